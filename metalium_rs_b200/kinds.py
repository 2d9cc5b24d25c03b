"""Element-wise kind numbers, read from csrc/kinds.h (the reference's numbering:
crates/tt-kernels/src/kind.rs:12-26, crates/tt-kernels/src/sfpu/ops.rs:24-251)."""
import re
from pathlib import Path

_text = (Path(__file__).resolve().parent / "csrc" / "kinds.h").read_text()
ARITY = {}
NAMES = {}
for _m in re.finditer(r"X\((\w+),\s*(0x[0-9a-fA-F]+|\d+),\s*(\d)\)", _text):
    _name, _val, _ar = _m.group(1), int(_m.group(2), 0), int(_m.group(3))
    globals()[_name] = _val
    ARITY[_val] = _ar
    NAMES[_val] = _name
del _m, _name, _val, _ar, _text
