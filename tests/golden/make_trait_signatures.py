"""Writes tests/golden/engine_trait.json: the method list of the reference's `pub trait Engine`
(crates/burn-tt/src/server.rs:42-786) -- every method's parameter types and result type, names of
modules dropped -- so a test can hold the Rust shim's `impl Engine for CudaEngine` to the trait
without a Rust compiler.  Run where the reference tree is mounted:

    python tests/golden/make_trait_signatures.py /path/to/reference

The same parser reads the shim in tests/test_abi.py.
"""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def block_after(text: str, start_pattern: str) -> str:
    """The text between the braces that follow the first match of `start_pattern`."""
    m = re.search(start_pattern, text)
    if not m:
        raise ValueError(f"{start_pattern!r} not found")
    i = text.index("{", m.end())
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i + 1:j]
    raise ValueError("unbalanced braces")


def _top_level_fns(body: str):
    body = re.sub(r"//[^\n]*", "", body)
    out, depth, i, n = [], 0, 0, len(body)
    while i < n:
        c = body[i]
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
        elif depth == 0 and body.startswith("fn ", i) and (i == 0 or not (body[i - 1].isalnum() or body[i - 1] == "_")):
            m = re.match(r"fn\s+([a-z0-9_]+)\s*(<[^>]*>)?\s*\(", body[i:])
            if m:
                j, d = i + m.end(), 1
                while d:
                    d += body[j] in "([" 
                    d -= body[j] in ")]"
                    j += 1
                params = body[i + m.end():j - 1]
                k, d = j, 0
                while not (d == 0 and body[k] in "{;"):     # the `;` of `[usize; 2]` sits inside brackets
                    d += body[k] in "([<"
                    d -= body[k] in ")]>" and not body.startswith("->", k - 1)
                    k += 1
                out.append((m.group(1), params, body[j:k]))
                i = k
                continue
        i += 1
    return out


def _split(params: str):
    parts, d, cur = [], 0, ""
    for ch in params:
        d += ch in "([<"
        d -= ch in ")]>"
        if ch == "," and d == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    parts.append(cur)
    return [p.strip() for p in parts if p.strip()]


def norm_type(t: str) -> str:
    t = re.sub(r"\s+", " ", t.strip())
    t = re.sub(r"^-> ?", "", t)
    t = re.sub(r"\b(?:[a-z_][a-z0-9_]*::)+", "", t)            # module paths: tt_kernels::tensor::Eltwise -> Eltwise
    t = re.sub(r"&'static ", "&", t)
    return re.sub(r"\s*([<>,\[\]\(\)&;:])\s*", r"\1", t)


def signatures(body: str) -> dict:
    res = {}
    for name, params, ret in _top_level_fns(body):
        ps = []
        for p in _split(params):
            ps.append(p if p in ("&self", "&mut self", "self") else norm_type(p.split(":", 1)[1]))
        res[name] = {"params": ps, "ret": norm_type(ret)}
    return res


def trait_signatures(reference_root: Path) -> dict:
    src = (reference_root / "crates" / "burn-tt" / "src" / "server.rs").read_text()
    return signatures(block_after(src, r"pub trait Engine\b"))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_trait_signatures.py <root of the metalium-rs tree>")
    root = Path(sys.argv[1])
    sig = trait_signatures(root)
    (HERE / "engine_trait.json").write_text(json.dumps(sig, indent=1, sort_keys=True) + "\n")
    print(f"{len(sig)} methods written")
