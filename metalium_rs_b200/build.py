"""Build libb200tt.so (the C-ABI engine) in-tree with nvcc for sm_100a.

The Rust crate that would bind this library runs the same nvcc command lines from its
`build.rs` (see rust/b200-sys/build.rs); this script is the stand-in where no Rust
toolchain exists.  nvcc cross-compiles without a GPU.

    python -m metalium_rs_b200.build [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libb200tt.so"
OBJ = HERE / "build"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# source -> extra flags.  -fmad=false where the reference defines separate roundings.
SOURCES = {
    "engine.cu": ["-Xcompiler", "-fvisibility=default"],
    "k_eltwise.cu": ["-fmad=false"],
    "k_reduce.cu": ["-fmad=false"],
    "k_index.cu": [],
    "k_gemm_simt.cu": [],
    "k_gemm_tc.cu": [],
    "k_gemm_tf32.cu": [],
    "k_gemm_tc2.cu": [],
    "k_gemm_addnorm.cu": ["-fmad=false"],
    "k_gemm_skinny.cu": [],
    "k_attention.cu": [],
    "k_attention_tc.cu": [],
    "k_convert.cu": [],
    "k_bfp.cu": [],
    "k_decode.cu": [],
    "k_pool.cu": ["-fmad=false"],
    "k_scan_sort.cu": ["-fmad=false"],
    "k_random.cu": ["-fmad=false"],
}


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the engine cannot be built")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile(src: str, flags, stamp: str) -> Path:
    obj = OBJ / (src.replace(".cu", ".o"))
    mark = OBJ / (src + ".stamp")
    if obj.exists() and mark.exists() and mark.read_text() == stamp:
        return obj
    cmd = [nvcc(), *ARCH, *COMMON, *flags, "-c", str(CSRC / src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    mark.write_text(stamp)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    # B200TT_SKIP_BUILD=1: use the library as shipped (a run that must not recompile).
    if os.environ.get("B200TT_SKIP_BUILD") == "1" and OUT.exists() and not force:
        return OUT
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "b200tt.h"]
    hstamp = _digest(headers)
    stamps = {s: hashlib.sha256((hstamp + (CSRC / s).read_text() + " ".join(f)).encode()).hexdigest()
              for s, f in SOURCES.items()}
    if force:
        for s in SOURCES:
            (OBJ / (s + ".stamp")).unlink(missing_ok=True)
    link_stamp = hashlib.sha256("".join(stamps[s] for s in sorted(stamps)).encode()).hexdigest()
    lmark = OBJ / "link.stamp"
    if OUT.exists() and lmark.exists() and lmark.read_text() == link_stamp and not force:
        return OUT
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda kv: _compile(kv[0], kv[1], stamps[kv[0]]), SOURCES.items()))
    tmp = OUT.with_suffix(".so.tmp")   # linked beside the target, then renamed: a reader never sees half a library
    cmd = [nvcc(), *ARCH, "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, OUT)
    lmark.write_text(link_stamp)
    if verbose:
        print(f"built {OUT}")
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
