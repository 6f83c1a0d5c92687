"""Build libtrb_kv.so (the C-ABI CUDA library) in-tree for sm_100a with nvcc.

    python -m tokenrush_b200.build [--force] [--verbose] [--timeline]

--timeline builds a second, diagnostic library (libtrb_kv_timeline.so) whose decode kernel records
per-CTA time stamps; `bench.py --workload timeline` loads it.

The library has no dependency on torch or Python; the host package loads it with ctypes.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtrb_kv.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]


def sources():
    out = [os.path.join(HERE, "..", "include", "trb_kv.h")]
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, f))
    return out


def up_to_date(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return False
    t = os.path.getmtime(lib)
    return all(os.path.getmtime(s) <= t for s in sources())


LIB_TIMELINE = os.path.join(HERE, "libtrb_kv_timeline.so")


def build(force: bool = False, verbose: bool = False, timeline: bool = False) -> str:
    lib = LIB_TIMELINE if timeline else LIB
    if not force and up_to_date(lib):
        return lib
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-DTRB_TIMELINE"] if timeline else []) + (["-Xptxas", "-v"] if verbose else []) + ["-o", lib, os.path.join(CSRC, "trb_kv.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed building libtrb_kv.so")
    if verbose:
        sys.stderr.write(r.stderr)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, timeline="--timeline" in sys.argv))
