"""Build liblkb.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python lfm2-ampere_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is written next to this file so
that it travels with the source tree; it is never installed into site-packages.
"""
import os
import pathlib
import shlex
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "liblkb.so"
SOURCES = ["lkb_decode.cu", "lkb_prefill.cu", "lkb_gemm_tc.cu", "lkb_fused.cu", "lkb_lmhead.cu", "lkb_mixer.cu", "lkb_pfmix.cu", "lkb_ep.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xcompiler", "-O3", "-shared", "-cudart", "static"]


def needs_build():
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "lkb.h", pathlib.Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return OUT
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    extra = shlex.split(os.environ.get("LKB_NVCC_EXTRA", ""))          # e.g. -DTC_MAGIC=0 while tuning
    cmd = ["nvcc"] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-o", str(OUT)] + srcs + ["-lcuda"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("nvcc failed building liblkb.so")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
