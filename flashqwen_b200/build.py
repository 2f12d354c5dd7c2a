"""Builds libfqb.so in-tree with nvcc for sm_100a: `python flashqwen_b200/build.py [-v]` (run as a file: importing the package needs the library)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["csrc/fqb_cuda.cu", "csrc/host/errors.cc", "csrc/host/allocator.cc", "csrc/host/layout.cc", "csrc/host/engine_shim.cc", "csrc/host/step_driver.cc"]
HEADERS = ["csrc/common.cuh", "csrc/decode.cuh", "csrc/umma.cuh", "csrc/prefill_tc_ks.cuh", "csrc/kv_append.cuh", "csrc/blocks.cuh",
           "csrc/errors.h", "../include/fqb.h"]


def out_path():
    return os.path.join(HERE, "libfqb.so")


def up_to_date():
    out = out_path()
    if not os.path.exists(out):
        return False
    t = os.path.getmtime(out)
    return all(os.path.getmtime(os.path.join(HERE, s)) <= t for s in SOURCES + HEADERS)


def build(verbose=False, force=False):
    if not force and up_to_date():
        return out_path()
    cmd = ["nvcc", "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "-o", out_path()] + [os.path.join(HERE, s) for s in SOURCES]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    cmd[1:1] = [x for x in sys.argv[1:] if x.startswith("-D")]  # build-time choices, e.g. -DFQB_DEFAULT_CTAS_PER_SM=1
    subprocess.run(cmd, check=True)
    return out_path()


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force=True))
