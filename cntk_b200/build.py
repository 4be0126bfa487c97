"""Builds cntk_b200/libqagg.so in-tree with nvcc for sm_100a.  No GPU is needed to build.

    python -m cntk_b200.build [--verbose]

NCCL: the header and library shipped inside the Python environment (the one PyTorch itself loads) are used when
present, else the system ones; the library is linked by SONAME (libnccl.so.2), so inside a process that has
already imported torch the copy torch loaded is reused.
"""
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libqagg.so")
SOURCES = ["qagg_kernels.cu", "qagg_stream.cu", "qagg_unquantize.cu", "qagg_owner.cu", "qagg_capi.cu", "qagg_aggregator.cu", "qagg_dense.cu", "qagg_f64.cu", "qagg_agg_f64.cu", "qagg_update.cu", "qagg_noalloc.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nccl_paths():
    try:
        import nvidia.nccl as m  # type: ignore
        base = list(m.__path__)[0]
        inc, lib = os.path.join(base, "include"), os.path.join(base, "lib")
        if os.path.exists(os.path.join(inc, "nccl.h")) and glob.glob(os.path.join(lib, "libnccl.so*")):
            return inc, lib
    except Exception:
        pass
    return None, None


def nvcc_path():
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def needs_build():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(os.path.dirname(HERE), "include", "qagg.h"), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    if not force and not needs_build():
        return OUT
    inc, lib = _nccl_paths()
    cmd = [nvcc_path(), "-O3", "-std=c++17", "-lineinfo", "--fmad=false", "-shared", "-Xcompiler", "-fPIC,-fvisibility=default"] + ARCH
    if verbose:
        cmd += ["-Xptxas", "-v"]
    if inc:
        cmd += ["-I", inc, "-L", lib, "-l:libnccl.so.2", "-Xlinker", "-rpath=" + lib]
    else:
        cmd += ["-lnccl"]
    cmd += ["-o", OUT] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libqagg.so")
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
