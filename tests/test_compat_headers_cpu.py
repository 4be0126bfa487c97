"""The C++ mirror of the reference interfaces (cntk_b200/csrc/cntk_compat) without a device: every header compiles on its
own, the driver program of the GPU tests links against the library, and the host-only logic -- the data-parallel
configuration checks and epoch bookkeeping of SGD (Source/SGDLib/SGD.cpp:3294-3343, SGD.h:634-637), DistGradHeader
(Source/SGDLib/DistGradHeader.h:5-95), the process-wide MPIWrapper slot -- behaves as the reference's."""
import glob
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
HEADERS = sorted(glob.glob(os.path.join(ROOT, "cntk_b200", "csrc", "cntk_compat", "*.h")))


def _link_args():
    libdir = os.path.join(ROOT, "cntk_b200")
    return ["-L", libdir, "-l:libqagg.so", f"-L{CUDA}/lib64", "-lcudart", "-lpthread", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{CUDA}/lib64"]


@pytest.fixture(scope="module")
def built():
    if not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime.h")):
        pytest.skip("CUDA headers not found")
    from cntk_b200 import build
    build.build()


@pytest.mark.parametrize("header", HEADERS, ids=[os.path.basename(h) for h in HEADERS])
def test_every_mirror_header_compiles_on_its_own(built, header, tmp_path):
    src = tmp_path / "tu.cpp"
    src.write_text(f'#include "{header}"\nint main() {{ return 0; }}\n')
    res = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", f"-I{CUDA}/include", str(src)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_driver_program_links_against_the_library(built, tmp_path):
    exe = str(tmp_path / "compat_check")
    res = subprocess.run(["g++", "-std=c++17", "-O0", f"-I{CUDA}/include", os.path.join(ROOT, "tests", "cpp", "compat_check.cpp"), "-o", exe] + _link_args(),
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_host_only_logic(built, tmp_path):
    exe = str(tmp_path / "host_logic_check")
    res = subprocess.run(["g++", "-std=c++17", "-O1", f"-I{CUDA}/include", os.path.join(ROOT, "tests", "cpp", "host_logic_check.cpp"), "-o", exe] + _link_args(),
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and "host logic ok" in run.stdout, (run.returncode, run.stdout, run.stderr)
