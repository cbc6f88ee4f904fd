"""The C ABI from C: a C99 embedder that includes only include/pfhe_b200.h and the CUDA runtime's C API is
compiled with gcc, linked against the library and (on a GPU) run; it compares what the library decodes with
the CPU oracle, bit for bit."""
import os
import shutil
import subprocess

import pytest

from pfhe_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
GCC = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")

pytestmark = pytest.mark.skipif(GCC is None or not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime_api.h")),
                                reason="needs gcc and the CUDA headers")


def _build(tmp_path):
    _native.lib()                                             # builds the library if it is missing
    exe = str(tmp_path / "c_embedder")
    libdir = os.path.join(ROOT, "pfhe_b200")
    cmd = [GCC, "-std=c11", "-Wall", "-Wextra", "-Werror", "-Wno-unknown-pragmas", "-O2", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           os.path.join(ROOT, "tests", "c_abi", "c_embedder.c"), os.path.join(ROOT, "oracle", "dequant_oracle.c"), "-o", exe,
           "-L", libdir, "-lpfhe_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-lm",
           f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_header_is_strict_c99(tmp_path):
    src = tmp_path / "hdr.c"
    src.write_text('#include "pfhe_b200.h"\nint main(void) { return pfhe_version() < 0; }\n')
    res = subprocess.run([GCC, "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_c_embedder_compiles_and_links(tmp_path):
    exe = _build(tmp_path)
    assert os.access(exe, os.X_OK)


@pytest.mark.gpu
def test_c_embedder_matches_the_oracle(tmp_path):
    exe = _build(tmp_path)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "c_embedder ok: " in res.stdout and int(res.stdout.rsplit("c_embedder ok: ", 1)[1].split()[0]) >= 60
