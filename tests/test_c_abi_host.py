"""The compiled C host (tests/c_abi/fa_data_host.c): a fa_data.h in the reference's array layout goes through the
C ABI as it lies.  Without a GPU the program is compiled and linked only (the header is plain C, every symbol
resolves); with one it runs and reports pass / fail like the reference's self-checking kernels."""
import os
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests" / "c_abi"))
import make_fa_data  # noqa: E402

import radiance_kernels_b200 as rk  # noqa: E402


def _cuda_home():
    for c in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if c and os.path.isdir(os.path.join(c, "include")):
            return c
    pytest.skip("no CUDA toolkit headers")


def _build(tmp_path, **shape):
    rk.lib()                                                     # raises if the library was never built
    make_fa_data.write_fa_data(tmp_path / "fa_data.h", **shape)
    cuda = _cuda_home()
    libdir = ROOT / "radiance-kernels_b200"
    exe = tmp_path / "fa_data_host"
    cmd = ["gcc", "-std=c11", "-O1", "-Wall", "-Werror", "-I", str(tmp_path), "-I", str(ROOT / "include"), "-I", f"{cuda}/include",
           str(ROOT / "tests" / "c_abi" / "fa_data_host.c"), "-o", str(exe), f"-L{libdir}", "-l:librk_mx_attn.so",
           f"-L{cuda}/lib64", "-lcudart", "-lm", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda}/lib64"]
    subprocess.run(cmd, check=True)
    return exe


def test_c_host_compiles_and_links_against_the_header(tmp_path):
    exe = _build(tmp_path, Sq=64, Sk=128, d=64, n_q=2, n_kv=1, q_pos0=64, Bk=64)
    assert exe.exists()


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [dict(Sq=64, Sk=256, d=64, n_q=8, n_kv=2, q_pos0=64, Bk=64),      # kernels/regen_data.sh:31-32
                                   dict(Sq=192, Sk=512, d=128, n_q=4, n_kv=2, q_pos0=320, Bk=64, seed=3)])
def test_c_host_runs_reference_layout_arrays(tmp_path, shape):
    exe = _build(tmp_path, **shape)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "errors 0" in r.stdout
