"""The exported C headers of the kernel library can be read by a C compiler."""

import os
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "thing_htn_2026_b200", "csrc")


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_no_alloc_header_is_valid_c(tmp_path):
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    if not os.path.exists(os.path.join(cuda, "include", "cuda_runtime.h")):
        pytest.skip("no CUDA headers")
    source = tmp_path / "use.c"
    source.write_text('#include "attention_no_alloc.h"\n'
                      "int (*entry)(void*, const void*, const int*, const int*, const void*, const int*, int, int, int,\n"
                      "             int, int, int, int, float, int, int*, cudaStream_t) = thn_attention_decode_bf16_no_alloc;\n")
    done = subprocess.run(["gcc", "-x", "c", "-std=c99", "-fsyntax-only", f"-I{CSRC}", f"-I{cuda}/include", str(source)],
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
