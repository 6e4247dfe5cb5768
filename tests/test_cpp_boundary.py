"""Runs the C++ test of the chatglm::BasicAttention mirror (tests/cpp/test_basic_attention.cpp) on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_cpp_basic_attention_mirror(tmp_path):
    from chatglm_cpp_b200 import build
    from oracle import attn_oracle
    build.build()
    attn_oracle.build()
    from cpp.build_cpp import build_cpp_test
    exe = build_cpp_test()
    # a model file in the converter's layout (ChatGLM3 shape with a P-Tuning prefix, f16 matrices) for the case that builds
    # the attention modules from a file
    import model_file_writer as W
    blob, _ = W.write_model(W.GLM3_PTUNING, W.F16, 2, seed=21)
    path = tmp_path / "glm3_ptuning.bin"
    path.write_bytes(blob)
    r = subprocess.run([exe, str(path)], capture_output=True, text=True, timeout=600)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL OK" in r.stdout and "forward from a model file" in r.stdout


def test_cpp_boundary_test_builds():
    """CPU check: the C++ mirror's test program compiles and links against the library and the oracle."""
    from chatglm_cpp_b200 import build
    from oracle import attn_oracle
    build.build()
    attn_oracle.build()
    from cpp.build_cpp import build_cpp_test
    assert os.path.exists(build_cpp_test())
