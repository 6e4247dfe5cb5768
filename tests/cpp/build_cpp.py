"""Builds the C++ boundary test programs under tests/cpp against the CUDA library and the CPU oracle (the checker)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def build_cpp_test(name: str = "test_basic_attention", sanitize: bool = False) -> str:
    """Compiles tests/cpp/<name>.cpp (test binary, in-tree under tests/cpp/bin)."""
    from chatglm_cpp_b200 import build
    src = os.path.join(ROOT, "tests", "cpp", name + ".cpp")
    out_dir = os.path.join(ROOT, "tests", "cpp", "bin")
    out = os.path.join(out_dir, name + ("_asan" if sanitize else ""))
    os.makedirs(out_dir, exist_ok=True)
    deps = [src, build.LIB_PATH, os.path.join(ROOT, "oracle", "liboracle_attn.so"),
            os.path.join(ROOT, "include", "chatglm_b200.h"), os.path.join(ROOT, "include", "cglm_attn.h")]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps if os.path.exists(d)):
        return out
    cmd = [build._nvcc(), "-std=c++17", "-O2", "-x", "cu", src, "-o", out, "-L" + build.LIB_DIR, "-lcglm_attn",
           "-L" + os.path.join(ROOT, "oracle"), "-loracle_attn", "-Xlinker", "-rpath", "-Xlinker",
           "$ORIGIN/../../../chatglm_cpp_b200/lib", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../oracle",
           "-cudart", "static"]
    if sanitize:
        cmd += ["-Xcompiler", "-fsanitize=address,undefined", "-Xcompiler", "-fno-omit-frame-pointer"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the C++ boundary test failed")
    return out
