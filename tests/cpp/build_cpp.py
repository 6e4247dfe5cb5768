"""Builds the C++ boundary test programs under tests/cpp against the CUDA library and the CPU oracle (the checker)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def build_cpp_test(name: str = "test_basic_attention", sanitize: bool = False, extra_sources=()) -> str:
    """Compiles tests/cpp/<name>.cpp (test binary, in-tree under tests/cpp/bin).  extra_sources: library sources (paths
    relative to the repository root) compiled INTO the test binary, so that -fsanitize instruments them; their symbols
    then take precedence over the library's."""
    from chatglm_cpp_b200 import build
    src = os.path.join(ROOT, "tests", "cpp", name + ".cpp")
    out_dir = os.path.join(ROOT, "tests", "cpp", "bin")
    out = os.path.join(out_dir, name + ("_asan" if sanitize else ""))
    os.makedirs(out_dir, exist_ok=True)
    deps = [src, build.LIB_PATH, os.path.join(ROOT, "oracle", "liboracle_attn.so"),
            os.path.join(ROOT, "include", "chatglm_b200.h"), os.path.join(ROOT, "include", "cglm_attn.h")]
    extra = [os.path.join(ROOT, e) for e in extra_sources]
    deps += extra
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps if os.path.exists(d)):
        return out
    if sanitize:
        # host-only sources, built by g++ so that the sanitizers instrument them
        cuda_home = os.path.dirname(os.path.dirname(build._nvcc()))
        cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer",
               "-I" + os.path.join(cuda_home, "include"), "-x", "c++", src, *extra, "-o", out, "-L" + build.LIB_DIR,
               "-lcglm_attn", "-L" + os.path.join(cuda_home, "lib64"), "-lcudart",
               "-Wl,-rpath,$ORIGIN/../../../chatglm_cpp_b200/lib", "-Wl,-rpath," + os.path.join(cuda_home, "lib64")]
    else:
        cmd = [build._nvcc(), "-std=c++17", "-O2", "-x", "cu", src, *extra, "-o", out, "-L" + build.LIB_DIR, "-lcglm_attn",
               "-L" + os.path.join(ROOT, "oracle"), "-loracle_attn", "-Xlinker", "-rpath", "-Xlinker",
               "$ORIGIN/../../../chatglm_cpp_b200/lib", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../oracle",
               "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the C++ boundary test failed")
    return out
