"""Builds libatb_b200.so (CUDA kernels + C ABI + the atb:: C++ operator layer) in-tree with nvcc for sm_100a."""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libatb_b200.so")

CU_SOURCES = ["reshape_and_cache.cu", "pa_generic.cu", "pa_combine.cu", "pa_tma_mma.cu", "atb_scale_convert.cu",
              "pa_noalloc.cu", "pa_tma_mma_i8.cu", "pa_mla_tc5.cu", "pa_mla_pair.cu", "pa_exchange.cu", "cache_ops.cu", "norm_rope_cache.cu"]
CPP_SOURCES = ["tma_encode.cpp", "pa_planner.cpp", "c_api.cpp", "atb_operation_base.cpp", "atb_paged_attention.cpp",
               "atb_reshape_and_cache.cpp", "atb_c_wrappers.cpp", "atb_cache_ops.cpp", "atb_mla.cpp"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=default", "--expt-relaxed-constexpr",
              "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def sources():
    return [os.path.join(CSRC, s) for s in CU_SOURCES + CPP_SOURCES]


def stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps += [os.path.join(ROOT, "include", "atb_b200.h")]
    deps += [os.path.join(ROOT, "include", "atb", f) for f in os.listdir(os.path.join(ROOT, "include", "atb"))]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every source with nvcc and link the shared library.  Objects go to csrc/build/."""
    if not force and not stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and not _obj_stale(obj, src):
            continue
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", OUT] + objs + ["-cudart", "shared" if os.environ.get("ATB_B200_SHARED_CUDART") else "static", "-ldl"])
    return OUT


def _obj_stale(obj, src):
    t = os.path.getmtime(obj)
    deps = [src] + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps += [os.path.join(ROOT, "include", "atb_b200.h")]
    deps += [os.path.join(ROOT, "include", "atb", f) for f in os.listdir(os.path.join(ROOT, "include", "atb"))]
    return any(os.path.getmtime(d) > t for d in deps)


def build_cpp_test():
    """Compiles tests/cpp/atb_cpp_api_test.cpp (a C++ caller of include/atb/) against the library."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    src = os.path.join(ROOT, "tests", "cpp", "atb_cpp_api_test.cpp")
    exe = os.path.join(ROOT, "tests", "cpp", "atb_cpp_api_test")
    if os.path.exists(exe) and os.path.getmtime(exe) > max(os.path.getmtime(src), os.path.getmtime(OUT)):
        return exe
    subprocess.check_call([nvcc, "-std=c++17", "-O2", "-Wno-deprecated-gpu-targets", "-I" + os.path.join(ROOT, "include"),
                           "-x", "cu", src, "-o", exe, "-L" + PKG, "-latb_b200", "-Xlinker", "-rpath=" + PKG])
    return exe


def build_host_emulation():
    """Compiles tests/cpp/cache_ops_host_emulation.cpp with g++: the bodies of the cache-management
    kernels run on the CPU so that the tests can compare them with the oracle and the golden fixtures."""
    src = os.path.join(ROOT, "tests", "cpp", "cache_ops_host_emulation.cpp")
    body = os.path.join(CSRC, "cache_ops_body.h")
    so = os.path.join(ROOT, "tests", "cpp", "libcache_ops_host_emulation.so")
    if os.path.exists(so) and os.path.getmtime(so) > max(os.path.getmtime(src), os.path.getmtime(body)):
        return so
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-g", "-shared", "-fPIC", src, "-o", so])
    return so


def build_body_selftest():
    """Compiles tests/cpp/cache_ops_body_selftest.cpp with AddressSanitizer and UBSan: randomized and
    adversarial cases of the same kernel bodies; an out-of-bounds access aborts the executable."""
    src = os.path.join(ROOT, "tests", "cpp", "cache_ops_body_selftest.cpp")
    body = os.path.join(CSRC, "cache_ops_body.h")
    exe = os.path.join(ROOT, "tests", "cpp", "cache_ops_body_selftest")
    if os.path.exists(exe) and os.path.getmtime(exe) > max(os.path.getmtime(src), os.path.getmtime(body)):
        return exe
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined",
                           "-fno-sanitize-recover=all", src, "-o", exe])
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
