"""In-tree build of the native parts: libbuda_cuda.so (CUDA kernels + C ABI, sm_100a only), the
pybind11 module pybuda._C (C++ host layer that calls the C ABI), and libbuda_probe.so (bare streaming
kernels that only the benchmark loads).

    python tt-buda_b200/build.py [--force]

Outputs stay inside the package (lib/libbuda_cuda.so, pybuda/_C*.so) so they travel with the
source tree; nothing is installed into site-packages.
"""
import concurrent.futures
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(CSRC, "build")
CUDA_LIB = os.path.join(LIB_DIR, "libbuda_cuda.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

PROBE_LIB = os.path.join(LIB_DIR, "libbuda_probe.so")
CU_SOURCES = ["capi.cu", "tilize_pack.cu", "unpack_untilize.cu", "quant.cu", "bfp8_gemm.cu", "gemm_pair.cu", "prestride.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE]

HOST_DIR = os.path.join(HERE, "pybuda", "csrc")
HOST_SOURCES = ["pybuda_bindings.cpp", "backend_api/backend_api.cpp", "backend_api/queue_store.cpp",
                "lower_to_buda/common.cpp", "balancer/tile_layout.cpp", "tt_torch_device/tt_device.cpp"]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _env():
    # the image exports CC/CXX pointing at a wrapper without OpenMP specs; use the PATH compilers
    return {k: v for k, v in os.environ.items() if k not in ("CC", "CXX", "CFLAGS", "CXXFLAGS")}


def _run(cmd):
    r = subprocess.run(cmd, env=_env(), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


def build_cuda(force=False, verbose=False):
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    headers.append(os.path.join(INCLUDE, "buda_cuda.h"))
    jobs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src[:-3] + ".o")
        if force or _newer(o, [s] + headers):
            jobs.append([_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out:
                print(out)
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in CU_SOURCES]
    if force or jobs or _newer(CUDA_LIB, objs):
        _run([_nvcc(), "-shared", "-o", CUDA_LIB] + objs + ["-Xcompiler", "-fPIC"])
    probe_src = os.path.join(CSRC, "bench", "stream_probe.cu")
    if force or _newer(PROBE_LIB, [probe_src]):
        _run([_nvcc()] + NVCC_FLAGS + ["-shared", "-o", PROBE_LIB, probe_src])
    return CUDA_LIB


def pybind_target():
    return os.path.join(HERE, "pybuda", "_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pybind(force=False):
    import pybind11

    target = pybind_target()
    srcs = [os.path.join(HOST_DIR, s) for s in HOST_SOURCES]
    deps = list(srcs)
    for root, _, files in os.walk(HOST_DIR):
        deps += [os.path.join(root, f) for f in files if f.endswith((".hpp", ".h"))]
    deps.append(os.path.join(INCLUDE, "buda_cuda.h"))
    if not (force or _newer(target, deps)):
        return target
    obj_dir = os.path.join(HOST_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)
    inc = ["-I", HOST_DIR, "-I", INCLUDE, "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.relpath(s, HOST_DIR).replace(os.sep, "_")[:-4] + ".o")
        objs.append(o)
        if force or _newer(o, deps):
            jobs.append(["g++"] + flags + inc + ["-c", s, "-o", o])
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        list(ex.map(_run, jobs))
    # the host module finds libbuda_cuda.so next to the package at run time ($ORIGIN/../lib)
    _run(["g++", "-shared", "-o", target] + objs +
         ["-L", LIB_DIR, "-lbuda_cuda", "-Wl,-rpath,$ORIGIN/../lib", "-ldl", "-lpthread"])
    return target


def build_all(force=False, verbose=False):
    lib = build_cuda(force=force, verbose=verbose)
    mod = build_pybind(force=force) if os.path.isdir(HOST_DIR) else None
    return lib, mod


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
