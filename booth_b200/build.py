"""Builds the sm_100a kernel image and libbooth_sm100.so in-tree.

    python -m booth_b200.build          (or booth_b200.build.build())

Steps:
  1. nvcc -gencode arch=compute_100a,code=sm_100a -cubin  csrc/kernels/image.cu
        -> lib/booth_sm100.cubin   (also the file bc_load_kernel is pointed at)
  2. nvcc -c  csrc/reduce_noalloc.cu  (the one runtime-API translation unit:
        its scratch is a __device__ array, so it carries its own device code)
  3. gcc -std=c99 -shared  csrc/*.c csrc/image.S (embeds the cubin) + that object
        -> lib/libbooth_sm100.so   (static cudart, libdl, libpthread; libcuda and
                                    libnccl are opened at run time)
nvcc cross-compiles without a GPU. Outputs are git-ignored build products.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
CUBIN = os.path.join(LIB, "booth_sm100.cubin")
SO = os.path.join(LIB, "libbooth_sm100.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo",
              "-std=c++17", "--fmad=true", "-Xptxas", "-v"]
C_SOURCES = ["sm100_shim.c", "bc_runtime.c", "sm100_ops.c", "sm100_comm.c", "rt_sm100.c", "lf_gpu_sm100.c", "nv_rt_sm100.c"]


def _cuda_home():
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return cand
    nvcc = shutil.which("nvcc")
    if nvcc:
        return os.path.dirname(os.path.dirname(nvcc))
    raise RuntimeError("nvcc not found: the sm_100a kernel image cannot be built")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd, log):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append("$ " + " ".join(cmd) + "\n" + res.stdout)
    if res.returncode != 0:
        sys.stderr.write(log[-1])
        raise RuntimeError("build step failed: " + " ".join(cmd[:3]))
    return res.stdout


def build(force=False, verbose=False):
    """Compile the kernel image for sm_100a and link the C-ABI library."""
    os.makedirs(LIB, exist_ok=True)
    cuda = _cuda_home()
    kdir = os.path.join(CSRC, "kernels")
    ksrc = [os.path.join(kdir, f) for f in sorted(os.listdir(kdir)) if f.endswith((".cu", ".cuh"))]
    log = []
    if force or not _newer(CUBIN, ksrc):
        _run([os.path.join(cuda, "bin", "nvcc")] + NVCC_FLAGS +
             ["-cubin", "-o", CUBIN, os.path.join(kdir, "image.cu")], log)
        with open(os.path.join(LIB, "ptxas.log"), "w") as f:
            f.write(log[-1])
    csrc = [os.path.join(CSRC, f) for f in C_SOURCES]
    noalloc_cu = os.path.join(CSRC, "reduce_noalloc.cu")
    noalloc_o = os.path.join(LIB, "reduce_noalloc.o")
    if force or not _newer(noalloc_o, [noalloc_cu, os.path.join(INCLUDE, "booth_sm100.h")]):
        _run([os.path.join(cuda, "bin", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo",
              "-std=c++17", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-c", noalloc_cu, "-o", noalloc_o], log)
    deps = csrc + [noalloc_o, CUBIN, os.path.join(CSRC, "image.S"), os.path.join(CSRC, "sm100_internal.h"),
                   os.path.join(INCLUDE, "booth_sm100.h"), os.path.join(INCLUDE, "bc_runtime.h"),
                   os.path.join(INCLUDE, "rt_sm100.h"), os.path.join(INCLUDE, "lf_gpu.h"), os.path.join(INCLUDE, "nv_rt.h")]
    if force or not _newer(SO, deps):
        _run(["gcc", "-std=c99", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra",
              "-Wno-unused-parameter", "-fvisibility=default",
              "-I", INCLUDE, "-I", CSRC, "-I", os.path.join(cuda, "include"),
              '-DBOOTH_SM100_IMAGE="%s"' % CUBIN,
              "-o", SO] + csrc + [os.path.join(CSRC, "image.S"), noalloc_o] +
             ["-Wl,-Bsymbolic", "-Wl,-z,noexecstack", "-Wl,--exclude-libs,ALL", "-L", os.path.join(cuda, "lib64"), "-lcudart_static",
              "-lstdc++", "-lrt", "-ldl", "-lpthread"], log)
    if verbose:
        sys.stdout.write("\n".join(log))
    return SO


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(SO)
