"""Builds libqwen3_5_cuda.so for sm_100a in-tree with nvcc (no JIT cache, no torch)."""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libqwen3_5_cuda.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

FLAGS = ["-O3", "-std=c++17", "--extended-lambda", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, ptxas_info=False):
    """Compile every source to an object (in parallel) and link the shared library."""
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    procs, objs = [], []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src}\n{out}\n")
        elif verbose or ptxas_info:
            sys.stderr.write(f"--- {src}\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(OUT, objs):
        lib64 = os.path.join(CUDA_HOME, "lib64")
        cmd = [NVCC, "-shared", "-o", OUT] + objs + ["-L" + lib64, "-ldl", "-Xlinker", "-rpath", "-Xlinker", lib64]
        subprocess.run(cmd, check=True)
    build_compare()
    return OUT


def build_compare():
    """The microbenchmark's comparison arm (the vendor library's GEMM) as a library of its own."""
    src = os.path.join(PKG, "compare", "library_gemm.cpp")
    out = os.path.join(PKG, "compare", "libs1_compare.so")
    if _stale(out, [src]):
        lib64 = os.path.join(CUDA_HOME, "lib64")
        subprocess.run([NVCC, "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-o", out, src, "-L" + lib64,
                        "-lcublasLt", "-Xlinker", "-rpath", "-Xlinker", lib64], check=True)
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv))
