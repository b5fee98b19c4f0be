"""Builds the CUDA library in-tree: zerocool_b200/libzc_moe.so (sm_100a only)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libzc_moe.so")
SOURCES = ["api.cu", "router.cu", "route.cu", "experts_decode.cu", "experts_prefill.cu", "combine.cu", "ep.cu", "synth.cu"]
HEADERS = ["common.cuh", os.path.join("..", "..", "include", "zc_moe.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, ptxas_info=False):
    """Compiles every .cu to an object and links the shared library. Returns the library path."""
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    objects = []
    env = dict(os.environ)
    env.pop("CXX", None)
    env.pop("CC", None)
    jobs = []
    for name in SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(CSRC, name[:-3] + ".o")
        objects.append(obj)
        if force or _stale(obj, [src] + headers):
            extra = os.environ.get("ZC_NVCC_FLAGS", "").split()
            jobs.append((name, [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]))

    def compile_one(job):
        name, cmd = job
        return name, cmd, subprocess.run(cmd, capture_output=True, text=True, env=env)

    # the translation units are independent: compile them side by side (the largest one takes minutes)
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, jobs))
    for name, cmd, r in results:
        if verbose or ptxas_info or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed on " + name)
    if force or _stale(LIB, objects):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objects + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
