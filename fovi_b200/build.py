"""Build recipe of the native library: ``python -m fovi_b200.build``.

Compiles ``fovi_b200/csrc/*.cu`` with nvcc for sm_100a (one object per source, in parallel, only the
stale ones) and links them into ``fovi_b200/libfovi_b200.so`` (in-tree; objects and the shared object
are not committed).
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libfovi_b200.so")
SOURCES = ["capi.cu", "sampler.cu", "knnconv.cu", "knnconv_tc.cu", "knnconv_tc2.cu", "knnpool.cu", "knnnorm.cu", "fused.cu", "tables.cu", "geometry.cu", "grad.cu", "depthwise.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "fovi_b200.h"))
    hs.append(os.path.abspath(__file__))
    return max(os.path.getmtime(h) for h in hs)


def build(force=False, verbose=False, defines=(), lib=None, obj_dir=None):
    """Compile what is stale and link.  `defines` ("NAME=value" strings), `lib` and `obj_dir` give a variant
    build beside the default one.  Returns the path of the shared object."""
    lib = lib or LIB
    obj_dir = obj_dir or OBJ
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdr_t = _headers_mtime()
    flags = NVCC_FLAGS + [f"-D{d}" for d in defines] + (["-Xptxas", "-v"] if verbose else [])
    jobs = []
    for s in SOURCES:
        src, obj = os.path.join(CSRC, s), os.path.join(obj_dir, s[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            jobs.append((s, [nvcc] + flags + ["-c", src, "-o", obj]))

    def run(job):
        return job[0], subprocess.run(job[1], capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for name, r in pool.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {name}")
    objs = [os.path.join(obj_dir, s[:-3] + ".o") for s in SOURCES]
    if jobs or not os.path.exists(lib) or os.path.getmtime(lib) < max(os.path.getmtime(o) for o in objs):
        r = subprocess.run([nvcc] + NVCC_FLAGS[:2] + ["-shared", "-o", lib] + objs, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libfovi_b200.so failed")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
