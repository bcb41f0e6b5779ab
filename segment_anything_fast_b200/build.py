"""Build the sm_100a kernel library in-tree: ``python -m segment_anything_fast_b200.build``.

Plain ``nvcc`` (cross-compiles without a GPU); the result
``segment_anything_fast_b200/lib/libsamb200.so`` exports only the C ABI declared in
``include/samb200.h`` and links the CUDA runtime statically, so it has no
load-time dependency on a driver or on torch.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libsamb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static"]
OBJ_DIR = os.path.join(PKG, "build")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(os.path.dirname(PKG), "include", "samb200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """One object per source (compiled in parallel, recompiled only when the source or a shared header is newer),
    then one link.  ``force`` recompiles everything."""
    if not force and not needs_build():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    shared = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith(".cu")]
    shared.append(os.path.join(os.path.dirname(PKG), "include", "samb200.h"))
    newest_shared = max(os.path.getmtime(h) for h in shared)

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src)
                and os.path.getmtime(obj) > newest_shared):
            return obj, 0, ""
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return obj, proc.returncode, proc.stdout + proc.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    for _, rc, log in results:
        if (verbose or rc) and log:
            sys.stderr.write(log)
    if any(rc for _, rc, _ in results):
        raise RuntimeError("nvcc failed building libsamb200.so")
    proc = subprocess.run([nvcc] + LINK_FLAGS + ["-o", LIB_PATH] + [o for o, _, _ in results], capture_output=True, text=True)
    if proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("linking libsamb200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
