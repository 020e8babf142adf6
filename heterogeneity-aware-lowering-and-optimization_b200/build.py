"""Builds libodla_b200.so in-tree with nvcc for sm_100a.

Every translation unit under csrc/ is compiled with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into one shared library next to
this file.  The CUDA runtime is linked statically and the driver API is reached through
cudaGetDriverEntryPoint, so the library loads (and exports every symbol) on a machine without a
GPU or libcuda; it simply reports zero devices there.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libodla_b200.so")
SOURCES = ["api.cc", "plan.cc", "quant_table.cc", "executable.cc", "kabi.cu", "noalloc.cu", "kernels_simt.cu", "kernels_detect.cu", "kernels_umma.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=default,-Wall,-Wno-unused-function", "-x", "cu",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"] + (["-DUMMA_DEBUG_TS"] if os.environ.get("UMMA_DEBUG_TS") else []) + (["-DUMMA_EPI_WARPS=" + os.environ["UMMA_EPI_WARPS"]] if os.environ.get("UMMA_EPI_WARPS") else [])


def _stale(obj, deps):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "odla_b200.h"))
    headers.append(os.path.abspath(__file__))
    objs, jobs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append([NVCC] + FLAGS + ["-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, len(jobs))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or not os.path.exists(OUT):
        cmd = [NVCC, "-shared", "-o", OUT] + objs + ["-cudart", "static", "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
