"""Builds librt_attn.so (the CUDA kernels and the C ABI) for sm_100a with nvcc.

nvcc cross-compiles without a GPU.  The library links the static CUDA runtime
and resolves driver entry points at run time, so it loads (and its symbols can
be listed) on a machine without a GPU or driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "librt_attn.so")
SOURCES = ["api.cu", "prefill_simt.cu", "prefill_tc.cu", "prefill_tc2.cu", "prefill_tc3.cu", "prefill_tc4.cu", "decode.cu", "exchange.cu", "misc.cu", "softmax.cu",
           "local_attn.cu", "matmul.cu",
           "matmul_tc.cu"]
HEADERS = ["common.cuh", "sm100.cuh", "tc_common.cuh", os.path.join(ROOT, "include", "rt_attn.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-O2,-fvisibility=hidden", "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES]
    deps += [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), target: str = LIB) -> str:
    """Compile the library if it is missing or older than its sources.  ``defines``
    (extra -D macros) and ``target`` build a variant beside the product library, for
    kernel experiments."""
    if not force and not defines and target == LIB and not _stale():
        return LIB
    objdir = (os.path.join(HERE, "build") if target == LIB else
              os.path.join(os.path.dirname(target), "build_" + os.path.basename(target)))
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    objs, procs = [], []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-ccbin", "/usr/bin/g++", "-I",
               os.path.join(ROOT, "include"), "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-shared", "-cudart", "static", "-ccbin", "/usr/bin/g++", "-o", target, *objs,
            "-Xlinker", "--exclude-libs,ALL", "-ldl", "-lpthread", "-lrt"]
    subprocess.check_call(link, env=env)
    return target


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
