"""In-tree build of libvyre_b200.so with nvcc for sm_100a (no JIT cache: the built library travels with the tree).

    python -m vyre_b200.build            # incremental
    python -m vyre_b200.build --force    # rebuild everything

Per-file flags matter: ref_ops.cu is compiled with -ftz=true so that f32 subnormals flush exactly like the
reference interpreter's canonicalisation; the bandwidth/tensor kernels use default (IEEE) modes.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libvyre_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall", "-Xptxas", "-v",
          "--expt-relaxed-constexpr"]

# source -> extra flags
SOURCES = {
    "host/blake3.cpp": [],
    "host/program.cpp": [],
    "host/artifact.cpp": [],
    "host/safetensors.cpp": [],
    "host/graph.cpp": [],
    "host/substrate.cpp": [],
    "host/frames.cpp": [],
    "host/runtime.cu": [],
    "kernels/ref_ops.cu": ["-ftz=true", "-prec-div=true", "-prec-sqrt=true", "-fmad=false"],
    "kernels/dropin_fast.cu": ["-ftz=true", "-fmad=false"],
    "kernels/int4_gemv.cu": [],
    "kernels/int4_gemv_halfsm.cu": [],
    "kernels/int4_gemv_batch8.cu": [],
    "kernels/int8_linear.cu": [],
    "kernels/int8_gemm_tcgen05.cu": [],
    "kernels/int8_gemm_pair_tcgen05.cu": [],
    "kernels/int4_prefill_tcgen05.cu": [],
    "kernels/int4_gemm_pair_tcgen05.cu": [],
    "kernels/moe_ffn.cu": [],
    "kernels/allgather_push.cu": [],
    "kernels/moe_ep.cu": [],
    "kernels/int8_dynamic_static_scratch.cu": [],
    "kernels/tensor_peak.cu": [],
}


def nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the native library cannot be built (there is no CPU fallback)")
    return cand


def _host_compiler_flags() -> list[str]:
    # the image exports CXX=/opt/gcc/bin/g++ (a wrapper); nvcc must use the distro g++
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def _deps_mtime() -> float:
    m = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".h", ".hpp", ".cuh")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    m = max(m, os.path.getmtime(os.path.join(HERE, "..", "include", "vyre_b200.h")))
    m = max(m, os.path.getmtime(os.path.abspath(__file__)))
    return m


def _compile(src: str, flags: list[str], force: bool, hdr_mtime: float) -> tuple[str, str]:
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ_DIR, src.replace("/", "_") + ".o")
    if (not force and os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(path)
            and os.path.getmtime(obj) >= hdr_mtime):
        return obj, ""
    cmd = [nvcc(), *_host_compiler_flags(), *ARCH, *COMMON, *flags, "-x", "cu", "-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr = _deps_mtime()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        futs = {ex.submit(_compile, s, f, force, hdr): s for s, f in SOURCES.items()}
        objs, logs = [], {}
        for fut in concurrent.futures.as_completed(futs):
            obj, log = fut.result()
            objs.append(obj)
            if log:
                logs[futs[fut]] = log
    if logs:
        with open(os.path.join(OUT_DIR, "ptxas.log"), "a") as fh:
            for s, log in logs.items():
                fh.write(f"==== {s}\n{log}\n")
        if verbose:
            for s, log in logs.items():
                print(f"==== {s}\n{log}")
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = [nvcc(), *_host_compiler_flags(), *ARCH, "-shared", "-o", LIB, *sorted(objs), "-lcudart_static", "-ldl",
               "-lpthread", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
