"""Build libmetallic_cuda.so (sm_100a) in-tree with nvcc.

    python test-burn_b200/build.py [--force] [--verbose]

The library is plain CUDA/C++ behind a C ABI (include/metallic_cuda.h); it links
the static CUDA runtime and nothing from PyTorch.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
OUT = HERE / "libmetallic_cuda.so"
OBJ = HERE / "build"
SOURCES = [
    HERE / "csrc" / "context.cu",
    HERE / "csrc" / "kv_append.cu",
    HERE / "csrc" / "fused_qkv_tc.cu",
    HERE / "csrc" / "decode.cu",
    HERE / "csrc" / "decode_kv8.cu",
    HERE / "csrc" / "prefill.cu",
    HERE / "csrc" / "prefill_tc.cu",
    HERE / "csrc" / "attention_api.cu",
    HERE / "csrc" / "peer_exchange.cu",
    HERE / "host" / "host_logic.cpp",
    HERE / "host" / "prefix_cache.cpp",
]
HEADERS = [HERE / "csrc" / "internal.hpp", HERE / "csrc" / "ptx.cuh", HERE / "csrc" / "tcgen05.cuh", HERE / "csrc" / "append.cuh", HERE / "csrc" / "push.cuh", ROOT / "include" / "metallic_cuda.h"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
EXTRA = os.environ.get("MF_EXTRA_NVCC_FLAGS", "").split()
FLAGS = EXTRA + ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-x", "cu"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for src in SOURCES:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *HEADERS]):
            cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            for r in ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed: " + " ".join(r.args))
    objs = [OBJ / (s.stem + ".o") for s in SOURCES]
    if force or jobs or _stale(OUT, objs):
        cmd = [NVCC, "-shared", "-o", str(OUT), *map(str, objs), "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
