"""In-tree build of the C-ABI CUDA libraries (sm_100a).

Separate libraries, so that a process compiles only what its model needs:
  core  omchat_b200/_lib/libomchat_b200.so      tcgen05 GEMMs, flash attention, the persistent decode kernel, the vision tower's
                                                row kernels, preprocessing (include/omchat_b200.h)
  seq   omchat_b200/_lib/libomchat_b200_seq.so  sequence-step kernels: latent and windowed attention over a paged cache, fp32
                                                residual row kernels, the score-corrected router, the any-shape linear layer,
                                                short convolutions and linear-state recurrences over state slots
                                                (include/omchat_b200_seq.h); built with IEEE division / square root / exp
  dense omchat_b200/_lib/libomchat_b200_dense.so  the GEMM / row-kernel / sampling subset of core, for a process that has no core
                                                library (lib.load_dense() prefers a built core library, which has the same symbols)
`python -m omchat_b200.build [core|seq ...]` or `__graft_entry__.build()` builds both; nvcc cross-compiles without a GPU. The
libraries are git-ignored but travel to the GPU box with the repo snapshot. `ensure(name)` builds one library on demand (first
use in a fresh checkout).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "_lib"
LIB = LIBDIR / "libomchat_b200.so"
SEQ_LIB = LIBDIR / "libomchat_b200_seq.so"
SOURCES = ["capi.cu", "gemm_sm100.cu", "gemm_skinny.cu", "gemm_stream.cu", "gemv.cu", "rowops.cu", "attention.cu", "attention_sm100.cu", "decode_mega.cu", "preprocess.cu", "model_capi.cu", "moe.cu"]
SEQ_SOURCES = ["capi.cu", "linear_any.cu", "rownorm32.cu", "latent_attention.cu", "router_moe.cu", "state_mixers.cu", "window_attention.cu"]
DENSE_LIB = LIBDIR / "libomchat_b200_dense.so"
DENSE_SOURCES = ["capi.cu", "gemm_sm100.cu", "gemm_skinny.cu", "rowops.cu", "moe.cu"]  # a subset of SOURCES that links on its own
BASE_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
NVCC_FLAGS = BASE_FLAGS + ["--use_fast_math"]
NVCC_FLAGS += os.environ.get("OMCHAT_B200_NVCC_EXTRA", "").split()  # e.g. -DOMC_MEGA_DETAIL=1 for tools/prof_mega.py
COMPONENTS = {
    "core": (LIB, SOURCES, NVCC_FLAGS),
    "seq": (SEQ_LIB, SEQ_SOURCES, BASE_FLAGS),  # no fast-math: its fp32 mode is true fp32
    # the core library's GEMMs (tcgen05, skinny, grouped), row kernels and sampling alone: what a sequence-step model needs of it
    # when a layer is wide enough for the tensor-core GEMMs and no full core library has been built
    "dense": (DENSE_LIB, DENSE_SOURCES, NVCC_FLAGS),
}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _headers():
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))


def build_component(name: str, force: bool = False, verbose: bool = False) -> Path:
    lib, sources, flags = COMPONENTS[name]
    LIBDIR.mkdir(exist_ok=True)
    objdir = LIBDIR if name == "core" else LIBDIR / name
    objdir.mkdir(exist_ok=True)
    stamp = LIBDIR / ("build.sha256" if name == "core" else f"build_{name}.sha256")
    digest = _digest([CSRC / s for s in sources] + _headers(), flags)
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == digest:
        return lib
    nvcc = _nvcc()

    def compile_one(src: str):
        obj = objdir / (src.replace(".cu", ".o"))
        cmd = [nvcc, *flags, "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (objdir / (src + ".log")).write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(sources)) as ex:
        objs = list(ex.map(compile_one, sources))
    tmp = lib.with_suffix(f".so.tmp{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)  # a concurrent process never sees a half-written library
    stamp.write_text(digest)
    return lib


def ensure(name: str) -> Path:
    """The library of component `name`, built first if it is missing or older than its sources."""
    return build_component(name)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Builds the seq and the core library (the dense subset is built on demand only); returns the core library's path."""
    build_component("seq", force, verbose)
    return build_component("core", force, verbose)


if __name__ == "__main__":
    names = [a for a in sys.argv[1:] if a in COMPONENTS]
    if names:
        for n in names:
            print(build_component(n, force="--force" in sys.argv, verbose="-v" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
