"""Build the in-tree shared libraries (sm_100a only) with nvcc.

`python -m promptcache_b200.build` or `build()` builds libpromptcache_b200.so (the prompt-cache hot path);
`build_seq()` builds libpromptcache_b200_seq.so (the sequence-batch kernels: slot-pool attention, recurrent scan, gated
norms), which is all a model of that family needs -- a first run in a fresh checkout compiles only the library its model
loads.  nvcc cross-compiles without a GPU.  The .so files are git-ignored but travel to the GPU box with the snapshot.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpromptcache_b200.so")
STAMP = os.path.join(HERE, ".libpromptcache_b200.stamp")
SOURCES = ["api.cu", "splice.cu", "rope_append.cu", "attn_simt.cu", "attn_combine.cu", "attn_tc_small.cu", "attn_tc2.cu", "support.cu", "linear_small.cu", "linear_chain.cu"]
HEADERS = [os.path.join(CSRC, "pc_common.cuh"), os.path.join(CSRC, "linear_common.cuh"), os.path.join(HERE, "..", "include", "promptcache_b200.h")]
SEQ_LIB = os.path.join(HERE, "libpromptcache_b200_seq.so")
SEQ_STAMP = os.path.join(HERE, ".libpromptcache_b200_seq.stamp")
SEQ_SOURCES = ["seq_norms.cu", "seq_attn.cu", "seq_attn_tc.cu", "seq_mlstm.cu", "seq_mlstm_chunk.cu", "seq_linear.cu", "seq_canon.cu", "seq_rope.cu", "seq_moe.cu", "seq_moe_gemm.cu",
               "seq_gla.cu", "seq_latent.cu", "seq_attn_latent.cu", "seq_layernorm.cu", "seq_gru.cu", "seq_attn_talk.cu", "seq_attn_talk_tc.cu"]
SEQ_HEADERS = [os.path.join(CSRC, "seq_common.cuh"), os.path.join(CSRC, "seq_mma.cuh"), os.path.join(HERE, "..", "include", "promptcache_b200_seq.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; promptcache_b200 needs the CUDA 12.9 toolchain to build")


def _digest(sources=None, headers=None) -> str:
    h = hashlib.sha256()
    for f in [os.path.join(CSRC, s) for s in (sources or SOURCES)] + (headers or HEADERS) + [os.path.abspath(__file__)]:
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    return _build(LIB, STAMP, SOURCES, HEADERS, force, verbose)


def build_seq(force: bool = False, verbose: bool = False) -> str:
    return _build(SEQ_LIB, SEQ_STAMP, SEQ_SOURCES, SEQ_HEADERS, force, verbose)


def _build(LIB: str, STAMP: str, SOURCES, HEADERS, force: bool, verbose: bool) -> str:
    extra = os.environ.get("PC_NVCC_EXTRA", "").split()  # experiments only (e.g. -DPC_EXP_...); empty in normal builds
    digest = _digest(SOURCES, HEADERS) + "|" + " ".join(extra)
    if not force and os.path.exists(LIB) and os.path.exists(STAMP):
        with open(STAMP) as fh:
            if fh.read().strip() == digest:
                return LIB
    nvcc = _nvcc()
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for s in SOURCES:
        obj = os.path.join(HERE, "build", s.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, s), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for s, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            failed.append(s)
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    tmp = LIB + f".{os.getpid()}.tmp"  # linked beside the target and renamed: a concurrent first run never loads half a file
    link = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static",
            "-Xcompiler", "-fPIC"]
    subprocess.run(link, check=True)
    os.replace(tmp, LIB)
    # a shared library links with unresolved symbols; make them a build error (dlopen resolves everything eagerly)
    import ctypes
    ctypes.CDLL(LIB, mode=ctypes.RTLD_LOCAL | os.RTLD_NOW)
    with open(STAMP, "w") as fh:
        fh.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_seq(force="--force" in sys.argv, verbose="-v" in sys.argv))
