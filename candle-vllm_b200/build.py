"""Builds libb200backend.so (the C-ABI library) with nvcc for sm_100a, in-tree.

``python candle-vllm_b200/build.py [--force] [--verbose]``.  Each ``csrc/*.cu`` is compiled to an
object (parallel), then linked into ``candle-vllm_b200/libb200backend.so`` (static cudart, so the
library has no run-time dependency beyond the driver).
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
SO = os.path.join(HERE, "libb200backend.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CCBIN = "/usr/bin/g++"

FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
         "-ccbin", CCBIN, "-Xcompiler", "-fPIC,-fvisibility=default", "--expt-relaxed-constexpr",
         "-I", os.path.join(HERE, "..", "include")]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


# Source groups that link into a library of their own: what one model family needs, so that a first start from a source-only checkout
# compiles that and nothing else.  "ragged" = the ragged-step decoders (seq_ops.py): error state, both linear kernels, norms /
# activations, recurrent, attention and latent-attention mixers, routed experts, argmax.
GROUPS = {"ragged": ["lib", "linear_generic", "dense_gemm", "norm_act", "gated_delta", "attention_varlen", "attention_prefill", "attention_decode", "attention_generic",
                     "attention_api", "elementwise"],
          # latent attention + routed experts: both linear kernels (the tcgen05 one also in its grouped form), norms, the latent mixers incl. the
          # split-KV latent decode kernel, the expert kernels, argmax
          "latent": ["lib", "linear_generic", "dense_gemm", "norm_act", "latent_attention", "moe_ragged", "mla", "elementwise"],
          # state-space / linear-attention mixers beside softmax attention, with dense or routed feed-forwards: both linear kernels (the tcgen05 one also
          # grouped), norms, the recurrences, the SIMT attention over the paged cache and the tensor-core prefill and split-KV decode kernels it hands 128-wide
          # heads to, the expert kernels
          "hybrid": ["lib", "linear_generic", "dense_gemm", "norm_act", "linear_recurrence", "attention_varlen", "attention_prefill", "attention_decode",
                     "attention_generic", "attention_api", "moe_ragged", "elementwise"],
          # softmax attention with a sink, attention without softmax over a window plus pooled blocks, latent attention, ungated routed experts: both linear
          # kernels (the tcgen05 one also grouped), norms, the per-head preparation and pooled-cache kernels, the SIMT attention over the paged cache and the
          # tensor-core kernels it hands 128-wide heads to, the latent mixers incl. the split-KV latent decode kernel, the expert kernels
          "window": ["lib", "linear_generic", "dense_gemm", "norm_act", "attention_window", "attention_varlen", "attention_prefill", "attention_decode",
                     "attention_generic", "attention_api", "latent_attention", "mla", "moe_ragged", "elementwise"]}


def so_path(group=None) -> str:
    return SO if group is None else os.path.join(HERE, f"libb200backend.{group}.so")


def build(force: bool = False, verbose: bool = False, group=None) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    if group is not None:
        srcs = [os.path.join(CSRC, n + ".cu") for n in GROUPS[group]]
    SO = so_path(group)
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    jobs = []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        if force or _newer(o, [s] + hdrs):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append((s, cmd))

    def run(job):
        s, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for s, r in ex.map(run, jobs):
                if verbose or r.returncode:
                    sys.stderr.write(f"== {os.path.basename(s)}\n{r.stdout}{r.stderr}\n")
                if r.returncode:
                    raise RuntimeError(f"nvcc failed on {s}")
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or _newer(SO, objs):
        tmp = f"{SO}.{os.getpid()}.tmp"
        cmd = [NVCC, "-shared", "-o", tmp, "-ccbin", CCBIN, "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "static"] + objs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
        os.replace(tmp, SO)              # a reader never sees a half-written library
    return SO


if __name__ == "__main__":
    grp = next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--group=")), None)
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, group=grp))
