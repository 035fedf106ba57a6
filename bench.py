#!/usr/bin/env python
"""bench.py -- headline benchmark: decode tokens/s, Llama-3-8B Q4_K (GGUF), batch 32, ctx 4096 -> 5120,
paged KV (bf16), on N B200s (tensor parallel = N), synthetic weights / KV / block tables.

One "step" = one decode step of the whole batch through the hot path (32 decoder layers of
quantised GEMMs + paged attention + lm_head + greedy argmax).  Prints ONE JSON line (see the
driver contract):  value = tokens/s with all inputs resident in HBM (CUDA-graph replay, metadata
advanced on the device); e2e = the same through the public host API (prepare_decode on the host,
H2D metadata copies, D2H token read-back inside the timed region); roofline = the paged-attention
decode kernel (HBM-bound) measured live with CUDA events; cpu_baseline = the C port of the
reference's CPU/GGML arithmetic (oracle/cpu_ref.c) on a bounded sample.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
  torchrun --nproc-per-node N bench.py --gpus N ...      (one rank per GPU; TP = N)
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "decode tokens/s Llama-3-8B Q4_K batch=32"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=4096, help="context length at the first decode step")
    ap.add_argument("--max-ctx", type=int, default=5120)
    ap.add_argument("--layers", type=int, default=32, help="debug only: fewer layers => number is INVALID")
    ap.add_argument("--kv", default=None, choices=["bf16", "fp8"])
    ap.add_argument("--config", default="q4k", choices=["q4k", "dense_bf16", "gptq_fp8kv"],
                    help="q4k = the metric (BASELINE config: Llama-3-8B Q4_K GGUF); dense_bf16 = BASELINE config 2 (Llama-3-8B BF16); "
                         "gptq_fp8kv = BASELINE config 3 (GPTQ/Marlin int4 + FP8 KV).  The extra configs are single-GPU.")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=20.0)
    ap.add_argument("--parity-steps", type=int, default=3, help="decode steps compared against a TP=1 engine before timing (0 = off)")
    ap.add_argument("--arch", default="llama", choices=["llama", "gobesun", "guvusun", "panarax", "dofevik"],
                    help="llama = the metric (default, unchanged).  gobesun = prefill / decode throughput of the Gobesun decoder at layer sizes of real "
                         "models (random weights), beside a dense bf16 Llama of equal width / heads / ff / depth, with a per-kernel roofline table; "
                         "one JSON line, single GPU.  guvusun / panarax / dofevik = the same for those decoders (panarax beside a Gobesun, dofevik beside a Guvusun of "
                         "equal size).")
    ap.add_argument("--arch-sizes", default="w2048,w4096")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# CPU arm: C port of the reference's CPU/GGML path (oracle/cpu_ref.c) on a bounded sample
# ------------------------------------------------------------------------------------------------
def cpu_sample_setup(batch: int, ctx: int):
    """Times ONE decoder layer (Q4_K x Q8_K integer-dot GEMMs + f32 paged attention over a bf16
    cache) for `batch` sequences at context `ctx`, plus a row slice of the Q6_K lm_head, and scales to
    the full model: t_step = 32 * t_layer + t_head * (vocab / rows).  Returns (tokens/s, info)."""
    import ctypes as C
    from oracle import cpu_ref
    from oracle import attention as OA
    lib = cpu_ref.lib()
    rng = np.random.default_rng(0)
    H, heads, kvh, hd, F, V, bs = 4096, 32, 8, 128, 14336, 128256, 64
    nblk = -(-(ctx + 1) // bs)

    def q4k(n, k):
        b = rng.integers(0, 256, (n * (k // 256), 144), dtype=np.uint8)
        b[:, 0:2] = (rng.uniform(0.5, 2, len(b)) * 2.0 ** -14).astype(np.float16).view(np.uint8).reshape(-1, 2)
        b[:, 2:4] = (rng.uniform(0.5, 2, len(b)) * 7.5 * 2.0 ** -14).astype(np.float16).view(np.uint8).reshape(-1, 2)
        return b.reshape(-1)

    ws = dict(wq=q4k(heads * hd, H), wk=q4k(kvh * hd, H), wv=q4k(kvh * hd, H), wo=q4k(H, heads * hd),
              w1=q4k(F, H), w2=q4k(H, F), w3=q4k(F, H))
    norms = dict(attn_norm=rng.uniform(0.5, 1.5, H).astype(np.float32), ffn_norm=rng.uniform(0.5, 1.5, H).astype(np.float32))
    nb = batch * nblk
    kc = rng.integers(0, 2 ** 16, (nb, bs, kvh, hd), dtype=np.uint16) & 0xBFFF     # finite bf16 bit patterns
    vc = rng.integers(0, 2 ** 16, (nb, bs, kvh, hd), dtype=np.uint16) & 0xBFFF
    kc = (kc & 0x807F) | 0x3F00; vc = (vc & 0x807F) | 0x3F00                         # |x| in [0.5, 1)
    bt = rng.permutation(nb).reshape(batch, nblk).astype(np.uint32)
    ctx_lens = np.full(batch, ctx + 1, np.uint32)
    pos = np.full(batch, ctx, np.int64)
    slots = (bt[:, ctx // bs].astype(np.int64) * bs + ctx % bs)
    cos, sin = OA.rope_tables(hd, ctx + 8, 500000.0)
    cfg = cpu_ref.RefCfg(H, heads, kvh, hd, F, bs, nblk, 1e-5)
    layer = cpu_ref.RefLayer(*[a.ctypes.data for a in (norms["attn_norm"], norms["ffn_norm"], ws["wq"], ws["wk"], ws["wv"],
                                                       ws["wo"], ws["w1"], ws["w2"], ws["w3"])])
    x = rng.standard_normal((batch, H)).astype(np.float32)
    lib.ref_layer_scratch_floats.restype = C.c_size_t
    scratch = np.empty(lib.ref_layer_scratch_floats(C.byref(cfg), batch), np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)

    def one_layer():
        t0 = time.perf_counter()
        rc = lib.ref_llama_layer_decode(C.byref(cfg), C.byref(layer), p(x), batch, p(pos), p(slots), p(bt), p(ctx_lens),
                                        p(kc), p(vc), p(cos), p(sin), p(scratch))
        assert rc == 0
        return time.perf_counter() - t0

    rows = 8192
    w6 = rng.integers(0, 256, (rows * (H // 256), 210), dtype=np.uint8)
    w6[:, 208:210] = (rng.uniform(0.5, 2, len(w6)) * 2.0 ** -16).astype(np.float16).view(np.uint8).reshape(-1, 2)
    w6 = w6.reshape(-1)
    xh = rng.standard_normal((batch, H)).astype(np.float32)

    keep = (ws, norms, kc, vc, bt, ctx_lens, pos, slots, cos, sin, x, scratch, layer, cfg)   # raw pointers inside

    # ONE thread count, chosen by rule and printed (r01 re-calibrated per run and moved 4x between boxes): the physical cores this
    # process may use = half the schedulable logical CPUs (SMT pairs; on the GPU box 128 logical threads ran 10x slower than 64)
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    n_thr = max(1, avail // 2) if avail >= 16 else max(1, avail)
    cpu_ref.set_num_threads(n_thr)
    one_layer()                                                    # warm the team and the page tables (not counted)

    def step():
        """one decode step of the whole model, nothing extrapolated: 32 decoder-layer passes (one layer's weights and KV reused -- 123 MB +
        1 GB per pass, far beyond the CPU caches) + the Q6_K lm_head over all `V` rows in slices of `rows`.  Returns seconds."""
        assert keep
        t_layers = sum(one_layer() for _ in range(32))
        t0 = time.perf_counter()
        done = 0
        while done < V:
            r = min(rows, V - done)
            cpu_ref.qmatmul_q8k(xh, w6[:r * (H // 256) * 210], 14, r, H)
            done += r
        t_head = time.perf_counter() - t0
        return t_layers + t_head, t_layers / 32, t_head

    info = dict(cores=cpu_ref.num_threads(), kind="port",
                sample=f"per step: all 32 decoder layers (batch {batch}, ctx {ctx}, Q4_K x Q8_K int dot + f32 paged attention; the "
                       f"weights and KV of one layer are reused for every pass) + the full {V}-row Q6_K lm_head -- a complete decode step, "
                       f"nothing scaled; {n_thr} threads = "
                       f"{'half the ' + str(avail) + ' schedulable logical CPUs' if avail >= 16 else 'all schedulable CPUs'}; mean over samples")
    return step, info


def cpu_decode_sample(batch: int, ctx: int, budget_s: float):
    step, info = cpu_sample_setup(batch, ctx)
    vals = []
    t_start = time.perf_counter()
    while len(vals) < 3 and (not vals or (time.perf_counter() - t_start) * (len(vals) + 1) / len(vals) < budget_s):
        vals.append(step()[0])
    mean = statistics.mean(vals)
    info = dict(info)
    info["sample"] += f"; {len(vals)} samples, mean {mean:.2f} s/step (min {min(vals):.2f}, max {max(vals):.2f})"
    return batch / mean, mean, info


def timed_window(args):
    """context lengths (including the decoded token) of the K timed steps: identical for both arms"""
    ctx0 = args.ctx + args.parity_steps
    return ctx0 + 1 + args.warmup + 1, ctx0 + 1 + args.warmup + args.steps


def workload_config(args, world: int, layers: int = 32) -> dict:
    """`config` of the JSON line -- the SAME dict from `--impl reference` and from the GPU arm (same workload, same window)."""
    first, last = timed_window(args)
    name = {"q4k": "Llama-3-8B Q4_K (lm_head Q6_K)", "dense_bf16": "Llama-3-8B BF16 (dense)",
            "gptq_fp8kv": "Llama-3-8B GPTQ int4 g128 (Marlin-prepared; lm_head Q6_K)"}[args.config]
    kv = args.kv or {"q4k": "bf16", "dense_bf16": "bf16", "gptq_fp8kv": "fp8"}[args.config]
    return {"workload": f"{name} decode, batch {args.batch}, ctx {first}->{last} of 4096->5120, block_size 64, {kv} paged KV, "
                        f"random non-contiguous block tables",
            "parallelism": f"tp{world}", "global_batch": args.batch, "layers": layers,
            "l2_policy": "inputs larger than L2 (KV 17+ GB and weights 4.4 GB streamed per step; 126 MB L2)"}


def run_reference(args):
    """--impl reference: the reference's CPU path (C port; the Rust reference cannot be built here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, info = cpu_sample_setup(args.batch, timed_window(args)[0])       # the first context of the timed window
    vals, t_begin = [], time.perf_counter()
    for i in range(args.warmup + args.steps):
        t_step, _, _ = step()
        if i >= args.warmup or (time.perf_counter() - t_begin) > 60:
            vals.append((args.batch / t_step, t_step))
        if vals and (time.perf_counter() - t_begin) > 170:       # keep the whole run within a few minutes (the line reports how many steps ran)
            break
    ms = statistics.mean(v[1] for v in vals) * 1e3                  # same statistic as the cpu_baseline leg: mean seconds per step
    tps = args.batch / (ms * 1e-3)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals),
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "q4_k weights x q8_k activations (int8 dot), f32 attention", "data": "synthetic",
            "config": workload_config(args, args.gpus),
            "note": "CPU arm (host cores only, rank 0): every step is a complete decode step of the same workload (one layer's weights / KV reused across the 32 layer passes)",
            "cpu_baseline": {"value": tps, "unit": UNIT, **info},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# clocks sampling during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.rows.append([c.strip() for c in ln.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 9 for i in range(4) if r[5 + i].lower().startswith("active")})
        pw = [float(r[3]) for r in self.rows if len(r) >= 9 and r[3].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": reasons}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
CONFIGS = {
    "q4k": dict(metric=METRIC, kv="bf16", dtype="f16 activations x q4_k/q6_k weights (fp32 accumulate), bf16 attention",
                name="Llama-3-8B Q4_K (lm_head Q6_K)"),
    "dense_bf16": dict(metric="decode tokens/s Llama-3-8B BF16 batch=32 (BASELINE config 2)", kv="bf16",
                       dtype="bf16 activations x bf16 weights (fp32 accumulate, tcgen05 dense GEMM), bf16 attention", name="Llama-3-8B BF16 (dense)"),
    "gptq_fp8kv": dict(metric="decode tokens/s Llama-3-8B GPTQ/Marlin int4 + FP8 KV batch=32 (BASELINE config 3)", kv="fp8",
                       dtype="f16 activations x int4 weights g128 (fp32 accumulate), f16 attention over e4m3 KV",
                       name="Llama-3-8B GPTQ int4 g128 (Marlin-prepared; lm_head Q6_K)"),
}


def run_b200(args):
    import torch
    import torch.distributed as dist
    import candle_vllm_b200 as pkg
    from candle_vllm_b200 import synthetic
    from candle_vllm_b200.distributed import Comm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N>1 must be launched with torchrun (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    comm = Comm(rank, world) if world > 1 else None

    conf = CONFIGS[args.config]
    if args.kv is None:
        args.kv = conf["kv"]
    if args.config != "q4k" and world > 1:
        raise SystemExit(f"bench.py --config {args.config} is a single-GPU configuration")
    B, bs = args.batch, 64
    K, W = args.steps, args.warmup
    PS = args.parity_steps
    args.max_ctx = max(args.max_ctx, args.ctx + 3 * (K + W) + PS + 16, 4608 + 2 * (K + W) + 16)      # room for every leg below
    blocks_per_seq = -(-args.max_ctx // bs)
    cfg = pkg.LlamaConfig(num_layers=args.layers, max_num_seqs=B, max_blocks_per_seq=blocks_per_seq, max_pos=args.max_ctx + 64,
                          block_size=bs)
    kv_dtype = pkg.DType.FP8_E4M3 if args.kv == "fp8" else pkg.DType.BF16
    num_blocks = B * blocks_per_seq + 16
    tables = synthetic.random_block_tables(B, blocks_per_seq, num_blocks, seed=2)
    tables_np = np.asarray(tables, np.int32)              # rectangular tables: prepare_decode's vectorised path
    stream = torch.cuda.Stream()

    def build(tp_rank, tp_world, nccl):
        """model + KV state for (tp_rank, tp_world): same seeds on every rank and for every tp_world, so a TP run and the TP = 1
        run see the same global weights and the same global KV cache (each rank holds its shard of both)."""
        if args.config == "dense_bf16":
            weights = synthetic.make_weights_16bit(cfg, dev, seed=0, dtype=torch.bfloat16)
        elif args.config == "gptq_fp8kv":
            weights, _ = synthetic.make_weights_gptq(cfg, dev, seed=0, group_size=128, dtype=torch.float16, with_oracle=False)
        else:
            weights = synthetic.make_weights(cfg, dev, seed=0, tp_rank=tp_rank, tp_world=tp_world)
        eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim,
                              pkg.CacheConfig(bs, num_blocks, kvcache_dtype="fp8" if args.kv == "fp8" else "auto"),
                              device=dev, num_shards=tp_world)
        synthetic.fill_kv_cache(eng.gpu_cache, seed=1, tp_rank=tp_rank, tp_world=tp_world, num_kv_heads=cfg.num_kv_heads)
        torch.cuda.synchronize()
        model = pkg.GGUFLLaMa(cfg, weights, eng.gpu_cache, kv_dtype=kv_dtype, tp_rank=tp_rank, tp_world=tp_world, nccl_comm=nccl,
                              stream=stream, rope_neox=args.config != "q4k")
        return model, eng, weights

    model, eng, weights = build(rank, world, comm.handle.value if comm else None)
    inboxes = None
    if world > 1:
        # row-parallel all-reduce + residual add + next RMSNorm as one kernel over NVLink peer memory (falls back to NCCL if
        # CUDA IPC is not available between the ranks, or with B200_TP_NCCL=1)
        from candle_vllm_b200.distributed import PeerInboxes
        inboxes = PeerInboxes(model, rank, world)
        if not inboxes.active and rank == 0:
            print(f"[bench] peer inboxes inactive, all-reduce through NCCL: {inboxes.error or 'B200_TP_NCCL set'}", file=sys.stderr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    toks0 = [int(t) for t in np.random.default_rng(3).integers(0, cfg.vocab, B)]

    # ---- (0) parity, OUTSIDE every timed region: the first PS decode steps of this run (graph replay, fused all-reduce and
    # all) against the same steps of a TP = 1 engine with the same seeds on rank 0: greedy tokens and full-vocabulary logits.
    # At N = 1 the second engine runs eagerly (no graph) -- that leg checks graph capture / replay and bounds the run-to-run
    # spread of the red.add reductions.
    def parity_steps(mdl, want, forced=None):
        """PS decode steps; with `forced` (the reference's tokens, [PS, B]) step s + 1 consumes forced[s] instead of the engine's own
        argmax -- teacher forcing, so that a greedy near-tie that flips under the run-to-run noise of the fp32 reductions cannot
        make the later steps decode different sequences and every step's logits stay comparable"""
        lens, toks, out_t, out_l = np.full(B, args.ctx + 1), list(toks0), [], []
        for st in range(PS):
            nxt, lg = mdl.decode(pkg.prepare_decode(lens, toks, tables_np, bs), want_logits=want)
            out_t.append(np.asarray(nxt).copy()); out_l.append(lg)
            toks, lens = [int(t) for t in (nxt if forced is None else forced[st])], lens + 1
        return np.stack(out_t), out_l

    parity = None
    if PS > 0:
        ref_t = torch.zeros(PS, B, dtype=torch.int64, device=dev)
        ref_l = None
        if rank == 0:
            if world == 1:
                ref_model = pkg.GGUFLLaMa(cfg, weights, eng.gpu_cache, kv_dtype=kv_dtype, use_graph=False, stream=stream,
                                          rope_neox=args.config != "q4k")
                ref_eng = None                                      # same cache: the steps rewrite the same slots with the same values
            else:
                ref_model, ref_eng, ref_w = build(0, 1, None)
            t, ref_l = parity_steps(ref_model, True)
            ref_t.copy_(torch.from_numpy(t.astype(np.int64)))
            del ref_model
            if world > 1:
                del ref_eng, ref_w
            torch.cuda.empty_cache()
        if world > 1:
            dist.broadcast(ref_t, src=0)
        ref_t = ref_t.cpu().numpy()
        got_t, got_l = parity_steps(model, True, forced=ref_t)      # collective at N > 1 (logits all-gather)
        barrier()
        if rank == 0:
            scale = max(float(np.abs(l).max()) for l in ref_l)
            tol = 3e-2 if args.config == "dense_bf16" else 5e-3
            errs = [float(np.abs(a - b).max()) / scale for a, b in zip(got_l, ref_l)]
            err = max(errs)
            # a greedy token may differ only on a near-tie inside the logit error
            flips = mismatches = 0
            for st in range(PS):
                for b in np.nonzero(got_t[st] != ref_t[st])[0]:
                    mismatches += 1
                    margin = float(ref_l[st][b].max() - ref_l[st][b, got_t[st][b]])
                    flips += int(margin > 2 * err * scale + 1e-6)
            parity = {"steps": PS, "logits_max_err": err, "logits_max_err_per_step": errs,
                      "tokens_equal_tp1": mismatches == 0, "token_mismatches": mismatches,
                      "token_mismatches_beyond_logit_error": flips, "logit_scale": scale,
                      "reference": "TP=1 engine, same seeds, rank 0" + (" (eager, no CUDA graph)" if world == 1 else "")
                                   + "; teacher-forced: every step of both engines consumes the reference's tokens",
                      "tolerance": tol, "within_tolerance": bool(err < tol and flips == 0),
                      "tolerance_note": ("bf16 activations (relative step 3.9e-3) amplify the fp32 reduction-order difference between the two "
                                         "engines layer by layer" if args.config == "dense_bf16" else
                                         "fp16 activations; fp32 reduction order differs between the two engines "
                                         "(profiles/r02_rounding_floor.md)") + "; unit: fraction of max|logit|"}
            del ref_l
        barrier()

    # ---- (1) device-resident: metadata advanced on the device, graph replay only ----------------
    def resident_leg(ctx0):
        prep = pkg.prepare_decode([ctx0 + 1] * B, toks0, tables, bs)   # context INCLUDING the token being decoded
        model.decode(prep)                                     # loads the static buffers (captures the graph on first use)
        for _ in range(W):
            model.decode_resident(B, advance=True)
        barrier()
        sampler = ClockSampler(local); sampler.start()
        l0 = model.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(K):
                model.decode_resident(B, advance=True)
            e1.record(stream)
        barrier()
        ms_total = max_over_ranks(e0.elapsed_time(e1))
        return ms_total / K, sampler.stop(), model.kernel_launches() - l0, (ctx0 + 1 + W + 1, ctx0 + 1 + W + K)

    ms_step, clocks, launches, (ctx_first, ctx_last) = resident_leg(args.ctx + PS)
    assert (ctx_first, ctx_last) == timed_window(args)
    value = B / (ms_step * 1e-3)
    # the metric is quoted over ctx 4096 -> 5120 (mean 4608): the same leg centred on the mean context
    mid0 = max(args.ctx, 4608 - (W + K) // 2 - 1)
    ms_mid, clocks_mid, _, (mid_first, mid_last) = resident_leg(mid0)

    # ---- (2) end to end through the host API -------------------------------------------------------
    # over the SAME context window as `value` (ctx_first -> ctx_last), so that the two numbers differ by the host path only
    n_warm = min(W, 3)
    cur = ctx_first - n_warm
    nxt = model.read_next_tokens(B)
    h2d = B * (8 + 8 + 8 + 4) + B * blocks_per_seq * 4
    d2h = B * 4
    for _ in range(n_warm):
        prep = pkg.prepare_decode(np.full(B, cur), nxt, tables_np, bs)
        nxt, _ = model.decode(prep); cur += 1
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record(stream)
    for _ in range(K):
        prep = pkg.prepare_decode(np.full(B, cur), nxt, tables_np, bs)              # host: block tables, slots
        nxt, _ = model.decode(prep); cur += 1                                       # H2D + replay + D2H + sync
    e1.record(stream)
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), wall_ms)) / K
    e2e = B / (e2e_ms * 1e-3)

    # ---- (3) rooflines: paged-attention decode alone per layer; the weight stream of all projections alone ---------
    roof = attention_roofline(pkg, model, cfg, eng, B, cur, tables, world, stream, dev)
    roof_gemm = gemm_roofline(model, cfg, B, world, stream, args.config)
    peer_ar = inboxes is not None and inboxes.active
    if inboxes is not None:
        timed_out = inboxes.timed_out()
        inboxes.close()                            # collective (barrier): before any rank leaves
        if timed_out:
            raise SystemExit("bench: the fused all-reduce timed out on a peer -- numbers invalid")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    src = "MEASURED_PEAKS.json hbm_gbs (measured copy bandwidth)" if peaks else "fallback 6.65 TB/s"
    roof.update(peak=hbm_peak, peak_source=src, frac=roof["achieved"] / hbm_peak)
    roof_gemm.update(peak=hbm_peak, peak_source=src, frac=roof_gemm["achieved"] / hbm_peak)
    line = {"metric": conf["metric"], "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": conf["dtype"], "data": "synthetic",
            "config": workload_config(args, world, cfg.num_layers),
            "all_reduce": None if world == 1 else ("fused all-reduce + add + norm over NVLink peer memory" if peer_ar else "NCCL all-reduce"),
            "value_mean_ctx": {"value": B / (ms_mid * 1e-3), "unit": UNIT, "ms_per_step": ms_mid, "ctx": f"{mid_first}->{mid_last}",
                               "note": "same leg centred on the metric's mean context 4608 (attention bytes +12 % over ctx 4096)",
                               "clocks": clocks_mid},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ctx": f"{cur - K}->{cur - 1}",
                    "api": "prepare_decode (host) + GGUFLLaMa.decode -> b200_llama_decode (C ABI, host buffers)"},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "roofline_gemm": roof_gemm}
    if parity is not None:
        line["parity"] = parity
    if cfg.num_layers != 32:
        line["invalid"] = "debug run with fewer layers"
    if not args.no_cpu_baseline and world == 1 and args.config == "q4k":      # the CPU arm is the reference's GGUF/GGML path
        tps, t_step, info = cpu_decode_sample(B, timed_window(args)[0], args.cpu_seconds)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, **info}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def ncu_traffic(csv_name: str, kernel_substr: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of the first launch of `kernel_substr` in a TRACKED `ncu --page raw --csv`
    export under profiles/ (None when the file or the metrics are missing): roofline.traffic is computed, never hard-coded."""
    import csv
    path = os.path.join(ROOT, "profiles", csv_name)
    try:
        rows = list(csv.reader(open(path, newline="")))
    except OSError:
        return None, None
    hdr = next((r for r in rows if "Kernel Name" in r), None)
    if hdr is None:
        return None, None
    ik = hdr.index("Kernel Name")
    units = rows[rows.index(hdr) + 1]
    def col(name):
        return hdr.index(name) if name in hdr else None
    ir, iw = col("dram__bytes_read.sum"), col("dram__bytes_write.sum")
    if ir is None or iw is None:
        return None, None
    mult = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    for r in rows[rows.index(hdr) + 2:]:
        if len(r) > max(ik, ir, iw) and kernel_substr in r[ik]:
            try:
                rd = float(r[ir].replace(",", "")) * mult.get(units[ir], 1.0)
                wr = float(r[iw].replace(",", "")) * mult.get(units[iw], 1.0)
                return rd + wr, os.path.join("profiles", csv_name)
            except ValueError:
                return None, None
    return None, None


def gemm_roofline(model, cfg, B, world, stream, config="q4k"):
    """The weight stream alone: every quantised projection of every layer + the lm_head + the small ops between them, without
    RoPE / cache write / attention (b200_llama_linear_chain), timed eagerly with CUDA events on the launching stream.  4.36 GB
    of weights per pass at TP = 1: far beyond the 126 MB L2."""
    import torch
    H, F, V = cfg.hidden, cfg.ffn, cfg.vocab
    qd, kd = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    params = (H * (qd + 2 * kd) + qd * H + 3 * H * F) * cfg.num_layers
    if config == "dense_bf16":
        alg = (params + V * H) * 2
    elif config == "gptq_fp8kv":
        alg = params // 2 + params // 128 * 2 + V * H * 210 // 256        # int4 + one f16 scale per 128 weights; lm_head Q6_K
    else:
        alg = (params * 144 // 256 + V * H * 210 // 256) // world
    with torch.cuda.stream(stream):
        for _ in range(3):
            model.linear_chain(B)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        stream.synchronize()
        e0.record(stream)
        for _ in range(reps):
            model.linear_chain(B)
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"kernel": "all quantised projections of one decode step (QKV, wo, gate|up, w2 per layer + lm_head) incl. norm / SiLU between them, eager launches",
            "bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes_per_launch": alg,
            "ms_per_launch": ms, "launch": f"one pass over all layers (weights {alg / 1e9:.2f} GB on this rank)",
            "traffic": None}


def attention_roofline(pkg, model, cfg, eng, B, ctx, tables, world, stream, dev):
    """Times PagedAttention decode alone (all layers round-robin, so every launch streams a different
    layer's KV: 0.5+ GB per launch >> 126 MB L2) with CUDA events on the launching stream."""
    import torch
    heads_l = cfg.num_heads // world
    kv_l = max(cfg.num_kv_heads // world, 1)
    attn = pkg.PagedAttention(heads_l, cfg.head_dim, cfg.head_dim ** -0.5, kv_l, fp8_kvcache=eng.dtype == torch.uint8)
    prep = pkg.prepare_decode([ctx] * B, [0] * B, tables, cfg.block_size)
    bt = np.zeros((B, cfg.max_blocks_per_seq), np.int32); bt[:, :prep["block_tables"].shape[1]] = prep["block_tables"]
    with torch.cuda.stream(stream):
        meta = pkg.InputMetadata(False, torch.zeros(0, dtype=torch.int64, device=dev), torch.from_numpy(bt).to(dev),
                                 torch.from_numpy(prep["context_lens"]).to(dev))
        q = torch.randn((B, heads_l, cfg.head_dim), device=dev, dtype=torch.float32).to(torch.bfloat16)
        for l in range(min(3, cfg.num_layers)):
            attn.forward(q, None, None, None, eng.gpu_cache[l][0], eng.gpu_cache[l][1], meta, out_dtype=torch.float16)
        reps = max(cfg.num_layers, 32)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def run_all():
            for i in range(reps):
                k, v = eng.gpu_cache[i % cfg.num_layers]
                attn.forward(q, None, None, None, k, v, meta, out_dtype=torch.float16)

        # the launches are captured once and replayed: at 50-100 us per launch an eager Python loop would measure the interpreter
        graph, how = None, "CUDA-graph replay of the launches"
        try:
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                run_all()
            graph.replay()                                   # warm replay
        except Exception as exc:                             # capture unavailable: eager launches (an upper bound on the kernel time)
            graph, how = None, f"eager launches ({type(exc).__name__})"
        stream.synchronize()
        e0.record(stream)
        if graph is not None:
            graph.replay()
        else:
            run_all()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    esz = eng.gpu_cache[0][0].element_size()
    kv_bytes = B * ctx * 2 * kv_l * cfg.head_dim * esz
    io_bytes = 2 * B * heads_l * cfg.head_dim * 2
    alg = kv_bytes + io_bytes
    return {"kernel": "paged_attention_decode (one layer: split-KV kernel + merge)", "bound": "hbm",
            "achieved": alg / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes_per_launch": alg,
            "ms_per_launch": ms, "ctx": ctx, "timed_as": how,
            # dram__bytes_read + dram__bytes_write of ONE `ncu --set full` capture of this kernel inside this benchmark, parsed
            # from the tracked raw export (profiles/); only quoted for the configuration it was captured on
            **traffic_fields(world, B, esz)}


def traffic_fields(world, B, esz):
    if not (world == 1 and B == 32):
        return {"traffic": None}
    if esz == 1:                                  # FP8 KV
        t, src = ncu_traffic("r02_attention_decode_fp8_raw.csv", "paged_attn_decode_kernel")
    else:
        t, src = ncu_traffic("r02_attention_decode_raw.csv", "paged_attn_decode_kernel")
        if not t:
            t, src = ncu_traffic("r01_attention_decode_raw.csv", "paged_attn_decode_kernel")
    return {"traffic": t, "traffic_source": src} if t else {"traffic": None, "traffic_source": "no tracked ncu export found"}


# ------------------------------------------------------------------------------------------------
# --arch gobesun: the new decoder beside the closest existing model at equal size
# ------------------------------------------------------------------------------------------------
ARCH_SIZES = {
    "w2048": dict(width=2048, heads=16, kv=4, ff=5632, vocab=32000, layers=8, chunk=2048),
    "w4096": dict(width=4096, heads=32, kv=8, ff=11008, vocab=32000, layers=4, chunk=2048),
}


def llama_beside(pkg, S, BK, z, hd, P, B, CTX, K, W, blocks_per, toks, timed, dev):
    """The dense bf16 Llama of the given width / heads / ff / depth: (prefill seconds per P-token prompt, decode seconds per step of B tokens at
    context CTX, per-kernel prefill times).  Decode runs on its C++ engine; prefill is the same layer written with the framework's operators."""
    import torch
    from candle_vllm_b200.inputs import prepare_prompt, to_device
    bf = torch.bfloat16
    D, H, G, ff, V, NL = z["width"], z["heads"], z["kv"], z["ff"], z["vocab"], z["layers"]
    # ---- Llama of equal size ---------------------------------------------------------------------------------------------------
    lcfg = pkg.LlamaConfig(hidden=D, num_layers=NL, num_heads=H, num_kv_heads=G, head_dim=hd, ffn=ff, vocab=V, rms_eps=1e-5, rope_theta=1e6,
                           max_pos=P + 64, block_size=64, max_num_seqs=B, max_blocks_per_seq=blocks_per)
    lw = S.make_weights_16bit(lcfg, dev, seed=0, dtype=bf)
    nblk = max(B * blocks_per, P // 64 + 1)
    eng = pkg.CacheEngine(NL, G, hd, pkg.CacheConfig(64, nblk), device=dev)
    S.fill_kv_cache(eng.gpu_cache, seed=1)
    lm = pkg.GGUFLLaMa(lcfg, lw, eng.gpu_cache, kv_dtype=pkg.DType.BF16, rope_neox=True)
    tables = S.random_block_tables(B, blocks_per, nblk, seed=2)
    prep = pkg.prepare_decode([CTX + 1] * B, toks[:B], tables, 64)
    lm.decode(prep)
    l_dec = timed(lambda: lm.decode_resident(B, advance=True), K, W)
    # prefill: the same layer written with the framework's operators (the decode engine has no prompt path of its own)
    lk = {}
    pp = prepare_prompt([toks], [list(range(P // 64 + 1))], 64)
    tok_d, pos_d, meta = to_device(pp, dev)
    inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = torch.arange(P + 64, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
    att = BK.PagedAttention(H, hd, hd ** -0.5, G)
    lin = {k: [BK.Linear(l[k]) for l in lw["layers"]] for k in ("wq", "wk", "wv", "wo", "w1", "w2", "w3")}
    lin_out = BK.Linear(lw["output"])
    emb = lw["tok_embeddings"]

    def op(key, fn, rec):
        if not rec:
            return fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); e0.record()
        r = fn()
        e1.record(); torch.cuda.synchronize()
        lk.setdefault(key, []).append(e0.elapsed_time(e1) * 1e-3)
        return r

    def l_prefill(rec=False):
        x = emb[tok_d]
        for i, l in enumerate(lw["layers"]):
            h = op("rms_norm", lambda: BK.rms_norm(x, l["attn_norm"], 1e-5, bf), rec)
            q = op(f"linear[{H * hd}x{D}]", lambda: lin["wq"][i].forward(h), rec)
            k = lin["wk"][i].forward(h); v = lin["wv"][i].forward(h)
            qf, kf = q.float().view(P, H, hd), k.float().view(P, G, hd)
            op("fused_rope", lambda: BK.fused_rope(qf, kf, cos, sin, pos_d, False), rec)
            kc, vc = eng.gpu_cache[i]
            qb, kb = qf.to(bf), kf.to(bf)
            op("reshape_and_cache", lambda: BK.reshape_and_cache(kb, v.view(P, G, hd), kc, vc, meta.slot_mapping), rec)
            a = op("paged_attention_prefill", lambda: att.forward(qb, None, None, None, kc, vc, meta), rec)
            x = x + lin["wo"][i].forward(a.view(P, H * hd)).float()
            h = BK.rms_norm(x, l["ffn_norm"], 1e-5, bf)
            g1 = op(f"linear[{ff}x{D}]", lambda: lin["w1"][i].forward(h), rec)
            u = lin["w3"][i].forward(h)
            m = op("silu_mul", lambda: BK.silu_mul(g1.float(), u.float(), torch.float32), rec).to(bf)
            x = x + op(f"linear[{D}x{ff}]", lambda: lin["w2"][i].forward(m), rec).float()
        return lin_out.forward(BK.rms_norm(x[-1:], lw["norm"], 1e-5, bf))
    l_pre = timed(l_prefill, 3, 2)
    l_prefill(True); lk.clear(); l_prefill(True)
    del lm, eng, lw, lin, lin_out
    torch.cuda.empty_cache()

    return l_pre, l_dec, lk


def run_gobesun(args):
    import torch
    import candle_vllm_b200 as pkg
    from candle_vllm_b200 import seq_ops as ops, synthetic as S
    from candle_vllm_b200 import backend as BK
    from candle_vllm_b200.engine import ModelRunner
    from candle_vllm_b200.gobesun import GobesunConfig, GobesunModel
    from candle_vllm_b200.inputs import prepare_prompt, to_device

    torch.cuda.set_device(0)
    dev = "cuda"
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else \
        {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}
    HBM, TC = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    K, W = max(args.steps, 1), max(args.warmup, 3)
    P, B, CTX, hd = 4096, 32, 1024, 128
    bf = torch.bfloat16
    l0 = pkg.lib().b200_total_kernel_launches()

    def timed(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3            # seconds per call

    sampler = ClockSampler(0); sampler.start()
    results = {}
    for name in [n for n in args.arch_sizes.split(",") if n in ARCH_SIZES]:
        z = ARCH_SIZES[name]
        D, H, G, ff, V, NL = z["width"], z["heads"], z["kv"], z["ff"], z["vocab"], z["layers"]
        # ---- Gobesun: three recurrent layers to one attention layer, every layer with a feed-forward -------------------------------
        layers = []
        for i in range(NL):
            layers.append(S.gobesun_attention_layer(H, G, hd, hd, z["chunk"], 64, ff=ff, base=1e6) if i % 4 == 3 else
                          S.gobesun_delta_layer(H, H // 2, hd, hd, conv=4, ff=ff))
        cfg = S.gobesun_config(D, V, layers)
        model = GobesunModel(GobesunConfig.from_dict(cfg), S.gobesun_weights(cfg, 0), dtype=bf, block_size=64, max_pos=P + 64, device=dev)
        blocks_per = -(-(CTX + K + W + 8) // 64)
        runner = ModelRunner(model, B * blocks_per + P // 64 + 1, B + 1, 64, decode_graphs=True, max_blocks_per_seq=blocks_per)
        toks = torch.randint(0, V, (P,), generator=torch.Generator().manual_seed(1)).tolist()

        def g_prefill():
            runner.admit(10 ** 6)
            runner.execute([dict(seq_id=10 ** 6, tokens=toks, want=[P - 1])])
            runner.release(10 ** 6)
        g_pre = timed(g_prefill, 3, 2)
        for i in range(B):
            runner.admit(i)
        for i in range(0, B, 4):
            runner.execute([dict(seq_id=j, tokens=toks[:CTX], want=[]) for j in range(i, i + 4)])
        step_entries = lambda: [dict(seq_id=j, tokens=[toks[j]], want=[0]) for j in range(B)]
        g_dec = timed(lambda: runner.execute(step_entries()), K, W)          # host metadata + 2 H2D copies + graph replay, per step
        g_dec_dev = timed(runner._graphs[B].graph.replay, K, 3)                  # the captured step alone (device time)
        # ---- per-kernel times of the Gobesun step, from the model's own call sequence (eager, CUDA events around every op) ------
        kern = {}
        names = ["linear", "rms_norm_ex", "gelu_tanh_mul", "embedding_scaled", "causal_conv_silu", "gated_delta_rule", "gated_rms_norm",
                 "qk_norm_rope_cache", "paged_attention_varlen", "paged_attention_decode_chunked"]
        orig = {n: getattr(ops, n) for n in names}

        def instrument(tag):
            def wrap(n):
                def f(*a, **k):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize(); e0.record()
                    r = orig[n](*a, **k)
                    e1.record(); torch.cuda.synchronize()
                    key = n if n != "linear" else f"linear[{a[1].shape[0]}x{a[1].shape[1]}]"
                    kern.setdefault((tag, key), []).append(e0.elapsed_time(e1) * 1e-3)
                    return r
                return f
            for n in names:
                setattr(ops, n, wrap(n))
        instrument("prefill")
        g_prefill(); kern.clear(); g_prefill()
        runner.decode_graphs = False
        instrument("decode")
        runner.execute(step_entries())
        for k in [k for k in kern if k[0] == "decode"]:
            kern.pop(k)
        runner.execute(step_entries())
        for n in names:
            setattr(ops, n, orig[n])
        del runner, model
        torch.cuda.empty_cache()

        l_pre, l_dec, lk = llama_beside(pkg, S, BK, z, hd, P, B, CTX, K, W, blocks_per, toks, timed, dev)
        med = lambda v: sorted(v)[len(v) // 2]
        esz = 2
        Gd = H // 2                                    # key heads of the recurrent layers
        Cd = 2 * Gd * hd + H * hd
        # algorithmic work per call: ("bytes", n) is set against the measured copy bandwidth, ("flops", n) against the measured bf16 GEMM rate
        def work(tag, key, T):
            if key.startswith("linear["):
                n, k = (int(v) for v in key[7:-1].split("x"))
                if n == V and tag == "prefill":
                    T = 1                           # only the last row of a prompt goes through the head
                return ("flops", 2.0 * T * n * k) if (tag == "prefill" and T > 1) else ("bytes", n * k * esz + T * (k * esz + n * 4))
            return {
                "rms_norm_ex": ("bytes", T * D * (4 + esz)), "rms_norm": ("bytes", T * D * (4 + esz)),
                "gelu_tanh_mul": ("bytes", T * ff * (8 + esz)), "silu_mul": ("bytes", T * ff * (8 + esz)),
                "embedding_scaled": ("bytes", T * D * (esz + 4)),
                "causal_conv_silu": ("bytes", T * Cd * 8),
                "gated_rms_norm": ("bytes", T * H * hd * (8 + esz)),
                "qk_norm_rope_cache": ("bytes", T * ((H + 2 * G) * hd * 4 + H * hd * esz + 2 * G * hd * esz)),
                "fused_rope": ("bytes", T * (H + G) * hd * 8), "reshape_and_cache": ("bytes", T * 2 * G * hd * esz * 2),
                # recurrence: q, k, v in and o out (f32) plus one read and one write of every entry's state
                "gated_delta_rule": ("bytes", T * (Cd + H * hd) * 4 + (1 if tag == "prefill" else T) * 2 * H * hd * hd * 4),
                # causal attention inside chunks of `chunk` keys
                "paged_attention_varlen": ("flops", 4.0 * H * hd * sum(min(i % z["chunk"] + 1, i + 1) for i in range(T))) if tag == "prefill"
                else ("bytes", T * (min(CTX, CTX % z["chunk"] + 1)) * 2 * G * hd * esz),
                "paged_attention_decode_chunked": ("bytes", T * (min(CTX, CTX % z["chunk"] + 1)) * 2 * G * hd * esz),
                "paged_attention_prefill": ("flops", 4.0 * H * hd * T * (T + 1) / 2),
            }.get(key)

        def table(rows, tag, T):
            out = {}
            for key, v in rows:
                w = work(tag, key, T)
                t = med(v)
                e = {"us": round(t * 1e6, 1), "calls_per_step": len(v)}
                if w:
                    roof = w[1] / (HBM if w[0] == "bytes" else TC)
                    e.update(bound=w[0], roofline_us=round(roof * 1e6, 2), frac_of_measured_peak=round(roof / t, 3))
                if key == "gated_delta_rule" and tag == "prefill":
                    # the recurrence is 32-bit by definition, so its arithmetic runs on the FMA pipe, not on tensor cores: three
                    # multiply-adds per state element per token against the nominal f32 rate (SMs x 128 lanes x 2 x max clock)
                    props = torch.cuda.get_device_properties(0)
                    f32_peak = props.multi_processor_count * 128 * 2 * 1.965e9
                    roof32 = 6.0 * T * H * hd * hd / f32_peak
                    e.update(f32_fma_roofline_us=round(roof32 * 1e6, 2), frac_of_nominal_f32_fma=round(roof32 / t, 3))
                out[key] = e
            return out
        results[name] = {
            "gobesun": {"prefill_tokens_per_s": round(P / g_pre), "prefill_ms": round(g_pre * 1e3, 2), "decode_tokens_per_s": round(B / g_dec),
                        "decode_ms_per_step": round(g_dec * 1e3, 3), "decode": "CUDA-graph replay incl. host metadata and H2D",
                        "decode_ms_per_step_device": round(g_dec_dev * 1e3, 3), "decode_tokens_per_s_device": round(B / g_dec_dev),
                        "kernels_prefill": table([(k[1], v) for k, v in kern.items() if k[0] == "prefill"], "prefill", P),
                        "kernels_decode": table([(k[1], v) for k, v in kern.items() if k[0] == "decode"], "decode", B)},
            "llama_dense_bf16": {"prefill_tokens_per_s": round(P / l_pre), "prefill_ms": round(l_pre * 1e3, 2), "decode_tokens_per_s": round(B / l_dec),
                                 "decode_ms_per_step": round(l_dec * 1e3, 3), "decode": "CUDA-graph replay, device-resident metadata",
                                 "prefill": "layer written with the framework's operators (f32 glue through torch)",
                                 "kernels_prefill": table(list(lk.items()), "prefill", P)},
            "shape": dict(z, prompt=P, decode_batch=B, decode_ctx=CTX, head_dim=hd),
        }
    clocks = sampler.stop()
    first = results[next(iter(results))]
    print(json.dumps({"metric": "Gobesun prefill / decode tokens/s beside dense bf16 Llama of equal size", "value": first["gobesun"]["decode_tokens_per_s"],
                      "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "arch": "gobesun",
                      "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": "fallback" if peaks.get("fallback") else "MEASURED_PEAKS.json"},
                      "l2": "weights and activations of a step exceed L2 (126 MB)", "clocks": clocks,
                      "gpu_launches": int(pkg.lib().b200_total_kernel_launches() - l0), "sizes": results}))


# ------------------------------------------------------------------------------------------------
# --arch guvusun: latent attention + routed experts beside the closest existing model and kernels at equal size
# ------------------------------------------------------------------------------------------------
GUVUSUN_SIZES = {
    # width, heads, unrotated / rotated / value sizes, latent, experts x ff (top + identity, groups), layers
    "w2048": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=512, experts=64, ff=1408, top=6, identity=4, groups=(4, 2), vocab=32000, layers=4, side=64),
    "w4096": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, rank=512, experts=32, ff=2048, top=4, identity=0, groups=None, vocab=32000, layers=2, side=64),
}


def run_guvusun(args):
    import torch
    import candle_vllm_b200 as pkg
    from candle_vllm_b200 import seq_ops as ops, synthetic as S, mla as MLA
    from candle_vllm_b200 import backend as BK
    from candle_vllm_b200.engine import ModelRunner
    from candle_vllm_b200.guvusun import GuvusunConfig, GuvusunModel

    torch.cuda.set_device(0)
    dev = "cuda"
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else \
        {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}
    HBM, TC = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    props = torch.cuda.get_device_properties(0)
    F32 = props.multi_processor_count * 128 * 2 * 1.965e9           # nominal f32 FMA rate: the bound of 32-bit SIMT arithmetic
    K, W = max(args.steps, 1), max(args.warmup, 3)
    P, B, CTX = 4096, 32, 1024
    bf = torch.bfloat16
    l0 = pkg.lib().b200_total_kernel_launches()

    def timed(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    sampler = ClockSampler(0); sampler.start()
    results = {}
    sizes = args.arch_sizes if args.arch_sizes != "w2048,w4096" else "w2048,w4096"
    for name in [n for n in sizes.split(",") if n in GUVUSUN_SIZES]:
        z = GUVUSUN_SIZES[name]
        D, H, dn, dr, dv, R, E, ff, top, NL, V = z["width"], z["heads"], z["dim"], z["rot"], z["vdim"], z["rank"], z["experts"], z["ff"], z["top"], z["layers"], z["vocab"]
        layers = [S.guvusun_layer(H, dn, dr, dv, R, experts=E, ff=ff, top=top, identity=z["identity"], groups=z["groups"], router_scale=1.8, base=1e6,
                                  kv_from=(0 if i == NL - 1 and NL > 1 else None)) for i in range(NL)]
        cfg = S.guvusun_config(D, V, layers, bigram=dict(buckets=65521, mul_prev=8191, mul_cur=131), side_dim=z["side"])
        model = GuvusunModel(GuvusunConfig.from_dict(cfg), S.guvusun_weights(cfg, 0), dtype=bf, block_size=64, max_pos=P + 64, device=dev)
        blocks_per = -(-(CTX + K + W + 8) // 64)
        runner = ModelRunner(model, B * blocks_per + P // 64 + 1, B + 1, 64, decode_graphs=True, max_blocks_per_seq=blocks_per)
        toks = torch.randint(0, V, (P,), generator=torch.Generator().manual_seed(1)).tolist()

        def g_prefill():
            runner.admit(10 ** 6)
            runner.execute([dict(seq_id=10 ** 6, tokens=toks, want=[P - 1])])
            runner.release(10 ** 6)
        g_pre = timed(g_prefill, 3, 2)
        for i in range(B):
            runner.admit(i)
        for i in range(0, B, 4):
            runner.execute([dict(seq_id=j, tokens=toks[:CTX], want=[]) for j in range(i, i + 4)])
        step_entries = lambda: [dict(seq_id=j, tokens=[toks[j]], want=[0]) for j in range(B)]
        g_dec = timed(lambda: runner.execute(step_entries()), K, W)
        g_dec_dev = timed(runner._graphs[B].graph.replay, K, 3)
        # ---- per-kernel times from the model's own call sequence (eager, CUDA events around every op) ----------------------------
        kern = {}
        names = ["linear", "linear_grouped", "rms_norm_ex", "residual_rms_norm", "embedding_bigram", "gelu_tanh_gather_mul", "latent_kv_rope_cache", "latent_q_absorb",
                 "latent_attention_varlen", "latent_out_gate", "moe_route", "moe_gate_up", "moe_down", "moe_sorted_rows", "moe_gather_rows", "silu_mul_packed",
                 "moe_combine_rows", "repack_heads", "latent_attention_decode", "token_tables"]
        orig = {n: getattr(ops, n) for n in names}

        def instrument(tag):
            def wrap(n):
                def f(*a, **k):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize(); e0.record()
                    r = orig[n](*a, **k)
                    e1.record(); torch.cuda.synchronize()
                    key = n
                    if n == "linear":
                        key = f"linear[{a[1].shape[0]}x{a[1].shape[1]}]"
                    elif n == "linear_grouped":
                        key = f"linear_grouped[{a[1].shape[0]}x{a[1].shape[1]}x{a[1].shape[2]}]"
                    kern.setdefault((tag, key), []).append(e0.elapsed_time(e1) * 1e-3)
                    return r
                return f
            for n in names:
                setattr(ops, n, wrap(n))
        instrument("prefill")
        g_prefill(); kern.clear(); g_prefill()
        runner.decode_graphs = False
        instrument("decode")
        runner.execute(step_entries())
        for k in [k for k in kern if k[0] == "decode"]:
            kern.pop(k)
        runner.execute(step_entries())
        for n in names:
            setattr(ops, n, orig[n])
        del runner, model
        torch.cuda.empty_cache()

        # ---- the closest existing kernels: latent attention of the DeepSeek path (absorbed form, R = 512, rotated part 64, bf16) -----
        like = {}
        if R == 512 and dr == 64:
            g = torch.Generator().manual_seed(3)
            nb = P // 64 + B * blocks_per
            ckv = (torch.randn(nb, 64, 1, R, generator=g) * 0.5).to(bf).to(dev)
            kpe = (torch.randn(nb, 64, 1, dr, generator=g) * 0.5).to(bf).to(dev)
            qa = (torch.randn(P, H, R, generator=g) * 0.1).to(bf).to(dev)
            qp = (torch.randn(P, H, dr, generator=g) * 0.1).to(bf).to(dev)
            bt = torch.arange(P // 64, dtype=torch.int32, device=dev)[None, :]
            ctx1 = torch.tensor([P], dtype=torch.int32, device=dev)
            cu = torch.tensor([0, P], dtype=torch.int32, device=dev)
            like["mla_paged_prefill"] = timed(lambda: MLA.mla_paged_prefill(qa, qp, ckv, kpe, bt, ctx1, cu, 0.07), 2, 1)
            btd = torch.from_numpy(np.asarray(S.random_block_tables(B, blocks_per, nb, seed=2), np.int32)).to(dev)
            ctxd = torch.full((B,), CTX + 1, dtype=torch.int32, device=dev)
            like["mla_paged_decode"] = timed(lambda: MLA.mla_paged_decode(qa[:B].contiguous(), qp[:B].contiguous(), ckv, kpe, btd, ctxd, 0.07), 20, 3)
            del ckv, kpe, qa, qp
        # ---- dense bf16 Llama of equal width / heads / depth, ff = the experts a token uses -----------------------------------------
        zl = dict(width=D, heads=H, kv=H // 4, ff=(top * ff + 127) // 128 * 128, vocab=V, layers=NL)
        l_pre, l_dec, lk = llama_beside(pkg, S, BK, zl, 128, P, B, CTX, K, W, blocks_per, toks, timed, dev)
        torch.cuda.empty_cache()

        med = lambda v: sorted(v)[len(v) // 2]
        esz = 2
        Wd = R + dr

        def work(tag, key, T):
            """algorithmic work per call: ("bytes", n) against the measured copy bandwidth, ("flops", n) against the measured bf16 GEMM rate,
            ("f32", n) against the nominal f32 FMA rate"""
            if key.startswith("linear["):
                n, k = (int(v) for v in key[7:-1].split("x"))
                if n == V and tag == "prefill":
                    T = 1
                return ("flops", 2.0 * T * n * k) if (tag == "prefill" and T > 1) else ("bytes", n * k * esz + T * (k * esz + n * 4))
            if key.startswith("linear_grouped["):
                gcount, n, k = (int(v) for v in key[15:-1].split("x"))
                rows = T * top if gcount == E else T * H
                if tag == "decode":                 # few rows per matrix: every matrix that has rows streams once (all of them, as an upper bound)
                    return ("bytes", min(rows, gcount) * n * k * esz)
                return ("flops", 2.0 * rows * n * k)
            ctx_sum = T * (T + 1) / 2 if tag == "prefill" else T * (CTX + 1)
            return {
                "rms_norm_ex": ("bytes", (1 if tag == "prefill" else T) * D * (4 + esz)), "rms_norm": ("bytes", T * D * (4 + esz)),
                "residual_rms_norm": ("bytes", T * D * (12 + esz)),
                "embedding_bigram": ("bytes", T * D * (2 * esz + 4)),
                "gelu_tanh_gather_mul": ("bytes", T * z["side"] * (4 + 2 * esz)),
                "latent_kv_rope_cache": ("bytes", T * Wd * (4 + esz)),
                "latent_q_absorb": ("bytes", T * H * ((dn + dr) * 4 + Wd * 4 + (dn * esz if tag == "prefill" else 0)) + (0 if tag == "prefill" else H * dn * R * esz)),
                "latent_out_gate": ("bytes", T * H * ((dv if tag == "prefill" else R) * 4 + dv * esz) + (0 if tag == "prefill" else H * dv * R * esz)),
                # scores and weighted sums over the latent: 2 (R + dr) + 2 R flops per key and head; in decode the cache rows of every
                # sequence are read once per group of 8 heads
                "latent_attention_varlen": ("f32", ctx_sum * H * (2 * Wd + 2 * R)) if tag == "prefill" else ("bytes", ctx_sum * Wd * esz),
                "mla_paged_prefill": ("f32", ctx_sum * H * (2 * Wd + 2 * R)), "mla_paged_decode": ("bytes", ctx_sum * Wd * esz),
                # rows on the split-KV tensor-core kernel: tensor work for prompts, cache bytes (once per 16 heads) for single tokens
                "latent_attention_decode": ("flops", ctx_sum * H * (2 * Wd + 2 * R)) if tag == "prefill" else ("bytes", ctx_sum * Wd * esz * -(-H // 16)),
                "repack_heads": ("bytes", T * H * (R * 6 + R * 4 + dr * 6) / 3), "token_tables": ("bytes", T * (blocks_per + 1) * 8),
                "moe_route": ("bytes", T * ((E + z["identity"]) * 4 + top * 8)),
                "moe_gate_up": ("bytes", min(T * top, E) * 2 * ff * D * esz), "moe_down": ("bytes", min(T * top, E) * ff * D * esz),
                "moe_gather_rows": ("bytes", T * top * D * esz * 2), "silu_mul_packed": ("bytes", T * top * ff * (8 + esz)),
                "moe_combine_rows": ("bytes", T * top * D * 4 + T * D * 8), "moe_sorted_rows": ("bytes", T * top * 12),
                "silu_mul": ("bytes", T * zl["ff"] * (8 + esz)), "fused_rope": ("bytes", T * (H + zl["kv"]) * 128 * 8),
                "reshape_and_cache": ("bytes", T * 2 * zl["kv"] * 128 * esz * 2), "paged_attention_prefill": ("flops", 4.0 * H * 128 * T * (T + 1) / 2),
            }.get(key)

        def table(rows, tag, T):
            out = {}
            for key, v in rows:
                w = work(tag, key, T)
                t = med(v)
                e = {"us": round(t * 1e6, 1), "calls_per_step": len(v)}
                if w:
                    roof = w[1] / {"bytes": HBM, "flops": TC, "f32": F32}[w[0]]
                    e.update(bound=w[0], roofline_us=round(roof * 1e6, 2), frac_of_peak=round(roof / t, 3))
                out[key] = e
            return out
        results[name] = {
            "guvusun": {"prefill_tokens_per_s": round(P / g_pre), "prefill_ms": round(g_pre * 1e3, 2), "decode_tokens_per_s": round(B / g_dec),
                        "decode_ms_per_step": round(g_dec * 1e3, 3), "decode": "CUDA-graph replay incl. host metadata and H2D",
                        "decode_ms_per_step_device": round(g_dec_dev * 1e3, 3), "decode_tokens_per_s_device": round(B / g_dec_dev),
                        "kernels_prefill": table([(k[1], v) for k, v in kern.items() if k[0] == "prefill"], "prefill", P),
                        "kernels_decode": table([(k[1], v) for k, v in kern.items() if k[0] == "decode"], "decode", B)},
            "like_kernels": {"prefill": table([("mla_paged_prefill", [like["mla_paged_prefill"]])] if like else [], "prefill", P),
                             "decode": table([("mla_paged_decode", [like["mla_paged_decode"]])] if like else [], "decode", B)},
            "llama_dense_bf16": {"prefill_tokens_per_s": round(P / l_pre), "prefill_ms": round(l_pre * 1e3, 2), "decode_tokens_per_s": round(B / l_dec),
                                 "decode_ms_per_step": round(l_dec * 1e3, 3), "decode": "CUDA-graph replay, device-resident metadata",
                                 "prefill": "layer written with the framework's operators (f32 glue through torch)", "ff": zl["ff"],
                                 "kernels_prefill": table(list(lk.items()), "prefill", P)},
            "shape": dict(z, prompt=P, decode_batch=B, decode_ctx=CTX),
        }
    clocks = sampler.stop()
    first = results[next(iter(results))]
    print(json.dumps({"metric": "Guvusun prefill / decode tokens/s beside dense bf16 Llama of equal size", "value": first["guvusun"]["decode_tokens_per_s"],
                      "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "arch": "guvusun",
                      "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "f32_fma_tflops_nominal": round(F32 / 1e12, 1),
                                "source": "fallback" if peaks.get("fallback") else "MEASURED_PEAKS.json"},
                      "l2": "weights and activations of a step exceed L2 (126 MB)", "clocks": clocks,
                      "gpu_launches": int(pkg.lib().b200_total_kernel_launches() - l0), "sizes": results}))


# ------------------------------------------------------------------------------------------------
# --arch panarax: recurrence / linear attention / softmax attention + matrix memory, dense and routed feed-forwards, beside a Gobesun of equal size
# ------------------------------------------------------------------------------------------------
PANARAX_SIZES = {
    "w2048": dict(width=2048, heads=16, kv=4, ff=5632, vocab=32000, layers=8, experts=8, top=2),
    "w4096": dict(width=4096, heads=32, kv=8, ff=11008, vocab=32000, layers=4, experts=8, top=2),
}


def run_panarax(args):
    import torch
    import candle_vllm_b200 as pkg
    from candle_vllm_b200 import seq_ops as ops, synthetic as S
    from candle_vllm_b200.engine import ModelRunner
    from candle_vllm_b200.gobesun import GobesunConfig, GobesunModel
    from candle_vllm_b200.panarax import PanaraxConfig, PanaraxModel

    torch.cuda.set_device(0)
    dev = "cuda"
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else \
        {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}
    HBM, TC = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    props = torch.cuda.get_device_properties(0)
    F32 = props.multi_processor_count * 128 * 2 * 1.965e9            # nominal f32 multiply-add rate: the recurrences are 32-bit by definition
    K, W = max(args.steps, 1), max(args.warmup, 3)
    P, B, CTX, hd = 4096, 32, 1024, 128
    bf = torch.bfloat16
    l0 = pkg.lib().b200_total_kernel_launches()

    def timed(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    names = ["linear", "linear_grouped", "rms_norm_ex", "layer_norm", "gelu_tanh_mul", "glu_packed", "embedding_scaled", "embedding_positional", "causal_conv_silu",
             "causal_conv", "gated_delta_rule", "gated_rms_norm", "group_rms_norm_gate", "block_diag_linear", "gated_linear_scan", "linear_attention", "qk_norm_rope_cache",
             "paged_attention_varlen", "paged_attention_decode_chunked", "head_gate", "gated_residual_add", "moe_route", "moe_sorted_rows", "moe_gather_rows",
             "moe_combine_rows", "moe_gate_up", "moe_down"]

    def measure(model, V):
        """(prefill s, decode s per step incl. host, decode s per step device, {(tag, kernel): [s]})"""
        blocks_per = -(-(CTX + K + W + 8) // 64)
        runner = ModelRunner(model, B * blocks_per + P // 64 + 1, B + 1, 64, decode_graphs=True, max_blocks_per_seq=blocks_per)
        toks = torch.randint(0, V, (P,), generator=torch.Generator().manual_seed(1)).tolist()

        def prefill():
            runner.admit(10 ** 6)
            runner.execute([dict(seq_id=10 ** 6, tokens=toks, want=[P - 1])])
            runner.release(10 ** 6)
        pre = timed(prefill, 3, 2)
        for i in range(B):
            runner.admit(i)
        for i in range(0, B, 4):
            runner.execute([dict(seq_id=j, tokens=toks[:CTX], want=[]) for j in range(i, i + 4)])
        step_entries = lambda: [dict(seq_id=j, tokens=[toks[j]], want=[0]) for j in range(B)]
        dec = timed(lambda: runner.execute(step_entries()), K, W)
        dec_dev = timed(runner._graphs[B].graph.replay, K, 3)
        kern = {}
        orig = {n: getattr(ops, n) for n in names}

        def instrument(tag):
            def wrap(n):
                def f(*a, **k):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize(); e0.record()
                    r = orig[n](*a, **k)
                    e1.record(); torch.cuda.synchronize()
                    key = n
                    if n == "linear":
                        key = f"linear[{a[1].shape[0]}x{a[1].shape[1]}]"
                    elif n == "linear_grouped":
                        key = f"linear_grouped[{a[1].shape[0]}x{a[1].shape[1]}x{a[1].shape[2]}]"
                    elif n == "linear_attention":
                        key = "linear_attention[" + ("decay" if k.get("decay") is not None else "exp") + "]"
                    kern.setdefault((tag, key), []).append(e0.elapsed_time(e1) * 1e-3)
                    return r
                return f
            for n in names:
                setattr(ops, n, wrap(n))
        instrument("prefill")
        prefill(); kern.clear(); prefill()
        runner.decode_graphs = False
        instrument("decode")
        runner.execute(step_entries())
        for k in [k for k in kern if k[0] == "decode"]:
            kern.pop(k)
        runner.execute(step_entries())
        for n in names:
            setattr(ops, n, orig[n])
        del runner
        torch.cuda.empty_cache()
        return pre, dec, dec_dev, kern

    sampler = ClockSampler(0); sampler.start()
    results = {}
    for name in [n for n in args.arch_sizes.split(",") if n in PANARAX_SIZES]:
        z = PANARAX_SIZES[name]
        D, H, G, ff, V, NL, E, top = z["width"], z["heads"], z["kv"], z["ff"], z["vocab"], z["layers"], z["experts"], z["top"]
        # ---- Panarax: parallel, recurrence, lightning, lightning in turn; dense and routed feed-forwards alternate (the routed ones with top x expert ff = ff)
        layers = []
        for i in range(NL):
            mlp = dict(ff=ff) if i % 2 == 0 else dict(ff=ff // top, experts=E, top=top)
            if i % 4 == 0:
                layers.append(S.panarax_parallel_layer(H, G, hd, hd, H // 2, hd, hd, q_temp=(0.1, 1024), **mlp))
            elif i % 4 == 1:
                layers.append(S.panarax_rglru_layer(D, H, conv=4, **mlp))
            else:
                layers.append(S.panarax_lightning_layer(H, hd, hd, **mlp))
        cfg = S.panarax_config(D, V, layers, max_positions=P + 64, taps=3)
        model = PanaraxModel(PanaraxConfig.from_dict(cfg), S.panarax_weights(cfg, 0), dtype=bf, block_size=64, device=dev)
        p_pre, p_dec, p_dec_dev, p_kern = measure(model, V)
        del model
        torch.cuda.empty_cache()
        # ---- Gobesun of equal width / heads / ff / depth: three recurrent layers to one attention layer
        glayers = [S.gobesun_attention_layer(H, G, hd, hd, 2048, 64, ff=ff, base=1e6) if i % 4 == 3 else S.gobesun_delta_layer(H, H // 2, hd, hd, conv=4, ff=ff)
                   for i in range(NL)]
        gcfg = S.gobesun_config(D, V, glayers)
        gmodel = GobesunModel(GobesunConfig.from_dict(gcfg), S.gobesun_weights(gcfg, 0), dtype=bf, block_size=64, max_pos=P + 64, device=dev)
        g_pre, g_dec, g_dec_dev, g_kern = measure(gmodel, V)
        del gmodel
        torch.cuda.empty_cache()
        med = lambda v: sorted(v)[len(v) // 2]
        esz, Hm, Gd = 2, H // 2, H // 2
        Cd = 2 * Gd * hd + H * hd
        n_blk = D // H

        def work(tag, key, T):
            """algorithmic work of one call: ("bytes", n) against the measured copy bandwidth, ("flops", n) against the measured bf16 GEMM rate, ("f32", n)
            against the nominal f32 multiply-add rate"""
            pre = tag == "prefill"
            if key.startswith("linear["):
                n, k = (int(v) for v in key[7:-1].split("x"))
                if n == V and pre:
                    T = 1
                return ("flops", 2.0 * T * n * k) if (pre and T > 1) else ("bytes", n * k * esz + T * (k * esz + n * 4))
            if key.startswith("linear_grouped["):
                g, n, k = (int(v) for v in key[15:-1].split("x"))
                return ("flops", 2.0 * T * top * n * k) if pre else ("bytes", min(g, T * top) * n * k * esz + T * top * (k * esz + n * 4))
            state = lambda per_seq: (1 if pre else T) * 2 * per_seq * 4            # one read and one write of every entry's state
            table = {
                "rms_norm_ex": ("bytes", T * D * (4 + esz)), "layer_norm": ("bytes", T * D * (4 + esz)),
                "gelu_tanh_mul": ("bytes", T * ff * (8 + esz)), "glu_packed": ("bytes", T * ff * (8 + esz)),
                "embedding_scaled": ("bytes", T * D * (esz + 4)), "embedding_positional": ("bytes", T * D * (2 * esz + 4)),
                "causal_conv_silu": ("bytes", T * Cd * 8), "causal_conv": ("bytes", T * D * (4 + esz)),
                "gated_rms_norm": ("bytes", T * H * hd * (8 + esz)), "group_rms_norm_gate": ("bytes", T * H * hd * (8 + esz)),
                "gated_residual_add": ("bytes", T * D * 16), "head_gate": ("bytes", T * H * hd * 2 * esz),
                "qk_norm_rope_cache": ("bytes", T * ((H + 2 * G) * hd * 4 + H * hd * esz + 2 * G * hd * esz)),
                "gated_delta_rule": ("bytes", T * (Cd + H * hd) * 4) if not pre else ("f32", 6.0 * T * H * hd * hd),
                "linear_attention[decay]": ("bytes", T * 4 * H * hd * 4 + state(H * hd * hd)) if not pre else ("f32", 4.0 * T * H * hd * hd),
                "linear_attention[exp]": ("bytes", T * 4 * Hm * hd * 4 + state(Hm * hd * hd)) if not pre else ("f32", 4.0 * T * Hm * hd * hd),
                "block_diag_linear": ("f32", 2.0 * T * D * 2 * n_blk) if pre else ("bytes", 2 * D * n_blk * 4 + T * D * 12),
                "gated_linear_scan": ("bytes", T * D * (16 + esz) + state(D)),
                "paged_attention_varlen": ("flops", 4.0 * H * hd * T * (T + 1) / 2) if pre else ("bytes", T * CTX * 2 * G * hd * esz),
                "paged_attention_decode_chunked": ("bytes", T * CTX * 2 * G * hd * esz),
            }
            if key == "gated_delta_rule" and not pre:
                return ("bytes", T * (Cd + H * hd) * 4 + state(H * hd * hd))
            return table.get(key)

        def table(kern, tag, T):
            out = {}
            for (tg, key), v in kern.items():
                if tg != tag:
                    continue
                t = med(v)
                e = {"us": round(t * 1e6, 1), "calls_per_step": len(v)}
                w = work(tag, key, T)
                if w:
                    roof = w[1] / {"bytes": HBM, "flops": TC, "f32": F32}[w[0]]
                    e.update(bound=w[0], roofline_us=round(roof * 1e6, 2), frac_of_roofline=round(roof / t, 3))
                out[key] = e
            return out
        results[name] = {
            "panarax": {"prefill_tokens_per_s": round(P / p_pre), "prefill_ms": round(p_pre * 1e3, 2), "decode_tokens_per_s": round(B / p_dec),
                        "decode_ms_per_step": round(p_dec * 1e3, 3), "decode": "CUDA-graph replay incl. host metadata and H2D",
                        "decode_ms_per_step_device": round(p_dec_dev * 1e3, 3), "decode_tokens_per_s_device": round(B / p_dec_dev),
                        "kernels_prefill": table(p_kern, "prefill", P), "kernels_decode": table(p_kern, "decode", B)},
            "gobesun": {"prefill_tokens_per_s": round(P / g_pre), "prefill_ms": round(g_pre * 1e3, 2), "decode_tokens_per_s": round(B / g_dec),
                        "decode_ms_per_step": round(g_dec * 1e3, 3), "decode_ms_per_step_device": round(g_dec_dev * 1e3, 3),
                        "decode_tokens_per_s_device": round(B / g_dec_dev),
                        "kernels_prefill": table(g_kern, "prefill", P), "kernels_decode": table(g_kern, "decode", B)},
            "shape": dict(z, prompt=P, decode_batch=B, decode_ctx=CTX, head_dim=hd, recurrence_blocks=H, memory_heads=Hm),
        }
    clocks = sampler.stop()
    first = results[next(iter(results))]
    print(json.dumps({"metric": "Panarax prefill / decode tokens/s beside a Gobesun of equal size", "value": first["panarax"]["decode_tokens_per_s"],
                      "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "arch": "panarax",
                      "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "f32_fma_tflops_nominal": round(F32 / 1e12, 1),
                                "source": "fallback" if peaks.get("fallback") else "MEASURED_PEAKS.json"},
                      "l2": "weights and activations of a step exceed L2 (126 MB)", "clocks": clocks,
                      "gpu_launches": int(pkg.lib().b200_total_kernel_launches() - l0), "sizes": results}))


# --arch dofevik: softmax attention with a sink, sigmoid attention over a window plus pooled blocks, latent attention, ungated routed experts beside a
# shared one -- beside a Guvusun (latent attention with a sink + routed experts) of equal size
# ------------------------------------------------------------------------------------------------
DOFEVIK_SIZES = {
    # width, heads / kv heads of 128, window, pool, latent sizes, experts x ff (top) + shared ff, layers (the three mixers in turn)
    "w2048": dict(width=2048, heads=16, kv=4, window=1024, pool=16, dim=128, rot=64, vdim=128, rank=512, q_rank=768, experts=64, ff=1408, top=6, shared=2816,
                  vocab=32000, layers=6),
    "w4096": dict(width=4096, heads=32, kv=8, window=1024, pool=16, dim=128, rot=64, vdim=128, rank=512, q_rank=1536, experts=32, ff=2048, top=4, shared=4096,
                  vocab=32000, layers=3),
}


def run_dofevik(args):
    import torch
    import candle_vllm_b200 as pkg
    from candle_vllm_b200 import seq_ops as ops, synthetic as S
    from candle_vllm_b200.engine import ModelRunner
    from candle_vllm_b200.dofevik import DofevikConfig, DofevikModel
    from candle_vllm_b200.guvusun import GuvusunConfig, GuvusunModel

    torch.cuda.set_device(0)
    dev = "cuda"
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else \
        {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}
    HBM, TC = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    props = torch.cuda.get_device_properties(0)
    F32 = props.multi_processor_count * 128 * 2 * 1.965e9           # nominal f32 multiply-add rate: the bound of 32-bit SIMT arithmetic
    K, W = max(args.steps, 1), max(args.warmup, 3)
    P, B, CTX, hd = 4096, 32, 2048, 128
    bf = torch.bfloat16
    l0 = pkg.lib().b200_total_kernel_launches()

    def timed(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    names = ["linear", "linear_grouped", "rms_norm_ex", "add_rms_norm", "residual_rms_norm", "embedding_scaled", "embedding_bigram", "gelu_tanh_gather_mul",
             "qk_head_norm_rope_cache", "pooled_cache_update", "paged_attention_varlen_sink", "paged_attention_sigmoid_pooled", "latent_kv_rope_cache",
             "latent_q_absorb", "latent_attention_varlen", "latent_attention_decode", "latent_out_gate", "repack_heads", "token_tables", "moe_route", "moe_sorted_rows",
             "moe_gather_rows", "moe_combine_rows", "moe_gate_up", "moe_down", "glu_packed", "silu_mul_packed"]

    def measure(model, V):
        """(prefill s, decode s per step incl. host, decode s per step device, {(tag, kernel): [s]})"""
        blocks_per = -(-(CTX + K + W + 8) // 64)
        runner = ModelRunner(model, B * blocks_per + P // 64 + 1, B + 1, 64, decode_graphs=True, max_blocks_per_seq=blocks_per)
        toks = torch.randint(0, V, (P,), generator=torch.Generator().manual_seed(1)).tolist()

        def prefill():
            runner.admit(10 ** 6)
            runner.execute([dict(seq_id=10 ** 6, tokens=toks, want=[P - 1])])
            runner.release(10 ** 6)
        pre = timed(prefill, 3, 2)
        for i in range(B):
            runner.admit(i)
        for i in range(0, B, 4):
            runner.execute([dict(seq_id=j, tokens=toks[:CTX], want=[]) for j in range(i, i + 4)])
        step_entries = lambda: [dict(seq_id=j, tokens=[toks[j]], want=[0]) for j in range(B)]
        dec = timed(lambda: runner.execute(step_entries()), K, W)
        dec_dev = timed(runner._graphs[B].graph.replay, K, 3)
        kern = {}
        orig = {n: getattr(ops, n) for n in names}

        def instrument(tag):
            def wrap(n):
                def f(*a, **k):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize(); e0.record()
                    r = orig[n](*a, **k)
                    e1.record(); torch.cuda.synchronize()
                    key = n
                    if n == "linear":
                        key = f"linear[{a[1].shape[0]}x{a[1].shape[1]}]"
                    elif n == "linear_grouped":
                        key = f"linear_grouped[{a[1].shape[0]}x{a[1].shape[1]}x{a[1].shape[2]}]"
                    elif n == "glu_packed":
                        key = f"glu_packed[{a[0].shape[1]}]"
                    kern.setdefault((tag, key), []).append(e0.elapsed_time(e1) * 1e-3)
                    return r
                return f
            for n in names:
                setattr(ops, n, wrap(n))
        instrument("prefill")
        prefill(); kern.clear(); prefill()
        runner.decode_graphs = False
        instrument("decode")
        runner.execute(step_entries())
        for k in [k for k in kern if k[0] == "decode"]:
            kern.pop(k)
        runner.execute(step_entries())
        for n in names:
            setattr(ops, n, orig[n])
        del runner
        torch.cuda.empty_cache()
        return pre, dec, dec_dev, kern

    sampler = ClockSampler(0); sampler.start()
    results = {}
    for name in [n for n in args.arch_sizes.split(",") if n in DOFEVIK_SIZES]:
        z = DOFEVIK_SIZES[name]
        D, H, G, Wn, Pl, dn, dr, dv, R, Rq = z["width"], z["heads"], z["kv"], z["window"], z["pool"], z["dim"], z["rot"], z["vdim"], z["rank"], z["q_rank"]
        E, ff, top, sff, V, NL = z["experts"], z["ff"], z["top"], z["shared"], z["vocab"], z["layers"]
        mlp = dict(experts=E, ff=ff, top=top, shared_ff=sff)
        layers = []
        for i in range(NL):
            if i % 3 == 0:
                layers.append(S.dofevik_pooled_layer(H, G, hd, window=Wn, pool=Pl, **mlp))
            elif i % 3 == 1:
                layers.append(S.dofevik_latent_layer(H, dn, dr, dv, R, Rq, window=Wn, base=1e6, **mlp))
            else:
                layers.append(S.dofevik_attention_layer(H, G, hd, hd, window=Wn, rot_dims=hd, base=1e6, factor=2.0, **mlp))
        cfg = S.dofevik_config(D, V, layers)
        model = DofevikModel(DofevikConfig.from_dict(cfg), S.dofevik_weights(cfg, 0), dtype=bf, block_size=64, max_pos=P + 64, device=dev)
        d_pre, d_dec, d_dec_dev, d_kern = measure(model, V)
        del model
        torch.cuda.empty_cache()
        # ---- Guvusun of equal width / heads / latent sizes / experts / depth (its experts are gated: three matrices each; no shared expert)
        glayers = [S.guvusun_layer(H, dn, dr, dv, R, experts=E, ff=ff, top=top, router_scale=1.8, base=1e6) for _ in range(NL)]
        gcfg = S.guvusun_config(D, V, glayers, bigram=dict(buckets=65521, mul_prev=8191, mul_cur=131))
        gmodel = GuvusunModel(GuvusunConfig.from_dict(gcfg), S.guvusun_weights(gcfg, 0), dtype=bf, block_size=64, max_pos=P + 64, device=dev)
        g_pre, g_dec, g_dec_dev, g_kern = measure(gmodel, V)
        del gmodel
        torch.cuda.empty_cache()
        # ---- the like kernel of the two paged attentions: the tensor-core kernel as the chunk-masked softmax attention of Gobesun calls it (no sink, no pooled
        # entries), same heads and window, one prompt of P rows and one step of B rows at context CTX
        like = {}
        g0 = torch.Generator().manual_seed(3)
        nbp = P // 64 + 1
        kc = (torch.randn(nbp, 64, G, hd, generator=g0) * 0.5).to(bf).to(dev)
        vc = (torch.randn(nbp, 64, G, hd, generator=g0) * 0.5).to(bf).to(dev)
        qq = (torch.randn(P, H * hd, generator=g0) * 0.1).to(bf).to(dev)
        from candle_vllm_b200.inputs import prepare_step
        bp = ops.StepBatch.from_host(prepare_step([dict(tokens=[0] * P, start=0, block_table=list(range(nbp)), state_slot=-1, want=[])], 64), dev)
        like[("prefill", "paged_attention_varlen")] = [timed(lambda: ops.paged_attention_varlen(qq, kc, vc, bp, H, G, hd, hd, 64, hd ** -0.5, 0, Wn, bf), 3, 2)]
        nbd = B * (CTX // 64 + 1)
        kc = (torch.randn(nbd, 64, G, hd, generator=g0) * 0.5).to(bf).to(dev)
        vc = (torch.randn(nbd, 64, G, hd, generator=g0) * 0.5).to(bf).to(dev)
        per = CTX // 64 + 1
        bd = ops.StepBatch.from_host(prepare_step([dict(tokens=[0], start=CTX, block_table=list(range(j * per, (j + 1) * per)), state_slot=-1, want=[]) for j in range(B)], 64), dev)
        like[("decode", "paged_attention_varlen")] = [timed(lambda: ops.paged_attention_varlen(qq[:B], kc, vc, bd, H, G, hd, hd, 64, hd ** -0.5, 0, Wn, bf), 20, 3)]
        del kc, vc, qq
        torch.cuda.empty_cache()
        med = lambda v: (sorted(v)[(len(v) - 1) // 2] + sorted(v)[len(v) // 2]) / 2
        esz, Wd = 2, R + dr

        def work(tag, key, T):
            """algorithmic work of one call: ("bytes", n) against the measured copy bandwidth, ("flops", n) against the measured bf16 GEMM rate, ("f32", n)
            against the nominal f32 multiply-add rate"""
            pre = tag == "prefill"
            if key.startswith("linear["):
                n, k = (int(v) for v in key[7:-1].split("x"))
                if n == V and pre:
                    T = 1
                return ("flops", 2.0 * T * n * k) if (pre and T > 1) else ("bytes", n * k * esz + T * (k * esz + n * 4))
            if key.startswith("linear_grouped["):
                g, n, k = (int(v) for v in key[15:-1].split("x"))
                rows = T * top if g == E else T * H
                return ("flops", 2.0 * rows * n * k) if pre else ("bytes", min(g, rows) * n * k * esz + rows * (k * esz + n * 4))
            if key.startswith("glu_packed["):
                n = int(key[11:-1])
                return ("bytes", T * (top if n == ff else 1) * n * (4 + esz))
            # keys a row sees: window tokens (all earlier ones while the context is shorter), plus pooled blocks wholly before the window
            win = sum(min(i + 1, Wn) for i in range(T)) if pre else T * min(CTX + 1, Wn)
            blk = sum(max(0, (i - Wn + 1) // Pl) for i in range(T)) if pre else T * max(0, (CTX - Wn + 1) // Pl)
            full = T * (T + 1) / 2 if pre else T * (CTX + 1)
            table = {
                "rms_norm_ex": ("bytes", T * Rq * (4 + esz)), "add_rms_norm": ("bytes", T * D * (16 + esz)),
                "residual_rms_norm": ("bytes", T * D * (12 + esz)), "embedding_scaled": ("bytes", T * D * (esz + 4)), "embedding_bigram": ("bytes", T * D * (2 * esz + 4)),
                "qk_head_norm_rope_cache": ("bytes", T * ((H + 2 * G) * hd * 4 + H * hd * esz + 2 * G * hd * esz)),
                "pooled_cache_update": ("bytes", (T / Pl) * 2 * G * hd * (Pl * esz + 4)),
                "paged_attention_varlen_sink": ("flops", 4.0 * H * hd * win) if pre else ("bytes", win * 2 * G * hd * esz),
                "paged_attention_varlen": ("flops", 4.0 * H * hd * win) if pre else ("bytes", win * 2 * G * hd * esz),
                "paged_attention_sigmoid_pooled": ("flops", 4.0 * H * hd * (win + blk)) if pre else ("bytes", win * 2 * G * hd * esz + blk * 2 * G * hd * 4),
                "latent_kv_rope_cache": ("bytes", T * Wd * (4 + esz)),
                "latent_q_absorb": ("bytes", T * H * ((dn + dr) * 4 + Wd * 4 + (dn * esz if pre else 0)) + (0 if pre else H * dn * R * esz)),
                "latent_out_gate": ("bytes", T * H * ((dv if pre else R) * 4 + dv * esz) + (0 if pre else H * dv * R * esz)),
                "repack_heads": ("bytes", T * H * (R * 6 + R * 4 + dr * 6) / 3), "token_tables": ("bytes", T * ((CTX + K + W + 8) // 64 + 2) * 8),
                "moe_route": ("bytes", T * (E * 4 + top * 8)), "moe_sorted_rows": ("bytes", T * top * 12),
                "moe_gather_rows": ("bytes", T * top * D * esz * 2), "moe_combine_rows": ("bytes", T * top * D * 4 + T * D * 8),
                "silu_mul_packed": ("bytes", T * top * ff * (8 + esz)),
            }
            return table.get(key)

        def work_model(which, tag, key, T):
            # latent attention: Dofevik's rows see a window (SIMT kernel over the latent cache), Guvusun's the whole context (split-KV tensor-core kernel);
            # the expert matrices in front of the activation: one per expert (ungated) against two (gated)
            pre = tag == "prefill"
            win = sum(min(i + 1, Wn) for i in range(T)) if pre else T * min(CTX + 1, Wn)
            full = T * (T + 1) / 2 if pre else T * (CTX + 1)
            keys = win if which == "dofevik" else full
            if key == "latent_attention_varlen":
                return ("f32", keys * H * (2 * Wd + 2 * R)) if pre else ("bytes", keys * Wd * esz)
            if key == "latent_attention_decode":
                return ("flops", keys * H * (2 * Wd + 2 * R)) if pre else ("bytes", keys * Wd * esz * -(-H // 16))
            if key == "moe_gate_up":
                return ("bytes", min(T * top, E) * (1 if which == "dofevik" else 2) * ff * D * esz)
            if key == "moe_down":
                return ("bytes", min(T * top, E) * ff * D * esz)
            return work(tag, key, T)

        def table(which, kern, tag, T):
            out = {}
            for (tg, key), v in kern.items():
                if tg != tag:
                    continue
                t = med(v)
                e = {"us": round(t * 1e6, 1), "calls_per_step": len(v)}
                w = work_model(which, tag, key, T)
                if w:
                    roof = w[1] / {"bytes": HBM, "flops": TC, "f32": F32}[w[0]]
                    e.update(bound=w[0], roofline_us=round(roof * 1e6, 2), frac_of_roofline=round(roof / t, 3))
                out[key] = e
            return out
        side = lambda which, pre, dec, dec_dev, kern: {
            "prefill_tokens_per_s": round(P / pre), "prefill_ms": round(pre * 1e3, 2), "decode_tokens_per_s": round(B / dec), "decode_ms_per_step": round(dec * 1e3, 3),
            "decode": "CUDA-graph replay incl. host metadata and H2D", "decode_ms_per_step_device": round(dec_dev * 1e3, 3),
            "decode_tokens_per_s_device": round(B / dec_dev), "kernels_prefill": table(which, kern, "prefill", P), "kernels_decode": table(which, kern, "decode", B)}
        results[name] = {"dofevik": side("dofevik", d_pre, d_dec, d_dec_dev, d_kern), "guvusun": side("guvusun", g_pre, g_dec, g_dec_dev, g_kern),
                         "like_kernels": {"prefill": table("like", like, "prefill", P), "decode": table("like", like, "decode", B)},
                         "shape": dict(z, prompt=P, decode_batch=B, decode_ctx=CTX, head_dim=hd)}
    clocks = sampler.stop()
    first = results[next(iter(results))]
    print(json.dumps({"metric": "Dofevik prefill / decode tokens/s beside a Guvusun of equal size", "value": first["dofevik"]["decode_tokens_per_s"],
                      "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "arch": "dofevik",
                      "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "f32_fma_tflops_nominal": round(F32 / 1e12, 1),
                                "source": "fallback" if peaks.get("fallback") else "MEASURED_PEAKS.json"},
                      "l2": "weights and activations of a step exceed L2 (126 MB)", "clocks": clocks,
                      "gpu_launches": int(pkg.lib().b200_total_kernel_launches() - l0), "sizes": results}))


def main():
    args = parse()
    if args.arch == "gobesun":
        run_gobesun(args)
        return
    if args.arch == "dofevik":
        run_dofevik(args)
        return
    if args.arch == "panarax":
        run_panarax(args)
        return
    if args.arch == "guvusun":
        run_guvusun(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
