"""Dofevik on the GPU against the plain float64 restatement in oracle/dofevik.py: every mechanism alone, then whole models through the runner
(portions down to two tokens, decoding, unequal batches, blocks handed from finished requests to new ones) and greedy generation through LLMEngine.
Configurations are small and made here; sizes that one model might happen to make equal or 1 (kv heads == heads, one kv head, value size == key
size, rotation over the whole head, pool == 1, pool larger than a page, top == experts, a layer without feed-forward or without a shared expert)
differ between them.  Windows are short, so every visible key carries weight: a window or a pooled block that is one position off moves a row by
far more than the f32 tolerance."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import candle_vllm_b200 as pkg
from candle_vllm_b200 import seq_ops as ops, synthetic as S
from candle_vllm_b200.dofevik import DofevikConfig, DofevikModel
from candle_vllm_b200.engine import LLMEngine, ModelRunner
from candle_vllm_b200.inputs import prepare_step
from candle_vllm_b200.mixers import LatentAttentionMixer, PagedAttentionMixer, PooledWindowAttentionMixer, RoutedExperts, UngatedMlp
from oracle import dofevik as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64


def dev(t, dt=torch.float32):
    return t.to(dt).to(DEV).contiguous()


def batch_of(entries, block_size=64):
    return ops.StepBatch.from_host(prepare_step(entries, block_size), DEV)


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err < tol, f"{what}: max-err/max = {err:.3e} (tolerance {tol})"


def _portions(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n)); at += n; i += 1
    return out


def _caches(mix, num_blocks, dtype, bs=64):
    g, dk, dv = mix.cache_shape()
    c = [torch.full((num_blocks, bs, g, dk), 7.0, dtype=dtype, device=DEV), torch.full((num_blocks, bs, g, dv), -7.0, dtype=dtype, device=DEV)]      # dirty pages
    pool = mix.pool_shape() if hasattr(mix, "pool_shape") else None
    if pool:
        n, g, dk, dv = pool
        c += [torch.full((num_blocks, n, g, dk), 5.0, device=DEV), torch.full((num_blocks, n, g, dv), -5.0, device=DEV)]
    return tuple(c)


def run_mixer(mix, h, sizes, table, dtype, bs=64):
    """the rows of one sequence through a mixer in portions, over pages in the order `table` gives"""
    cache = _caches(mix, max(table) + 1, dtype, bs)
    out = []
    for at, n in _portions(h.shape[0], sizes):
        b = batch_of([dict(tokens=[0] * n, start=at, block_table=table, state_slot=-1, want=[])], bs)
        out.append(mix.forward(dev(h[at:at + n], dtype), b, cache))
    return torch.cat(out)


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [5, 96, 321, 1030])
def test_sum_then_norm_with_one_number(n):
    g = torch.Generator().manual_seed(n)
    x, y1, y2 = torch.randn(9, n, generator=g) * 3, torch.randn(9, n + 3, generator=g), torch.randn(9, n, generator=g) * 0.5
    num = torch.tensor(1.37)
    w = num.reshape(1).expand(n).contiguous()
    for pending in ((), (y1[:, :n],), (y1[:, :n], y2)):
        xd = dev(x)
        out = ops.add_rms_norm(xd, tuple(dev(p) if p.is_contiguous() else dev(y1)[:, :n] for p in pending), dev(w), 1e-6, torch.float32)
        tot = x.to(F64) + sum(p.to(F64) for p in pending)
        close(xd, tot, 1e-6, f"the sum of {len(pending)} addends")
        close(out, O.scalar_norm(tot, num, 1e-6), 2e-6, "its norm")
    xd = dev(x)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out = ops.add_rms_norm(xd, (dev(y2),), dev(w), 1e-5, torch.bfloat16, row_index=rows)
    close(xd, x, 1e-9, "selected rows leave the stream alone")
    close(out, O.scalar_norm((x + y2).to(F64)[[8, 0, 3]], num, 1e-5), 6e-3, "selected rows")
    xd = dev(x)
    assert ops.add_rms_norm(xd, (dev(y2),), None, 1e-6) is None
    close(xd, (x + y2).to(F64), 1e-6, "the sum alone")


@pytest.mark.parametrize("H,G,dk,dv,rot,inter,norm", [(4, 2, 12, 10, 8, True, "after"), (3, 3, 16, 16, 16, True, "after"), (5, 1, 10, 6, 4, False, "before"),
                                                      (2, 2, 34, 40, 0, False, "before"), (6, 2, 8, 8, 8, False, "none")])
def test_head_preparation_against_the_plain_rotation_and_norm(H, G, dk, dv, rot, inter, norm):
    g = torch.Generator().manual_seed(H * 100 + dk)
    T, eps, base, factor = 37, 1e-5, 777.0, 3.0
    proj = torch.randn(T, (H + G) * dk + G * dv + 5, generator=g)
    bias = torch.randn((H + G) * dk + G * dv, generator=g)
    qw, kw = 1 + torch.randn(dk, generator=g) * 0.3, 1 + torch.randn(dk, generator=g) * 0.3
    from candle_vllm_b200.mixers import yarn_rotary_tables
    cos, sin = yarn_rotary_tables(rot, base, 256, dict(factor=factor), DEV) if rot else (None, None)
    start = 130
    b = batch_of([dict(tokens=[0] * T, start=start, block_table=[2, 0, 1], state_slot=-1, want=[])])
    kc, vc = torch.zeros(3, 64, G, dk, device=DEV), torch.zeros(3, 64, G, dv, device=DEV)
    q = ops.qk_head_norm_rope_cache(dev(proj), dev(bias), dev(qw) if norm == "before" else None, dev(kw) if norm == "before" else None, cos, sin, b, kc, vc, H, G, dk, dv, rot,
                                    eps, interleaved=inter, norm=norm)
    pos = torch.arange(start, start + T)
    full = proj[:, :bias.numel()].to(F64) + bias.to(F64)
    wq, wk, wv = full[:, :H * dk].reshape(T, H, dk), full[:, H * dk:(H + G) * dk].reshape(T, G, dk), full[:, (H + G) * dk:].reshape(T, G, dv)
    if norm == "before":
        wq, wk = O.rms(wq, eps) * qw.to(F64), O.rms(wk, eps) * kw.to(F64)
    if rot:
        wq, wk = (O.rotate(t, pos, rot, base, factor, "interleaved" if inter else "half") for t in (wq, wk))
    if norm == "after":
        wq, wk = O.rms(wq, eps), O.rms(wk, eps)
    close(q.view(T, H, dk), wq, 3e-6, "queries")
    slots = [([2, 0, 1][p // 64], p % 64) for p in pos.tolist()]
    close(torch.stack([kc[a, o] for a, o in slots]), wk, 3e-6, "cached keys")
    close(torch.stack([vc[a, o] for a, o in slots]), wv, 1e-6, "cached values")


ATT = [  # H, G, dk, dv, window, rot_dims, factor
    (4, 2, 12, 10, 9, 8, 2.0), (3, 3, 16, 16, 70, 16, 0.0), (6, 1, 10, 24, 1, 4, 8.0), (2, 2, 20, 6, 0, 0, 0.0), (8, 4, 8, 8, 130, 6, 1.5),
]


@pytest.mark.parametrize("H,G,dk,dv,window,rot,factor", ATT)
@pytest.mark.parametrize("sizes", [[300], [2], [61, 1, 1, 2, 70, 3]])
def test_softmax_attention_with_sink_window_and_neighbour_pairs(H, G, dk, dv, window, rot, factor, sizes):
    g = torch.Generator().manual_seed(dk + window)
    L = S.dofevik_attention_layer(H, G, dk, dv, window=window, rot_dims=rot, factor=factor, base=300.0, scale=1.7 * dk ** -0.5)
    cfg = S.dofevik_config(48, 10, [L])
    w = {k[7:]: v for k, v in S.dofevik_weights(cfg, 3).items() if k.startswith("l0.mix.")}
    T = 150 if sizes == [2] else 300
    h = torch.randn(T, 48, generator=g)
    m = L["mixer"]
    mix = PagedAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, G, dk, dv, m["scale"], 1e-6, torch.float32, rot=m.get("rot"), window=window, max_pos=64,
                              head_norm="after", interleaved=True)
    got = run_mixer(mix, h, sizes, [3, 1, 4, 0, 2], torch.float32)
    close(got, O.mixer_attention(h.to(F64), torch.arange(T), w, m, 1e-6), 2e-5, f"attention, portions {sizes}")
    # the sink does take weight: without it the rows move by far more than the tolerance
    w2 = dict(w); w2["sink"] = torch.full((H,), -40.0)
    far = O.mixer_attention(h.to(F64), torch.arange(T), w2, m, 1e-6)
    assert float((got.cpu().to(F64) - far).abs().max()) > 1e-2 * float(far.abs().max())


POOLED = [  # H, G, dk, window, pool
    (4, 2, 12, 20, 7), (3, 3, 16, 64, 64), (6, 1, 10, 5, 1), (2, 2, 20, 9, 70), (4, 4, 8, 33, 12), (5, 1, 6, 0, 0), (2, 1, 14, 16, 0), (3, 3, 8, 1, 3), (2, 2, 8, 128, 5),
]


@pytest.mark.parametrize("H,G,dk,window,pool", POOLED)
@pytest.mark.parametrize("sizes", [[300], [2], [61, 1, 1, 2, 70, 3]])
def test_sigmoid_attention_over_window_and_pooled_blocks(H, G, dk, window, pool, sizes):
    """every row against the oracle: rows just before and after a block joins, windows that cross pages, pools that straddle pages and portions"""
    g = torch.Generator().manual_seed(dk + window + pool)
    L = S.dofevik_pooled_layer(H, G, dk, window=window, pool=pool, scale=1.3 * dk ** -0.5)
    cfg = S.dofevik_config(40, 10, [L])
    w = {k[7:]: v for k, v in S.dofevik_weights(cfg, 5).items() if k.startswith("l0.mix.")}
    T = 150 if sizes == [2] else 300
    h = torch.randn(T, 40, generator=g)
    m = L["mixer"]
    mix = PooledWindowAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, G, dk, m["scale"], 1e-6, torch.float32, window=window, pool=pool)
    got = run_mixer(mix, h, sizes, [3, 1, 4, 0, 2], torch.float32)
    close(got, O.mixer_attention_2(h.to(F64), torch.arange(T), w, m, 1e-6), 2e-5, f"window {window} pool {pool}, portions {sizes}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("G,dk,dv,pool", [(2, 16, 8, 7), (3, 5, 6, 12), (1, 128, 128, 16), (2, 24, 40, 70), (4, 8, 8, 1), (1, 4, 12, 64)])
def test_pooled_entries_are_the_means_of_their_blocks_at_their_places(G, dk, dv, pool, dtype):
    """the pooled cache after a prompt fed in portions: the entry of block b sits in the page of the block's last position at index b - floor(page bs / pool) and
    equals the mean of the cached rows (rows of 16-byte groups and rows of any other length take different kernels); places no block owns keep what they held"""
    g = torch.Generator().manual_seed(G * 1000 + dk + pool)
    bs, T, table = 64, 200, [3, 0, 2, 1]
    per = -(-bs // pool)
    keys, vals = torch.randn(T, G, dk, generator=g).to(dtype), torch.randn(T, G, dv, generator=g).to(dtype)
    kc, vc = torch.zeros(4, bs, G, dk, dtype=dtype, device=DEV), torch.zeros(4, bs, G, dv, dtype=dtype, device=DEV)
    for p in range(T):
        kc[table[p // bs], p % bs], vc[table[p // bs], p % bs] = keys[p].to(DEV), vals[p].to(DEV)
    kp, vp = torch.full((4, per, G, dk), 9.0, device=DEV), torch.full((4, per, G, dv), -9.0, device=DEV)
    for at, n in _portions(T, [61, 1, 2, 70, 3]):
        ops.pooled_cache_update(kc, vc, kp, vp, batch_of([dict(tokens=[0] * n, start=at, block_table=table, state_slot=-1, want=[])]), pool)
    owned = set()
    for b in range(T // pool):
        end = b * pool + pool - 1
        page = end // bs
        place = (table[page], b - (page * bs) // pool)
        owned.add(place)
        close(kp[place], keys[b * pool:end + 1].to(F64).mean(0), 2e-6, f"mean key of block {b}")
        close(vp[place], vals[b * pool:end + 1].to(F64).mean(0), 2e-6, f"mean value of block {b}")
    for blk in range(4):
        for j in range(per):
            if (blk, j) not in owned:
                assert float(kp[blk, j].min()) == 9.0 and float(vp[blk, j].max()) == -9.0


def test_a_loud_token_is_seen_through_its_window_then_not_then_through_its_block():
    """one token with a loud value: inside the window it dominates the row, after leaving the window it is invisible until its block of `pool`
    positions is wholly before the window, from then on it counts with weight 1 / pool inside the block's mean -- in a prompt and token by token"""
    H, G, dk, window, pool, loud = 2, 1, 8, 10, 6, 61            # block 10 = positions 60..65 straddles the border between the first two pages
    L = S.dofevik_pooled_layer(H, G, dk, window=window, pool=pool)
    w = {k[7:]: v for k, v in S.dofevik_weights(S.dofevik_config(24, 10, [L]), 1).items() if k.startswith("l0.mix.")}
    g = torch.Generator().manual_seed(0)
    h = torch.randn(140, 24, generator=g) * 0.1
    h[loud] *= 3000.0
    mix = PooledWindowAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, G, dk, L["mixer"]["scale"], 1e-6, torch.float32, window=window, pool=pool)
    want = O.mixer_attention_2(h.to(F64), torch.arange(140), w, L["mixer"], 1e-6)
    for sizes in ([140], [66, 1], [3]):
        got = run_mixer(mix, h, sizes, [1, 0, 2], torch.float32)
        close(got, want, 2e-5, f"portions {sizes}")
    size = want.abs().max(-1).values
    assert float(size[loud + window - 1]) > 5 * float(size[loud + window])           # the last row that sees the token itself, the first that does not
    first_block_row = 65 + window                                                      # block 60..65 ends at 65: seen from position 65 + window on
    assert first_block_row > loud + window                                             # rows in between see neither the token nor its block
    assert float(size[first_block_row]) > 5 * float(size[first_block_row - 1])
    assert float(size[139]) > 5 * float(size[first_block_row - 1])                     # and it stays visible, far away


LATENT = [  # H, dn, dr, dv, R, Rq, window
    (4, 12, 8, 20, 40, 28, 33), (1, 32, 4, 24, 136, 9, 0), (3, 6, 2, 10, 34, 50, 1), (5, 10, 6, 6, 20, 16, 64), (2, 8, 8, 8, 24, 24, 100),
]


@pytest.mark.parametrize("H,dn,dr,dv,R,Rq,window", LATENT)
@pytest.mark.parametrize("sizes", [[260], [2], [61, 1, 1, 2, 70, 3]])
def test_latent_attention_with_query_latent_window_and_element_gate(H, dn, dr, dv, R, Rq, window, sizes):
    g = torch.Generator().manual_seed(R + window)
    L = S.dofevik_latent_layer(H, dn, dr, dv, R, Rq, window=window, base=500.0)
    w = {k[7:]: v for k, v in S.dofevik_weights(S.dofevik_config(56, 10, [L]), 7).items() if k.startswith("l0.mix.")}
    T = 130 if sizes == [2] else 260
    h = torch.randn(T, 56, generator=g)
    m = L["mixer"]
    mix = LatentAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, dn, dr, dv, R, m["scale"], 1e-6, torch.float32, rot=m["rot"], window=window, max_pos=64, q_rank=Rq,
                               gate="element")
    got = run_mixer(mix, h, sizes, [3, 1, 4, 0, 2], torch.float32)
    close(got, O.mixer_latent_attention(h.to(F64), torch.arange(T), w, m, 1e-6), 3e-5, f"latent attention, portions {sizes}")


MOE = [  # D, experts, ff, top, shared_ff
    (40, 5, 24, 2, 36), (64, 8, 64, 3, 0), (52, 3, 18, 3, 10), (72, 7, 10, 1, 48), (128, 6, 64, 2, 128),
]


@pytest.mark.parametrize("D,E,ff,top,sff", MOE)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_biased_router_ungated_experts_and_shared_expert(D, E, ff, top, sff, dtype, tol):
    """router biases large enough to change the choice; T = 3 rows (every pair streams its expert) and T = 200 (bf16 with 8-aligned sizes: pairs sorted by
    expert on the tensor-core GEMM).  The inputs are bf16-representable and the router is peaked, so both dtypes choose the same experts."""
    g = torch.Generator().manual_seed(D + E)
    L = S.dofevik_attention_layer(2, 1, 8, 8, experts=E, ff=ff, top=top, shared_ff=sff)
    w = {k[7:]: v for k, v in S.dofevik_weights(S.dofevik_config(D, 10, [L]), 11).items() if k.startswith("l0.mlp.")}
    w["router.b"] = (torch.randn(E, generator=g) * 2).to(torch.bfloat16)
    wd = {k: v.to(DEV) for k, v in w.items()}
    moe = RoutedExperts(wd, E, 0, top, 1.0, dtype, act="relu2")
    shared = UngatedMlp({"up": wd["shared.up"], "down": wd["shared.down"]}, dtype) if sff else None
    for T in (3, 200):
        h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
        z = h.to(F64) @ w["router"].to(F64).T + w["router.b"].to(F64)
        srt = z.sort(-1, descending=True).values
        keep = (srt[:, top - 1] - srt[:, top]) > 0.05 if top < E else torch.ones(T, dtype=torch.bool)       # rows without a near-tie at the cut
        assert int(keep.sum()) > 0.7 * T
        hd = dev(h, dtype)
        got = moe.forward(hd, dev(h))
        if shared is not None:
            got = got + shared.forward(hd)
        want = O.moe(h.to(F64), w, L["mlp"])
        close(got[keep.to(DEV)], want[keep], tol, f"{T} rows")
        without_bias = O.moe(h.to(F64), {k: v for k, v in w.items() if k != "router.b"}, L["mlp"])
        if T == 200:                                         # among many rows the bias changes choices: the result moves by far more than rounding
            assert float((want - without_bias).abs().max()) > 0.05 * float(want.abs().max())


# ----------------------------------------------------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------------------------------------------------
CONFIGS = {
    # all three mixers, pools that straddle pages, partial rotation with scaling, a layer without a shared expert
    "mix": S.dofevik_config(96, 131, [S.dofevik_pooled_layer(6, 3, 16, window=40, pool=7, experts=5, ff=24, top=2, shared_ff=40),
                                      S.dofevik_latent_layer(4, 12, 8, 20, 40, 28, window=33, experts=4, ff=16, top=3),
                                      S.dofevik_attention_layer(6, 2, 20, 12, window=50, rot_dims=12, factor=4.0, base=5000.0, experts=6, ff=32, top=2, shared_ff=24),
                                      S.dofevik_pooled_layer(2, 2, 24, window=70, pool=64, experts=3, ff=40, top=1, shared_ff=8)]),
    # odd sizes everywhere, attention first, a pool of one and one larger than a page, a window of one, rotation over the whole head without scaling,
    # layers without feed-forward and without masks, top == experts, one kv head, kv heads == heads
    "odd": S.dofevik_config(52, 61, [S.dofevik_attention_layer(3, 3, 10, 14, window=1, rot_dims=10, experts=3, ff=18, top=3),
                                     S.dofevik_pooled_layer(5, 1, 6, window=9, pool=1),
                                     S.dofevik_latent_layer(2, 6, 2, 22, 34, 11, experts=2, ff=44, top=1, shared_ff=6),
                                     S.dofevik_pooled_layer(3, 3, 14, window=11, pool=70, experts=7, ff=10, top=4, shared_ff=30),
                                     S.dofevik_attention_layer(4, 1, 6, 6, experts=2, ff=12, top=2, shared_ff=12),
                                     S.dofevik_pooled_layer(2, 1, 10)], eps=1e-5),
    # 8-aligned sizes: in bf16 the expert products and the latent up-projections take the tensor-core routes
    "aligned": S.dofevik_config(128, 200, [S.dofevik_latent_layer(4, 64, 16, 32, 64, 72, window=90, experts=6, ff=64, top=2, shared_ff=64),
                                           S.dofevik_pooled_layer(4, 2, 32, window=48, pool=16, experts=4, ff=128, top=2, shared_ff=128),
                                           S.dofevik_attention_layer(4, 2, 32, 32, window=100, rot_dims=32, factor=2.0, experts=3, ff=64, top=2)]),
}
_CACHE = {}
TOL = {torch.float32: 2e-4, torch.bfloat16: 8e-2}


def model_and_oracle(name, dtype, n_tokens, seed=0):
    cfg = CONFIGS[name]
    key = (name, seed)
    if key not in _CACHE:
        w = S.dofevik_weights(cfg, seed)
        toks = torch.randint(0, cfg["vocab"], (300,), generator=torch.Generator().manual_seed(seed + 1)).tolist()
        _CACHE[key] = (w, toks, O.forward(toks, cfg, w))
    w, toks, ref = _CACHE[key]
    model = DofevikModel(DofevikConfig.from_dict(cfg), w, dtype=dtype, block_size=64, max_pos=128, device=DEV)
    return model, toks[:n_tokens], ref[:n_tokens]


def run_schedule(runner, seq_id, toks, sizes):
    runner.admit(seq_id)
    out = []
    for at, n in _portions(len(toks), sizes):
        out.append(runner.execute([dict(seq_id=seq_id, tokens=toks[at:at + n], want=list(range(n)))]))
    runner.release(seq_id)
    return torch.cat(out)


def row_errors(got, want):
    """per position: rms over the vocabulary of the centred difference, relative to the rms of the reference logits"""
    d = got.detach().cpu().to(F64) - want
    d = d - d.mean(-1, keepdim=True)
    return torch.sqrt((d * d).mean(-1)) / torch.sqrt((want * want).mean())


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_oracle(name):
    model, toks, ref = model_and_oracle(name, torch.float32, 230)
    runner = ModelRunner(model, 8, 2, 64)
    trace = []
    runner.admit(0)
    got = runner.execute([dict(seq_id=0, tokens=toks, want=list(range(len(toks))))], hidden_trace=trace)
    close(got, ref, TOL[torch.float32], f"{name} logits")
    want_trace = []
    O.forward(toks, CONFIGS[name], _CACHE[(name, 0)][0], want_trace)
    assert len(trace) == len(want_trace) == len(CONFIGS[name]["layers"])
    for i, (a, b) in enumerate(zip(trace, want_trace)):
        close(a, b, 1e-4, f"{name} stream after layer {i}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bf16_stays_within_rounding(name):
    """bf16 operands may flip a router's near-tie at a few positions, so the bound is on the typical position, with a loose cap on all"""
    model, toks, ref = model_and_oracle(name, torch.bfloat16, 230)
    runner = ModelRunner(model, 8, 2, 64)
    whole = run_schedule(runner, 0, toks, [230])
    parts = run_schedule(runner, 1, toks, [37, 2, 1, 1, 64])
    for got in (whole, parts):
        e = row_errors(got, ref)
        assert float(e.median()) < 0.03 and float(e.quantile(0.9)) < 0.08, (float(e.median()), float(e.quantile(0.9)))


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("sizes", [[1], [2], [3, 2, 7], [64, 1, 1, 5], [39, 1, 41, 2, 63]])
def test_portions_and_decoding_match_the_whole_prompt(name, sizes):
    model, toks, ref = model_and_oracle(name, torch.float32, 200)
    runner = ModelRunner(model, 4, 1, 64)
    close(run_schedule(runner, 5, toks, sizes), ref, TOL[torch.float32], f"{name} portions {sizes}")


@pytest.mark.parametrize("name", ["mix", "odd"])
def test_unequal_batches_match_each_request_alone(name):
    """Requests of different lengths advance together, portions of some beside single tokens of others; the pool of pages is smaller than the sum of
    all requests, so pages (with the pooled entries they carry) go from finished requests to later ones."""
    cfg = CONFIGS[name]
    w = S.dofevik_weights(cfg, 0)
    model = DofevikModel(DofevikConfig.from_dict(cfg), w, dtype=torch.float32, block_size=64, max_pos=512, device=DEV)
    g = torch.Generator().manual_seed(9)
    lens = [130, 7, 64, 201, 65, 1, 90]
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    refs = [O.forward(s, cfg, w) for s in seqs]
    runner = ModelRunner(model, 9, 3, 64)
    plans = [[64, 1, 1, 30, 2, 1], [2, 1], [63, 1], [100, 3, 1, 1, 50, 2], [64, 1], [1], [1, 1, 1, 80, 2]]
    waiting, live, got = list(range(len(seqs))), {}, {i: [] for i in range(len(seqs))}
    guard = 0
    while waiting or live:
        guard += 1
        assert guard < 500
        while waiting and runner.state.pool.num_free() > 0 and runner.can_admit(lens[waiting[0]], sum(-(-lens[i] // 64) - len(runner.blocks.tables.get(i, ())) for i in live)):
            i = waiting.pop(0)
            runner.admit(i)
            live[i] = [0, 0]
        entries = []
        for i, (fed, pi) in live.items():
            n = min(plans[i][pi % len(plans[i])] if pi < len(plans[i]) else 1, lens[i] - fed)
            entries.append(dict(seq_id=i, tokens=seqs[i][fed:fed + n], want=list(range(n))))
        out = runner.execute(entries)
        at = 0
        for e in entries:
            i, n = e["seq_id"], len(e["tokens"])
            got[i].append(out[at:at + n]); at += n
            live[i][0] += n; live[i][1] += 1
        for i in [i for i, (fed, _) in live.items() if fed == lens[i]]:
            runner.release(i); del live[i]
    for i in range(len(seqs)):
        close(torch.cat(got[i]), refs[i], TOL[torch.float32], f"{name} request {i} in a batch")
    runner.blocks.check_invariants()
    assert runner.blocks.num_free_gpu_blocks() == 9 and runner.state.pool.num_free() == 3


def test_long_decoding_across_pages_windows_and_pooled_blocks():
    model, toks, ref = model_and_oracle("mix", torch.float32, 300)
    runner = ModelRunner(model, 5, 1, 64)
    runner.admit(0)
    got = [runner.execute([dict(seq_id=0, tokens=toks[:20], want=list(range(20)))])]
    for t in range(20, 300):
        got.append(runner.execute([dict(seq_id=0, tokens=[toks[t]], want=[0])]))
    close(torch.cat(got), ref, TOL[torch.float32], "280 decoded tokens")


def test_first_tokens_and_single_token_requests():
    model, toks, ref = model_and_oracle("odd", torch.float32, 230)
    runner = ModelRunner(model, 4, 2, 64)
    for n in (1, 2, 3):
        runner.admit(n)
        close(runner.execute([dict(seq_id=n, tokens=toks[:n], want=list(range(n)))]), ref[:n], TOL[torch.float32], f"first {n} tokens")
        runner.release(n)


def test_many_rows_take_the_tensor_core_routes():
    """a bf16 step with hundreds of rows and 8-aligned sizes against the same rows in steps of a few tokens (streaming kernels): both stay within rounding of
    the oracle and of each other"""
    cfg = CONFIGS["aligned"]
    w = S.dofevik_weights(cfg, 2)
    toks = torch.randint(0, 200, (420,), generator=torch.Generator().manual_seed(4)).tolist()
    ref = O.forward(toks, cfg, w)
    model = DofevikModel(DofevikConfig.from_dict(cfg), w, dtype=torch.bfloat16, block_size=64, max_pos=512, device=DEV)
    assert model.layers[0].mixer.grouped and model.layers[0].mlp.grouped
    runner = ModelRunner(model, 14, 2, 64)
    big = run_schedule(runner, 0, toks, [420])
    mid = run_schedule(runner, 1, toks, [300, 1, 119])
    small = run_schedule(runner, 2, toks, [9, 1, 30])
    for got in (big, mid, small):
        e = row_errors(got, ref)
        assert float(e.median()) < 0.03 and float(e.quantile(0.9)) < 0.08, (float(e.median()), float(e.quantile(0.9)))
    e = row_errors(big, small.detach().cpu().to(F64))
    assert float(e.median()) < 0.03


def test_wide_heads_and_wide_latent_as_a_whole_model_in_unequal_batches():
    """128-wide heads and a 512 + 64 latent: in bf16 the paged attentions run on the tensor-core kernel and the latent rows on the split-KV kernel, in f32
    on the plain kernels.  Every expert is chosen (top == experts), so no near-tie of a router can move a row: all rows of all requests stay within rounding
    of the oracle, whole, in portions, and side by side with other requests over pages that change hands."""
    cfg = S.dofevik_config(256, 333, [S.dofevik_pooled_layer(4, 2, 128, window=130, pool=9, scale=0.09, experts=3, ff=64, top=3, shared_ff=128),
                                      S.dofevik_attention_layer(4, 1, 128, 128, window=200, rot_dims=64, base=3e5, factor=2.0, scale=0.09, experts=3, ff=64, top=3),
                                      S.dofevik_latent_layer(2, 128, 64, 128, 512, 192, window=150, scale=0.07, experts=3, ff=64, top=3, shared_ff=64)])
    w = S.dofevik_weights(cfg, 6)
    g = torch.Generator().manual_seed(8)
    lens = [470, 131, 3, 260]
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    refs = [O.forward(s, cfg, w) for s in seqs]
    plans = [[300, 1, 1, 64, 2], [1, 1, 129], [2, 1], [130, 1, 1, 1, 70, 57]]
    for dtype, cap in ((torch.float32, 2e-4), (torch.bfloat16, 0.05)):
        model = DofevikModel(DofevikConfig.from_dict(cfg), w, dtype=dtype, block_size=64, max_pos=512, device=DEV)
        runner = ModelRunner(model, 18, 4, 64)
        whole = run_schedule(runner, 9, seqs[0], [lens[0]])
        assert float(row_errors(whole, refs[0]).max()) < cap, (dtype, "whole", float(row_errors(whole, refs[0]).max()))
        fed, step, got = [0] * 4, 0, [[] for _ in lens]
        for i in range(4):
            runner.admit(i)
        while any(f < n for f, n in zip(fed, lens)):
            entries = []
            for i, n in enumerate(lens):
                if fed[i] < n and not (i == 1 and step % 3 == 1):               # request 1 sits out every third step
                    k = min(plans[i][step] if step < len(plans[i]) else 1, n - fed[i])
                    entries.append(dict(seq_id=i, tokens=seqs[i][fed[i]:fed[i] + k], want=list(range(k))))
            out, at = runner.execute(entries), 0
            for e in entries:
                k = len(e["tokens"])
                got[e["seq_id"]].append(out[at:at + k]); at += k; fed[e["seq_id"]] += k
            step += 1
        for i in range(4):
            e = row_errors(torch.cat(got[i]), refs[i])
            assert float(e.max()) < cap, (dtype, i, int(e.argmax()), float(e.max()))


WIDE = [  # kind, H, G, window, pool: 128-wide heads in bf16 take the tensor-core kernel (its sink, its sigmoid form, its pooled tiles)
    ("attention", 4, 2, 100, 0), ("attention", 2, 2, 0, 0), ("attention", 4, 1, 64, 0),
    ("pooled", 4, 2, 70, 2), ("pooled", 2, 1, 100, 16), ("pooled", 2, 2, 0, 0), ("pooled", 3, 3, 33, 0), ("pooled", 2, 2, 5, 1), ("pooled", 2, 1, 64, 64),
]


@pytest.mark.parametrize("kind,H,G,window,pool", WIDE)
def test_wide_heads_on_the_tensor_core_kernel_match_the_oracle_and_the_plain_kernel(kind, H, G, window, pool):
    """bf16 with 128-wide heads: whole prompt, portions (tiles that start inside a page, single rows) and the f32 run of the SIMT kernels all agree with the
    oracle; pool 2 with window 70 gives a row up to 175 pooled entries (three pooled tiles), pool 1 entries in every page slot"""
    g = torch.Generator().manual_seed(H * 7 + window + pool)
    D, T, dk = 64, 420, 128
    if kind == "attention":
        L = S.dofevik_attention_layer(H, G, dk, dk, window=window, rot_dims=64, factor=2.0, scale=2.0 * dk ** -0.5)
    else:
        L = S.dofevik_pooled_layer(H, G, dk, window=window, pool=pool, scale=2.0 * dk ** -0.5)
    w = {k[7:]: v for k, v in S.dofevik_weights(S.dofevik_config(D, 10, [L]), 13).items() if k.startswith("l0.mix.")}
    if kind == "attention":
        w["sink"] = torch.tensor([3.0, -1.0, 5.0, 0.5][:H]).to(torch.bfloat16)
    elif pool == 16:
        w["pb"] = torch.tensor([-6.0, -5.5]).to(torch.bfloat16)            # weights of a few thousandths: their relative accuracy must hold
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    m = L["mixer"]
    want = (O.mixer_attention if kind == "attention" else O.mixer_attention_2)(h.to(F64), torch.arange(T), w, m, 1e-6)

    def make(dtype):
        wd = {k: v.to(DEV) for k, v in w.items()}
        if kind == "attention":
            return PagedAttentionMixer(wd, H, G, dk, dk, m["scale"], 1e-6, dtype, rot=m.get("rot"), window=window, max_pos=512, head_norm="after", interleaved=True)
        return PooledWindowAttentionMixer(wd, H, G, dk, m["scale"], 1e-6, dtype, window=window, pool=pool)
    close(run_mixer(make(torch.float32), h, [420], [3, 1, 4, 0, 2, 6, 5], torch.float32), want, 3e-5, "f32 on the plain kernel")
    mix = make(torch.bfloat16)
    assert mix.q_dtype == torch.bfloat16
    scale = float(want.abs().max())
    for sizes in ([420], [100, 1, 37, 2, 64]):
        got = run_mixer(mix, h, sizes, [3, 1, 4, 0, 2, 6, 5], torch.bfloat16).float().cpu().to(F64)
        err = (got - want).abs().max(-1).values / scale
        assert float(err.max()) < 4e-2 and float(err.median()) < 1.2e-2, (sizes, float(err.max()), float(err.median()))


@pytest.mark.parametrize("window", [0, 1, 31, 100, 256, 300])
def test_latent_rows_on_the_split_kv_kernel_with_a_window(window):
    """latent 512 + rotated 64 in bf16: steps of 16 and more rows run on the split-KV tensor-core kernel of the latent cache, every row as a sequence of its
    own whose keys start at the window's edge (inside a tile, at a tile's border, beyond one 256-key run); fewer rows stay on the SIMT kernel"""
    g = torch.Generator().manual_seed(window)
    H, dn, dr, dv, R, Rq, D, T = 3, 64, 64, 32, 512, 96, 64, 420
    L = S.dofevik_latent_layer(H, dn, dr, dv, R, Rq, window=window, base=1e4)
    w = {k[7:]: v for k, v in S.dofevik_weights(S.dofevik_config(D, 10, [L]), 17).items() if k.startswith("l0.mix.")}
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    m = L["mixer"]
    want = O.mixer_latent_attention(h.to(F64), torch.arange(T), w, m, 1e-6)
    mix = LatentAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, dn, dr, dv, R, m["scale"], 1e-6, torch.bfloat16, rot=m["rot"], window=window, max_pos=512, q_rank=Rq,
                               gate="element")
    assert mix.decode_kernel
    scale = float(want.abs().max())
    for sizes in ([420], [100, 1, 37, 2, 64, 16]):
        got = run_mixer(mix, h, sizes, [3, 1, 4, 0, 2, 6, 5], torch.bfloat16).float().cpu().to(F64)
        err = (got - want).abs().max(-1).values / scale
        assert float(err.max()) < 4e-2 and float(err.median()) < 1.2e-2, (sizes, float(err.max()), float(err.median()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_engine(dtype, tmp_path):
    """checkpoint on disk -> registry -> LLMEngine (scheduler, chunked prefill, sampler) against the oracle's greedy continuation"""
    from candle_vllm_b200.safetensors_io import save_file
    cfg = CONFIGS["mix"]
    w = S.dofevik_weights(cfg, 4)
    save_file(w, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (70, 3, 33, 1, 129)]
    eng = LLMEngine.from_pretrained(str(tmp_path), dtype=dtype, num_blocks=7, max_num_seqs=2, prefill_chunk=48, max_batch_tokens=64, max_model_len=256)
    assert type(eng.model).__name__ == "DofevikModel"
    outs = eng.generate(prompts, pkg.SamplingParams(max_tokens=6))
    assert eng.runner.blocks.num_free_gpu_blocks() == 7 and eng.runner.state.pool.num_free() == 2
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        if dtype == torch.float32:
            assert o == O.greedy(cfg, w, p, 6)
        else:
            assert all(0 <= t < cfg["vocab"] for t in o)


def test_graph_replay_of_decode_steps_matches_eager():
    cfg = CONFIGS["mix"]
    w = S.dofevik_weights(cfg, 0)
    model = DofevikModel(DofevikConfig.from_dict(cfg), w, dtype=torch.float32, block_size=64, max_pos=64, device=DEV)      # tables must grow
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (100, 140)]
    refs = [O.forward(s, cfg, w) for s in seqs]
    runner = ModelRunner(model, 6, 2, 64, decode_graphs=True)
    got = [[], []]
    runner.admit(0); runner.admit(1)
    out = runner.execute([dict(seq_id=0, tokens=seqs[0][:50], want=list(range(50))), dict(seq_id=1, tokens=seqs[1][:61], want=list(range(61)))])
    got[0].append(out[:50]); got[1].append(out[50:])
    fed = [50, 61]
    while fed[0] < 100 or fed[1] < 140:
        live = [i for i in (0, 1) if fed[i] < len(seqs[i])]
        out = runner.execute([dict(seq_id=i, tokens=[seqs[i][fed[i]]], want=[0]) for i in live]).clone()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1]); fed[i] += 1
    assert 1 in runner._graphs
    for i in (0, 1):
        close(torch.cat(got[i]), refs[i], TOL[torch.float32], f"graph replay, request {i}")


def test_command_line_and_trace_runner(tmp_path):
    """the two programs a user starts, as child processes on a checkpoint on disk"""
    from candle_vllm_b200.safetensors_io import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CONFIGS["odd"]
    w = S.dofevik_weights(cfg, 1)
    save_file(w, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "candle_vllm_b200", "generate", "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids", "5,6,7,8", "--max-new-tokens", "5"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout.strip().splitlines()[-1])["output"] == O.greedy(cfg, w, [5, 6, 7, 8], 5)
    a, b = list(range(3, 43)), [9, 8, 7]
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:30], want=[0, 29]), dict(id="b", tokens=b[:1], want=[0])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[30:], want=[9]), dict(id="b", tokens=b[1:2], want=[])], end=["a"]),
             dict(step=2, entries=[dict(id="b", tokens=b[2:], want=[0]), dict(id="c", tokens=a[:2], want=[1])], end=["b"]),
             # a step in which nothing is wanted, by a new request under the name of a finished one; then its next token
             dict(step=3, entries=[dict(id="a", tokens=b[:2], want=[]), dict(id="c", tokens=a[2:5], want=[])], end=[]),
             dict(step=4, entries=[dict(id="a", tokens=b[2:], want=[0])], end=["a", "c"])]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    assert not (out / "3.f32").exists()
    ra, rb = O.forward(a, cfg, w), O.forward(b, cfg, w)
    V = cfg["vocab"]
    s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    close(s0, torch.stack([ra[0], ra[29], rb[0]]), TOL[torch.float32], "step 0")
    s1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
    close(s1, ra[39:40], TOL[torch.float32], "step 1")
    s2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    close(s2, torch.stack([rb[2], ra[1]]), TOL[torch.float32], "step 2")
    s4 = torch.from_numpy(np.fromfile(out / "4.f32", dtype="<f4").reshape(-1, V))
    close(s4, rb[2:3], TOL[torch.float32], "step 4")
