"""GPU parity: the whole decode step (GGUFLLaMa::forward_inner) through b200_llama_decode vs the
numpy oracle on a small synthetic model; greedy tokens and logits.  Tolerance: logits within 1e-3
(normalised by max|logit|) of the fp oracle."""
import numpy as np
import pytest
import torch

import candle_vllm_b200 as pkg
from candle_vllm_b200 import synthetic
from oracle import llama as OL
from tests.gpu_util import DEV, weights_to_oracle

pytestmark = pytest.mark.gpu


def _small_cfg(**kw):
    d = dict(hidden=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128, ffn=1024, vocab=768,
             max_pos=512, block_size=16, max_num_seqs=8, max_blocks_per_seq=16)
    d.update(kw)
    return pkg.LlamaConfig(**d)


def _ocfg(cfg):
    return dict(hidden=cfg.hidden, heads=cfg.num_heads, kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                rms_eps=cfg.rms_eps, max_pos=cfg.max_pos, rope_theta=cfg.rope_theta)


@pytest.fixture(params=[0, 1, 2], ids=["per_gemm", "layer_kernel", "split_phases"])
def engine_path(request, monkeypatch):
    """both engine paths: one launch per GEMM (default) and the persistent layer kernel (B200_MEGA=1, read at model creation)"""
    monkeypatch.setenv("B200_MEGA", str(request.param))
    return request.param


@pytest.mark.parametrize("use_graph", [False, True])
def test_decode_steps_match_oracle(use_graph, engine_path):
    cfg = _small_cfg()
    w = synthetic.make_weights(cfg, DEV, seed=0)
    ow = weights_to_oracle(w)
    nb = 40
    eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, pkg.CacheConfig(cfg.block_size, nb))
    synthetic.fill_kv_cache(eng.gpu_cache, seed=1)
    okc = [k.float().cpu().numpy().copy() for k, _ in eng.gpu_cache]
    ovc = [v.float().cpu().numpy().copy() for _, v in eng.gpu_cache]
    model = pkg.GGUFLLaMa(cfg, w, eng.gpu_cache, use_graph=use_graph)
    assert model.uses_layer_kernel(5) == bool(engine_path)
    B = 5
    lens = [1, 16, 17, 40, 100]
    tables = synthetic.random_block_tables(B, 8, nb, seed=2)
    tokens = [5, 700, 33, 0, 123]
    for step in range(3):
        prep = pkg.prepare_decode(lens, tokens, tables, cfg.block_size)
        nxt, logits = model.decode(prep, want_logits=True)
        ref = OL.forward(_ocfg(cfg), ow, prep["tokens"].astype(np.int64), prep["positions"], okc, ovc,
                         dict(slot_mapping=prep["slot_mapping"], block_tables=prep["block_tables"], context_lens=prep["context_lens"]))
        scale = np.abs(ref).max()
        err = np.abs(logits - ref).max() / scale
        assert err < 1e-3, (step, err)
        # greedy tokens agree wherever the oracle's top-1 margin exceeds the logit error bound
        for b in range(B):
            if nxt[b] != ref[b].argmax():
                assert ref[b].max() - ref[b, nxt[b]] <= 2 * err * scale, (step, b)
        # the engine wrote this step's K/V into the paged cache exactly where the oracle did
        for l in range(cfg.num_layers):
            assert np.abs(eng.gpu_cache[l][0].float().cpu().numpy() - okc[l]).max() < 2e-2
        tokens = [int(t) for t in ref.argmax(axis=1)]
        lens = [L + 1 for L in lens]


def test_decode_at_metric_shapes_matches_oracle(engine_path):
    """The exact code path bench.py times, at the metric's shapes: hidden 4096, ffn 14336, 32 q / 8 kv
    heads, fused 3-segment QKV (n = 4096 + 1024 + 1024), stream-K splits accumulating into the residual, Q6_K lm_head
    (16 384 rows), B = 32, ctx ~ 4 k over 80-block tables, CUDA graph on.  Two layers keep the numpy oracle to ~1 minute;
    layer count does not change any kernel's shape.
    Tolerance: rel-Frobenius < 2e-3 and max|err| / max|logit| < 5e-3 (the worst of 524 288 logits) against the exact (fp64
    dequant-matmul) oracle; measured on B200: 1.2e-3 / 1.5e-3 at step 0, 1.4e-3 / 3.2e-3 at step 1.  Why not the
    1e-3 of the small-model test: at these sizes the QMatMul contract itself (activations and dequantised weights rounded once to
    fp16, exact accumulation) is 0.8e-3 / 0.8e-3 away from the exact result and the reference's own
    Q8-activation arithmetic is 5e-3 away (tools/emulate_rounding.py, CPU only; numbers in profiles/r02_rounding_floor.md); the bf16
    roundings of q, k, v, P and the attention output add the rest."""
    cfg = pkg.LlamaConfig(hidden=4096, num_layers=2, num_heads=32, num_kv_heads=8, head_dim=128, ffn=14336, vocab=16384,
                          max_pos=5248, block_size=64, max_num_seqs=32, max_blocks_per_seq=80)
    w = synthetic.make_weights(cfg, DEV, seed=0)
    ow = weights_to_oracle(w)
    B, nb = 32, 32 * 80 + 8
    eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, pkg.CacheConfig(cfg.block_size, nb))
    synthetic.fill_kv_cache(eng.gpu_cache, seed=1)
    okc = [k.float().cpu().numpy() for k, _ in eng.gpu_cache]
    ovc = [v.float().cpu().numpy() for _, v in eng.gpu_cache]
    model = pkg.GGUFLLaMa(cfg, w, eng.gpu_cache, use_graph=True)
    assert model.uses_layer_kernel(B) == bool(engine_path)
    rng = np.random.default_rng(5)
    lens = [int(x) for x in rng.integers(3900, 4300, B)]
    lens[0], lens[1], lens[2], lens[3] = 1, 4096, 4097, 5118          # a fresh sequence, a block boundary, one past it, the table's last block
    tables = synthetic.random_block_tables(B, 80, nb, seed=2)
    tokens = [int(t) for t in rng.integers(0, cfg.vocab, B)]
    for step in range(2):                                             # step 0 captures the graph, step 1 replays it
        prep = pkg.prepare_decode(lens, tokens, tables, cfg.block_size)
        nxt, logits = model.decode(prep, want_logits=True)
        ref = OL.forward(_ocfg(cfg), ow, prep["tokens"].astype(np.int64), prep["positions"], okc, ovc,
                         dict(slot_mapping=prep["slot_mapping"], block_tables=prep["block_tables"], context_lens=prep["context_lens"]))
        scale = np.abs(ref).max()
        err = np.abs(logits - ref).max() / scale
        fro = np.linalg.norm(logits - ref) / np.linalg.norm(ref)
        print(f"metric shapes step {step}: max err / max = {err:.2e}, rel-Fro = {fro:.2e}, layer kernel = {model.uses_layer_kernel(B)}")
        assert err < 5e-3 and fro < 2e-3, (step, err, fro)
        for b in range(B):
            if nxt[b] != ref[b].argmax():
                assert ref[b].max() - ref[b, nxt[b]] <= 2 * err * scale, (step, b)
        tokens = [int(t) for t in ref.argmax(axis=1)]
        lens = [L + 1 for L in lens]
    # run-to-run: on the persistent layer kernel the split-K partial sums of the layers are added in a fixed order; what is left is the
    # lm_head, which at THIS vocabulary (128 tiles < 4 per SM) splits its tiles over K and meets in fp32 atomics -- at Llama's 128 256
    # rows every CTA owns whole tiles and bench.py's parity leg reports bit-identical logits.  The one-launch-per-GEMM path has
    # atomics in every layer: tiny differences in the fp32 residual flip 16-bit roundings downstream (measured spread 6e-4 here, after
    # two layers).
    prep = pkg.prepare_decode(lens, tokens, tables, cfg.block_size)
    a = model.decode(prep, want_logits=True)[1].copy()
    b_ = model.decode(prep, want_logits=True)[1]      # same inputs again (the step rewrites the same slots with the same values)
    spread = np.abs(a - b_).max() / np.abs(a).max()
    print(f"run-to-run spread {spread:.2e}")
    assert spread < (1e-6 if model.uses_layer_kernel(B) else 2e-3)


@pytest.mark.parametrize("use_graph", [False, True])
def test_decode_with_fp8_kv_cache_matches_oracle(use_graph, engine_path):
    """FP8 (e4m3, scale 1.0) KV cache through the engine: vectorised e4m3 cache write in the fused RoPE kernel + FP8 attention
    (config 3 of BASELINE.json) against the oracle with fp8_kv=True.  The cache bytes must be bit-exact."""
    cfg = _small_cfg(block_size=64, max_blocks_per_seq=8)
    w = synthetic.make_weights(cfg, DEV, seed=0)
    ow = weights_to_oracle(w)
    nb = 32
    eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, pkg.CacheConfig(cfg.block_size, nb, kvcache_dtype="fp8"))
    synthetic.fill_kv_cache(eng.gpu_cache, seed=1)
    okc = [k.cpu().numpy().copy() for k, _ in eng.gpu_cache]          # u8 e4m3 bits
    ovc = [v.cpu().numpy().copy() for _, v in eng.gpu_cache]
    model = pkg.GGUFLLaMa(cfg, w, eng.gpu_cache, kv_dtype=pkg.DType.FP8_E4M3, use_graph=use_graph)
    lens, tokens = [1, 64, 65, 200, 300], [5, 700, 33, 0, 123]
    tables = synthetic.random_block_tables(5, 5, nb, seed=2)
    for step in range(3):
        prep = pkg.prepare_decode(lens, tokens, tables, cfg.block_size)
        nxt, logits = model.decode(prep, want_logits=True)
        ref = OL.forward(_ocfg(cfg), ow, prep["tokens"].astype(np.int64), prep["positions"], okc, ovc,
                         dict(slot_mapping=prep["slot_mapping"], block_tables=prep["block_tables"], context_lens=prep["context_lens"]), fp8_kv=True)
        err = np.abs(logits - ref).max() / np.abs(ref).max()
        assert err < 2e-3, (step, err)
        for l in range(cfg.num_layers):
            mism = (eng.gpu_cache[l][0].cpu().numpy() != okc[l]).mean()
            assert mism < 2e-3, (step, l, mism)         # e4m3 bytes: identical except where our f32 k differs from the oracle's by an ulp
        tokens = [int(t) for t in ref.argmax(axis=1)]
        lens = [L + 1 for L in lens]


def _oracle_dense(w):
    f = lambda t: ("dense", t.float().cpu().numpy())
    return dict(tok_embeddings=w["tok_embeddings"].cpu().numpy(), norm=w["norm"].cpu().numpy(), output=f(w["output"]),
                layers=[dict(attn_norm=l["attn_norm"].cpu().numpy(), ffn_norm=l["ffn_norm"].cpu().numpy(),
                             **{k: f(l[k]) for k in ("wq", "wk", "wv", "wo", "w1", "w2", "w3")}) for l in w["layers"]])


@pytest.mark.parametrize("kind", ["dense_bf16", "dense_f16", "gptq_f16", "gptq_bf16_fp8kv"])
def test_decode_with_other_linear_kinds_matches_oracle(kind):
    """The safetensors models of the reference through the same engine (b200_llama_set_layer_ex): dense 16-bit linears on the tcgen05
    dense GEMM (BASELINE config 2) and GPTQ int4 prepared for Marlin (config 3, here also with the FP8 KV cache), NeoX RoPE.
    Tolerance: 2e-3 of max|logit| (bf16 weights and activations carry 8-bit mantissas; the oracle sees the same 16-bit weight values)."""
    cfg = _small_cfg(block_size=64, max_blocks_per_seq=8)
    fp8 = kind.endswith("fp8kv")
    if kind.startswith("dense"):
        w = synthetic.make_weights_16bit(cfg, DEV, seed=0, dtype=torch.bfloat16 if "bf16" in kind else torch.float16)
        ow = _oracle_dense(w)
    else:
        w, ow = synthetic.make_weights_gptq(cfg, DEV, seed=0, group_size=128, dtype=torch.bfloat16 if "bf16" in kind else torch.float16)
    nb = 32
    eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, pkg.CacheConfig(cfg.block_size, nb, kvcache_dtype="fp8" if fp8 else "auto"))
    synthetic.fill_kv_cache(eng.gpu_cache, seed=1)
    okc = [(k.cpu().numpy() if fp8 else k.float().cpu().numpy()).copy() for k, _ in eng.gpu_cache]
    ovc = [(v.cpu().numpy() if fp8 else v.float().cpu().numpy()).copy() for _, v in eng.gpu_cache]
    model = pkg.GGUFLLaMa(cfg, w, eng.gpu_cache, kv_dtype=pkg.DType.FP8_E4M3 if fp8 else pkg.DType.BF16, rope_neox=True)
    assert not model.uses_layer_kernel(5)
    ocfg = dict(_ocfg(cfg), rope_neox=True)
    lens, tokens = [1, 64, 65, 200, 300], [5, 700, 33, 0, 123]
    tables = synthetic.random_block_tables(5, 5, nb, seed=2)
    for step in range(3):
        prep = pkg.prepare_decode(lens, tokens, tables, cfg.block_size)
        nxt, logits = model.decode(prep, want_logits=True)
        ref = OL.forward(ocfg, ow, prep["tokens"].astype(np.int64), prep["positions"], okc, ovc,
                         dict(slot_mapping=prep["slot_mapping"], block_tables=prep["block_tables"], context_lens=prep["context_lens"]), fp8_kv=fp8)
        scale = np.abs(ref).max()
        err = np.abs(logits - ref).max() / scale
        fro = np.linalg.norm(logits - ref) / np.linalg.norm(ref)
        print(f"{kind} step {step}: max err / max = {err:.2e}, rel-Fro = {fro:.2e}")
        # the synthetic GPTQ model (uniform int4) has weights of mean -s/2: sums with heavy cancellation, so the same operand
        # rounding shows up ~4x larger in the max-normalised error than with the zero-mean dense / GGML models
        assert err < (8e-3 if kind.startswith("gptq") else 2e-3) and fro < (6e-3 if kind.startswith("gptq") else 2e-3), (kind, step, err, fro)
        for b in range(5):
            if nxt[b] != ref[b].argmax():
                assert ref[b].max() - ref[b, nxt[b]] <= 2 * err * scale, (step, b)
        tokens = [int(t) for t in ref.argmax(axis=1)]
        lens = [L + 1 for L in lens]


def test_resident_replay_equals_host_driven_steps():
    cfg = _small_cfg()
    w = synthetic.make_weights(cfg, DEV, seed=3)
    nb = 40
    tables = synthetic.random_block_tables(4, 8, nb, seed=4)

    def run(resident):
        eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, pkg.CacheConfig(cfg.block_size, nb))
        synthetic.fill_kv_cache(eng.gpu_cache, seed=5)
        model = pkg.GGUFLLaMa(cfg, w, eng.gpu_cache)
        lens, toks, out = [10, 31, 32, 50], [1, 2, 3, 4], []
        nxt, _ = model.decode(pkg.prepare_decode(lens, toks, tables, cfg.block_size))
        out.append(nxt.copy())
        for _ in range(4):
            if resident:
                model.decode_resident(4, advance=True)
                nxt = model.read_next_tokens(4)
            else:
                lens = [L + 1 for L in lens]
                nxt, _ = model.decode(pkg.prepare_decode(lens, [int(x) for x in nxt], tables, cfg.block_size))
            out.append(np.asarray(nxt).copy())
        return np.stack(out)

    a, b = run(False), run(True)
    assert np.array_equal(a, b)


def test_engine_argument_errors():
    cfg = _small_cfg()
    w = synthetic.make_weights(cfg, DEV, seed=0)
    eng = pkg.CacheEngine(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, pkg.CacheConfig(cfg.block_size, 8))
    model = pkg.GGUFLLaMa(cfg, w, eng.gpu_cache)
    prep = pkg.prepare_decode([3], [cfg.vocab + 5], [[1]], cfg.block_size)
    with pytest.raises(pkg.BackendError, match="vocab"):
        model.decode(prep)
    prep = pkg.prepare_decode([3] * 9, [1] * 9, [[1]] * 9, cfg.block_size)
    with pytest.raises(pkg.BackendError, match="num_seqs"):
        model.decode(prep)
