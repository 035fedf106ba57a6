"""Dofevik without a GPU: configuration reading, the registry and build group, the synthetic checkpoints, the rotary tables with linear scaling, where
pooled entries live in their pages, the cache engine's pooled tensors, and properties of the float64 oracle that the GPU tests rely on."""
import json

import numpy as np
import pytest
import torch

import candle_vllm_b200 as pkg
from candle_vllm_b200 import _lib, registry, seq_ops as ops, synthetic as S
from candle_vllm_b200.dofevik import DofevikConfig
from candle_vllm_b200.mixers import yarn_rotary_tables
from oracle import dofevik as O

F64 = torch.float64


def _cfg():
    return S.dofevik_config(48, 37, [S.dofevik_attention_layer(4, 2, 8, 6, window=5, rot_dims=4, factor=2.0, experts=3, ff=8, top=2, shared_ff=12),
                                     S.dofevik_pooled_layer(2, 1, 6, window=7, pool=3), S.dofevik_latent_layer(2, 4, 2, 6, 10, 8, window=4, experts=2, ff=6, top=1)])


def test_registered_with_a_build_group_of_its_own(tmp_path):
    assert "Dofevik" in registry.registered()
    (tmp_path / "config.json").write_text(json.dumps(_cfg()))
    group = registry.build_group_of(str(tmp_path))
    assert group == "window" and set(_lib.GROUP_SYMBOLS[group]) <= set(_lib.SYMBOLS)
    import importlib.util, os
    spec = importlib.util.spec_from_file_location("b200_build", os.path.join(os.path.dirname(_lib.__file__), "build.py"))
    b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b)
    assert all(os.path.exists(os.path.join(b.CSRC, n + ".cu")) for n in b.GROUPS[group])


def test_config_is_read_and_checked():
    cfg = DofevikConfig.from_dict(_cfg())
    assert (cfg.vocab, cfg.width, len(cfg.layers)) == (37, 48, 3)
    for breaker, text in [(lambda d: d["layers"][0].update(type="conv"), "unknown mixer"), (lambda d: d["layers"][1]["mixer"].update(vdim=9), "values are the keys"),
                          (lambda d: d["layers"][2]["mixer"].pop("q_rank"), "lacks"), (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "feed-forward kind"),
                          (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=4), "rotation spans"), (lambda d: d.pop("norm"), "lacks")]:
        d = json.loads(json.dumps(_cfg()))
        breaker(d)
        with pytest.raises(pkg.BackendError, match=text):
            DofevikConfig.from_dict(d)


def test_synthetic_checkpoint_has_the_tensors_the_oracle_reads():
    cfg = _cfg()
    w = S.dofevik_weights(cfg, 0)
    assert w["l0.norm1"].shape == () and w["final.norm"].shape == () and w["l0.mix.sink"].shape == (4,) and w["l1.mix.pb"].shape == (2,)
    assert "l1.mlp.router" not in w and "l2.mlp.shared.up" not in w and w["l0.mlp.shared.up"].shape == (12, 48)
    hidden = []
    lg = O.forward(list(range(20)), cfg, w, hidden)
    assert lg.shape == (20, 37) and len(hidden) == 3 and bool(torch.isfinite(lg).all())
    # causal: a later token changes no earlier row
    lg2 = O.forward(list(range(19)) + [5], cfg, w)
    assert float((lg[:19] - lg2[:19]).abs().max()) == 0.0 and float((lg[19] - lg2[19]).abs().max()) > 0


@pytest.mark.parametrize("dims,base,factor", [(8, 10000.0, 1.0), (6, 300.0, 4.0), (32, 5e5, 2.0)])
def test_rotary_table_with_linear_scaling(dims, base, factor):
    cos, sin = yarn_rotary_tables(dims, base, 50, dict(factor=factor) if factor != 1.0 else None, device="cpu")
    x = torch.randn(50, 3, dims + 2, dtype=F64, generator=torch.Generator().manual_seed(0))
    for layout in ("interleaved", "half"):
        want = O.rotate(x, torch.arange(50), dims, base, factor, layout)
        ia = torch.arange(0, dims, 2) if layout == "interleaved" else torch.arange(dims // 2)
        ib = ia + 1 if layout == "interleaved" else ia + dims // 2
        got = x.clone()
        c, s = cos.to(F64)[:, None, :], sin.to(F64)[:, None, :]
        got[..., ia], got[..., ib] = x[..., ia] * c - x[..., ib] * s, x[..., ib] * c + x[..., ia] * s
        assert float((got - want).abs().max()) < 1e-6
        assert float((got[..., dims:] - x[..., dims:]).abs().max()) == 0.0


@pytest.mark.parametrize("bs,pool", [(64, 12), (64, 1), (64, 64), (64, 70), (64, 7), (16, 5), (32, 200), (64, 63), (64, 65)])
def test_every_pooled_block_has_a_place_of_its_own_in_the_page_of_its_last_position(bs, pool):
    per = ops.pooled_entries_per_block(bs, pool)
    seen = set()
    for b in range(0, 40 * max(1, bs // pool + 1)):
        page, idx = ops.pooled_entry_location(b, pool, bs)
        assert page == (b * pool + pool - 1) // bs and 0 <= idx < per
        assert (page, idx) not in seen
        seen.add((page, idx))


@pytest.mark.parametrize("window,pool", [(5, 3), (8, 1), (4, 9), (0, 3), (6, 0), (1, 2)])
def test_oracle_visibility_rule_by_enumeration(window, pool):
    """the oracle's sigmoid attention against a sum over explicitly enumerated (token | block) sets"""
    g = torch.Generator().manual_seed(window * 10 + pool)
    T, H, G, d = 31, 2, 1, 4
    q, k = torch.randn(T, H, d, dtype=F64, generator=g), torch.randn(T, G, d, dtype=F64, generator=g)
    got = O.sigmoid_pooled_attention(q, k, k, 0.5, window, pool, torch.tensor([-1.0, 0.5]))
    for i in range(T):
        toks = [j for j in range(i + 1) if window <= 0 or i - j < window]
        blocks = [b for b in range(T) if pool > 0 and window > 0 and b * pool + pool - 1 <= i - window]
        assert O.pooled_blocks_seen(i, window, pool) == len(blocks)
        for h in range(H):
            tot = torch.zeros(d, dtype=F64)
            for j in toks:
                tot += torch.sigmoid(q[i, h] @ k[j, 0] * 0.5 + (-1.0, 0.5)[h]) * k[j, 0]
            for b in blocks:
                kb = k[b * pool:(b + 1) * pool, 0].mean(0)
                tot += torch.sigmoid(q[i, h] @ kb * 0.5 + (-1.0, 0.5)[h]) * kb
            assert float((tot - got[i, h]).abs().max()) < 1e-12


def test_cache_engine_keeps_pooled_tensors_beside_the_pages():
    from candle_vllm_b200.cache_engine import CacheConfig, CacheEngine
    eng = CacheEngine(2, 0, 0, CacheConfig(64, 5), dtype=torch.bfloat16, device="cpu", layer_shapes=[(2, 8, 8), (1, 16, 4)], pool_shapes=[(6, 2, 8, 8), None])
    k, v, kp, vp = eng.gpu_cache[0]
    assert k.shape == (5, 64, 2, 8) and kp.shape == (5, 6, 2, 8) and vp.shape == (5, 6, 2, 8) and kp.dtype == torch.float32 and k.dtype == torch.bfloat16
    assert len(eng.gpu_cache[1]) == 2
    assert eng.bytes_per_block() == (64 * 2 * 8 * 2) * 2 + (6 * 2 * 8 * 2) * 4 + 64 * (16 + 4) * 2
    with pytest.raises(pkg.BackendError):
        CacheEngine(2, 0, 0, CacheConfig(64, 5), device="cpu", layer_shapes=[(2, 8, 8), (1, 16, 4)], pool_shapes=[None])
