"""Host-side pieces of Panarax on the CPU: configuration checks, the registry entry and its build group, the shapes of the synthetic
checkpoints, and properties of the float64 restatement that the GPU tests lean on (so that a fault there is not taken for a fault of
the product): every recurrence against its closed form over the whole history."""
import copy
import math

import pytest
import torch

from candle_vllm_b200 import _lib, synthetic as S
from candle_vllm_b200._lib import BackendError
from candle_vllm_b200.panarax import PanaraxConfig
from candle_vllm_b200.registry import registered
from oracle import panarax as P

F64 = torch.float64
CFG = S.panarax_config(40, 50, [S.panarax_parallel_layer(4, 2, 12, 20, 3, 10, 18, ff=24),
                                S.panarax_rglru_layer(48, 3, conv=5, ff=16, experts=5, top=2, limit=1.0),
                                S.panarax_lightning_layer(3, 12, 20)], max_positions=64, taps=2)


def test_registered_with_a_build_group_of_its_own(tmp_path):
    import json
    from candle_vllm_b200.registry import build_group_of
    assert "Panarax" in registered()
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    group = build_group_of(str(tmp_path))
    assert group == "hybrid" and set(_lib.GROUP_SYMBOLS[group]) <= set(_lib.SYMBOLS)
    c = PanaraxConfig.from_dict(copy.deepcopy(CFG))
    assert (c.vocab, c.width, c.max_positions, c.canon_taps, len(c.layers)) == (50, 40, 64, 2, 3)


@pytest.mark.parametrize("edit,needle", [
    (lambda d: d["layers"][0].update(type="other"), "unknown mixer"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "feed-forward kind"),
    (lambda d: d["layers"][2]["mixer"].update(decay=[0.5]), "decays for"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("scale"), "lacks"),
    (lambda d: d["layers"][0]["mixer"]["right"].pop("gate_cap"), "lacks"),
    (lambda d: d["layers"][1]["mixer"].pop("blocks"), "lacks"),
    (lambda d: d["layers"][1]["mlp"]["expert"].pop("limit"), "lacks"),
    (lambda d: d.pop("max_positions"), "lacks"),
])
def test_config_faults_are_named(edit, needle):
    d = copy.deepcopy(CFG)
    edit(d)
    with pytest.raises(BackendError, match=needle):
        PanaraxConfig.from_dict(d)


def test_synthetic_checkpoint_runs_through_the_oracle():
    w = S.panarax_weights(CFG, 0)
    assert w["l0.mix.left.g"].shape == (4, 40) and w["l0.mix.right.i.b"].shape == (3,) and w["l1.mix.ra"].shape == (3, 16, 16)
    assert w["l1.canon1"].shape == (40, 2) and w["l1.mlp.e4.down"].shape == (40, 16) and "l2.norm2" not in w
    trace = []
    lg = P.forward(CFG, w, list(range(30)), trace)
    assert lg.shape == (30, 50) and len(trace) == 3 and bool(torch.isfinite(lg).all())
    # causal: a later token changes nothing before it
    lg2 = P.forward(CFG, w, list(range(29)) + [7])
    assert torch.allclose(lg[:29], lg2[:29])


def test_oracle_fixed_decay_against_the_sum_over_all_keys():
    g = torch.Generator().manual_seed(0)
    D, H, dk, dv, T = 10, 2, 6, 5, 40
    w = {k: torch.randn(n, D, generator=g, dtype=F64) for k, n in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv))}
    w["norm"], w["o"] = torch.ones(H * dv, dtype=F64), torch.eye(H * dv, dtype=F64)
    h = torch.randn(T, D, generator=g, dtype=F64)
    decay = [0.9, 0.5]
    got = P.lightning_mixer(h, w, H, dk, dv, decay, 1e-6)
    q, k, v = (P.silu(h @ w[n].T).view(T, H, -1) for n in ("q", "k", "v"))
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for j in range(t + 1):
            for hh in range(H):
                o[t, hh] += decay[hh] ** (t - j) * (q[t, hh] @ k[j, hh]) * v[j, hh]
    want = P.rms(o.reshape(T, -1), 1e-6) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-12)


def test_oracle_matrix_memory_against_unstabilised_sums():
    """without the running maximum: C_t = sum_j exp(sum_{s>j} f_s + i_j) k_j v_j^T; the stabilised recurrence returns C_t^T q over
    max(|n_t . q|, 1) up to the factor exp(-m_t) in numerator, denominator and the floor"""
    g = torch.Generator().manual_seed(1)
    D, H, dk, dv, T, cap = 8, 2, 4, 3, 25, 6.0
    w = {k: torch.randn(n, D, generator=g, dtype=F64) for k, n in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv), ("i", H), ("f", H))}
    w["i.b"], w["f.b"] = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64) + 2.0
    w["norm"], w["o"] = torch.ones(H * dv, dtype=F64), torch.eye(H * dv, dtype=F64)
    h = torch.randn(T, D, generator=g, dtype=F64)
    got = P.matrix_memory(h, w, H, dk, dv, cap, 1e-6)
    q = (h @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k, v = (h @ w["k"].T).view(T, H, dk), (h @ w["v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    o = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        m = 0.0
        for t in range(T):
            m = max(float(fg[t, hh]) + m, float(ig[t, hh]))
            logw = torch.tensor([float(fg[j + 1:t + 1, hh].sum() + ig[j, hh]) for j in range(t + 1)], dtype=F64)
            assert float(logw.max()) <= m + 1e-12                 # the maximum bounds every weight (it may be held up by its start at zero)
            wt = torch.exp(logw - m)
            num = ((q[t, hh] @ k[:t + 1, hh].T) * wt) @ v[:t + 1, hh]
            den = max(abs(float(((q[t, hh] @ k[:t + 1, hh].T) * wt).sum())), math.exp(-m)) + 1e-6
            o[t, hh] = num / den
    want = (P.rms(o, 1e-6).reshape(T, -1)) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want, rtol=1e-8, atol=1e-10)


def test_oracle_gated_recurrence_is_bounded_and_keeps_its_scale():
    """sqrt(1 - a^2) keeps a unit-variance input at unit variance: with constant gates the state of a constant input u converges to i u"""
    Cn, nb = 12, 3
    w = dict(y=torch.zeros(Cn, 4, dtype=F64), x=torch.zeros(Cn, 4, dtype=F64), conv=torch.zeros(Cn, 3, dtype=F64), ra=torch.zeros(nb, 4, 4, dtype=F64),
             ri=torch.zeros(nb, 4, 4, dtype=F64), lam=torch.linspace(-3, 1, Cn, dtype=F64), o=torch.eye(Cn, dtype=F64))
    w["y.b"], w["x.b"], w["conv.b"] = torch.full((Cn,), 3.0, dtype=F64), torch.zeros(Cn, dtype=F64), torch.linspace(0.5, 2.0, Cn, dtype=F64)
    w["ra.b"], w["ri.b"] = torch.zeros(nb, 4, dtype=F64), torch.full((nb, 4), 1.0, dtype=F64)
    out = P.rglru_mixer(torch.zeros(400, 4, dtype=F64), w, nb)
    a = torch.exp(-8.0 * 0.5 * torch.nn.functional.softplus(w["lam"]))
    fixed = torch.sqrt(1 - a * a) * torch.sigmoid(torch.tensor(1.0, dtype=F64)) * w["conv.b"] / (1 - a)
    assert torch.allclose(out[-1], fixed * P.gelu_tanh(torch.tensor(3.0, dtype=F64)), rtol=1e-6)


def test_oracle_experts_see_the_weighted_token():
    g = torch.Generator().manual_seed(2)
    D, E, ff = 6, 4, 5
    w = {"router": torch.randn(E, D, generator=g, dtype=F64)}
    for j in range(E):
        w[f"e{j}.gate"], w[f"e{j}.up"], w[f"e{j}.down"] = (torch.randn(ff, D, generator=g, dtype=F64), torch.randn(ff, D, generator=g, dtype=F64),
                                                          torch.randn(D, ff, generator=g, dtype=F64))
    h = torch.randn(9, D, generator=g, dtype=F64)
    s = torch.sigmoid(h @ w["router"].T)
    one = P.sigmoid_moe(h, w, E, 1, 0.7)
    for t in range(9):
        e = int(torch.argmax(s[t]))
        assert torch.allclose(one[t], P.clamped_expert(s[t, e] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], 0.7))
    allofthem = P.sigmoid_moe(h, w, E, E, 0.7)
    want = sum(P.clamped_expert(s[:, e:e + 1] * h, w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], 0.7) for e in range(E))
    assert torch.allclose(allofthem, want)
