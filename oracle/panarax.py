"""Plain, slow restatement of the Panarax decoder (test infrastructure only; shares no code with the product path).

One function per mechanism, float64 torch on the CPU, whole sequences only: a sequence is processed from position 0 with empty
state, token by token where the mechanism is a recurrence.  The product (paged cache, state slots, batched steps, CUDA kernels)
is compared against this.

Notation: T tokens, D model width, H query heads, G key / value heads, dk key size, dv value size; linear weights are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b with the biased variance."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time on each channel.  x [T, C], taps [C, K]: y_t = sum_j taps[:, j] x_(t - K + 1 + j); tokens before
    the start count as zero."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * x[s]
    return y


def rglru_mixer(h, w: Dict[str, torch.Tensor], blocks: int):
    """Recurrent block with a real-gated linear recurrent unit.  One branch is gelu_tanh(W_y h + b_y); the other is W_x h + b_x run
    through a short convolution (with bias) and then through the recurrence  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t  with
    a_t = exp(-8 r_t softplus(lam)), the gates r, i = sigmoid of block-diagonal maps of u.  Output: W_o (S * y branch)."""
    T = h.shape[0]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = short_conv(h @ w["x"].T + w["x.b"], w["conv"]) + w["conv.b"]
    C = u.shape[1]
    n = C // blocks
    ub = u.view(T, blocks, n)
    r = torch.sigmoid(torch.einsum("bij,tbj->tbi", w["ra"], ub) + w["ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("bij,tbj->tbi", w["ri"], ub) + w["ri.b"]).reshape(T, C)
    log_a = -8.0 * r * torch.nn.functional.softplus(w["lam"])
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=F)
    out = torch.zeros(T, C, dtype=F)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
        out[t] = S
    return (out * y) @ w["o"].T


def lightning_mixer(h, w, heads: int, dk: int, dv: int, decay: List[float], eps: float):
    """Linear attention with a fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, on silu'd q, k, v; all heads'
    outputs normed together, gated by sigmoid(W_g h), projected."""
    T = h.shape[0]
    q = silu(h @ w["q"].T).view(T, heads, dk)
    k = silu(h @ w["k"].T).view(T, heads, dk)
    v = silu(h @ w["v"].T).view(T, heads, dv)
    S = torch.zeros(heads, dk, dv, dtype=F)
    lam = torch.tensor(decay, dtype=F).view(heads, 1, 1)
    o = torch.zeros(T, heads, dv, dtype=F)
    for t in range(T):
        S = lam * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    z = rms(o.reshape(T, heads * dv), eps) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return z @ w["o"].T


def softmax_attention(h, w, H: int, G: int, dk: int, dv: int, scale: float, eps: float, q_temp: Optional[dict]):
    """Causal grouped-query softmax attention without rotation: the query is stretched by 1 + coef ln(floor((p + 1) / every) + 1), every
    value head is brought to unit root mean square, each head's output is gated by one sigmoid per head."""
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, dk)
    k = (h @ w["k"].T).view(T, G, dk)
    v = rms((h @ w["v"].T).view(T, G, dv), eps)
    if q_temp:
        p = torch.arange(T, dtype=F)
        q = q * (1.0 + float(q_temp["coef"]) * torch.log(torch.floor((p + 1.0) / float(q_temp["every"])) + 1.0)).view(T, 1, 1)
    gate = torch.sigmoid(h @ w["g"].T)                     # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    rep = H // G
    for hh in range(H):
        g = hh // rep
        s = (q[:, hh] @ k[:, g].T) * scale
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    out = out * gate.unsqueeze(-1)
    return out.reshape(T, H * dv) @ w["o"].T


def matrix_memory(h, w, heads: int, dk: int, dv: int, cap: float, eps: float):
    """Matrix memory with exponential gating held stable by a running maximum m (m_0 = 0):  i = cap tanh(. / cap),
    f = logsigmoid(cap tanh(. / cap)),  m_t = max(f + m_(t-1), i),  S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T,  n_t alike
    with k,  o = S^T q / (max(|n . q|, e^(-m_t)) + 1e-6)."""
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, heads, dk) * dk ** -0.5
    k = (h @ w["k"].T).view(T, heads, dk)
    v = (h @ w["v"].T).view(T, heads, dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    S = torch.zeros(heads, dk, dv, dtype=F)
    n = torch.zeros(heads, dk, dtype=F)
    m = torch.zeros(heads, dtype=F)
    o = torch.zeros(T, heads, dv, dtype=F)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a = torch.exp(fg[t] + m - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a.view(-1, 1, 1) * S + b.view(-1, 1, 1) * k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        n = a.view(-1, 1) * n + b.view(-1, 1) * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = num / den.view(-1, 1)
    z = rms(o, eps).reshape(T, heads * dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return z @ w["o"].T


def parallel_mixer(h, w, cfg: dict, eps: float):
    """Softmax attention and matrix memory side by side on the same input; half the sum of their normed outputs."""
    sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
    L, R = cfg["left"], cfg["right"]
    a = softmax_attention(h, sub("left."), int(L["heads"]), int(L["kv_heads"]), int(L["dim"]), int(L["vdim"]), float(L["scale"]), eps, L.get("q_temp"))
    b = matrix_memory(h, sub("right."), int(R["heads"]), int(R["dim"]), int(R["vdim"]), float(R["gate_cap"]), eps)
    return 0.5 * (rms(a, eps) * w["left.out"] + rms(b, eps) * w["right.out"])


def dense_mlp(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def clamped_expert(x, gate, up, down, limit: float):
    g = torch.clamp(x @ gate.T, max=limit)
    u = torch.clamp(x @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def sigmoid_moe(h, w, experts: int, top: int, limit: float):
    """Every token goes to the `top` experts of largest sigmoid(router logit); an expert sees the token times that score."""
    s = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            out[t] += clamped_expert(s[t, e] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, trace: Optional[list] = None) -> torch.Tensor:
    """tokens of ONE sequence from position 0 -> logits [T, vocab] (float64); `trace` collects the stream after every layer."""
    w = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] + w["pos"][:T]
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        sub = {k[len(p) + 4:]: v for k, v in w.items() if k.startswith(p + "mix.")}
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        gate = torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"]) if p + "rg1" in w else 1.0
        hc = h + short_conv(h, w[p + "canon1"]) if p + "canon1" in w else h
        m = L["mixer"]
        if L["type"] == "rglru":
            y = rglru_mixer(hc, sub, int(m["blocks"]))
        elif L["type"] == "lightning":
            y = lightning_mixer(hc, sub, int(m["heads"]), int(m["dim"]), int(m["vdim"]), [float(d) for d in m["decay"]], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(hc, sub, m, eps)
        else:
            raise ValueError(L["type"])
        x = x + gate * y
        if L.get("mlp"):
            sub = {k[len(p) + 4:]: v for k, v in w.items() if k.startswith(p + "mlp.")}
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            gate = torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"]) if p + "rg2" in w else 1.0
            if L["mlp"]["kind"] == "dense":
                y = dense_mlp(h, sub)
            else:
                y = sigmoid_moe(h, sub, int(L["mlp"]["router"]["experts"]), int(L["mlp"]["router"]["top"]), float(L["mlp"]["expert"]["limit"]))
            x = x + gate * y
        if trace is not None:
            trace.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T


def greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt, n: int) -> List[int]:
    """n tokens of greedy continuation (the whole sequence is run again for every token)."""
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(forward(cfg, weights, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
