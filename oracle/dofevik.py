"""Plain, slow restatement of the Dofevik decoder (test infrastructure only; shares no code with the product path).

One function per mechanism, float64 torch on the CPU, whole sequences only (a sequence is processed from position 0, every query loops
over the keys it sees).  The product (paged caches, pooled-block cache, ragged steps, CUDA kernels) is compared against this.

Dofevik in short: a pre-norm decoder (x <- x + mixer(norm(x)), x <- x + ff(norm(x))) whose norms carry ONE learned number instead of a
weight vector.  A layer's mixer is one of

  attention         grouped-query softmax attention: biased q / k / v projections, interleaved rotary pairs (2i, 2i + 1) on the first
                    rot.dims entries with every frequency divided by a linear factor, then q and k over their root mean square per head,
                    a sliding window, and a per-head sink in the softmax denominator;
  attention_2       grouped-query attention WITHOUT softmax: per-head weighted RMS norm on q and k, no rotation, values = the keys as
                    projected, a sliding window plus one mean key / mean value per block of P tokens that lies wholly before the window,
                    weight of a visible key = sigmoid(score + pb[h]);
  latent_attention  queries through a normed low-rank latent, keys and values from a cached normed latent plus one rotated key part shared
                    by the heads (rotate-half pairs (i, i + dims/2)), a sliding window, ordinary softmax, an element-wise sigmoid output gate.

The feed-forward is a mixture of ungated experts down(relu(up h)^2): biased router logits, the `top` largest chosen, softmax over the chosen
logits, plus a shared expert of the same form that every token uses.

Notation: T tokens, D width, H query heads, G key/value heads, dk / dv key / value sizes, W window, P pool size, R latent sizes.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is one number for all coordinates"""
    return rms(x, eps) * g.to(F).reshape(())


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float, layout: str) -> torch.Tensor:
    """x [T, ..., d]: the first `dims` entries of the last axis are turned by a = p f_i, f_i = base^(-2i / dims) / factor; the pair of frequency i is
    (2i, 2i + 1) for layout "interleaved" and (i, i + dims/2) for "half"."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = float(base) ** (-2.0 * i / dims) / float(factor)
    ang = positions.to(F)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def window_lo(i: int, window: int) -> int:
    return 0 if window <= 0 else max(0, i - window + 1)


def softmax_attention(q, k, v, scale: float, window: int, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; query i sees j with 0 <= i - j < window; exp(sink[h]) joins the denominator"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    for i in range(T):
        lo = window_lo(i, window)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h].to(F))
            e = torch.exp(s - m)
            den = e.sum() + (0.0 if sink is None else torch.exp(sink[h].to(F) - m))
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def pooled_blocks_seen(i: int, window: int, pool: int) -> int:
    """number of blocks of `pool` positions that end at or before i - window"""
    if pool <= 0 or window <= 0:
        return 0
    return max(0, (i - window + 1) // pool)


def sigmoid_pooled_attention(q, k, v, scale: float, window: int, pool: int, pb: Optional[torch.Tensor]) -> torch.Tensor:
    """No softmax: out_i = sum_j sigmoid(q_i . k_j scale + pb[h]) v_j over the window's tokens and, treated alike, the mean key / mean value of every
    block of `pool` positions that ends at or before i - window."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    nb = T // pool if pool > 0 else 0
    kp = k[:nb * pool].reshape(nb, pool, G, -1).mean(1) if nb else None
    vp = v[:nb * pool].reshape(nb, pool, G, -1).mean(1) if nb else None
    for i in range(T):
        lo = window_lo(i, window)
        seen = pooled_blocks_seen(i, window, pool)
        for h in range(H):
            g = h // (H // G)
            keys, vals = k[lo:i + 1, g], v[lo:i + 1, g]
            if seen:
                keys, vals = torch.cat([kp[:seen, g], keys], 0), torch.cat([vp[:seen, g], vals], 0)
            s = (keys @ q[i, h]) * scale + (0.0 if pb is None else pb[h].to(F))
            out[i, h] = torch.sigmoid(s) @ vals
    return out


def mixer_attention(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    lin = lambda name: h @ w[name].to(F).T + (w[name + ".b"].to(F) if name + ".b" in w else 0.0)
    q, k, v = lin("q").reshape(T, H, dk), lin("k").reshape(T, G, dk), lin("v").reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate(q, positions, int(rot["dims"]), float(rot["base"]), factor, "interleaved")
        k = rotate(k, positions, int(rot["dims"]), float(rot["base"]), factor, "interleaved")
    q, k = rms(q, eps), rms(k, eps)
    a = softmax_attention(q, k, v, float(m["scale"]), int((m.get("mask") or {}).get("size", 0)), w.get("sink"))
    return a.reshape(T, H * dv) @ w["o"].to(F).T


def mixer_attention_2(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w["q"].to(F).T).reshape(T, H, dk)
    k = (h @ w["k"].to(F).T).reshape(T, G, dk)
    v = k                                                       # the values are the keys as projected
    q = rms(q, eps) * w["q.norm"].to(F)
    k = rms(k, eps) * w["k.norm"].to(F)
    mask = m.get("mask") or {}
    a = sigmoid_pooled_attention(q, k, v, float(m["scale"]), int(mask.get("size", 0)), int(mask.get("pool", 0)), w.get("pb"))
    return a.reshape(T, H * dk) @ w["o"].to(F).T


def mixer_latent_attention(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dn, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m.get("rot")
    cq = rms(h @ w["dq"].to(F).T, eps) * w["dq.norm"].to(F)
    q = (cq @ w["uq"].to(F).T).reshape(T, H, dn + dr)
    ckv = h @ w["dkv"].to(F).T
    c = rms(ckv[:, :R], eps) * w["dkv.norm"].to(F)
    kr = ckv[:, R:]                                             # one rotated key part for all heads
    qn, qr = q[..., :dn], q[..., dn:]
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        qr = rotate(qr, positions, int(rot["dims"]), float(rot["base"]), factor, "half")
        kr = rotate(kr, positions, int(rot["dims"]), float(rot["base"]), factor, "half")
    kn = (c @ w["uk"].to(F).T).reshape(T, H, dn)
    v = (c @ w["uv"].to(F).T).reshape(T, H, dv)
    window = int((m.get("mask") or {}).get("size", 0))
    scale = float(m["scale"])
    out = torch.zeros((T, H, dv), dtype=F)
    for i in range(T):
        lo = window_lo(i, window)
        for hh in range(H):
            s = (kn[lo:i + 1, hh] @ qn[i, hh] + kr[lo:i + 1] @ qr[i, hh]) * scale
            out[i, hh] = torch.softmax(s, 0) @ v[lo:i + 1, hh]
    a = out.reshape(T, H * dv)
    if "g" in w:
        a = a * torch.sigmoid(h @ w["g"].to(F).T)
    return a @ w["o"].to(F).T


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.to(F).T) ** 2 @ down.to(F).T


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ w["router"].to(F).T + (w["router.b"].to(F) if "router.b" in w else 0.0)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(z[t], top).indices
        p = torch.softmax(z[t, chosen], 0)
        for e, pe in zip(chosen.tolist(), p):
            out[t] += pe * relu2_expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if "shared.up" in w:
        out = out + relu2_expert(h, w["shared.up"], w["shared.down"])
    return out


MIXERS = {"attention": mixer_attention, "attention_2": mixer_attention_2, "latent_attention": mixer_latent_attention}


def forward(tokens: List[int], cfg: dict, w: Dict[str, torch.Tensor], hidden: Optional[list] = None) -> torch.Tensor:
    """-> logits f64 [T, vocab]; ``hidden`` receives the stream after every layer"""
    eps = float(cfg["norm"]["eps"])
    sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
    x = w["embed"].to(F)[torch.tensor(tokens, dtype=torch.long)]
    positions = torch.arange(len(tokens))
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[L["type"]](scalar_norm(x, w[p + "norm1"], eps), positions, sub(p + "mix."), L["mixer"], eps)
        if L.get("mlp"):
            x = x + moe(scalar_norm(x, w[p + "norm2"], eps), sub(p + "mlp."), L["mlp"])
        if hidden is not None:
            hidden.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].to(F).T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    """the n tokens that follow `prompt` when the largest logit is taken every time (the whole sequence is run again for every token)"""
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(forward(toks, cfg, w)[-1]))
        out.append(t)
        toks.append(t)
    return out
