"""Dofevik: a pre-norm decoder (x <- x + mixer(norm1 x), x <- x + ff(norm2 x)) whose norms carry one learned number instead of a weight vector, whose
layers mix the sequence with one of three kinds of attention, and whose feed-forward is a mixture of ungated experts beside a shared one:

  attention         grouped-query softmax attention over a sliding window: biased q / k / v projections, rotation of neighbouring pairs (2i, 2i + 1) on the
                    first rot.dims entries with every frequency divided by rot.scaling.factor, then q and k divided by their root mean square head by head,
                    and a learned sink per head in the softmax denominator;
  attention_2       grouped-query attention without a softmax: the weight of a visible key is sigmoid(score + pb[h]); q and k normed head by head with a
                    weight, no rotation, the values are the keys as projected; a query sees the tokens of its window and one mean key / value per block of
                    mask.pool positions that lies wholly before the window;
  latent_attention  queries through a normed latent of their own, keys and values from a cached normed latent plus one rotated key part shared by the heads,
                    sliding window, softmax, and an element-wise sigmoid gate on the heads' outputs.

Experts are down(relu(up h)^2); the router's logits carry a bias, the `top` largest are chosen and weighted by a softmax over the chosen logits; a shared
expert of the same form runs for every token.  Everything size- or constant-like comes from ``config.json``:

  architecture, vocab, width, norm.eps,
  layers[i] = {type, mixer: {...}, mlp: null | {kind: "moe", expert: {ff}, router: {experts, top}, shared: {ff}}}
    attention         mixer = {heads, kv_heads, dim, vdim, scale, mask: {size}, rot: {base, dims, scaling: {factor}}}
    attention_2       mixer = {heads, kv_heads, dim, vdim, scale, mask: {size, pool}}
    latent_attention  mixer = {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask: {size}, rot: {base, dims}}
  (mask, rot, rot.scaling, mask.pool and mlp.shared may be absent: no window, no rotation, no scaling, no pooled blocks, no shared expert.)

Tensor names: embed, l<i>.norm1 / norm2 (one number each), l<i>.mix.{q, k, v (+ .b), sink, o} | {q, k, q.norm, k.norm, pb, o} |
{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}, l<i>.mlp.{router, router.b, e<j>.up / down, shared.up / down}, final.norm, head.
The model object holds weights only; the paged caches (keys / values, latents, pooled blocks) are allocated by the engine from ``cache_plan()``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ._lib import BackendError, require_device
from . import seq_ops as ops
from .mixers import LatentAttentionMixer, PagedAttentionMixer, PooledWindowAttentionMixer, RoutedExperts, UngatedMlp
from .seq_ops import StepBatch

MIXERS = ("attention", "attention_2", "latent_attention")


@dataclass
class DofevikConfig:
    vocab: int
    width: int
    eps: float
    layers: List[dict]
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "DofevikConfig":
        try:
            cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), layers=list(d["layers"]), raw=d)
            for i, L in enumerate(cfg.layers):
                m = L["mixer"]
                if L.get("type") not in MIXERS:
                    raise BackendError(f"layer {i}: unknown mixer type {L.get('type')!r}")
                if L["type"] == "latent_attention":
                    for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"):
                        m[key]
                    rot = m.get("rot")
                    if rot and int(rot.get("dims", m["rot_dim"])) != int(m["rot_dim"]):
                        raise BackendError(f"layer {i}: the rotation spans {rot['dims']} entries, the rotated part has {m['rot_dim']}")
                else:
                    for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                        m[key]
                    if L["type"] == "attention_2" and int(m["vdim"]) != int(m["dim"]):
                        raise BackendError(f"layer {i}: the values are the keys, so vdim {m['vdim']} must equal dim {m['dim']}")
                    if m.get("rot"):
                        m["rot"]["base"], m["rot"]["dims"]
                mlp = L.get("mlp")
                if mlp:
                    if mlp.get("kind") != "moe":
                        raise BackendError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
                    mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"]
        except KeyError as e:
            raise BackendError(f"Dofevik config lacks {e}")
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "DofevikConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


def _scalar_weight(t: torch.Tensor, n: int) -> torch.Tensor:
    """a norm's single learned number as the weight row the norm kernels take"""
    if t.numel() != 1:
        raise BackendError(f"a norm of this model carries one number, the tensor has {t.numel()}")
    return t.float().reshape(1).expand(n).contiguous()


class _Layer:
    def __init__(self, cfg: DofevikConfig, i: int, w: Dict[str, torch.Tensor], dtype: torch.dtype, block_size: int, max_pos: int):
        L, p, D = cfg.layers[i], f"l{i}.", cfg.width
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        m, mw = L["mixer"], sub(p + "mix.")
        self.type = L["type"]
        self.norm1 = _scalar_weight(w[p + "norm1"], D)
        window = int((m.get("mask") or {}).get("size", 0))
        if self.type == "attention":
            self.mixer = PagedAttentionMixer(mw, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]), cfg.eps, dtype,
                                             rot=m.get("rot") or None, window=window, block_size=block_size, max_pos=max_pos, head_norm="after", interleaved=True)
        elif self.type == "attention_2":
            self.mixer = PooledWindowAttentionMixer(mw, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), float(m["scale"]), cfg.eps, dtype, window=window,
                                                    pool=int((m.get("mask") or {}).get("pool", 0)), block_size=block_size)
        else:
            self.mixer = LatentAttentionMixer(mw, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), float(m["scale"]), cfg.eps,
                                              dtype, rot=m.get("rot") or None, window=window, block_size=block_size, max_pos=max_pos, q_rank=int(m["q_rank"]),
                                              gate="element")
        # feed-forward: the router's product and the shared expert's first product read the same normed row and run as one
        self.mlp = self.shared = self.mlp_in = self.norm2 = None
        mlp = L.get("mlp")
        if mlp:
            self.norm2 = _scalar_weight(w[p + "norm2"], D)
            r, fw = mlp["router"], sub(p + "mlp.")
            self.mlp = RoutedExperts(fw, int(r["experts"]), 0, int(r["top"]), 1.0, dtype, act="relu2")
            if self.mlp.ff != int(mlp["expert"]["ff"]):
                raise BackendError(f"layer {i}: expert tensors have ff {self.mlp.ff}, the config says {mlp['expert']['ff']}")
            self.n_router = self.mlp.N
            if "shared.up" in fw:
                self.shared = UngatedMlp({"up": fw["shared.up"], "down": fw["shared.down"]}, dtype)
                if mlp.get("shared") and self.shared.ff != int(mlp["shared"]["ff"]):
                    raise BackendError(f"layer {i}: the shared expert has ff {self.shared.ff}, the config says {mlp['shared']['ff']}")
                self.mlp_in = torch.cat([self.mlp.router, self.shared.w_in], 0).contiguous()


class DofevikModel:
    architecture = "Dofevik"

    def __init__(self, cfg: DofevikConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16, block_size: int = 64,
                 max_pos: int = 4096, device="cuda"):
        require_device()
        if dtype not in (torch.bfloat16, torch.float32):
            raise BackendError("Dofevik runs in bfloat16 or float32")
        self.cfg, self.dtype, self.block_size, self.device = cfg, dtype, block_size, torch.device(device)
        w = {k: v.to(self.device) for k, v in weights.items()}
        self.embed = w["embed"].to(dtype).contiguous()
        self.head = w["head"].to(dtype).contiguous()
        if self.embed.shape != (cfg.vocab, cfg.width) or self.head.shape != (cfg.vocab, cfg.width):
            raise BackendError(f"embed {tuple(self.embed.shape)} / head {tuple(self.head.shape)} against vocab {cfg.vocab}, width {cfg.width}")
        self.final_norm = _scalar_weight(w["final.norm"], cfg.width)
        self.layers = [_Layer(cfg, i, w, dtype, block_size, max_pos) for i in range(len(cfg.layers))]
        self.vocab = cfg.vocab

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, **kw) -> "DofevikModel":
        from .safetensors_io import load_file
        cfg = DofevikConfig.from_json(os.path.join(path, "config.json"))
        return cls(cfg, load_file(os.path.join(path, "model.safetensors")), dtype=dtype, **kw)

    def ensure_positions(self, max_pos: int) -> bool:
        """grow the rotary tables (outside any graph capture) to cover positions below ``max_pos``; True if a table moved"""
        moved = False
        for L in self.layers:
            cos = getattr(L.mixer, "cos", None)
            if cos is not None and cos.shape[0] < max_pos:
                L.mixer.ensure_positions(max(2 * cos.shape[0], max_pos))
                moved = True
        return moved

    def cache_plan(self) -> dict:
        """What the engine allocates, one entry per layer: (kv heads, key size, value size) of the paged cache -- for a latent layer (1, latent size,
        rotated size) -- and, for layers that see pooled blocks, (pooled entries per page, kv heads, key size, value size) of the f32 pooled cache."""
        return dict(kv_layers=[L.mixer.cache_shape() for L in self.layers], state_layers=[],
                    pool_layers=[L.mixer.pool_shape() if L.type == "attention_2" else None for L in self.layers])

    def forward(self, batch: StepBatch, kv_cache, state_cache, hidden_trace: Optional[list] = None) -> Optional[torch.Tensor]:
        """Runs the step's rows through every layer, advancing the caches; returns f32 logits [R, vocab] of the wanted rows (None when nothing is wanted)."""
        cfg, dt = self.cfg, self.dtype
        x = ops.embedding_scaled(self.embed, batch.tokens, 1.0)
        pending = ()                      # a sublayer's output that has not joined the f32 stream yet: the next norm's kernel adds it first
        for li, L in enumerate(self.layers):
            h = ops.add_rms_norm(x, pending, L.norm1, cfg.eps, dt)
            pending = (L.mixer.forward(h, batch, kv_cache[li]),)
            if L.mlp is not None:
                h = ops.add_rms_norm(x, pending, L.norm2, cfg.eps, dt)
                if L.shared is not None:
                    proj = ops.linear(h, L.mlp_in)
                    pending = (L.mlp.forward(h, x, logits=proj[:, :L.n_router]), L.shared.forward(h, proj=proj[:, L.n_router:]))
                else:
                    pending = (L.mlp.forward(h, x),)
            if hidden_trace is not None:
                ops.add_rms_norm(x, pending, None, cfg.eps)
                pending = ()
                hidden_trace.append(x.clone())
        if batch.num_want == 0:
            return None
        hn = ops.add_rms_norm(x, pending, self.final_norm, cfg.eps, dt, row_index=batch.want_rows)
        return ops.linear(hn, self.head)
