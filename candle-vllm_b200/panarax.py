"""Panarax: a pre-norm decoder whose layers mix the sequence with one of three mixers -- a real-gated linear recurrence ("rglru"), linear
attention with a fixed decay per head ("lightning"), or softmax attention and an exponentially gated matrix memory side by side
("parallel") -- and whose feed-forward is dense (SiLU) or a sigmoid-routed mixture of clamped experts.  Learned position vectors are
added to the token embedding, norms are layer norms with weight and bias, the mixer reads its input plus a short causal convolution of
it, every sublayer's output passes a sigmoid gate computed from the sublayer's input before it joins the f32 stream, and the head is
the embedding table.  Everything size- or constant-like comes from ``config.json``:

  architecture, vocab, width, max_positions, norm.eps, canon.taps,
  layers[i] = {type: "rglru" | "lightning" | "parallel", mixer: {...}, mlp: null | {kind: "dense", ff} |
               {kind: "moe", expert: {ff, limit}, router: {experts, top}}}
    rglru      mixer = {width, blocks, conv}
    lightning  mixer = {heads, dim, vdim, decay: [per head]}
    parallel   mixer = {left: {heads, kv_heads, dim, vdim, scale, q_temp: {coef, every}}, right: {heads, dim, vdim, gate_cap}}

Tensor names: embed, pos, l<i>.norm1 / norm1.b / norm2 / norm2.b, l<i>.canon1, l<i>.rg1 / rg1.b / rg2 / rg2.b, l<i>.mix.*,
l<i>.mlp.{gate, up, down} or l<i>.mlp.{router, e<j>.gate / up / down}, final.norm / final.norm.b.
The model object holds weights only; the paged cache of the attention side and the per-sequence state (the convolutions' last inputs, the
recurrences' f32 state) are allocated by the engine from ``cache_plan()`` and handed to ``forward``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ._lib import BackendError, require_device
from . import seq_ops as ops
from .mixers import (DecayLinearAttention, GatedLinearRecurrence, GatedMlp, MatrixMemoryMixer, PagedAttentionMixer, ParallelMixer, RoutedExperts)
from .seq_ops import StepBatch

MIXERS = ("rglru", "lightning", "parallel")


@dataclass
class PanaraxConfig:
    vocab: int
    width: int
    max_positions: int
    eps: float
    canon_taps: int
    layers: List[dict]
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "PanaraxConfig":
        try:
            cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), max_positions=int(d["max_positions"]), eps=float(d["norm"]["eps"]),
                      canon_taps=int((d.get("canon") or {}).get("taps", 0)), layers=list(d["layers"]), raw=d)
            for i, L in enumerate(cfg.layers):
                m = L["mixer"]
                if L.get("type") not in MIXERS:
                    raise BackendError(f"layer {i}: unknown mixer type {L.get('type')!r}")
                if L["type"] == "rglru":
                    m["width"], m["blocks"], m["conv"]
                elif L["type"] == "lightning":
                    if len(m["decay"]) != int(m["heads"]):
                        raise BackendError(f"layer {i}: {len(m['decay'])} decays for {m['heads']} heads")
                    m["dim"], m["vdim"]
                else:
                    for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                        m["left"][key]
                    for key in ("heads", "dim", "vdim", "gate_cap"):
                        m["right"][key]
                mlp = L.get("mlp")
                if mlp:
                    if mlp.get("kind") == "dense":
                        mlp["ff"]
                    elif mlp.get("kind") == "moe":
                        mlp["expert"]["ff"], mlp["expert"]["limit"], mlp["router"]["experts"], mlp["router"]["top"]
                    else:
                        raise BackendError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        except KeyError as e:
            raise BackendError(f"Panarax config lacks {e}")
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "PanaraxConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


class _Layer:
    def __init__(self, cfg: PanaraxConfig, i: int, w: Dict[str, torch.Tensor], dtype: torch.dtype, block_size: int, max_pos: int):
        L, p = cfg.layers[i], f"l{i}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        f32 = lambda name: w[p + name].float().contiguous() if p + name in w else None
        m, D = L["mixer"], cfg.width
        self.type = L["type"]
        self.norm1, self.norm1_b = f32("norm1"), f32("norm1.b")
        self.canon = f32("canon1")
        if self.canon is not None and tuple(self.canon.shape) != (D, cfg.canon_taps):
            raise BackendError(f"layer {i}: input convolution {tuple(self.canon.shape)}, the config says {(D, cfg.canon_taps)}")
        self.rg1 = w[p + "rg1"].to(dtype).contiguous() if p + "rg1" in w else None
        self.rg1_b = f32("rg1.b")
        mw = sub(p + "mix.")
        if self.type == "rglru":
            self.mixer = GatedLinearRecurrence(mw, int(m["blocks"]), int(m["conv"]), dtype)
            if self.mixer.C != int(m["width"]):
                raise BackendError(f"layer {i}: the recurrence has {self.mixer.C} channels, the config says {m['width']}")
        elif self.type == "lightning":
            self.mixer = DecayLinearAttention(mw, int(m["heads"]), int(m["dim"]), int(m["vdim"]), m["decay"], cfg.eps, dtype)
        else:
            lm, rm = m["left"], m["right"]
            lw = {k[5:]: v for k, v in mw.items() if k.startswith("left.") and k != "left.out"}
            rw = {k[6:]: v for k, v in mw.items() if k.startswith("right.") and k != "right.out"}
            left = PagedAttentionMixer(lw, int(lm["heads"]), int(lm["kv_heads"]), int(lm["dim"]), int(lm["vdim"]), float(lm["scale"]), cfg.eps, dtype,
                                       block_size=block_size, max_pos=max_pos, q_temp=lm.get("q_temp") or None, value_norm=True)
            right = MatrixMemoryMixer(rw, int(rm["heads"]), int(rm["dim"]), int(rm["vdim"]), float(rm["gate_cap"]), cfg.eps, dtype)
            self.mixer = ParallelMixer(left, right, mw["left.out"], mw["right.out"], cfg.eps)
        # feed-forward: its gate's projection (and the router's) joins the first product of the sublayer, all of them read the same normed row
        self.mlp = self.mlp_in = None
        mlp = L.get("mlp")
        if mlp:
            self.norm2, self.norm2_b = f32("norm2"), f32("norm2.b")
            self.rg2_b = f32("rg2.b")
            self.has_rg2 = p + "rg2" in w
            head = [w[p + "rg2"].to(dtype)] if self.has_rg2 else []
            self.off_mlp = D if self.has_rg2 else 0
            if mlp["kind"] == "dense":
                self.mlp = GatedMlp(sub(p + "mlp."), dtype, act="silu")
                if self.mlp.w_down.shape[1] != int(mlp["ff"]):
                    raise BackendError(f"layer {i}: feed-forward tensors have ff {self.mlp.w_down.shape[1]}, the config says {mlp['ff']}")
                self.mlp_in = torch.cat(head + [self.mlp.w_in], 0).contiguous()
            else:
                r = mlp["router"]
                self.mlp = RoutedExperts(sub(p + "mlp."), int(r["experts"]), 0, int(r["top"]), 1.0, dtype, score="sigmoid", normalise=False, weight_input=True,
                                         act="clamped", limit=float(mlp["expert"]["limit"]))
                if self.mlp.ff != int(mlp["expert"]["ff"]):
                    raise BackendError(f"layer {i}: expert tensors have ff {self.mlp.ff}, the config says {mlp['expert']['ff']}")
                self.mlp_in = torch.cat(head + [self.mlp.router], 0).contiguous()


class PanaraxModel:
    architecture = "Panarax"

    def __init__(self, cfg: PanaraxConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16, block_size: int = 64,
                 max_pos: int = 4096, device="cuda"):
        require_device()
        if dtype not in (torch.bfloat16, torch.float32):
            raise BackendError("Panarax runs in bfloat16 or float32")
        self.cfg, self.dtype, self.block_size, self.device = cfg, dtype, block_size, torch.device(device)
        w = {k: v.to(self.device) for k, v in weights.items()}
        self.embed = w["embed"].to(dtype).contiguous()
        self.pos = w["pos"].to(dtype).contiguous()
        if self.pos.shape[0] != cfg.max_positions or self.embed.shape != (cfg.vocab, cfg.width):
            raise BackendError(f"embed {tuple(self.embed.shape)} / pos {tuple(self.pos.shape)} against vocab {cfg.vocab}, width {cfg.width}, {cfg.max_positions} positions")
        self.final_norm = w["final.norm"].float().contiguous()
        self.final_norm_b = w["final.norm.b"].float().contiguous() if "final.norm.b" in w else None
        self.layers = [_Layer(cfg, i, w, dtype, block_size, max_pos) for i in range(len(cfg.layers))]
        # every layer has a state entry (the input convolution's last rows, then the mixer's own state); parallel layers also a paged cache
        self.kv_index, n = [], 0
        for L in self.layers:
            self.kv_index.append(n if L.type == "parallel" else None)
            n += L.type == "parallel"
        self.vocab = cfg.vocab

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, **kw) -> "PanaraxModel":
        from .safetensors_io import load_file
        cfg = PanaraxConfig.from_json(os.path.join(path, "config.json"))
        return cls(cfg, load_file(os.path.join(path, "model.safetensors")), dtype=dtype, **kw)

    def ensure_positions(self, max_pos: int) -> bool:
        """positions are a learned table of fixed length: nothing to grow"""
        if max_pos > self.cfg.max_positions:
            raise BackendError(f"position {max_pos - 1} is outside the model's {self.cfg.max_positions} learned positions")
        return False

    def cache_plan(self) -> dict:
        """What the engine allocates: one (kv heads, key size, value size) per parallel layer, and per layer a tuple of per-slot state shapes: the input
        convolution's last taps - 1 rows (when the layer has one), then the mixer's state."""
        D, K = self.cfg.width, self.cfg.canon_taps
        kv = [L.mixer.cache_shape() for L in self.layers if L.type == "parallel"]
        st = [(((max(K - 1, 1), D),) if L.canon is not None else ()) + tuple(L.mixer.state_shapes()) for L in self.layers]
        return dict(kv_layers=kv, state_layers=st)

    def forward(self, batch: StepBatch, kv_cache, state_cache, hidden_trace: Optional[list] = None) -> Optional[torch.Tensor]:
        """Runs the step's rows through every layer, advancing the cache and the states; returns f32 logits [R, vocab] of the wanted rows (None when
        nothing is wanted)."""
        cfg, dt, D = self.cfg, self.dtype, self.cfg.width
        x = ops.embedding_positional(self.embed, self.pos, batch)
        pending = None                    # a sublayer's gated output that has not joined the stream yet: the next norm's kernel adds it first
        for li, L in enumerate(self.layers):
            st = state_cache[li]
            h, h32 = ops.layer_norm(x, L.norm1, L.norm1_b, cfg.eps, dt, also_f32=True, pending=pending) if L.canon is not None else \
                (ops.layer_norm(x, L.norm1, L.norm1_b, cfg.eps, dt, pending=pending), None)
            z = ops.linear(h, L.rg1) if L.rg1 is not None else None
            if L.canon is not None:
                hc = ops.causal_conv(h32, L.canon, st[0], batch, out_dtype=dt, add_input=True)
                st = st[1:]
            else:
                hc = h
            if L.type == "parallel":
                y = L.mixer.forward(hc, batch, kv_cache[self.kv_index[li]], st)
            else:
                y = L.mixer.forward(hc, batch, st)
            pending = (y, z, L.rg1_b)
            if L.mlp is not None:
                h = ops.layer_norm(x, L.norm2, L.norm2_b, cfg.eps, dt, pending=pending)
                proj = ops.linear(h, L.mlp_in)
                z = proj[:, :D] if L.has_rg2 else None
                if isinstance(L.mlp, GatedMlp):
                    y = L.mlp.forward(h, proj=proj[:, L.off_mlp:])
                else:
                    y = L.mlp.forward(h, x, logits=proj[:, L.off_mlp:])
                pending = (y, z, L.rg2_b)
            if hidden_trace is not None:
                ops.gated_residual_add(x, *pending)
                pending = None
                hidden_trace.append(x.clone())
        if pending is not None:
            ops.gated_residual_add(x, *pending)
        if batch.num_want == 0:
            return None
        hn = ops.layer_norm(x, self.final_norm, self.final_norm_b, cfg.eps, dt, row_index=batch.want_rows)
        return ops.linear(hn, self.embed)
