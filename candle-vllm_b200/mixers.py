"""Sequence mixers and feed-forward blocks for ragged-step models, each a thin object that owns its (fused) weights and calls the
kernels of ``seq_ops``.  Sizes and constants are constructor arguments so that any decoder built from these parts can use them:

  GatedDeltaMixer      short causal convolution + SiLU on q / k / v, unit-norm q and k, gated delta rule over an f32 state, per-head
                       RMS norm times a SiLU gate, output projection (csrc/gated_delta.cu)
  PagedAttentionMixer  grouped-query attention over the paged cache with optional whole-row q / k RMS norm, partial rotary with
                       optional YaRN scaling, a chunk and / or sliding-window mask, an optional query temperature, values cached at unit
                       root mean square, and one sigmoid gate per head (csrc/attention_varlen.cu)
  GatedMlp             down(act(gate x) * (up x)) with the tanh GELU or SiLU (csrc/norm_act.cu)
  LatentAttentionMixer attention over a cached low-rank latent plus one shared rotated key part, softmax sink, sigmoid head gates, optionally
                       over another layer's cache (csrc/latent_attention.cu)
  RoutedExperts        softmax-routed mixture of SiLU experts: group-limited top-k with a choice-only correction, identity experts
                       (csrc/moe_ragged.cu)
  TokenSideInput       a per-token embedding gated by the stream and added back through a norm
  GatedLinearRecurrence  two branches: gelu(W_y h) and a short convolution of W_x h run through a per-channel recurrence whose decay and
                       input gates are block-diagonal maps of the convolved branch (csrc/linear_recurrence.cu)
  DecayLinearAttention linear attention over an f32 matrix state with one fixed decay per head, SiLU on q / k / v, all heads normed together, sigmoid gate
  MatrixMemoryMixer    linear attention with exponential input / forget gates held stable by a running maximum, a normaliser vector, per-head norm
  ParallelMixer        two mixers side by side on one input (one fused projection), half the sum of their normed outputs

Activations that feed a matrix product are of the model's compute dtype (bf16 or f32); products come back in f32 and everything
between them (norms, convolution, recurrence, softmax) is 32-bit.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from ._lib import BackendError
from . import seq_ops as ops
from .seq_ops import StepBatch


def yarn_rotary_tables(dims: int, base: float, max_pos: int, scaling: Optional[dict] = None, device="cuda") -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin f32 [max_pos, dims/2] for the rotate-half layout, angles computed in float64.  ``scaling`` = dict(factor, original, fast,
    slow) applies YaRN: with c(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)),
    dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes f_i / factor * r_i + f_i * (1 - r_i), and cos /
    sin are multiplied by 0.1 * ln(factor) + 1.  A ``scaling`` of dict(factor) alone is linear scaling: every frequency is divided by the factor.
    Row p holds the angles p f_i whatever the pairing of the entries (neighbours or half apart) the kernel that reads the table uses."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    mag = 1.0
    if scaling and "original" not in scaling:
        f = f / float(scaling.get("factor", 1.0))
    elif scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])
        corr = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(corr(float(scaling["fast"]))), 0)
        hi = min(math.ceil(corr(float(scaling["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(ang) * mag).float().to(device), (torch.sin(ang) * mag).float().to(device)


class GatedDeltaMixer:
    """weights: q, k [G dk, D], v, g [H dv, D], b, a [H, D], o [D, H dv] (compute dtype); q.conv / k.conv / v.conv [channels, taps], A_log,
    dt_bias [H], norm [dv].  One fused projection q|k|v|g|b|a per step."""
    kind = "state"

    def __init__(self, w: Dict[str, torch.Tensor], heads: int, kv_heads: int, dk: int, dv: int, taps: int, eps: float, dtype: torch.dtype):
        if heads % kv_heads:
            raise BackendError("GatedDeltaMixer: heads must be a multiple of kv_heads")
        self.H, self.G, self.dk, self.dv, self.taps, self.eps, self.dtype = heads, kv_heads, dk, dv, taps, eps, dtype
        self.C = 2 * kv_heads * dk + heads * dv
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"], w["b"], w["a"]], 0).to(dtype).contiguous()
        self.off_g = self.C
        self.off_b = self.C + heads * dv
        self.off_a = self.off_b + heads
        self.conv = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0).float().contiguous()
        if self.conv.shape != (self.C, taps):
            raise BackendError(f"GatedDeltaMixer: convolution taps {tuple(self.conv.shape)} != {(self.C, taps)}")
        self.A_log, self.dt_bias, self.norm = w["A_log"].float().contiguous(), w["dt_bias"].float().contiguous(), w["norm"].float().contiguous()
        self.w_o = w["o"].to(dtype).contiguous()

    def state_shapes(self):
        return ((max(self.taps - 1, 1), self.C), (self.H, self.dv, self.dk))     # state stored column-major per head; a 1-tap convolution keeps no inputs; one unused row

    def forward(self, h: torch.Tensor, batch: StepBatch, cache) -> torch.Tensor:
        conv_state, S = cache
        proj = ops.linear(h, self.w_in)
        y = ops.causal_conv_silu(proj[:, :self.C], self.conv, conv_state, batch)
        o = ops.gated_delta_rule(y, proj, self.off_b, self.off_a, self.A_log, self.dt_bias, S, batch, self.H, self.G, self.dk, self.dv)
        z = ops.gated_rms_norm(o, proj[:, self.off_g:], self.norm, self.H, self.dv, self.eps, self.dtype)
        return ops.linear(z, self.w_o)


class PagedAttentionMixer:
    """weights: q [H dk, D], k [G dk, D], v [G dv, D], o [D, H dv]; optional q.norm [H dk], k.norm [G dk] (plain weights, RMS over the whole
    row), optional g [H, D] (head h's output times sigmoid(g x)[h]).  rot = dict(dims, base, scaling) or None; chunk / window = 0 for none;
    q_temp = dict(coef, every): the query at position p times 1 + coef ln(floor((p + 1) / every) + 1); value_norm: every value head is
    cached divided by its root mean square.

    ``head_norm`` "before" / "after": q and k are normed head by head over dk, before or after the rotation (q.norm / k.norm are then [dk], shared by the
    heads, or absent for a norm without weight); ``interleaved``: the rotation pairs neighbours (2i, 2i + 1) instead of (i, i + dims/2); biases q.b / k.b /
    v.b are added in the projection; sink [H]: exp(sink[h]) joins the softmax denominator of head h (a key without a value whose score is not scaled)."""
    kind = "kv"

    def __init__(self, w: Dict[str, torch.Tensor], heads: int, kv_heads: int, dk: int, dv: int, scale: float, eps: float, dtype: torch.dtype,
                 rot: Optional[dict] = None, chunk: int = 0, window: int = 0, block_size: int = 64, max_pos: int = 4096, q_temp: Optional[dict] = None,
                 value_norm: bool = False, head_norm: str = "none", interleaved: bool = False):
        if heads % kv_heads:
            raise BackendError("PagedAttentionMixer: heads must be a multiple of kv_heads")
        if head_norm not in ("none", "before", "after") or (head_norm != "none" and (q_temp or value_norm)):
            raise BackendError(f"PagedAttentionMixer: head_norm {head_norm!r} (none / before / after; not with a query temperature or normed values)")
        self.H, self.G, self.dk, self.dv, self.scale, self.eps, self.dtype = heads, kv_heads, dk, dv, float(scale), eps, dtype
        self.chunk, self.window, self.block_size, self.rot = int(chunk), int(window), block_size, rot
        self.head_norm, self.interleaved = head_norm, bool(interleaved)
        self.sink = w["sink"].float().contiguous() if "sink" in w else None
        self.bias = None
        if any(n + ".b" in w for n in "qkv"):
            zero = lambda n: torch.zeros(w[n].shape[0], dtype=torch.float32, device=w[n].device)
            self.bias = torch.cat([w[n + ".b"].float() if n + ".b" in w else zero(n) for n in "qkv"], 0).contiguous()
        # the per-head preparation kernel serves head norms, neighbour pairs and biases; the whole-row one the rest
        self.per_head = head_norm != "none" or self.interleaved or self.bias is not None
        if self.per_head and (q_temp or value_norm):
            raise BackendError("PagedAttentionMixer: biases / neighbour pairs do not combine with a query temperature or normed values")
        self.has_gate = "g" in w
        self.off_g = heads * dk + kv_heads * (dk + dv)
        self.w_in = torch.cat([w["q"], w["k"], w["v"]] + ([w["g"]] if self.has_gate else []), 0).to(dtype).contiguous()
        self.q_temp = (float(q_temp["coef"]), int(q_temp["every"])) if q_temp else None
        self.value_norm = bool(value_norm)
        self.q_norm = w["q.norm"].float().contiguous() if "q.norm" in w else None
        self.k_norm = w["k.norm"].float().contiguous() if "k.norm" in w else None
        self.w_o = w["o"].to(dtype).contiguous()
        self.rot_dims = int(rot["dims"]) if rot else 0
        if self.rot_dims % 2 or self.rot_dims > dk:
            raise BackendError(f"PagedAttentionMixer: {self.rot_dims} rotary dims do not fit a head of {dk}")
        # 16-bit q for the tensor-core attention kernel (128-wide heads, 64-token blocks, bf16 cache); f32 q for the SIMT one
        self.q_dtype = torch.bfloat16 if (dtype == torch.bfloat16 and dk == dv == 128 and block_size == 64) else torch.float32
        # steps of single tokens: the split-KV decode kernel, when chunks start on block borders and the head layout is one it takes
        self.decode_kernel = (self.q_dtype == torch.bfloat16 and self.chunk % block_size == 0 and self.window == 0 and heads // kv_heads in (1, 2, 4, 8) and
                              self.sink is None)
        self._scratch = {}
        self.cos = self.sin = None
        self._device = self.w_in.device
        if rot:
            self.ensure_positions(max_pos)
        if self.q_norm is not None and self.q_norm.numel() != (dk if head_norm != "none" else heads * dk):
            raise BackendError(f"PagedAttentionMixer: q.norm has {self.q_norm.numel()} entries for head_norm {head_norm!r}")

    def ensure_positions(self, max_pos: int) -> None:
        if self.rot and (self.cos is None or self.cos.shape[0] < max_pos):
            self.cos, self.sin = yarn_rotary_tables(self.rot_dims, float(self.rot["base"]), max_pos, self.rot.get("scaling"), self._device)

    def cache_shape(self):
        return (self.G, self.dk, self.dv)

    def forward(self, h: torch.Tensor, batch: StepBatch, cache, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``proj``: the product of ``w_in`` with the input when the caller has it already (columns of a wider fused projection)"""
        k_cache, v_cache = cache
        if self.rot and batch.max_position >= self.cos.shape[0]:
            self.ensure_positions(max(2 * self.cos.shape[0], batch.max_position + 1))
        if proj is None:
            proj = ops.linear(h, self.w_in)
        if self.per_head:
            q = ops.qk_head_norm_rope_cache(proj, self.bias, self.q_norm, self.k_norm, self.cos, self.sin, batch, k_cache, v_cache, self.H, self.G, self.dk, self.dv,
                                            self.rot_dims, self.eps, interleaved=self.interleaved, norm=self.head_norm, q_dtype=self.q_dtype)
        else:
            q = ops.qk_norm_rope_cache(proj, self.q_norm, self.k_norm, self.cos, self.sin, batch, k_cache, v_cache, self.H, self.G, self.dk, self.dv,
                                       self.rot_dims, self.eps, self.q_dtype, q_temp=self.q_temp, v_unit_rms=self.value_norm)
        if self.decode_kernel and batch.pure_decode and batch.num_seqs <= 256:
            # without a chunk mask the whole table is one chunk
            a = ops.paged_attention_decode_chunked(q, k_cache, v_cache, batch, self.H, self.G, self.dk, self.block_size, self.scale,
                                                   self.chunk or batch.block_tables.shape[1] * self.block_size, self._scratch)
        else:
            # on the SIMT kernel gated head outputs stay f32 until the gate has been applied and take the compute dtype once; the tensor-core kernel
            # (16-bit q) returns 16 bits
            a = ops.paged_attention_varlen_sink(q, k_cache, v_cache, batch, self.H, self.G, self.dk, self.dv, self.block_size, self.scale, self.chunk,
                                                self.window, self.sink, torch.float32 if (self.has_gate and self.q_dtype == torch.float32) else self.dtype)
        if self.has_gate:
            a = ops.head_gate(a, proj[:, self.off_g:], self.H, self.dv, self.dtype)
        return ops.linear(a, self.w_o)


class PooledWindowAttentionMixer:
    """Grouped-query attention without a softmax: the weight of a visible key is sigmoid(q . k scale + pb[h]), and the weights are not normalised over the
    keys.  A query at position i sees the tokens j with 0 <= i - j < window and, beside them and treated like them, one mean key / mean value per block of
    ``pool`` positions that lies wholly before the window (block b = positions b pool .. b pool + pool - 1, seen once b pool + pool - 1 <= i - window).
    q and k are normed head by head (weights q.norm / k.norm [dk] shared by the heads), nothing is rotated, and the value of a token is its key as projected
    (there is no value projection), so dv = dk.  The paged cache holds the normed keys and the raw keys (as values); a pooled cache beside it holds, page by
    page, the means of the blocks that end in the page (csrc/attention_window.cu).

    weights: q [H dk, D], k [G dk, D], o [D, H dk]; optional q.norm, k.norm [dk], pb [H].  window = 0: every earlier token is seen (and no pooled block)."""
    kind = "kv"

    def __init__(self, w: Dict[str, torch.Tensor], heads: int, kv_heads: int, dk: int, scale: float, eps: float, dtype: torch.dtype, window: int = 0, pool: int = 0,
                 block_size: int = 64):
        if heads % kv_heads:
            raise BackendError("PooledWindowAttentionMixer: heads must be a multiple of kv_heads")
        if tuple(w["q"].shape)[0] != heads * dk or tuple(w["k"].shape)[0] != kv_heads * dk or tuple(w["o"].shape)[1] != heads * dk:
            raise BackendError(f"PooledWindowAttentionMixer: q {tuple(w['q'].shape)}, k {tuple(w['k'].shape)}, o {tuple(w['o'].shape)} for {heads} / {kv_heads} heads of {dk}")
        self.H, self.G, self.dk, self.dv, self.scale, self.eps, self.dtype = heads, kv_heads, dk, dk, float(scale), eps, dtype
        self.window, self.block_size = int(window), block_size
        self.pool = int(pool) if self.window > 0 else 0
        self.w_in = torch.cat([w["q"], w["k"]], 0).to(dtype).contiguous()
        self.q_norm = w["q.norm"].float().contiguous() if "q.norm" in w else None
        self.k_norm = w["k.norm"].float().contiguous() if "k.norm" in w else None
        self.head_bias = w["pb"].float().contiguous() if "pb" in w else None
        self.w_o = w["o"].to(dtype).contiguous()
        # 16-bit q for the tensor-core attention kernel (128-wide heads, 64-token blocks, bf16 cache); f32 q for the SIMT one
        self.q_dtype = torch.bfloat16 if (dtype == torch.bfloat16 and dk == 128 and block_size == 64) else torch.float32

    def cache_shape(self):
        return (self.G, self.dk, self.dk)

    def pool_shape(self):
        """(pooled entries per page, kv heads, key size, value size) of the f32 pooled cache, None without pooling"""
        return (ops.pooled_entries_per_block(self.block_size, self.pool), self.G, self.dk, self.dk) if self.pool else None

    def forward(self, h: torch.Tensor, batch: StepBatch, cache, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        k_cache, v_cache = cache[0], cache[1]
        k_pool, v_pool = (cache[2], cache[3]) if self.pool else (None, None)
        if proj is None:
            proj = ops.linear(h, self.w_in)
        q = ops.qk_head_norm_rope_cache(proj, None, self.q_norm, self.k_norm, None, None, batch, k_cache, v_cache, self.H, self.G, self.dk, self.dk, 0, self.eps,
                                        norm="before", v_from_k=True, q_dtype=self.q_dtype)
        if self.pool:
            ops.pooled_cache_update(k_cache, v_cache, k_pool, v_pool, batch, self.pool)
        a = ops.paged_attention_sigmoid_pooled(q, k_cache, v_cache, k_pool, v_pool, batch, self.head_bias, self.H, self.scale, self.window, self.pool, self.dtype)
        return ops.linear(a, self.w_o)


class GatedMlp:
    """down(act(gate x) * (up x)), act the tanh GELU or SiLU; gate, up [ff, D], down [D, ff]."""

    def __init__(self, w: Dict[str, torch.Tensor], dtype: torch.dtype, act: str = "gelu_tanh"):
        if act not in ("gelu_tanh", "silu"):
            raise BackendError(f"GatedMlp: unknown activation {act!r}")
        self.dtype, self.act = dtype, act
        self.w_in = torch.cat([w["gate"], w["up"]], 0).to(dtype).contiguous()
        self.w_down = w["down"].to(dtype).contiguous()

    def forward(self, h: torch.Tensor, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``proj``: the product of ``w_in`` with the input when the caller has it already (columns of a wider fused projection)"""
        if proj is None:
            proj = ops.linear(h, self.w_in)
        if self.act == "gelu_tanh":
            return ops.linear(ops.gelu_tanh_mul(proj, self.dtype), self.w_down)
        return ops.linear(ops.glu_packed(proj, self.act, self.dtype), self.w_down)


class UngatedMlp:
    """down(act(up x)) with act = relu(.)^2; up [ff, D], down [D, ff]."""

    def __init__(self, w: Dict[str, torch.Tensor], dtype: torch.dtype, act: str = "relu2"):
        if act != "relu2":
            raise BackendError(f"UngatedMlp: unknown activation {act!r}")
        self.dtype, self.act = dtype, act
        self.w_in = w["up"].to(dtype).contiguous()
        self.w_down = w["down"].to(dtype).contiguous()
        self.ff = self.w_in.shape[0]

    def forward(self, h: torch.Tensor, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``proj``: the product of ``w_in`` with the input when the caller has it already (columns of a wider fused projection)"""
        if proj is None:
            proj = ops.linear(h, self.w_in)
        return ops.linear(ops.glu_packed(proj, self.act, self.dtype), self.w_down)


GROUPED_MIN_ROWS = 256        # token-choice pairs from which the expert products take 128-row tiles per expert (below: 32-row tiles, weights on the 128-row side)
GROUPED_MIN_TOKENS = 16       # rows from which the latent up-projections run head by head on the tensor-core GEMM (each head's rows padded to 128)


class LatentAttentionMixer:
    """Multi-head attention over a low-rank latent: per token the cache holds the normed latent c [rank] and one rotated key part [rot_dim] shared by
    all heads; head h's key is (W_uk[h] c | rotated part), its value W_uv[h] c; the softmax denominator may hold a per-head sink, the head outputs
    may be gated by sigmoid(W_g x)[h] (csrc/latent_attention.cu, absorbed form: W_uk is folded into the query, W_uv applied after the sum).

    weights: q [H (dn + rot_dim), D] (per head: dn unrotated then rot_dim rotated), dkv [rank + rot_dim, D] and dkv.norm [rank] (absent when
    ``shared``: the layer then attends over the cache another layer writes), uk [H dn, rank], uv [H dv, rank], o [D, H dv]; optional sink [H], g [H, D].
    With ``q_rank`` the queries go through a latent of their own: dq [q_rank, D], dq.norm [q_rank], uq [H (dn + rot_dim), q_rank] take the place of q
    (q = uq rms_norm(dq h)).  ``gate`` "element": g is [H dv, D], one sigmoid gate per output entry instead of one per head.
    rot = dict(base, scaling) or None (the rotation always spans the whole rot_dim part); window = 0 for none."""
    kind = "kv"

    def __init__(self, w: Dict[str, torch.Tensor], heads: int, dn: int, rot_dim: int, dv: int, rank: int, scale: float, eps: float, dtype: torch.dtype,
                 rot: Optional[dict] = None, shared: bool = False, window: int = 0, block_size: int = 64, max_pos: int = 4096, q_rank: int = 0,
                 gate: str = "head"):
        if rot_dim % 2:
            raise BackendError(f"LatentAttentionMixer: the rotated part has {rot_dim} entries, not an even number")
        if gate not in ("head", "element"):
            raise BackendError(f"LatentAttentionMixer: gate {gate!r} (head / element)")
        self.H, self.dn, self.dr, self.dv, self.R, self.scale, self.eps, self.dtype = heads, dn, rot_dim, dv, rank, float(scale), eps, dtype
        self.shared, self.window, self.block_size, self.rot = bool(shared), int(window), block_size, rot
        self.q_rank, self.gate_per_element = int(q_rank), gate == "element"
        if self.q_rank:
            if tuple(w["dq"].shape)[0] != self.q_rank or tuple(w["uq"].shape) != (heads * (dn + rot_dim), self.q_rank):
                raise BackendError(f"LatentAttentionMixer: dq {tuple(w['dq'].shape)} / uq {tuple(w['uq'].shape)} for a query latent of {self.q_rank}")
            self.q_norm = w["dq.norm"].float().contiguous() if "dq.norm" in w else torch.ones(self.q_rank, dtype=torch.float32, device=w["dq"].device)
            self.w_uq = w["uq"].to(dtype).contiguous()
        parts = [w["dq"] if self.q_rank else w["q"]]
        self.off_dkv = self.q_rank if self.q_rank else heads * (dn + rot_dim)
        self.off_g = self.off_dkv
        if not shared:
            parts.append(w["dkv"])
            self.off_g += rank + rot_dim
        self.has_gate = "g" in w
        if self.has_gate:
            parts.append(w["g"])
        self.w_in = torch.cat(parts, 0).to(dtype).contiguous()
        want = {"uk": (heads * dn, rank), "uv": (heads * dv, rank), "o": (None, heads * dv)}
        if not self.q_rank:
            want["q"] = (heads * (dn + rot_dim),)
        if self.has_gate:
            want["g"] = (heads * (dv if self.gate_per_element else 1),)
        if not shared:
            want["dkv"] = (rank + rot_dim,)
        for name, shape in want.items():
            got = tuple(w[name].shape)
            if any(s is not None and s != g for s, g in zip(shape, got)):
                raise BackendError(f"LatentAttentionMixer: {name} is {got}, expected {shape}")
        self.c_norm = None if shared or "dkv.norm" not in w else w["dkv.norm"].float().contiguous()
        self.sink = w["sink"].float().contiguous() if "sink" in w else None
        self.w_uk = w["uk"].to(dtype).contiguous()
        self.w_uv = w["uv"].to(dtype).contiguous()
        self.w_o = w["o"].to(dtype).contiguous()
        # steps with many rows (bf16, TMA-sized operands): both up-projections run head by head as ONE grouped product on the tensor-core GEMM;
        # its weight operand is [n, k] per head: W_uk[h]^T [rank, dn] and W_uv[h] [dv, rank]
        self.grouped = dtype == torch.bfloat16 and dn % 8 == 0 and rank % 8 == 0 and dn >= 64 and rank >= 64
        self.uk_t = self.w_uk.view(heads, dn, rank).transpose(1, 2).contiguous() if self.grouped else None
        self._tile_heads = {}
        self.decode_kernel = self.grouped and ops.latent_decode_kernel_supported(rank, rot_dim, block_size, dtype)
        self.cos = self.sin = None
        self._device = self.w_in.device
        if rot and rot_dim:
            self.ensure_positions(max_pos)

    def ensure_positions(self, max_pos: int) -> None:
        if self.rot and self.dr and (self.cos is None or self.cos.shape[0] < max_pos):
            self.cos, self.sin = yarn_rotary_tables(self.dr, float(self.rot["base"]), max_pos, self.rot.get("scaling"), self._device)

    def cache_shape(self):
        return (1, self.R, max(self.dr, 1))             # "keys" = latents, "values" = the shared rotated key part

    def forward(self, h: torch.Tensor, batch: StepBatch, cache) -> torch.Tensor:
        c_cache, kr_cache = cache
        if self.cos is not None and batch.max_position >= self.cos.shape[0]:
            self.ensure_positions(max(2 * self.cos.shape[0], batch.max_position + 1))
        proj = ops.linear(h, self.w_in)
        if not self.shared:
            ops.latent_kv_rope_cache(proj, self.off_dkv, self.c_norm, self.cos, self.sin, batch, c_cache, kr_cache, self.R, self.dr, self.eps)
        gate = proj[:, self.off_g:] if self.has_gate else None
        if self.q_rank:
            # the queries' own latent: normed in f32, then up to the heads; from here on `proj` holds q at column 0 like a direct projection
            proj = ops.linear(ops.rms_norm_ex(proj[:, :self.q_rank], self.q_norm, self.eps, 0.0, self.dtype), self.w_uq)
        T = proj.shape[0]
        if self.grouped and T >= GROUPED_MIN_TOKENS:
            # head-major buffers, every head's rows padded to whole 128-row tiles; tile i belongs to head i // (tiles per head)
            Tp = -(-T // 128) * 128
            if Tp not in self._tile_heads:
                self._tile_heads[Tp] = (torch.arange(self.H * Tp // 128, dtype=torch.int32, device=proj.device) // (Tp // 128)).to(torch.int32)
            heads_of = self._tile_heads[Tp]
            qn16 = torch.zeros((self.H, Tp, self.dn), dtype=torch.bfloat16, device=proj.device) if Tp != T else torch.empty((self.H, Tp, self.dn), dtype=torch.bfloat16,
                                                                                                                         device=proj.device)
            q_hm = torch.empty((self.H, Tp, self.R + self.dr), dtype=torch.float32, device=proj.device)
            q_lat = q_hm.transpose(0, 1)                                     # [Tp, H, R + dr] view: token stride R + dr, head stride Tp (R + dr)
            ops.latent_q_absorb(proj, None, self.cos, self.sin, batch, self.H, self.dn, self.dr, self.R, q_lat=q_lat, qn16=qn16)
            ops.linear_grouped(qn16.view(self.H * Tp, self.dn), self.uk_t, heads_of, q_hm.view(self.H * Tp, self.R + self.dr))
            o16 = torch.zeros((self.H, Tp, self.R), dtype=torch.bfloat16, device=proj.device) if Tp != T else torch.empty((self.H, Tp, self.R), dtype=torch.bfloat16,
                                                                                                                       device=proj.device)
            if self.decode_kernel:
                # the sizes the split-KV tensor-core kernel of the latent cache takes: every row (a decoded token or a row of a prompt) goes in as a
                # one-row sequence with its own context length; token-major 16-bit queries in, latents out
                qa = ops.repack_heads(q_lat[:T, :, :self.R], torch.empty((T, self.H, self.R), dtype=torch.bfloat16, device=proj.device))
                qr = ops.repack_heads(q_lat[:T, :, self.R:], torch.empty((T, self.H, self.dr), dtype=torch.bfloat16, device=proj.device))
                tables, ctx = ops.token_tables(batch)
                ops.repack_heads(ops.latent_attention_decode(qa, qr, c_cache, kr_cache, tables, ctx, self.sink, self.scale, self.window), o16.transpose(0, 1)[:T])
            else:
                ops.latent_attention_varlen(q_lat[:T], c_cache, kr_cache, batch, self.sink, self.H, self.R, self.dr, self.block_size, self.scale, self.window,
                                            out=o16.transpose(0, 1)[:T])
            v_hm = torch.empty((self.H, Tp, self.dv), dtype=torch.float32, device=proj.device)
            ops.linear_grouped(o16.view(self.H * Tp, self.R), self.w_uv.view(self.H, self.dv, self.R), heads_of, v_hm.view(self.H * Tp, self.dv))
            a = ops.latent_out_gate(v_hm.transpose(0, 1)[:T], None, gate, self.H, self.dv, self.R, self.dtype, self.gate_per_element)
        else:
            q_lat = ops.latent_q_absorb(proj, self.w_uk, self.cos, self.sin, batch, self.H, self.dn, self.dr, self.R)
            o_lat = ops.latent_attention_varlen(q_lat, c_cache, kr_cache, batch, self.sink, self.H, self.R, self.dr, self.block_size, self.scale, self.window)
            a = ops.latent_out_gate(o_lat, self.w_uv, gate, self.H, self.dv, self.R, self.dtype, self.gate_per_element)
        return ops.linear(a, self.w_o)


class RoutedExperts:
    """Mixture of experts with a softmax router: down(silu(gate x) * (up x)) per expert, weights e<j>.gate / e<j>.up [ff, D], e<j>.down [D, ff],
    router [N, D], optional correction [N] (added to the scores for the choice only).  N = experts + identity: the last ``identity`` router outputs
    are experts without weights whose output is the input itself.  ``groups`` / ``keep`` restrict the choice to the best groups of neighbouring
    outputs (0 = off); the chosen scores are normalised and multiplied by ``scale`` (csrc/moe_ragged.cu).

    ``score`` "sigmoid" scores every output by itself; ``normalise`` False keeps the chosen scores as they are; ``weight_input`` feeds an expert its token
    times the score instead of scaling what the expert returns; ``act`` "clamped" is g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u,
    +-limit); ``act`` "relu2" makes the experts ungated, down(relu(up x)^2) with weights e<j>.up / e<j>.down only.  An optional router.b [N] is a bias of
    the logits (it counts for the choice and for the weights; softmax scores normalised over the chosen = a softmax over the chosen logits)."""

    def __init__(self, w: Dict[str, torch.Tensor], experts: int, identity: int, top: int, scale: float, dtype: torch.dtype, groups: int = 0, keep: int = 0,
                 score: str = "softmax", normalise: bool = True, weight_input: bool = False, act: str = "silu", limit: float = 0.0):
        self.E, self.I, self.top, self.scale, self.groups, self.keep, self.dtype = experts, identity, top, float(scale), int(groups), int(keep), dtype
        if score not in ("softmax", "sigmoid") or act not in ("silu", "clamped", "relu2") or (weight_input and identity):
            raise BackendError(f"RoutedExperts: score {score!r} / activation {act!r} / weighted input with identity experts")
        self.score, self.normalise, self.weight_input, self.act, self.limit = score, bool(normalise), bool(weight_input), act, float(limit)
        self.N = experts + identity
        if tuple(w["router"].shape)[0] != self.N:
            raise BackendError(f"RoutedExperts: the router has {w['router'].shape[0]} outputs, expected {experts} + {identity}")
        if top > self.N or (self.groups > 1 and (self.N % self.groups or not 0 < self.keep <= self.groups)):
            raise BackendError(f"RoutedExperts: top {top} / groups {groups} / keep {keep} do not fit {self.N} router outputs")
        self.router = w["router"].to(dtype).contiguous()
        self.correction = w["correction"].float().contiguous() if "correction" in w else None
        self.router_bias = w["router.b"].float().contiguous() if "router.b" in w else None
        self.w_gu = self.w_d = None
        self.ff = 0
        if experts:
            first = (lambda j: w[f"e{j}.up"]) if act == "relu2" else (lambda j: torch.cat([w[f"e{j}.gate"], w[f"e{j}.up"]], 0))
            self.w_gu = torch.stack([first(j) for j in range(experts)], 0).to(dtype).contiguous()
            self.w_d = torch.stack([w[f"e{j}.down"] for j in range(experts)], 0).to(dtype).contiguous()
            self.ff = self.w_d.shape[2]
        D = self.router.shape[1]
        # steps with many rows (bf16, TMA-sized operands): pairs sorted by expert, both expert products as grouped products on the tensor-core GEMM
        self.grouped = bool(experts) and dtype == torch.bfloat16 and D % 8 == 0 and self.ff % 8 == 0 and D >= 64 and self.ff >= 64

    def forward(self, h: torch.Tensor, x: torch.Tensor, logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h: the input in the compute dtype, x: the same rows in f32 (what an identity expert returns); ``logits``: the router's product when the caller has
        it already (columns of a wider fused projection)"""
        if logits is None:
            logits = ops.linear(h, self.router)
        ids, wts = ops.moe_route(logits, self.correction, self.top, self.groups, self.keep, self.scale, self.score, self.normalise, bias=self.router_bias)
        # a weight on the expert's input is applied to both of its first products (W (s h) = s W h), in f32, before the activation
        pre, post = (wts, None) if self.weight_input else (None, wts)
        if self.grouped:
            # pairs sorted by expert into tiles of 128 rows, or of 32 while experts have few rows each (the weights then take the 128-row side of the MMA and
            # stream once per tile)
            tile = 128 if h.shape[0] * self.top >= GROUPED_MIN_ROWS else 32
            pair_row, row_pair, tile_expert = ops.moe_sorted_rows(ids, self.E, tile)
            xg = ops.moe_gather_rows(h, row_pair, self.top)
            gu = ops.linear_grouped(xg, self.w_gu, tile_expert, torch.empty((xg.shape[0], self.w_gu.shape[1]), dtype=torch.float32, device=h.device), tile)
            if self.act == "silu" and pre is None:
                act = ops.silu_mul_packed(gu, torch.bfloat16)
            else:
                act = ops.glu_packed(gu, self.act, torch.bfloat16, self.limit, row_scale=None if pre is None else pre.view(-1), scale_index=None if pre is None else row_pair)
            y = ops.linear_grouped(act, self.w_d, tile_expert, torch.empty((xg.shape[0], self.w_d.shape[1]), dtype=torch.float32, device=h.device), tile)
            return ops.moe_combine_rows(y, pair_row, post, x)
        if not self.E:                                       # identity experts only
            return ops.moe_combine_rows(x, torch.full((ids.numel(),), -1, dtype=torch.int32, device=ids.device), wts, x)
        # few rows: every pair streams its expert; the blocks walk the pairs expert by expert, so that those running together read the same weights
        pair_row, order, _ = ops.moe_sorted_rows(ids, self.E, tile=1)
        act = ops.moe_gate_up(h, self.w_gu, ids, order, self.act, self.limit, None if pre is None else pre.view(-1))
        return ops.moe_combine_rows(ops.moe_down(act, self.w_d, ids, order), pair_row, post, x)


class TokenSideInput:
    """A per-layer, per-token embedding let in by the stream: e = table[token, col0 : col0 + dim]; y = proj (gelu_tanh(gate x) * e);
    x <- x + rms_norm(y) * norm.  weights: gate [dim, D], proj [D, dim], norm [D]; the table [vocab, layers * dim] is shared by the layers."""

    def __init__(self, w: Dict[str, torch.Tensor], table: torch.Tensor, col0: int, dim: int, eps: float, dtype: torch.dtype):
        self.table, self.col0, self.dim, self.eps = table, int(col0), int(dim), eps
        self.w_gate = w["gate"].to(dtype).contiguous()
        self.w_proj = w["proj"].to(dtype).contiguous()
        self.norm = w["norm"].float().contiguous()

    def forward(self, x: torch.Tensor, h: torch.Tensor, batch: StepBatch, out16: Optional[torch.Tensor]) -> None:
        g = ops.gelu_tanh_gather_mul(ops.linear(h, self.w_gate), self.table, self.col0, batch.tokens, self.dim)
        ops.residual_rms_norm(x, ops.linear(g, self.w_proj), self.norm, 1.0, self.eps, False, out16)


class GatedLinearRecurrence:
    """Recurrent block with a real-gated linear recurrent unit.  weights: y, x [C, D] with biases y.b, x.b [C]; conv [C, taps], conv.b [C]; ra, ri
    [blocks, C / blocks, C / blocks] with biases ra.b, ri.b [blocks, C / blocks]; lam [C]; o [D, C].  With u = conv(x h + x.b) + conv.b, per block r =
    sigmoid(ra u + ra.b), i = sigmoid(ri u + ri.b); S <- a S + sqrt(1 - a^2) i u with a = exp(-decay_scale r softplus(lam)); out = o (S * gelu_tanh(y h + y.b)).
    The gates and the recurrence are f32 whatever the compute dtype."""
    kind = "state"

    def __init__(self, w: Dict[str, torch.Tensor], blocks: int, taps: int, dtype: torch.dtype, decay_scale: float = 8.0):
        C = w["x"].shape[0]
        if C % blocks or tuple(w["ra"].shape) != (blocks, C // blocks, C // blocks) or tuple(w["conv"].shape) != (C, taps):
            raise BackendError(f"GatedLinearRecurrence: {C} channels in {blocks} blocks, gates {tuple(w['ra'].shape)}, convolution {tuple(w['conv'].shape)}")
        self.C, self.blocks, self.n, self.taps, self.dtype, self.decay_scale = C, blocks, C // blocks, taps, dtype, float(decay_scale)
        f32 = lambda name: w[name].float().contiguous() if name in w else None
        self.w_in = torch.cat([w["y"], w["x"]], 0).to(dtype).contiguous()
        self.y_bias, self.x_bias, self.conv, self.conv_bias, self.lam = f32("y.b"), f32("x.b"), f32("conv"), f32("conv.b"), f32("lam")
        self.w_gates = torch.cat([w["ra"], w["ri"]], 1).float().contiguous()                        # [blocks, 2 n, n]: recurrence gate rows, then input gate rows
        self.gate_bias = torch.cat([w["ra.b"], w["ri.b"]], 1).float().contiguous() if "ra.b" in w else None
        self.w_o = w["o"].to(dtype).contiguous()

    def state_shapes(self):
        return ((max(self.taps - 1, 1), self.C), (self.C,))

    def forward(self, h: torch.Tensor, batch: StepBatch, cache, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        conv_state, S = cache
        if proj is None:
            proj = ops.linear(h, self.w_in)
        u = ops.causal_conv(proj[:, self.C:], self.conv, conv_state, batch, in_bias=self.x_bias, out_bias=self.conv_bias)
        gates = ops.block_diag_linear(u, self.w_gates, None if self.gate_bias is None else self.gate_bias.view(-1))
        z = ops.gated_linear_scan(u, gates, self.lam, proj[:, :self.C], self.y_bias, S, batch, self.n, self.decay_scale, self.dtype)
        return ops.linear(z, self.w_o)


class DecayLinearAttention:
    """Linear attention with one fixed decay per head: q, k = silu(W h) [H dk], v = silu(W h) [H dv]; S <- decay[h] S + k v^T, o = S^T q; the heads'
    outputs are normed together (RMS, weight norm [H dv]), times sigmoid(g h), projected by o [D, H dv]."""
    kind = "state"

    def __init__(self, w: Dict[str, torch.Tensor], heads: int, dk: int, dv: int, decay, eps: float, dtype: torch.dtype):
        if len(decay) != heads:
            raise BackendError(f"DecayLinearAttention: {len(decay)} decays for {heads} heads")
        self.H, self.dk, self.dv, self.eps, self.dtype = heads, dk, dv, eps, dtype
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"]], 0).to(dtype).contiguous()
        self.off_g = 2 * heads * dk + heads * dv
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=self.w_in.device)
        self.kernel = None                       # None: chosen by the step's shape (tests force one)
        self.norm = w["norm"].float().contiguous()
        self.w_o = w["o"].to(dtype).contiguous()

    def state_shapes(self):
        return ((self.H, self.dv, self.dk),)

    def forward(self, h: torch.Tensor, batch: StepBatch, cache, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        if proj is None:
            proj = ops.linear(h, self.w_in)
        o = ops.linear_attention(proj, 0, self.H * self.dk, 2 * self.H * self.dk, cache[0], batch, self.H, self.dk, self.dv, act="silu", decay=self.decay,
                                 kernel=self.kernel)
        z = ops.group_rms_norm_gate(o, self.norm, proj[:, self.off_g:], 1, self.eps, self.dtype)
        return ops.linear(z, self.w_o)


class MatrixMemoryMixer:
    """Linear attention with exponential gating: q = W_q h dk^-1/2, k, v plain; log input gate i = cap tanh((W_i h + i.b) / cap), log forget gate
    f = logsigmoid(cap tanh((W_f h + f.b) / cap)); with the running maximum m (0 at the start): m' = max(f + m, i), S <- e^(f + m - m') S + e^(i - m') k v^T,
    n alike with k, o = S^T q / (max(|n . q|, e^(-m')) + 1e-6); each head's o over its root mean square, times norm [H dv], times sigmoid(g h), then o [D, H dv]."""
    kind = "state"

    def __init__(self, w: Dict[str, torch.Tensor], heads: int, dk: int, dv: int, cap: float, eps: float, dtype: torch.dtype):
        self.H, self.dk, self.dv, self.cap, self.eps, self.dtype = heads, dk, dv, float(cap), eps, dtype
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"], w["i"], w["f"]], 0).to(dtype).contiguous()
        self.off_g = 2 * heads * dk + heads * dv
        self.off_i = self.off_g + heads * dv
        self.off_f = self.off_i + heads
        self.kernel = None                       # None: chosen by the step's shape (tests force one)
        self.i_bias = w["i.b"].float().contiguous() if "i.b" in w else None
        self.f_bias = w["f.b"].float().contiguous() if "f.b" in w else None
        self.norm = w["norm"].float().contiguous()
        self.w_o = w["o"].to(dtype).contiguous()

    def state_shapes(self):
        nvb = -(-self.dv // 16)                     # the normaliser and the maximum are kept once per block of 16 value columns
        return ((self.H, self.dv, self.dk), (self.H, nvb, self.dk), (self.H, nvb))

    def forward(self, h: torch.Tensor, batch: StepBatch, cache, proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        S, n, m = cache
        if proj is None:
            proj = ops.linear(h, self.w_in)
        gates = dict(off_i=self.off_i, off_f=self.off_f, i_bias=self.i_bias, f_bias=self.f_bias, cap=self.cap, normaliser=n, maximum=m)
        o = ops.linear_attention(proj, 0, self.H * self.dk, 2 * self.H * self.dk, S, batch, self.H, self.dk, self.dv, q_scale=self.dk ** -0.5, gates=gates,
                                 kernel=self.kernel)
        z = ops.group_rms_norm_gate(o, self.norm, proj[:, self.off_g:], self.H, self.eps, self.dtype)
        return ops.linear(z, self.w_o)


class ParallelMixer:
    """Two mixers on the same input, one fused input projection; result = (rms(left) * left_out + rms(right) * right_out) / 2 over the model width.
    ``left`` keeps a paged cache, ``right`` a state."""
    kind = "both"

    def __init__(self, left, right, left_out: torch.Tensor, right_out: torch.Tensor, eps: float):
        self.left, self.right, self.eps = left, right, eps
        self.w_in = torch.cat([left.w_in, right.w_in], 0).contiguous()
        self.split = left.w_in.shape[0]
        self.left_out, self.right_out = (0.5 * left_out.float()).contiguous(), (0.5 * right_out.float()).contiguous()       # the halving is exact in the weights

    def cache_shape(self):
        return self.left.cache_shape()

    def state_shapes(self):
        return self.right.state_shapes()

    def forward(self, h: torch.Tensor, batch: StepBatch, kv, state) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        a = self.left.forward(h, batch, kv, proj=proj[:, :self.split])
        b = self.right.forward(h, batch, state, proj=proj[:, self.split:])
        y = ops.rms_norm_ex(a, self.left_out, self.eps, 0.0, torch.float32)
        return ops.rms_norm_ex(b, self.right_out, self.eps, 0.0, torch.float32, residual=y, out=y)
