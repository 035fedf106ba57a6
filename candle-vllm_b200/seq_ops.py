"""Operator wrappers for ragged-step models: the C entry points that serve portions of prompts beside single decoded tokens in one
launch (include/b200_backend.h: linear_f32out ... paged_attention_varlen).  Same conventions as ``backend.py``: torch tensors are
device memory and stream plumbing only, every op is one hand-written kernel launch on the current stream, errors raise
``BackendError``; nothing here allocates on the host or synchronises, so a step can be captured into a CUDA graph.

``StepBatch`` is the device-side description of one step that ``inputs.prepare_step`` builds on the host.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ._lib import BackendError, check, lib
from .backend import DType, _ptr, _stream

_B200 = {torch.float32: DType.F32, torch.bfloat16: DType.BF16}


def _tag(dt: torch.dtype) -> int:
    try:
        return _B200[dt]
    except KeyError:
        raise BackendError(f"ragged-step ops take f32 / bf16, not {dt}")


@dataclass
class StepBatch:
    """One step on the device (all i32 unless said): T rows, B entries, R wanted rows."""
    tokens: torch.Tensor          # [T]
    positions: torch.Tensor       # [T] position of each row in its sequence
    token_seq: torch.Tensor       # [T] entry that owns the row
    slot_mapping: torch.Tensor    # [T] i64, flat cache slot = block * block_size + offset
    cu_seqlens: torch.Tensor      # [B + 1] rows
    cu_seqlens_k: torch.Tensor    # [B + 1] context lengths (start + rows), cumulative
    seq_slots: torch.Tensor       # [B] state slot of each entry's sequence
    seq_start: torch.Tensor       # [B] position of each entry's first row (0 = new sequence)
    block_tables: torch.Tensor    # [B, W]
    want_rows: torch.Tensor       # [R] rows whose logits are returned
    num_tokens: int = 0
    num_seqs: int = 0
    num_want: int = 0
    max_position: int = 0
    pure_decode: bool = False     # every entry brings exactly one token
    max_rows: int = 1             # the most rows any entry brings

    @classmethod
    def from_host(cls, prep: dict, device="cuda") -> "StepBatch":
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dt)).to(device, non_blocking=True)
        return cls(tokens=t(prep["tokens"], np.int32), positions=t(prep["positions"], np.int32), token_seq=t(prep["token_seq"], np.int32),
                   slot_mapping=t(prep["slot_mapping"], np.int64), cu_seqlens=t(prep["cu_seqlens"], np.int32), cu_seqlens_k=t(prep["cu_seqlens_k"], np.int32),
                   seq_slots=t(prep["seq_slots"], np.int32), seq_start=t(prep["seq_start"], np.int32),
                   block_tables=t(prep["block_tables"], np.int32), want_rows=t(prep["want_rows"], np.int32),
                   num_tokens=len(prep["tokens"]), num_seqs=len(prep["seq_slots"]), num_want=len(prep["want_rows"]),
                   max_position=int(prep["max_position"]), pure_decode=len(prep["tokens"]) == len(prep["seq_slots"]),
                   max_rows=int(np.diff(np.asarray(prep["cu_seqlens"], np.int64)).max()) if len(prep["seq_slots"]) else 1)


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [m, k] (rows may be strided) . weight [n, k]^T -> f32 [m, n]; both operands f32 (true 32-bit product) or both bf16."""
    if x.dtype != weight.dtype or x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or not weight.is_contiguous():
        raise BackendError(f"linear: x {tuple(x.shape)} {x.dtype} vs weight {tuple(weight.shape)} {weight.dtype}")
    m, k = x.shape
    n = weight.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    lib().linear_f32out(_ptr(x), _ptr(weight), _ptr(out), C.c_int32(m), C.c_int32(n), C.c_int32(k), C.c_int64(x.stride(0) if m > 1 else max(k, x.stride(0))),
                        C.c_int64(out.stride(0) if m > 1 else max(n, out.stride(0))), C.c_int32(_tag(x.dtype)), _stream(x.device))
    check("linear")
    return out


def rms_norm_ex(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype, residual: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of f32 rows times (offset + weight); with ``residual`` the result is added to it (pass out=residual for in place);
    ``row_index`` (i32) selects the rows to normalise."""
    n = x.shape[-1]
    rows = x.shape[0] if row_index is None else row_index.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or x.stride(-1) != 1:
        raise BackendError("rms_norm_ex: x and weight are f32")
    if out is None:
        out = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    lib().rms_norm_ex(_ptr(x), _ptr(weight), _ptr(out), _ptr(residual), _ptr(row_index), C.c_int32(rows), C.c_int32(n), C.c_int64(x.stride(0) if x.shape[0] > 1 else n),
                      C.c_float(eps), C.c_float(offset), C.c_int32(_tag(out.dtype)), _stream(x.device))
    check("rms_norm_ex")
    return out


def gelu_tanh_mul(gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    rows, two_ff = gate_up.shape
    ff = two_ff // 2
    out = torch.empty((rows, ff), dtype=out_dtype, device=gate_up.device)
    lib().gelu_tanh_mul(_ptr(gate_up), _ptr(out), C.c_int64(rows), C.c_int32(ff), C.c_int64(gate_up.stride(0) if rows > 1 else two_ff),
                        C.c_int32(_tag(out_dtype)), _stream(gate_up.device))
    check("gelu_tanh_mul")
    return out


def embedding_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    vocab, dim = table.shape
    out = torch.empty((ids.shape[0], dim), dtype=torch.float32, device=table.device)
    lib().embedding_scaled(_ptr(table), _ptr(ids), _ptr(out), C.c_int32(ids.shape[0]), C.c_int32(dim), C.c_int32(vocab), C.c_float(scale),
                           C.c_int32(_tag(table.dtype)), _stream(table.device))
    check("embedding_scaled")
    return out


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor, conv_state: torch.Tensor, batch: StepBatch) -> torch.Tensor:
    """x: f32 view [T, C] of the fused projection (row stride allowed); taps f32 [C, K]; conv_state f32 [slots, K-1, C], advanced in place."""
    T, Cn = x.shape
    K = taps.shape[1]
    if T > 65535:
        raise BackendError("causal_conv_silu: at most 65535 rows per step")
    y = torch.empty((T, Cn), dtype=torch.float32, device=x.device)
    lib().causal_conv_silu(_ptr(x), C.c_int64(x.stride(0) if T > 1 else max(Cn, x.stride(0))), _ptr(taps), _ptr(conv_state), _ptr(y), _ptr(batch.token_seq),
                           _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T), C.c_int32(batch.num_seqs), C.c_int32(Cn),
                           C.c_int32(K), _stream(x.device))
    check("causal_conv_silu")
    return y


TILED_DELTA_MIN_ROWS = 8      # steps in which some entry brings at least this many rows take the tiled form of the rule


def gated_delta_rule(qkv: torch.Tensor, proj: torch.Tensor, off_b: int, off_a: int, A_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
                     batch: StepBatch, heads: int, kv_heads: int, dk: int, dv: int, kernel: Optional[str] = None) -> torch.Tensor:
    """qkv f32 [T, G dk | G dk | H dv]; b / a read from columns off_b.. / off_a.. of ``proj``; state f32 [slots, H, dv, dk] advanced in place.
    Three kernels compute the same rule: "step" (every entry brings one token: one pass over the state, nothing staged), "tiled" (over
    tiles of 16 tokens, for portions of prompts; key sizes up to 128) and "token" (token by token, any step).  ``kernel`` forces one;
    None chooses by the step's shape."""
    T = qkv.shape[0]
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=qkv.device)
    ld_proj = C.c_int64(proj.stride(0) if T > 1 else proj.shape[1])
    if kernel is None:
        kernel = "step" if batch.pure_decode else "tiled" if (dk <= 128 and batch.max_rows >= TILED_DELTA_MIN_ROWS) else "token"
    if kernel == "step":
        if T != batch.num_seqs:
            raise BackendError("gated_delta_rule: the single-token kernel takes one row per entry")
        lib().gated_delta_rule_step(_ptr(qkv), _ptr(proj), ld_proj, C.c_int32(off_b), C.c_int32(off_a), _ptr(A_log), _ptr(dt_bias), _ptr(state), _ptr(out),
                                    _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(batch.num_seqs), C.c_int32(heads), C.c_int32(kv_heads),
                                    C.c_int32(dk), C.c_int32(dv), _stream(qkv.device))
        check("gated_delta_rule_step")
    elif kernel == "tiled":
        scratch = torch.empty((T * (2 * kv_heads * dk + 35 * heads),), dtype=torch.float32, device=qkv.device)
        lib().gated_delta_rule_tiled(_ptr(qkv), _ptr(proj), ld_proj, C.c_int32(off_b), C.c_int32(off_a), _ptr(A_log), _ptr(dt_bias), _ptr(state), _ptr(out),
                                     _ptr(scratch), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T),
                                     C.c_int32(batch.num_seqs), C.c_int32(batch.max_rows), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk),
                                     C.c_int32(dv), _stream(qkv.device))
        check("gated_delta_rule_tiled")
    elif kernel == "token":
        lib().gated_delta_rule(_ptr(qkv), _ptr(proj), ld_proj, C.c_int32(off_b), C.c_int32(off_a), _ptr(A_log),
                               _ptr(dt_bias), _ptr(state), _ptr(out), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start),
                               C.c_int32(batch.num_seqs), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), _stream(qkv.device))
        check("gated_delta_rule")
    else:
        raise BackendError(f"gated_delta_rule: unknown kernel {kernel!r}")
    return out


def gated_rms_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, heads: int, dv: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    T = o.shape[0]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=o.device)
    lib().gated_rms_norm(_ptr(o), _ptr(gate), C.c_int64(gate.stride(0) if T > 1 else max(heads * dv, gate.stride(0))), _ptr(weight), _ptr(out), C.c_int32(T),
                         C.c_int32(heads), C.c_int32(dv), C.c_float(eps), C.c_int32(_tag(out_dtype)), _stream(o.device))
    check("gated_rms_norm")
    return out


def qk_norm_rope_cache(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                       sin: Optional[torch.Tensor], batch: StepBatch, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, dk: int,
                       dv: int, rot_dims: int, eps: float, q_dtype: torch.dtype = torch.float32, q_temp: Optional[tuple] = None,
                       v_unit_rms: bool = False) -> torch.Tensor:
    """``q_temp`` = (coef, every): the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1); ``v_unit_rms``: every value head is
    cached divided by its root mean square."""
    T = qkv.shape[0]
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise BackendError(f"position {batch.max_position} is outside the rotary table ({cos.shape[0]} rows)")
    q = torch.empty((T, heads * dk), dtype=q_dtype, device=qkv.device)
    coef, every = q_temp if q_temp else (0.0, 0)
    lib().qk_norm_rope_cache_ex(_ptr(qkv), C.c_int64(qkv.stride(0) if T > 1 else qkv.shape[1]), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin),
                                C.c_int32(0 if cos is None else cos.shape[0]), _ptr(batch.positions), _ptr(batch.slot_mapping), _ptr(q), _ptr(k_cache),
                                _ptr(v_cache), C.c_int32(T), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), C.c_int32(rot_dims),
                                C.c_float(eps), C.c_float(coef), C.c_int32(every), C.c_int32(1 if v_unit_rms else 0), C.c_int32(_tag(k_cache.dtype)),
                                C.c_int32(_tag(q_dtype)), _stream(qkv.device))
    check("qk_norm_rope_cache")
    return q


def paged_attention_varlen(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: StepBatch, heads: int, kv_heads: int, dk: int, dv: int,
                           block_size: int, scale: float, chunk: int, window: int, out_dtype: torch.dtype) -> torch.Tensor:
    T = q.shape[0]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=q.device)
    lib().paged_attention_varlen(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]),
                                 _ptr(batch.token_seq), _ptr(batch.positions), _ptr(batch.cu_seqlens), _ptr(batch.cu_seqlens_k), C.c_int32(batch.num_seqs),
                                 C.c_int32(T), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), C.c_int32(block_size), C.c_float(scale),
                                 C.c_int32(chunk), C.c_int32(window), C.c_int32(_tag(q.dtype)), C.c_int32(_tag(k_cache.dtype)), C.c_int32(_tag(out_dtype)),
                                 _stream(q.device))
    check("paged_attention_varlen")
    return out


def paged_attention_decode_chunked(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: StepBatch, heads: int, kv_heads: int, hd: int,
                                   block_size: int, scale: float, chunk: int, scratch: dict) -> torch.Tensor:
    """A step of single tokens under a chunk mask with chunk % block_size == 0, on the split-KV decode kernel of ``PagedAttention``: the
    block tables are viewed from each sequence's chunk start (``chunk_decode_view``).  q bf16 [B, H * hd]; ``scratch`` keeps the view
    and the kernel's workspace between calls (allocated on first use, so call once before capturing a graph)."""
    B = q.shape[0]
    width = chunk // block_size
    key = (B, width)
    if key not in scratch:
        if len(scratch) >= 8:                   # tables that grow step by step: keep a few views, not one per width ever seen
            scratch.clear()
        need = lib().paged_attention_decode_workspace_bytes(C.c_int32(B), C.c_int32(heads), C.c_int32(hd), C.c_int32(width), C.c_int32(block_size))
        scratch[key] = (torch.zeros((B, width), dtype=torch.int32, device=q.device), torch.zeros(B, dtype=torch.int32, device=q.device),
                        torch.zeros(int(need), dtype=torch.uint8, device=q.device))
    tables, ctx, ws = scratch[key]
    out = torch.empty((B, heads * hd), dtype=q.dtype, device=q.device)
    L = lib()
    L.chunk_decode_view(_ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]), _ptr(batch.positions), _ptr(tables), _ptr(ctx), C.c_int32(B),
                        C.c_int32(width), C.c_int32(block_size), C.c_int32(chunk), _stream(q.device))
    L.paged_attention_decode(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(tables), _ptr(ctx), C.c_int32(B), C.c_int32(heads), C.c_int32(kv_heads),
                             C.c_int32(hd), C.c_int32(block_size), C.c_int32(width), C.c_int64(k_cache.shape[0]), C.c_float(scale), C.c_float(0.0),
                             C.c_int32(0), C.c_int32(_tag(q.dtype)), C.c_int32(_tag(k_cache.dtype)), C.c_int32(0), C.c_int32(_tag(q.dtype)), _ptr(ws),
                             C.c_size_t(ws.numel()), _stream(q.device))
    check("paged_attention_decode_chunked")
    return out


# ---- latent attention, routed experts, post-sum norms -----------------------------------------------------------------------------------

def embedding_bigram(table: torch.Tensor, bigram: Optional[torch.Tensor], batch: StepBatch, prev_state: Optional[torch.Tensor], buckets: int, mul_prev: int,
                     mul_cur: int) -> torch.Tensor:
    """table[token] + bigram[hash(previous token, token)] -> f32 [T, dim]; ``prev_state`` i32 [slots, 1] carries each sequence's last token
    from step to step (read for an entry's first row, then set to the entry's last token)."""
    vocab, dim = table.shape
    T = batch.tokens.shape[0]
    out = torch.empty((T, dim), dtype=torch.float32, device=table.device)
    if bigram is not None and (bigram.dtype != table.dtype or bigram.shape != (buckets + 1, dim) or prev_state is None or prev_state.dtype != torch.int32):
        raise BackendError(f"embedding_bigram: bigram table {tuple(bigram.shape)} for {buckets} buckets, or no i32 previous-token state")
    lib().embedding_bigram(_ptr(table), _ptr(bigram), _ptr(batch.tokens), _ptr(batch.positions), _ptr(batch.token_seq), _ptr(batch.cu_seqlens),
                           _ptr(batch.seq_slots), _ptr(prev_state), _ptr(out), C.c_int32(T), C.c_int32(dim), C.c_int32(vocab), C.c_int32(buckets),
                           C.c_int32(mul_prev), C.c_int32(mul_cur), C.c_int32(_tag(table.dtype)), _stream(table.device))
    check("embedding_bigram")
    return out


def residual_rms_norm(x: torch.Tensor, y: Optional[torch.Tensor], weight: torch.Tensor, alpha: float, eps: float, after_sum: bool,
                      out16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place on the f32 stream x [T, n]: ``after_sum`` x <- norm(alpha x + y) * w (y None = no sublayer output), else x <- x + norm(y) * w.
    ``out16`` (bf16 [T, n]) also receives the new x."""
    T, n = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or weight.dtype != torch.float32 or (y is not None and (y.dtype != torch.float32 or y.stride(1) != 1)):
        raise BackendError("residual_rms_norm: f32 tensors, x contiguous")
    if out16 is not None and (out16.dtype != torch.bfloat16 or not out16.is_contiguous() or out16.shape != x.shape):
        raise BackendError("residual_rms_norm: out16 is bf16 of x's shape")
    lib().residual_rms_norm(_ptr(x), _ptr(y), C.c_int64(0 if y is None else (y.stride(0) if T > 1 else max(n, y.stride(0)))), _ptr(weight), _ptr(out16), C.c_int32(T),
                            C.c_int32(n), C.c_float(alpha), C.c_float(eps), C.c_int32(0 if after_sum else 1), _stream(x.device))
    check("residual_rms_norm")
    return x


def gelu_tanh_gather_mul(z: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, dim: int) -> torch.Tensor:
    """gelu_tanh(z[t, :dim]) * table[ids[t], col0 : col0 + dim] -> [T, dim] of the table's dtype"""
    T = z.shape[0]
    out = torch.empty((T, dim), dtype=table.dtype, device=z.device)
    lib().gelu_tanh_gather_mul(_ptr(z), C.c_int64(z.stride(0) if T > 1 else max(dim, z.stride(0))), _ptr(table), C.c_int64(table.stride(0)), C.c_int32(col0), _ptr(ids),
                               _ptr(out), C.c_int32(T), C.c_int32(dim), C.c_int32(table.shape[0]), C.c_int32(_tag(table.dtype)), C.c_int32(_tag(table.dtype)),
                               _stream(z.device))
    check("gelu_tanh_gather_mul")
    return out


def latent_kv_rope_cache(proj: torch.Tensor, off: int, norm_w: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], batch: StepBatch,
                         c_cache: torch.Tensor, kr_cache: torch.Tensor, rank: int, rot_dim: int, eps: float) -> None:
    T = proj.shape[0]
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise BackendError(f"position {batch.max_position} is outside the rotary table ({cos.shape[0]} rows)")
    lib().latent_kv_rope_cache(_ptr(proj), C.c_int64(proj.stride(0) if T > 1 else proj.shape[1]), C.c_int32(off), _ptr(norm_w), _ptr(cos), _ptr(sin),
                               C.c_int32(0 if cos is None else cos.shape[0]), _ptr(batch.positions), _ptr(batch.slot_mapping), _ptr(c_cache), _ptr(kr_cache),
                               C.c_int32(T), C.c_int32(rank), C.c_int32(rot_dim), C.c_float(eps), C.c_int32(_tag(c_cache.dtype)), _stream(proj.device))
    check("latent_kv_rope_cache")


def latent_q_absorb(proj: torch.Tensor, w_uk: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], batch: StepBatch, heads: int,
                    dn: int, rot_dim: int, rank: int, q_lat: Optional[torch.Tensor] = None, qn16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """-> q_lat f32 [T, H, rank + rot_dim] (or the given tensor of any token / head strides whose last axis is contiguous); w_uk None writes only
    the rotated part (the caller fills [..., :rank]); ``qn16`` bf16 [H, rows, dn] also receives the unrotated part, head by head."""
    T = proj.shape[0]
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise BackendError(f"position {batch.max_position} is outside the rotary table ({cos.shape[0]} rows)")
    if q_lat is None:
        q_lat = torch.empty((T, heads, rank + rot_dim), dtype=torch.float32, device=proj.device)
    if q_lat.stride(2) != 1 or q_lat.dtype != torch.float32 or (qn16 is not None and (qn16.dtype != torch.bfloat16 or not qn16.is_contiguous())):
        raise BackendError("latent_q_absorb: q_lat is f32 with a contiguous last axis, qn16 contiguous bf16")
    lib().latent_q_absorb(_ptr(proj), C.c_int64(proj.stride(0) if T > 1 else proj.shape[1]), _ptr(w_uk), _ptr(cos), _ptr(sin), C.c_int32(0 if cos is None else cos.shape[0]),
                          _ptr(batch.positions), _ptr(q_lat), C.c_int64(q_lat.stride(0)), C.c_int64(q_lat.stride(1)), _ptr(qn16),
                          C.c_int64(0 if qn16 is None else qn16.shape[1]), C.c_int32(T), C.c_int32(heads), C.c_int32(dn), C.c_int32(rot_dim), C.c_int32(rank),
                          C.c_int32(_tag(w_uk.dtype) if w_uk is not None else DType.F32), _stream(proj.device))
    check("latent_q_absorb")
    return q_lat


LATENT_SPLIT_BLOCKS = 296      # two blocks per SM: steps with fewer (token, head group) blocks cut the keys of every row into runs


def latent_attention_varlen(q_lat: torch.Tensor, c_cache: torch.Tensor, kr_cache: torch.Tensor, batch: StepBatch, sink: Optional[torch.Tensor], heads: int,
                            rank: int, rot_dim: int, block_size: int, scale: float, window: int = 0, out: Optional[torch.Tensor] = None,
                            splits: Optional[int] = None) -> torch.Tensor:
    """q_lat f32 [T, H, rank + rot_dim] (any token / head strides) -> o f32 [T, H, rank], or into ``out`` (f32 or bf16, any token / head strides).
    ``splits``: runs every row's keys are cut into (None: enough blocks to fill the device when the step has few rows, from the table width, so that
    a captured step keeps its choice)."""
    T = q_lat.shape[0]
    if splits is None:
        blocks = T * -(-heads // (8 if heads >= 8 else 4))
        longest = batch.block_tables.shape[1] * block_size if window <= 0 else min(window, batch.block_tables.shape[1] * block_size)
        splits = max(1, min(-(-LATENT_SPLIT_BLOCKS // blocks), longest // 128, 64)) if blocks < LATENT_SPLIT_BLOCKS else 1
    part = torch.empty((T * heads * splits * (rank + 2),), dtype=torch.float32, device=q_lat.device) if splits > 1 else None
    if out is None:
        out = torch.empty((T, heads, rank), dtype=torch.float32, device=q_lat.device)
    if q_lat.stride(2) != 1 or out.stride(2) != 1:
        raise BackendError("latent_attention_varlen: the last axis of q_lat and out is contiguous")
    lib().latent_attention_varlen(_ptr(out), C.c_int64(out.stride(0)), C.c_int64(out.stride(1)), C.c_int32(_tag(out.dtype)), _ptr(q_lat), C.c_int64(q_lat.stride(0)),
                                  C.c_int64(q_lat.stride(1)), _ptr(c_cache), _ptr(kr_cache), _ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]),
                                  _ptr(batch.token_seq), _ptr(batch.positions), _ptr(sink), C.c_int32(T), C.c_int32(heads), C.c_int32(rank), C.c_int32(rot_dim),
                                  C.c_int32(block_size), C.c_float(scale), C.c_int32(window), C.c_int32(_tag(c_cache.dtype)), C.c_int32(splits), _ptr(part),
                                  _stream(q_lat.device))
    check("latent_attention_varlen")
    return out


def latent_out_gate(src: torch.Tensor, w_uv: Optional[torch.Tensor], gate: Optional[torch.Tensor], heads: int, dv: int, rank: int, out_dtype: torch.dtype,
                    gate_per_element: bool = False) -> torch.Tensor:
    """sigmoid(gate[t, h]) * (w_uv[h] src[t, h]) -> [T, H dv]; src f32 [T, H, rank] of any token / head strides; w_uv None: src is [T, H, dv] already;
    ``gate_per_element``: gate is [T, H dv], one per output entry"""
    T = src.shape[0]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=src.device)
    if src.dtype != torch.float32 or src.stride(2) != 1:
        raise BackendError("latent_out_gate: src is f32 with a contiguous last axis")
    lib().latent_out_gate_ex(_ptr(src), C.c_int64(src.stride(0)), C.c_int64(src.stride(1)), _ptr(w_uv), _ptr(gate),
                          C.c_int64(0 if gate is None else (gate.stride(0) if T > 1 else max(heads * (dv if gate_per_element else 1), gate.stride(0)))),
                          C.c_int32(1 if gate_per_element else 0), _ptr(out),
                          C.c_int32(T), C.c_int32(heads), C.c_int32(dv), C.c_int32(rank), C.c_int32(_tag(w_uv.dtype) if w_uv is not None else _tag(out_dtype)),
                          C.c_int32(_tag(out_dtype)), _stream(src.device))
    check("latent_out_gate")
    return out


def linear_grouped(x: torch.Tensor, weight: torch.Tensor, tile_group: torch.Tensor, out: torch.Tensor, tile: int = 128) -> torch.Tensor:
    """out[r, :n] = x[r] . weight[tile_group[r // tile]]^T on the tcgen05 GEMM: x bf16 [m_pad, k] (m_pad % tile == 0, rows may be strided), weight bf16
    [groups, n, k], tile_group i32 [m_pad / tile] (negative = skip the tile), out f32 or bf16 [m_pad, >= n] (rows may be strided).  tile = 128, or
    32 / 64 when groups have few rows (the weights then take the 128-row side of the MMA)."""
    m, k = x.shape
    G, n, _ = weight.shape
    if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1 or m % tile or
            tile_group.dtype != torch.int32 or tile_group.numel() < m // tile or weight.shape[2] != k or out.shape[0] != m or out.shape[1] < n):
        raise BackendError(f"linear_grouped: x {tuple(x.shape)} {x.dtype}, weight {tuple(weight.shape)} {weight.dtype}, out {tuple(out.shape)}")
    lib().linear_grouped(_ptr(x), _ptr(weight), _ptr(out), _ptr(tile_group), C.c_int32(tile), C.c_int32(m), C.c_int32(n), C.c_int32(k), C.c_int32(G), C.c_int64(x.stride(0)),
                         C.c_int64(out.stride(0)), C.c_int32(_tag(out.dtype)), _stream(x.device))
    check("linear_grouped")
    return out


def moe_route(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int, scale: float, score: str = "softmax",
              normalise: bool = True, bias: Optional[torch.Tensor] = None):
    """f32 [T, N] -> (ids i32 [T, top], weights f32 [T, top]); ``score`` softmax over the outputs or a sigmoid per output; ``normalise`` False leaves the
    chosen scores (times scale) as they are; ``bias`` (f32 [N]) is added to the logits first (``correction`` only to the scores the choice is made by)"""
    T, N = logits.shape
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    lib().moe_route_bias(_ptr(logits), C.c_int64(logits.stride(0) if T > 1 else max(N, logits.stride(0))), _ptr(bias), _ptr(correction), _ptr(ids), _ptr(w), C.c_int32(T), C.c_int32(N),
                       C.c_int32(top), C.c_int32(groups), C.c_int32(keep), C.c_float(scale), C.c_int32({"softmax": 0, "sigmoid": 1}[score]), C.c_int32(1 if normalise else 0),
                       _stream(logits.device))
    check("moe_route")
    return ids, w


def moe_gate_up(h: torch.Tensor, w_gate_up: torch.Tensor, ids: torch.Tensor, order: Optional[torch.Tensor] = None, act: str = "silu", limit: float = 0.0,
                pair_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, D], w_gate_up [E, 2 ff, D] of one dtype -> act [T * top, ff] (rows of identity choices are left unwritten); ``order`` i32 [T * top]: the
    pairs in the order the blocks take them (sorted by expert, so that neighbours share weights)"""
    T, D = h.shape
    E, ff2, _ = w_gate_up.shape
    top = ids.shape[1]
    ff = ff2 if act == "relu2" else ff2 // 2            # ungated experts: w_gate_up is the one matrix [E, ff, D] in front of the activation
    out = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
    lib().moe_gate_up_ex(_ptr(h), C.c_int64(h.stride(0) if T > 1 else max(D, h.stride(0))), _ptr(w_gate_up), _ptr(ids), _ptr(order), _ptr(out), C.c_int32(T), C.c_int32(top),
                         C.c_int32(E), C.c_int32(ff), C.c_int32(D), C.c_int32(GLU_ACTS[act]), C.c_float(limit), _ptr(pair_scale), C.c_int32(_tag(h.dtype)), _stream(h.device))
    check("moe_gate_up")
    return out


def moe_down(act: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    """y f32 [rows, D]: y[r] = w_down[e] act[order[r]] for the pairs in the order given (rows of padding or identity choices stay unwritten)"""
    E, D, ff = w_down.shape
    rows = order.shape[0]
    y = torch.empty((rows, D), dtype=torch.float32, device=act.device)
    lib().moe_down(_ptr(act), _ptr(w_down), _ptr(ids), _ptr(order), _ptr(y), C.c_int32(rows), C.c_int32(E), C.c_int32(ff), C.c_int32(D), C.c_int32(_tag(w_down.dtype)),
                   _stream(act.device))
    check("moe_down")
    return y


def moe_sorted_rows(ids: torch.Tensor, num_experts: int, tile: int = 128):
    """pairs (token, choice) sorted by expert into tiles of ``tile`` rows -> (pair_row i32 [T * top] (-1 for identity choices), row_pair i32 [rows] (-1
    = padding), tile_group i32 [rows / tile] (-1 = unused tile)); rows = an upper bound that depends on the counts only through their number"""
    P = ids.numel()
    rows = int(lib().moe_align_rows(C.c_int64(P), C.c_int32(num_experts), C.c_int32(tile)))
    pair_row = torch.empty((P,), dtype=torch.int32, device=ids.device)
    row_pair = torch.empty((rows,), dtype=torch.int32, device=ids.device)
    tile_group = torch.empty((rows // tile,), dtype=torch.int32, device=ids.device)
    lib().moe_align(_ptr(ids), _ptr(pair_row), _ptr(row_pair), _ptr(tile_group), C.c_int32(P), C.c_int32(num_experts), C.c_int32(rows), C.c_int32(tile),
                    _stream(ids.device))
    check("moe_align")
    return pair_row, row_pair, tile_group


def moe_gather_rows(h: torch.Tensor, row_pair: torch.Tensor, top: int) -> torch.Tensor:
    rows, D = row_pair.shape[0], h.shape[1]
    xg = torch.empty((rows, D), dtype=torch.bfloat16, device=h.device)
    lib().moe_gather_rows(_ptr(h), C.c_int64(h.stride(0)), _ptr(row_pair), _ptr(xg), C.c_int32(rows), C.c_int32(top), C.c_int32(D), _stream(h.device))
    check("moe_gather_rows")
    return xg


def silu_mul_packed(gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    rows, two_ff = gate_up.shape
    out = torch.empty((rows, two_ff // 2), dtype=out_dtype, device=gate_up.device)
    lib().silu_mul_packed(_ptr(gate_up), _ptr(out), C.c_int64(rows), C.c_int32(two_ff // 2), C.c_int64(gate_up.stride(0)), C.c_int32(_tag(out_dtype)), _stream(gate_up.device))
    check("silu_mul_packed")
    return out


def moe_combine_rows(y: torch.Tensor, pair_row: torch.Tensor, weights: Optional[torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    """weights None: every choice counts once (the weight was applied elsewhere)"""
    T, D = x.shape
    top = pair_row.numel() // T
    out = torch.empty((T, D), dtype=torch.float32, device=x.device)
    lib().moe_combine_rows(_ptr(y), _ptr(pair_row), _ptr(weights), _ptr(x), C.c_int64(x.stride(0) if T > 1 else max(D, x.stride(0))), _ptr(out), C.c_int32(T),
                           C.c_int32(top), C.c_int32(D), _stream(x.device))
    check("moe_combine_rows")
    return out


def repack_heads(src: torch.Tensor, dst: torch.Tensor, positions: Optional[torch.Tensor] = None, context_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dst[t, h, :] (bf16) = src[t, h, :] (f32 / bf16), each with its own token / head strides; with ``context_lens`` (i32 [T]) also positions + 1"""
    T, H, n = dst.shape
    if dst.dtype != torch.bfloat16 or src.shape != dst.shape or src.stride(2) != 1 or dst.stride(2) != 1:
        raise BackendError("repack_heads: [T, H, n] tensors with a contiguous last axis, bf16 destination")
    lib().repack_heads(_ptr(src), C.c_int32(_tag(src.dtype)), C.c_int64(src.stride(0)), C.c_int64(src.stride(1)), _ptr(dst), C.c_int64(dst.stride(0)),
                       C.c_int64(dst.stride(1)), C.c_int32(T), C.c_int32(H), C.c_int32(n), _ptr(positions), _ptr(context_lens), _stream(dst.device))
    check("repack_heads")
    return dst


def latent_decode_kernel_supported(rank: int, rot_dim: int, block_size: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and bool(lib().mla_decode_kernel_supported(C.c_int32(rank), C.c_int32(rot_dim), C.c_int32(block_size), C.c_int32(DType.BF16)))


def token_tables(batch: StepBatch):
    """-> (tables i32 [T, W], context_lens i32 [T]): every row of the step with its sequence's block table and position + 1"""
    T, W = batch.tokens.shape[0], batch.block_tables.shape[1]
    tables = torch.empty((T, W), dtype=torch.int32, device=batch.tokens.device)
    ctx = torch.empty((T,), dtype=torch.int32, device=batch.tokens.device)
    lib().token_tables(_ptr(batch.block_tables), C.c_int32(W), _ptr(batch.token_seq), _ptr(batch.positions), _ptr(tables), _ptr(ctx), C.c_int32(T),
                       _stream(tables.device))
    check("token_tables")
    return tables, ctx


LATENT_DECODE_WORKSPACE = 1 << 31      # bytes of partials one call of the split-KV kernel may use; steps with more rows go in slabs


def latent_attention_decode(q_abs: torch.Tensor, q_rot: torch.Tensor, c_cache: torch.Tensor, kr_cache: torch.Tensor, tables: torch.Tensor, context_lens: torch.Tensor,
                            sink: Optional[torch.Tensor], scale: float, window: int = 0) -> torch.Tensor:
    """Rows as one-row sequences (``token_tables``) on the split-KV tensor-core kernel of the latent cache (csrc/mla.cu: TMA tiles, 16 heads per MMA,
    runs of 256 keys folded by a merge kernel that also takes the sink): q_abs bf16 [T, H, 512], q_rot bf16 [T, H, 64], bf16 caches of 64-token
    blocks -> bf16 [T, H, 512].  Serves single decoded tokens and rows of prompts alike (each row has its own context length); ``window`` > 0: a row sees
    only the last ``window`` keys of its context."""
    T, H, R = q_abs.shape
    W = tables.shape[1]
    bs = c_cache.shape[1]
    out = torch.empty((T, H, R), dtype=torch.bfloat16, device=q_abs.device)
    L = lib()
    per_row = int(L.mla_paged_decode_workspace_bytes(C.c_int32(1), C.c_int32(H), C.c_int32(W), C.c_int32(bs)))
    slab = max(1, min(T, 65535, LATENT_DECODE_WORKSPACE // per_row))
    need = int(L.mla_paged_decode_workspace_bytes(C.c_int32(slab), C.c_int32(H), C.c_int32(W), C.c_int32(bs)))
    ws = torch.empty(need, dtype=torch.uint8, device=q_abs.device)
    for r0 in range(0, T, slab):
        n = min(slab, T - r0)
        L.mla_paged_attention_window(_ptr(out[r0:]), _ptr(q_abs[r0:]), _ptr(q_rot[r0:]), _ptr(c_cache), _ptr(kr_cache), _ptr(tables[r0:]), _ptr(context_lens[r0:]), _ptr(None),
                                   _ptr(sink), C.c_int32(window), C.c_int32(n), C.c_int32(n), C.c_int32(H), C.c_int32(R), C.c_int32(q_rot.shape[2]), C.c_int32(bs), C.c_int32(W),
                                   C.c_int64(c_cache.shape[0]), C.c_float(scale), C.c_int32(DType.BF16), _ptr(ws), C.c_size_t(need), _stream(q_abs.device))
        check("latent_attention_decode")
    return out


# ---- position embeddings, layer norm, gated residuals, state-space and linear-attention mixers ----------------------------------------------

def embedding_positional(table: torch.Tensor, pos_table: torch.Tensor, batch: StepBatch, scale: float = 1.0) -> torch.Tensor:
    """table[token] * scale + pos_table[position] -> f32 [T, dim]; both tables of one dtype"""
    vocab, dim = table.shape
    if pos_table.dtype != table.dtype or pos_table.shape[1] != dim or not pos_table.is_contiguous():
        raise BackendError(f"embedding_positional: position table {tuple(pos_table.shape)} {pos_table.dtype} beside {tuple(table.shape)} {table.dtype}")
    if batch.max_position >= pos_table.shape[0]:
        raise BackendError(f"position {batch.max_position} is outside the position table ({pos_table.shape[0]} rows)")
    T = batch.tokens.shape[0]
    out = torch.empty((T, dim), dtype=torch.float32, device=table.device)
    lib().embedding_positional(_ptr(table), _ptr(pos_table), _ptr(batch.tokens), _ptr(batch.positions), _ptr(out), C.c_int32(T), C.c_int32(dim), C.c_int32(vocab),
                               C.c_int32(pos_table.shape[0]), C.c_float(scale), C.c_int32(_tag(table.dtype)), _stream(table.device))
    check("embedding_positional")
    return out


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None,
               also_f32: bool = False, pending: Optional[tuple] = None):
    """Layer norm of f32 rows with weight and bias -> rows of ``out_dtype``; ``also_f32`` returns (out, f32 copy) -- the same tensor twice when
    out_dtype is f32.  ``row_index`` (i32) selects the rows.  ``pending`` = (y, gate_logits, gate_bias): the sum x += sigmoid(gate_logits + gate_bias) * y
    (see ``gated_residual_add``) is done first, in the same kernel, and x (contiguous) is updated in place."""
    n = x.shape[-1]
    rows = x.shape[0] if row_index is None else row_index.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or x.stride(-1) != 1:
        raise BackendError("layer_norm: x and weight are f32")
    out = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    out32 = torch.empty((rows, n), dtype=torch.float32, device=x.device) if also_f32 and out_dtype != torch.float32 else None
    if pending is not None:
        y, z, zb = pending
        T = x.shape[0]
        if row_index is not None or not x.is_contiguous() or y.dtype != torch.float32 or y.stride(1) != 1 or (z is not None and z.stride(1) != 1):
            raise BackendError("layer_norm: a pending sum needs the whole contiguous stream and f32 operands")
        pitch = lambda t: t.stride(0) if T > 1 else max(n, t.stride(0))
        lib().gated_add_layer_norm(_ptr(x), _ptr(y), C.c_int64(pitch(y)), _ptr(z), C.c_int64(0 if z is None else pitch(z)), _ptr(zb), _ptr(weight), _ptr(bias), _ptr(out),
                                   _ptr(out32), C.c_int32(T), C.c_int32(n), C.c_float(eps), C.c_int32(_tag(out_dtype)), _stream(x.device))
        check("gated_add_layer_norm")
        return (out, (out if out32 is None else out32)) if also_f32 else out
    lib().layer_norm_ex(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(out32), _ptr(row_index), C.c_int32(rows), C.c_int32(n),
                        C.c_int64(x.stride(0) if x.shape[0] > 1 else n), C.c_float(eps), C.c_int32(_tag(out_dtype)), _stream(x.device))
    check("layer_norm_ex")
    if also_f32:
        return out, (out if out32 is None else out32)
    return out


def gated_residual_add(x: torch.Tensor, y: torch.Tensor, gate_logits: Optional[torch.Tensor], gate_bias: Optional[torch.Tensor]) -> torch.Tensor:
    """x += sigmoid(gate_logits + gate_bias) * y in place on the f32 stream x [T, n] (gate_logits None: x += y)"""
    T, n = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or y.dtype != torch.float32 or y.stride(1) != 1 or (gate_logits is not None and gate_logits.stride(1) != 1):
        raise BackendError("gated_residual_add: f32 tensors, x contiguous")
    pitch = lambda t: t.stride(0) if T > 1 else max(n, t.stride(0))
    lib().gated_residual_add(_ptr(x), _ptr(y), C.c_int64(pitch(y)), _ptr(gate_logits), C.c_int64(0 if gate_logits is None else pitch(gate_logits)), _ptr(gate_bias),
                             C.c_int32(T), C.c_int32(n), _stream(x.device))
    check("gated_residual_add")
    return x


GLU_ACTS = {"silu": 0, "gelu_tanh": 1, "clamped": 2, "relu2": 3}      # "relu2" is ungated: relu(x)^2 from rows of ff entries


def glu_packed(gate_up: torch.Tensor, act: str, out_dtype: torch.dtype, limit: float = 0.0, row_scale: Optional[torch.Tensor] = None,
               scale_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(gate) * up from f32 [rows, ff | ff]; ``row_scale`` (f32) first multiplies both halves of row r by row_scale[scale_index[r]] (or [r])"""
    rows, two_ff = gate_up.shape
    ff = two_ff if act == "relu2" else two_ff // 2
    out = torch.empty((rows, ff), dtype=out_dtype, device=gate_up.device)
    lib().glu_packed(_ptr(gate_up), _ptr(out), C.c_int64(rows), C.c_int32(ff), C.c_int64(gate_up.stride(0) if rows > 1 else two_ff), C.c_int32(GLU_ACTS[act]),
                     C.c_float(limit), _ptr(row_scale), _ptr(scale_index), C.c_int32(_tag(out_dtype)), _stream(gate_up.device))
    check("glu_packed")
    return out


def group_rms_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], groups: int, eps: float, out_dtype: torch.dtype,
                        gate_act: str = "sigmoid") -> torch.Tensor:
    """o f32 [T, n] -> o / rms(o over each of ``groups`` equal runs) * weight * act(gate)"""
    T, n = o.shape
    out = torch.empty((T, n), dtype=out_dtype, device=o.device)
    pitch = lambda t: t.stride(0) if T > 1 else max(n, t.stride(0))
    lib().group_rms_norm_gate(_ptr(o), C.c_int64(pitch(o)), _ptr(weight), _ptr(gate), C.c_int64(0 if gate is None else pitch(gate)), _ptr(out), C.c_int32(T), C.c_int32(n),
                              C.c_int32(groups), C.c_float(eps), C.c_int32({"sigmoid": 0, "silu": 1}[gate_act]), C.c_int32(_tag(out_dtype)), _stream(o.device))
    check("group_rms_norm_gate")
    return out


def head_gate(src: torch.Tensor, gate: torch.Tensor, heads: int, dv: int, out_dtype: torch.dtype) -> torch.Tensor:
    """src [T, H dv] (f32 or bf16, contiguous) times sigmoid(gate[t, h]) (f32 view [T, H], row stride allowed) -> [T, H dv] of ``out_dtype``"""
    T = src.shape[0]
    if not src.is_contiguous() or src.shape[1] != heads * dv or gate.dtype != torch.float32 or gate.stride(1) != 1:
        raise BackendError(f"head_gate: src {tuple(src.shape)}, gate {tuple(gate.shape)} {gate.dtype}")
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=src.device)
    lib().head_gate(_ptr(src), C.c_int32(_tag(src.dtype)), _ptr(gate), C.c_int64(gate.stride(0) if T > 1 else max(heads, gate.stride(0))), _ptr(out), C.c_int32(_tag(out_dtype)),
                    C.c_int32(T), C.c_int32(heads), C.c_int32(dv), _stream(src.device))
    check("head_gate")
    return out


def causal_conv(x: torch.Tensor, taps: torch.Tensor, conv_state: torch.Tensor, batch: StepBatch, out_dtype: torch.dtype = torch.float32,
                in_bias: Optional[torch.Tensor] = None, out_bias: Optional[torch.Tensor] = None, act: str = "none", add_input: bool = False) -> torch.Tensor:
    """Causal convolution over time on each channel of x (f32 view [T, C], row stride allowed): act(taps * inputs + out_bias) (+ the input itself), the
    inputs being x + in_bias; conv_state f32 [slots, max(K - 1, 1), C] is advanced in place."""
    T, Cn = x.shape
    K = taps.shape[1]
    if T > 65535:
        raise BackendError("causal_conv: at most 65535 rows per step")
    if x.dtype != torch.float32 or taps.dtype != torch.float32 or taps.shape[0] != Cn or conv_state.shape[1:] != (max(K - 1, 1), Cn):
        raise BackendError(f"causal_conv: x {tuple(x.shape)}, taps {tuple(taps.shape)}, state {tuple(conv_state.shape)}")
    y = torch.empty((T, Cn), dtype=out_dtype, device=x.device)
    lib().causal_conv_ex(_ptr(x), C.c_int64(x.stride(0) if T > 1 else max(Cn, x.stride(0))), _ptr(in_bias), _ptr(taps), _ptr(out_bias), _ptr(conv_state), _ptr(y),
                         C.c_int64(Cn), _ptr(batch.token_seq), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T),
                         C.c_int32(batch.num_seqs), C.c_int32(1 if batch.pure_decode else 0), C.c_int32(Cn), C.c_int32(K), C.c_int32({"none": 0, "silu": 1}[act]), C.c_int32(1 if add_input else 0),
                         C.c_int32(_tag(out_dtype)), _stream(x.device))
    check("causal_conv_ex")
    return y


def block_diag_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """x f32 [T, blocks * N] (row stride allowed), weight f32 [blocks, M, N] -> f32 [T, blocks * M]: every block of N neighbouring channels times its own matrix"""
    T = x.shape[0]
    nb, M, N = weight.shape
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not weight.is_contiguous() or x.shape[1] != nb * N or x.stride(1) != 1:
        raise BackendError(f"block_diag_linear: x {tuple(x.shape)} {x.dtype}, weight {tuple(weight.shape)} {weight.dtype}")
    out = torch.empty((T, nb * M), dtype=torch.float32, device=x.device)
    lib().block_diag_linear(_ptr(x), C.c_int64(x.stride(0) if T > 1 else max(nb * N, x.stride(0))), _ptr(weight), _ptr(bias), _ptr(out), C.c_int64(nb * M), C.c_int32(T),
                            C.c_int32(nb), C.c_int32(M), C.c_int32(N), _stream(x.device))
    check("block_diag_linear")
    return out


def gated_linear_scan(u: torch.Tensor, gates: torch.Tensor, lam: torch.Tensor, y_pre: torch.Tensor, y_bias: Optional[torch.Tensor], state: torch.Tensor, batch: StepBatch,
                      block_channels: int, decay_scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """u f32 [T, C]; gates f32 [T, blocks, 2 n] (recurrence gate, then input gate, per block); y_pre f32 view [T, C]; state f32 [slots, C] advanced in place
    -> S_t * gelu_tanh(y_pre + y_bias) of ``out_dtype``.  ``gates`` and ``y_pre`` are scratch: steps with portions of prompts overwrite them."""
    T, Cn = u.shape
    out = torch.empty((T, Cn), dtype=out_dtype, device=u.device)
    pitch = lambda t, n: t.stride(0) if T > 1 else max(n, t.stride(0))
    # long portions: room for a (product, partial scan) pair per chunk of 128 rows and channel
    scratch = torch.empty((2 * Cn * (-(-T // 128) + batch.num_seqs),), dtype=torch.float32, device=u.device) if batch.max_rows >= 512 else None
    lib().gated_linear_scan(_ptr(u), C.c_int64(pitch(u, Cn)), _ptr(gates), C.c_int64(pitch(gates, 2 * Cn)), _ptr(lam), _ptr(y_pre), C.c_int64(pitch(y_pre, Cn)), _ptr(y_bias),
                            _ptr(state), _ptr(out), _ptr(scratch), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T), C.c_int32(batch.num_seqs),
                            C.c_int32(batch.max_rows), C.c_int32(Cn), C.c_int32(block_channels), C.c_float(decay_scale), C.c_int32(_tag(out_dtype)), _stream(u.device))
    check("gated_linear_scan")
    return out


CHUNKED_LINEAR_ATTENTION_MIN_ROWS = 64          # steps in which some entry brings at least this many rows take the chunked form
CHUNKED_LINEAR_ATTENTION_SCRATCH = 1 << 30      # bytes of scratch above which a step stays on the token-by-token kernel


def linear_attention(proj: torch.Tensor, off_q: int, off_k: int, off_v: int, state: torch.Tensor, batch: StepBatch, heads: int, dk: int, dv: int, act: str = "none",
                     q_scale: float = 1.0, decay: Optional[torch.Tensor] = None, gates: Optional[dict] = None, kernel: Optional[str] = None) -> torch.Tensor:
    """S <- a S + b k v^T, o = S^T q per head on columns of ``proj`` (f32 [T, ld]); state f32 [slots, H, dv, dk] advanced in place.  ``decay`` f32 [H]: a fixed
    decay per head.  ``gates`` = dict(off_i, off_f, i_bias, f_bias, cap, normaliser, maximum): exponential gating with a running maximum and a normaliser
    (states [slots, H, ceil(dv / 16), dk] and [slots, H, ceil(dv / 16)]).  -> f32 [T, H dv].  Three kernels compute the same rule: "step" (every entry brings
    one token), "token" (token by token in tiles of 16, any step) and "chunked" (over chunks of 64 tokens, all chunks at once, for portions of prompts);
    ``kernel`` forces one, None chooses by the step's shape."""
    T = proj.shape[0]
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=proj.device)
    if (decay is None) == (gates is None):
        raise BackendError("linear_attention: either a fixed decay or exponential gates")
    g = gates or {}
    if kernel is None:
        kernel = "step" if batch.pure_decode else "token"
        if batch.max_rows >= CHUNKED_LINEAR_ATTENTION_MIN_ROWS and -(-batch.max_rows // 64) * batch.num_seqs <= 65535:
            need = int(lib().linear_attention_chunked_scratch(C.c_int32(T), C.c_int32(batch.num_seqs), C.c_int32(heads), C.c_int32(dk), C.c_int32(dv)))
            if need * 4 <= CHUNKED_LINEAR_ATTENTION_SCRATCH:
                kernel = "chunked"
    if kernel == "chunked":
        need = int(lib().linear_attention_chunked_scratch(C.c_int32(T), C.c_int32(batch.num_seqs), C.c_int32(heads), C.c_int32(dk), C.c_int32(dv)))
        scratch = torch.empty((need,), dtype=torch.float32, device=proj.device)
        lib().linear_attention_chunked(_ptr(proj), C.c_int64(proj.stride(0) if T > 1 else proj.shape[1]), C.c_int32(off_q), C.c_int32(off_k), C.c_int32(off_v),
                                       C.c_int32(g.get("off_i", 0)), C.c_int32(g.get("off_f", 0)), _ptr(decay), _ptr(g.get("i_bias")), _ptr(g.get("f_bias")),
                                       C.c_float(g.get("cap", 0.0)), C.c_float(q_scale), C.c_int32({"none": 0, "silu": 1}[act]), C.c_int32(0 if gates is None else 1),
                                       _ptr(state), _ptr(g.get("normaliser")), _ptr(g.get("maximum")), _ptr(out), _ptr(scratch), _ptr(batch.cu_seqlens),
                                       _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T), C.c_int32(batch.num_seqs), C.c_int32(batch.max_rows), C.c_int32(heads),
                                       C.c_int32(dk), C.c_int32(dv), _stream(proj.device))
        check("linear_attention_chunked")
        return out
    if kernel not in ("step", "token"):
        raise BackendError(f"linear_attention: unknown kernel {kernel!r}")
    lib().linear_attention(_ptr(proj), C.c_int64(proj.stride(0) if T > 1 else proj.shape[1]), C.c_int32(off_q), C.c_int32(off_k), C.c_int32(off_v),
                           C.c_int32(g.get("off_i", 0)), C.c_int32(g.get("off_f", 0)), _ptr(decay), _ptr(g.get("i_bias")), _ptr(g.get("f_bias")),
                           C.c_float(g.get("cap", 0.0)), C.c_float(q_scale), C.c_int32({"none": 0, "silu": 1}[act]), C.c_int32(0 if gates is None else 1), _ptr(state),
                           _ptr(g.get("normaliser")), _ptr(g.get("maximum")), _ptr(out), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start),
                           C.c_int32(T), C.c_int32(batch.num_seqs), C.c_int32(1 if kernel == "step" else 0), C.c_int32(heads), C.c_int32(dk), C.c_int32(dv),
                           _stream(proj.device))
    check("linear_attention")
    return out


# ---- per-head q / k preparation, softmax sink, attention without softmax over a window plus pooled blocks, ungated experts, pre-norm sum ------

def add_rms_norm(x: torch.Tensor, pending: Sequence[Optional[torch.Tensor]], weight: Optional[torch.Tensor], eps: float, out_dtype: Optional[torch.dtype] = None,
                 row_index: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The pre-norm step on the f32 stream x [T, n] (contiguous): x += sum of ``pending`` (up to two f32 tensors [T, n], row stride allowed) in place,
    then rms_norm(x) * weight -> [T, n] of ``out_dtype``.  ``weight`` None: the sum alone (returns None).  ``row_index`` (i32 [R]): only those rows are
    summed and normed ([R, n] comes back) and x is left as it is."""
    T, n = x.shape
    ys = [y for y in pending if y is not None]
    if len(ys) > 2 or x.dtype != torch.float32 or not x.is_contiguous() or any(y.dtype != torch.float32 or y.stride(1) != 1 or y.shape != x.shape for y in ys):
        raise BackendError("add_rms_norm: an f32 contiguous stream and at most two f32 addends of its shape")
    if weight is None and (not ys or row_index is not None):
        return None
    ys += [None] * (2 - len(ys))
    rows = T if row_index is None else row_index.shape[0]
    out = None if weight is None else torch.empty((rows, n), dtype=out_dtype, device=x.device)
    pitch = lambda t: 0 if t is None else (t.stride(0) if T > 1 else max(n, t.stride(0)))
    lib().add_rms_norm(_ptr(x), _ptr(ys[0]), C.c_int64(pitch(ys[0])), _ptr(ys[1]), C.c_int64(pitch(ys[1])), _ptr(weight), _ptr(out), _ptr(row_index), C.c_int32(rows),
                       C.c_int32(n), C.c_float(eps), C.c_int32(_tag(out_dtype) if out is not None else DType.F32), _stream(x.device))
    check("add_rms_norm")
    return out


def qk_head_norm_rope_cache(proj: torch.Tensor, bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                            sin: Optional[torch.Tensor], batch: StepBatch, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int,
                            rot_dims: int, eps: float, interleaved: bool = False, norm: str = "none", v_from_k: bool = False,
                            q_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """proj f32 [T, H dk | G dk | G dv] (+ bias f32 of that length): every q and k head normed over dk (``norm`` "before" / "after" the rotation / "none"; weights
    [dk] shared by the heads or None), rotated on its first ``rot_dims`` entries (pairs (i, i + rot_dims/2) or, ``interleaved``, (2i, 2i + 1)); k and v go to the
    paged cache, q [T, H dk] comes back.  ``v_from_k``: no value columns, the value is the key head as projected."""
    T = proj.shape[0]
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise BackendError(f"position {batch.max_position} is outside the rotary table ({cos.shape[0]} rows)")
    q = torch.empty((T, heads * dk), dtype=q_dtype, device=proj.device)
    lib().qk_head_norm_rope_cache(_ptr(proj), C.c_int64(proj.stride(0) if T > 1 else proj.shape[1]), _ptr(bias), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin),
                                  C.c_int32(0 if cos is None else cos.shape[0]), _ptr(batch.positions), _ptr(batch.slot_mapping), _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                  C.c_int32(T), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), C.c_int32(rot_dims if cos is not None else 0),
                                  C.c_int32(1 if interleaved else 0), C.c_int32({"none": 0, "before": 1, "after": 2}[norm]), C.c_int32(1 if v_from_k else 0), C.c_float(eps),
                                  C.c_int32(_tag(k_cache.dtype)), C.c_int32(_tag(q_dtype)), _stream(proj.device))
    check("qk_head_norm_rope_cache")
    return q


def paged_attention_varlen_sink(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: StepBatch, heads: int, kv_heads: int, dk: int, dv: int,
                                block_size: int, scale: float, chunk: int, window: int, sink: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """``paged_attention_varlen`` with exp(sink[h]) (f32 [H]) in the softmax denominator of head h"""
    T = q.shape[0]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=q.device)
    lib().paged_attention_varlen_sink(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]),
                                      _ptr(batch.token_seq), _ptr(batch.positions), _ptr(batch.cu_seqlens), _ptr(batch.cu_seqlens_k), C.c_int32(batch.num_seqs),
                                      C.c_int32(T), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), C.c_int32(block_size), C.c_float(scale),
                                      C.c_int32(chunk), C.c_int32(window), _ptr(sink), C.c_int32(_tag(q.dtype)), C.c_int32(_tag(k_cache.dtype)), C.c_int32(_tag(out_dtype)),
                                      _stream(q.device))
    check("paged_attention_varlen_sink")
    return out


def pooled_entries_per_block(block_size: int, pool: int) -> int:
    """pooled entries a page must hold: the blocks of ``pool`` positions whose last position falls into one page"""
    return -(-block_size // pool)


def pooled_entry_location(block: int, pool: int, block_size: int):
    """(page of the sequence, index inside the page) of the pooled entry of block ``block`` (positions block * pool .. block * pool + pool - 1): the page that
    holds the block's last position, and the block's rank among the blocks that end in that page.  The kernels compute the same."""
    page = (block * pool + pool - 1) // block_size
    return page, block - (page * block_size) // pool


def pooled_cache_update(k_cache: torch.Tensor, v_cache: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatch, pool: int) -> None:
    """After the step's keys and values are in the cache: every row whose position closes a block of ``pool`` positions writes the block's mean key and mean value
    (f32) into the pooled caches [nb, per_block, G, dk | dv]."""
    nb, bs, G, dk = k_cache.shape
    dv = v_cache.shape[3]
    if k_pool.dtype != torch.float32 or v_pool.dtype != torch.float32 or k_pool.shape[0] != nb or k_pool.shape[2:] != (G, dk) or v_pool.shape[2:] != (G, dv):
        raise BackendError(f"pooled_cache_update: pooled caches {tuple(k_pool.shape)} / {tuple(v_pool.shape)} beside {tuple(k_cache.shape)} / {tuple(v_cache.shape)}")
    lib().pooled_cache_update(_ptr(k_cache), _ptr(v_cache), _ptr(k_pool), _ptr(v_pool), _ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]), _ptr(batch.token_seq),
                              _ptr(batch.positions), _ptr(batch.slot_mapping), C.c_int32(batch.tokens.shape[0]), C.c_int32(G), C.c_int32(dk), C.c_int32(dv), C.c_int32(bs),
                              C.c_int32(pool), C.c_int32(k_pool.shape[1]), C.c_int32(_tag(k_cache.dtype)), _stream(k_cache.device))
    check("pooled_cache_update")


def paged_attention_sigmoid_pooled(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                                   batch: StepBatch, head_bias: Optional[torch.Tensor], heads: int, scale: float, window: int, pool: int,
                                   out_dtype: torch.dtype) -> torch.Tensor:
    """out[t, h] = sum_j sigmoid(q . k_j scale + head_bias[h]) v_j over the window's tokens and the pooled entries of the blocks wholly before the window;
    q f32 [T, H dk] -> [T, H dv]; a bf16 q (128-wide heads, 64-token blocks, bf16 cache and output) takes the tensor-core kernel"""
    T = q.shape[0]
    nb, bs, G, dk = k_cache.shape
    dv = v_cache.shape[3]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=q.device)
    lib().paged_attention_sigmoid_pooled(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(k_pool), _ptr(v_pool), _ptr(batch.block_tables),
                                         C.c_int32(batch.block_tables.shape[1]), _ptr(batch.token_seq), _ptr(batch.positions), _ptr(batch.cu_seqlens), _ptr(batch.cu_seqlens_k),
                                         C.c_int32(batch.num_seqs), _ptr(head_bias), C.c_int32(T), C.c_int32(heads),
                                         C.c_int32(G), C.c_int32(dk), C.c_int32(dv), C.c_int32(bs), C.c_float(scale), C.c_int32(window), C.c_int32(pool if k_pool is not None else 0),
                                         C.c_int32(0 if k_pool is None else k_pool.shape[1]), C.c_int32(_tag(q.dtype)), C.c_int32(_tag(k_cache.dtype)), C.c_int32(_tag(out_dtype)),
                                         _stream(q.device))
    check("paged_attention_sigmoid_pooled")
    return out
