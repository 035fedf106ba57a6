"""ctypes loader for libb200backend.so (include/b200_backend.h).  Fails loudly if missing."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libb200backend.so")
_lib = None


class BackendError(RuntimeError):
    """Raised where the reference would ``candle_core::bail!`` or surface a CUDA error."""


def lib_path() -> str:
    return _SO


# every symbol include/b200_backend.h declares (checked by tests/test_abi.py against the header)
SYMBOLS = [
    "b200_abi_version", "b200_last_error", "b200_last_error_message", "b200_device_sm_count", "b200_device_cc",
    "copy_blocks_bf16", "copy_blocks_f16", "copy_blocks_f32", "copy_blocks_u8", "swap_blocks", "flashinfer_csr_to_paged", "reshape_and_cache",
    "paged_attention_decode_workspace_bytes", "paged_attention_decode", "paged_attention_prefill",
    "qmatmul_workspace_bytes", "qmatmul_f32", "qmatmul_f16act", "qmatmul_slab_count", "qmatmul_f16act_slabs", "b200_llama_peer_inbox_bytes", "b200_llama_set_peer_inboxes", "b200_llama_peer_timeouts", "b200_ipc_alloc", "b200_ipc_open", "b200_ipc_close", "b200_ipc_free",
    "dequantize_f32", "linear_16bit", "fp8_matmul", "nvfp4_matmul", "mxfp4_matmul",
    "concat_and_cache_mla", "mla_paged_decode_workspace_bytes", "mla_paged_attention",
    "topk_softmax", "sort_expert_assignments", "moe_gemm_workspace_bytes", "moe_gemm_gguf", "moe_gemm_fp8_workspace_bytes", "moe_gemm_fp8",
    "rms_norm", "fused_rope_f32", "silu_mul", "add_f32", "cast", "embedding_f32", "argmax_f32", "rope_and_cache",
    "b200_llama_create", "b200_llama_destroy", "b200_llama_set_layer", "b200_llama_set_globals", "b200_llama_set_layer_ex", "b200_llama_set_globals_ex",
    "b200_llama_set_kv_cache", "b200_llama_set_comm", "b200_llama_decode", "b200_llama_decode_resident", "b200_llama_linear_chain", "b200_llama_uses_layer_kernel", "b200_llama_mega_trace",
    "b200_llama_logits", "b200_llama_next_tokens", "b200_llama_kernel_launches",
    "b200_llama_read_next_tokens", "b200_llama_read_logits",
    "b200_total_kernel_launches", "b200_allreduce_f32",
    "gptq_repack", "marlin_checkpoint_repack", "awq_repack", "marlin_4bit_f16", "marlin_4bit_bf16", "marlin_awq_4bit_f16", "marlin_awq_4bit_bf16",
    "gemm_half_q_half_alt", "b200_set_scratch",
    "linear_f32out", "rms_norm_ex", "gelu_tanh_mul", "embedding_scaled", "causal_conv_silu", "gated_delta_rule", "gated_delta_rule_tiled", "gated_delta_rule_step", "gated_rms_norm",
    "qk_norm_rope_cache", "paged_attention_varlen", "chunk_decode_view",
    "embedding_bigram", "residual_rms_norm", "gelu_tanh_gather_mul", "latent_kv_rope_cache", "latent_q_absorb", "latent_attention_varlen", "latent_out_gate", "latent_out_gate_ex", "moe_route", "moe_route_bias", "moe_gate_up", "moe_gate_up_ex", "moe_down", "mla_decode_kernel_supported", "mla_paged_attention_sink", "repack_heads", "token_tables", "linear_grouped", "moe_align_rows", "moe_align", "moe_gather_rows", "silu_mul_packed", "moe_combine_rows",
    "embedding_positional", "layer_norm_ex", "gated_residual_add", "gated_add_layer_norm", "glu_packed", "group_rms_norm_gate", "head_gate", "causal_conv_ex", "block_diag_linear", "gated_linear_scan",
    "linear_attention", "linear_attention_chunked", "linear_attention_chunked_scratch", "qk_norm_rope_cache_ex", "moe_route_ex", "moe_gate_up_ex",
    "qk_head_norm_rope_cache", "paged_attention_varlen_sink", "pooled_cache_update", "paged_attention_sigmoid_pooled", "latent_out_gate_ex", "moe_route_bias", "add_rms_norm",
    "mla_paged_attention_window",
]


# what a library built from one source group (build.GROUPS) exports
_COMMON = ["b200_abi_version", "b200_last_error", "b200_last_error_message", "b200_device_sm_count", "b200_device_cc", "b200_total_kernel_launches", "linear_16bit",
           "linear_f32out", "rms_norm_ex", "gelu_tanh_mul", "embedding_scaled", "argmax_f32", "rms_norm", "cast", "embedding_positional", "layer_norm_ex",
           "gated_residual_add", "gated_add_layer_norm", "glu_packed", "group_rms_norm_gate", "head_gate", "add_rms_norm"]
GROUP_SYMBOLS = {
    "ragged": _COMMON + ["causal_conv_silu", "gated_delta_rule", "gated_delta_rule_tiled", "gated_delta_rule_step", "gated_rms_norm", "qk_norm_rope_cache",
                         "paged_attention_varlen", "chunk_decode_view", "paged_attention_decode", "paged_attention_decode_workspace_bytes"],
    "latent": _COMMON + ["embedding_bigram", "residual_rms_norm", "gelu_tanh_gather_mul", "latent_kv_rope_cache", "latent_q_absorb", "latent_attention_varlen",
                         "latent_out_gate", "latent_out_gate_ex", "moe_route", "moe_route_bias", "moe_gate_up", "moe_gate_up_ex", "moe_down", "mla_decode_kernel_supported", "mla_paged_attention_sink",
                         "mla_paged_decode_workspace_bytes", "repack_heads", "token_tables", "linear_grouped", "moe_align_rows", "moe_align", "moe_gather_rows", "silu_mul_packed",
                         "moe_combine_rows"],
    "hybrid": _COMMON + ["causal_conv_ex", "block_diag_linear", "gated_linear_scan", "linear_attention", "linear_attention_chunked", "linear_attention_chunked_scratch", "qk_norm_rope_cache", "qk_norm_rope_cache_ex",
                         "paged_attention_varlen", "chunk_decode_view", "paged_attention_decode", "paged_attention_decode_workspace_bytes", "moe_route", "moe_route_ex", "moe_route_bias", "moe_gate_up", "moe_gate_up_ex", "moe_down", "linear_grouped",
                         "moe_align_rows", "moe_align", "moe_gather_rows", "silu_mul_packed", "moe_combine_rows"],
    "window": _COMMON + ["qk_head_norm_rope_cache", "paged_attention_varlen_sink", "pooled_cache_update", "paged_attention_sigmoid_pooled", "latent_kv_rope_cache",
                         "latent_q_absorb", "latent_attention_varlen", "latent_out_gate_ex", "repack_heads", "token_tables", "mla_decode_kernel_supported",
                         "mla_paged_attention_sink", "mla_paged_attention_window", "mla_paged_decode_workspace_bytes", "moe_route_bias", "moe_gate_up_ex", "moe_down", "linear_grouped", "moe_align_rows",
                         "moe_align", "moe_gather_rows", "moe_combine_rows"],
}
_RESTYPES = {"b200_last_error_message": C.c_char_p, "paged_attention_decode_workspace_bytes": C.c_size_t, "qmatmul_workspace_bytes": C.c_size_t,
             "moe_gemm_workspace_bytes": C.c_size_t, "moe_gemm_fp8_workspace_bytes": C.c_size_t, "mla_paged_decode_workspace_bytes": C.c_size_t,
             "b200_llama_create": C.c_void_p, "b200_llama_peer_inbox_bytes": C.c_size_t, "b200_ipc_alloc": C.c_void_p, "b200_ipc_open": C.c_void_p,
             "b200_llama_logits": C.c_void_p, "b200_llama_next_tokens": C.c_void_p, "b200_llama_kernel_launches": C.c_int64,
             "b200_total_kernel_launches": C.c_longlong, "moe_align_rows": C.c_int64, "linear_attention_chunked_scratch": C.c_int64}


def _open(path: str, symbols) -> C.CDLL:
    L = C.CDLL(path)
    for name in symbols:
        getattr(L, name)            # AttributeError if the library lacks a declared symbol
    for name, rt in _RESTYPES.items():
        if name in symbols:
            getattr(L, name).restype = rt
    return L


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise BackendError(
                f"{_SO} not found: build it with `python candle-vllm_b200/build.py` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        _lib = _open(_SO, SYMBOLS)
    return _lib


def ensure_built(group: str) -> C.CDLL:
    """For programs that start from a source-only checkout: use the full library when it is there, otherwise compile (once) and load the
    library of ``group`` alone -- the kernels one model family needs (``registry.build_group_of`` names the group of a checkpoint)."""
    global _lib
    if _lib is None and not os.path.exists(_SO):
        import importlib.util
        spec = importlib.util.spec_from_file_location("b200_build", os.path.join(_HERE, "build.py"))
        b = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(b)
        path = b.so_path(group)
        if not os.path.exists(path):
            b.build(group=group)
        _lib = _open(path, GROUP_SYMBOLS[group])
    return lib()


def check(what: str = "") -> None:
    """Raise BackendError if the last call on this thread recorded an error."""
    L = lib()
    code = L.b200_last_error()
    if code:
        raise BackendError(f"{what}: {L.b200_last_error_message().decode()} (code {code})")


def device_ok() -> bool:
    """True when the current CUDA device is an sm_100 part."""
    try:
        return lib().b200_device_cc() >= 100
    except Exception:
        return False


def require_device() -> None:
    cc = lib().b200_device_cc()
    if cc < 100:
        raise BackendError(f"no sm_100 (B200) device available (compute capability {cc / 10:.1f}); "
                           "this backend has no CPU or other-GPU fallback")
