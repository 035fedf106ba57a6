"""KV-cache allocator and block-op entry points: mirror of ``CacheEngine``
(src/scheduler/cache_engine.rs).

  allocate_kv_cache   cache_engine.rs:122-294   (flash layout by default, legacy paged optional)
  shapes              cache_engine.rs:298-341
  swap_in / swap_out  cache_engine.rs:345-385   -> swap_blocks (K5), K then V of every layer
  copy                cache_engine.rs:387-399   -> copy_blocks (K4)

Unlike the reference the block ops must be applied on EVERY tensor-parallel rank:
each rank owns its kv-head shard of every block.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ._lib import BackendError
from .backend import KvLayout, copy_blocks, swap_blocks


@dataclass
class CacheConfig:
    block_size: int
    num_gpu_blocks: int
    num_cpu_blocks: int = 0
    fully_init: bool = True
    kvcache_dtype: str = "auto"        # "auto" (model dtype) | "fp8" (e4m3 stored as u8, main.rs:263-267)


def kv_head_shard(num_kv_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """(src/openai/distributed.rs:725-765) -> (local kv heads, first global head)."""
    if world <= 1:
        return num_kv_heads, 0
    if num_kv_heads >= world:
        if num_kv_heads % world:
            raise BackendError(f"num_key_value_heads {num_kv_heads} not divisible by world {world}")
        n = num_kv_heads // world
        return n, rank * n
    if world % num_kv_heads:
        raise BackendError(f"world {world} not divisible by num_key_value_heads {num_kv_heads}")
    return 1, rank // (world // num_kv_heads)      # replicate each head over world/kvh ranks


def allocate_mla_cache(num_layers: int, num_blocks: int, block_size: int, kv_lora_rank: int, qk_rope_head_dim: int,
                       dtype: torch.dtype = torch.bfloat16, device="cuda") -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """MLA models (cache_engine.rs:172-185): per layer the compressed KV ``[nb, bs, 1, kv_lora_rank]`` and the rope keys
    ``[nb, bs, 1, qk_rope_head_dim]`` -- what ``mla.concat_and_cache_mla`` writes and ``mla.mla_paged_decode`` reads."""
    return [(torch.zeros((num_blocks, block_size, 1, kv_lora_rank), dtype=dtype, device=device),
             torch.zeros((num_blocks, block_size, 1, qk_rope_head_dim), dtype=dtype, device=device)) for _ in range(num_layers)]


def turboquant_layer_shapes(mode: str, num_blocks: int, block_size: int, num_kv_heads: int, head_dim: int, num_shards: int = 1) -> Dict[str, tuple]:
    """STORAGE shapes of the TurboQuant KV cache (cache_engine.rs:401-482); ``mode`` in {"turbo8", "turbo4", "turbo3"}.  Only the
    allocation is visible in the reference -- the transform (WHT + absmax quantisation) lives in attention-rs -- so this backend
    offers the shapes for sizing and block bookkeeping, and no kernels."""
    if mode not in ("turbo8", "turbo4", "turbo3"):
        raise BackendError(f"unknown TurboQuant mode {mode!r}")
    kvh = max(num_kv_heads // max(num_shards, 1), 1)
    shapes = {"v_absmax": (num_blocks, block_size, kvh), "v_quant": (num_blocks, block_size, kvh, head_dim // 2)}
    if mode == "turbo4":
        shapes.update(k_absmax=(num_blocks, block_size, kvh), k_quant=(num_blocks, block_size, kvh, head_dim // 2))
    elif mode == "turbo3":
        shapes.update(k_absmax=(num_blocks, block_size, kvh), k_quant=(num_blocks, block_size, kvh, (head_dim * 3 + 7) // 8))
    return shapes            # turbo8: K stays in the regular FP8 cache (no k_* tensors), as upstream


class CacheEngine:
    layer_shapes = None          # per-layer (kv heads, key size, value size); None = uniform layers
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, cache_config: CacheConfig,
                 dtype: torch.dtype = torch.bfloat16, device="cuda", num_shards: int = 1,
                 layout: int = KvLayout.FLASH, pin_cpu: bool = True,
                 layer_shapes: Optional[Sequence[Tuple[int, int, int]]] = None, pool_shapes: Optional[Sequence[Optional[Tuple[int, int, int, int]]]] = None):
        """``layer_shapes`` (optional): one (kv heads, key size, value size) per cached layer for models whose layers differ or whose
        keys and values have different sizes; flash layout only.  Without it every layer is (num_kv_heads, head_dim, head_dim).
        ``pool_shapes`` (optional): per cached layer None or (entries per block, kv heads, key size, value size): the layer also keeps f32 pooled
        keys / values [num_blocks, entries, kv heads, size] page by page (means over runs of positions that end in the page), and its cache entry
        is the 4-tuple (K, V, pooled K, pooled V).  Pooled tensors travel with their blocks in swaps and copies."""
        self.num_layers = num_layers
        self.head_dim = head_dim
        self.num_kv_heads = max(num_kv_heads // max(num_shards, 1), 1)       # cache_engine.rs:306,320,335
        self.layer_shapes = None if layer_shapes is None else [tuple(int(v) for v in s) for s in layer_shapes]
        if self.layer_shapes is not None and (len(self.layer_shapes) != num_layers or layout != KvLayout.FLASH):
            raise BackendError("CacheEngine: layer_shapes needs one entry per layer and the flash layout")
        self.pool_shapes = None if pool_shapes is None else [None if p is None else tuple(int(v) for v in p) for p in pool_shapes]
        if self.pool_shapes is not None and len(self.pool_shapes) != num_layers:
            raise BackendError("CacheEngine: pool_shapes needs one entry (or None) per layer")
        self.cfg = cache_config
        self.block_size = cache_config.block_size
        self.layout = layout
        self.device = torch.device(device)
        self.dtype = torch.uint8 if cache_config.kvcache_dtype == "fp8" else dtype
        self.cpu_swap_enabled = cache_config.num_cpu_blocks > 0
        self.gpu_cache = self._allocate(cache_config.num_gpu_blocks, self.device, False)
        self.cpu_cache = self._allocate(cache_config.num_cpu_blocks, torch.device("cpu"), pin_cpu) if self.cpu_swap_enabled else []

    # shapes: cache_engine.rs:298-341
    def key_block_shape(self, layer: int = 0):
        if self.layer_shapes is not None:
            g, dk, _ = self.layer_shapes[layer]
            return (self.block_size, g, dk)
        if self.layout == KvLayout.FLASH:
            return (self.block_size, self.num_kv_heads, self.head_dim)
        x = 16 // torch.empty((), dtype=self.dtype).element_size()
        return (self.num_kv_heads, self.head_dim // x, self.block_size, x)

    def value_block_shape(self, layer: int = 0):
        if self.layer_shapes is not None:
            g, _, dv = self.layer_shapes[layer]
            return (self.block_size, g, dv)
        if self.layout == KvLayout.FLASH:
            return (self.block_size, self.num_kv_heads, self.head_dim)
        return (self.num_kv_heads, self.head_dim, self.block_size)

    def _allocate(self, num_blocks: int, device, pin: bool) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        out = []
        for i in range(self.num_layers):
            kw = dict(dtype=self.dtype, device=device)
            if device.type == "cpu" and pin and torch.cuda.is_available():
                kw["pin_memory"] = True
            k = torch.zeros((num_blocks,) + self.key_block_shape(i), **kw)
            v = torch.zeros((num_blocks,) + self.value_block_shape(i), **kw)
            pool = self.pool_shapes[i] if self.pool_shapes is not None else None
            if pool is not None:
                n, g, dk, dv = pool
                kw["dtype"] = torch.float32
                out.append((k, v, torch.zeros((num_blocks, n, g, dk), **kw), torch.zeros((num_blocks, n, g, dv), **kw)))
            else:
                out.append((k, v))
        return out

    def get_kv_cache(self):
        return self.gpu_cache

    def bytes_per_block(self) -> int:
        return sum(t[0].numel() * t.element_size() for layer in self.gpu_cache for t in layer)

    def swap_in(self, src_to_dst: Dict[int, int]) -> int:
        if not self.cpu_swap_enabled:
            raise BackendError("CPU KV cache swap-in is disabled for this device")
        nbytes = 0
        for src_layer, dst_layer in zip(self.cpu_cache, self.gpu_cache):
            for s, d in zip(src_layer, dst_layer):
                swap_blocks(s, d, src_to_dst)
                nbytes += s[0].numel() * s.element_size() * len(src_to_dst)
        return nbytes

    def swap_out(self, src_to_dst: Dict[int, int]) -> int:
        if not self.cpu_swap_enabled:
            raise BackendError("CPU KV cache swap-out is disabled for this device")
        nbytes = 0
        for src_layer, dst_layer in zip(self.gpu_cache, self.cpu_cache):
            for s, d in zip(src_layer, dst_layer):
                swap_blocks(s, d, src_to_dst)
                nbytes += s[0].numel() * s.element_size() * len(src_to_dst)
        return nbytes

    def copy(self, src_to_dst: Dict[int, List[int]]) -> None:
        copy_blocks([layer[0] for layer in self.gpu_cache], [layer[1] for layer in self.gpu_cache], src_to_dst)
        for layer in self.gpu_cache:                 # pooled entries follow their page, layer by layer (their sizes differ from layer to layer)
            if len(layer) == 4:
                copy_blocks([layer[2]], [layer[3]], src_to_dst)
