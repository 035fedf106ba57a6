"""Synthetic GGUF-LLaMA weights and KV state: no model files, no network.

Weights are random but VALID GGML blocks generated on the device with a seeded torch generator:
Q4_K: 12 scale bytes + 128 nibble bytes uniform, d ~ U(0.5,2)*2^-14, dmin ~ 7.5*U(0.5,2)*2^-14
(zero-mean weights of std ~0.02, so activations stay O(1) through 32 layers); Q6_K: 208 bytes
uniform, d ~ U(0.5,2)*2^-16.  Norm weights ~ U(0.5,1.5), embeddings N(0,1).
Tensor-parallel shards follow the reference: column split dim 0, row split dim 1 by raw blocks
(src/openai/models/layers/quantized_var_builder.rs:234-269).
"""
from __future__ import annotations

import torch

from .backend import GgmlType, QTensor
from .llama import LlamaConfig


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).view(torch.uint8).reshape(*x.shape, 2)


def random_q4k(gen, n: int, k: int, device) -> torch.Tensor:
    nb = n * (k // 256)
    blocks = torch.randint(0, 256, (nb, 144), dtype=torch.uint8, device=device, generator=gen)
    d = (torch.rand(nb, device=device, generator=gen) * 1.5 + 0.5) * 2.0 ** -14
    dmin = (torch.rand(nb, device=device, generator=gen) * 1.5 + 0.5) * 7.5 * 2.0 ** -14
    blocks[:, 0:2] = _f16_bytes(d)
    blocks[:, 2:4] = _f16_bytes(dmin)
    return blocks.reshape(-1)


def random_q6k(gen, n: int, k: int, device) -> torch.Tensor:
    nb = n * (k // 256)
    blocks = torch.randint(0, 256, (nb, 210), dtype=torch.uint8, device=device, generator=gen)
    d = (torch.rand(nb, device=device, generator=gen) * 1.5 + 0.5) * 2.0 ** -16
    blocks[:, 208:210] = _f16_bytes(d)
    return blocks.reshape(-1)


def random_qtensor(gen, ggml_type: int, n: int, k: int, device) -> QTensor:
    fn = {GgmlType.Q4_K: random_q4k, GgmlType.Q6_K: random_q6k}[ggml_type]
    return QTensor(fn(gen, n, k, device), ggml_type, (n, k), allow_cpu=True)


def shard_rows(w: QTensor, rank: int, world: int) -> QTensor:
    """column-parallel: split dim 0 (distributed.rs:767-811)."""
    n, k = w.shape
    be, bb = GgmlType.BLOCK[w.ggml_type]
    rows = w.data.reshape(n, (k // be) * bb)
    nl = n // world
    return QTensor(rows[rank * nl:(rank + 1) * nl].contiguous().reshape(-1), w.ggml_type, (nl, k), allow_cpu=True)


def pad_rows(w: QTensor, n_pad: int) -> QTensor:
    """append all-zero GGML blocks (d = 0 -> weights 0) so that the tensor has n_pad rows."""
    n, k = w.shape
    if n_pad == n:
        return w
    be, bb = GgmlType.BLOCK[w.ggml_type]
    extra = torch.zeros((n_pad - n) * (k // be) * bb, dtype=torch.uint8, device=w.data.device)
    return QTensor(torch.cat([w.data, extra]), w.ggml_type, (n_pad, k), allow_cpu=True)


def shard_cols(w: QTensor, rank: int, world: int) -> QTensor:
    """row-parallel: split dim 1 along whole blocks (raw-byte shard, quantized_var_builder.rs:234-269)."""
    n, k = w.shape
    be, bb = GgmlType.BLOCK[w.ggml_type]
    nbk = k // be
    if nbk % world:
        raise ValueError(f"k={k}: {nbk} blocks per row not divisible by world {world}")
    blocks = w.data.reshape(n, nbk, bb)
    bl = nbk // world
    return QTensor(blocks[:, rank * bl:(rank + 1) * bl].contiguous().reshape(-1), w.ggml_type, (n, k // world), allow_cpu=True)


def make_weights(cfg: LlamaConfig, device="cuda", seed: int = 0, tp_rank: int = 0, tp_world: int = 1,
                 linear_type: int = GgmlType.Q4_K, output_type: int = GgmlType.Q6_K) -> dict:
    """Full (unsharded) tensors are drawn from the seeded stream on every rank, then sharded, so all
    ranks agree on the global model (embedding + norms replicated)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    H, hd = cfg.hidden, cfg.head_dim
    qd, kd = cfg.num_heads * hd, cfg.num_kv_heads * hd
    col = (lambda w: shard_rows(w, tp_rank, tp_world)) if tp_world > 1 else (lambda w: w)
    row = (lambda w: shard_cols(w, tp_rank, tp_world)) if tp_world > 1 else (lambda w: w)
    kcol = col
    if tp_world > 1 and cfg.num_kv_heads < tp_world:
        # kv_head_shard with fewer kv heads than ranks (src/openai/distributed.rs:753-764): every rank holds ONE
        # kv head, replicated over world / kvh consecutive ranks
        if tp_world % cfg.num_kv_heads:
            raise ValueError(f"world {tp_world} not a multiple of {cfg.num_kv_heads} kv heads")
        kcol = lambda w: shard_rows(w, tp_rank * cfg.num_kv_heads // tp_world, cfg.num_kv_heads)
    w = dict(tok_embeddings=torch.randn((cfg.vocab, H), device=device, generator=gen, dtype=torch.float32),
             norm=torch.rand(H, device=device, generator=gen) + 0.5, layers=[])
    for _ in range(cfg.num_layers):
        w["layers"].append(dict(
            attn_norm=torch.rand(H, device=device, generator=gen) + 0.5,
            ffn_norm=torch.rand(H, device=device, generator=gen) + 0.5,
            wq=col(random_qtensor(gen, linear_type, qd, H, device)),
            wk=kcol(random_qtensor(gen, linear_type, kd, H, device)),
            wv=kcol(random_qtensor(gen, linear_type, kd, H, device)),
            wo=row(random_qtensor(gen, linear_type, H, qd, device)),
            w1=col(random_qtensor(gen, linear_type, cfg.ffn, H, device)),
            w2=row(random_qtensor(gen, linear_type, H, cfg.ffn, device)),
            w3=col(random_qtensor(gen, linear_type, cfg.ffn, H, device)),
        ))
    out = random_qtensor(gen, output_type, cfg.vocab, H, device)
    if tp_world > 1:
        # vocab-parallel lm_head: rows padded with zero blocks to pad_vocab_size (distributed.rs:1448-1454), then split
        from .llama import padded_vocab
        out = shard_rows(pad_rows(out, padded_vocab(cfg.vocab, tp_world)), tp_rank, tp_world)
    w["output"] = out
    return w


def make_weights_16bit(cfg: LlamaConfig, device="cuda", seed: int = 0, dtype=torch.bfloat16):
    """Dense 16-bit Llama (BASELINE config 2; the safetensors path of the reference, llama.rs): every linear a [n, k] tensor of
    ``dtype`` ~ N(0, 0.02), lm_head included.  Returns (engine weights, oracle weights); the oracle sees exactly the 16-bit values."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    H, hd = cfg.hidden, cfg.head_dim
    qd, kd = cfg.num_heads * hd, cfg.num_kv_heads * hd
    mk = lambda n, k: (torch.randn((n, k), device=device, generator=gen, dtype=torch.float32) * 0.02).to(dtype).contiguous()
    w = dict(tok_embeddings=torch.randn((cfg.vocab, H), device=device, generator=gen, dtype=torch.float32),
             norm=torch.rand(H, device=device, generator=gen) + 0.5, layers=[])
    for _ in range(cfg.num_layers):
        w["layers"].append(dict(attn_norm=torch.rand(H, device=device, generator=gen) + 0.5, ffn_norm=torch.rand(H, device=device, generator=gen) + 0.5,
                                wq=mk(qd, H), wk=mk(kd, H), wv=mk(kd, H), wo=mk(H, qd), w1=mk(cfg.ffn, H), w2=mk(H, cfg.ffn), w3=mk(cfg.ffn, H)))
    w["output"] = mk(cfg.vocab, H)
    return w


def make_weights_gptq(cfg: LlamaConfig, device="cuda", seed: int = 0, group_size: int = 128, dtype=torch.float16, output_type: int = GgmlType.Q6_K,
                      with_oracle: bool = True):
    """GPTQ symmetric int4 Llama prepared for Marlin like the reference does at load time (linear.rs:300-413: ``gptq_repack`` +
    ``marlin_permute_scales``): BASELINE config 3.  int4 uniform, scales ~ U(0.005, 0.02) of ``dtype``; the lm_head stays a GGML tensor
    (the reference never quantises it to int4).  Returns (engine weights, oracle weights)."""
    import numpy as np
    from .gptq import marlin_permute_scales, marlin_weight_repack
    from .llama import MarlinWeight
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    H, hd = cfg.hidden, cfg.head_dim
    qd, kd = cfg.num_heads * hd, cfg.num_kv_heads * hd

    def mk(n, k):
        q = torch.randint(0, 16, (k, n), device=device, generator=gen, dtype=torch.int32)          # [K, N] like the checkpoint
        packed = torch.zeros((k // 8, n), dtype=torch.int32, device=device)
        for i in range(8):
            packed |= q[i::8] << (4 * i)                                                              # nibble i of word kp = q[8 kp + i]
        ng = 1 if group_size == -1 else k // group_size
        scales = (torch.rand((ng, n), device=device, generator=gen) * 0.015 + 0.005).to(dtype)
        eng = MarlinWeight(marlin_weight_repack(packed, 4, False), marlin_permute_scales(scales, k, n, group_size).contiguous(), group_size)
        orc = ("gptq", packed.cpu().numpy().view(np.uint32), scales.float().cpu().numpy(), group_size) if with_oracle else None
        return eng, orc

    w = dict(tok_embeddings=torch.randn((cfg.vocab, H), device=device, generator=gen, dtype=torch.float32),
             norm=torch.rand(H, device=device, generator=gen) + 0.5, layers=[])
    ow = dict(tok_embeddings=w["tok_embeddings"].cpu().numpy() if with_oracle else None, norm=w["norm"].cpu().numpy(), layers=[])
    for _ in range(cfg.num_layers):
        lw = dict(attn_norm=torch.rand(H, device=device, generator=gen) + 0.5, ffn_norm=torch.rand(H, device=device, generator=gen) + 0.5)
        lo = dict(attn_norm=lw["attn_norm"].cpu().numpy(), ffn_norm=lw["ffn_norm"].cpu().numpy())
        for name, (n, k) in dict(wq=(qd, H), wk=(kd, H), wv=(kd, H), wo=(H, qd), w1=(cfg.ffn, H), w2=(H, cfg.ffn), w3=(cfg.ffn, H)).items():
            lw[name], lo[name] = mk(n, k)
        w["layers"].append(lw); ow["layers"].append(lo)
    out = random_qtensor(gen, output_type, cfg.vocab, H, device)
    w["output"] = out
    ow["output"] = (out.data.cpu().numpy(), out.ggml_type, cfg.vocab, H) if with_oracle else None
    return w, ow


def fill_kv_cache(kv_cache, seed: int = 1, tp_rank: int = 0, tp_world: int = 1, num_kv_heads: int = 0) -> None:
    """KV contents N(0,1) in the cache dtype (bf16, or e4m3 bits for u8 caches).  With tp_world > 1 (and the model's total
    ``num_kv_heads``) every rank draws the FULL layer [nb, bs, kvh, hd] from the same seeded stream and keeps its own kv heads
    (kv_head_shard: a slice, or one replicated head when kvh < world), so the sharded caches are exactly the shards of the
    tp_world = 1 cache -- which is what lets bench.py compare a TP run with a TP = 1 run of the same seed."""
    dev = kv_cache[0][0].device
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    for k, v in kv_cache:
        for t in (k, v):
            if tp_world > 1 and num_kv_heads > 0:
                nb, bs, kl, hd = t.shape
                full = torch.randn((nb, bs, num_kv_heads, hd), device=dev, generator=gen, dtype=torch.float32)
                h0 = tp_rank * kl if num_kv_heads >= tp_world else tp_rank * num_kv_heads // tp_world
                r = full[:, :, h0:h0 + kl, :]
                del full
            else:
                r = torch.randn(t.shape, device=dev, generator=gen, dtype=torch.float32)
            if t.dtype == torch.uint8:
                t.copy_(r.to(torch.float8_e4m3fn).view(torch.uint8))
            else:
                t.copy_(r)
            del r


def random_block_tables(num_seqs: int, blocks_per_seq: int, num_blocks: int, seed: int = 2):
    """Random permutation of physical blocks (non-contiguous pages), seeded; list of lists."""
    import numpy as np
    rng = np.random.default_rng(seed)
    perm = rng.permutation(num_blocks)[: num_seqs * blocks_per_seq]
    return perm.reshape(num_seqs, blocks_per_seq).tolist()


# ---------------------------------------------------------------------------------------------------------------------
# Gobesun: random checkpoints of any shape (tests and bench.py; there is no network for real ones)
# ---------------------------------------------------------------------------------------------------------------------
def gobesun_delta_layer(heads: int, kv_heads: int, dim: int, vdim: int, conv: int = 4, ff: int = 0) -> dict:
    return dict(type="delta", mixer=dict(conv=conv, dim=dim, heads=heads, kv_heads=kv_heads, vdim=vdim), mlp=dict(ff=ff, kind="dense") if ff else None)


def gobesun_attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, chunk: int, rot_dims: int, ff: int = 0, base: float = 10000.0,
                            scaling: dict = None, scale: float = None) -> dict:
    rot = dict(base=base, dims=rot_dims)
    if scaling:
        rot["scaling"] = scaling
    return dict(type="attention", mixer=dict(dim=dim, heads=heads, kv_heads=kv_heads, vdim=vdim, mask=dict(size=chunk), rot=rot,
                                             scale=dim ** -0.5 if scale is None else scale), mlp=dict(ff=ff, kind="dense") if ff else None)


def gobesun_config(width: int, vocab: int, layers: list, loop: dict = None, eps: float = 1e-6, embedding_scale: float = None) -> dict:
    return dict(architecture="Gobesun", embedding=dict(scale=width ** 0.5 if embedding_scale is None else embedding_scale), layers=layers,
                loop=loop or dict(start=0, stop=0, times=1), norm=dict(eps=eps), vocab=vocab, width=width)


def gobesun_weights(cfg: dict, seed: int = 0, device="cpu") -> dict:
    """name -> bf16 tensor, with the magnitudes of a model at initialisation (unit-variance activations through every sublayer)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    out = {}
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std)
    lin = lambda n, k: rnd(n, k, std=k ** -0.5)
    out["embed"] = rnd(cfg["vocab"], D, std=D ** -0.5)
    out["head"] = lin(cfg["vocab"], D)
    out["final.norm"] = rnd(D, std=0.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "norm1"], out[p + "norm1b"] = rnd(D, std=0.2), rnd(D, std=0.2)
        if L["type"] == "delta":
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"], out[p + "mix.g"] = lin(G * dk, D), lin(G * dk, D), lin(H * dv, D), lin(H * dv, D)
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + f"mix.{n}.conv"] = rnd(c, m["conv"], std=0.6) + 0.2
            out[p + "mix.b"], out[p + "mix.a"] = lin(H, D), lin(H, D)
            out[p + "mix.A_log"] = torch.rand(H, generator=g) * 4.0 - 4.0
            out[p + "mix.dt_bias"] = torch.rand(H, generator=g) * 3.0 - 4.0
            out[p + "mix.norm"] = 1.0 + rnd(dv, std=0.2)
            out[p + "mix.o"] = lin(D, H * dv)
        else:
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = lin(H * dk, D), lin(G * dk, D), lin(G * dv, D)
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = 1.2 + rnd(H * dk, std=0.4), 1.2 + rnd(G * dk, std=0.4)
            out[p + "mix.o"] = lin(D, H * dv)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out[p + "norm2"], out[p + "norm2b"] = rnd(D, std=0.2), rnd(D, std=0.2)
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = lin(ff, D), lin(ff, D), lin(D, ff)
    return {k: v.to(torch.bfloat16).to(device) for k, v in out.items()}


# ---------------------------------------------------------------------------------------------------------------------
# Guvusun: random checkpoints of any shape (tests and bench.py)
# ---------------------------------------------------------------------------------------------------------------------
def guvusun_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, experts: int = 0, ff: int = 0, top: int = 1, identity: int = 0,
                  groups: tuple = None, router_scale: float = 1.0, kv_from: int = None, base: float = 10000.0, scaling: dict = None, scale: float = None) -> dict:
    rot = dict(base=base, dims=rot_dim)
    if scaling:
        rot["scaling"] = scaling
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, rot=rot, scale=(dim + rot_dim) ** -0.5 if scale is None else scale)
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    mlp = None
    if experts or identity:
        router = dict(experts=experts, top=top, scale=router_scale)
        if identity:
            router["identity"] = identity
        if groups:
            router["groups"] = dict(count=groups[0], keep=groups[1])
        mlp = dict(kind="moe", expert=dict(ff=ff), router=router)
    return dict(type="latent_attention", mixer=mixer, mlp=mlp)


def guvusun_config(width: int, vocab: int, layers: list, alpha: float = 1.5, bigram: dict = None, side_dim: int = 0, eps: float = 1e-6) -> dict:
    cfg = dict(architecture="Guvusun", layers=layers, norm=dict(eps=eps), postln_alpha=alpha, vocab=vocab, width=width)
    if bigram:
        cfg["embedding"] = dict(bigram=dict(bigram))
    if side_dim:
        cfg["token_side"] = dict(dim=side_dim)
    return cfg


def guvusun_weights(cfg: dict, seed: int = 0, device="cpu") -> dict:
    """name -> bf16 tensor with magnitudes that keep every mechanism visible in the logits: sinks of the order of the scores, corrections large
    enough to change the router's choice (and negative on average), a peaked router."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    out = {}
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std)
    lin = lambda n, k, gain=1.0: rnd(n, k, std=gain * k ** -0.5)
    out["embed"] = rnd(V, D)
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = rnd(bg["buckets"] + 1, D, std=0.7)
    out["embed.norm"] = 1.0 + rnd(D, std=0.2)
    out["head"] = lin(V, D)
    out["final.norm"] = 1.0 + rnd(D, std=0.2)
    side = int((cfg.get("token_side") or {}).get("dim", 0))
    if side:
        out["side.embed"] = rnd(V, side * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out[p + "norm1"] = 1.0 + rnd(D, std=0.2)
        out[p + "mix.q"] = lin(H * (dn + dr), D, 1.5)
        if m.get("kv_from") is None:
            out[p + "mix.dkv"] = lin(R + dr, D)
            out[p + "mix.dkv.norm"] = 1.0 + rnd(R, std=0.3)
        out[p + "mix.uk"], out[p + "mix.uv"] = lin(H * dn, R, 1.5), lin(H * dv, R)
        out[p + "mix.sink"] = rnd(H, std=1.5)
        out[p + "mix.g"] = lin(H, D, 2.0)
        out[p + "mix.o"] = lin(D, H * dv)
        if L.get("mlp"):
            r = L["mlp"]["router"]
            E, I, ff = r["experts"], r.get("identity", 0), L["mlp"]["expert"]["ff"]
            out[p + "norm2"] = 1.0 + rnd(D, std=0.2)
            out[p + "mlp.router"] = lin(E + I, D, 3.0)
            out[p + "mlp.correction"] = rnd(E + I, std=0.15) - 0.4
            for j in range(E):
                out[p + f"mlp.e{j}.gate"], out[p + f"mlp.e{j}.up"], out[p + f"mlp.e{j}.down"] = lin(ff, D), lin(ff, D), lin(D, ff)
        if side:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = lin(side, D), lin(D, side), 0.5 + rnd(D, std=0.1)
    return {k: v.to(torch.bfloat16).to(device) for k, v in out.items()}


# ---------------------------------------------------------------------------------------------------------------------
# Panarax: random checkpoints of any shape (tests and bench.py)
# ---------------------------------------------------------------------------------------------------------------------
def _panarax_mlp(ff: int, experts: int, top: int, limit: float):
    if not ff:
        return None
    if experts:
        return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))
    return dict(kind="dense", ff=ff)


def panarax_rglru_layer(width: int, blocks: int, conv: int = 4, ff: int = 0, experts: int = 0, top: int = 1, limit: float = 7.0) -> dict:
    return dict(type="rglru", mixer=dict(width=width, blocks=blocks, conv=conv), mlp=_panarax_mlp(ff, experts, top, limit))


def panarax_lightning_layer(heads: int, dim: int, vdim: int, decay=None, ff: int = 0, experts: int = 0, top: int = 1, limit: float = 7.0) -> dict:
    decay = list(decay) if decay is not None else [1.0 - 2.0 ** (-1.5 - 6.0 * h / max(heads - 1, 1)) for h in range(heads)]
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay), mlp=_panarax_mlp(ff, experts, top, limit))


def panarax_parallel_layer(heads: int, kv_heads: int, dim: int, vdim: int, m_heads: int, m_dim: int, m_vdim: int, q_temp=(0.2, 32), gate_cap: float = 12.0,
                           scale: float = None, ff: int = 0, experts: int = 0, top: int = 1, limit: float = 7.0) -> dict:
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale)
    if q_temp:
        left["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return dict(type="parallel", mixer=dict(left=left, right=dict(heads=m_heads, dim=m_dim, vdim=m_vdim, gate_cap=gate_cap)), mlp=_panarax_mlp(ff, experts, top, limit))


def panarax_config(width: int, vocab: int, layers: list, max_positions: int = 4096, taps: int = 3, eps: float = 1e-6) -> dict:
    return dict(architecture="Panarax", canon=dict(taps=taps), layers=layers, max_positions=max_positions, norm=dict(eps=eps), vocab=vocab, width=width)


def panarax_weights(cfg: dict, seed: int = 0, device="cpu") -> dict:
    """name -> bf16 tensor, with the magnitudes of a model at initialisation (unit-variance activations through every sublayer)."""
    g = torch.Generator().manual_seed(seed)
    D, K = cfg["width"], cfg["canon"]["taps"]
    out = {}
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std)
    lin = lambda n, k: rnd(n, k, std=k ** -0.5)
    out["embed"] = rnd(cfg["vocab"], D)
    out["pos"] = rnd(cfg["max_positions"], D, std=0.5)
    out["final.norm"], out["final.norm.b"] = 1.0 + rnd(D, std=0.2), rnd(D, std=0.1)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"], out[p + "norm1.b"] = 1.0 + rnd(D, std=0.2), rnd(D, std=0.1)
        out[p + "canon1"] = rnd(D, K, std=0.4)
        out[p + "rg1"], out[p + "rg1.b"] = lin(D, D), rnd(D, std=0.5)
        if L["type"] == "rglru":
            C, nb, taps = m["width"], m["blocks"], m["conv"]
            n = C // nb
            out[p + "mix.y"], out[p + "mix.y.b"], out[p + "mix.x"], out[p + "mix.x.b"] = lin(C, D), rnd(C, std=0.3), lin(C, D), rnd(C, std=0.3)
            out[p + "mix.conv"], out[p + "mix.conv.b"] = rnd(C, taps, std=0.5) + 0.2, rnd(C, std=0.2)
            out[p + "mix.ra"], out[p + "mix.ra.b"] = rnd(nb, n, n, std=n ** -0.5), rnd(nb, n, std=0.5)
            out[p + "mix.ri"], out[p + "mix.ri.b"] = rnd(nb, n, n, std=n ** -0.5), rnd(nb, n, std=0.5)
            out[p + "mix.lam"] = torch.rand(C, generator=g) * 6.0 - 5.0
            out[p + "mix.o"] = lin(D, C)
        elif L["type"] == "lightning":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"], out[p + "mix.g"] = lin(H * dk, D), lin(H * dk, D), lin(H * dv, D), lin(H * dv, D)
            out[p + "mix.norm"] = 1.0 + rnd(H * dv, std=0.2)
            out[p + "mix.o"] = lin(D, H * dv)
        else:
            l, r = m["left"], m["right"]
            H, G, dk, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            q = "mix.left."
            out[p + q + "q"], out[p + q + "k"], out[p + q + "v"], out[p + q + "g"] = lin(H * dk, D) * 2.0, lin(G * dk, D) * 2.0, lin(G * dv, D), lin(H, D)
            out[p + q + "o"], out[p + q + "out"] = lin(D, H * dv), 1.0 + rnd(D, std=0.2)
            H, dk, dv = r["heads"], r["dim"], r["vdim"]
            q = "mix.right."
            out[p + q + "q"], out[p + q + "k"], out[p + q + "v"], out[p + q + "g"] = lin(H * dk, D), lin(H * dk, D), lin(H * dv, D), lin(H * dv, D)
            out[p + q + "i"], out[p + q + "i.b"], out[p + q + "f"], out[p + q + "f.b"] = lin(H, D) * 2.0, rnd(H), lin(H, D) * 2.0, rnd(H) + 3.0
            out[p + q + "norm"], out[p + q + "o"], out[p + q + "out"] = 1.0 + rnd(H * dv, std=0.2), lin(D, H * dv), 1.0 + rnd(D, std=0.2)
        mlp = L.get("mlp")
        if mlp:
            out[p + "norm2"], out[p + "norm2.b"] = 1.0 + rnd(D, std=0.2), rnd(D, std=0.1)
            out[p + "rg2"], out[p + "rg2.b"] = lin(D, D), rnd(D, std=0.5)
            if mlp["kind"] == "dense":
                ff = mlp["ff"]
                out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = lin(ff, D), lin(ff, D), lin(D, ff)
            else:
                ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
                out[p + "mlp.router"] = lin(E, D) * 2.0
                for j in range(E):
                    out[p + f"mlp.e{j}.gate"], out[p + f"mlp.e{j}.up"], out[p + f"mlp.e{j}.down"] = lin(ff, D) * 2.0, lin(ff, D) * 2.0, lin(D, ff)
    return {k: v.to(torch.bfloat16).to(device) for k, v in out.items()}


# ---------------------------------------------------------------------------------------------------------------------
# Dofevik: random checkpoints of any shape (tests and bench.py)
# ---------------------------------------------------------------------------------------------------------------------
def _dofevik_mlp(experts: int, ff: int, top: int, shared_ff: int):
    if not experts:
        return None
    mlp = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared_ff:
        mlp["shared"] = dict(ff=shared_ff)
    return mlp


def dofevik_attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, window: int = 0, rot_dims: int = 0, base: float = 10000.0, factor: float = 0.0,
                            scale: float = None, experts: int = 0, ff: int = 0, top: int = 1, shared_ff: int = 0) -> dict:
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale)
    if window:
        mixer["mask"] = dict(size=window)
    if rot_dims:
        mixer["rot"] = dict(base=base, dims=rot_dims)
        if factor:
            mixer["rot"]["scaling"] = dict(factor=factor)
    return dict(type="attention", mixer=mixer, mlp=_dofevik_mlp(experts, ff, top, shared_ff))


def dofevik_pooled_layer(heads: int, kv_heads: int, dim: int, window: int = 0, pool: int = 0, scale: float = None, experts: int = 0, ff: int = 0, top: int = 1,
                         shared_ff: int = 0) -> dict:
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5 if scale is None else scale)
    if window:
        mixer["mask"] = dict(size=window)
        if pool:
            mixer["mask"]["pool"] = pool
    return dict(type="attention_2", mixer=mixer, mlp=_dofevik_mlp(experts, ff, top, shared_ff))


def dofevik_latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, window: int = 0, base: float = 10000.0, scale: float = None,
                         experts: int = 0, ff: int = 0, top: int = 1, shared_ff: int = 0) -> dict:
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, rot=dict(base=base, dims=rot_dim),
                 scale=(dim + rot_dim) ** -0.5 if scale is None else scale)
    if window:
        mixer["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=mixer, mlp=_dofevik_mlp(experts, ff, top, shared_ff))


def dofevik_config(width: int, vocab: int, layers: list, eps: float = 1e-6) -> dict:
    return dict(architecture="Dofevik", layers=layers, norm=dict(eps=eps), vocab=vocab, width=width)


def dofevik_weights(cfg: dict, seed: int = 0, device="cpu") -> dict:
    """name -> bf16 tensor with magnitudes that keep every mechanism visible in the logits: sinks of the order of the scores, sigmoid biases that leave the
    weights away from 0 and 1, router biases large enough to change the choice, a peaked router, norm numbers away from one."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    out = {}
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std)
    lin = lambda n, k, gain=1.0: rnd(n, k, std=gain * k ** -0.5)
    one = lambda: (0.7 + torch.rand((), generator=g) * 0.8)
    out["embed"], out["head"], out["final.norm"] = rnd(V, D), lin(V, D), one()
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = one()
        H = m["heads"]
        if L["type"] == "attention":
            G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = lin(H * dk, D), lin(G * dk, D), lin(G * dv, D)
            out[p + "mix.q.b"], out[p + "mix.k.b"], out[p + "mix.v.b"] = rnd(H * dk, std=0.3), rnd(G * dk, std=0.3), rnd(G * dv, std=0.3)
            out[p + "mix.sink"] = rnd(H, std=1.5) + 1.0
            out[p + "mix.o"] = lin(D, H * dv)
        elif L["type"] == "attention_2":
            G, dk = m["kv_heads"], m["dim"]
            out[p + "mix.q"], out[p + "mix.k"] = lin(H * dk, D), lin(G * dk, D)
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = 1.0 + rnd(dk, std=0.3), 1.0 + rnd(dk, std=0.3)
            out[p + "mix.pb"] = rnd(H, std=0.8) - 2.0
            out[p + "mix.o"] = lin(D, H * dk, 0.5)
        else:
            dn, dr, dv, R, Rq = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"], out[p + "mix.uq"] = lin(Rq, D), 1.0 + rnd(Rq, std=0.3), lin(H * (dn + dr), Rq, 1.5)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = lin(R + dr, D), 1.0 + rnd(R, std=0.3)
            out[p + "mix.uk"], out[p + "mix.uv"] = lin(H * dn, R, 1.5), lin(H * dv, R)
            out[p + "mix.g"] = lin(H * dv, D, 2.0)
            out[p + "mix.o"] = lin(D, H * dv)
        if L.get("mlp"):
            r, ff = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            out[p + "norm2"] = one()
            out[p + "mlp.router"], out[p + "mlp.router.b"] = lin(r["experts"], D, 3.0), rnd(r["experts"], std=1.0)
            for j in range(r["experts"]):
                out[p + f"mlp.e{j}.up"], out[p + f"mlp.e{j}.down"] = lin(ff, D), lin(D, ff)
            if L["mlp"].get("shared"):
                sf = L["mlp"]["shared"]["ff"]
                out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = lin(sf, D), lin(D, sf)
    return {k: v.to(torch.bfloat16).to(device) for k, v in out.items()}
