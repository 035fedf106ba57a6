// attention_window.cu -- per-head query / key preparation and attention without a softmax over a sliding window plus pooled blocks, for
// ragged steps (portions of prompts beside single decoded tokens in one launch), any sizes, f32 or bf16 cache.
//
//   qk_head_norm_rope_cache  from the packed f32 product [T, H dk | G dk | G dv] of a fused q|k|v projection (plus an optional bias row of
//                            that length): every q and k head is, in this order, RMS-normed (norm_mode 1; weights of length dk shared by
//                            the heads, null = no weight), rotated on its first rot_dims entries by a cos / sin table [max_pos, rot_dims/2]
//                            (frequency i pairs entries (i, i + rot_dims/2), or (2i, 2i + 1) when `interleaved`), and RMS-normed after the
//                            rotation (norm_mode 2).  q goes out in f32 or bf16, k and v into the paged cache at slot_mapping[t]
//                            (K [nb, bs, G, dk], V [nb, bs, G, dv]).  `v_from_k`: the projection has no value columns and the value of a
//                            token is its key head as projected (bias added, before norm and rotation), so dv = dk.
//   pooled_cache_update      the sequence positions are cut into blocks of `pool`; block b (positions b pool .. b pool + pool - 1) is complete
//                            once its last position is in the cache.  A row of the step whose position closes a block averages the block's
//                            `pool` cached keys and values (f32) into the pooled cache KP / VP [nb, per_block, G, dk | dv]: the entry lives
//                            in the page that holds the block's last position, at index b - floor(page bs / pool), so pages that change
//                            hands carry their pooled entries with them and no entry is read before its sequence wrote it.
//   paged_attention_sigmoid_pooled   out[t, h] = sum_j sigmoid(q . k_j scale + head_bias[h]) v_j over the tokens j of the window
//                            (0 <= i - j < window; window 0 = all) and, treated like tokens, the pooled entries of all blocks that end at or
//                            before i - window.  Tokens that left the window whose block is not complete yet are not seen.  One warp per
//                            (token, head): a lane scores one key, then the tile's values are accumulated with lanes across the value
//                            columns; no normalisation over the keys.  With 16-bit q / cache / out, 128-wide heads and 64-token blocks the step runs on the
//                            tensor-core kernel of attention_prefill.cu in its sigmoid form instead.
#include <stdlib.h>

#include "attention.cuh"
#include "common.cuh"

namespace b200 {
namespace {

template <typename TC, typename TQ>
__global__ void __launch_bounds__(256)
qk_head_norm_rope_cache_kernel(const float* __restrict__ proj, int64_t ld, const float* __restrict__ bias, const float* __restrict__ q_w,
                               const float* __restrict__ k_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                               const int32_t* __restrict__ positions, const int64_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                               TC* __restrict__ k_cache, TC* __restrict__ v_cache, int H, int G, int dk, int dv, int rot_dims, int interleaved,
                               int norm_mode, int v_from_k, float eps) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float sm[];                          // [8 warps][dk]
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = sm + warp * dk;
    const float* row = proj + (int64_t)t * ld;
    const int pos = positions[t];
    const int64_t slot = slot_mapping[t];
    const int half = rot_dims >> 1;
    const int units = H + G + (v_from_k ? 0 : G);
    for (int u = warp; u < units; u += 8) {
        if (u >= H + G) {                                  // a value head: bias, then the cache
            const int g = u - H - G;
            const int col0 = (H + G) * dk + g * dv;
            if (slot >= 0)
                for (int i = lane; i < dv; i += 32)
                    v_cache[(slot * G + g) * dv + i] = from_f32<TC>(row[col0 + i] + (bias ? bias[col0 + i] : 0.f));
            continue;
        }
        const bool is_q = u < H;
        const int col0 = u * dk;                           // q heads, then k heads, back to back
        const float* w = is_q ? q_w : k_w;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) {
            const float v = row[col0 + i] + (bias ? bias[col0 + i] : 0.f);
            buf[i] = v;
            ss = fmaf(v, v, ss);
            if (!is_q && v_from_k && slot >= 0) v_cache[(slot * G + (u - H)) * dk + i] = from_f32<TC>(v);
        }
        __syncwarp();
        if (norm_mode == 1) {
            const float sc = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
            for (int i = lane; i < dk; i += 32) buf[i] = buf[i] * sc * (w ? w[i] : 1.0f);
            __syncwarp();
        }
        if (cos_t) {
            for (int f = lane; f < half; f += 32) {
                const int ia = interleaved ? 2 * f : f, ib = interleaved ? 2 * f + 1 : f + half;
                const float c = cos_t[(int64_t)pos * half + f], s = sin_t[(int64_t)pos * half + f];
                const float a = buf[ia], b = buf[ib];
                buf[ia] = a * c - b * s;
                buf[ib] = b * c + a * s;
            }
            __syncwarp();
        }
        float sc = 1.0f;
        if (norm_mode == 2) {
            float s2 = 0.f;
            for (int i = lane; i < dk; i += 32) s2 = fmaf(buf[i], buf[i], s2);
            sc = 1.0f / sqrtf(warp_sum(s2) / (float)dk + eps);
        }
        for (int i = lane; i < dk; i += 32) {
            const float v = norm_mode == 2 ? buf[i] * sc * (w ? w[i] : 1.0f) : buf[i];
            if (is_q) q_out[((int64_t)t * H + u) * dk + i] = from_f32<TQ>(v);
            else if (slot >= 0) k_cache[(slot * G + (u - H)) * dk + i] = from_f32<TC>(v);
        }
        __syncwarp();
    }
}

template <typename TC>
__global__ void __launch_bounds__(256)
pooled_cache_update_kernel(const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, float* __restrict__ kp, float* __restrict__ vp,
                           const int32_t* __restrict__ block_tables, int table_width, const int32_t* __restrict__ token_seq,
                           const int32_t* __restrict__ positions, const int64_t* __restrict__ slot_mapping, int nk, int nv, int block_size, int pool,
                           int per_block) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if ((pos + 1) % pool) return;                          // this row closes no block
    const int64_t slot = slot_mapping[t];
    if (slot < 0) return;
    const int i = blockIdx.y * 256 + threadIdx.x;          // one entry of the key row, then of the value row, per thread
    if (i >= nk + nv) return;
    const int b = (pos + 1) / pool - 1;
    const int page = pos / block_size;
    const int64_t dst = (slot / block_size) * per_block + (b - (int)(((int64_t)page * block_size) / pool));
    const int32_t* table = block_tables + (int64_t)token_seq[t] * table_width;
    const bool is_k = i < nk;
    const TC* src = is_k ? k_cache + i : v_cache + (i - nk);
    const int n = is_k ? nk : nv;
    float a = 0.f;
#pragma unroll 8
    for (int j = pos - pool + 1; j <= pos; ++j) {          // a fixed order: the mean does not depend on how the prompt was cut
        const int64_t phys = (int64_t)table[j / block_size] * block_size + j % block_size;
        a += to_f32<TC>(src[phys * n]);
    }
    a *= 1.0f / (float)pool;
    if (is_k) kp[dst * nk + i] = a;
    else vp[dst * nv + (i - nk)] = a;
}

// The same update with 16-byte reads: a warp per row of the step, a lane per group of 16 / sizeof(TC) neighbouring entries of the key row or the value
// row (nk and nv are multiples of the group).  Every entry is still the sum of its block's positions in ascending order, so both kernels give the same bits.
template <typename TC>
__global__ void __launch_bounds__(256)
pooled_cache_update_vec_kernel(const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, float* __restrict__ kp, float* __restrict__ vp,
                               const int32_t* __restrict__ block_tables, int table_width, const int32_t* __restrict__ token_seq,
                               const int32_t* __restrict__ positions, const int64_t* __restrict__ slot_mapping, int num_tokens, int nk, int nv,
                               int block_size, int pool, int per_block) {
    pdl_wait();
    pdl_trigger();
    constexpr int VEC = 16 / (int)sizeof(TC);
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= num_tokens) return;
    const int pos = positions[t];
    if ((pos + 1) % pool) return;                          // this row closes no block
    const int64_t slot = slot_mapping[t];
    if (slot < 0) return;
    const int i = (blockIdx.y * 32 + (threadIdx.x & 31)) * VEC;        // first entry of the lane's group in [key row | value row]
    if (i >= nk + nv) return;
    const int b = (pos + 1) / pool - 1;
    const int page = pos / block_size;
    const int64_t dst = (slot / block_size) * per_block + (b - (int)(((int64_t)page * block_size) / pool));
    const int32_t* table = block_tables + (int64_t)token_seq[t] * table_width;
    const bool is_k = i < nk;
    const TC* src = is_k ? k_cache + i : v_cache + (i - nk);
    const int n = is_k ? nk : nv;
    float a[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) a[c] = 0.f;
#pragma unroll 8
    for (int j = pos - pool + 1; j <= pos; ++j) {
        const int64_t phys = (int64_t)table[j / block_size] * block_size + j % block_size;
        const uint4 raw = *reinterpret_cast<const uint4*>(src + phys * n);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if constexpr (sizeof(TC) == 4) {
                a[c] += __uint_as_float(w[c]);
            } else {                                       // two bf16 in a word: the low half is the earlier entry
                a[2 * c] += __uint_as_float(w[c] << 16);
                a[2 * c + 1] += __uint_as_float(w[c] & 0xffff0000u);
            }
        }
    }
    const float inv = 1.0f / (float)pool;
    float* out = is_k ? kp + dst * nk + i : vp + dst * nv + (i - nk);
#pragma unroll
    for (int c = 0; c < VEC; c += 4) *reinterpret_cast<float4*>(out + c) = make_float4(a[c] * inv, a[c + 1] * inv, a[c + 2] * inv, a[c + 3] * inv);
}

constexpr int kMaxVPerLane = 8;      // value size <= 256

template <typename TC, typename TOut, typename TQ>
__global__ void __launch_bounds__(128)
paged_attention_sigmoid_pooled_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, const float* __restrict__ kp,
                                      const float* __restrict__ vp, const int32_t* __restrict__ block_tables, int table_width,
                                      const int32_t* __restrict__ token_seq, const int32_t* __restrict__ positions, const float* __restrict__ head_bias,
                                      TOut* __restrict__ out, int64_t items, int H, int G, int dk, int dv, int block_size, float scale, int window, int pool,
                                      int per_block) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float qsm[];                  // [4 warps][dk]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + warp;
    if (item >= items) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const int g = h / (H / G);
    const int pos = positions[t];
    const int32_t* table = block_tables + (int64_t)token_seq[t] * table_width;
    float* qs = qsm + warp * dk;
    for (int i = lane; i < dk; i += 32) qs[i] = to_f32<TQ>(q[((int64_t)t * H + h) * dk + i]) * scale;
    __syncwarp();
    const float hb = head_bias ? head_bias[h] : 0.f;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int seen = (pool > 0 && lo > 0) ? lo / pool : 0;                // blocks whose last position is <= pos - window
    const int total = seen + (pos - lo + 1);
    float acc[kMaxVPerLane];
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) acc[c] = 0.f;
    for (int n0 = 0; n0 < total; n0 += 32) {
        const int n = n0 + lane;
        int64_t ent = 0;
        float p = 0.f;
        if (n < total) {
            float d = 0.f;
            if (n < seen) {
                const int last = n * pool + pool - 1;
                const int page = last / block_size;
                ent = (int64_t)table[page] * per_block + (n - (int)(((int64_t)page * block_size) / pool));
                const float* kr = kp + (ent * G + g) * dk;
                for (int i = 0; i < dk; ++i) d = fmaf(qs[i], kr[i], d);
            } else {
                const int j = lo + (n - seen);
                ent = (int64_t)table[j / block_size] * block_size + j % block_size;
                const TC* kr = k_cache + (ent * G + g) * dk;
                for (int i = 0; i < dk; ++i) d = fmaf(qs[i], to_f32<TC>(kr[i]), d);
            }
            p = 1.0f / (1.0f + expf(-(d + hb)));
        }
        const int cnt = min(32, total - n0);
        for (int kk = 0; kk < cnt; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const int64_t e = __shfl_sync(0xffffffffu, ent, kk);
            if (n0 + kk < seen) {
                const float* vr = vp + (e * G + g) * dv;
#pragma unroll
                for (int c = 0; c < kMaxVPerLane; ++c) {
                    const int i = lane + 32 * c;
                    if (i < dv) acc[c] = fmaf(pk, vr[i], acc[c]);
                }
            } else {
                const TC* vr = v_cache + (e * G + g) * dv;
#pragma unroll
                for (int c = 0; c < kMaxVPerLane; ++c) {
                    const int i = lane + 32 * c;
                    if (i < dv) acc[c] = fmaf(pk, to_f32<TC>(vr[i]), acc[c]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) out[((int64_t)t * H + h) * dv + i] = from_f32<TOut>(acc[c]);
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void qk_head_norm_rope_cache(const float* proj, int64_t ld, const float* bias, const float* q_norm_w, const float* k_norm_w, const float* cos_t,
                             const float* sin_t, int32_t max_pos, const int32_t* positions, const int64_t* slot_mapping, void* q_out, void* key_cache,
                             void* value_cache, int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t dk, int32_t dv, int32_t rot_dims,
                             int32_t interleaved, int32_t norm_mode, int32_t v_from_k, float eps, int32_t cache_dtype, int32_t q_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(proj && positions && slot_mapping && q_out && key_cache && value_cache, kErrBadArg, "qk_head_norm_rope_cache: null pointer");
    B200_REQUIRE((cos_t == nullptr) == (sin_t == nullptr) && norm_mode >= 0 && norm_mode <= 2, kErrBadArg, "qk_head_norm_rope_cache: tables come in pairs, norm_mode 0..2");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && dk > 0 && dv > 0 && rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0 && (!v_from_k || dv == dk) &&
                 ld >= (int64_t)(num_heads + num_kv_heads) * dk + (v_from_k ? 0 : (int64_t)num_kv_heads * dv) && (!cos_t || max_pos > 0) && dk <= 4096,
                 kErrBadArg, "qk_head_norm_rope_cache: bad sizes");
    cudaStream_t st = as_stream(stream);
    const size_t smem = (size_t)8 * dk * sizeof(float);
#define QHP(TC, TQ) do { ensure_dynamic_smem((const void*)qk_head_norm_rope_cache_kernel<TC, TQ>, (int)smem); \
        launch_pdl(qk_head_norm_rope_cache_kernel<TC, TQ>, dim3(num_tokens), dim3(256), smem, st, proj, ld, bias, q_norm_w, k_norm_w, cos_t, sin_t, positions, \
        slot_mapping, (TQ*)q_out, (TC*)key_cache, (TC*)value_cache, num_heads, num_kv_heads, dk, dv, rot_dims, interleaved, norm_mode, v_from_k, eps); } while (0)
    if (cache_dtype == B200_F32 && q_dtype == B200_F32) QHP(float, float);
    else if (cache_dtype == B200_BF16 && q_dtype == B200_F32) QHP(__nv_bfloat16, float);
    else if (cache_dtype == B200_BF16 && q_dtype == B200_BF16) QHP(__nv_bfloat16, __nv_bfloat16);
    else { set_error(kErrUnsupported, "qk_head_norm_rope_cache: cache dtype %d / q dtype %d", cache_dtype, q_dtype); return; }
#undef QHP
    count_launch();
    check_launch("qk_head_norm_rope_cache");
}

void pooled_cache_update(const void* key_cache, const void* value_cache, float* pooled_keys, float* pooled_values, const int32_t* block_tables,
                         int32_t table_width, const int32_t* token_seq, const int32_t* positions, const int64_t* slot_mapping, int32_t num_tokens,
                         int32_t num_kv_heads, int32_t dk, int32_t dv, int32_t block_size, int32_t pool, int32_t per_block, int32_t cache_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(key_cache && value_cache && pooled_keys && pooled_values && block_tables && token_seq && positions && slot_mapping, kErrBadArg,
                 "pooled_cache_update: null pointer");
    B200_REQUIRE(num_kv_heads > 0 && dk > 0 && dv > 0 && block_size > 0 && table_width > 0 && pool > 0 && per_block >= (block_size + pool - 1) / pool, kErrBadArg,
                 "pooled_cache_update: bad sizes (a page needs ceil(block_size / pool) pooled entries)");
    cudaStream_t st = as_stream(stream);
    const int nk = num_kv_heads * dk, nv = num_kv_heads * dv;
    B200_REQUIRE((nk + nv + 255) / 256 <= 65535, kErrUnsupported, "pooled_cache_update: rows of %d entries", nk + nv);
    const int vec = cache_dtype == B200_F32 ? 4 : 8;      // entries in 16 bytes
    const bool wide = nk % vec == 0 && nv % vec == 0 && ((uintptr_t)key_cache | (uintptr_t)value_cache | (uintptr_t)pooled_keys | (uintptr_t)pooled_values) % 16 == 0;
    const dim3 grid((unsigned)num_tokens, (unsigned)((nk + nv + 255) / 256));
    const dim3 grid_v((unsigned)((num_tokens + 7) / 8), (unsigned)(((nk + nv) / vec + 31) / 32));
    if (cache_dtype == B200_F32 && wide)
        launch_pdl(pooled_cache_update_vec_kernel<float>, grid_v, dim3(256), 0, st, (const float*)key_cache, (const float*)value_cache, pooled_keys, pooled_values,
                   block_tables, table_width, token_seq, positions, slot_mapping, num_tokens, nk, nv, block_size, pool, per_block);
    else if (cache_dtype == B200_BF16 && wide)
        launch_pdl(pooled_cache_update_vec_kernel<__nv_bfloat16>, grid_v, dim3(256), 0, st, (const __nv_bfloat16*)key_cache, (const __nv_bfloat16*)value_cache,
                   pooled_keys, pooled_values, block_tables, table_width, token_seq, positions, slot_mapping, num_tokens, nk, nv, block_size, pool, per_block);
    else if (cache_dtype == B200_F32)
        launch_pdl(pooled_cache_update_kernel<float>, grid, dim3(256), 0, st, (const float*)key_cache, (const float*)value_cache, pooled_keys, pooled_values,
                   block_tables, table_width, token_seq, positions, slot_mapping, nk, nv, block_size, pool, per_block);
    else if (cache_dtype == B200_BF16)
        launch_pdl(pooled_cache_update_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (const __nv_bfloat16*)key_cache, (const __nv_bfloat16*)value_cache,
                   pooled_keys, pooled_values, block_tables, table_width, token_seq, positions, slot_mapping, nk, nv, block_size, pool, per_block);
    else { set_error(kErrUnsupported, "pooled_cache_update: cache dtype %d", cache_dtype); return; }
    count_launch();
    check_launch("pooled_cache_update");
}

void paged_attention_sigmoid_pooled(void* out, const void* q, const void* key_cache, const void* value_cache, const float* pooled_keys, const float* pooled_values,
                                    const int32_t* block_tables, int32_t table_width, const int32_t* token_seq, const int32_t* positions, const int32_t* cu_seqlens_q,
                                    const int32_t* cu_seqlens_k, int32_t num_seqs, const float* head_bias, int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads,
                                    int32_t dk, int32_t dv, int32_t block_size, float scale, int32_t window, int32_t pool, int32_t per_block, int32_t q_dtype,
                                    int32_t cache_dtype, int32_t out_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(out && q && key_cache && value_cache && block_tables && token_seq && positions, kErrBadArg, "paged_attention_sigmoid_pooled: null pointer");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0 && block_size > 0 && table_width > 0 && window >= 0 &&
                 pool >= 0 && (pool == 0 || (pooled_keys && pooled_values && per_block >= (block_size + pool - 1) / pool)), kErrBadArg,
                 "paged_attention_sigmoid_pooled: bad sizes");
    cudaStream_t st = as_stream(stream);
    // 16-bit q / cache / out with 128-wide heads and 64-token blocks: the tensor-core kernel of the softmax models in its sigmoid form (attention_prefill.cu);
    // pooled entries are gathered into tiles of 64 and take the same MMA path as a page
    static const bool no_tc = [] { const char* e = getenv("B200_VARLEN_SIMT"); return e && atoi(e) != 0; }();
    if (!no_tc && q_dtype == B200_BF16 && out_dtype == B200_BF16 && dk == dv && cu_seqlens_q && cu_seqlens_k && num_seqs > 0 &&
        paged_attention_prefill_tc_supported(dk, block_size, B200_BF16, cache_dtype, B200_KV_FLASH, 0.f, 1, q, key_cache, value_cache)) {
        PrefillExtras extras;
        extras.sigmoid = true; extras.head_bias = head_bias;
        extras.pooled_keys = pooled_keys; extras.pooled_values = pooled_values; extras.pool = pool; extras.per_block = per_block;
        paged_attention_prefill_tc(out, q, key_cache, value_cache, (const uint32_t*)block_tables, (const uint32_t*)cu_seqlens_q, (const uint32_t*)cu_seqlens_k,
                                   num_seqs, num_tokens, num_heads, num_kv_heads, table_width, (int64_t)1 << 22, scale, window, B200_BF16, st, 0, &extras);
        return;
    }
    B200_REQUIRE(dv <= 32 * kMaxVPerLane && dk <= 2048, kErrUnsupported, "paged_attention_sigmoid_pooled: value size %d > %d or key size %d > 2048", dv,
                 32 * kMaxVPerLane, dk);
    const int64_t items = (int64_t)num_tokens * num_heads;
    const unsigned grid = (unsigned)((items + 3) / 4);
    const size_t smem = (size_t)4 * dk * sizeof(float);
#define PSP(TC, TO, TQ) launch_pdl(paged_attention_sigmoid_pooled_kernel<TC, TO, TQ>, dim3(grid), dim3(128), smem, st, (const TQ*)q, (const TC*)key_cache, \
        (const TC*)value_cache, pooled_keys, pooled_values, block_tables, table_width, token_seq, positions, head_bias, (TO*)out, items, num_heads, num_kv_heads, \
        dk, dv, block_size, scale, window, pool, per_block)
    if (cache_dtype == B200_F32 && out_dtype == B200_F32 && q_dtype == B200_F32) PSP(float, float, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_BF16 && q_dtype == B200_F32) PSP(__nv_bfloat16, __nv_bfloat16, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_F32 && q_dtype == B200_F32) PSP(__nv_bfloat16, float, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_BF16 && q_dtype == B200_BF16) PSP(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else { set_error(kErrUnsupported, "paged_attention_sigmoid_pooled: cache dtype %d / out dtype %d / q dtype %d", cache_dtype, out_dtype, q_dtype); return; }
#undef PSP
    count_launch();
    check_launch("paged_attention_sigmoid_pooled");
}

}  // extern "C"
