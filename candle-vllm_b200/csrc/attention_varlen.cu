// attention_varlen.cu -- softmax attention over the paged cache for ragged steps (portions of prompts beside single decoded
// tokens in one launch), with separate key and value sizes, an f32 or bf16 cache, and a visibility rule per query:
//     key j is seen by the query at position i  iff  j <= i, floor(j / chunk) == floor(i / chunk) when chunk > 0, and
//     i - j < window when window > 0.
// Chunks and windows are counted in sequence positions, so the result does not depend on where a prompt was cut.
//
//   qk_norm_rope_cache      from the packed f32 product [T, H dk | G dk | G dv] of a fused q|k|v projection: RMS norm over the WHOLE
//                           q row and the whole k row (weights of that length; optional), rotation of the first rot_dims entries
//                           of every head, entry i paired with i + rot_dims/2, by a cos/sin table [max_pos, rot_dims/2] that
//                           already carries any frequency scaling and magnitude factor (optional), q written out in f32, k and v
//                           written into the paged cache at slot_mapping[t] (K [nb, bs, G, dk], V [nb, bs, G, dv]).  The _ex form
//                           adds a query temperature (q times 1 + coef ln(floor((p + 1) / every) + 1) at position p) and values
//                           stored at unit root mean square per head.
//   paged_attention_varlen  one warp per (token, head); keys in tiles of 32 (a lane scores one key, the tile's values are then
//                           accumulated with lanes across the value columns), online softmax in f32.  The _sink form puts exp(sink[h]) into
//                           the denominator of head h (a key without a value; its score is not scaled).
#include <stdlib.h>

#include "attention.cuh"
#include "common.cuh"

namespace b200 {
namespace {

template <typename TC, typename TQ>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_kernel(const float* __restrict__ qkv, int64_t ld, const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int32_t* __restrict__ positions,
                          const int64_t* __restrict__ slot_mapping, TQ* __restrict__ q_out, TC* __restrict__ k_cache,
                          TC* __restrict__ v_cache, int H, int G, int dk, int dv, int rot_dims, float eps, float q_temp_coef, int q_temp_every,
                          int v_unit_rms) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[2][8];
    const int t = blockIdx.x;
    const float* row = qkv + (int64_t)t * ld;
    const int nq = H * dk, nk = G * dk, nv = G * dv;
    float sq = 0.f, sk = 0.f;
    if (q_norm_w) {
        for (int i = threadIdx.x; i < nq; i += 256) { const float v = row[i]; sq = fmaf(v, v, sq); }
        for (int i = threadIdx.x; i < nk; i += 256) { const float v = row[nq + i]; sk = fmaf(v, v, sk); }
        sq = warp_sum(sq); sk = warp_sum(sk);
        if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = sq; red[1][threadIdx.x >> 5] = sk; }
        __syncthreads();
        sq = 0.f; sk = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { sq += red[0][i]; sk += red[1][i]; }
    }
    const int pos = positions[t];
    // query temperature: the whole query grows with the logarithm of the number of full runs of `every` places before it
    const float q_temp = q_temp_every > 0 ? 1.0f + q_temp_coef * logf((float)((pos + 1) / q_temp_every) + 1.0f) : 1.0f;
    const float qsc = (q_norm_w ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.0f) * q_temp;
    const float ksc = k_norm_w ? 1.0f / sqrtf(sk / (float)nk + eps) : 1.0f;
    const int half = rot_dims >> 1;
    const int64_t slot = slot_mapping[t];
    for (int e = threadIdx.x; e < nq + nk; e += 256) {
        const bool is_q = e < nq;
        const int idx = is_q ? e : e - nq;                     // index inside the q (or k) row
        const float* w = is_q ? q_norm_w : k_norm_w;
        const float sc = is_q ? qsc : ksc;
        const int d = idx % dk;
        float val = row[e] * sc * (w ? w[idx] : 1.0f);
        if (cos_t && d < rot_dims) {
            const int pd = d < half ? d + half : d - half;     // partner inside the head
            const int pidx = idx - d + pd;
            const float other = row[e - d + pd] * sc * (w ? w[pidx] : 1.0f);
            const float c = cos_t[(int64_t)pos * half + (d < half ? d : d - half)];
            const float s = sin_t[(int64_t)pos * half + (d < half ? d : d - half)];
            val = d < half ? val * c - other * s : val * c + other * s;
        }
        if (is_q) q_out[(int64_t)t * nq + idx] = from_f32<TQ>(val);
        else if (slot >= 0) k_cache[slot * nk + idx] = from_f32<TC>(val);
    }
    if (slot < 0) return;
    if (v_unit_rms) {
        // every value head is stored at unit root mean square: a warp takes whole heads
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int g = warp; g < G; g += 8) {
            const float* vr = row + nq + nk + g * dv;
            float ss = 0.f;
            for (int i = lane; i < dv; i += 32) { const float v = vr[i]; ss = fmaf(v, v, ss); }
            const float sc = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
            for (int i = lane; i < dv; i += 32) v_cache[slot * nv + g * dv + i] = from_f32<TC>(vr[i] * sc);
        }
        return;
    }
    for (int i = threadIdx.x; i < nv; i += 256) v_cache[slot * nv + i] = from_f32<TC>(row[nq + nk + i]);
}

// Steps made of single tokens: a query at position i sees the keys chunk_start .. i with chunk_start = floor(i / chunk) * chunk.  When
// chunks start on block borders that is an ordinary decode over a context of i - chunk_start + 1 keys whose block table is the
// sequence's table moved left by chunk_start / block_size blocks -- so the split-KV decode kernel of the other models serves it.
__global__ void chunk_decode_view_kernel(const int32_t* __restrict__ block_tables, int table_width, const int32_t* __restrict__ positions,
                                         uint32_t* __restrict__ out_tables, uint32_t* __restrict__ out_ctx, int num_seqs, int out_width,
                                         int block_size, int chunk) {
    pdl_wait();
    pdl_trigger();
    const int b = blockIdx.x;
    const int pos = positions[b];
    const int cs = (pos / chunk) * chunk;
    const int first = cs / block_size;
    if (threadIdx.x == 0) out_ctx[b] = (uint32_t)(pos - cs + 1);
    for (int j = threadIdx.x; j < out_width; j += blockDim.x)
        out_tables[(int64_t)b * out_width + j] = first + j < table_width ? (uint32_t)block_tables[(int64_t)b * table_width + first + j] : 0u;
}

constexpr int kMaxVPerLane = 8;      // value size <= 256

template <typename TC, typename TOut, typename TQ>
__global__ void __launch_bounds__(128)
paged_attention_varlen_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                              const int32_t* __restrict__ block_tables, int table_width, const int32_t* __restrict__ token_seq,
                              const int32_t* __restrict__ positions, TOut* __restrict__ out, int64_t items, int H, int G, int dk, int dv,
                              int block_size, float scale, int chunk, int window, const float* __restrict__ sink) {
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
    int lo = 0;
    if (chunk > 0) lo = (pos / chunk) * chunk;
    if (window > 0 && pos - window + 1 > lo) lo = pos - window + 1;
    // a sink is a key without a value whose score is sink[h] as it stands: the running maximum and sum start from it
    float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f;
    float acc[kMaxVPerLane];
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) acc[c] = 0.f;
    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= pos;
        int64_t phys = 0;
        float s = -INFINITY;
        if (valid) {
            phys = (int64_t)table[j / block_size] * block_size + j % block_size;
            const TC* kr = k_cache + (phys * G + g) * dk;
            float d = 0.f;
            for (int i = 0; i < dk; ++i) d = fmaf(qs[i], to_f32<TC>(kr[i]), d);
            s = d;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);          // m = -inf on the first tile: exp(-inf) = 0, acc and l are 0 anyway
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < kMaxVPerLane; ++c) acc[c] *= corr;
        const int cnt = min(32, pos - j0 + 1);
        for (int kk = 0; kk < cnt; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const int64_t ph = __shfl_sync(0xffffffffu, phys, kk);
            const TC* vr = v_cache + (ph * G + g) * dv;
#pragma unroll
            for (int c = 0; c < kMaxVPerLane; ++c) {
                const int i = lane + 32 * c;
                if (i < dv) acc[c] = fmaf(pk, to_f32<TC>(vr[i]), acc[c]);
            }
        }
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) out[((int64_t)t * H + h) * dv + i] = from_f32<TOut>(acc[c] * inv);
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void qk_norm_rope_cache(const float* qkv, int64_t ld, const float* q_norm_w, const float* k_norm_w, const float* cos_t, const float* sin_t,
                        int32_t max_pos, const int32_t* positions, const int64_t* slot_mapping, void* q_out, void* key_cache, void* value_cache,
                        int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t dk, int32_t dv, int32_t rot_dims, float eps,
                        int32_t cache_dtype, int32_t q_dtype, int64_t stream) {
    qk_norm_rope_cache_ex(qkv, ld, q_norm_w, k_norm_w, cos_t, sin_t, max_pos, positions, slot_mapping, q_out, key_cache, value_cache, num_tokens, num_heads,
                          num_kv_heads, dk, dv, rot_dims, eps, 0.f, 0, 0, cache_dtype, q_dtype, stream);
}

void qk_norm_rope_cache_ex(const float* qkv, int64_t ld, const float* q_norm_w, const float* k_norm_w, const float* cos_t, const float* sin_t,
                           int32_t max_pos, const int32_t* positions, const int64_t* slot_mapping, void* q_out, void* key_cache, void* value_cache,
                           int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t dk, int32_t dv, int32_t rot_dims, float eps,
                           float q_temp_coef, int32_t q_temp_every, int32_t v_unit_rms, int32_t cache_dtype, int32_t q_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(qkv && positions && slot_mapping && q_out && key_cache && value_cache, kErrBadArg, "qk_norm_rope_cache: null pointer");
    B200_REQUIRE((q_norm_w == nullptr) == (k_norm_w == nullptr) && (cos_t == nullptr) == (sin_t == nullptr), kErrBadArg,
                 "qk_norm_rope_cache: norm weights / tables come in pairs");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && dk > 0 && dv > 0 && rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0 &&
                 ld >= (int64_t)num_heads * dk + (int64_t)num_kv_heads * (dk + dv) && (!cos_t || max_pos > 0),
                 kErrBadArg, "qk_norm_rope_cache: bad sizes");
    cudaStream_t st = as_stream(stream);
#define QNRC(TC, TQ) launch_pdl(qk_norm_rope_cache_kernel<TC, TQ>, dim3(num_tokens), dim3(256), 0, st, qkv, ld, q_norm_w, k_norm_w, cos_t, sin_t, positions, \
        slot_mapping, (TQ*)q_out, (TC*)key_cache, (TC*)value_cache, num_heads, num_kv_heads, dk, dv, rot_dims, eps, q_temp_coef, q_temp_every, v_unit_rms)
    if (cache_dtype == B200_F32 && q_dtype == B200_F32) QNRC(float, float);
    else if (cache_dtype == B200_BF16 && q_dtype == B200_F32) QNRC(__nv_bfloat16, float);
    else if (cache_dtype == B200_BF16 && q_dtype == B200_BF16) QNRC(__nv_bfloat16, __nv_bfloat16);
    else { set_error(kErrUnsupported, "qk_norm_rope_cache: cache dtype %d / q dtype %d", cache_dtype, q_dtype); return; }
#undef QNRC
    count_launch();
    check_launch("qk_norm_rope_cache");
}

void chunk_decode_view(const int32_t* block_tables, int32_t table_width, const int32_t* positions, uint32_t* out_tables, uint32_t* out_ctx,
                       int32_t num_seqs, int32_t out_width, int32_t block_size, int32_t chunk, int64_t stream) {
    if (num_seqs == 0) return;
    B200_REQUIRE(block_tables && positions && out_tables && out_ctx && table_width > 0 && out_width > 0 && block_size > 0 && chunk > 0 &&
                 chunk % block_size == 0, kErrBadArg, "chunk_decode_view: bad arguments (chunk must be a multiple of the block size)");
    launch_pdl(chunk_decode_view_kernel, dim3(num_seqs), dim3(64), 0, as_stream(stream), block_tables, table_width, positions, out_tables, out_ctx, num_seqs,
               out_width, block_size, chunk);
    count_launch();
    check_launch("chunk_decode_view");
}

void paged_attention_varlen(void* out, const void* q, const void* key_cache, const void* value_cache, const int32_t* block_tables,
                            int32_t table_width, const int32_t* token_seq, const int32_t* positions, const int32_t* cu_seqlens_q,
                            const int32_t* cu_seqlens_k, int32_t num_seqs, int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t dk,
                            int32_t dv, int32_t block_size, float scale, int32_t chunk, int32_t window, int32_t q_dtype, int32_t cache_dtype,
                            int32_t out_dtype, int64_t stream) {
    paged_attention_varlen_sink(out, q, key_cache, value_cache, block_tables, table_width, token_seq, positions, cu_seqlens_q, cu_seqlens_k, num_seqs, num_tokens,
                                num_heads, num_kv_heads, dk, dv, block_size, scale, chunk, window, nullptr, q_dtype, cache_dtype, out_dtype, stream);
}

void paged_attention_varlen_sink(void* out, const void* q, const void* key_cache, const void* value_cache, const int32_t* block_tables,
                                 int32_t table_width, const int32_t* token_seq, const int32_t* positions, const int32_t* cu_seqlens_q,
                                 const int32_t* cu_seqlens_k, int32_t num_seqs, int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t dk,
                                 int32_t dv, int32_t block_size, float scale, int32_t chunk, int32_t window, const float* sink, int32_t q_dtype,
                                 int32_t cache_dtype, int32_t out_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(out && q && key_cache && value_cache && block_tables && token_seq && positions, kErrBadArg, "paged_attention_varlen: null pointer");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0 && block_size > 0 && table_width > 0,
                 kErrBadArg, "paged_attention_varlen: bad sizes");
    cudaStream_t st = as_stream(stream);
    // 16-bit q / cache / out with 128-wide heads and 64-token blocks: the tensor-core kernel that serves the other models' prefill
    // (attention_prefill.cu), with the chunk rule added to its mask; it covers portions and single tokens alike
    static const bool no_tc = [] { const char* e = getenv("B200_VARLEN_SIMT"); return e && atoi(e) != 0; }();
    PrefillExtras extras;
    extras.sink = sink;
    if (!no_tc && q_dtype == B200_BF16 && out_dtype == B200_BF16 && dk == dv && cu_seqlens_q && cu_seqlens_k && num_seqs > 0 &&
        paged_attention_prefill_tc_supported(dk, block_size, B200_BF16, cache_dtype, B200_KV_FLASH, 0.f, 1, q, key_cache, value_cache)) {
        paged_attention_prefill_tc(out, q, key_cache, value_cache, (const uint32_t*)block_tables, (const uint32_t*)cu_seqlens_q,
                                   (const uint32_t*)cu_seqlens_k, num_seqs, num_tokens, num_heads, num_kv_heads, table_width, (int64_t)1 << 22, scale,
                                   window, B200_BF16, st, chunk, &extras);
        return;
    }
    B200_REQUIRE(dv <= 32 * kMaxVPerLane && dk <= 2048, kErrUnsupported, "paged_attention_varlen: value size %d > %d or key size %d > 2048", dv,
                 32 * kMaxVPerLane, dk);
    const int64_t items = (int64_t)num_tokens * num_heads;
    const unsigned grid = (unsigned)((items + 3) / 4);
    const size_t smem = (size_t)4 * dk * sizeof(float);
#define PAV(TC, TO, TQ) launch_pdl(paged_attention_varlen_kernel<TC, TO, TQ>, dim3(grid), dim3(128), smem, st, (const TQ*)q, (const TC*)key_cache, \
        (const TC*)value_cache, block_tables, table_width, token_seq, positions, (TO*)out, items, num_heads, num_kv_heads, dk, dv, block_size, scale, chunk, window, sink)
    if (cache_dtype == B200_F32 && out_dtype == B200_F32 && q_dtype == B200_F32) PAV(float, float, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_BF16 && q_dtype == B200_F32) PAV(__nv_bfloat16, __nv_bfloat16, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_BF16 && q_dtype == B200_BF16) PAV(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_F32 && q_dtype == B200_F32) PAV(__nv_bfloat16, float, float);
    else { set_error(kErrUnsupported, "paged_attention_varlen: cache dtype %d / out dtype %d / q dtype %d", cache_dtype, out_dtype, q_dtype); return; }
#undef PAV
    count_launch();
    check_launch("paged_attention_varlen");
}

}  // extern "C"
