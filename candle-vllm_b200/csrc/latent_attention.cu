// latent_attention.cu -- multi-head attention over a low-rank latent for ragged steps (portions of prompts beside single decoded
// tokens in one launch), any sizes, f32 or bf16 cache.  Per token the paged cache keeps only the normed latent c [R] and ONE rotated key
// part k_r [dr] shared by all heads; head h's key is (W_uk[h] c, k_r), its value W_uv[h] c.  The step runs in the "absorbed" form:
//     q_lat[t, h] = (W_uk[h]^T q_n[t, h]  |  rot(q_r[t, h]))                      [R + dr]
//     s_j         = (q_lat[t, h] . (c_j | k_r_j)) * scale,   j <= position(t)  (and position(t) - j < window when window > 0)
//     p_j         = exp(s_j) / (sum_i exp(s_i) + exp(sink[h]))                    -- the sink joins the denominator only
//     o_lat[t, h] = sum_j p_j c_j                                                 [R]
//     out[t, h]   = sigmoid(gate[t, h]) * W_uv[h] o_lat[t, h]                     [dv]
// so every head of a token reads the same (R + dr) numbers per key, and W_uk / W_uv are touched once per token, not once per key.
//
//   latent_kv_rope_cache     from columns [off, off + R + dr) of the step's packed f32 projection: RMS norm of the first R (plain
//                            weight), rotation of the last dr (entry i with i + dr/2, cos / sin table rows by position), both
//                            written into the paged cache at slot_mapping[t].
//   latent_q_absorb          q_lat as above from the packed projection (SIMT: one block per (token, head); steps with many rows do the
//                            W_uk product on the tensor-core GEMM instead and call this with w_uk = null for the rotation alone).
//   latent_attention_varlen  one block per (token, group of heads): tiles of 32 keys are staged once in shared memory for all heads of
//                            the group, a lane scores one key, then the tile's latents are accumulated with lanes across the
//                            latent columns; online softmax in f32 that starts from the sink.  Steps of few rows cut every row's keys into
//                            `splits` runs (one block each) whose (max, sum, weighted sum) a second kernel folds.
//   latent_out_gate          out as above (w_uv = null: the product was done by the GEMM, only the gate and the cast remain).  The _ex form may take
//                            one gate per output entry (gate [T, H dv]) instead of one per head.
#include "common.cuh"

namespace b200 {
namespace {

template <typename TC>
__global__ void __launch_bounds__(128)
latent_kv_rope_cache_kernel(const float* __restrict__ proj, int64_t ld, int off, const float* __restrict__ norm_w, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int32_t* __restrict__ positions, const int64_t* __restrict__ slot_mapping,
                            TC* __restrict__ c_cache, TC* __restrict__ kr_cache, int R, int dr, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[4];
    const int t = blockIdx.x;
    const int64_t slot = slot_mapping[t];
    if (slot < 0) return;
    const float* row = proj + (int64_t)t * ld + off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += 128) { const float v = row[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float sc = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)R + eps);
    for (int i = threadIdx.x; i < R; i += 128) c_cache[slot * R + i] = from_f32<TC>(row[i] * sc * (norm_w ? norm_w[i] : 1.0f));
    const int half = dr >> 1;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < dr; i += 128) {
        float v = row[R + i];
        if (cos_t) {
            const int f = i < half ? i : i - half;
            const float c = cos_t[(int64_t)pos * half + f], s = sin_t[(int64_t)pos * half + f];
            const float other = row[R + (i < half ? i + half : i - half)];
            v = i < half ? v * c - other * s : v * c + other * s;
        }
        kr_cache[slot * dr + i] = from_f32<TC>(v);
    }
}

template <typename TW>
__global__ void __launch_bounds__(128)
latent_q_absorb_kernel(const float* __restrict__ proj, int64_t ld, const TW* __restrict__ w_uk, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, const int32_t* __restrict__ positions, float* __restrict__ q_lat, int64_t q_st, int64_t q_sh,
                       __nv_bfloat16* __restrict__ qn16, int64_t rows16, int H, int dn, int dr, int R) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float qn[];                          // [dn]
    const int t = blockIdx.x, h = blockIdx.y;
    const float* q = proj + (int64_t)t * ld + (int64_t)h * (dn + dr);
    float* o = q_lat + (int64_t)t * q_st + (int64_t)h * q_sh;
    const int half = dr >> 1;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < dr; i += 128) {
        float v = q[dn + i];
        if (cos_t) {
            const int f = i < half ? i : i - half;
            const float c = cos_t[(int64_t)pos * half + f], s = sin_t[(int64_t)pos * half + f];
            const float other = q[dn + (i < half ? i + half : i - half)];
            v = i < half ? v * c - other * s : v * c + other * s;
        }
        o[R + i] = v;
    }
    if (qn16)                                              // [H, rows16, dn]: the unrotated part as the 16-bit operand of the grouped product
        for (int i = threadIdx.x; i < dn; i += 128) qn16[((int64_t)h * rows16 + t) * dn + i] = __float2bfloat16_rn(q[i]);
    if (!w_uk) return;
    for (int i = threadIdx.x; i < dn; i += 128) qn[i] = q[i];
    __syncthreads();
    const TW* w = w_uk + (int64_t)h * dn * R;               // [dn, R]: column r of all rows is coalesced over the threads
    for (int r = threadIdx.x; r < R; r += 128) {
        float a = 0.f;
        for (int d = 0; d < dn; ++d) a = fmaf(qn[d], to_f32<TW>(w[(int64_t)d * R + r]), a);
        o[r] = a;
    }
}

template <typename TC, typename TO, int NR>
__global__ void __launch_bounds__(256)
latent_attention_varlen_kernel(const float* __restrict__ q_lat, int64_t q_st, int64_t q_sh, const TC* __restrict__ c_cache, const TC* __restrict__ kr_cache,
                               const int32_t* __restrict__ block_tables, int table_width, const int32_t* __restrict__ token_seq,
                               const int32_t* __restrict__ positions, const float* __restrict__ sink, TO* __restrict__ o_lat, int64_t o_st, int64_t o_sh,
                               int H, int R, int dr, int block_size, float scale, int window, int groups_per_token, int splits, float* __restrict__ part) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float sm[];
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = R + dr, stride = W | 1;                  // odd row pitch: a warp reading one column of 32 rows hits 32 banks
    float* qs = sm;                                        // [nw][W]
    float* tile = sm + nw * W;                             // [32][stride]
    const int t = blockIdx.x / groups_per_token;
    const int h = (blockIdx.x - t * groups_per_token) * nw + warp;
    const bool live = h < H;
    int pos = positions[t];
    const int32_t* table = block_tables + (int64_t)token_seq[t] * table_width;
    if (live) {
        const float* q = q_lat + (int64_t)t * q_st + (int64_t)h * q_sh;
        for (int i = lane; i < W; i += 32) qs[warp * W + i] = q[i] * scale;
    }
    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    int hi = pos;
    const int split = blockIdx.y;
    if (splits > 1) {
        // the row's keys are cut into `splits` runs of whole 32-key tiles; this block takes run blockIdx.y and leaves (m, l, sum) for the merge
        const int run = (((pos - lo + 1) + splits - 1) / splits + 31) / 32 * 32;
        lo += split * run;
        hi = min(pos, lo + run - 1);
    }
    // the sink is a key without a value whose score is sink[h] as it stands (it joins the first run only)
    const bool with_sink = live && sink && split == 0;
    float m = with_sink ? sink[h] : -INFINITY, l = with_sink ? 1.f : 0.f;
    float acc[NR];
#pragma unroll
    for (int c = 0; c < NR; ++c) acc[c] = 0.f;
    pos = hi;
    for (int j0 = lo; j0 <= pos; j0 += 32) {
        __syncthreads();                                   // q staged / previous tile consumed
        for (int kk = warp; kk < 32; kk += nw) {
            const int j = j0 + kk;
            float* dst = tile + kk * stride;
            if (j <= pos) {
                const int64_t phys = (int64_t)table[j / block_size] * block_size + j % block_size;
                const TC* cr = c_cache + phys * R;
                const TC* kr = kr_cache + phys * dr;
                for (int i = lane; i < R; i += 32) dst[i] = to_f32<TC>(cr[i]);
                for (int i = lane; i < dr; i += 32) dst[R + i] = to_f32<TC>(kr[i]);
            } else {
                for (int i = lane; i < W; i += 32) dst[i] = 0.f;
            }
        }
        __syncthreads();
        if (!live) continue;
        const bool valid = j0 + lane <= pos;
        float s = -INFINITY;
        if (valid) {
            const float* kr = tile + lane * stride;
            const float* qw = qs + warp * W;
            float d0 = 0.f, d1 = 0.f;
            int i = 0;
            for (; i + 1 < W; i += 2) { d0 = fmaf(qw[i], kr[i], d0); d1 = fmaf(qw[i + 1], kr[i + 1], d1); }
            if (i < W) d0 = fmaf(qw[i], kr[i], d0);
            s = d0 + d1;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);      // m = -inf only before the first tile of a sink-less run: l and acc are 0
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < NR; ++c) acc[c] *= corr;
        const int cnt = min(32, pos - j0 + 1);
        for (int kk = 0; kk < cnt; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const float* cr = tile + kk * stride;
#pragma unroll
            for (int c = 0; c < NR; ++c) {
                const int i = lane + 32 * c;
                if (i < R) acc[c] = fmaf(pk, cr[i], acc[c]);
            }
        }
    }
    if (!live) return;
    if (splits > 1) {
        float* dst = part + (((int64_t)t * H + h) * splits + split) * (R + 2);
        if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
        for (int c = 0; c < NR; ++c) {
            const int i = lane + 32 * c;
            if (i < R) dst[2 + i] = acc[c];
        }
        return;
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int c = 0; c < NR; ++c) {
        const int i = lane + 32 * c;
        if (i < R) o_lat[(int64_t)t * o_st + (int64_t)h * o_sh + i] = from_f32<TO>(acc[c] * inv);
    }
}

// folds the runs of a split row: with M = max m_s, out = sum_s exp(m_s - M) sum_s / sum_s exp(m_s - M) l_s (a run without keys has m = -inf, l = 0)
template <typename TO>
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ part, TO* __restrict__ o_lat, int64_t o_st, int64_t o_sh, int H, int R, int splits) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = part + ((int64_t)t * H + h) * splits * (R + 2);
    float M = -INFINITY;
    for (int s2 = 0; s2 < splits; ++s2) M = fmaxf(M, src[(int64_t)s2 * (R + 2)]);
    float L = 0.f;
    for (int s2 = 0; s2 < splits; ++s2) {
        const float ms = src[(int64_t)s2 * (R + 2)];
        if (ms != -INFINITY) L = fmaf(expf(ms - M), src[(int64_t)s2 * (R + 2) + 1], L);
    }
    const float inv = 1.0f / L;
    for (int i = threadIdx.x; i < R; i += 128) {
        float a = 0.f;
        for (int s2 = 0; s2 < splits; ++s2) {
            const float ms = src[(int64_t)s2 * (R + 2)];
            if (ms != -INFINITY) a = fmaf(expf(ms - M), src[(int64_t)s2 * (R + 2) + 2 + i], a);
        }
        o_lat[(int64_t)t * o_st + (int64_t)h * o_sh + i] = from_f32<TO>(a * inv);
    }
}

template <typename TW, typename TOut>
__global__ void __launch_bounds__(128)
latent_out_gate_kernel(const float* __restrict__ src, int64_t s_st, int64_t s_sh, const TW* __restrict__ w_uv, const float* __restrict__ gate,
                       int64_t ld_gate, TOut* __restrict__ out, int H, int dv, int R, int gate_per_element) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float ol[];                          // [R]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // one gate per head, or (gate_per_element) one per output entry: gate [T, H dv]
    const float* ge = gate && gate_per_element ? gate + (int64_t)t * ld_gate + (int64_t)h * dv : nullptr;
    const float gv = gate && !ge ? 1.0f / (1.0f + expf(-gate[(int64_t)t * ld_gate + h])) : 1.0f;
    TOut* o = out + ((int64_t)t * H + h) * dv;
    const float* sp = src + (int64_t)t * s_st + (int64_t)h * s_sh;
    if (!w_uv) {                                           // src holds the dv values already
        for (int i = threadIdx.x; i < dv; i += 128) o[i] = from_f32<TOut>(sp[i] * (ge ? 1.0f / (1.0f + expf(-ge[i])) : gv));
        return;
    }
    for (int i = threadIdx.x; i < R; i += 128) ol[i] = sp[i];
    __syncthreads();
    const TW* w = w_uv + (int64_t)h * dv * R;               // [dv, R]
    for (int d = warp; d < dv; d += 4) {
        float a = 0.f;
        for (int r = lane; r < R; r += 32) a = fmaf(ol[r], to_f32<TW>(w[(int64_t)d * R + r]), a);
        a = warp_sum(a);
        if (lane == 0) o[d] = from_f32<TOut>(a * (ge ? 1.0f / (1.0f + expf(-ge[d])) : gv));
    }
}

// out[t, h, :n] (bf16, any token / head strides) = src[t, h, :n] (f32 or bf16, any strides): moves rows between the head-major buffers of the grouped
// products and the token-major ones of the split-KV decode kernel; optionally also ctx[t] = positions[t] + 1
template <typename TS>
__global__ void __launch_bounds__(128)
repack_heads_kernel(const TS* __restrict__ src, int64_t s_st, int64_t s_sh, __nv_bfloat16* __restrict__ dst, int64_t d_st, int64_t d_sh, int n,
                    const int32_t* __restrict__ positions, uint32_t* __restrict__ ctx) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const TS* s = src + (int64_t)t * s_st + (int64_t)h * s_sh;
    __nv_bfloat16* d = dst + (int64_t)t * d_st + (int64_t)h * d_sh;
    for (int i = threadIdx.x; i < n; i += 128) d[i] = __float2bfloat16_rn(to_f32<TS>(s[i]));
    if (ctx && h == 0 && threadIdx.x == 0) ctx[t] = (uint32_t)(positions[t] + 1);
}

// every row of a step as a one-row "sequence": its own copy of its sequence's block table and its context length (position + 1), the form in
// which the split-KV decode kernel serves rows of prompts as well
__global__ void __launch_bounds__(64)
token_tables_kernel(const int32_t* __restrict__ block_tables, int table_width, const int32_t* __restrict__ token_seq, const int32_t* __restrict__ positions,
                    uint32_t* __restrict__ out_tables, uint32_t* __restrict__ ctx) {
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    const int32_t* src = block_tables + (int64_t)token_seq[t] * table_width;
    for (int i = threadIdx.x; i < table_width; i += 64) out_tables[t * table_width + i] = (uint32_t)src[i];
    if (threadIdx.x == 0) ctx[t] = (uint32_t)(positions[t] + 1);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void latent_kv_rope_cache(const float* proj, int64_t ld, int32_t off, const float* norm_w, const float* cos_t, const float* sin_t, int32_t max_pos,
                          const int32_t* positions, const int64_t* slot_mapping, void* c_cache, void* kr_cache, int32_t num_tokens, int32_t rank,
                          int32_t rot_dim, float eps, int32_t cache_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(proj && positions && slot_mapping && c_cache && kr_cache, kErrBadArg, "latent_kv_rope_cache: null pointer");
    B200_REQUIRE(rank > 0 && rot_dim >= 0 && rot_dim % 2 == 0 && off >= 0 && ld >= (int64_t)off + rank + rot_dim && (cos_t == nullptr) == (sin_t == nullptr) &&
                 (!cos_t || max_pos > 0), kErrBadArg, "latent_kv_rope_cache: bad sizes");
    cudaStream_t st = as_stream(stream);
    if (cache_dtype == B200_F32)
        launch_pdl(latent_kv_rope_cache_kernel<float>, dim3(num_tokens), dim3(128), 0, st, proj, ld, off, norm_w, cos_t, sin_t, positions, slot_mapping,
                   (float*)c_cache, (float*)kr_cache, rank, rot_dim, eps);
    else if (cache_dtype == B200_BF16)
        launch_pdl(latent_kv_rope_cache_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, st, proj, ld, off, norm_w, cos_t, sin_t, positions, slot_mapping,
                   (__nv_bfloat16*)c_cache, (__nv_bfloat16*)kr_cache, rank, rot_dim, eps);
    else { set_error(kErrUnsupported, "latent_kv_rope_cache: cache dtype %d (f32 / bf16)", cache_dtype); return; }
    count_launch();
    check_launch("latent_kv_rope_cache");
}

void latent_q_absorb(const float* proj, int64_t ld, const void* w_uk, const float* cos_t, const float* sin_t, int32_t max_pos, const int32_t* positions,
                     float* q_lat, int64_t q_stride_token, int64_t q_stride_head, void* qn16, int64_t rows16, int32_t num_tokens, int32_t num_heads, int32_t dn,
                     int32_t rot_dim, int32_t rank, int32_t w_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(proj && positions && q_lat, kErrBadArg, "latent_q_absorb: null pointer");
    B200_REQUIRE(num_heads > 0 && num_heads <= 65535 && dn > 0 && rank > 0 && rot_dim >= 0 && rot_dim % 2 == 0 && ld >= (int64_t)num_heads * (dn + rot_dim) &&
                 (cos_t == nullptr) == (sin_t == nullptr) && (!cos_t || max_pos > 0) && dn <= 8192 && (!qn16 || rows16 >= num_tokens), kErrBadArg,
                 "latent_q_absorb: bad sizes");
    cudaStream_t st = as_stream(stream);
    const size_t smem = (size_t)dn * sizeof(float);
    const dim3 grid(num_tokens, num_heads);
    if (w_dtype == B200_F32)
        launch_pdl(latent_q_absorb_kernel<float>, grid, dim3(128), smem, st, proj, ld, (const float*)w_uk, cos_t, sin_t, positions, q_lat, q_stride_token,
                   q_stride_head, (__nv_bfloat16*)qn16, rows16, num_heads, dn, rot_dim, rank);
    else if (w_dtype == B200_BF16)
        launch_pdl(latent_q_absorb_kernel<__nv_bfloat16>, grid, dim3(128), smem, st, proj, ld, (const __nv_bfloat16*)w_uk, cos_t, sin_t, positions, q_lat, q_stride_token,
                   q_stride_head, (__nv_bfloat16*)qn16, rows16, num_heads, dn, rot_dim, rank);
    else { set_error(kErrUnsupported, "latent_q_absorb: weight dtype %d (f32 / bf16)", w_dtype); return; }
    count_launch();
    check_launch("latent_q_absorb");
}

void latent_attention_varlen(void* o_lat, int64_t o_stride_token, int64_t o_stride_head, int32_t out_dtype, const float* q_lat, int64_t q_stride_token,
                             int64_t q_stride_head, const void* c_cache, const void* kr_cache, const int32_t* block_tables, int32_t table_width,
                             const int32_t* token_seq, const int32_t* positions, const float* sink, int32_t num_tokens, int32_t num_heads, int32_t rank,
                             int32_t rot_dim, int32_t block_size, float scale, int32_t window, int32_t cache_dtype, int32_t splits, float* partials,
                             int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(o_lat && q_lat && c_cache && kr_cache && block_tables && token_seq && positions, kErrBadArg, "latent_attention_varlen: null pointer");
    B200_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || partials) && num_heads <= 65535, kErrBadArg, "latent_attention_varlen: %d runs need a partials buffer",
                 splits);
    B200_REQUIRE(num_heads > 0 && rank > 0 && rot_dim >= 0 && block_size > 0 && table_width > 0 && window >= 0, kErrBadArg, "latent_attention_varlen: bad sizes");
    B200_REQUIRE(rank <= 1024, kErrUnsupported, "latent_attention_varlen: latent size %d > 1024", rank);
    cudaStream_t st = as_stream(stream);
    const int nw = num_heads >= 8 ? 8 : 4;
    const int groups = (num_heads + nw - 1) / nw;
    const int W = rank + rot_dim;
    const size_t smem = ((size_t)nw * W + (size_t)32 * (W | 1)) * sizeof(float);
    B200_REQUIRE(smem <= 200 * 1024, kErrUnsupported, "latent_attention_varlen: latent + rotated size %d does not fit shared memory", W);
    const dim3 grid((unsigned)((int64_t)num_tokens * groups), (unsigned)splits);
#define LAV(TC, TO, NR)                                                                                                                             \
    do {                                                                                                                                            \
        auto kern = latent_attention_varlen_kernel<TC, TO, NR>;                                                                                     \
        ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem);                                                                        \
        launch_pdl(kern, grid, dim3(nw * 32), smem, st, q_lat, q_stride_token, q_stride_head, (const TC*)c_cache, (const TC*)kr_cache, block_tables, table_width,  \
                   token_seq, positions, sink, (TO*)o_lat, o_stride_token, o_stride_head, num_heads, rank, rot_dim, block_size, scale, window, groups, splits, \
                   partials);                                                                                                                       \
    } while (0)
#define LAV_R(TC, TO)                                                                                                                               \
    do {                                                                                                                                            \
        if (rank <= 128) LAV(TC, TO, 4); else if (rank <= 256) LAV(TC, TO, 8); else if (rank <= 512) LAV(TC, TO, 16); else LAV(TC, TO, 32);         \
    } while (0)
    if (cache_dtype == B200_F32 && out_dtype == B200_F32) LAV_R(float, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_F32) LAV_R(__nv_bfloat16, float);
    else if (cache_dtype == B200_BF16 && out_dtype == B200_BF16) LAV_R(__nv_bfloat16, __nv_bfloat16);
    else { set_error(kErrUnsupported, "latent_attention_varlen: cache dtype %d / out dtype %d", cache_dtype, out_dtype); return; }
#undef LAV_R
#undef LAV
    count_launch();
    if (splits > 1) {
        const dim3 mg(num_tokens, num_heads);
        if (out_dtype == B200_F32)
            launch_pdl(latent_attention_merge_kernel<float>, mg, dim3(128), 0, st, (const float*)partials, (float*)o_lat, o_stride_token, o_stride_head, num_heads, rank, splits);
        else
            launch_pdl(latent_attention_merge_kernel<__nv_bfloat16>, mg, dim3(128), 0, st, (const float*)partials, (__nv_bfloat16*)o_lat, o_stride_token, o_stride_head,
                       num_heads, rank, splits);
        count_launch();
    }
    check_launch("latent_attention_varlen");
}

void latent_out_gate(const float* src, int64_t src_stride_token, int64_t src_stride_head, const void* w_uv, const float* gate, int64_t ld_gate, void* out,
                     int32_t num_tokens, int32_t num_heads, int32_t dv, int32_t rank, int32_t w_dtype, int32_t out_dtype, int64_t stream) {
    latent_out_gate_ex(src, src_stride_token, src_stride_head, w_uv, gate, ld_gate, 0, out, num_tokens, num_heads, dv, rank, w_dtype, out_dtype, stream);
}

void latent_out_gate_ex(const float* src, int64_t src_stride_token, int64_t src_stride_head, const void* w_uv, const float* gate, int64_t ld_gate,
                        int32_t gate_per_element, void* out, int32_t num_tokens, int32_t num_heads, int32_t dv, int32_t rank, int32_t w_dtype, int32_t out_dtype,
                        int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(src && out && num_heads > 0 && num_heads <= 65535 && dv > 0 && rank > 0 && rank <= 8192 &&
                 (!gate || ld_gate >= (int64_t)num_heads * (gate_per_element ? dv : 1)), kErrBadArg, "latent_out_gate: bad arguments");
    cudaStream_t st = as_stream(stream);
    const size_t smem = (size_t)rank * sizeof(float);
    const dim3 grid(num_tokens, num_heads);
#define LOG(TW, TO) launch_pdl(latent_out_gate_kernel<TW, TO>, grid, dim3(128), smem, st, src, src_stride_token, src_stride_head, (const TW*)w_uv, gate, ld_gate, (TO*)out, \
                               num_heads, dv, rank, gate_per_element)
    if (w_dtype == B200_F32 && out_dtype == B200_F32) LOG(float, float);
    else if (w_dtype == B200_BF16 && out_dtype == B200_BF16) LOG(__nv_bfloat16, __nv_bfloat16);
    else if (w_dtype == B200_BF16 && out_dtype == B200_F32) LOG(__nv_bfloat16, float);
    else { set_error(kErrUnsupported, "latent_out_gate: weight dtype %d / out dtype %d", w_dtype, out_dtype); return; }
#undef LOG
    count_launch();
    check_launch("latent_out_gate");
}

void repack_heads(const void* src, int32_t src_dtype, int64_t src_stride_token, int64_t src_stride_head, void* dst, int64_t dst_stride_token, int64_t dst_stride_head,
                  int32_t num_tokens, int32_t num_heads, int32_t n, const int32_t* positions, uint32_t* context_lens, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(src && dst && num_heads > 0 && num_heads <= 65535 && n > 0 && (!context_lens || positions), kErrBadArg, "repack_heads: bad arguments");
    cudaStream_t st = as_stream(stream);
    const dim3 grid(num_tokens, num_heads);
    if (src_dtype == B200_F32)
        launch_pdl(repack_heads_kernel<float>, grid, dim3(128), 0, st, (const float*)src, src_stride_token, src_stride_head, (__nv_bfloat16*)dst, dst_stride_token,
                   dst_stride_head, n, positions, context_lens);
    else if (src_dtype == B200_BF16)
        launch_pdl(repack_heads_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, (const __nv_bfloat16*)src, src_stride_token, src_stride_head, (__nv_bfloat16*)dst,
                   dst_stride_token, dst_stride_head, n, positions, context_lens);
    else { set_error(kErrUnsupported, "repack_heads: source dtype %d (f32 / bf16)", src_dtype); return; }
    count_launch();
    check_launch("repack_heads");
}

void token_tables(const int32_t* block_tables, int32_t table_width, const int32_t* token_seq, const int32_t* positions, uint32_t* out_tables,
                  uint32_t* context_lens, int32_t num_tokens, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(block_tables && token_seq && positions && out_tables && context_lens && table_width > 0, kErrBadArg, "token_tables: bad arguments");
    launch_pdl(token_tables_kernel, dim3(num_tokens), dim3(64), 0, as_stream(stream), block_tables, table_width, token_seq, positions, out_tables, context_lens);
    count_launch();
    check_launch("token_tables");
}

}  // extern "C"
