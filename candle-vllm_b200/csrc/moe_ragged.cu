// moe_ragged.cu -- mixture of experts on dense f32 / bf16 expert weights for ragged steps: the router's choice and the expert
// feed-forward for steps of few rows (every (token, choice) pair streams its expert once; steps with many rows sort the pairs by
// expert and run the expert products on the tensor-core GEMM instead).
//
//   moe_route         per token, from f32 router logits z [N]: s = softmax(z) over all N outputs; choice score = s + correction; the
//                     outputs form `groups` equal runs of neighbours, a group's score is its best choice score, and only members of the
//                     `keep` best groups can be chosen (the others count as -inf); the `top` best choice scores are taken (ties: the lower
//                     index); weights = s of the chosen / (their sum + 1e-20) * scale.  groups <= 1 switches the restriction off.
//                     The _ex form takes the scores from a sigmoid per output instead of the softmax, and may leave the chosen scores as they are; the
//                     _bias form first adds a bias to the logits (softmax over all outputs, renormalised over the chosen = softmax over the chosen logits).
//   moe_gate_up       act[p] = silu(W_gate[e] h) * (W_up[e] h); the _ex form may first multiply both products by the pair's weight (an expert fed its
//                     token times the router's score) and has the clamped activation of glu_packed, and the ungated form act[p] = relu(W_up[e] h)^2 with
//                     one matrix [ff, D] per expert.  Pair p = (token, choice) with expert e < E; outputs
//                     e >= E are identity experts (no weights) and are skipped.
//   moe_down          y[row] = W_down[e] act[p] for the pairs in expert order (moe_align with tiles of one row);
//   moe_combine_rows  out[t] = sum over the token's choices, in choice order, of weight * y[row of the pair], or weight * x[t] for an
//                     identity expert.
// Steps with many rows (bf16): moe_align sorts the pairs by expert into tiles of 128 rows (padding each expert's run), moe_gather_rows copies
// the tokens' rows into that order, the two expert products run as grouped tcgen05 GEMMs (dense_gemm.cu, the weight tile chosen per row tile),
// silu_mul_packed sits between them, and the same moe_combine_rows adds each token's choices in choice order.
#include "common.cuh"

namespace b200 {
namespace {

__global__ void __launch_bounds__(32)
moe_route_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ correction, int32_t* __restrict__ ids, float* __restrict__ weights,
                 int N, int top, int groups, int keep, float scale, int score_fn, int normalise, const float* __restrict__ logit_bias) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float sm[];
    float* s = sm;                 // [N] softmax
    float* pick = sm + N;          // [N] choice scores, -inf once masked or taken
    float* gbest = sm + 2 * N;     // [groups]
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* z = logits + (int64_t)t * ld;
    if (logit_bias) {                                      // a bias that belongs to the logits: it counts for the choice and for the weights
        float* zb = sm + 2 * N + (groups > 1 ? groups : 1);
        for (int i = lane; i < N; i += 32) zb[i] = z[i] + logit_bias[i];
        __syncwarp();
        z = zb;
    }
    if (score_fn == 1) {
        for (int i = lane; i < N; i += 32) { s[i] = 1.0f / (1.0f + expf(-z[i])); pick[i] = s[i] + (correction ? correction[i] : 0.f); }
    } else {
        float mx = -INFINITY;
        for (int i = lane; i < N; i += 32) mx = fmaxf(mx, z[i]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int i = lane; i < N; i += 32) { const float e = expf(z[i] - mx); s[i] = e; sum += e; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int i = lane; i < N; i += 32) { s[i] *= inv; pick[i] = s[i] + (correction ? correction[i] : 0.f); }
    }
    __syncwarp();
    if (groups > 1) {
        const int per = N / groups;
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int i = 0; i < per; ++i) b = fmaxf(b, pick[g * per + i]);
            gbest[g] = b;
        }
        __syncwarp();
        // take the `keep` best groups one at a time; a taken group is marked +inf, the rest are masked afterwards
        for (int r = 0; r < keep; ++r) {
            float b = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) { const float v = gbest[g]; if (v != INFINITY && (v > b || bi == 0x7fffffff)) { b = v; bi = g; } }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, b, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > b || (ob == b && oi < bi))) { b = ob; bi = oi; }
            }
            if (lane == 0 && bi != 0x7fffffff) gbest[bi] = INFINITY;
            __syncwarp();
        }
        for (int i = lane; i < N; i += 32) if (gbest[i / per] != INFINITY) pick[i] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int r = 0; r < top; ++r) {
        float b = -INFINITY; int bi = 0x7fffffff;
        for (int i = lane; i < N; i += 32) { const float v = pick[i]; if (!isnan(v) && (bi == 0x7fffffff ? v > -INFINITY : v > b)) { b = v; bi = i; } }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, b, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > b || (ob == b && oi < bi))) { b = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                      // fewer eligible outputs than `top` (a configuration error): repeat output 0 with weight s[0]
        if (lane == 0) { ids[(int64_t)t * top + r] = bi; pick[bi] = NAN; }
        wsum += s[bi];
        __syncwarp();
    }
    const float norm = normalise ? scale / (wsum + 1e-20f) : scale;
    for (int r = lane; r < top; r += 32) weights[(int64_t)t * top + r] = s[ids[(int64_t)t * top + r]] * norm;
}

// Dot of a weight row with a vector staged in shared memory as f32, lanes striding over the row.  When rows allow 16-byte loads (`vec`) a lane
// takes kVec consecutive weights at once and the vector is staged so that element i sits at (i % kVec) * (n / kVec) + i / kVec: for each of
// the kVec sub-steps the lanes then read consecutive words (no bank conflicts).
template <typename T>
__device__ __forceinline__ bool rows_vectorise(const T* base, int n, int64_t pitch) {
    constexpr int kVec = 16 / (int)sizeof(T);
    return n % kVec == 0 && pitch % kVec == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}
template <typename T>
__device__ __forceinline__ int staged_at(int i, int n, bool vec) {
    constexpr int kVec = 16 / (int)sizeof(T);
    return vec ? (i % kVec) * (n / kVec) + i / kVec : i;
}
template <typename T>
__device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* __restrict__ v, int n, int lane, bool vec) {
    float a = 0.f;
    constexpr int kVec = 16 / (int)sizeof(T);
    if (vec) {
        const int nv = n / kVec;
        for (int i = lane; i < nv; i += 32) {
            const uint4 raw = reinterpret_cast<const uint4*>(w)[i];
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int c = 0; c < kVec; ++c) a = fmaf(v[c * nv + i], to_f32<T>(e[c]), a);
        }
    } else {
        for (int i = lane; i < n; i += 32) a = fmaf(v[i], to_f32<T>(w[i]), a);
    }
    return a;
}

constexpr int kGuRows = 32;        // gate / up rows per block of moe_gate_up
constexpr int kDownCols = 64;      // output columns per block of moe_down

template <typename T>
__global__ void __launch_bounds__(128)
moe_gate_up_kernel(const T* __restrict__ h, int64_t ldh, const T* __restrict__ w_gu, const int32_t* __restrict__ ids, const int32_t* __restrict__ order,
                   T* __restrict__ act, int top, int E, int ff, int D, int act_fn, float limit, const float* __restrict__ pair_scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float hs[];                          // [D]
    const int64_t p = order ? (int64_t)order[blockIdx.x] : (int64_t)blockIdx.x;      // `order` walks the pairs expert by expert: blocks running together share weights
    if (p < 0) return;
    const int e = ids[p];
    if (e < 0 || e >= E) return;                           // identity expert: nothing to compute
    const int64_t t = p / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = rows_vectorise<T>(w_gu, D, D);
    for (int i = threadIdx.x; i < D; i += 128) hs[staged_at<T>(i, D, vec)] = to_f32<T>(h[t * ldh + i]);
    __syncthreads();
    const bool gated = act_fn != 3;                         // ungated experts keep one matrix [ff, D] in front of the activation
    const T* wg = w_gu + (int64_t)e * (gated ? 2 : 1) * ff * D;           // [gate rows | up rows][D]
    const int j1 = min(ff, (int)(blockIdx.y + 1) * kGuRows);
    for (int j = blockIdx.y * kGuRows + warp; j < j1; j += 4) {
        float a = row_dot<T>(wg + (int64_t)j * D, hs, D, lane, vec), b = gated ? row_dot<T>(wg + (int64_t)(ff + j) * D, hs, D, lane, vec) : 0.f;
        a = warp_sum(a);
        if (gated) b = warp_sum(b);
        if (lane == 0) {
            if (pair_scale) { const float sc = pair_scale[p]; a *= sc; b *= sc; }         // the expert sees its token times the pair's weight
            float v;
            if (act_fn == 3) {
                a = fmaxf(a, 0.f);
                v = a * a;
            } else if (act_fn == 2) {
                a = fminf(a, limit); b = fminf(fmaxf(b, -limit), limit);
                v = a / (1.0f + expf(-1.702f * a)) * (b + 1.0f);
            } else {
                v = a / (1.0f + expf(-a)) * b;
            }
            act[p * ff + j] = from_f32<T>(v);
        }
    }
}

// y[row] = W_down[e] act[p] for the pair p = order[row] (rows in expert order), f32 out
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_d, const int32_t* __restrict__ ids, const int32_t* __restrict__ order, float* __restrict__ y,
                int E, int ff, int D) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float as[];                          // [ff]
    const int64_t row = blockIdx.x;
    const int64_t p = order[row];
    if (p < 0) return;
    const int e = ids[p];
    if (e < 0 || e >= E) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = rows_vectorise<T>(w_d, ff, ff);
    for (int i = threadIdx.x; i < ff; i += 256) as[staged_at<T>(i, ff, vec)] = to_f32<T>(act[p * ff + i]);
    __syncthreads();
    const int d1 = min(D, (int)(blockIdx.y + 1) * kDownCols);
    for (int d = blockIdx.y * kDownCols + warp; d < d1; d += 8) {
        const float a = warp_sum(row_dot<T>(w_d + ((int64_t)e * D + d) * ff, as, ff, lane, vec));
        if (lane == 0) y[row * D + d] = a;
    }
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ pair_row, int32_t* __restrict__ row_pair, int32_t* __restrict__ tile_group, int pairs,
                 int E, int max_rows, int kTile) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ int sh[];
    int* count = sh;               // [E]
    int* start = sh + E;           // [E + 1] first row of every expert's padded run
    int* cursor = sh + 2 * E + 1;  // [E]
    for (int e = threadIdx.x; e < E; e += 1024) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += 1024) { const int e = ids[p]; if (e >= 0 && e < E) atomicAdd(&count[e], 1); }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) { start[e] = at; at += (count[e] + kTile - 1) / kTile * kTile; }
        start[E] = at;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < max_rows; r += 1024) row_pair[r] = -1;
    if (tile_group)
        for (int i = threadIdx.x; i < max_rows / kTile; i += 1024) tile_group[i] = -1;
    __syncthreads();
    if (tile_group)
        for (int e = threadIdx.x; e < E; e += 1024)
            for (int i = start[e] / kTile; i < start[e + 1] / kTile; ++i) tile_group[i] = e;
    for (int p = threadIdx.x; p < pairs; p += 1024) {
        const int e = ids[p];
        int row = -1;
        if (e >= 0 && e < E) { row = start[e] + atomicAdd(&cursor[e], 1); row_pair[row] = p; }
        pair_row[p] = row;
    }
}

__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ h, int64_t ldh, const int32_t* __restrict__ row_pair, __nv_bfloat16* __restrict__ xg, int top, int D) {
    pdl_wait();
    pdl_trigger();
    const int64_t r = blockIdx.x;
    const int p = row_pair[r];
    __nv_bfloat16* dst = xg + r * D;
    if (p < 0) { for (int i = threadIdx.x; i < D; i += 128) dst[i] = __float2bfloat16_rn(0.f); return; }
    const __nv_bfloat16* src = h + (int64_t)(p / top) * ldh;
    for (int i = threadIdx.x; i < D; i += 128) dst[i] = src[i];
}

template <typename TOut>
__global__ void silu_mul_packed_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int64_t rows, int ff, int64_t ld) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * ff) return;
    const int64_t r = i / ff;
    const int c = (int)(i - r * ff);
    const float g = gu[r * ld + c], u = gu[r * ld + ff + c];
    out[i] = from_f32<TOut>(g / (1.0f + expf(-g)) * u);
}

__global__ void __launch_bounds__(256)
moe_combine_rows_kernel(const float* __restrict__ y, const int32_t* __restrict__ pair_row, const float* __restrict__ weights, const float* __restrict__ x,
                        int64_t ldx, float* __restrict__ out, int top, int D) {
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += 256) {
        float tot = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = pair_row[t * top + k];
            tot = fmaf(weights ? weights[t * top + k] : 1.0f, row >= 0 ? y[(int64_t)row * D + d] : x[t * ldx + d], tot);
        }
        out[t * D + d] = tot;
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void moe_route(const float* logits, int64_t ld, const float* correction, int32_t* ids, float* weights, int32_t num_tokens, int32_t num_outputs, int32_t top,
               int32_t groups, int32_t keep, float scale, int64_t stream) {
    moe_route_ex(logits, ld, correction, ids, weights, num_tokens, num_outputs, top, groups, keep, scale, 0, 1, stream);
}

void moe_route_ex(const float* logits, int64_t ld, const float* correction, int32_t* ids, float* weights, int32_t num_tokens, int32_t num_outputs, int32_t top,
                  int32_t groups, int32_t keep, float scale, int32_t score_fn, int32_t normalise, int64_t stream) {
    moe_route_bias(logits, ld, nullptr, correction, ids, weights, num_tokens, num_outputs, top, groups, keep, scale, score_fn, normalise, stream);
}

void moe_route_bias(const float* logits, int64_t ld, const float* logit_bias, const float* correction, int32_t* ids, float* weights, int32_t num_tokens,
                    int32_t num_outputs, int32_t top, int32_t groups, int32_t keep, float scale, int32_t score_fn, int32_t normalise, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(logits && ids && weights && num_outputs > 0 && top > 0 && top <= num_outputs && ld >= num_outputs, kErrBadArg, "moe_route: bad arguments");
    B200_REQUIRE(groups <= 1 || (num_outputs % groups == 0 && keep > 0 && keep <= groups), kErrBadArg, "moe_route: %d outputs do not form %d equal groups (keep %d)",
                 num_outputs, groups, keep);
    B200_REQUIRE(num_outputs <= 8192, kErrUnsupported, "moe_route: more than 8192 router outputs");
    const size_t smem = ((size_t)(logit_bias ? 3 : 2) * num_outputs + (groups > 1 ? groups : 1)) * sizeof(float);
    ensure_dynamic_smem(reinterpret_cast<const void*>(moe_route_kernel), (int)smem);
    launch_pdl(moe_route_kernel, dim3(num_tokens), dim3(32), smem, as_stream(stream), logits, ld, correction, ids, weights, num_outputs, top, groups, keep, scale,
               score_fn, normalise, logit_bias);
    count_launch();
    check_launch("moe_route");
}

void moe_gate_up(const void* h, int64_t ldh, const void* w_gate_up, const int32_t* ids, const int32_t* order, void* act, int32_t num_tokens, int32_t top,
                 int32_t num_experts, int32_t ff, int32_t width, int32_t dtype, int64_t stream) {
    moe_gate_up_ex(h, ldh, w_gate_up, ids, order, act, num_tokens, top, num_experts, ff, width, 0, 0.f, nullptr, dtype, stream);
}

void moe_gate_up_ex(const void* h, int64_t ldh, const void* w_gate_up, const int32_t* ids, const int32_t* order, void* act, int32_t num_tokens, int32_t top,
                    int32_t num_experts, int32_t ff, int32_t width, int32_t act_fn, float limit, const float* pair_scale, int32_t dtype, int64_t stream) {
    if (num_tokens == 0 || num_experts == 0) return;
    B200_REQUIRE(act_fn == 0 || act_fn == 2 || act_fn == 3, kErrBadArg, "moe_gate_up: activation %d (0 = SiLU, 2 = clamped, 3 = ungated squared ReLU)", act_fn);
    B200_REQUIRE(h && w_gate_up && ids && act && top > 0 && ff > 0 && width > 0 && width <= 16384 && ldh >= width, kErrBadArg, "moe_gate_up: bad arguments");
    cudaStream_t st = as_stream(stream);
    const dim3 grid((unsigned)((int64_t)num_tokens * top), (unsigned)((ff + kGuRows - 1) / kGuRows));
    const size_t smem = (size_t)width * sizeof(float);
    ensure_dynamic_smem(reinterpret_cast<const void*>(moe_gate_up_kernel<float>), (int)smem);
    ensure_dynamic_smem(reinterpret_cast<const void*>(moe_gate_up_kernel<__nv_bfloat16>), (int)smem);
    if (dtype == B200_F32)
        launch_pdl(moe_gate_up_kernel<float>, grid, dim3(128), smem, st, (const float*)h, ldh, (const float*)w_gate_up, ids, order, (float*)act, top, num_experts, ff, width,
                   act_fn, limit, pair_scale);
    else if (dtype == B200_BF16)
        launch_pdl(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(128), smem, st, (const __nv_bfloat16*)h, ldh, (const __nv_bfloat16*)w_gate_up, ids, order,
                   (__nv_bfloat16*)act, top, num_experts, ff, width, act_fn, limit, pair_scale);
    else { set_error(kErrUnsupported, "moe_gate_up: dtype %d (f32 / bf16)", dtype); return; }
    count_launch();
    check_launch("moe_gate_up");
}

void moe_down(const void* act, const void* w_down, const int32_t* ids, const int32_t* order, float* y, int32_t rows, int32_t num_experts, int32_t ff, int32_t width,
              int32_t dtype, int64_t stream) {
    if (rows == 0 || num_experts == 0) return;
    B200_REQUIRE(act && w_down && ids && order && y && ff > 0 && ff <= 40960 && width > 0, kErrBadArg, "moe_down: bad arguments");
    cudaStream_t st = as_stream(stream);
    const size_t smem = (size_t)ff * sizeof(float);
    const dim3 grid(rows, (width + kDownCols - 1) / kDownCols);
    if (dtype == B200_F32) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(moe_down_kernel<float>), (int)smem);
        launch_pdl(moe_down_kernel<float>, grid, dim3(256), smem, st, (const float*)act, (const float*)w_down, ids, order, y, num_experts, ff, width);
    } else if (dtype == B200_BF16) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(moe_down_kernel<__nv_bfloat16>), (int)smem);
        launch_pdl(moe_down_kernel<__nv_bfloat16>, grid, dim3(256), smem, st, (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, ids, order, y, num_experts, ff,
                   width);
    } else { set_error(kErrUnsupported, "moe_down: dtype %d (f32 / bf16)", dtype); return; }
    count_launch();
    check_launch("moe_down");
}

int64_t moe_align_rows(int64_t pairs, int32_t num_experts, int32_t tile) {
    // every expert's run is padded to whole tiles: at most tile - 1 rows of padding each
    if (tile < 1) tile = 1;
    return (pairs + (int64_t)num_experts * (tile - 1) + tile - 1) / tile * tile;
}

void moe_align(const int32_t* ids, int32_t* pair_row, int32_t* row_pair, int32_t* tile_group, int32_t pairs, int32_t num_experts, int32_t max_rows, int32_t tile,
               int64_t stream) {
    if (pairs == 0) return;
    B200_REQUIRE(ids && pair_row && row_pair && (tile_group || tile == 1) && pairs > 0 && num_experts > 0 && num_experts <= 4096 && tile >= 1 &&
                 max_rows % tile == 0 && max_rows >= moe_align_rows(pairs, num_experts, tile), kErrBadArg, "moe_align: bad arguments");
    launch_pdl(moe_align_kernel, dim3(1), dim3(1024), (size_t)(3 * num_experts + 1) * sizeof(int), as_stream(stream), ids, pair_row, row_pair, tile_group, pairs,
               num_experts, max_rows, tile);
    count_launch();
    check_launch("moe_align");
}

void moe_gather_rows(const void* h, int64_t ldh, const int32_t* row_pair, void* xg, int32_t max_rows, int32_t top, int32_t width, int64_t stream) {
    if (max_rows == 0) return;
    B200_REQUIRE(h && row_pair && xg && top > 0 && width > 0 && ldh >= width, kErrBadArg, "moe_gather_rows: bad arguments");
    launch_pdl(moe_gather_rows_kernel, dim3(max_rows), dim3(128), 0, as_stream(stream), (const __nv_bfloat16*)h, ldh, row_pair, (__nv_bfloat16*)xg, top, width);
    count_launch();
    check_launch("moe_gather_rows");
}

void silu_mul_packed(const float* gate_up, void* out, int64_t rows, int32_t ff, int64_t ld, int32_t out_dtype, int64_t stream) {
    if (rows == 0 || ff == 0) return;
    B200_REQUIRE(gate_up && out && rows > 0 && ff > 0 && ld >= 2 * (int64_t)ff, kErrBadArg, "silu_mul_packed: bad arguments");
    const unsigned grid = (unsigned)((rows * ff + 255) / 256);
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32) launch_pdl(silu_mul_packed_kernel<float>, dim3(grid), dim3(256), 0, st, gate_up, (float*)out, rows, ff, ld);
    else if (out_dtype == B200_BF16) launch_pdl(silu_mul_packed_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, gate_up, (__nv_bfloat16*)out, rows, ff, ld);
    else { set_error(kErrUnsupported, "silu_mul_packed: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("silu_mul_packed");
}

void moe_combine_rows(const float* y, const int32_t* pair_row, const float* weights, const float* x, int64_t ldx, float* out, int32_t num_tokens, int32_t top,
                      int32_t width, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(y && pair_row && x && out && top > 0 && width > 0 && ldx >= width, kErrBadArg, "moe_combine_rows: bad arguments");
    launch_pdl(moe_combine_rows_kernel, dim3(num_tokens), dim3(256), 0, as_stream(stream), y, pair_row, weights, x, ldx, out, top, width);
    count_launch();
    check_launch("moe_combine_rows");
}

}  // extern "C"
