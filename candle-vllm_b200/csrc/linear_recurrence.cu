// linear_recurrence.cu -- sequence mixers whose memory is a fixed-size f32 state per sequence, for ragged steps (portions of prompts
// beside single decoded tokens in one launch).  Entry b's rows continue the sequence whose state sits in slot seq_slots[b];
// seq_start[b] == 0 means "new sequence": what the slot holds is ignored (taken as zero), so a slot is never cleared.
//
//   causal_conv_ex        y[t, c] = act(sum_j taps[c, j] * in[t - K + 1 + j, c] + out_bias[c]) (+ in[t, c]), in = x + in_bias, zeros before
//                         the sequence's start; the K - 1 inputs before a portion come from conv_state [slots, K-1, C], which is then
//                         rolled forward over the portion.  act = none or SiLU; the "+ in" form is a convolution added to its own input.
//   block_diag_linear     out[t, b M + j] = sum_i w[b, j, i] x[t, b N + i] + bias[b M + j]: one matrix per block of N neighbouring
//                         channels, true 32-bit products (the gates of a recurrence).
//   gated_linear_scan     per channel  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t,  a_t = exp(-c r_t softplus(lam)),  r, i = sigmoid of
//                         the block-diagonal products;  out_t = S_t * gelu_tanh(y_t + y_bias).  One kernel for steps of few rows per entry;
//                         for portions of prompts a row-parallel pass first turns gates and y into a_t, the input term and the GELU (in place);
//                         from 512 rows per entry the bare scan that follows runs over chunks of 128 rows, all chunks at once.
//   linear_attention      per head, S [dk, dv]:  S_t = a_t S_(t-1) + b_t k_t v_t^T,  o_t = S_t^T q_t, in two gatings:
//                           fixed decay      a = decay[h], b = 1;
//                           exponential      a_t = e^(f_t + m_(t-1) - m_t), b_t = e^(i_t - m_t) with the running maximum m_t = max(f_t + m_(t-1), i_t),
//                                            m_0 = 0, i = cap tanh(. / cap), f = logsigmoid(cap tanh(. / cap)); a normaliser n_t = a_t n_(t-1) + b_t k_t
//                                            rides along and o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6).  n and m are stored once per
//                                            block of 16 value columns, so that no block reads what another one writes.
//                         A block of four warps owns 16 value columns of one head of one entry; inside a warp the key rows are split eight
//                         ways (lane = 4 * part + column) with the lane's rows of S (and of n) in registers; tokens come in tiles of 16
//                         staged through shared memory with the activation already applied, the per-token coefficients worked out once
//                         per tile (the chain of maxima by one lane, the exponentials by sixteen).  Every sum has a fixed order, so
//                         portions of any size leave the same state bit for bit.  State S is stored [slot, head, column, row].
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    const float c = 0.7978845608028654f;       // sqrt(2 / pi)
    return 0.5f * z * (1.0f + tanhf(c * (z + 0.044715f * z * z * z)));
}

template <typename TOut>
__global__ void __launch_bounds__(128)
causal_conv_ex_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ in_bias, const float* __restrict__ taps,
                      const float* __restrict__ out_bias, const float* __restrict__ conv_state, TOut* __restrict__ y, int64_t ldy,
                      const int32_t* __restrict__ token_seq, const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots,
                      const int32_t* __restrict__ seq_start, int C, int K, int act, int add_input) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= C) return;
    const int b = token_seq[t];
    const int i = t - cu_seqlens[b];
    const bool fresh = seq_start[b] == 0;
    const float* st = conv_state + (int64_t)seq_slots[b] * (K > 1 ? K - 1 : 1) * C;
    const float ib = in_bias ? in_bias[c] : 0.f;
    float acc = 0.f, cur = 0.f;
    for (int d = K - 1; d >= 0; --d) {            // oldest input first
        const int src = i - d;
        float v;
        if (src >= 0) v = x[(int64_t)(t - d) * ldx + c] + ib;
        else v = fresh ? 0.f : st[(int64_t)(K - 1 + src) * C + c];
        if (d == 0) cur = v;
        acc = fmaf(taps[(int64_t)c * K + (K - 1 - d)], v, acc);
    }
    if (out_bias) acc += out_bias[c];
    if (act == 1) acc = silu_f(acc);
    if (add_input) acc += cur;
    y[(int64_t)t * ldy + c] = from_f32<TOut>(acc);
}

__global__ void __launch_bounds__(128)
causal_conv_roll_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ in_bias, float* __restrict__ conv_state,
                        const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int C, int K) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (n <= 0) return;
    const bool fresh = seq_start[b] == 0;
    const float ib = in_bias ? in_bias[c] : 0.f;
    float* st = conv_state + (int64_t)seq_slots[b] * (K - 1) * C;
    // the sequence's inputs so far are [old state rows 0 .. K-2][portion rows 0 .. n-1]; the last K-1 of them stay.  Row j of the new
    // state is element n + j of that list: j ascends and n >= 1, so an old row is read before it is overwritten.
    for (int j = 0; j < K - 1; ++j) {
        const int e = n + j;
        float v;
        if (e >= K - 1) v = x[(int64_t)(t0 + e - (K - 1)) * ldx + c] + ib;
        else v = fresh ? 0.f : st[(int64_t)e * C + c];
        st[(int64_t)j * C + c] = v;
    }
}

// Steps in which every entry brings one row: the convolution and the roll of the state in one kernel (a thread owns its channel's state column)
template <typename TOut>
__global__ void __launch_bounds__(128)
causal_conv_step_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ in_bias, const float* __restrict__ taps,
                        const float* __restrict__ out_bias, float* __restrict__ conv_state, TOut* __restrict__ y, int64_t ldy,
                        const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int C, int K, int act, int add_input) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const bool fresh = seq_start[b] == 0;
    float* st = conv_state + (int64_t)seq_slots[b] * (K > 1 ? K - 1 : 1) * C;
    const float cur = x[(int64_t)b * ldx + c] + (in_bias ? in_bias[c] : 0.f);
    float acc = 0.f;
    for (int j = 0; j < K - 1; ++j) {             // oldest input first; row j moves to row j - 1
        const float v = fresh ? 0.f : st[(int64_t)j * C + c];
        acc = fmaf(taps[(int64_t)c * K + j], v, acc);
        if (j > 0) st[(int64_t)(j - 1) * C + c] = v;
    }
    if (K > 1) st[(int64_t)(K - 2) * C + c] = cur;
    acc = fmaf(taps[(int64_t)c * K + K - 1], cur, acc);
    if (out_bias) acc += out_bias[c];
    if (act == 1) acc = silu_f(acc);
    if (add_input) acc += cur;
    y[(int64_t)b * ldy + c] = from_f32<TOut>(acc);
}

// ---- block-diagonal f32 product ---------------------------------------------------------------------------------------------------
constexpr int kBM = 64, kBN = 64, kBK = 16;

__global__ void __launch_bounds__(256)
block_diag_linear_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ y,
                         int64_t ldy, int T, int M, int N) {
    pdl_wait();
    pdl_trigger();
    __shared__ float xs[kBK][kBM + 4], ws[kBK][kBN + 4];
    const int blk = blockIdx.z;
    const float* xb = x + (int64_t)blk * N;
    const float* wb = w + (int64_t)blk * M * N;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * kBM, col0 = blockIdx.x * kBN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < N; k0 += kBK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256, r = idx >> 4, c = idx & 15;
            const int gr = row0 + r, gc = k0 + c, wr = col0 + r;
            xs[c][r] = (gr < T && gc < N) ? xb[(int64_t)gr * ldx + gc] : 0.f;
            ws[c][r] = (wr < M && gc < N) ? wb[(int64_t)wr * N + gc] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = xs[kk][ty * 4 + i]; b[i] = ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < M) y[(int64_t)gr * ldy + (int64_t)blk * M + gc] = acc[i][j] + (bias ? bias[(int64_t)blk * M + gc] : 0.f);
        }
    }
}

// few rows: a warp owns one output column of one block and up to 4 rows, lanes stride the block's inputs
__global__ void __launch_bounds__(256)
block_diag_rows_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ y,
                       int64_t ldy, int T, int M, int N) {
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.z;
    const int col = blockIdx.x * 8 + warp;
    const int r0 = blockIdx.y * 4;
    if (col >= M) return;
    const float* wr = w + ((int64_t)blk * M + col) * N;
    const float* xb = x + (int64_t)blk * N;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = lane; i < N; i += 32) {
        const float wv = wr[i];
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r0 + r < T) acc[r] = fmaf(xb[(int64_t)(r0 + r) * ldx + i], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float s = warp_sum(acc[r]);
        if (lane == 0 && r0 + r < T) y[(int64_t)(r0 + r) * ldy + (int64_t)blk * M + col] = s + (bias ? bias[(int64_t)blk * M + col] : 0.f);
    }
}

// ---- the gated scan ------------------------------------------------------------------------------------------------------------------
// One thread per (entry, channel); the next rows' operands are fetched while the current row is applied.  gates f32 [T, blocks, 2 n]: per
// block the recurrence gate's pre-activations, then the input gate's.
template <typename TOut>
__global__ void __launch_bounds__(64)
gated_linear_scan_kernel(const float* __restrict__ u, int64_t ldu, const float* __restrict__ gates, int64_t ldg, const float* __restrict__ lam,
                         const float* __restrict__ ypre, int64_t ldy, const float* __restrict__ y_bias, float* __restrict__ state, TOut* __restrict__ out,
                         const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int C, int n,
                         float decay_scale) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 64 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    if (t1 <= t0) return;
    float* sp = state + (int64_t)seq_slots[b] * C + c;
    float S = seq_start[b] == 0 ? 0.f : *sp;
    const float k = -decay_scale * softplus_f(lam[c]);
    const float yb = y_bias ? y_bias[c] : 0.f;
    const int blk = c / n, j = c - blk * n;
    const int rc = blk * 2 * n + j, ic = rc + n;
    constexpr int kAhead = 4;
    float gr[kAhead], gi[kAhead], uu[kAhead], yy[kAhead];
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
        const int t = min(t0 + a, t1 - 1);
        gr[a] = gates[(int64_t)t * ldg + rc]; gi[a] = gates[(int64_t)t * ldg + ic]; uu[a] = u[(int64_t)t * ldu + c]; yy[a] = ypre[(int64_t)t * ldy + c];
    }
    for (int tb = t0; tb < t1; tb += kAhead) {
        float cr[kAhead], ci[kAhead], cu[kAhead], cy[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) { cr[a] = gr[a]; ci[a] = gi[a]; cu[a] = uu[a]; cy[a] = yy[a]; }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int t = min(tb + kAhead + a, t1 - 1);
            gr[a] = gates[(int64_t)t * ldg + rc]; gi[a] = gates[(int64_t)t * ldg + ic]; uu[a] = u[(int64_t)t * ldu + c]; yy[a] = ypre[(int64_t)t * ldy + c];
        }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            if (tb + a >= t1) break;
            const float la = k * sigmoid_f(cr[a]);                     // log a_t <= 0
            const float at = expf(la);
            const float mult = sqrtf(-expm1f(2.0f * la));               // sqrt(1 - a^2) without cancellation near a = 1
            S = fmaf(at, S, mult * sigmoid_f(ci[a]) * cu[a]);
            out[(int64_t)(tb + a) * C + c] = from_f32<TOut>(S * gelu_tanh_f(cy[a] + yb));
        }
    }
    *sp = S;
}

// Portions of prompts: the per-token part (two sigmoids, the decay and its square-root complement, the GELU of the other branch) is done for all
// rows at once, in place -- gates[t, blk, j] <- a_t, gates[t, blk, n + j] <- sqrt(1 - a_t^2) i_t u_t, y[t, c] <- gelu_tanh(y + bias) -- and the scan
// itself is two multiply-adds per row with the next rows' operands in flight.
__global__ void gated_scan_prepare_kernel(const float* __restrict__ u, int64_t ldu, float* __restrict__ gates, int64_t ldg, const float* __restrict__ lam,
                                          float* __restrict__ y, int64_t ldy, const float* __restrict__ y_bias, int64_t rows, int C, int n, float decay_scale) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const int64_t t = i / C;
    const int c = (int)(i - t * C);
    const int blk = c / n, j = c - blk * n;
    float* gr = gates + t * ldg + blk * 2 * n + j;
    const float la = -decay_scale * softplus_f(lam[c]) * sigmoid_f(gr[0]);
    const float b = sqrtf(-expm1f(2.0f * la)) * sigmoid_f(gr[n]) * u[t * ldu + c];
    gr[0] = expf(la);
    gr[n] = b;
    y[t * ldy + c] = gelu_tanh_f(y[t * ldy + c] + (y_bias ? y_bias[c] : 0.f));
}

template <typename TOut>
__global__ void __launch_bounds__(32)
linear_scan_kernel(const float* __restrict__ gates, int64_t ldg, const float* __restrict__ y, int64_t ldy, float* __restrict__ state, TOut* __restrict__ out,
                   const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int C, int n) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 32 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    if (t1 <= t0) return;
    float* sp = state + (int64_t)seq_slots[b] * C + c;
    float S = seq_start[b] == 0 ? 0.f : *sp;
    const int blk = c / n, j = c - blk * n;
    const float* ga = gates + blk * 2 * n + j;
    constexpr int kAhead = 16;
    float na[kAhead], nb[kAhead], ny[kAhead];
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
        const int64_t t = min(t0 + a, t1 - 1);
        na[a] = ga[t * ldg]; nb[a] = ga[t * ldg + n]; ny[a] = y[t * ldy + c];
    }
    for (int tb = t0; tb < t1; tb += kAhead) {
        float ca[kAhead], cb[kAhead], cy[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) { ca[a] = na[a]; cb[a] = nb[a]; cy[a] = ny[a]; }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int64_t t = min(tb + kAhead + a, t1 - 1);
            na[a] = ga[t * ldg]; nb[a] = ga[t * ldg + n]; ny[a] = y[t * ldy + c];
        }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            if (tb + a >= t1) break;
            S = fmaf(ca[a], S, cb[a]);
            out[(int64_t)(tb + a) * C + c] = from_f32<TOut>(S * cy[a]);
        }
    }
    *sp = S;
}

// Long portions: the bare scan cut into chunks of 128 rows, all chunks at once.  A chunk's rows compose to S_out = P S_in + Q with P the product of
// its a_t and Q its own scan from zero: one kernel takes (P, Q) of every chunk, one walks an entry's chunks per channel and leaves every chunk's S_in,
// one replays every chunk from its S_in and writes the outputs.  The association of the sums differs from the row-by-row scan by rounding only.
constexpr int kScanChunk = 128;

__device__ __forceinline__ int scan_chunk_base(const int32_t* cu, int b) {
    int s = 0;
    for (int i = 0; i < b; ++i) s += (cu[i + 1] - cu[i] + kScanChunk - 1) / kScanChunk;
    return s;
}

__global__ void __launch_bounds__(128)
scan_chunk_compose_kernel(const float* __restrict__ gates, int64_t ldg, float* __restrict__ pq, const int32_t* __restrict__ cu_seqlens, int C, int n) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 128 + threadIdx.x, ch = blockIdx.y, b = blockIdx.z;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], rows = cu_seqlens[b + 1] - t0;
    if (ch * kScanChunk >= rows) return;
    const int tf = t0 + ch * kScanChunk, nt = min(kScanChunk, rows - ch * kScanChunk);
    const int blk = c / n, j = c - blk * n;
    const float* ga = gates + (int64_t)tf * ldg + blk * 2 * n + j;
    float P = 1.f, Q = 0.f;
#pragma unroll 8
    for (int t = 0; t < nt; ++t) {
        const float a = ga[(int64_t)t * ldg], bb = ga[(int64_t)t * ldg + n];
        Q = fmaf(a, Q, bb);
        P *= a;
    }
    const int64_t at = ((int64_t)(scan_chunk_base(cu_seqlens, b) + ch) * C + c) * 2;
    pq[at] = P; pq[at + 1] = Q;
}

__global__ void __launch_bounds__(128)
scan_chunk_carry_kernel(float* __restrict__ pq, float* __restrict__ state, const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots,
                        const int32_t* __restrict__ seq_start, int C) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
    if (c >= C) return;
    const int rows = cu_seqlens[b + 1] - cu_seqlens[b];
    if (rows <= 0) return;
    const int nc = (rows + kScanChunk - 1) / kScanChunk;
    float* sp = state + (int64_t)seq_slots[b] * C + c;
    float S = seq_start[b] == 0 ? 0.f : *sp;
    float2* p0 = reinterpret_cast<float2*>(pq) + (int64_t)scan_chunk_base(cu_seqlens, b) * C + c;
    constexpr int kAhead = 8;
    float2 nx[kAhead];
#pragma unroll
    for (int a = 0; a < kAhead; ++a) nx[a] = p0[(int64_t)min(a, nc - 1) * C];
    for (int cb = 0; cb < nc; cb += kAhead) {
        float2 cur[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) cur[a] = nx[a];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) nx[a] = p0[(int64_t)min(cb + kAhead + a, nc - 1) * C];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            if (cb + a >= nc) break;
            p0[(int64_t)(cb + a) * C].y = S;                 // the state that enters the chunk
            S = fmaf(cur[a].x, S, cur[a].y);
        }
    }
    *sp = S;
}

template <typename TOut>
__global__ void __launch_bounds__(128)
scan_chunk_replay_kernel(const float* __restrict__ gates, int64_t ldg, const float* __restrict__ y, int64_t ldy, const float* __restrict__ pq, TOut* __restrict__ out,
                         const int32_t* __restrict__ cu_seqlens, int C, int n) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * 128 + threadIdx.x, ch = blockIdx.y, b = blockIdx.z;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], rows = cu_seqlens[b + 1] - t0;
    if (ch * kScanChunk >= rows) return;
    const int tf = t0 + ch * kScanChunk, nt = min(kScanChunk, rows - ch * kScanChunk);
    const int blk = c / n, j = c - blk * n;
    const float* ga = gates + (int64_t)tf * ldg + blk * 2 * n + j;
    const float* yp = y + (int64_t)tf * ldy + c;
    TOut* op = out + (int64_t)tf * C + c;
    float S = pq[((int64_t)(scan_chunk_base(cu_seqlens, b) + ch) * C + c) * 2 + 1];
#pragma unroll 8
    for (int t = 0; t < nt; ++t) {
        S = fmaf(ga[(int64_t)t * ldg], S, ga[(int64_t)t * ldg + n]);
        op[(int64_t)t * C] = from_f32<TOut>(S * yp[(int64_t)t * ldy]);
    }
}

// ---- linear attention with a matrix state ---------------------------------------------------------------------------------------------
constexpr int kTile = 16;
constexpr int kScanChunkedRows = 512;    // entries with at least this many rows (and a scratch buffer): the bare scan runs over chunks of 128 rows, all at once
constexpr int kScanSplitRows = 16;     // entries with at least this many rows: the gated scan runs as a row-parallel pass plus a bare scan

struct LinAttnArgs {
    const float* proj; int64_t ld;
    int off_q, off_k, off_v, off_i, off_f;      // columns of proj: q, k [H dk], v [H dv], gate pre-activations [H] (exponential gating only)
    const float* decay;                          // [H] (fixed decay)
    const float* i_bias; const float* f_bias;    // [H]
    float cap, q_scale; int act;
    float* S; float* nrm; float* mx;             // [slots, H, dv, dk], [slots, H, ceil(dv / 16), dk], [slots, H, ceil(dv / 16)]
    float* out;                                  // [T, H dv]
    const int32_t* cu_seqlens; const int32_t* seq_slots; const int32_t* seq_start;
    int H, dk, dv;
};

template <int kR, bool kExp>
__global__ void __launch_bounds__(128)
linear_attention_kernel(const LinAttnArgs A) {
    pdl_wait();
    pdl_trigger();
    constexpr int kP = 8 * kR;                   // padded key rows
    extern __shared__ __align__(16) float smem[];
    float* sq = smem;                            // [kTile][kP]
    float* sk = sq + kTile * kP;                 // [kTile][kP]
    float* sv = sk + kTile * kP;                 // [kTile][16]
    float* sa = sv + kTile * 16;                 // [kTile] decay of the state
    float* sb = sa + kTile;                      // [kTile] weight of the new outer product
    float* se = sb + kTile;                      // [kTile] e^(-m_t)
    float* sf = se + kTile;                      // [kTile] f_t
    float* si = sf + kTile;                      // [kTile] i_t
    float* sm = si + kTile;                      // [kTile + 1] m before the tile's first token, then m_t
    const int h = blockIdx.y, b = blockIdx.z;
    const int H = A.H, dk = A.dk, dv = A.dv;
    const int t0 = A.cu_seqlens[b], t1 = A.cu_seqlens[b + 1];
    if (t1 <= t0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int part = lane >> 2, cl = lane & 3;
    const int colb = warp * 4 + cl;              // column inside the block's 16
    const int col = blockIdx.x * 16 + colb;
    const bool col_ok = col < dv;
    const bool fresh = A.seq_start[b] == 0;
    const int64_t slot = A.seq_slots[b];
    const bool vec = (dk & 3) == 0;              // a lane's rows of the state are then whole 16-byte words
    float* Sp = A.S + ((slot * H + h) * dv + (col_ok ? col : 0)) * (int64_t)dk + part * kR;
    // the normaliser and the maximum are kept once per block of 16 columns: every block reads and writes a copy of its own
    const int64_t own = (slot * H + h) * (int64_t)gridDim.x + blockIdx.x;
    float* np = kExp ? A.nrm + own * dk + part * kR : nullptr;
    float S[kR], nv[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) { S[r] = 0.f; nv[r] = 0.f; }
    if (!fresh) {
        if (vec) {
#pragma unroll
            for (int r4 = 0; r4 < kR / 4; ++r4) {
                if (part * kR + r4 * 4 >= dk) continue;
                if (col_ok) { const float4 v = reinterpret_cast<const float4*>(Sp)[r4]; S[r4 * 4] = v.x; S[r4 * 4 + 1] = v.y; S[r4 * 4 + 2] = v.z; S[r4 * 4 + 3] = v.w; }
                if (kExp) { const float4 v = reinterpret_cast<const float4*>(np)[r4]; nv[r4 * 4] = v.x; nv[r4 * 4 + 1] = v.y; nv[r4 * 4 + 2] = v.z; nv[r4 * 4 + 3] = v.w; }
            }
        } else {
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                const bool ok = part * kR + r < dk;
                if (col_ok && ok) S[r] = Sp[r];
                if (kExp && ok) nv[r] = np[r];
            }
        }
    }
    if (kExp && threadIdx.x == 0) sm[0] = fresh ? 0.f : A.mx[own];
    const float fixed_a = kExp ? 0.f : A.decay[h];
    // the next tile's operands travel in registers while the current tile is walked: element e = thread + 128 i of the tile's [16][kP] q and k
    // rows, two of its [16][16] values, and (lanes 0..15 of the last warp) the two gate pre-activations of a token
    float pq[kR], pk[kR], pv[2], pgi = 0.f, pgf = 0.f;
    auto fetch = [&](int tb) {
        const int nt = min(kTile, t1 - tb);
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            const int e = threadIdx.x + 128 * i, tt = e / kP, r = e - tt * kP;
            const bool ok = tt < nt && r < dk;
            const float* row = A.proj + (int64_t)(tb + (ok ? tt : 0)) * A.ld;
            pq[i] = ok ? row[A.off_q + h * dk + r] : 0.f;
            pk[i] = ok ? row[A.off_k + h * dk + r] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int e = threadIdx.x + 128 * i, tt = e >> 4, gc = blockIdx.x * 16 + (e & 15);
            pv[i] = (tt < nt && gc < dv) ? A.proj[(int64_t)(tb + tt) * A.ld + A.off_v + h * dv + gc] : 0.f;
        }
        if (kExp && warp == 3 && lane < nt) {
            const float* row = A.proj + (int64_t)(tb + lane) * A.ld;
            pgi = row[A.off_i + h] + (A.i_bias ? A.i_bias[h] : 0.f);
            pgf = row[A.off_f + h] + (A.f_bias ? A.f_bias[h] : 0.f);
        }
    };
    fetch(t0);
    for (int tb = t0; tb < t1; tb += kTile) {
        const int nt = min(kTile, t1 - tb);
        __syncthreads();                         // the previous tile has been walked
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            const int e = threadIdx.x + 128 * i;
            float qv = pq[i], kv = pk[i];
            if (A.act == 1) { qv = silu_f(qv); kv = silu_f(kv); }
            sq[e] = qv * A.q_scale; sk[e] = kv;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) sv[threadIdx.x + 128 * i] = A.act == 1 ? silu_f(pv[i]) : pv[i];
        if (kExp && warp == 3) {
            // gate values of the tile's tokens, the chain of maxima, then the coefficients
            if (lane < nt) {
                si[lane] = A.cap * tanhf(pgi / A.cap);
                sf[lane] = log_sigmoid_f(A.cap * tanhf(pgf / A.cap));
            }
            __syncwarp();
            if (lane == 0) {
                float m = sm[0];
                for (int tt = 0; tt < nt; ++tt) { m = fmaxf(sf[tt] + m, si[tt]); sm[tt + 1] = m; }
            }
            __syncwarp();
            if (lane < nt) {
                const float m_prev = sm[lane], m_new = sm[lane + 1];
                sa[lane] = expf(sf[lane] + m_prev - m_new);
                sb[lane] = expf(si[lane] - m_new);
                se[lane] = expf(-m_new);
            }
        }
        __syncthreads();
        if (tb + kTile < t1) fetch(tb + kTile);
        // the tile's tokens one after the other; every token leaves a partial sum per lane, and the butterflies that join the eight parts run
        // afterwards for all tokens together (sixteen independent chains instead of one per token on the serial path)
        float osum[kTile], nsum[kTile];
#pragma unroll
        for (int tt = 0; tt < kTile; ++tt) {
            osum[tt] = 0.f; nsum[tt] = 0.f;
            if (tt >= nt) continue;
            const float a = kExp ? sa[tt] : fixed_a;
            const float bv = (kExp ? sb[tt] : 1.0f) * sv[tt * 16 + colb];
            const float bn = kExp ? sb[tt] : 0.f;
            float acc[2] = {0.f, 0.f}, nq[2] = {0.f, 0.f};
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * kP + part * kR);
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * kP + part * kR);
#pragma unroll
            for (int r4 = 0; r4 < kR / 4; ++r4) {
                const float4 qq = q4[r4], kk = k4[r4];
                const float qa[4] = {qq.x, qq.y, qq.z, qq.w}, ka[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = r4 * 4 + j;
                    S[r] = fmaf(a, S[r], ka[j] * bv);
                    acc[j & 1] = fmaf(S[r], qa[j], acc[j & 1]);
                    if (kExp) { nv[r] = fmaf(a, nv[r], ka[j] * bn); nq[j & 1] = fmaf(nv[r], qa[j], nq[j & 1]); }
                }
            }
            osum[tt] = acc[0] + acc[1];
            if (kExp) nsum[tt] = nq[0] + nq[1];
        }
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
#pragma unroll
            for (int tt = 0; tt < kTile; ++tt) {
                osum[tt] += __shfl_xor_sync(0xffffffffu, osum[tt], sh);
                if (kExp) nsum[tt] += __shfl_xor_sync(0xffffffffu, nsum[tt], sh);
            }
        }
        if (part == 0 && col_ok) {
#pragma unroll
            for (int tt = 0; tt < kTile; ++tt) {
                if (tt >= nt) continue;
                float o = osum[tt];
                if (kExp) o = o / (fmaxf(fabsf(nsum[tt]), se[tt]) + 1e-6f);
                A.out[(int64_t)(tb + tt) * H * dv + h * dv + col] = o;
            }
        }
        if (kExp) {
            __syncthreads();
            if (threadIdx.x == 0) sm[0] = sm[nt];
        }
    }
    if (vec) {
#pragma unroll
        for (int r4 = 0; r4 < kR / 4; ++r4) {
            if (part * kR + r4 * 4 >= dk) continue;
            if (col_ok) reinterpret_cast<float4*>(Sp)[r4] = make_float4(S[r4 * 4], S[r4 * 4 + 1], S[r4 * 4 + 2], S[r4 * 4 + 3]);
            if (kExp && warp == 0 && cl == 0) reinterpret_cast<float4*>(np)[r4] = make_float4(nv[r4 * 4], nv[r4 * 4 + 1], nv[r4 * 4 + 2], nv[r4 * 4 + 3]);
        }
    } else {
#pragma unroll
        for (int r = 0; r < kR; ++r) {
            const bool ok = part * kR + r < dk;
            if (col_ok && ok) Sp[r] = S[r];
            if (kExp && ok && warp == 0 && cl == 0) np[r] = nv[r];
        }
    }
    if (kExp) {
        __syncthreads();
        if (threadIdx.x == 0) A.mx[own] = sm[0];
    }
}

// Steps in which every entry brings one token (row b belongs to entry b): nothing is staged and no thread waits for another -- a lane reads its
// own rows of q and k, its column's value and (exponential gating) the two gate values straight from the projection, takes one pass over its
// rows of the state and writes them back.  Same lane layout and state layout as the kernel above.
template <int kR, bool kExp>
__global__ void __launch_bounds__(128)
linear_attention_step_kernel(const LinAttnArgs A) {
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.y, b = blockIdx.z;
    const int H = A.H, dk = A.dk, dv = A.dv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int part = lane >> 2, cl = lane & 3;
    const int col = blockIdx.x * 16 + warp * 4 + cl;
    const bool col_ok = col < dv;
    const bool fresh = A.seq_start[b] == 0;
    const int64_t slot = A.seq_slots[b];
    const bool vec = (dk & 3) == 0;
    float* Sp = A.S + ((slot * H + h) * dv + (col_ok ? col : 0)) * (int64_t)dk + part * kR;
    const int64_t own = (slot * H + h) * (int64_t)gridDim.x + blockIdx.x;
    float* np = kExp ? A.nrm + own * dk + part * kR : nullptr;
    const float* row = A.proj + (int64_t)b * A.ld;
    float S[kR], nv[kR], q[kR], k[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) {
        const int g = part * kR + r;
        const bool ok = g < dk;
        S[r] = 0.f; nv[r] = 0.f;
        q[r] = ok ? row[A.off_q + h * dk + g] : 0.f;
        k[r] = ok ? row[A.off_k + h * dk + g] : 0.f;
    }
    float v = col_ok ? row[A.off_v + h * dv + col] : 0.f;
    float zi = 0.f, zf = 0.f, m_prev = 0.f;
    if (kExp) {
        zi = row[A.off_i + h] + (A.i_bias ? A.i_bias[h] : 0.f);
        zf = row[A.off_f + h] + (A.f_bias ? A.f_bias[h] : 0.f);
        if (!fresh) m_prev = A.mx[own];
    }
    if (!fresh) {
        if (vec) {
#pragma unroll
            for (int r4 = 0; r4 < kR / 4; ++r4) {
                if (part * kR + r4 * 4 >= dk) continue;
                if (col_ok) { const float4 t = reinterpret_cast<const float4*>(Sp)[r4]; S[r4 * 4] = t.x; S[r4 * 4 + 1] = t.y; S[r4 * 4 + 2] = t.z; S[r4 * 4 + 3] = t.w; }
                if (kExp) { const float4 t = reinterpret_cast<const float4*>(np)[r4]; nv[r4 * 4] = t.x; nv[r4 * 4 + 1] = t.y; nv[r4 * 4 + 2] = t.z; nv[r4 * 4 + 3] = t.w; }
            }
        } else {
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                const bool ok = part * kR + r < dk;
                if (col_ok && ok) S[r] = Sp[r];
                if (kExp && ok) nv[r] = np[r];
            }
        }
    }
    float a = kExp ? 0.f : A.decay[h], bw = 1.0f, em = 0.f, m_new = 0.f;
    if (kExp) {
        const float gi = A.cap * tanhf(zi / A.cap), gf = log_sigmoid_f(A.cap * tanhf(zf / A.cap));
        m_new = fmaxf(gf + m_prev, gi);
        a = expf(gf + m_prev - m_new); bw = expf(gi - m_new); em = expf(-m_new);
    }
    if (A.act == 1) v = silu_f(v);
    const float bv = bw * v;
    float acc[2] = {0.f, 0.f}, nq[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kR; ++r) {
        float qv = q[r], kv = k[r];
        if (A.act == 1) { qv = silu_f(qv); kv = silu_f(kv); }
        qv *= A.q_scale;
        S[r] = fmaf(a, S[r], kv * bv);
        acc[r & 1] = fmaf(S[r], qv, acc[r & 1]);
        if (kExp) { nv[r] = fmaf(a, nv[r], kv * bw); nq[r & 1] = fmaf(nv[r], qv, nq[r & 1]); }
    }
    float o = acc[0] + acc[1], nqs = nq[0] + nq[1];
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
        o += __shfl_xor_sync(0xffffffffu, o, sh);
        if (kExp) nqs += __shfl_xor_sync(0xffffffffu, nqs, sh);
    }
    if (part == 0 && col_ok) {
        if (kExp) o = o / (fmaxf(fabsf(nqs), em) + 1e-6f);
        A.out[(int64_t)b * H * dv + h * dv + col] = o;
    }
    if (vec) {
#pragma unroll
        for (int r4 = 0; r4 < kR / 4; ++r4) {
            if (part * kR + r4 * 4 >= dk) continue;
            if (col_ok) reinterpret_cast<float4*>(Sp)[r4] = make_float4(S[r4 * 4], S[r4 * 4 + 1], S[r4 * 4 + 2], S[r4 * 4 + 3]);
            if (kExp && warp == 0 && cl == 0) reinterpret_cast<float4*>(np)[r4] = make_float4(nv[r4 * 4], nv[r4 * 4 + 1], nv[r4 * 4 + 2], nv[r4 * 4 + 3]);
        }
    } else {
#pragma unroll
        for (int r = 0; r < kR; ++r) {
            const bool ok = part * kR + r < dk;
            if (col_ok && ok) Sp[r] = S[r];
            if (kExp && ok && warp == 0 && cl == 0) np[r] = nv[r];
        }
    }
    if (kExp && threadIdx.x == 0) A.mx[own] = m_new;
}

// ---- portions of prompts: the same recurrence over chunks of 64 tokens, all chunks at once -----------------------------------------------------
// With F_t the sum of the log decays from the chunk's first token to t, li_t the log input weight and m_t the running maximum (F_t = (t + 1) ln decay,
// li = 0, m = 0 for a fixed decay), token t of a chunk that is entered with the (stabilised) state S_in and maximum m_in returns
//     o_t = e^(F_t + m_in - m_t) S_in^T q_t + sum_{j <= t} e^(F_t - F_j + li_j - m_t) (q_t . k_j) v_j
// and the chunk leaves  S_out = e^(F_L + m_in - m_L) S_in + sum_j e^(F_L - F_j + li_j - m_L) k_j v_j^T  (the normaliser alike, with k_j alone).  So:
//   la_gate_values   (exponential gating) log gates of every token, all rows at once;
//   la_gate_chain    per (entry, head) the chain of maxima m_t, exactly as the token-by-token kernel takes it, and F_t;
//   la_chunk_state   per chunk the second term of S_out, a [dv, dk] product over the chunk's tokens, all chunks at once;
//   la_chunk_scan    per state element the walk over an entry's chunks that turns those terms into the state entering every chunk (in place);
//   la_chunk_output  per chunk the two terms of o_t: scores against the chunk's own keys, then values and entering state in one accumulation.
// All arithmetic is f32 on the FMA pipe; the results differ from the token-by-token kernel by rounding only.
constexpr int kChunk = 64;

struct ChunkArgs {
    LinAttnArgs A;
    float* gc;            // [T, H, 3]: F_t, li_t, m_t (exponential gating)
    float* U;             // [chunk slots, H, dv, dk]
    float* un;            // [chunk slots, H, dk] a chunk's own term of the normaliser
    float* un_in;         // [chunk slots, H, dk] the normaliser that enters the chunk
    float* m0;            // [entries, H] the maximum every entry starts this step with (the slot's copy changes while the kernels run)
    int max_chunks;       // the most chunks any entry has
    int gating;
};

__device__ __forceinline__ int chunk_base(const int32_t* cu, int b) {      // chunk slots of the entries before b
    int s = 0;
    for (int i = 0; i < b; ++i) s += (cu[i + 1] - cu[i] + kChunk - 1) / kChunk;
    return s;
}
__device__ __forceinline__ float log_decay(float d) { return fmaxf(logf(d), -80.f); }

__global__ void la_gate_values_kernel(const ChunkArgs C, int T) {
    pdl_wait();
    pdl_trigger();
    const LinAttnArgs& A = C.A;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * A.H) return;
    const int t = i / A.H, h = i - t * A.H;
    const float* row = A.proj + (int64_t)t * A.ld;
    const float zi = row[A.off_i + h] + (A.i_bias ? A.i_bias[h] : 0.f), zf = row[A.off_f + h] + (A.f_bias ? A.f_bias[h] : 0.f);
    C.gc[(int64_t)i * 3 + 1] = A.cap * tanhf(zi / A.cap);
    C.gc[(int64_t)i * 3 + 0] = log_sigmoid_f(A.cap * tanhf(zf / A.cap));
}

__global__ void la_gate_chain_kernel(const ChunkArgs C) {
    pdl_wait();
    pdl_trigger();
    const LinAttnArgs& A = C.A;
    const int h = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (h >= A.H) return;
    const int t0 = A.cu_seqlens[b], t1 = A.cu_seqlens[b + 1];
    if (t1 <= t0) return;
    const int nvb = (A.dv + 15) / 16;
    float m = A.seq_start[b] == 0 ? 0.f : A.mx[((int64_t)A.seq_slots[b] * A.H + h) * nvb];
    C.m0[(int64_t)b * A.H + h] = m;
    float F = 0.f;
    // the chain itself is an add and a maximum per token; the log gates of the next sixteen tokens are in flight meanwhile
    constexpr int kAhead = 16;
    float nf[kAhead], ni[kAhead];
    float* g0 = C.gc + (int64_t)h * 3;
    const int64_t pitch = (int64_t)A.H * 3;
#pragma unroll
    for (int a = 0; a < kAhead; ++a) { const int64_t t = min(t0 + a, t1 - 1); nf[a] = g0[t * pitch]; ni[a] = g0[t * pitch + 1]; }
    for (int tb = t0; tb < t1; tb += kAhead) {
        float cf[kAhead], ci[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) { cf[a] = nf[a]; ci[a] = ni[a]; }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) { const int64_t t = min(tb + kAhead + a, t1 - 1); nf[a] = g0[t * pitch]; ni[a] = g0[t * pitch + 1]; }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int t = tb + a;
            if (t >= t1) break;
            if ((t - t0) % kChunk == 0) F = 0.f;
            F += cf[a];
            m = fmaxf(cf[a] + m, ci[a]);
            g0[(int64_t)t * pitch] = F; g0[(int64_t)t * pitch + 2] = m;
        }
    }
}

// F, li, m of row t (tt = its index inside the chunk)
__device__ __forceinline__ void token_gate(const ChunkArgs& C, int h, int t, int tt, float lnd, float& F, float& li, float& m) {
    if (C.gating == 0) { F = (float)(tt + 1) * lnd; li = 0.f; m = 0.f; return; }
    const float* g = C.gc + ((int64_t)t * C.A.H + h) * 3;
    F = g[0]; li = g[1]; m = g[2];
}
__device__ __forceinline__ float chunk_m_in(const ChunkArgs& C, int b, int h, int t_first, int c) {
    if (C.gating == 0) return 0.f;
    if (c > 0) return C.gc[((int64_t)(t_first - 1) * C.A.H + h) * 3 + 2];
    return C.m0[(int64_t)b * C.A.H + h];
}

// U[slot, h, cv, r] = sum_j w_j v_j[cv] k_j[r], w_j = e^(F_L - F_j + li_j - m_L); a block makes a 64 x 64 tile, a thread 4 x 4 of it
__global__ void __launch_bounds__(256)
la_chunk_state_kernel(const ChunkArgs C) {
    pdl_wait();
    pdl_trigger();
    const LinAttnArgs& A = C.A;
    __shared__ __align__(16) float vs[kChunk][64 + 4], ks[kChunk][64 + 4];          // rows of 68 floats: 16-byte reads of four neighbours
    __shared__ float ws[kChunk];
    const int h = blockIdx.y, b = blockIdx.z / C.max_chunks, c = blockIdx.z % C.max_chunks;
    const int t0 = A.cu_seqlens[b], rows = A.cu_seqlens[b + 1] - t0;
    if (c * kChunk >= rows) return;
    const int tf = t0 + c * kChunk, nt = min(kChunk, rows - c * kChunk);
    const int dk = A.dk, dv = A.dv, H = A.H;
    const int tiles_r = (dk + 63) / 64;
    const int cv0 = (blockIdx.x / tiles_r) * 64, r0 = (blockIdx.x % tiles_r) * 64;
    const int slot = chunk_base(A.cu_seqlens, b) + c;
    const float lnd = C.gating == 0 ? log_decay(A.decay[h]) : 0.f;
    if (threadIdx.x < kChunk) {
        float w = 0.f;
        if ((int)threadIdx.x < nt) {
            float F, li, m, FL, liL, mL;
            token_gate(C, h, tf + threadIdx.x, threadIdx.x, lnd, F, li, m);
            token_gate(C, h, tf + nt - 1, nt - 1, lnd, FL, liL, mL);
            w = expf(FL - F + li - mL);
        }
        ws[threadIdx.x] = w;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kChunk * 64; e += 256) {
        const int j = e >> 6, x = e & 63;
        float v = 0.f, k = 0.f;
        if (j < nt) {
            const float* row = A.proj + (int64_t)(tf + j) * A.ld;
            if (cv0 + x < dv) { v = row[A.off_v + h * dv + cv0 + x]; if (A.act == 1) v = silu_f(v); }
            if (r0 + x < dk) { k = row[A.off_k + h * dk + r0 + x]; if (A.act == 1) k = silu_f(k); }
        }
        vs[j][x] = v * ws[j]; ks[j][x] = k;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int j = 0; j < nt; ++j) {
        const float4 a4 = *reinterpret_cast<const float4*>(&vs[j][ty * 4]), k4 = *reinterpret_cast<const float4*>(&ks[j][tx * 4]);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w}, k[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int l = 0; l < 4; ++l) acc[i][l] = fmaf(a[i], k[l], acc[i][l]);
    }
    float* U = C.U + ((int64_t)slot * H + h) * dv * dk;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int cv = cv0 + ty * 4 + i;
        if (cv >= dv) continue;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const int r = r0 + tx * 4 + l;
            if (r < dk) U[(int64_t)cv * dk + r] = acc[i][l];
        }
    }
    if (C.gating == 1 && cv0 == 0 && threadIdx.x < 64 && r0 + (int)threadIdx.x < dk) {
        float s = 0.f;
        for (int j = 0; j < nt; ++j) s = fmaf(ws[j], ks[j][threadIdx.x], s);
        C.un[((int64_t)slot * H + h) * dk + r0 + threadIdx.x] = s;
    }
}

// a thread owns one state element (h, cv, r): U[c] <- the state that enters chunk c, the state slot <- the state after the last chunk
__global__ void __launch_bounds__(256)
la_chunk_scan_kernel(const ChunkArgs C) {
    pdl_wait();
    pdl_trigger();
    const LinAttnArgs& A = C.A;
    const int b = blockIdx.y;
    const int dk = A.dk, dv = A.dv, H = A.H;
    const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (e >= (int64_t)H * dv * dk) return;
    const int h = (int)(e / ((int64_t)dv * dk));
    const int cv = (int)((e / dk) % dv), r = (int)(e % dk);
    const int t0 = A.cu_seqlens[b], rows = A.cu_seqlens[b + 1] - t0;
    if (rows <= 0) return;
    const int nc = (rows + kChunk - 1) / kChunk;
    const int base = chunk_base(A.cu_seqlens, b);
    const bool fresh = A.seq_start[b] == 0;
    const int64_t slot = A.seq_slots[b];
    const int nvb = (dv + 15) / 16;
    float* Sp = A.S + ((slot * H + h) * dv + cv) * (int64_t)dk + r;
    const bool carries_n = C.gating == 1 && (cv & 15) == 0;            // one copy of the normaliser and of the maximum per 16 value columns
    float* np = carries_n ? A.nrm + ((slot * H + h) * nvb + (cv >> 4)) * (int64_t)dk + r : nullptr;
    float S = fresh ? 0.f : *Sp;
    float n = (carries_n && !fresh) ? *np : 0.f;
    const float lnd = C.gating == 0 ? log_decay(A.decay[h]) : 0.f;
    float m_in = chunk_m_in(C, b, h, t0, 0);
    // a chunk's term does not depend on the walk: the terms of the next eight chunks are in flight while the current one is applied
    constexpr int kAhead = 8;
    const int64_t ustride = (int64_t)H * dv * dk, nstride = (int64_t)H * dk;
    float* u0 = C.U + (((int64_t)base * H + h) * dv + cv) * dk + r;
    const int64_t n0 = ((int64_t)base * H + h) * dk + r;
    float nu[kAhead], nn[kAhead];
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
        const int c = min(a, nc - 1);
        nu[a] = u0[c * ustride];
        nn[a] = carries_n ? C.un[n0 + c * nstride] : 0.f;
    }
    for (int cb = 0; cb < nc; cb += kAhead) {
        float cu[kAhead], cn[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) { cu[a] = nu[a]; cn[a] = nn[a]; }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int c = min(cb + kAhead + a, nc - 1);
            nu[a] = u0[c * ustride];
            nn[a] = carries_n ? C.un[n0 + c * nstride] : 0.f;
        }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int c = cb + a;
            if (c >= nc) break;
            const int nt = min(kChunk, rows - c * kChunk);
            float FL, liL, mL;
            token_gate(C, h, t0 + c * kChunk + nt - 1, nt - 1, lnd, FL, liL, mL);
            const float g = expf(FL + m_in - mL);
            u0[c * ustride] = S;
            S = fmaf(g, S, cu[a]);
            if (carries_n) {
                if (cv == 0) C.un_in[n0 + c * nstride] = n;               // the output kernel reads the entering normaliser from here
                n = fmaf(g, n, cn[a]);
            }
            m_in = mL;
        }
    }
    *Sp = S;
    if (carries_n) {
        *np = n;
        if (r == 0) A.mx[(slot * H + h) * nvb + (cv >> 4)] = m_in;
    }
}

// o for the 64 tokens of a chunk and 64 value columns: scores against the chunk's own keys, weights, then values and entering state
__global__ void __launch_bounds__(256, 3)
la_chunk_output_kernel(const ChunkArgs C) {
    pdl_wait();
    pdl_trigger();
    const LinAttnArgs& A = C.A;
    extern __shared__ __align__(16) float sm[];
    // every tile is stored so that the four neighbours a thread multiplies together are one 16-byte read (rows of 68 floats)
    float (*qs)[68] = reinterpret_cast<float (*)[68]>(sm);                          // [32][68] a slab of 32 key rows of q: [key row][token]
    float (*ks)[68] = reinterpret_cast<float (*)[68]>(sm + 32 * 68);                // [32][68] the same slab of k: [key row][token]; later of the entering state
    float (*pw)[68] = reinterpret_cast<float (*)[68]>(sm + 2 * 32 * 68);            // [64][68] weighted scores: [key token j][query token t]
    float (*vs)[68] = reinterpret_cast<float (*)[68]>(sm + 2 * 32 * 68 + 64 * 68);  // [64][68] values: [token][column]
    float* sF = sm + 2 * 32 * 68 + 2 * 64 * 68;                                     // [64] F_t, li_t, m_t, c_t, n_in . q_t
    float* sL = sF + 64; float* sM = sL + 64; float* sC = sM + 64; float* sN = sC + 64;
    const int h = blockIdx.y, b = blockIdx.z / C.max_chunks, c = blockIdx.z % C.max_chunks;
    const int t0 = A.cu_seqlens[b], rows = A.cu_seqlens[b + 1] - t0;
    if (c * kChunk >= rows) return;
    const int tf = t0 + c * kChunk, nt = min(kChunk, rows - c * kChunk);
    const int dk = A.dk, dv = A.dv, H = A.H;
    const int cv0 = blockIdx.x * 64;
    const int slot = chunk_base(A.cu_seqlens, b) + c;
    const float lnd = C.gating == 0 ? log_decay(A.decay[h]) : 0.f;
    const float m_in = chunk_m_in(C, b, h, tf, c);
    const float* Uin = C.U + ((int64_t)slot * H + h) * dv * dk;
    const float* nin = C.un_in + ((int64_t)slot * H + h) * dk;
    if (threadIdx.x < 64) {
        float F = 0.f, li = 0.f, m = 0.f, nq = 0.f;
        if ((int)threadIdx.x < nt) {
            token_gate(C, h, tf + threadIdx.x, threadIdx.x, lnd, F, li, m);
            if (C.gating == 1) {
                const float* row = A.proj + (int64_t)(tf + threadIdx.x) * A.ld + A.off_q + h * dk;
                for (int r = 0; r < dk; ++r) nq = fmaf(nin[r], (A.act == 1 ? silu_f(row[r]) : row[r]) * A.q_scale, nq);
            }
        }
        sF[threadIdx.x] = F; sL[threadIdx.x] = li; sM[threadIdx.x] = m; sC[threadIdx.x] = expf(F + m_in - m); sN[threadIdx.x] = nq;
    }
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    // a thread's eight elements of a 64 x 32 slab: (j, x) = (e >> 5, e & 31), e = thread + 256 i.  The next slab's elements are fetched into registers
    // before the current slab is multiplied, so that the loads are in flight during the products.
    float rq[8], rk[8];
    auto fetch_qk = [&](int r0, bool with_k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = threadIdx.x + 256 * i, j = e >> 5, x = e & 31;
            const bool ok = j < nt && r0 + x < dk;
            const float* row = A.proj + (int64_t)(tf + (ok ? j : 0)) * A.ld;
            rq[i] = ok ? row[A.off_q + h * dk + r0 + x] : 0.f;
            if (with_k) rk[i] = ok ? row[A.off_k + h * dk + r0 + x] : 0.f;
        }
    };
    // scores: rows ty * 4 .., keys tx * 4 ..
    fetch_qk(0, true);
    for (int r0 = 0; r0 < dk; r0 += 32) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = threadIdx.x + 256 * i, j = e >> 5, x = e & 31;
            float q = rq[i], k = rk[i];
            if (A.act == 1) { q = silu_f(q); k = silu_f(k); }
            qs[x][j] = q * A.q_scale; ks[x][j] = k;
        }
        __syncthreads();
        if (r0 + 32 < dk) fetch_qk(r0 + 32, true);
#pragma unroll 8
        for (int x = 0; x < 32; ++x) {
            const float4 a4 = *reinterpret_cast<const float4*>(&qs[x][ty * 4]), k4 = *reinterpret_cast<const float4*>(&ks[x][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w}, k[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int l = 0; l < 4; ++l) acc[i][l] = fmaf(a[i], k[l], acc[i][l]);
        }
    }
    // the values of the chunk travel while the weights are worked out
    float rv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int e = threadIdx.x + 256 * i, j = e >> 6, x = e & 63;
        rv[i] = (j < nt && cv0 + x < dv) ? A.proj[(int64_t)(tf + j) * A.ld + A.off_v + h * dv + cv0 + x] : 0.f;
    }
#pragma unroll
    for (int l = 0; l < 4; ++l) {
        const int j = tx * 4 + l;
        float w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = ty * 4 + i;
            w[i] = (j <= t && t < nt) ? acc[i][l] * expf(sF[t] - sF[j] + sL[j] - sM[t]) : 0.f;
        }
        *reinterpret_cast<float4*>(&pw[j][ty * 4]) = make_float4(w[0], w[1], w[2], w[3]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int e = threadIdx.x + 256 * i;
        vs[e >> 6][e & 63] = A.act == 1 ? silu_f(rv[i]) : rv[i];
    }
    __syncthreads();
    // the first slab of q and of the entering state for the second term travels during the first term's products
    float ru[8];
    auto fetch_u = [&](int r0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = threadIdx.x + 256 * i, j = e >> 5, x = e & 31;
            ru[i] = (cv0 + j < dv && r0 + x < dk) ? Uin[(int64_t)(cv0 + j) * dk + r0 + x] : 0.f;
        }
    };
    fetch_qk(0, false);
    fetch_u(0);
    // first term of the output: weighted scores times values (rows ty * 4 .., columns tx * 4 ..)
    float o1[4][4] = {}, o2[4][4] = {};
    for (int j = 0; j < nt; ++j) {
        const float4 p4 = *reinterpret_cast<const float4*>(&pw[j][ty * 4]), v4 = *reinterpret_cast<const float4*>(&vs[j][tx * 4]);
        const float p[4] = {p4.x, p4.y, p4.z, p4.w}, v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int l = 0; l < 4; ++l) o1[i][l] = fmaf(p[i], v[l], o1[i][l]);
    }
    // second term: q against the state that entered the chunk, a slab of 32 key rows at a time
    float (*ss)[68] = ks;                                                           // [32][68] the entering state: [key row][column], over the k slab
    for (int r0 = 0; r0 < dk; r0 += 32) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = threadIdx.x + 256 * i, j = e >> 5, x = e & 31;
            qs[x][j] = (A.act == 1 ? silu_f(rq[i]) : rq[i]) * A.q_scale;
            ss[x][j] = ru[i];                        // the same index pair read the other way: column j of the tile, key row x
        }
        __syncthreads();
        if (r0 + 32 < dk) { fetch_qk(r0 + 32, false); fetch_u(r0 + 32); }
#pragma unroll 8
        for (int x = 0; x < 32; ++x) {
            const float4 a4 = *reinterpret_cast<const float4*>(&qs[x][ty * 4]), u4 = *reinterpret_cast<const float4*>(&ss[x][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int l = 0; l < 4; ++l) o2[i][l] = fmaf(a[i], u[l], o2[i][l]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = ty * 4 + i;
        if (t >= nt) continue;
        float den = 1.0f;
        if (C.gating == 1) {
            float nq = sC[t] * sN[t];
            for (int j = 0; j <= t; ++j) nq += pw[j][t];
            den = fmaxf(fabsf(nq), expf(-sM[t])) + 1e-6f;
        }
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const int cv = cv0 + tx * 4 + l;
            if (cv < dv) A.out[(int64_t)(tf + t) * H * dv + h * dv + cv] = fmaf(sC[t], o2[i][l], o1[i][l]) / den;
        }
    }
}

template <int kR, bool kExp>
void launch_linear_attention(const LinAttnArgs& A, int num_seqs, bool single_rows, cudaStream_t st) {
    if (single_rows) {
        launch_pdl(linear_attention_step_kernel<kR, kExp>, dim3(ceil_div(A.dv, 16), A.H, num_seqs), dim3(128), 0, st, A);
        return;
    }
    const int smem = (2 * kTile * 8 * kR + kTile * 16 + 6 * kTile + 1) * (int)sizeof(float);
    ensure_dynamic_smem(reinterpret_cast<const void*>(linear_attention_kernel<kR, kExp>), smem);
    launch_pdl(linear_attention_kernel<kR, kExp>, dim3(ceil_div(A.dv, 16), A.H, num_seqs), dim3(128), (size_t)smem, st, A);
}

template <bool kExp>
bool dispatch_linear_attention(const LinAttnArgs& A, int num_seqs, bool single_rows, cudaStream_t st) {
    if (A.dk <= 32) launch_linear_attention<4, kExp>(A, num_seqs, single_rows, st);
    else if (A.dk <= 64) launch_linear_attention<8, kExp>(A, num_seqs, single_rows, st);
    else if (A.dk <= 128) launch_linear_attention<16, kExp>(A, num_seqs, single_rows, st);
    else if (A.dk <= 256) launch_linear_attention<32, kExp>(A, num_seqs, single_rows, st);
    else if (A.dk <= 512) launch_linear_attention<64, kExp>(A, num_seqs, single_rows, st);      // spills its staging registers: a path for correctness, not speed
    else return false;
    return true;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void causal_conv_ex(const float* x, int64_t ldx, const float* in_bias, const float* taps, const float* out_bias, float* conv_state, void* y, int64_t ldy,
                    const int32_t* token_seq, const int32_t* cu_seqlens, const int32_t* seq_slots, const int32_t* seq_start, int32_t num_tokens,
                    int32_t num_seqs, int32_t single_rows, int32_t channels, int32_t num_taps, int32_t act, int32_t add_input, int32_t out_dtype, int64_t stream) {
    if (num_tokens == 0 || num_seqs == 0) return;
    B200_REQUIRE(x && taps && conv_state && y && token_seq && cu_seqlens && seq_slots && seq_start && channels > 0 && num_taps >= 1 && ldx >= channels &&
                 ldy >= channels && num_tokens <= 65535 && num_seqs <= 65535 && (act == 0 || act == 1), kErrBadArg, "causal_conv_ex: bad arguments");
    cudaStream_t st = as_stream(stream);
    const dim3 grid(ceil_div(channels, 128), num_tokens);
    if (single_rows) {
        B200_REQUIRE(num_tokens == num_seqs, kErrBadArg, "causal_conv_ex: the single-row kernel takes one row per entry");
        if (out_dtype == B200_F32)
            launch_pdl(causal_conv_step_kernel<float>, grid, dim3(128), 0, st, x, ldx, in_bias, taps, out_bias, conv_state, (float*)y, ldy, seq_slots, seq_start, channels,
                       num_taps, act, add_input);
        else if (out_dtype == B200_BF16)
            launch_pdl(causal_conv_step_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, x, ldx, in_bias, taps, out_bias, conv_state, (__nv_bfloat16*)y, ldy, seq_slots,
                       seq_start, channels, num_taps, act, add_input);
        else { set_error(kErrUnsupported, "causal_conv_ex: out dtype %d (f32 / bf16)", out_dtype); return; }
        count_launch();
        check_launch("causal_conv_ex");
        return;
    }
    if (out_dtype == B200_F32)
        launch_pdl(causal_conv_ex_kernel<float>, grid, dim3(128), 0, st, x, ldx, in_bias, taps, out_bias, (const float*)conv_state, (float*)y, ldy, token_seq,
                   cu_seqlens, seq_slots, seq_start, channels, num_taps, act, add_input);
    else if (out_dtype == B200_BF16)
        launch_pdl(causal_conv_ex_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, x, ldx, in_bias, taps, out_bias, (const float*)conv_state, (__nv_bfloat16*)y, ldy,
                   token_seq, cu_seqlens, seq_slots, seq_start, channels, num_taps, act, add_input);
    else { set_error(kErrUnsupported, "causal_conv_ex: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    if (num_taps > 1) {
        launch_pdl(causal_conv_roll_kernel, dim3(ceil_div(channels, 128), num_seqs), dim3(128), 0, st, x, ldx, in_bias, conv_state, cu_seqlens, seq_slots, seq_start,
                   channels, num_taps);
        count_launch();
    }
    check_launch("causal_conv_ex");
}

void block_diag_linear(const float* x, int64_t ldx, const float* weight, const float* bias, float* out, int64_t ldy, int32_t num_tokens, int32_t blocks,
                       int32_t rows_per_block, int32_t cols_per_block, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(x && weight && out && blocks > 0 && blocks <= 65535 && rows_per_block > 0 && cols_per_block > 0 && ldx >= (int64_t)blocks * cols_per_block &&
                 ldy >= (int64_t)blocks * rows_per_block, kErrBadArg, "block_diag_linear: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (num_tokens <= 8)
        launch_pdl(block_diag_rows_kernel, dim3(ceil_div(rows_per_block, 8), ceil_div(num_tokens, 4), blocks), dim3(256), 0, st, x, ldx, weight, bias, out, ldy,
                   num_tokens, rows_per_block, cols_per_block);
    else
        launch_pdl(block_diag_linear_kernel, dim3(ceil_div(rows_per_block, kBN), ceil_div(num_tokens, kBM), blocks), dim3(256), 0, st, x, ldx, weight, bias, out, ldy,
                   num_tokens, rows_per_block, cols_per_block);
    count_launch();
    check_launch("block_diag_linear");
}

void gated_linear_scan(const float* u, int64_t ldu, float* gates, int64_t ld_gates, const float* lam, float* y_pre, int64_t ldy, const float* y_bias,
                       float* state, void* out, float* scratch, const int32_t* cu_seqlens, const int32_t* seq_slots, const int32_t* seq_start, int32_t num_tokens, int32_t num_seqs,
                       int32_t max_rows, int32_t channels, int32_t block_channels, float decay_scale, int32_t out_dtype, int64_t stream) {
    if (num_seqs == 0 || num_tokens == 0) return;
    B200_REQUIRE(u && gates && lam && y_pre && state && out && cu_seqlens && seq_slots && seq_start && channels > 0 && block_channels > 0 &&
                 channels % block_channels == 0 && ldu >= channels && ldy >= channels && ld_gates >= 2 * (int64_t)channels && num_seqs <= 65535, kErrBadArg,
                 "gated_linear_scan: bad arguments");
    B200_REQUIRE(out_dtype == B200_F32 || out_dtype == B200_BF16, kErrUnsupported, "gated_linear_scan: out dtype %d (f32 / bf16)", out_dtype);
    cudaStream_t st = as_stream(stream);
    if (max_rows >= kScanSplitRows) {
        // portions of prompts: everything but the recurrence itself for all rows at once (in place), then a scan of two multiply-adds per row
        const int64_t total = (int64_t)num_tokens * channels;
        launch_pdl(gated_scan_prepare_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, u, ldu, gates, ld_gates, lam, y_pre, ldy, y_bias,
                   (int64_t)num_tokens, channels, block_channels, decay_scale);
        if (max_rows >= kScanChunkedRows && scratch && (int64_t)ceil_div(max_rows, kScanChunk) * num_seqs <= 65535) {
            const int max_chunks = ceil_div(max_rows, kScanChunk);
            const dim3 cgrid(ceil_div(channels, 128), max_chunks, num_seqs);
            launch_pdl(scan_chunk_compose_kernel, cgrid, dim3(128), 0, st, (const float*)gates, ld_gates, scratch, cu_seqlens, channels, block_channels);
            launch_pdl(scan_chunk_carry_kernel, dim3(ceil_div(channels, 128), num_seqs), dim3(128), 0, st, scratch, state, cu_seqlens, seq_slots, seq_start, channels);
            if (out_dtype == B200_F32)
                launch_pdl(scan_chunk_replay_kernel<float>, cgrid, dim3(128), 0, st, (const float*)gates, ld_gates, (const float*)y_pre, ldy, (const float*)scratch,
                           (float*)out, cu_seqlens, channels, block_channels);
            else
                launch_pdl(scan_chunk_replay_kernel<__nv_bfloat16>, cgrid, dim3(128), 0, st, (const float*)gates, ld_gates, (const float*)y_pre, ldy,
                           (const float*)scratch, (__nv_bfloat16*)out, cu_seqlens, channels, block_channels);
            count_launch(4);
            check_launch("gated_linear_scan");
            return;
        }
        const dim3 grid(ceil_div(channels, 32), num_seqs);
        if (out_dtype == B200_F32)
            launch_pdl(linear_scan_kernel<float>, grid, dim3(32), 0, st, (const float*)gates, ld_gates, (const float*)y_pre, ldy, state, (float*)out, cu_seqlens, seq_slots,
                       seq_start, channels, block_channels);
        else
            launch_pdl(linear_scan_kernel<__nv_bfloat16>, grid, dim3(32), 0, st, (const float*)gates, ld_gates, (const float*)y_pre, ldy, state, (__nv_bfloat16*)out,
                       cu_seqlens, seq_slots, seq_start, channels, block_channels);
        count_launch(2);
        check_launch("gated_linear_scan");
        return;
    }
    const dim3 grid(ceil_div(channels, 64), num_seqs);
    if (out_dtype == B200_F32)
        launch_pdl(gated_linear_scan_kernel<float>, grid, dim3(64), 0, st, u, ldu, (const float*)gates, ld_gates, lam, (const float*)y_pre, ldy, y_bias, state, (float*)out,
                   cu_seqlens, seq_slots, seq_start, channels, block_channels, decay_scale);
    else
        launch_pdl(gated_linear_scan_kernel<__nv_bfloat16>, grid, dim3(64), 0, st, u, ldu, (const float*)gates, ld_gates, lam, (const float*)y_pre, ldy, y_bias, state,
                   (__nv_bfloat16*)out, cu_seqlens, seq_slots, seq_start, channels, block_channels, decay_scale);
    count_launch();
    check_launch("gated_linear_scan");
}

void linear_attention(const float* proj, int64_t ld, int32_t off_q, int32_t off_k, int32_t off_v, int32_t off_i, int32_t off_f, const float* decay,
                      const float* i_bias, const float* f_bias, float gate_cap, float q_scale, int32_t act, int32_t gating, float* state, float* normaliser,
                      float* maximum, float* out, const int32_t* cu_seqlens, const int32_t* seq_slots, const int32_t* seq_start, int32_t num_tokens,
                      int32_t num_seqs, int32_t single_rows, int32_t num_heads, int32_t dk, int32_t dv, int64_t stream) {
    if (num_seqs == 0) return;
    B200_REQUIRE(!single_rows || num_tokens == num_seqs, kErrBadArg, "linear_attention: the single-row kernel takes one row per entry");
    B200_REQUIRE(proj && state && out && cu_seqlens && seq_slots && seq_start && num_heads > 0 && num_heads <= 65535 && num_seqs <= 65535 && dk > 0 && dv > 0 &&
                 (act == 0 || act == 1) && (gating == 0 || gating == 1), kErrBadArg, "linear_attention: bad arguments");
    B200_REQUIRE(gating == 0 ? decay != nullptr : (normaliser && maximum && gate_cap > 0.f), kErrBadArg,
                 "linear_attention: fixed decay needs decay[H]; exponential gating needs the normaliser, the maximum and a positive cap");
    B200_REQUIRE(dk <= 512, kErrUnsupported, "linear_attention: key size %d > 512", dk);
    LinAttnArgs A{proj, ld, off_q, off_k, off_v, off_i, off_f, decay, i_bias, f_bias, gate_cap, q_scale, act, state, normaliser, maximum, out,
                  cu_seqlens, seq_slots, seq_start, num_heads, dk, dv};
    cudaStream_t st = as_stream(stream);
    if (gating == 0) dispatch_linear_attention<false>(A, num_seqs, single_rows != 0, st);
    else dispatch_linear_attention<true>(A, num_seqs, single_rows != 0, st);
    count_launch();
    check_launch("linear_attention");
}

int64_t linear_attention_chunked_scratch(int32_t num_tokens, int32_t num_seqs, int32_t num_heads, int32_t dk, int32_t dv) {
    // floats: per chunk slot a [dv, dk] term per head and two normaliser rows, per token three gate values per head, per entry a maximum per head
    const int64_t slots = (int64_t)(num_tokens + kChunk - 1) / kChunk + num_seqs;
    return slots * num_heads * ((int64_t)dv * dk + 2 * dk) + (int64_t)num_tokens * num_heads * 3 + (int64_t)num_seqs * num_heads;
}


void linear_attention_chunked(const float* proj, int64_t ld, int32_t off_q, int32_t off_k, int32_t off_v, int32_t off_i, int32_t off_f, const float* decay,
                              const float* i_bias, const float* f_bias, float gate_cap, float q_scale, int32_t act, int32_t gating, float* state, float* normaliser,
                              float* maximum, float* out, float* scratch, const int32_t* cu_seqlens, const int32_t* seq_slots, const int32_t* seq_start,
                              int32_t num_tokens, int32_t num_seqs, int32_t max_rows, int32_t num_heads, int32_t dk, int32_t dv, int64_t stream) {
    if (num_seqs == 0 || num_tokens == 0) return;
    B200_REQUIRE(proj && state && out && scratch && cu_seqlens && seq_slots && seq_start && num_heads > 0 && num_heads <= 65535 && dk > 0 && dv > 0 && max_rows > 0 &&
                 (act == 0 || act == 1) && (gating == 0 || gating == 1), kErrBadArg, "linear_attention_chunked: bad arguments");
    B200_REQUIRE(gating == 0 ? decay != nullptr : (normaliser && maximum && gate_cap > 0.f), kErrBadArg,
                 "linear_attention_chunked: fixed decay needs decay[H]; exponential gating needs the normaliser, the maximum and a positive cap");
    const int max_chunks = (max_rows + kChunk - 1) / kChunk;
    B200_REQUIRE((int64_t)max_chunks * num_seqs <= 65535, kErrUnsupported, "linear_attention_chunked: %d chunks x %d entries exceed the grid", max_chunks, num_seqs);
    const int64_t slots = (int64_t)(num_tokens + kChunk - 1) / kChunk + num_seqs;
    ChunkArgs C;
    C.A = LinAttnArgs{proj, ld, off_q, off_k, off_v, off_i, off_f, decay, i_bias, f_bias, gate_cap, q_scale, act, state, normaliser, maximum, out,
                      cu_seqlens, seq_slots, seq_start, num_heads, dk, dv};
    C.U = scratch;
    C.un = C.U + slots * num_heads * dv * dk;
    C.un_in = C.un + slots * num_heads * dk;
    C.gc = C.un_in + slots * num_heads * dk;
    C.m0 = C.gc + (int64_t)num_tokens * num_heads * 3;
    C.max_chunks = max_chunks;
    C.gating = gating;
    cudaStream_t st = as_stream(stream);
    int launches = 3;
    if (gating == 1) {
        launch_pdl(la_gate_values_kernel, dim3(ceil_div((int64_t)num_tokens * num_heads, 256)), dim3(256), 0, st, C, (int)num_tokens);
        launch_pdl(la_gate_chain_kernel, dim3(ceil_div(num_heads, 32), num_seqs), dim3(32), 0, st, C);
        launches += 2;
    }
    const unsigned z = (unsigned)(max_chunks * num_seqs);
    launch_pdl(la_chunk_state_kernel, dim3(ceil_div(dv, 64) * ceil_div(dk, 64), num_heads, z), dim3(256), 0, st, C);
    launch_pdl(la_chunk_scan_kernel, dim3(ceil_div((int64_t)num_heads * dv * dk, 256), num_seqs), dim3(256), 0, st, C);
    const int smem = (2 * 32 * 68 + 2 * 64 * 68 + 5 * 64) * (int)sizeof(float);
    ensure_dynamic_smem(reinterpret_cast<const void*>(la_chunk_output_kernel), smem);
    launch_pdl(la_chunk_output_kernel, dim3(ceil_div(dv, 64), num_heads, z), dim3(256), (size_t)smem, st, C);
    count_launch(launches);
    check_launch("linear_attention_chunked");
}

}  // extern "C"
