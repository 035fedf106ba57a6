// norm_act.cu -- the row-wise pieces between the matrix products of the pre+post-norm decoder family, all 32-bit inside:
//   rms_norm_ex      out[r] = (residual[r] +) x[src(r)] / sqrt(mean(x^2) + eps) * (offset + w)   -- offset 1 for weights stored
//                    around zero; `residual` makes it the closing norm of a sublayer (the sum stays f32, in place is fine);
//                    `row_index` gathers the rows whose result is wanted (the logits of a step);
//   gelu_tanh_mul    out = gelu_tanh(gate) * up from the packed [rows, 2 ff] product of a fused gate|up projection;
//   embedding_scaled out[t] = table[ids[t]] * scale, table f32 or bf16.
//   embedding_bigram out[t] = table[ids[t]] + bigram[row(t)]: row = (previous token * mul_prev + token * mul_cur) mod buckets, the extra
//                    row `buckets` for a sequence's first token; the previous token of an entry's first row comes from (and the entry's
//                    last token goes to) a per-slot i32 state, so a sequence may be cut into steps anywhere;
//   residual_rms_norm  the two closing forms of a sublayer on the f32 stream x, in place: mode 0 "norm after the sum"
//                    x <- norm(alpha x + y) * w, mode 1 x <- x + norm(y) * w; optionally also x in 16 bits for the next product;
//   gelu_tanh_gather_mul  out[t, i] = gelu_tanh(z[t, i]) * table[ids[t], col0 + i] (a per-token embedding gated by the stream).
//   embedding_positional  out[t] = table[ids[t]] * scale + pos_table[positions[t]] (a learned position vector per place);
//   layer_norm_ex    out[r] = (x[src(r)] - mean) / sqrt(var + eps) * w + b with the biased variance, in up to two copies: one of the
//                    compute dtype for the next product, one f32 for whatever else reads the normed row;
//   gated_residual_add  x <- x + sigmoid(z + bias) * y, the gate's pre-activation z being a product of its own (z null: x <- x + y);
//   gated_add_layer_norm  both of the above in one pass over the row: the closing sum of a sublayer, then the next sublayer's norm of the new x;
//   glu_packed       out = act(gate) * up from a packed [rows, 2 ff] product, act one of silu, tanh GELU, or the clamped form
//                    g' = min(g, limit), u' = clamp(u, +-limit), g' sigmoid(1.702 g') (u' + 1); a per-row factor may multiply gate and
//                    up first (an expert that sees its token times the router's score); act 3 is ungated: out = relu(g)^2 from rows of ff entries;
//   add_rms_norm     the pre-norm step on the f32 stream: x <- x + y1 + y2 (each optional; x in place), then out = x / sqrt(mean(x^2) + eps) * w
//                    in the compute dtype for the next product -- the closing sum of one sublayer and the opening norm of the next in one pass;
//                    with `row_index` only the selected rows are summed and normed and x is left as it is; w null = the sum alone;
//   group_rms_norm_gate  out = o / rms(o over a group of neighbours) * w * act(gate): the closing norm of the linear-attention mixers,
//                    one group per head or one for the whole row;
//   head_gate        out[t, h, :] = src[t, h, :] * sigmoid(gate[t, h]): one gate per attention head.
// Any row length (no vector-width rule): the rows these models use are a few hundred to a few thousand floats and every kernel
// here is one pass over them from L2.
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    __syncthreads();
    return t;
}

template <typename TOut>
__global__ void __launch_bounds__(256)
rms_norm_ex_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* out, const float* residual,
                   const int32_t* __restrict__ row_index, int n, int64_t ldx, float eps, float offset) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const int row = blockIdx.x;
    const int64_t src = row_index ? row_index[row] : row;
    const float* xr = x + src * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    const float tot = block_sum_256(ss, red);
    const float sc = 1.0f / sqrtf(tot / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = xr[i] * sc * (offset + w[i]);
        if (residual) v += residual[(int64_t)row * n + i];
        out[(int64_t)row * n + i] = from_f32<TOut>(v);
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    const float c = 0.7978845608028654f;       // sqrt(2 / pi)
    return 0.5f * z * (1.0f + tanhf(c * (z + 0.044715f * z * z * z)));
}

template <typename TOut>
__global__ void gelu_tanh_mul_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int64_t rows, int ff, int64_t ld) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * ff) return;
    const int64_t r = i / ff;
    const int c = (int)(i - r * ff);
    const float g = gu[r * ld + c], u = gu[r * ld + ff + c];
    out[i] = from_f32<TOut>(gelu_tanh_f(g) * u);
}

template <typename TTab>
__global__ void embedding_scaled_kernel(const TTab* __restrict__ table, const int32_t* __restrict__ ids, float* __restrict__ out, int dim,
                                        int vocab, float scale) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) out[(int64_t)t * dim + i] = to_f32<TTab>(table[(int64_t)id * dim + i]) * scale;
}

template <typename TTab>
__global__ void __launch_bounds__(128)
embedding_bigram_kernel(const TTab* __restrict__ table, const TTab* __restrict__ bigram, const int32_t* __restrict__ ids,
                        const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq, const int32_t* __restrict__ cu_seqlens,
                        const int32_t* __restrict__ seq_slots, int32_t* prev_state, float* __restrict__ out, int dim, int vocab, int buckets,
                        int mul_prev, int mul_cur) {
    pdl_wait();
    pdl_trigger();
    __shared__ int s_prev;
    const int t = blockIdx.x;
    auto clampv = [&](int id) { return id < 0 ? 0 : (id >= vocab ? vocab - 1 : id); };
    const int id = clampv(ids[t]);
    if (threadIdx.x == 0) {
        const int b = token_seq[t];
        const int first = cu_seqlens[b], last = cu_seqlens[b + 1] - 1;
        int prev = -1;
        if (t == first) {
            // only this block touches the entry's slot: read what the last step left, then leave the entry's last token
            const int slot = seq_slots[b];
            if (prev_state && slot >= 0) {
                if (positions[t] > 0) prev = prev_state[slot];
                prev_state[slot] = ids[last];
            }
        } else {
            prev = ids[t - 1];
        }
        if (positions[t] == 0) prev = -1;
        s_prev = prev;
    }
    __syncthreads();
    const int prev = s_prev;
    const int64_t row = prev < 0 ? (int64_t)buckets : (int64_t)(((int64_t)clampv(prev) * mul_prev + (int64_t)id * mul_cur) % buckets);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[(int64_t)t * dim + i] = to_f32<TTab>(table[(int64_t)id * dim + i]) + (bigram ? to_f32<TTab>(bigram[row * dim + i]) : 0.f);
}

template <typename T16>
__global__ void __launch_bounds__(256)
residual_rms_norm_kernel(float* x, const float* __restrict__ y, int64_t ldy, const float* __restrict__ w, T16* out16, int n, float alpha, float eps,
                         int mode) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    float* xr = x + row * n;
    const float* yr = y ? y + row * ldy : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = mode == 0 ? fmaf(alpha, xr[i], yr ? yr[i] : 0.f) : yr[i];
        ss = fmaf(v, v, ss);
    }
    const float sc = 1.0f / sqrtf(block_sum_256(ss, red) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        float v;
        if (mode == 0) v = fmaf(alpha, xr[i], yr ? yr[i] : 0.f) * sc * w[i];
        else v = xr[i] + yr[i] * sc * w[i];
        xr[i] = v;
        if (out16) out16[row * n + i] = from_f32<T16>(v);
    }
}

template <typename TTab, typename TOut>
__global__ void gelu_tanh_gather_mul_kernel(const float* __restrict__ z, int64_t ldz, const TTab* __restrict__ table, int64_t ld_table, int col0,
                                            const int32_t* __restrict__ ids, TOut* __restrict__ out, int64_t rows, int dim, int vocab) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * dim) return;
    const int64_t r = i / dim;
    const int c = (int)(i - r * dim);
    int id = ids[r];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    out[i] = from_f32<TOut>(gelu_tanh_f(z[r * ldz + c]) * to_f32<TTab>(table[(int64_t)id * ld_table + col0 + c]));
}


template <typename TTab>
__global__ void embedding_positional_kernel(const TTab* __restrict__ table, const TTab* __restrict__ pos_table, const int32_t* __restrict__ ids,
                                            const int32_t* __restrict__ positions, float* __restrict__ out, int dim, int vocab, int max_pos, float scale) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    int p = positions[t];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[(int64_t)t * dim + i] = fmaf(to_f32<TTab>(table[(int64_t)id * dim + i]), scale, to_f32<TTab>(pos_table[(int64_t)p * dim + i]));
}

template <typename TOut>
__global__ void __launch_bounds__(256)
layer_norm_ex_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, TOut* out, float* out32,
                     const int32_t* __restrict__ row_index, int n, int64_t ldx, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const int row = blockIdx.x;
    const int64_t src = row_index ? row_index[row] : row;
    const float* xr = x + src * ldx;
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) s += xr[i];
    const float mean = block_sum_256(s, red) / (float)n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { const float d = xr[i] - mean; ss = fmaf(d, d, ss); }
    const float sc = 1.0f / sqrtf(block_sum_256(ss, red) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = fmaf((xr[i] - mean) * sc, w[i], b ? b[i] : 0.f);
        if (out) out[(int64_t)row * n + i] = from_f32<TOut>(v);
        if (out32) out32[(int64_t)row * n + i] = v;
    }
}

__global__ void gated_residual_add_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t ldy, const float* __restrict__ z, int64_t ldz,
                                          const float* __restrict__ bias, int64_t rows, int n) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * n) return;
    const int64_t r = i / n;
    const int c = (int)(i - r * n);
    float v = y[r * ldy + c];
    if (z) v *= 1.0f / (1.0f + expf(-(z[r * ldz + c] + (bias ? bias[c] : 0.f))));
    x[i] += v;
}

__device__ __forceinline__ float glu_value(float g, float u, int act, float limit) {
    if (act == 0) return g / (1.0f + expf(-g)) * u;
    if (act == 1) return gelu_tanh_f(g) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

template <typename TOut>
__global__ void glu_packed_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int64_t rows, int ff, int64_t ld, int act, float limit,
                                  const float* __restrict__ row_scale, const int32_t* __restrict__ scale_index) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * ff) return;
    const int64_t r = i / ff;
    const int c = (int)(i - r * ff);
    float g = gu[r * ld + c], u = act == 3 ? 0.f : gu[r * ld + ff + c];        // act 3 is ungated: the row holds ff entries only
    if (row_scale) {
        const int64_t j = scale_index ? scale_index[r] : r;
        if (j < 0) { out[i] = from_f32<TOut>(0.f); return; }          // a padding row of a sorted, tiled order
        const float s = row_scale[j];
        g *= s; u *= s;
    }
    if (act == 3) { g = fmaxf(g, 0.f); out[i] = from_f32<TOut>(g * g); return; }
    out[i] = from_f32<TOut>(glu_value(g, u, act, limit));
}

template <typename TOut>
__global__ void __launch_bounds__(128)
group_rms_norm_gate_kernel(const float* __restrict__ o, int64_t ldo, const float* __restrict__ w, const float* __restrict__ gate, int64_t ldg, TOut* __restrict__ out,
                           int n, int glen, float eps, int gate_act) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[4];
    const int64_t t = blockIdx.y;
    const int c0 = blockIdx.x * glen;
    const float* orow = o + t * ldo + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < glen; i += 128) { const float v = orow[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float sc = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)glen + eps);
    for (int i = threadIdx.x; i < glen; i += 128) {
        float v = orow[i] * sc * (w ? w[c0 + i] : 1.0f);
        if (gate) {
            const float z = gate[t * ldg + c0 + i];
            v *= gate_act == 0 ? 1.0f / (1.0f + expf(-z)) : z / (1.0f + expf(-z));
        }
        out[t * n + c0 + i] = from_f32<TOut>(v);
    }
}


template <typename TS, typename TOut>
__global__ void head_gate_kernel(const TS* __restrict__ src, const float* __restrict__ gate, int64_t ldg, TOut* __restrict__ out, int H, int dv) {
    pdl_wait();
    pdl_trigger();
    // a thread takes four neighbours of one row (of one head when dv is a multiple of four)
    const int64_t r = blockIdx.y;
    const int n = H * dv;
    const int i0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i0 >= n) return;
    const TS* sp = src + r * n;
    TOut* op = out + r * n;
    if ((dv & 3) == 0) {
        const float g = 1.0f / (1.0f + expf(-gate[r * ldg + i0 / dv]));
        float v[4];
        if (sizeof(TS) == 4) { const float4 t = *reinterpret_cast<const float4*>(sp + i0); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
        else { const uint2 t = *reinterpret_cast<const uint2*>(sp + i0); const TS* e = reinterpret_cast<const TS*>(&t); for (int j = 0; j < 4; ++j) v[j] = to_f32<TS>(e[j]); }
        if (sizeof(TOut) == 4) *reinterpret_cast<float4*>(op + i0) = make_float4(v[0] * g, v[1] * g, v[2] * g, v[3] * g);
        else {
            TOut o[4];
            for (int j = 0; j < 4; ++j) o[j] = from_f32<TOut>(v[j] * g);
            *reinterpret_cast<uint2*>(op + i0) = *reinterpret_cast<const uint2*>(o);
        }
        return;
    }
    for (int i = i0; i < min(i0 + 4, n); ++i) op[i] = from_f32<TOut>(to_f32<TS>(sp[i]) / (1.0f + expf(-gate[r * ldg + i / dv])));
}

// the closing sum of one sublayer and the opening norm of the next in one pass over the row: x <- x + sigmoid(z + zb) * y, then the layer norm of the new x
template <typename TOut>
__global__ void __launch_bounds__(256)
gated_add_layer_norm_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t ldy, const float* __restrict__ z, int64_t ldz, const float* __restrict__ zb,
                            const float* __restrict__ w, const float* __restrict__ b, TOut* out, float* out32, int n, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    float* xr = x + row * n;
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = y[row * ldy + i];
        if (z) v *= 1.0f / (1.0f + expf(-(z[row * ldz + i] + (zb ? zb[i] : 0.f))));
        v += xr[i];
        xr[i] = v;                                 // read again below by the thread that wrote it
        s += v;
    }
    const float mean = block_sum_256(s, red) / (float)n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { const float d = xr[i] - mean; ss = fmaf(d, d, ss); }
    const float sc = 1.0f / sqrtf(block_sum_256(ss, red) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = fmaf((xr[i] - mean) * sc, w[i], b ? b[i] : 0.f);
        if (out) out[row * n + i] = from_f32<TOut>(v);
        if (out32) out32[row * n + i] = v;
    }
}


template <typename TOut>
__global__ void __launch_bounds__(256)
add_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ y1, int64_t ld1, const float* __restrict__ y2, int64_t ld2, const float* __restrict__ w,
                    TOut* __restrict__ out, const int32_t* __restrict__ row_index, int n, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const int row = blockIdx.x;
    const int64_t src = row_index ? row_index[row] : row;
    float* xr = x + src * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = xr[i];
        if (y1) v += y1[src * ld1 + i];
        if (y2) v += y2[src * ld2 + i];
        if (!row_index && (y1 || y2)) xr[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!out) return;
    const float tot = block_sum_256(ss, red);
    const float sc = 1.0f / sqrtf(tot / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = xr[i];
        if (row_index) {                                   // x was not updated: form the sum again
            if (y1) v += y1[src * ld1 + i];
            if (y2) v += y2[src * ld2 + i];
        }
        out[(int64_t)row * n + i] = from_f32<TOut>(v * sc * w[i]);
    }
}


// act 3 of glu_packed without a row factor: out = relu(x)^2 over rows of ff entries (pitch ld), four entries per thread when rows allow 16-byte loads
template <typename TOut>
__global__ void __launch_bounds__(256)
relu2_rows_kernel(const float* __restrict__ x, TOut* __restrict__ out, int ff, int64_t ld, int vec) {
    pdl_wait();
    pdl_trigger();
    const int64_t r = blockIdx.x;
    const int c = (blockIdx.y * 256 + threadIdx.x) * 4;
    if (c >= ff) return;
    const float* src = x + r * ld + c;
    TOut* dst = out + r * ff + c;
    if (vec) {
        float4 v = *reinterpret_cast<const float4*>(src);
        v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
        dst[0] = from_f32<TOut>(v.x * v.x); dst[1] = from_f32<TOut>(v.y * v.y); dst[2] = from_f32<TOut>(v.z * v.z); dst[3] = from_f32<TOut>(v.w * v.w);
    } else {
        for (int i = 0; i < 4 && c + i < ff; ++i) { const float v = fmaxf(src[i], 0.f); dst[i] = from_f32<TOut>(v * v); }
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void rms_norm_ex(const float* x, const float* weight, void* out, const float* residual, const int32_t* row_index, int32_t rows, int32_t n,
                 int64_t ldx, float eps, float weight_offset, int32_t out_dtype, int64_t stream) {
    if (rows == 0) return;
    B200_REQUIRE(x && weight && out && rows > 0 && n > 0 && ldx >= n, kErrBadArg, "rms_norm_ex: bad arguments");
    B200_REQUIRE(!residual || out_dtype == B200_F32, kErrUnsupported, "rms_norm_ex: the residual sum is f32");
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32) launch_pdl(rms_norm_ex_kernel<float>, dim3(rows), dim3(256), 0, st, x, weight, (float*)out, residual, row_index, n, ldx, eps, weight_offset);
    else if (out_dtype == B200_BF16) launch_pdl(rms_norm_ex_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, st, x, weight, (__nv_bfloat16*)out, residual, row_index, n, ldx, eps, weight_offset);
    else { set_error(kErrUnsupported, "rms_norm_ex: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("rms_norm_ex");
}

void gelu_tanh_mul(const float* gate_up, void* out, int64_t rows, int32_t ff, int64_t ld, int32_t out_dtype, int64_t stream) {
    if (rows == 0 || ff == 0) return;
    B200_REQUIRE(gate_up && out && rows > 0 && ff > 0 && ld >= 2 * (int64_t)ff, kErrBadArg, "gelu_tanh_mul: bad arguments");
    const int64_t total = rows * ff;
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32) launch_pdl(gelu_tanh_mul_kernel<float>, dim3(grid), dim3(256), 0, st, gate_up, (float*)out, rows, ff, ld);
    else if (out_dtype == B200_BF16) launch_pdl(gelu_tanh_mul_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, gate_up, (__nv_bfloat16*)out, rows, ff, ld);
    else { set_error(kErrUnsupported, "gelu_tanh_mul: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("gelu_tanh_mul");
}

void embedding_scaled(const void* table, const int32_t* ids, float* out, int32_t num_tokens, int32_t dim, int32_t vocab, float scale,
                      int32_t table_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(table && ids && out && dim > 0 && vocab > 0, kErrBadArg, "embedding_scaled: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (table_dtype == B200_F32) launch_pdl(embedding_scaled_kernel<float>, dim3(num_tokens), dim3(128), 0, st, (const float*)table, ids, out, dim, vocab, scale);
    else if (table_dtype == B200_BF16) launch_pdl(embedding_scaled_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, st, (const __nv_bfloat16*)table, ids, out, dim, vocab, scale);
    else { set_error(kErrUnsupported, "embedding_scaled: table dtype %d (f32 / bf16)", table_dtype); return; }
    count_launch();
    check_launch("embedding_scaled");
}

void embedding_bigram(const void* table, const void* bigram, const int32_t* ids, const int32_t* positions, const int32_t* token_seq,
                      const int32_t* cu_seqlens, const int32_t* seq_slots, int32_t* prev_state, float* out, int32_t num_tokens, int32_t dim,
                      int32_t vocab, int32_t buckets, int32_t mul_prev, int32_t mul_cur, int32_t table_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(table && ids && positions && token_seq && cu_seqlens && seq_slots && out && dim > 0 && vocab > 0, kErrBadArg,
                 "embedding_bigram: bad arguments");
    B200_REQUIRE(!bigram || (prev_state && buckets > 0), kErrBadArg, "embedding_bigram: a bigram table needs buckets and the previous-token state");
    cudaStream_t st = as_stream(stream);
    if (table_dtype == B200_F32)
        launch_pdl(embedding_bigram_kernel<float>, dim3(num_tokens), dim3(128), 0, st, (const float*)table, (const float*)bigram, ids, positions, token_seq,
                   cu_seqlens, seq_slots, prev_state, out, dim, vocab, buckets, mul_prev, mul_cur);
    else if (table_dtype == B200_BF16)
        launch_pdl(embedding_bigram_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, st, (const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, ids,
                   positions, token_seq, cu_seqlens, seq_slots, prev_state, out, dim, vocab, buckets, mul_prev, mul_cur);
    else { set_error(kErrUnsupported, "embedding_bigram: table dtype %d (f32 / bf16)", table_dtype); return; }
    count_launch();
    check_launch("embedding_bigram");
}

void residual_rms_norm(float* x, const float* y, int64_t ldy, const float* weight, void* out16, int32_t rows, int32_t n, float alpha, float eps,
                       int32_t mode, int64_t stream) {
    if (rows == 0) return;
    B200_REQUIRE(x && weight && rows > 0 && n > 0 && (mode == 0 || (mode == 1 && y)) && (!y || ldy >= n), kErrBadArg, "residual_rms_norm: bad arguments");
    launch_pdl(residual_rms_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, as_stream(stream), x, y, ldy, weight, (__nv_bfloat16*)out16, n, alpha, eps, mode);
    count_launch();
    check_launch("residual_rms_norm");
}

void gelu_tanh_gather_mul(const float* z, int64_t ldz, const void* table, int64_t ld_table, int32_t col0, const int32_t* ids, void* out, int32_t rows,
                          int32_t dim, int32_t vocab, int32_t table_dtype, int32_t out_dtype, int64_t stream) {
    if (rows == 0 || dim == 0) return;
    B200_REQUIRE(z && table && ids && out && rows > 0 && dim > 0 && vocab > 0 && ldz >= dim && col0 >= 0 && ld_table >= col0 + dim, kErrBadArg,
                 "gelu_tanh_gather_mul: bad arguments");
    B200_REQUIRE(table_dtype == out_dtype && (out_dtype == B200_F32 || out_dtype == B200_BF16), kErrUnsupported,
                 "gelu_tanh_gather_mul: table and out share a dtype (f32 / bf16)");
    const unsigned grid = (unsigned)(((int64_t)rows * dim + 255) / 256);
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32)
        launch_pdl(gelu_tanh_gather_mul_kernel<float, float>, dim3(grid), dim3(256), 0, st, z, ldz, (const float*)table, ld_table, col0, ids, (float*)out,
                   (int64_t)rows, dim, vocab);
    else
        launch_pdl(gelu_tanh_gather_mul_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(256), 0, st, z, ldz, (const __nv_bfloat16*)table, ld_table, col0,
                   ids, (__nv_bfloat16*)out, (int64_t)rows, dim, vocab);
    count_launch();
    check_launch("gelu_tanh_gather_mul");
}

void embedding_positional(const void* table, const void* pos_table, const int32_t* ids, const int32_t* positions, float* out, int32_t num_tokens, int32_t dim,
                          int32_t vocab, int32_t max_pos, float scale, int32_t table_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(table && pos_table && ids && positions && out && dim > 0 && vocab > 0 && max_pos > 0, kErrBadArg, "embedding_positional: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (table_dtype == B200_F32)
        launch_pdl(embedding_positional_kernel<float>, dim3(num_tokens), dim3(128), 0, st, (const float*)table, (const float*)pos_table, ids, positions, out, dim, vocab,
                   max_pos, scale);
    else if (table_dtype == B200_BF16)
        launch_pdl(embedding_positional_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, st, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, ids,
                   positions, out, dim, vocab, max_pos, scale);
    else { set_error(kErrUnsupported, "embedding_positional: table dtype %d (f32 / bf16)", table_dtype); return; }
    count_launch();
    check_launch("embedding_positional");
}

void layer_norm_ex(const float* x, const float* weight, const float* bias, void* out, float* out32, const int32_t* row_index, int32_t rows, int32_t n, int64_t ldx,
                   float eps, int32_t out_dtype, int64_t stream) {
    if (rows == 0) return;
    B200_REQUIRE(x && weight && (out || out32) && rows > 0 && n > 0 && ldx >= n, kErrBadArg, "layer_norm_ex: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32) launch_pdl(layer_norm_ex_kernel<float>, dim3(rows), dim3(256), 0, st, x, weight, bias, (float*)out, out32, row_index, n, ldx, eps);
    else if (out_dtype == B200_BF16)
        launch_pdl(layer_norm_ex_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, st, x, weight, bias, (__nv_bfloat16*)out, out32, row_index, n, ldx, eps);
    else { set_error(kErrUnsupported, "layer_norm_ex: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("layer_norm_ex");
}

void gated_residual_add(float* x, const float* y, int64_t ldy, const float* gate_logits, int64_t ld_gate, const float* gate_bias, int32_t rows, int32_t n,
                        int64_t stream) {
    if (rows == 0) return;
    B200_REQUIRE(x && y && rows > 0 && n > 0 && ldy >= n && (!gate_logits || ld_gate >= n), kErrBadArg, "gated_residual_add: bad arguments");
    const unsigned grid = (unsigned)(((int64_t)rows * n + 255) / 256);
    launch_pdl(gated_residual_add_kernel, dim3(grid), dim3(256), 0, as_stream(stream), x, y, ldy, gate_logits, ld_gate, gate_bias, (int64_t)rows, n);
    count_launch();
    check_launch("gated_residual_add");
}

void glu_packed(const float* gate_up, void* out, int64_t rows, int32_t ff, int64_t ld, int32_t act, float limit, const float* row_scale, const int32_t* scale_index,
                int32_t out_dtype, int64_t stream) {
    if (rows == 0 || ff == 0) return;
    B200_REQUIRE(gate_up && out && rows > 0 && ff > 0 && ld >= (act == 3 ? 1 : 2) * (int64_t)ff && act >= 0 && act <= 3 && (row_scale || !scale_index), kErrBadArg,
                 "glu_packed: bad arguments");
    const unsigned grid = (unsigned)((rows * ff + 255) / 256);
    cudaStream_t st = as_stream(stream);
    if (act == 3 && !row_scale && rows <= 0x7fffffff && (out_dtype == B200_F32 || out_dtype == B200_BF16)) {
        const int vec = ff % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0;
        const dim3 g2((unsigned)rows, (unsigned)((ff + 1023) / 1024));
        if (out_dtype == B200_F32) launch_pdl(relu2_rows_kernel<float>, g2, dim3(256), 0, st, gate_up, (float*)out, ff, ld, vec);
        else launch_pdl(relu2_rows_kernel<__nv_bfloat16>, g2, dim3(256), 0, st, gate_up, (__nv_bfloat16*)out, ff, ld, vec);
        count_launch();
        check_launch("glu_packed");
        return;
    }
    if (out_dtype == B200_F32) launch_pdl(glu_packed_kernel<float>, dim3(grid), dim3(256), 0, st, gate_up, (float*)out, rows, ff, ld, act, limit, row_scale, scale_index);
    else if (out_dtype == B200_BF16)
        launch_pdl(glu_packed_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, gate_up, (__nv_bfloat16*)out, rows, ff, ld, act, limit, row_scale, scale_index);
    else { set_error(kErrUnsupported, "glu_packed: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("glu_packed");
}

void group_rms_norm_gate(const float* o, int64_t ldo, const float* weight, const float* gate, int64_t ld_gate, void* out, int32_t num_tokens, int32_t n,
                         int32_t groups, float eps, int32_t gate_act, int32_t out_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(o && out && n > 0 && groups > 0 && n % groups == 0 && ldo >= n && (!gate || ld_gate >= n) && groups <= 65535 && (gate_act == 0 || gate_act == 1),
                 kErrBadArg, "group_rms_norm_gate: bad arguments");
    cudaStream_t st = as_stream(stream);
    const dim3 grid(groups, num_tokens);
    if (out_dtype == B200_F32)
        launch_pdl(group_rms_norm_gate_kernel<float>, grid, dim3(128), 0, st, o, ldo, weight, gate, ld_gate, (float*)out, n, n / groups, eps, gate_act);
    else if (out_dtype == B200_BF16)
        launch_pdl(group_rms_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, o, ldo, weight, gate, ld_gate, (__nv_bfloat16*)out, n, n / groups, eps, gate_act);
    else { set_error(kErrUnsupported, "group_rms_norm_gate: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("group_rms_norm_gate");
}

void head_gate(const void* src, int32_t src_dtype, const float* gate, int64_t ld_gate, void* out, int32_t out_dtype, int32_t num_tokens, int32_t num_heads, int32_t dv,
               int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(src && gate && out && num_heads > 0 && dv > 0 && ld_gate >= num_heads, kErrBadArg, "head_gate: bad arguments");
    B200_REQUIRE(num_tokens <= 65535, kErrUnsupported, "head_gate: at most 65535 rows per call");
    const dim3 grid((unsigned)(((int64_t)num_heads * dv + 1023) / 1024), (unsigned)num_tokens);
    cudaStream_t st = as_stream(stream);
#define HG(TS, TO) launch_pdl(head_gate_kernel<TS, TO>, grid, dim3(256), 0, st, (const TS*)src, gate, ld_gate, (TO*)out, num_heads, dv)
    if (src_dtype == B200_F32 && out_dtype == B200_F32) HG(float, float);
    else if (src_dtype == B200_F32 && out_dtype == B200_BF16) HG(float, __nv_bfloat16);
    else if (src_dtype == B200_BF16 && out_dtype == B200_BF16) HG(__nv_bfloat16, __nv_bfloat16);
    else { set_error(kErrUnsupported, "head_gate: source dtype %d / out dtype %d", src_dtype, out_dtype); return; }
#undef HG
    count_launch();
    check_launch("head_gate");
}

void gated_add_layer_norm(float* x, const float* y, int64_t ldy, const float* gate_logits, int64_t ld_gate, const float* gate_bias, const float* weight, const float* bias,
                          void* out, float* out32, int32_t rows, int32_t n, float eps, int32_t out_dtype, int64_t stream) {
    if (rows == 0) return;
    B200_REQUIRE(x && y && weight && (out || out32) && rows > 0 && n > 0 && ldy >= n && (!gate_logits || ld_gate >= n), kErrBadArg, "gated_add_layer_norm: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32)
        launch_pdl(gated_add_layer_norm_kernel<float>, dim3(rows), dim3(256), 0, st, x, y, ldy, gate_logits, ld_gate, gate_bias, weight, bias, (float*)out, out32, n, eps);
    else if (out_dtype == B200_BF16)
        launch_pdl(gated_add_layer_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, st, x, y, ldy, gate_logits, ld_gate, gate_bias, weight, bias, (__nv_bfloat16*)out,
                   out32, n, eps);
    else { set_error(kErrUnsupported, "gated_add_layer_norm: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("gated_add_layer_norm");
}

void add_rms_norm(float* x, const float* y1, int64_t ld1, const float* y2, int64_t ld2, const float* weight, void* out, const int32_t* row_index, int32_t rows,
                  int32_t n, float eps, int32_t out_dtype, int64_t stream) {
    if (rows == 0) return;
    B200_REQUIRE(x && rows > 0 && n > 0 && (!y1 || ld1 >= n) && (!y2 || ld2 >= n) && ((weight == nullptr) == (out == nullptr)), kErrBadArg, "add_rms_norm: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (!out || out_dtype == B200_F32) launch_pdl(add_rms_norm_kernel<float>, dim3(rows), dim3(256), 0, st, x, y1, ld1, y2, ld2, weight, (float*)out, row_index, n, eps);
    else if (out_dtype == B200_BF16) launch_pdl(add_rms_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, st, x, y1, ld1, y2, ld2, weight, (__nv_bfloat16*)out, row_index, n, eps);
    else { set_error(kErrUnsupported, "add_rms_norm: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("add_rms_norm");
}

}  // extern "C"
