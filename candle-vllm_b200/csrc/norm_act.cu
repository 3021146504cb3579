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

}  // extern "C"
