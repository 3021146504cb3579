// linear_generic.cu -- y[m, n] (f32) = x[m, k] . w[n, k]^T for operands of one type, f32 or bf16, any m / n / k.
//
// Two jobs:
//   * models served in true 32-bit (no tensor-core mode rounds an fp32 operand): a tiled SIMT kernel, one fmaf per product, the
//     k index walked in ascending order by a single thread per output element, so a row's result does not depend on how many
//     other rows the call carries;
//   * bf16 operands whose shape the tcgen05 kernel of dense_gemm.cu cannot take (k not a multiple of 8, unaligned rows).
// `linear_f32out` is the dispatcher: bf16 operands that satisfy the TMA rules go to dense_gemm_16 with an f32 epilogue
// (16-bit products, fp32 accumulation in TMEM), everything else runs here.
#include "common.cuh"
#include "qmatmul.cuh"

namespace b200 {
namespace {

constexpr int kTM = 64, kTN = 64, kTK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
linear_generic_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ y, int m, int n, int k, int64_t ldx,
                      int64_t ldw, int64_t ldy) {
    pdl_wait();
    pdl_trigger();
    __shared__ float xs[kTK][kTM + 4], ws[kTK][kTN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * kTM, col0 = blockIdx.x * kTN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < k; k0 += kTK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256, r = idx >> 4, c = idx & 15;
            const int gr = row0 + r, gc = k0 + c, wr = col0 + r;
            xs[c][r] = (gr < m && gc < k) ? to_f32<T>(x[(int64_t)gr * ldx + gc]) : 0.f;
            ws[c][r] = (wr < n && gc < k) ? to_f32<T>(w[(int64_t)wr * ldw + gc]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTK; ++kk) {
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
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < n) y[(int64_t)gr * ldy + gc] = acc[i][j];
        }
    }
}

// few rows (decode): one warp per output element pair would waste the tile above; here a warp owns one weight row and up to
// 4 activation rows, lanes stride k, fixed-order butterfly at the end.
template <typename T>
__global__ void __launch_bounds__(256)
linear_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ y, int m, int n, int k, int64_t ldx, int64_t ldw,
                   int64_t ldy) {
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 8 + warp;
    const int r0 = blockIdx.y * 4;
    if (col >= n) return;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const T* wr = w + (int64_t)col * ldw;
    for (int i = lane; i < k; i += 32) {
        const float wv = to_f32<T>(wr[i]);
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r0 + r < m) acc[r] = fmaf(to_f32<T>(x[(int64_t)(r0 + r) * ldx + i]), wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float s = warp_sum(acc[r]);
        if (lane == 0 && r0 + r < m) y[(int64_t)(r0 + r) * ldy + col] = s;
    }
}

template <typename T>
void launch_generic(const void* x, const void* w, float* y, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldy, cudaStream_t st) {
    if (m <= 8)
        launch_pdl(linear_rows_kernel<T>, dim3(ceil_div(n, 8), ceil_div(m, 4)), dim3(256), 0, st, (const T*)x, (const T*)w, y, m, n, k, ldx, ldw, ldy);
    else
        launch_pdl(linear_generic_kernel<T>, dim3(ceil_div(n, kTN), ceil_div(m, kTM)), dim3(256), 0, st, (const T*)x, (const T*)w, y, m, n, k, ldx, ldw, ldy);
    count_launch();
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void linear_f32out(const void* x, const void* weight, float* out, int32_t m, int32_t n, int32_t k, int64_t ldx, int64_t ldy, int32_t dtype,
                   int64_t stream) {
    if (m == 0 || n == 0) return;
    B200_REQUIRE(x && weight && out && m > 0 && n > 0 && k > 0 && ldx >= k && ldy >= n, kErrBadArg, "linear_f32out: bad arguments");
    cudaStream_t st = as_stream(stream);
    if (dtype == B200_BF16) {
        const bool tma_ok = k % 8 == 0 && ldx % 8 == 0 && ((((uintptr_t)x) | ((uintptr_t)weight)) & 15) == 0 && k >= 64;
        if (tma_ok) {
            // few rows = a pure weight stream: with fewer 128-row weight tiles than SMs the kernel cuts k so that every SM streams a part and
            // the parts meet in fp32 atomics on a zeroed output (the condition mirrors dense_gemm_16's own)
            int split = 0;
            if (m <= 64) {
                const int tiles = (n + 127) / 128, nkb = (k + 63) / 64;
                int ks = tiles < sm_count() ? sm_count() / tiles : 1;
                if (ks > nkb / 4) ks = nkb / 4;
                split = ks > 1 ? 1 : 0;
            }
            if (split) {
                if (ldy == n) cudaMemsetAsync(out, 0, (size_t)m * n * sizeof(float), st);
                else cudaMemset2DAsync(out, (size_t)ldy * sizeof(float), 0, (size_t)n * sizeof(float), (size_t)m, st);
            }
            dense_gemm_16(x, weight, nullptr, out, m, n, k, ldx, k, ldy, B200_BF16, B200_F32, st, 0, split);
            return;
        }
        launch_generic<__nv_bfloat16>(x, weight, out, m, n, k, ldx, k, ldy, st);
    } else if (dtype == B200_F32) {
        launch_generic<float>(x, weight, out, m, n, k, ldx, k, ldy, st);
    } else {
        set_error(kErrUnsupported, "linear_f32out: dtype %d (f32 / bf16)", dtype);
        return;
    }
    check_launch("linear_f32out");
}

}  // extern "C"
