// gated_delta.cu -- the recurrent mixer family "short convolution -> gated delta rule -> gated norm", for ragged steps.
//
// A step carries B entries; entry b owns the rows cu_seqlens[b] .. cu_seqlens[b+1] of the flat token arrays (a portion of a
// prompt or one decoded token), continues the sequence whose state lives in slot seq_slots[b], and starts at position
// seq_start[b] of that sequence.  seq_start[b] == 0 means "new sequence": the slot's old contents are ignored (treated as
// zero), so a slot needs no clearing when it is handed to another request.  All state is f32.
//
//   causal_conv_silu        y[t, c] = silu(sum_d taps[c, K-1-d] * x[t-d, c]); inputs before the portion come from
//                           conv_state[slot] = the last K-1 input rows of the sequence ([slots, K-1, C]).
//   causal_conv_update      rolls conv_state[slot] forward over the portion (run after causal_conv_silu: it overwrites
//                           what that kernel reads).
//   gated_delta_rule        per head, S [dk, dv]:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                           with q, k made unit vectors (q also times dk^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) *
//                           softplus(a + dt_bias)).  One warp owns 32 value columns of one head of one entry and walks the
//                           portion token by token with its slice of S in registers (dk <= 128) or shared memory; the next
//                           token's operands are fetched while the current one is applied.  Decode (one token per entry) is
//                           one read and one write of the state.
//   gated_rms_norm          out = o / rms(o over dv) * w * silu(gate), per (token, head).
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__global__ void __launch_bounds__(128)
causal_conv_silu_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ taps, const float* __restrict__ conv_state,
                        float* __restrict__ y, const int32_t* __restrict__ token_seq, const int32_t* __restrict__ cu_seqlens,
                        const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int C, int K) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= C) return;
    const int b = token_seq[t];
    const int i = t - cu_seqlens[b];
    const bool fresh = seq_start[b] == 0;
    const float* st = conv_state + (int64_t)seq_slots[b] * (K - 1) * C;
    float acc = 0.f;
    for (int d = K - 1; d >= 0; --d) {            // oldest input first
        const int src = i - d;
        float v;
        if (src >= 0) v = x[(int64_t)(t - d) * ldx + c];
        else v = fresh ? 0.f : st[(int64_t)(K - 1 + src) * C + c];
        acc = fmaf(taps[(int64_t)c * K + (K - 1 - d)], v, acc);
    }
    y[(int64_t)t * C + c] = silu_f(acc);
}

__global__ void __launch_bounds__(128)
causal_conv_update_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ conv_state, const int32_t* __restrict__ cu_seqlens,
                          const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int C, int K) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (n <= 0) return;
    const bool fresh = seq_start[b] == 0;
    float* st = conv_state + (int64_t)seq_slots[b] * (K - 1) * C;
    // the sequence's inputs so far are [old state rows 0 .. K-2][portion rows 0 .. n-1]; keep the last K-1 of them.  Row j of the
    // new state is element n + j of that list: j ascends and n >= 1, so an old row is read before it is overwritten.
    for (int j = 0; j < K - 1; ++j) {
        const int e = n + j;
        float v;
        if (e >= K - 1) v = x[(int64_t)(t0 + e - (K - 1)) * ldx + c];
        else v = fresh ? 0.f : st[(int64_t)e * C + c];
        st[(int64_t)j * C + c] = v;
    }
}

// kDK > 0: dk == kDK, state slice in registers.  kDK == 0: any dk <= 256, state slice in shared memory [dk][32].
template <int kDK>
__global__ void __launch_bounds__(32)
gated_delta_rule_kernel(const float* __restrict__ qkv, const float* __restrict__ proj, int64_t ld_proj, int off_b, int off_a,
                        const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ state, float* __restrict__ out,
                        const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start,
                        int H, int G, int dk_rt, int dv) {
    extern __shared__ float smem[];
    const int dk = kDK > 0 ? kDK : dk_rt;
    constexpr int kPer = kDK > 0 ? (kDK + 31) / 32 : 8;       // q / k elements a lane stages per token
    float* ks = smem;                 // [dk] unit key of the current token
    float* qs = smem + dk;            // [dk] scaled unit query
    float* Ss = smem + 2 * dk;        // [dk][32] when kDK == 0
    const int lane = threadIdx.x;
    const int b = blockIdx.z, h = blockIdx.y;
    const int col = blockIdx.x * 32 + lane;
    const bool live = col < dv;
    const int g = h / (H / G);
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (n <= 0) return;
    const int C = 2 * G * dk + H * dv;
    float* Sg = state + (((int64_t)seq_slots[b] * H + h) * dk) * dv + col;
    const bool fresh = seq_start[b] == 0;
    float S[kDK > 0 ? kDK : 1];
    if constexpr (kDK > 0) {
#pragma unroll
        for (int i = 0; i < kDK; ++i) S[i] = (live && !fresh) ? Sg[(int64_t)i * dv] : 0.f;
    } else {
        for (int i = 0; i < dk; ++i) Ss[i * 32 + lane] = (live && !fresh) ? Sg[(int64_t)i * dv] : 0.f;
    }
    const float neg_rate = -expf(A_log[h]);
    const float bias = dt_bias[h];
    const float qscale = 1.0f / sqrtf((float)dk);

    float kr[kPer], qr[kPer], vr, ar, br;
    auto fetch = [&](int t) {
        const float* row = qkv + (int64_t)t * C;
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const int i = lane + 32 * e;
            qr[e] = i < dk ? row[g * dk + i] : 0.f;
            kr[e] = i < dk ? row[G * dk + g * dk + i] : 0.f;
        }
        vr = live ? row[2 * G * dk + h * dv + col] : 0.f;
        br = proj[(int64_t)t * ld_proj + off_b + h];
        ar = proj[(int64_t)t * ld_proj + off_a + h];
    };
    fetch(t0);
    for (int s = 0; s < n; ++s) {
        const int t = t0 + s;
        // unit vectors (32-bit), staged for broadcast
        float qq = 0.f, kk = 0.f;
#pragma unroll
        for (int e = 0; e < kPer; ++e) { qq = fmaf(qr[e], qr[e], qq); kk = fmaf(kr[e], kr[e], kk); }
        qq = warp_sum(qq); kk = warp_sum(kk);
        const float qn = qscale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
        __syncwarp();
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const int i = lane + 32 * e;
            if (i < dk) { qs[i] = qr[e] * qn; ks[i] = kr[e] * kn; }
        }
        const float v = vr;
        const float beta = 1.0f / (1.0f + expf(-br));
        const float decay = expf(neg_rate * softplus_f(ar + bias));
        __syncwarp();
        if (s + 1 < n) fetch(t + 1);
        float pred = 0.f, o = 0.f;
        if constexpr (kDK > 0) {
#pragma unroll
            for (int i = 0; i < kDK; ++i) { S[i] *= decay; pred = fmaf(S[i], ks[i], pred); }
            const float u = beta * (v - pred);
#pragma unroll
            for (int i = 0; i < kDK; ++i) { S[i] = fmaf(ks[i], u, S[i]); o = fmaf(S[i], qs[i], o); }
        } else {
            for (int i = 0; i < dk; ++i) { const float sv = Ss[i * 32 + lane] * decay; Ss[i * 32 + lane] = sv; pred = fmaf(sv, ks[i], pred); }
            const float u = beta * (v - pred);
            for (int i = 0; i < dk; ++i) { const float sv = fmaf(ks[i], u, Ss[i * 32 + lane]); Ss[i * 32 + lane] = sv; o = fmaf(sv, qs[i], o); }
        }
        if (live) out[(int64_t)t * H * dv + h * dv + col] = o;
    }
    if (live) {
        if constexpr (kDK > 0) {
#pragma unroll
            for (int i = 0; i < kDK; ++i) Sg[(int64_t)i * dv] = S[i];
        } else {
            for (int i = 0; i < dk; ++i) Sg[(int64_t)i * dv] = Ss[i * 32 + lane];
        }
    }
}

template <typename TOut>
__global__ void __launch_bounds__(128)
gated_rms_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int64_t ld_gate, const float* __restrict__ w,
                      TOut* __restrict__ out, int64_t items, int H, int dv, float eps) {
    const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= items) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const float* orow = o + (t * H + h) * dv;
    const float* grow = gate + t * ld_gate + (int64_t)h * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) { const float v = orow[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float sc = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) out[(t * H + h) * dv + i] = from_f32<TOut>(orow[i] * sc * w[i] * silu_f(grow[i]));
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void causal_conv_silu(const float* x, int64_t ldx, const float* taps, float* conv_state, float* y, const int32_t* token_seq,
                      const int32_t* cu_seqlens, const int32_t* seq_slots, const int32_t* seq_start, int32_t num_tokens, int32_t num_seqs,
                      int32_t channels, int32_t num_taps, int64_t stream) {
    if (num_tokens == 0 || num_seqs == 0) return;
    B200_REQUIRE(x && taps && conv_state && y && token_seq && cu_seqlens && seq_slots && seq_start && channels > 0 && num_taps >= 1 &&
                 ldx >= channels, kErrBadArg, "causal_conv_silu: bad arguments");
    cudaStream_t st = as_stream(stream);
    causal_conv_silu_kernel<<<dim3(ceil_div(channels, 128), num_tokens), 128, 0, st>>>(x, ldx, taps, conv_state, y, token_seq, cu_seqlens,
                                                                                         seq_slots, seq_start, channels, num_taps);
    count_launch();
    if (num_taps > 1) {
        causal_conv_update_kernel<<<dim3(ceil_div(channels, 128), num_seqs), 128, 0, st>>>(x, ldx, conv_state, cu_seqlens, seq_slots, seq_start,
                                                                                            channels, num_taps);
        count_launch();
    }
    check_launch("causal_conv_silu");
}

void gated_delta_rule(const float* qkv, const float* proj, int64_t ld_proj, int32_t off_b, int32_t off_a, const float* A_log,
                      const float* dt_bias, float* state, float* out, const int32_t* cu_seqlens, const int32_t* seq_slots,
                      const int32_t* seq_start, int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t dk, int32_t dv,
                      int64_t stream) {
    if (num_seqs == 0) return;
    B200_REQUIRE(qkv && proj && A_log && dt_bias && state && out && cu_seqlens && seq_slots && seq_start, kErrBadArg, "gated_delta_rule: null pointer");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0, kErrBadArg, "gated_delta_rule: bad head counts");
    B200_REQUIRE(dk <= 256, kErrUnsupported, "gated_delta_rule: key size %d > 256", dk);
    cudaStream_t st = as_stream(stream);
    const dim3 grid(ceil_div(dv, 32), num_heads, num_seqs);
#define GDR(DK, SMEM) gated_delta_rule_kernel<DK><<<grid, 32, (SMEM), st>>>(qkv, proj, ld_proj, off_b, off_a, A_log, dt_bias, state, out, cu_seqlens, \
                                                                          seq_slots, seq_start, num_heads, num_kv_heads, dk, dv)
    if (dk == 32) GDR(32, 2 * 32 * 4);
    else if (dk == 64) GDR(64, 2 * 64 * 4);
    else if (dk == 128) GDR(128, 2 * 128 * 4);
    else GDR(0, (2 * dk + 32 * dk) * 4);
#undef GDR
    count_launch();
    check_launch("gated_delta_rule");
}

void gated_rms_norm(const float* o, const float* gate, int64_t ld_gate, const float* weight, void* out, int32_t num_tokens, int32_t num_heads,
                    int32_t dv, float eps, int32_t out_dtype, int64_t stream) {
    if (num_tokens == 0) return;
    B200_REQUIRE(o && gate && weight && out && num_heads > 0 && dv > 0, kErrBadArg, "gated_rms_norm: bad arguments");
    const int64_t items = (int64_t)num_tokens * num_heads;
    const unsigned grid = (unsigned)((items + 3) / 4);
    cudaStream_t st = as_stream(stream);
    if (out_dtype == B200_F32) gated_rms_norm_kernel<float><<<grid, 128, 0, st>>>(o, gate, ld_gate, weight, (float*)out, items, num_heads, dv, eps);
    else if (out_dtype == B200_BF16) gated_rms_norm_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(o, gate, ld_gate, weight, (__nv_bfloat16*)out, items, num_heads, dv, eps);
    else { set_error(kErrUnsupported, "gated_rms_norm: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("gated_rms_norm");
}

}  // extern "C"
