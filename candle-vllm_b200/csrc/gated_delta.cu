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
//                           softplus(a + dt_bias)).  A block owns 16 value columns of one head of one entry with its slice of S in
//                           registers and walks the portion in tiles of 16 tokens staged through shared memory, the next
//                           tile in flight while the current one is applied.  Decode (one token per entry) is one read and
//                           one write of the state.
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
    pdl_wait();
    pdl_trigger();
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
    pdl_wait();
    pdl_trigger();
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

// A block of four warps owns 16 value columns of one head of one entry (4 per warp); inside a warp the key rows are split eight ways
// (lane = 4 * part + column, part p holds rows p * kR .. p * kR + kR - 1 of its column in registers), so a token costs kR multiply-adds
// per lane per pass instead of dk and three butterfly steps join the eight partial sums.  kR = rows per part (dk <= 8 * kR; rows past dk
// are zero and stay zero).  The state is stored [slot, head, column, row]: a lane's rows are contiguous (16-byte loads and stores).
// Tokens are taken in tiles of 16: the block loads the NEXT tile's q, k, v, a, b into registers (coalesced, all in flight at once) while
// it walks the current tile out of shared memory, where q and k were made unit vectors and beta, decay and k . q were worked out for all
// 16 tokens in parallel.  Both read-outs of a token are taken from the state as the previous token left it (S0^T k and S0^T q; the
// current token's write enters the output as u (k . q)), so the serial part of a token is one pass of multiply-adds, one butterfly
// round that joins both sums, and the update pass.
// Every sum has a fixed order, so portions of any size give the same state bit for bit.
constexpr int kTile = 16;

template <int kR>
__global__ void __launch_bounds__(128)
gated_delta_rule_kernel(const float* __restrict__ qkv, const float* __restrict__ proj, int64_t ld_proj, int off_b, int off_a,
                        const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ state, float* __restrict__ out,
                        const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start,
                        int H, int G, int dk, int dv) {
    pdl_wait();
    pdl_trigger();
    constexpr int kDP = 8 * kR;                       // padded key size
    constexpr int kNQ = kTile * kDP / 128;            // q (and k) elements a thread stages per tile
    extern __shared__ float sm[];
    float* qs = sm;                                   // [kTile][kDP]
    float* ks = qs + kTile * kDP;                     // [kTile][kDP]
    float* vs = ks + kTile * kDP;                     // [kTile][16]
    float* bs = vs + kTile * 16;                      // [kTile] b, then beta
    float* ds = bs + kTile;                           // [kTile] a, then decay
    float* kqs = ds + kTile;                          // [kTile] k . q of the unit vectors
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, part = lane >> 2;
    const int b = blockIdx.z, h = blockIdx.y;
    const int col = blockIdx.x * 16 + warp * 4 + (lane & 3);
    const bool live = col < dv;
    const int g = h / (H / G);
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (n <= 0) return;
    const int C = 2 * G * dk + H * dv;
    const int row0 = part * kR;
    float* Sg = state + (((int64_t)seq_slots[b] * H + h) * dv + (live ? col : 0)) * dk + row0;
    const bool fresh = seq_start[b] == 0;
    const bool vec = (dk & 3) == 0 && row0 + kR <= dk;           // this lane's rows: whole float4s inside the key size
    float S[kR];
    if (live && !fresh && vec) {
#pragma unroll
        for (int r = 0; r < kR; r += 4) {
            const float4 t4 = *reinterpret_cast<const float4*>(Sg + r);
            S[r] = t4.x; S[r + 1] = t4.y; S[r + 2] = t4.z; S[r + 3] = t4.w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < kR; ++r) S[r] = (live && !fresh && row0 + r < dk) ? Sg[r] : 0.f;
    }
    const float neg_rate = -expf(A_log[h]);
    const float bias = dt_bias[h];
    const float qscale = 1.0f / sqrtf((float)dk);

    float rq[kNQ], rk[kNQ], rv[kTile * 16 / 128], ra = 0.f, rb = 0.f;
    auto load_tile = [&](int first, int cnt) {        // global -> registers
#pragma unroll
        for (int j = 0; j < kNQ; ++j) {
            const int e = tid + 128 * j, tt = e / kDP, i = e - tt * kDP;
            const bool in = tt < cnt && i < dk;
            const float* row = qkv + (int64_t)(first + tt) * C + g * dk + i;
            rq[j] = in ? row[0] : 0.f;
            rk[j] = in ? row[G * dk] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kTile * 16 / 128; ++j) {
            const int e = tid + 128 * j, tt = e >> 4, c = blockIdx.x * 16 + (e & 15);
            rv[j] = (tt < cnt && c < dv) ? qkv[(int64_t)(first + tt) * C + 2 * G * dk + h * dv + c] : 0.f;
        }
        if (tid < kTile && tid < cnt) {
            rb = proj[(int64_t)(first + tid) * ld_proj + off_b + h];
            ra = proj[(int64_t)(first + tid) * ld_proj + off_a + h];
        }
    };
    auto store_tile = [&]() {                          // registers -> shared memory
#pragma unroll
        for (int j = 0; j < kNQ; ++j) { qs[tid + 128 * j] = rq[j]; ks[tid + 128 * j] = rk[j]; }
#pragma unroll
        for (int j = 0; j < kTile * 16 / 128; ++j) vs[tid + 128 * j] = rv[j];
        if (tid < kTile) { bs[tid] = rb; ds[tid] = ra; }
    };
    auto prepare_tile = [&](int cnt) {                 // unit vectors, beta, decay: 4 tokens per warp, in parallel
        for (int tt = warp; tt < cnt; tt += 4) {
            float qq = 0.f, kk = 0.f, qk = 0.f;
            for (int i = lane; i < kDP; i += 32) {
                const float a = qs[tt * kDP + i], c = ks[tt * kDP + i];
                qq = fmaf(a, a, qq); kk = fmaf(c, c, kk); qk = fmaf(a, c, qk);
            }
            qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
            const float qn = qscale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
            for (int i = lane; i < kDP; i += 32) { qs[tt * kDP + i] *= qn; ks[tt * kDP + i] *= kn; }
            if (lane == 0) {
                kqs[tt] = qk * qn * kn;
                bs[tt] = 1.0f / (1.0f + expf(-bs[tt]));
                ds[tt] = expf(neg_rate * softplus_f(ds[tt] + bias));
            }
        }
    };
    auto join8 = [](float& a, float& c) {              // sums over the eight parts (lanes that differ in bits 2, 3 and 4), two at a time
#pragma unroll
        for (int m = 4; m <= 16; m <<= 1) {
            const float x = __shfl_xor_sync(0xffffffffu, a, m), y = __shfl_xor_sync(0xffffffffu, c, m);
            a += x; c += y;
        }
    };

    const int tiles = (n + kTile - 1) / kTile;
    load_tile(t0, min(kTile, n));
    for (int tile = 0; tile < tiles; ++tile) {
        const int first = t0 + tile * kTile, cnt = min(kTile, n - tile * kTile);
        __syncthreads();                               // every warp has finished the previous tile
        store_tile();
        __syncthreads();
        prepare_tile(cnt);
        __syncthreads();
        if (tile + 1 < tiles) load_tile(first + kTile, min(kTile, n - (tile + 1) * kTile));
        for (int tt = 0; tt < cnt; ++tt) {
            const float4* k4 = reinterpret_cast<const float4*>(ks + tt * kDP + row0);
            const float4* q4 = reinterpret_cast<const float4*>(qs + tt * kDP + row0);
            const float decay = ds[tt], beta = bs[tt], kq = kqs[tt], v = vs[tt * 16 + warp * 4 + (lane & 3)];
            // both read-outs of the state as the previous token left it, S0: with S = g S0 + k u^T,
            //   S0^T k -> u = beta (v - g S0^T k)   and   S^T q = g S0^T q + u (k . q),
            // so one butterfly round per token joins both sums and the update is one pass
            float kd[kR];
            float p[4] = {0.f, 0.f, 0.f, 0.f}, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < kR; r += 4) {
                const float4 c = k4[r >> 2], a = q4[r >> 2];
                kd[r] = c.x; kd[r + 1] = c.y; kd[r + 2] = c.z; kd[r + 3] = c.w;
                p[0] = fmaf(S[r], c.x, p[0]); p[1] = fmaf(S[r + 1], c.y, p[1]); p[2] = fmaf(S[r + 2], c.z, p[2]); p[3] = fmaf(S[r + 3], c.w, p[3]);
                o[0] = fmaf(S[r], a.x, o[0]); o[1] = fmaf(S[r + 1], a.y, o[1]); o[2] = fmaf(S[r + 2], a.z, o[2]); o[3] = fmaf(S[r + 3], a.w, o[3]);
            }
            float pk = (p[0] + p[1]) + (p[2] + p[3]), pq = (o[0] + o[1]) + (o[2] + o[3]);
            join8(pk, pq);
            const float u = beta * (v - decay * pk);
            const float ov = fmaf(u, kq, decay * pq);
#pragma unroll
            for (int r = 0; r < kR; ++r) S[r] = fmaf(kd[r], u, decay * S[r]);
            if (live && part == 0) out[(int64_t)(first + tt) * H * dv + h * dv + col] = ov;
        }
    }
    if (live) {
        if (vec) {
#pragma unroll
            for (int r = 0; r < kR; r += 4) *reinterpret_cast<float4*>(Sg + r) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
        } else {
#pragma unroll
            for (int r = 0; r < kR; ++r)
                if (row0 + r < dk) Sg[r] = S[r];
        }
    }
}

template <typename TOut>
__global__ void __launch_bounds__(128)
gated_rms_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int64_t ld_gate, const float* __restrict__ w,
                      TOut* __restrict__ out, int64_t items, int H, int dv, float eps) {
    pdl_wait();
    pdl_trigger();
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
    launch_pdl(causal_conv_silu_kernel, dim3(ceil_div(channels, 128), num_tokens), dim3(128), 0, st, x, ldx, taps, (const float*)conv_state, y, token_seq,
               cu_seqlens, seq_slots, seq_start, channels, num_taps);
    count_launch();
    if (num_taps > 1) {
        launch_pdl(causal_conv_update_kernel, dim3(ceil_div(channels, 128), num_seqs), dim3(128), 0, st, x, ldx, conv_state, cu_seqlens, seq_slots, seq_start,
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
    const dim3 grid(ceil_div(dv, 16), num_heads, num_seqs);
#define GDR(R) do { \
        const int smem = (2 * kTile * 8 * R + kTile * 16 + 3 * kTile) * (int)sizeof(float); \
        ensure_dynamic_smem(reinterpret_cast<const void*>(gated_delta_rule_kernel<R>), smem); \
        launch_pdl(gated_delta_rule_kernel<R>, grid, dim3(128), smem, st, qkv, proj, ld_proj, off_b, off_a, A_log, dt_bias, state, out, cu_seqlens, seq_slots, \
                   seq_start, num_heads, num_kv_heads, dk, dv); } while (0)
    if (dk <= 32) GDR(4);
    else if (dk <= 64) GDR(8);
    else if (dk <= 128) GDR(16);
    else GDR(32);
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
    if (out_dtype == B200_F32) launch_pdl(gated_rms_norm_kernel<float>, dim3(grid), dim3(128), 0, st, o, gate, ld_gate, weight, (float*)out, items, num_heads, dv, eps);
    else if (out_dtype == B200_BF16) launch_pdl(gated_rms_norm_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, o, gate, ld_gate, weight, (__nv_bfloat16*)out, items, num_heads, dv, eps);
    else { set_error(kErrUnsupported, "gated_rms_norm: out dtype %d (f32 / bf16)", out_dtype); return; }
    count_launch();
    check_launch("gated_rms_norm");
}

}  // extern "C"
