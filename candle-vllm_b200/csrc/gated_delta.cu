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

// ---- steps of single tokens ------------------------------------------------------------------------------------------------------
// Every entry brings one token: the work is one read and one write of the state.  Same lane layout as above (4 columns x 8 parts of kR
// rows per warp, 16 columns per block), but nothing is staged: a lane's state loads go out first, every warp works out the token's unit
// norms, k . q, beta and decay for itself (the q / k rows are a few hundred bytes and stay in L1), and a lane reads its own kR entries
// of q and k straight from the rows.  No shared memory, no block-wide barrier, ~80 registers: six and more blocks per SM keep the state
// traffic in flight.  The sums are those of gated_delta_rule_kernel in the same order.
template <int kR>
__global__ void __launch_bounds__(128)
gated_delta_step_kernel(const float* __restrict__ qkv, const float* __restrict__ proj, int64_t ld_proj, int off_b, int off_a,
                        const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ state, float* __restrict__ out,
                        const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start, int H, int G, int dk, int dv) {
    pdl_wait();
    pdl_trigger();
    constexpr int kDP = 8 * kR;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, part = lane >> 2;
    const int t = blockIdx.z, h = blockIdx.y;          // entry = row
    const int col = blockIdx.x * 16 + warp * 4 + (lane & 3);
    const bool live = col < dv;
    const int g = h / (H / G);
    const int C = 2 * G * dk + H * dv;
    const int row0 = part * kR;
    float* Sg = state + (((int64_t)seq_slots[t] * H + h) * dv + (live ? col : 0)) * dk + row0;
    const bool fresh = seq_start[t] == 0;
    const bool vec = (dk & 3) == 0 && row0 + kR <= dk;
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
    const float* qrow = qkv + (int64_t)t * C + g * dk;
    const float* krow = qrow + G * dk;
    float kd[kR], qd[kR];
    if (vec && (C & 3) == 0) {
#pragma unroll
        for (int r = 0; r < kR; r += 4) {
            const float4 c = *reinterpret_cast<const float4*>(krow + row0 + r), a = *reinterpret_cast<const float4*>(qrow + row0 + r);
            kd[r] = c.x; kd[r + 1] = c.y; kd[r + 2] = c.z; kd[r + 3] = c.w;
            qd[r] = a.x; qd[r + 1] = a.y; qd[r + 2] = a.z; qd[r + 3] = a.w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < kR; ++r) {
            const bool in = row0 + r < dk;
            kd[r] = in ? krow[row0 + r] : 0.f;
            qd[r] = in ? qrow[row0 + r] : 0.f;
        }
    }
    const float v = live ? qkv[(int64_t)t * C + 2 * G * dk + h * dv + col] : 0.f;
    float qq = 0.f, kk = 0.f, qk = 0.f;
    for (int i = lane; i < kDP; i += 32) {
        const float a = i < dk ? qrow[i] : 0.f, c = i < dk ? krow[i] : 0.f;
        qq = fmaf(a, a, qq); kk = fmaf(c, c, kk); qk = fmaf(a, c, qk);
    }
    qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
    const float qn = (1.0f / sqrtf((float)dk)) / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
    const float kq = qk * qn * kn;
    const float beta = 1.0f / (1.0f + expf(-proj[(int64_t)t * ld_proj + off_b + h]));
    const float decay = expf(-expf(A_log[h]) * softplus_f(proj[(int64_t)t * ld_proj + off_a + h] + dt_bias[h]));
    float p[4] = {0.f, 0.f, 0.f, 0.f}, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kR; r += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            kd[r + j] *= kn; qd[r + j] *= qn;
            p[j] = fmaf(S[r + j], kd[r + j], p[j]);
            o[j] = fmaf(S[r + j], qd[r + j], o[j]);
        }
    }
    float pk = (p[0] + p[1]) + (p[2] + p[3]), pq = (o[0] + o[1]) + (o[2] + o[3]);
#pragma unroll
    for (int m = 4; m <= 16; m <<= 1) {
        const float x = __shfl_xor_sync(0xffffffffu, pk, m), y = __shfl_xor_sync(0xffffffffu, pq, m);
        pk += x; pq += y;
    }
    const float u = beta * (v - decay * pk);
    const float ov = fmaf(u, kq, decay * pq);
#pragma unroll
    for (int r = 0; r < kR; ++r) S[r] = fmaf(kd[r], u, decay * S[r]);
    if (live) {
        if (part == 0) out[(int64_t)t * H * dv + h * dv + col] = ov;
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

// ---- the rule over tiles of 16 tokens -------------------------------------------------------------------------------------------
// Inside a tile that starts from state S0, with decays g_i, P_i = g_0 ... g_i and R_is = g_{s+1} ... g_i:
//     S_i = P_i S0 + sum_{s<=i} R_is k_s u_s^T
//     u_i = beta_i (v_i - P_i S0^T k_i - sum_{s<i} R_is (k_s . k_i) u_s)            (a triangular system, one per value column)
//     o_i = P_i S0^T q_i + sum_{s<=i} R_is (k_s . q_i) u_s
// so the state is read for all 16 tokens at once (32 independent sums per lane), the serial part is 16 short steps on scalars, and the
// state is written once per tile.  Everything that does not depend on the value column -- unit vectors, beta, decays and their
// products, M_is = R_is (k_s . k_i), N_is = R_is (k_s . q_i) -- is worked out by gated_delta_prepare_kernel for all tiles in parallel
// and handed over in `scratch` (floats per step, T rows):
//     kn [T, G, dk] | qn [T, G, dk] | M [T, H, 16] | N [T, H, 16] | P [T, H] | E [T, H] (decay from the token to its tile's end) | beta [T, H]
struct DeltaScratch { float *kn, *qn, *M, *N, *P, *E, *beta; };
__host__ __device__ __forceinline__ DeltaScratch delta_scratch(float* base, int64_t T, int H, int G, int dk) {
    DeltaScratch d;
    d.kn = base;
    d.qn = d.kn + T * G * dk;
    d.M = d.qn + T * G * dk;
    d.N = d.M + T * H * kTile;
    d.P = d.N + T * H * kTile;
    d.E = d.P + T * H;
    d.beta = d.E + T * H;
    return d;
}

// one block per (tile, key/value group, entry)
__global__ void __launch_bounds__(128)
gated_delta_prepare_kernel(const float* __restrict__ qkv, const float* __restrict__ proj, int64_t ld_proj, int off_b, int off_a,
                           const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ scratch,
                           const int32_t* __restrict__ cu_seqlens, int T, int H, int G, int dk, int dv) {
    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, g = blockIdx.y;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if ((int)blockIdx.x * kTile >= n) return;
    const int first = t0 + blockIdx.x * kTile, cnt = min(kTile, n - (int)blockIdx.x * kTile);
    const int ld = ((dk + 3) & ~3) + 4;               // row pitch: whole float4s, rows 4 banks apart
    extern __shared__ float sm[];
    float* qs = sm;                                   // [kTile][ld]
    float* ks = qs + kTile * ld;                      // [kTile][ld]
    float* KK = ks + kTile * ld;                      // [kTile][kTile] k_i . k_s
    float* KQ = KK + kTile * kTile;                   // [kTile][kTile] q_i . k_s
    float* gs = KQ + kTile * kTile;                   // [kTile] decays of one head
    const DeltaScratch sc = delta_scratch(scratch, T, H, G, dk);
    const int C = 2 * G * dk + H * dv;
    for (int e = tid; e < kTile * ld; e += 128) {
        const int tt = e / ld, i = e - tt * ld;
        const bool in = tt < cnt && i < dk;
        const float* row = qkv + (int64_t)(first + tt) * C + g * dk + i;
        qs[e] = in ? row[0] : 0.f;
        ks[e] = in ? row[G * dk] : 0.f;
    }
    __syncthreads();
    const float qscale = 1.0f / sqrtf((float)dk);
    for (int tt = warp; tt < cnt; tt += 4) {
        float qq = 0.f, kk = 0.f;
        for (int i = lane; i < ld; i += 32) { const float a = qs[tt * ld + i], c = ks[tt * ld + i]; qq = fmaf(a, a, qq); kk = fmaf(c, c, kk); }
        qq = warp_sum(qq); kk = warp_sum(kk);
        const float qn = qscale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
        for (int i = lane; i < dk; i += 32) {
            const float a = qs[tt * ld + i] * qn, c = ks[tt * ld + i] * kn;
            qs[tt * ld + i] = a; ks[tt * ld + i] = c;
            sc.qn[((int64_t)(first + tt) * G + g) * dk + i] = a;
            sc.kn[((int64_t)(first + tt) * G + g) * dk + i] = c;
        }
    }
    __syncthreads();
    for (int p = tid; p < kTile * kTile; p += 128) {
        const int i = p >> 4, s = p & 15;
        float kk = 0.f, kq = 0.f;
        if (s <= i && i < cnt) {
            const float4* ki = reinterpret_cast<const float4*>(ks + i * ld);
            const float4* qi = reinterpret_cast<const float4*>(qs + i * ld);
            const float4* kr = reinterpret_cast<const float4*>(ks + s * ld);
            float k2[4] = {0.f, 0.f, 0.f, 0.f}, q2[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < (ld >> 2) - 1; ++r) {
                const float4 x = ki[r], y = qi[r], z = kr[r];
                k2[0] = fmaf(x.x, z.x, k2[0]); k2[1] = fmaf(x.y, z.y, k2[1]); k2[2] = fmaf(x.z, z.z, k2[2]); k2[3] = fmaf(x.w, z.w, k2[3]);
                q2[0] = fmaf(y.x, z.x, q2[0]); q2[1] = fmaf(y.y, z.y, q2[1]); q2[2] = fmaf(y.z, z.z, q2[2]); q2[3] = fmaf(y.w, z.w, q2[3]);
            }
            kk = (k2[0] + k2[1]) + (k2[2] + k2[3]);
            kq = (q2[0] + q2[1]) + (q2[2] + q2[3]);
        }
        KK[p] = kk; KQ[p] = kq;
    }
    const int rep = H / G;
    for (int hh = 0; hh < rep; ++hh) {
        const int h = g * rep + hh;
        __syncthreads();                               // KK / KQ written; the previous head's decays no longer read
        if (tid < kTile) {
            float dec = 1.0f;
            if (tid < cnt) {
                const float a = proj[(int64_t)(first + tid) * ld_proj + off_a + h], bb = proj[(int64_t)(first + tid) * ld_proj + off_b + h];
                dec = expf(-expf(A_log[h]) * softplus_f(a + dt_bias[h]));
                sc.beta[(int64_t)(first + tid) * H + h] = 1.0f / (1.0f + expf(-bb));
            }
            gs[tid] = dec;
        }
        __syncthreads();
        for (int p = tid; p < kTile * kTile; p += 128) {
            const int i = p >> 4, s = p & 15;
            if (i >= cnt) continue;
            float R = 1.0f;
            for (int r = s + 1; r <= i; ++r) R *= gs[r];
            const int64_t at = ((int64_t)(first + i) * H + h) * kTile + s;
            sc.M[at] = s < i ? R * KK[p] : 0.f;
            sc.N[at] = s <= i ? R * KQ[p] : 0.f;
        }
        if (tid < cnt) {
            float P = 1.0f, E = 1.0f;
            for (int r = 0; r <= tid; ++r) P *= gs[r];
            for (int r = tid + 1; r < cnt; ++r) E *= gs[r];
            sc.P[(int64_t)(first + tid) * H + h] = P;
            sc.E[(int64_t)(first + tid) * H + h] = E;
        }
    }
}

// The recurrence itself.  The split is that of gated_delta_rule_kernel: a warp holds 32 / kParts value columns of one head of one entry,
// each column's key rows cut into kParts parts of kR rows (lane = columns-per-warp * part + column), state in registers; a block is four
// warps (kParts = 8: 16 columns per block).  q / k rows sit in shared memory with the parts kR + 4 floats apart, so the 16-byte loads
// of a warp's parts fall on different banks.
template <int kR, int kParts>
__global__ void __launch_bounds__(128)
gated_delta_tiled_kernel(const float* __restrict__ qkv, float* __restrict__ scratch, float* __restrict__ state, float* __restrict__ out,
                         const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_start,
                         int T, int H, int G, int dk, int dv) {
    pdl_wait();
    pdl_trigger();
    constexpr int kPS = kR + 4;                       // floats between parts
    constexpr int kRow = kParts * kPS;                // floats between tokens
    constexpr int kCW = 32 / kParts;                  // value columns per warp
    constexpr int kCB = 4 * kCW;                      // value columns per block
    constexpr int kNQ = kTile * kParts * kR / 128;    // q (and k) elements a thread stages per tile
    constexpr int kNV = kTile * kCB / 128;            // v elements a thread stages per tile
    constexpr int kNS = 20;                           // row pitch of N
    extern __shared__ float sm[];
    float* qs = sm;                                   // [kTile][kParts][kPS]
    float* ks = qs + kTile * kRow;                    // [kTile][kParts][kPS]
    float* vs = ks + kTile * kRow;                    // [kTile][kCB]
    float* Mt = vs + kTile * kCB;                     // [s][i]: M transposed
    float* Ns = Mt + kTile * kTile;                   // [i][kNS]
    float* Ps = Ns + kTile * kNS;                     // [kTile]
    float* Es = Ps + kTile;                           // [kTile]
    float* bs = Es + kTile;                           // [kTile]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, part = lane / kCW;
    const int b = blockIdx.z, h = blockIdx.y;
    const int ci = warp * kCW + lane % kCW;
    const int col = blockIdx.x * kCB + ci;
    const bool live = col < dv;
    const int g = h / (H / G);
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (n <= 0) return;
    const int C = 2 * G * dk + H * dv;
    const int row0 = part * kR;
    const DeltaScratch sc = delta_scratch(scratch, T, H, G, dk);
    float* Sg = state + (((int64_t)seq_slots[b] * H + h) * dv + (live ? col : 0)) * dk + row0;
    const bool fresh = seq_start[b] == 0;
    const bool vec = (dk & 3) == 0 && row0 + kR <= dk;
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

    float rq[kNQ], rk[kNQ], rv[kNV], rM[2], rN[2], rP = 1.f, rE = 0.f, rb = 0.f;
    auto load_tile = [&](int first, int cnt) {        // global -> registers
#pragma unroll
        for (int j = 0; j < kNQ; ++j) {
            const int e = tid + 128 * j, tt = e / (kParts * kR), i = e % (kParts * kR);
            const bool in = tt < cnt && i < dk;
            const int64_t at = ((int64_t)(first + tt) * G + g) * dk + i;
            rq[j] = in ? sc.qn[at] : 0.f;
            rk[j] = in ? sc.kn[at] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kNV; ++j) {
            const int e = tid + 128 * j, tt = e / kCB, c = blockIdx.x * kCB + e % kCB;
            rv[j] = (tt < cnt && c < dv) ? qkv[(int64_t)(first + tt) * C + 2 * G * dk + h * dv + c] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int e = tid + 128 * j, tt = e >> 4;
            const int64_t at = ((int64_t)(first + tt) * H + h) * kTile + (e & 15);
            rM[j] = tt < cnt ? sc.M[at] : 0.f;
            rN[j] = tt < cnt ? sc.N[at] : 0.f;
        }
        if (tid < kTile) {
            const bool in = tid < cnt;
            const int64_t at = (int64_t)(first + tid) * H + h;
            rP = in ? sc.P[at] : 1.f;
            rE = in ? sc.E[at] : 0.f;
            rb = in ? sc.beta[at] : 0.f;
        }
    };
    auto store_tile = [&]() {                          // registers -> shared memory
#pragma unroll
        for (int j = 0; j < kNQ; ++j) {
            const int e = tid + 128 * j, tt = e / (kParts * kR), i = e % (kParts * kR);
            const int at = tt * kRow + (i / kR) * kPS + (i % kR);
            qs[at] = rq[j]; ks[at] = rk[j];
        }
#pragma unroll
        for (int j = 0; j < kNV; ++j) vs[tid + 128 * j] = rv[j];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int e = tid + 128 * j, i = e >> 4, c = e & 15;
            Mt[c * kTile + i] = rM[j];
            Ns[i * kNS + c] = rN[j];
        }
        if (tid < kTile) { Ps[tid] = rP; Es[tid] = rE; bs[tid] = rb; }
    };

    const float* kp = ks + part * kPS;
    const float* qp = qs + part * kPS;
    const int tiles = (n + kTile - 1) / kTile;
    load_tile(t0, min(kTile, n));
    for (int tile = 0; tile < tiles; ++tile) {
        const int first = t0 + tile * kTile, cnt = min(kTile, n - tile * kTile);
        __syncthreads();                               // every warp has finished the previous tile
        store_tile();
        __syncthreads();
        // S0^T k_i and S0^T q_i for the 16 tokens: this lane's rows, then the eight parts joined
        float a[kTile], bq[kTile];
#pragma unroll
        for (int i = 0; i < kTile; ++i) { a[i] = 0.f; bq[i] = 0.f; }
#pragma unroll
        for (int r = 0; r < kR; r += 4) {
#pragma unroll
            for (int i = 0; i < kTile; ++i) {
                const float4 c = *reinterpret_cast<const float4*>(kp + i * kRow + r);
                const float4 d = *reinterpret_cast<const float4*>(qp + i * kRow + r);
                a[i] = fmaf(S[r], c.x, a[i]); a[i] = fmaf(S[r + 1], c.y, a[i]); a[i] = fmaf(S[r + 2], c.z, a[i]); a[i] = fmaf(S[r + 3], c.w, a[i]);
                bq[i] = fmaf(S[r], d.x, bq[i]); bq[i] = fmaf(S[r + 1], d.y, bq[i]); bq[i] = fmaf(S[r + 2], d.z, bq[i]); bq[i] = fmaf(S[r + 3], d.w, bq[i]);
                // at most eight 16-byte loads in flight: without the barrier the compiler hoists the tile's loads and spills
                if ((i & 3) == 3) asm volatile("" ::: "memory");
            }
        }
#pragma unroll
        for (int m = kCW; m <= 16; m <<= 1) {
#pragma unroll
            for (int i = 0; i < kTile; ++i) {
                const float x = __shfl_xor_sync(0xffffffffu, a[i], m), y = __shfl_xor_sync(0xffffffffu, bq[i], m);
                a[i] += x; bq[i] += y;
            }
        }
        if (tile + 1 < tiles) load_tile(first + kTile, min(kTile, n - (tile + 1) * kTile));     // in flight under the rest of this tile
        // the triangular system, column by column of M: every lane of a value column solves it (the same sums in the same order)
        float u[kTile];
#pragma unroll
        for (int i = 0; i < kTile; i += 4) {
            const float4 P4 = *reinterpret_cast<const float4*>(Ps + i);
            a[i] = fmaf(-P4.x, a[i], vs[i * kCB + ci]); a[i + 1] = fmaf(-P4.y, a[i + 1], vs[(i + 1) * kCB + ci]);
            a[i + 2] = fmaf(-P4.z, a[i + 2], vs[(i + 2) * kCB + ci]); a[i + 3] = fmaf(-P4.w, a[i + 3], vs[(i + 3) * kCB + ci]);
        }
#pragma unroll
        for (int s = 0; s < kTile; ++s) {
            u[s] = bs[s] * a[s];
#pragma unroll
            for (int i4 = (s + 1) >> 2; i4 < 4; ++i4) {
                const float4 m = *reinterpret_cast<const float4*>(Mt + s * kTile + 4 * i4);
                if (4 * i4 > s) a[4 * i4] = fmaf(-m.x, u[s], a[4 * i4]);
                if (4 * i4 + 1 > s) a[4 * i4 + 1] = fmaf(-m.y, u[s], a[4 * i4 + 1]);
                if (4 * i4 + 2 > s) a[4 * i4 + 2] = fmaf(-m.z, u[s], a[4 * i4 + 2]);
                a[4 * i4 + 3] = fmaf(-m.w, u[s], a[4 * i4 + 3]);
            }
        }
        // outputs: part p takes tokens p, p + kParts, ...
#pragma unroll
        for (int half = 0; half < kTile / kParts; ++half) {
            const int i = part + kParts * half;
            float b0 = 0.f;
#pragma unroll
            for (int j = 0; j < kParts; ++j) b0 = (j == part) ? bq[j + kParts * half] : b0;
            const float4* nr = reinterpret_cast<const float4*>(Ns + i * kNS);
            float o[4] = {Ps[i] * b0, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s4 = 0; s4 < 4; ++s4) {
                const float4 w = nr[s4];
                o[0] = fmaf(w.x, u[4 * s4], o[0]); o[1] = fmaf(w.y, u[4 * s4 + 1], o[1]); o[2] = fmaf(w.z, u[4 * s4 + 2], o[2]); o[3] = fmaf(w.w, u[4 * s4 + 3], o[3]);
            }
            if (live && i < cnt) out[(int64_t)(first + i) * H * dv + h * dv + col] = (o[0] + o[1]) + (o[2] + o[3]);
        }
        // the state at the tile's end
        const float pend = Ps[cnt - 1];
#pragma unroll
        for (int r = 0; r < kR; ++r) S[r] *= pend;
#pragma unroll
        for (int s = 0; s < kTile; ++s) {
            const float w = Es[s] * u[s];
#pragma unroll
            for (int r = 0; r < kR; r += 4) {
                const float4 c = *reinterpret_cast<const float4*>(kp + s * kRow + r);
                S[r] = fmaf(c.x, w, S[r]); S[r + 1] = fmaf(c.y, w, S[r + 1]); S[r + 2] = fmaf(c.z, w, S[r + 2]); S[r + 3] = fmaf(c.w, w, S[r + 3]);
            }
            if (s & 1) asm volatile("" ::: "memory");
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
    B200_REQUIRE(dk <= 512, kErrUnsupported, "gated_delta_rule: key size %d > 512", dk);
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
    else if (dk <= 256) GDR(32);
    else GDR(64);                                      // spills its staging registers: a path for correctness, not speed
#undef GDR
    count_launch();
    check_launch("gated_delta_rule");
}

void gated_delta_rule_step(const float* qkv, const float* proj, int64_t ld_proj, int32_t off_b, int32_t off_a, const float* A_log, const float* dt_bias,
                           float* state, float* out, const int32_t* seq_slots, const int32_t* seq_start, int32_t num_seqs, int32_t num_heads,
                           int32_t num_kv_heads, int32_t dk, int32_t dv, int64_t stream) {
    if (num_seqs == 0) return;
    B200_REQUIRE(qkv && proj && A_log && dt_bias && state && out && seq_slots && seq_start, kErrBadArg, "gated_delta_rule_step: null pointer");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0 && num_seqs <= 65535, kErrBadArg,
                 "gated_delta_rule_step: bad sizes");
    B200_REQUIRE(dk <= 512, kErrUnsupported, "gated_delta_rule_step: key size %d > 512", dk);
    cudaStream_t st = as_stream(stream);
    const dim3 grid(ceil_div(dv, 16), num_heads, num_seqs);
#define GDS(R) launch_pdl(gated_delta_step_kernel<R>, grid, dim3(128), 0, st, qkv, proj, ld_proj, off_b, off_a, A_log, dt_bias, state, out, seq_slots, seq_start, \
                          num_heads, num_kv_heads, dk, dv)
    if (dk <= 32) GDS(4);
    else if (dk <= 64) GDS(8);
    else if (dk <= 128) GDS(16);
    else if (dk <= 256) GDS(32);
    else GDS(64);
#undef GDS
    count_launch();
    check_launch("gated_delta_rule_step");
}

void gated_delta_rule_tiled(const float* qkv, const float* proj, int64_t ld_proj, int32_t off_b, int32_t off_a, const float* A_log, const float* dt_bias,
                            float* state, float* out, float* scratch, const int32_t* cu_seqlens, const int32_t* seq_slots, const int32_t* seq_start,
                            int32_t num_tokens, int32_t num_seqs, int32_t max_rows, int32_t num_heads, int32_t num_kv_heads, int32_t dk, int32_t dv,
                            int64_t stream) {
    if (num_seqs == 0 || num_tokens == 0) return;
    B200_REQUIRE(qkv && proj && A_log && dt_bias && state && out && scratch && cu_seqlens && seq_slots && seq_start, kErrBadArg,
                 "gated_delta_rule_tiled: null pointer");
    B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0 && max_rows > 0, kErrBadArg,
                 "gated_delta_rule_tiled: bad sizes");
    B200_REQUIRE(dk <= 128, kErrUnsupported, "gated_delta_rule_tiled: key size %d > 128", dk);
    cudaStream_t st = as_stream(stream);
    {
        const int ld = ((dk + 3) & ~3) + 4;
        const int smem = (2 * kTile * ld + 2 * kTile * kTile + kTile) * (int)sizeof(float);
        ensure_dynamic_smem(reinterpret_cast<const void*>(gated_delta_prepare_kernel), smem);
        launch_pdl(gated_delta_prepare_kernel, dim3(ceil_div(max_rows, kTile), num_kv_heads, num_seqs), dim3(128), smem, st, qkv, proj, ld_proj, off_b, off_a,
                   A_log, dt_bias, scratch, cu_seqlens, num_tokens, num_heads, num_kv_heads, dk, dv);
        count_launch();
        if (!check_launch("gated_delta_prepare")) return;
    }
#define GDT(R, P) do { \
        constexpr int kCB = 4 * (32 / P); \
        const dim3 grid(ceil_div(dv, kCB), num_heads, num_seqs); \
        const int smem = (2 * kTile * P * (R + 4) + kTile * kCB + kTile * kTile + kTile * 20 + 3 * kTile) * (int)sizeof(float); \
        ensure_dynamic_smem(reinterpret_cast<const void*>(gated_delta_tiled_kernel<R, P>), smem); \
        launch_pdl(gated_delta_tiled_kernel<R, P>, grid, dim3(128), smem, st, qkv, scratch, state, out, cu_seqlens, seq_slots, seq_start, num_tokens, num_heads, \
                   num_kv_heads, dk, dv); } while (0)
    // eight parts per column: sixteen (twice the blocks, half the work per lane) measured no faster at 16 heads of 128 and slower at 32
    if (dk <= 32) GDT(4, 8);
    else if (dk <= 64) GDT(8, 8);
    else GDT(16, 8);
#undef GDT
    count_launch();
    check_launch("gated_delta_rule_tiled");
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
