// Recurrent mixers whose inputs pass a short causal convolution first, and their recurrences:
//
//   causal_conv_kernel        y[t, c] = act(sum_j w[c, j] x[t - (J - 1) + j, c] + b[c]) over the tokens of a request, the
//                             J - 1 inputs before a step's first token read from the request's state slot (zero at
//                             admission, which is "zeros before the start") and the step's last J - 1 inputs left there
//   gate_blocks_kernel        the gates of a real-gated linear recurrent unit from block-diagonal products of the
//                             convolved branch u:  r = sigmoid(Wa_b u_b + ba), i = sigmoid(Wi_b u_b + bi),
//                             log a = -c r softplus(lam), and what the recurrence adds, sqrt(1 - a^2) i u
//   linear_recurrence_kernel  S_t = a_t S_(t-1) + b_t per channel from the state slot, result S_t * gelu_tanh(y_t + by)
//   gated_delta_scan_kernel   the gated delta rule per head on a matrix S [dk, dv]:
//                                 S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//                             with q and k made unit vectors here, g_t = exp(-exp(A) softplus(z_t + dt_bias)) per key
//                             channel and beta_t = sigmoid(.)
//
// States, decays and their logarithms, softplus and exponentials, gates, unit norms and every sum are float whatever the
// type T of the projections is.  The reference has no recurrent mixer (src/layers/attention.cpp is its only mixer).
#include "common.cuh"

#define CONV_MAX_TAPS 8
#define CONV_SEG 32            // tokens a thread walks; at least CONV_MAX_TAPS - 1, so that only a request's first segment reads the state

__device__ __forceinline__ float gr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float gr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gr_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gr_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

struct ConvArgs {
    const void* x;              // [n, C] rows of T, row stride ldx
    long long ldx;
    const float* pre_bias;      // [C] or null: added to every input (never to the zeros before the start)
    const float* w;             // [C, J]
    const float* bias;          // [C] or null: added to the sum
    float* state;               // slot s, row j (0 .. J - 2), channel c at state[s * slot_stride + j * C + c]
    long long slot_stride;
    float* out;                 // [n, C] float, row stride ldo
    long long ldo;
    const int* q_start;
    const int* state_slots;
    int C, J, act;
};

// Grid (segments of the longest portion, requests, tiles of 128 channels); a thread per channel.
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_kernel(ConvArgs a) {
    const int c = blockIdx.z * 128 + threadIdx.x;
    float w[CONV_MAX_TAPS];
    const int J = a.J;
    const bool live = c < a.C;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = (live && j < J) ? a.w[(size_t)c * J + j] : 0.0f;
    const float pb = (live && a.pre_bias) ? a.pre_bias[c] : 0.0f, cb = (live && a.bias) ? a.bias[c] : 0.0f;
    pdl_start();
    const int r = blockIdx.y;
    const int row0 = a.q_start[r], len = a.q_start[r + 1] - row0;
    const int seg0 = blockIdx.x * CONV_SEG;
    if (seg0 >= len || !live) return;
    const T* x = (const T*)a.x + (size_t)row0 * a.ldx + c;
    float* st = a.state + (size_t)a.state_slots[r] * a.slot_stride + c;
    // win[j]: the input J - 1 - j places before the current token, oldest first
    float win[CONV_MAX_TAPS - 1], old[CONV_MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        win[j] = old[j] = 0.0f;
        if (j < J - 1) {
            const int li = seg0 - (J - 1) + j;
            win[j] = li >= 0 ? to_f32<T>(x[(size_t)li * a.ldx]) + pb : st[(size_t)(J - 1 + li) * a.C];
            old[j] = win[j];
        }
    }
    const int end = min(seg0 + CONV_SEG, len);
    float* out = a.out + (size_t)row0 * a.ldo + c;
    for (int t = seg0; t < end; ++t) {
        const float cur = to_f32<T>(x[(size_t)t * a.ldx]) + pb;
        float acc = cb;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < J - 1) acc = fmaf(w[j], win[j], acc);
        acc = fmaf(w[J - 1], cur, acc);
        out[(size_t)t * a.ldo] = a.act ? gr_silu(acc) : acc;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 2; ++j) win[j] = win[j + 1];
        if (J >= 2) {
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
                if (j == J - 2) win[j] = cur;
        }
    }
    if (seg0 == 0) {
        // this thread alone reads and writes the channel's state: what it read is in old[]
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
            if (j >= J - 1) break;
            const int li = len - (J - 1) + j;
            st[(size_t)j * a.C] = li >= 0 ? to_f32<T>(x[(size_t)li * a.ldx]) + pb : old[J - 1 + li];
        }
    }
}

VCB_EXPORT int vcb_causal_conv(const void* x, long long ldx, const float* pre_bias, const float* w, const float* bias,
                               float* state, long long slot_stride, float* out, long long ldo, const int* q_start,
                               const int* state_slots, int n_reqs, int max_q_len, int C, int J, int act, int dtype,
                               void* stream) {
    if (n_reqs <= 0 || max_q_len <= 0) return 0;
    if (!x || !w || (!state && J > 1) || !out || C <= 0 || J <= 0 || J > CONV_MAX_TAPS || n_reqs > 65535) return VCB_ERR_BAD_ARG;
    ConvArgs a{x, ldx, pre_bias, w, bias, state, slot_stride, out, ldo, q_start, state_slots, C, J, act};
    dim3 grid((max_q_len + CONV_SEG - 1) / CONV_SEG, n_reqs, (C + 127) / 128);
    if (grid.z > 65535) return VCB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) vcb_launch(causal_conv_kernel<float>, grid, 128, 0, s, a);
    else if (dtype == VCB_BF16) vcb_launch(causal_conv_kernel<__nv_bfloat16>, grid, 128, 0, s, a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------------------------- gates of the recurrent unit
// u: float [n, W]; W = B blocks of bs channels; wa, wi: [B, bs, bs] of T ([out, in]); ba, bi: float [W]; lam: float [W].
// decay[t, c] = exp(-c_gate * r * softplus(lam[c])),  drive[t, c] = sqrt(1 - decay^2) * i * u[t, c].
// A CTA owns 64 tokens x 64 channels of one block; 16-deep slices of the block's inputs through shared memory; float FMA.
template <typename T>
__global__ void __launch_bounds__(256)
gate_blocks_kernel(const float* __restrict__ u, long long ldu, const T* __restrict__ wa, const T* __restrict__ wi,
                   const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ lam,
                   float* __restrict__ decay, float* __restrict__ drive, long long ldo, int n, int bs, int tiles_per_block,
                   float c_gate) {
    __shared__ float Us[16][64 + 1];
    __shared__ float As[16][64 + 1];
    __shared__ float Is[16][64 + 1];
    pdl_start();
    const int b = blockIdx.y / tiles_per_block, n0 = (blockIdx.y % tiles_per_block) * 64;
    const int t0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* Wa = wa + (size_t)b * bs * bs;
    const T* Wi = wi + (size_t)b * bs * bs;
    const float* ub = u + (size_t)b * bs;
    float accr[4][4], acci[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) accr[i][j] = acci[i][j] = 0.0f;
    for (int k0 = 0; k0 < bs; k0 += 16) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = threadIdx.x + q * 256;
            const int r = idx >> 4, kk = idx & 15, k = k0 + kk;
            Us[kk][r] = (t0 + r < n && k < bs) ? ub[(size_t)(t0 + r) * ldu + k] : 0.0f;
            const bool ok = n0 + r < bs && k < bs;
            As[kk][r] = ok ? to_f32<T>(Wa[(size_t)(n0 + r) * bs + k]) : 0.0f;
            Is[kk][r] = ok ? to_f32<T>(Wi[(size_t)(n0 + r) * bs + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float uv[4], av[4], iv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) uv[i] = Us[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { av[j] = As[kk][tx * 4 + j]; iv[j] = Is[kk][tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    accr[i][j] = fmaf(uv[i], av[j], accr[i][j]);
                    acci[i][j] = fmaf(uv[i], iv[j], acci[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= n) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cb = n0 + tx * 4 + j;
            if (cb >= bs) continue;
            const int c = b * bs + cb;
            const float r = gr_sigmoid(accr[i][j] + ba[c]), g = gr_sigmoid(acci[i][j] + bi[c]);
            const float la = -c_gate * r * gr_softplus(lam[c]);
            decay[(size_t)t * ldo + c] = expf(la);
            drive[(size_t)t * ldo + c] = sqrtf(-expm1f(2.0f * la)) * g * u[(size_t)t * ldu + c];
        }
    }
}

// The same for a few tokens (single tokens of a batch) and blocks of up to GATE_ROWS_BS channels: the tiles above would
// fill a fraction of the SMs and walk the block's inputs in dependent slices.  A warp per output channel: its lanes split
// the block's inputs and keep their weights of both matrices in registers, every token costs two warp sums, and lane t % 32
// finishes token t (gates, decay, drive).
constexpr int GATE_ROWS_MAX = 16, GATE_ROWS_BS = 256;      // measured: at 64 tokens the tiles above are faster (29 against 42 us)
template <typename T>
__global__ void __launch_bounds__(256)
gate_rows_kernel(const float* __restrict__ u, long long ldu, const T* __restrict__ wa, const T* __restrict__ wi,
                 const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ lam,
                 float* __restrict__ decay, float* __restrict__ drive, long long ldo, int n, int bs, float c_gate) {
    constexpr int M = GATE_ROWS_BS / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y, cb = blockIdx.x * 8 + warp;
    const bool live = cb < bs;
    const int c = b * bs + (live ? cb : 0);
    float wa_r[M], wi_r[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const int k = lane + 32 * m;
        const bool ok = live && k < bs;
        wa_r[m] = ok ? to_f32<T>(wa[((size_t)b * bs + cb) * bs + k]) : 0.0f;
        wi_r[m] = ok ? to_f32<T>(wi[((size_t)b * bs + cb) * bs + k]) : 0.0f;
    }
    const float bav = ba[c], biv = bi[c], sp = gr_softplus(lam[c]);
    pdl_start();
    if (!live) return;
    const float* ub = u + (size_t)b * bs;
    for (int t0 = 0; t0 < n; t0 += 32) {
        float mine_a = 0.0f, mine_i = 0.0f;
        const int t1 = min(t0 + 32, n);
        for (int t = t0; t < t1; t += 4) {          // four tokens' loads and sums in flight
            float sa[4], si[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                sa[q] = si[q] = 0.0f;
                const int tq = min(t + q, t1 - 1);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const int k = lane + 32 * m;
                    if (k < bs) {
                        const float uv = ub[(size_t)tq * ldu + k];
                        sa[q] = fmaf(uv, wa_r[m], sa[q]);
                        si[q] = fmaf(uv, wi_r[m], si[q]);
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    sa[q] += __shfl_xor_sync(0xffffffffu, sa[q], o);
                    si[q] += __shfl_xor_sync(0xffffffffu, si[q], o);
                }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (lane == t + q - t0) { mine_a = sa[q]; mine_i = si[q]; }
        }
        const int t = t0 + lane;
        if (t < t1) {
            const float r = gr_sigmoid(mine_a + bav), g = gr_sigmoid(mine_i + biv);
            const float la = -c_gate * r * sp;
            decay[(size_t)t * ldo + c] = expf(la);
            drive[(size_t)t * ldo + c] = sqrtf(-expm1f(2.0f * la)) * g * u[(size_t)t * ldu + c];
        }
    }
}

VCB_EXPORT int vcb_gate_blocks(const float* u, long long ldu, const void* wa, const void* wi, const float* ba, const float* bi,
                               const float* lam, float* decay, float* drive, long long ldo, int n, int W, int B, float c_gate,
                               int dtype, void* stream) {
    if (n <= 0) return 0;
    if (!u || !wa || !wi || !ba || !bi || !lam || !decay || !drive || W <= 0 || B <= 0 || W % B) return VCB_ERR_BAD_ARG;
    const int bs = W / B, tiles = (bs + 63) / 64;
    if ((long long)B * tiles > 65535) return VCB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (n <= GATE_ROWS_MAX && bs <= GATE_ROWS_BS && B <= 65535) {
        dim3 rows((bs + 7) / 8, B);
        if (dtype == VCB_F32)
            vcb_launch(gate_rows_kernel<float>, rows, 256, 0, s, u, ldu, (const float*)wa, (const float*)wi, ba, bi, lam, decay, drive, ldo, n, bs, c_gate);
        else if (dtype == VCB_BF16)
            vcb_launch(gate_rows_kernel<__nv_bfloat16>, rows, 256, 0, s, u, ldu, (const __nv_bfloat16*)wa, (const __nv_bfloat16*)wi, ba, bi,
                       lam, decay, drive, ldo, n, bs, c_gate);
        else return VCB_ERR_BAD_ARG;
        return vcb_last_error();
    }
    dim3 grid((n + 63) / 64, B * tiles);
    if (dtype == VCB_F32)
        vcb_launch(gate_blocks_kernel<float>, grid, 256, 0, s, u, ldu, (const float*)wa, (const float*)wi, ba, bi, lam, decay, drive, ldo, n, bs, tiles, c_gate);
    else if (dtype == VCB_BF16)
        vcb_launch(gate_blocks_kernel<__nv_bfloat16>, grid, 256, 0, s, u, ldu, (const __nv_bfloat16*)wa, (const __nv_bfloat16*)wi, ba, bi, lam,
                   decay, drive, ldo, n, bs, tiles, c_gate);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------------------------- S_t = a_t S_(t-1) + b_t
// decay, drive: float [n, W]; y: [n, W] rows of T (row stride ldy) with bias by (float [W] or null); state: slot s,
// channel c at state[s * slot_stride + c]; out [n, W] of T = S_t * gelu_tanh(y_t + by).  A thread per channel walks
// its request's tokens, four tokens' loads in flight.
template <typename T>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const float* __restrict__ decay, const float* __restrict__ drive, long long ldd, const T* __restrict__ y,
                         long long ldy, const float* __restrict__ by, float* __restrict__ state, long long slot_stride,
                         T* __restrict__ out, long long ldo, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                         int W) {
    const int c = blockIdx.y * 128 + threadIdx.x;
    const float yb = (c < W && by) ? by[c] : 0.0f;
    pdl_start();
    if (c >= W) return;
    const int r = blockIdx.x;
    const int row0 = q_start[r], row1 = q_start[r + 1];
    float* st = state + (size_t)state_slots[r] * slot_stride + c;
    float S = *st;
    int t = row0;
    for (; t + 4 <= row1; t += 4) {
        float a[4], b[4], g[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            a[k] = decay[(size_t)(t + k) * ldd + c];
            b[k] = drive[(size_t)(t + k) * ldd + c];
            g[k] = to_f32<T>(y[(size_t)(t + k) * ldy + c]);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            S = fmaf(a[k], S, b[k]);
            out[(size_t)(t + k) * ldo + c] = from_f32<T>(S * gr_gelu_tanh(g[k] + yb));
        }
    }
    for (; t < row1; ++t) {
        S = fmaf(decay[(size_t)t * ldd + c], S, drive[(size_t)t * ldd + c]);
        out[(size_t)t * ldo + c] = from_f32<T>(S * gr_gelu_tanh(to_f32<T>(y[(size_t)t * ldy + c]) + yb));
    }
    *st = S;
}

// The same for portions of many tokens: a CTA owns 32 channels (the lanes) of a request, its SCAN_WARPS warps a
// stretch of the portion each.  Every warp first walks its stretch from an empty state and keeps the stretch's total decay
// A and its own contribution B (S_end = A S_start + B); one warp then carries the request's state through the stretches
// in order; then every warp walks its stretch again from the state it starts with and writes the outputs.  Within a
// stretch the recurrence runs token by token as above; only the states at the stretches' starts are summed in another
// order.
constexpr int SCAN_WARPS = 32, SCAN_AHEAD = 8;
template <typename T>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
linear_recurrence_stretches_kernel(const float* __restrict__ decay, const float* __restrict__ drive, long long ldd,
                                   const T* __restrict__ y, long long ldy, const float* __restrict__ by, float* __restrict__ state,
                                   long long slot_stride, T* __restrict__ out, long long ldo, const int* __restrict__ q_start,
                                   const int* __restrict__ state_slots, int W) {
    __shared__ float As[SCAN_WARPS][32], Bs[SCAN_WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.y * 32 + lane;
    const bool ok = c < W;
    const float yb = (ok && by) ? by[c] : 0.0f;
    pdl_start();
    const int r = blockIdx.x;
    const int row0 = q_start[r], len = q_start[r + 1] - row0;
    const int per = (len + SCAN_WARPS - 1) / SCAN_WARPS;
    const int t0 = row0 + min(warp * per, len), t1 = row0 + min((warp + 1) * per, len);
    float A = 1.0f, B = 0.0f;
    if (ok) {
        int t = t0;
        for (; t + SCAN_AHEAD <= t1; t += SCAN_AHEAD) {
            float a[SCAN_AHEAD], b[SCAN_AHEAD];
#pragma unroll
            for (int k = 0; k < SCAN_AHEAD; ++k) { a[k] = decay[(size_t)(t + k) * ldd + c]; b[k] = drive[(size_t)(t + k) * ldd + c]; }
#pragma unroll
            for (int k = 0; k < SCAN_AHEAD; ++k) { B = fmaf(a[k], B, b[k]); A *= a[k]; }
        }
        for (; t < t1; ++t) { const float a = decay[(size_t)t * ldd + c]; B = fmaf(a, B, drive[(size_t)t * ldd + c]); A *= a; }
    }
    As[warp][lane] = A;
    Bs[warp][lane] = B;
    __syncthreads();
    if (warp == 0 && ok) {
        float* st = state + (size_t)state_slots[r] * slot_stride + c;
        float S = *st;
        for (int w = 0; w < SCAN_WARPS; ++w) {
            const float a = As[w][lane], b = Bs[w][lane];
            As[w][lane] = S;                              // the state the stretch starts with
            S = fmaf(a, S, b);
        }
        *st = S;
    }
    __syncthreads();
    if (!ok) return;
    float S = As[warp][lane];
    int t = t0;
    for (; t + SCAN_AHEAD <= t1; t += SCAN_AHEAD) {
        float a[SCAN_AHEAD], b[SCAN_AHEAD], g[SCAN_AHEAD];
#pragma unroll
        for (int k = 0; k < SCAN_AHEAD; ++k) {
            a[k] = decay[(size_t)(t + k) * ldd + c];
            b[k] = drive[(size_t)(t + k) * ldd + c];
            g[k] = to_f32<T>(y[(size_t)(t + k) * ldy + c]);
        }
#pragma unroll
        for (int k = 0; k < SCAN_AHEAD; ++k) {
            S = fmaf(a[k], S, b[k]);
            out[(size_t)(t + k) * ldo + c] = from_f32<T>(S * gr_gelu_tanh(g[k] + yb));
        }
    }
    for (; t < t1; ++t) {
        S = fmaf(decay[(size_t)t * ldd + c], S, drive[(size_t)t * ldd + c]);
        out[(size_t)t * ldo + c] = from_f32<T>(S * gr_gelu_tanh(to_f32<T>(y[(size_t)t * ldy + c]) + yb));
    }
}

constexpr int SCAN_STRETCHES_FROM = 64;      // portions of at least this many tokens in a step: the kernel above

VCB_EXPORT int vcb_linear_recurrence(const float* decay, const float* drive, long long ldd, const void* y, long long ldy,
                                     const float* by, float* state, long long slot_stride, void* out, long long ldo,
                                     const int* q_start, const int* state_slots, int n_reqs, int max_q_len, int W, int dtype,
                                     void* stream) {
    if (n_reqs <= 0) return 0;
    if (!decay || !drive || !y || !state || !out || W <= 0 || (W + 31) / 32 > 65535) return VCB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (max_q_len >= SCAN_STRETCHES_FROM) {
        dim3 grid(n_reqs, (W + 31) / 32);
        if (dtype == VCB_F32)
            vcb_launch(linear_recurrence_stretches_kernel<float>, grid, SCAN_WARPS * 32, 0, s, decay, drive, ldd, (const float*)y, ldy, by,
                       state, slot_stride, (float*)out, ldo, q_start, state_slots, W);
        else if (dtype == VCB_BF16)
            vcb_launch(linear_recurrence_stretches_kernel<__nv_bfloat16>, grid, SCAN_WARPS * 32, 0, s, decay, drive, ldd,
                       (const __nv_bfloat16*)y, ldy, by, state, slot_stride, (__nv_bfloat16*)out, ldo, q_start, state_slots, W);
        else return VCB_ERR_BAD_ARG;
        return vcb_last_error();
    }
    dim3 grid(n_reqs, (W + 127) / 128);
    if (dtype == VCB_F32)
        vcb_launch(linear_recurrence_kernel<float>, grid, 128, 0, s, decay, drive, ldd, (const float*)y, ldy, by, state, slot_stride,
                   (float*)out, ldo, q_start, state_slots, W);
    else if (dtype == VCB_BF16)
        vcb_launch(linear_recurrence_kernel<__nv_bfloat16>, grid, 128, 0, s, decay, drive, ldd, (const __nv_bfloat16*)y, ldy, by, state,
                   slot_stride, (__nv_bfloat16*)out, ldo, q_start, state_slots, W);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------------------------- the gated delta rule
struct DeltaArgs {
    const float* q;             // [n, G * dk] float (convolved, activated), row stride ldq
    const float* k;
    const float* v;             // [n, H * dv], row stride ldv
    long long ldq, ldk, ldv;
    const void* beta_pre;       // [n, H] rows of T, row stride ldb: beta = sigmoid(.)
    long long ldb;
    const void* decay_pre;      // [n, H * dk] rows of T, row stride lda
    long long lda;
    const float* a_log;         // [H]
    const float* dt_bias;       // [H * dk]
    float* state;               // [slots][H][dk][dv]
    float* out;                 // [n, H * dv] float, row stride ldo
    long long ldo;
    const int* q_start;
    const int* state_slots;
    int H, G, dk, dv;
    float q_scale, unit_eps;
    int chunk;                  // tokens staged in shared memory at a time
};

// Grid (request, head, tile of DVT value channels).  A thread keeps DKP rows of one column of S in registers; the P
// threads that share a column are neighbouring lanes of a warp and add their partial sums up by shuffles, so a token
// costs no block-wide barrier.  Key channels beyond dk are padded with q = k = 0, g = 1.
template <typename T, int DKP>
__global__ void gated_delta_scan_kernel(DeltaArgs a, int P, int DVT) {
    extern __shared__ __align__(16) float sm[];
    pdl_start();
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DVT;
    const int kvh = h / (a.H / a.G);
    const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const int part = tid % P, cl = tid / P;
    const int col = col0 + cl;
    const bool col_ok = cl < DVT && col < a.dv;
    const int TC = a.chunk;
    const int pstride = DKP + 4;                  // a part's slice of a token's q, k, g; padded against bank conflicts
    const int tstride = P * pstride;
    float* qs = sm;
    float* ks = qs + TC * tstride;
    float* gs = ks + TC * tstride;
    float* vs = gs + TC * tstride;                // [TC][DVT]
    float* os = vs + TC * DVT;                    // [TC][DVT]
    float* bs = os + TC * DVT;                    // [TC]
    const int row0 = a.q_start[r], row1 = a.q_start[r + 1];
    float* st = a.state + (((size_t)a.state_slots[r] * a.H + h) * a.dk) * a.dv;
    float S[DKP];
#pragma unroll
    for (int i = 0; i < DKP; ++i) {
        const int kr = part * DKP + i;
        S[i] = (col_ok && kr < a.dk) ? st[(size_t)kr * a.dv + col] : 0.0f;
    }
    const float rate = expf(a.a_log[h]);
    const T* bp = (const T*)a.beta_pre;
    const T* dp = (const T*)a.decay_pre;
    for (int c0 = row0; c0 < row1; c0 += TC) {
        const int tc = min(TC, row1 - c0);
        __syncthreads();                          // the chunk before has been read
        // a warp per token: unit q and k, the decays, beta
        for (int tt = warp; tt < tc; tt += nwarps) {
            const size_t row = (size_t)(c0 + tt);
            const float* qr = a.q + row * a.ldq + kvh * a.dk;
            const float* kr = a.k + row * a.ldk + kvh * a.dk;
            float sq = 0.0f, sk = 0.0f;
            for (int i = lane; i < a.dk; i += 32) { const float x = qr[i], y = kr[i]; sq = fmaf(x, x, sq); sk = fmaf(y, y, sk); }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            const float rq = a.q_scale / sqrtf(sq + a.unit_eps), rk = 1.0f / sqrtf(sk + a.unit_eps);
            for (int i = lane; i < P * DKP; i += 32) {
                const int p = i / DKP, j = i - p * DKP;
                float qv = 0.0f, kv = 0.0f, gv = 1.0f;
                if (i < a.dk) {
                    qv = qr[i] * rq;
                    kv = kr[i] * rk;
                    const float z = to_f32<T>(dp[row * a.lda + h * a.dk + i]) + a.dt_bias[h * a.dk + i];
                    gv = expf(-rate * gr_softplus(z));
                }
                const int at = tt * tstride + p * pstride + j;
                qs[at] = qv;
                ks[at] = kv;
                gs[at] = gv;
            }
            if (lane == 0) bs[tt] = gr_sigmoid(to_f32<T>(bp[row * a.ldb + h]));
        }
        for (int idx = tid; idx < tc * DVT; idx += nthreads) {
            const int tt = idx / DVT, j = idx - tt * DVT, c = col0 + j;
            vs[idx] = c < a.dv ? a.v[(size_t)(c0 + tt) * a.ldv + h * a.dv + c] : 0.0f;
        }
        __syncthreads();
        if (cl < DVT) {
            for (int tt = 0; tt < tc; ++tt) {
                const float4* qq = reinterpret_cast<const float4*>(qs + tt * tstride + part * pstride);
                const float4* kk = reinterpret_cast<const float4*>(ks + tt * tstride + part * pstride);
                const float4* gg = reinterpret_cast<const float4*>(gs + tt * tstride + part * pstride);
                float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
                for (int i = 0; i < DKP / 4; ++i) {
                    const float4 g4 = gg[i], k4 = kk[i];
                    S[4 * i] *= g4.x; S[4 * i + 1] *= g4.y; S[4 * i + 2] *= g4.z; S[4 * i + 3] *= g4.w;
                    p0 = fmaf(S[4 * i], k4.x, p0);
                    p1 = fmaf(S[4 * i + 1], k4.y, p1);
                    p0 = fmaf(S[4 * i + 2], k4.z, p0);
                    p1 = fmaf(S[4 * i + 3], k4.w, p1);
                }
                float p = p0 + p1;
                for (int o = 1; o < P; o <<= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
                const float u = bs[tt] * (vs[tt * DVT + cl] - p);
                float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
                for (int i = 0; i < DKP / 4; ++i) {
                    const float4 k4 = kk[i], q4 = qq[i];
                    S[4 * i] = fmaf(k4.x, u, S[4 * i]);
                    S[4 * i + 1] = fmaf(k4.y, u, S[4 * i + 1]);
                    S[4 * i + 2] = fmaf(k4.z, u, S[4 * i + 2]);
                    S[4 * i + 3] = fmaf(k4.w, u, S[4 * i + 3]);
                    o0 = fmaf(S[4 * i], q4.x, o0);
                    o1 = fmaf(S[4 * i + 1], q4.y, o1);
                    o0 = fmaf(S[4 * i + 2], q4.z, o0);
                    o1 = fmaf(S[4 * i + 3], q4.w, o1);
                }
                float o = o0 + o1;
                for (int d = 1; d < P; d <<= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
                if (part == 0) os[tt * DVT + cl] = o;
            }
        }
        __syncthreads();
        for (int idx = tid; idx < tc * DVT; idx += nthreads) {
            const int tt = idx / DVT, j = idx - tt * DVT, c = col0 + j;
            if (c < a.dv) a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + c] = os[idx];
        }
    }
#pragma unroll
    for (int i = 0; i < DKP; ++i) {
        const int kr = part * DKP + i;
        if (col_ok && kr < a.dk) st[(size_t)kr * a.dv + col] = S[i];
    }
}

// ---- the same for steps that bring portions of many tokens, in two kernels.
// delta_prepare_kernel, a warp per token and head: what the recurrence reads per token, into rows of float
//   work[t] = [ q: G * dk | k: G * dk | g: H * dk | beta: H | qk: G ]   (q, k unit vectors, q scaled; qk = q . k)
// so that nothing but the recurrence itself is left in the walk over the tokens.
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(DeltaArgs a, float* __restrict__ work, long long ldw, int n) {
    pdl_start();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (long long)n * a.H) return;
    const size_t row = (size_t)(item / a.H);
    const int h = (int)(item % a.H);
    float* w = work + row * ldw;
    const int per = a.H / a.G, dk = a.dk;
    if (h % per == 0) {                                   // the first head of a group norms the group's q and k
        const int kvh = h / per;
        const float* qr = a.q + row * a.ldq + kvh * dk;
        const float* kr = a.k + row * a.ldk + kvh * dk;
        float sq = 0.0f, sk = 0.0f, qk = 0.0f;
        for (int i = lane; i < dk; i += 32) { const float x = qr[i], y = kr[i]; sq = fmaf(x, x, sq); sk = fmaf(y, y, sk); qk = fmaf(x, y, qk); }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        qk = warp_sum(qk);
        const float rq = a.q_scale / sqrtf(sq + a.unit_eps), rk = 1.0f / sqrtf(sk + a.unit_eps);
        for (int i = lane; i < dk; i += 32) { w[kvh * dk + i] = qr[i] * rq; w[(a.G + kvh) * dk + i] = kr[i] * rk; }
        if (lane == 0) w[(2 * a.G + a.H) * dk + a.H + kvh] = qk * rq * rk;
    }
    const float rate = expf(a.a_log[h]);
    const T* dp = (const T*)a.decay_pre + row * a.lda + h * dk;
    for (int i = lane; i < dk; i += 32)
        w[(2 * a.G + h) * dk + i] = expf(-rate * gr_softplus(to_f32<T>(dp[i]) + a.dt_bias[h * dk + i]));
    if (lane == 0) w[(2 * a.G + a.H) * dk + h] = gr_sigmoid(to_f32<T>(((const T*)a.beta_pre)[row * a.ldb + h]));
}

// delta_walk_kernel, grid (request, head, tile of DVT value channels), P lanes of a warp per column of S, DKP rows of
// the column in a thread's registers.  With S' = diag(g) S, both sums over key channels that a token needs come from S':
//   p = k . S'[:, c],  r = q . S'[:, c];   u = beta (v_c - p);   S[:, c] = S'[:, c] + k u;   o_c = r + (q . k) u
// so a token costs one round of shuffles, for two sums at once.  Chunks of a.chunk tokens' rows go through shared memory.
__device__ __forceinline__ void walk_copy(float* smem, const float* gmem, int bytes) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem) : "memory");
}

template <int DKP>
__global__ void __launch_bounds__(128)
delta_walk_kernel(DeltaArgs a, const float* __restrict__ work, long long ldw, int P, int DVT) {
    extern __shared__ __align__(16) float sm[];
    pdl_start();
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DVT;
    const int kvh = h / (a.H / a.G);
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int part = tid % P, cl = tid / P;
    const int col = col0 + cl;
    const bool col_ok = cl < DVT && col < a.dv;
    const int pstride = DKP + 4, tstride = P * pstride, dk = a.dk, TC = a.chunk;
    // two buffers of a chunk's rows, filled by asynchronous copies while the chunk before is walked:
    // [q, k, g: TC x tstride each][v: TC x DVT][beta, q . k: TC x 2], then the chunk's outputs [TC x DVT]
    const int buf_floats = TC * (3 * tstride + DVT + 2);
    float* os = sm + 2 * buf_floats;
    const int row0 = a.q_start[r], row1 = a.q_start[r + 1];
    float* st = a.state + (((size_t)a.state_slots[r] * a.H + h) * dk) * a.dv;
    float S[DKP];
#pragma unroll
    for (int i = 0; i < DKP; ++i) {
        const int kr = part * DKP + i;
        S[i] = (col_ok && kr < dk) ? st[(size_t)kr * a.dv + col] : 0.0f;
    }
    const int off_q = kvh * dk, off_k = (a.G + kvh) * dk, off_g = (2 * a.G + h) * dk, off_b = (2 * a.G + a.H) * dk;
    // key channels beyond dk: q = k = 0, g = 1, written once (the copies never touch them)
    for (int idx = tid; idx < 2 * TC * P * DKP; idx += nthreads) {
        const int b = idx / (TC * P * DKP), rest = idx - b * (TC * P * DKP);
        const int tt = rest / (P * DKP), i = rest - tt * (P * DKP);
        if (i >= dk) {
            float* base = sm + b * buf_floats + tt * tstride + (i / DKP) * pstride + i % DKP;
            base[0] = 0.0f;
            base[TC * tstride] = 0.0f;
            base[2 * TC * tstride] = 1.0f;
        }
    }
    const bool wide = (dk & 3) == 0;               // rows of the prepared inputs start on 16 bytes, so do their heads then
    const int piece = wide ? 4 : 1, pieces = dk / piece;
    auto fetch = [&](int c0, int b) {
        const int tc = min(TC, row1 - c0);
        float* qs = sm + b * buf_floats;
        float* vs = qs + 3 * TC * tstride;
        float* bs = vs + TC * DVT;
        for (int idx = tid; idx < tc * pieces; idx += nthreads) {
            const int tt = idx / pieces, i = (idx - tt * pieces) * piece;
            const float* w = work + (size_t)(c0 + tt) * ldw;
            float* at = qs + tt * tstride + (i / DKP) * pstride + i % DKP;
            walk_copy(at, w + off_q + i, 4 * piece);
            walk_copy(at + TC * tstride, w + off_k + i, 4 * piece);
            walk_copy(at + 2 * TC * tstride, w + off_g + i, 4 * piece);
        }
        for (int idx = tid; idx < tc * DVT; idx += nthreads) {
            const int tt = idx / DVT, j = idx - tt * DVT, c = col0 + j;
            if (c < a.dv) walk_copy(vs + idx, a.v + (size_t)(c0 + tt) * a.ldv + h * a.dv + c, 4);
        }
        for (int idx = tid; idx < 2 * tc; idx += nthreads) {
            const int tt = idx >> 1;
            walk_copy(bs + idx, work + (size_t)(c0 + tt) * ldw + off_b + ((idx & 1) ? a.H + kvh : h), 4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (row0 < row1) fetch(row0, 0);
    int b = 0;
    for (int c0 = row0; c0 < row1; c0 += TC, b ^= 1) {
        const int tc = min(TC, row1 - c0);
        if (c0 + TC < row1) {
            fetch(c0 + TC, b ^ 1);                 // its buffer was walked two chunks ago; the barriers since cover it
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                           // everybody's copies of this chunk have landed; the outputs before are stored
        const float* qs = sm + b * buf_floats;
        const float* ks = qs + TC * tstride;
        const float* gs = ks + TC * tstride;
        const float* vs = gs + TC * tstride;
        const float* bs = vs + TC * DVT;
        if (cl < DVT) {
            // the rows of the token after this one are read from shared memory while this one's sums run; two sets of
            // registers take turns, so nothing is copied between them
            struct Rows { float4 q[DKP / 4], k[DKP / 4], g[DKP / 4]; float beta, qk, v; };
            const float* mine = qs + part * pstride;
            auto read = [&](Rows& w, int tt) {
                const float* at = mine + tt * tstride;
#pragma unroll
                for (int i = 0; i < DKP / 4; ++i) {
                    w.q[i] = reinterpret_cast<const float4*>(at)[i];
                    w.k[i] = reinterpret_cast<const float4*>(at + TC * tstride)[i];
                    w.g[i] = reinterpret_cast<const float4*>(at + 2 * TC * tstride)[i];
                }
                w.beta = bs[2 * tt];
                w.qk = bs[2 * tt + 1];
                w.v = col_ok ? vs[tt * DVT + cl] : 0.0f;
            };
            auto token = [&](const Rows& w, Rows& next, int tt) {
                if (tt + 1 < tc) read(next, tt + 1);
                float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f, r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f;
#pragma unroll
                for (int i = 0; i < DKP / 4; ++i) {
                    S[4 * i] *= w.g[i].x; S[4 * i + 1] *= w.g[i].y; S[4 * i + 2] *= w.g[i].z; S[4 * i + 3] *= w.g[i].w;
                    p0 = fmaf(S[4 * i], w.k[i].x, p0);     r0 = fmaf(S[4 * i], w.q[i].x, r0);
                    p1 = fmaf(S[4 * i + 1], w.k[i].y, p1); r1 = fmaf(S[4 * i + 1], w.q[i].y, r1);
                    p2 = fmaf(S[4 * i + 2], w.k[i].z, p2); r2 = fmaf(S[4 * i + 2], w.q[i].z, r2);
                    p3 = fmaf(S[4 * i + 3], w.k[i].w, p3); r3 = fmaf(S[4 * i + 3], w.q[i].w, r3);
                }
                float p = (p0 + p1) + (p2 + p3), rr = (r0 + r1) + (r2 + r3);
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    if (o < P) {
                        p += __shfl_xor_sync(0xffffffffu, p, o);
                        rr += __shfl_xor_sync(0xffffffffu, rr, o);
                    }
                }
                const float u = w.beta * (w.v - p);
#pragma unroll
                for (int i = 0; i < DKP / 4; ++i) {
                    S[4 * i] = fmaf(w.k[i].x, u, S[4 * i]);
                    S[4 * i + 1] = fmaf(w.k[i].y, u, S[4 * i + 1]);
                    S[4 * i + 2] = fmaf(w.k[i].z, u, S[4 * i + 2]);
                    S[4 * i + 3] = fmaf(w.k[i].w, u, S[4 * i + 3]);
                }
                if (part == 0) os[tt * DVT + cl] = fmaf(w.qk, u, rr);
            };
            Rows even, odd;
            read(even, 0);
            for (int tt = 0; tt < tc; tt += 2) {
                token(even, odd, tt);
                if (tt + 1 < tc) token(odd, even, tt + 1);
            }
        }
        __syncthreads();
        for (int idx = tid; idx < tc * DVT; idx += nthreads) {
            const int tt = idx / DVT, j = idx - tt * DVT, c = col0 + j;
            if (c < a.dv) a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + c] = os[idx];
        }
    }
#pragma unroll
    for (int i = 0; i < DKP; ++i) {
        const int kr = part * DKP + i;
        if (col_ok && kr < dk) st[(size_t)kr * a.dv + col] = S[i];
    }
}

// Floats of a token's row of the prepared inputs (ops.py has the same formula).
static long long delta_work_row(int H, int G, int dk) { return ((long long)(2 * G + H) * dk + H + G + 3) / 4 * 4; }

template <typename T>
static int launch_delta(const DeltaArgs& a, int n_reqs, cudaStream_t s);

constexpr int WALK_SMEM = 64 * 1024;

template <int DKP>
static int launch_walk(const DeltaArgs& b, dim3 grid, int threads, size_t bytes, const float* work, long long ldw, int P, int dvt,
                       cudaStream_t s) {
    static unsigned long long configured = 0;
    if (int e = vcb_allow_dynamic_smem(delta_walk_kernel<DKP>, WALK_SMEM, &configured)) return e;
    vcb_launch(delta_walk_kernel<DKP>, grid, threads, bytes, s, b, work, ldw, P, dvt);
    return vcb_last_error();
}

template <typename T>
static int launch_delta_portions(const DeltaArgs& a, int n_reqs, int n_tokens, float* work, cudaStream_t s) {
    // 8 rows of a column per thread where the key channels fill 16 lanes (keys of 128), fewer lanes for shorter keys, 16 rows
    // for longer ones; CTAs of four warps, so that a head's columns spread over many SMs.  Measured at 16 heads of 128 x 128
    // over 2,048 tokens: 16 rows a thread or 4 rows in CTAs of 16 warps are both slower.
    const int dkp = a.dk > 256 ? 16 : 8;
    int P = 1;
    while (P * dkp < a.dk) P <<= 1;
    const int dvt = 128 / P >= 32 ? 32 : 128 / P;
    int chunk = 16;
    auto bytes = [&](int tc) { return (size_t)tc * (2 * (3 * P * (dkp + 4) + dvt + 2) + dvt) * sizeof(float); };
    while (chunk > 4 && bytes(chunk) > WALK_SMEM) chunk >>= 1;
    if (P > 32 || bytes(chunk) > WALK_SMEM) return launch_delta<T>(a, n_reqs, s);      // keys beyond 512 channels: the kernel above
    const long long ldw = delta_work_row(a.H, a.G, a.dk);
    const long long items = (long long)n_tokens * a.H;
    vcb_launch(delta_prepare_kernel<T>, dim3((unsigned)((items + 3) / 4)), 128, 0, s, a, work, ldw, n_tokens);
    if (int e = vcb_last_error()) return e;
    DeltaArgs b = a;
    b.chunk = chunk;
    dim3 grid(n_reqs, a.H, (a.dv + dvt - 1) / dvt);
    const int threads = dvt * P;
    if (dkp == 8) return launch_walk<8>(b, grid, threads, bytes(chunk), work, ldw, P, dvt, s);
    return launch_walk<16>(b, grid, threads, bytes(chunk), work, ldw, P, dvt, s);
}

template <typename T>
static int launch_delta(const DeltaArgs& a, int n_reqs, cudaStream_t s) {
    const int dkp = a.dk <= 32 ? 8 : a.dk <= 64 ? 16 : 32;
    int P = 1;
    while (P * dkp < a.dk) P <<= 1;
    if (P > 32) return VCB_ERR_UNSUPPORTED;
    const int dvt = P <= 8 ? 32 : 256 / P;
    const int threads = ((dvt * P + 31) / 32) * 32;
    int chunk = 16;
    auto bytes = [&](int tc) { return ((size_t)tc * (3 * P * (dkp + 4) + 2 * dvt + 1)) * sizeof(float); };
    while (chunk > 1 && bytes(chunk) > 48 * 1024) chunk >>= 1;
    DeltaArgs b = a;
    b.chunk = chunk;
    dim3 grid(n_reqs, a.H, (a.dv + dvt - 1) / dvt);
    if (dkp == 8) vcb_launch(gated_delta_scan_kernel<T, 8>, grid, threads, bytes(chunk), s, b, P, dvt);
    else if (dkp == 16) vcb_launch(gated_delta_scan_kernel<T, 16>, grid, threads, bytes(chunk), s, b, P, dvt);
    else vcb_launch(gated_delta_scan_kernel<T, 32>, grid, threads, bytes(chunk), s, b, P, dvt);
    return vcb_last_error();
}

VCB_EXPORT int vcb_gated_delta_scan(const float* q, const float* k, const float* v, long long ldq, long long ldk, long long ldv,
                                    const void* beta_pre, long long ldb, const void* decay_pre, long long lda,
                                    const float* a_log, const float* dt_bias, float* state, float* out, long long ldo,
                                    const int* q_start, const int* state_slots, int n_reqs, int H, int G, int dk, int dv,
                                    float q_scale, float unit_eps, int dtype, float* work, int n_tokens, void* stream) {
    if (n_reqs <= 0) return 0;
    if (!q || !k || !v || !beta_pre || !decay_pre || !a_log || !dt_bias || !state || !out || H <= 0 || G <= 0 || H % G ||
        dk <= 0 || dv <= 0 || H > 65535 || (dv + 7) / 8 > 65535)
        return VCB_ERR_BAD_ARG;
    DeltaArgs a{q, k, v, ldq, ldk, ldv, beta_pre, ldb, decay_pre, lda, a_log, dt_bias, state, out, ldo, q_start, state_slots,
                H, G, dk, dv, q_scale, unit_eps, 0};
    cudaStream_t s = (cudaStream_t)stream;
    if (work && n_tokens > 0) {                   // a step with portions: inputs prepared for all tokens at once, then the walk
        if (dtype == VCB_F32) return launch_delta_portions<float>(a, n_reqs, n_tokens, work, s);
        if (dtype == VCB_BF16) return launch_delta_portions<__nv_bfloat16>(a, n_reqs, n_tokens, work, s);
        return VCB_ERR_BAD_ARG;
    }
    if (dtype == VCB_F32) return launch_delta<float>(a, n_reqs, s);
    if (dtype == VCB_BF16) return launch_delta<__nv_bfloat16>(a, n_reqs, s);
    return VCB_ERR_BAD_ARG;
}
