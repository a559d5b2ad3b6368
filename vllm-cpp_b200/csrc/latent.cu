// Kernels of latent attention: keys and values of all heads are projections of one low-rank row per
// token (the latent), and only that row is cached.
//
//   latent_cache_write_kernel   c = raw / sqrt(mean(raw^2) + eps) * gain  ->  the token's slot of a cache
//                               whose pages hold one plane of rows (kv_pos layout, common.cuh)
//   headwise_linear_kernel      out[t, h, :] = x[t, h, :] W_h^T for every head h (a block-diagonal product):
//                               queries into the latent space (W_h = Wuk_h^T) so that scores are taken against
//                               the cached rows directly, and attention's result back out of it (W_h = Wuv_h),
//                               there with an optional sigmoid gate on the result
//
// With the queries absorbed, attention over the latent rows is multi-query attention with one shared
// key/value row of `rank` elements per token, and runs on the engine's attention kernels with the value
// plane of a page being its key plane.  The reference has no such layer.
#include "common.cuh"

// ------------------------------------------------------ norm of the latent + cache write
// One warp per token.  raw: [n, ld] rows of the product that made it (the latent's columns start at raw).
template <typename T>
__global__ void latent_cache_write_kernel(const T* __restrict__ raw, int ld, const float* __restrict__ gain,
                                          const int* __restrict__ positions, const int* __restrict__ req_of_token,
                                          const int* __restrict__ block_table, int bt_stride, T* __restrict__ cache,
                                          size_t page_stride, int n_tokens, int rank, int page, float eps,
                                          int num_pages, int* status) {
    pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    const T* row = raw + (size_t)t * ld;
    float ss = 0.0f;
    for (int i = lane; i < rank; i += 32) {
        const float v = to_f32<T>(row[i]);
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)rank + eps);
    const int pos = positions[t];
    const int lp = pos / page, slot = pos - lp * page;
    const int pg = lp < bt_stride ? block_table[(size_t)req_of_token[t] * bt_stride + lp] : -1;
    if ((unsigned)pg >= (unsigned)num_pages) {
        if (status && lane == 0) atomicCAS(status, 0, VCB_STATUS_BAD_PAGE);
        return;
    }
    T* dst = cache + (size_t)pg * page_stride;
    for (int i = lane; i < rank; i += 32)
        dst[kv_pos(i, slot, rank, page, (int)sizeof(T))] = from_f32<T>((to_f32<T>(row[i]) * r) * gain[i]);
}

VCB_EXPORT int vcb_latent_cache_write(const void* raw, int ld, const float* gain, const int* positions,
                                      const int* req_of_token, const int* block_table, int bt_stride, void* cache,
                                      long long page_stride, int n_tokens, int rank, int page, float eps, int num_pages,
                                      int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || page <= 0 || ld < rank || page_stride < (long long)page * rank || num_pages <= 0) return VCB_ERR_BAD_ARG;
    const int warps = 4, blocks = (n_tokens + warps - 1) / warps;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        vcb_launch(latent_cache_write_kernel<float>, blocks, warps * 32, 0, s, (const float*)raw, ld, gain, positions,
                   req_of_token, block_table, bt_stride, (float*)cache, (size_t)page_stride, n_tokens, rank, page, eps,
                   num_pages, status);
    else if (dtype == VCB_BF16)
        vcb_launch(latent_cache_write_kernel<__nv_bfloat16>, blocks, warps * 32, 0, s, (const __nv_bfloat16*)raw, ld, gain,
                   positions, req_of_token, block_table, bt_stride, (__nv_bfloat16*)cache, (size_t)page_stride, n_tokens,
                   rank, page, eps, num_pages, status);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------ per-head products
// out[t, h, n] = sum_k x[t, h, k] * w[h, n, k]   (w: [heads, N, K] contiguous; x rows ldx apart with head h
// at column h * K + x0; out rows ldo apart with head h at column h * N), float accumulation.
// gate (may be null; rows ldg apart, head h at column h * N): out *= sigmoid(gate).
// 64 x 64 output tile per CTA and head, 32-deep k slices in shared memory, a 4 x 4 register tile per thread,
// every edge guarded.  With few tokens the weights are read once and the kernel runs at the rate they
// stream at; long portions in bfloat16 go to the library's batched product instead (ops.headwise_linear).
#define HT 64
#define HK 32

template <typename T>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, const T* __restrict__ gate,
                       int M, int N, int K, int ldx, int ldo, int ldg, int gate_per_head) {
    // rows 68 floats apart: a thread's four values of a k are one 16-byte load (the loop is bound by shared-memory
    // loads, not by the multiplications)
    __shared__ __align__(16) float As[HK][HT + 4];
    __shared__ __align__(16) float Ws[HK][HT + 4];
    pdl_start();
    const int h = blockIdx.z;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * HT, n0 = blockIdx.x * HT;
    const T* xh = x + (size_t)h * K;
    const T* wh = w + (size_t)h * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    // a slice is 64 rows x 32 k per operand, 8 elements a thread; the next slice is fetched into registers
    // while this one is multiplied, so a global load's latency is paid once, not once per slice
    float pa[8], pw[8];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int idx = threadIdx.x + e * 256;
            const int r = idx / HK, k = k0 + idx % HK;
            pa[e] = (m0 + r < M && k < K) ? to_f32<T>(xh[(size_t)(m0 + r) * ldx + k]) : 0.0f;
            pw[e] = (n0 + r < N && k < K) ? to_f32<T>(wh[(size_t)(n0 + r) * K + k]) : 0.0f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += HK) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int idx = threadIdx.x + e * 256;
            As[idx % HK][idx / HK] = pa[e];
            Ws[idx % HK][idx / HK] = pw[e];
        }
        __syncthreads();
        if (k0 + HK < K) fetch(k0 + HK);
#pragma unroll
        for (int kk = 0; kk < HK; ++kk) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (gate) v *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)m * ldg + (gate_per_head ? (size_t)h : (size_t)h * N + n)])));
            out[(size_t)m * ldo + (size_t)h * N + n] = from_f32<T>(v);
        }
    }
}

// The same product on tensor cores for bfloat16 steps of few tokens (mma.sync m16n8k16, float accumulation): a warp
// owns 16 tokens x 32 features of one head and walks K in steps of 16, its fragments loaded straight from global
// memory as 32-bit pairs (both operands have K innermost, which is the layout the instruction's row x col form wants;
// the operands of a step of few tokens are small and stay in L1/L2).  K a multiple of 16, N of 8, even strides.
#define HW_WARPS 2
__device__ __forceinline__ void hw_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(HW_WARPS * 32)
headwise_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate,
                           int M, int N, int K, int ldx, int ldo, int ldg, int gate_per_head) {
    pdl_start();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * 16, n0 = (blockIdx.x * HW_WARPS + warp) * 32;
    if (n0 >= N) return;
    const int qr = lane >> 2, qc = (lane & 3) * 2;
    const __nv_bfloat16* xa = x + (size_t)h * K + (size_t)(m0 + qr) * ldx + qc;        // rows qr and qr + 8 of the token tile
    const bool ra = m0 + qr < M, rb = m0 + qr + 8 < M;
    const __nv_bfloat16* wb = w + ((size_t)h * N + n0 + qr) * K + qc;                  // feature n0 + 8 * j + qr
    bool nb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) nb[j] = n0 + 8 * j + qr < N;
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
#pragma unroll 4
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t a[4], b[4][2];
        a[0] = ra ? *reinterpret_cast<const uint32_t*>(xa + k0) : 0u;
        a[1] = rb ? *reinterpret_cast<const uint32_t*>(xa + (size_t)8 * ldx + k0) : 0u;
        a[2] = ra ? *reinterpret_cast<const uint32_t*>(xa + k0 + 8) : 0u;
        a[3] = rb ? *reinterpret_cast<const uint32_t*>(xa + (size_t)8 * ldx + k0 + 8) : 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            b[j][0] = nb[j] ? *reinterpret_cast<const uint32_t*>(wb + (size_t)8 * j * K + k0) : 0u;
            b[j][1] = nb[j] ? *reinterpret_cast<const uint32_t*>(wb + (size_t)8 * j * K + k0 + 8) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) hw_mma(acc[j], a, b[j][0], b[j][1]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int n = n0 + 8 * j + qc;
        if (n >= N) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + qr + 8 * half;
            if (m >= M) continue;
            float v0 = acc[j][2 * half], v1 = acc[j][2 * half + 1];
            if (gate && gate_per_head) {
                const float g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)m * ldg + h])));
                v0 *= g;
                v1 *= g;
            } else if (gate) {
                const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + (size_t)m * ldg + (size_t)h * N + n));
                v0 *= 1.0f / (1.0f + expf(-g.x));
                v1 *= 1.0f / (1.0f + expf(-g.y));
            }
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)m * ldo + (size_t)h * N + n) = __floats2bfloat162_rn(v0, v1);
        }
    }
}

// gate_per_head 1: the gate holds one number per head ([M, heads] rows ldg apart) instead of one per output.
VCB_EXPORT int vcb_headwise_linear(const void* x, const void* w, void* out, const void* gate, int M, int heads, int N,
                                   int K, int ldx, int ldo, int ldg, int gate_per_head, int dtype, void* stream) {
    if (M <= 0 || heads <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < heads * K || ldo < heads * N || (gate && ldg < (gate_per_head ? heads : heads * N)) || heads > 65535)
        return VCB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t addrs = (uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (gate_per_head ? 0 : (uintptr_t)gate);
    if (dtype == VCB_BF16 && K % 16 == 0 && N % 8 == 0 && !(addrs & 3) && !((ldx | ldo | (gate_per_head ? 0 : ldg)) & 1) && (M + 15) / 16 <= 65535) {
        dim3 mgrid((N + 32 * HW_WARPS - 1) / (32 * HW_WARPS), (M + 15) / 16, heads);
        vcb_launch(headwise_linear_mma_kernel, mgrid, HW_WARPS * 32, 0, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                   (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, M, N, K, ldx, ldo, ldg, gate_per_head);
        return vcb_last_error();
    }
    dim3 grid((N + HT - 1) / HT, (M + HT - 1) / HT, heads);
    if (grid.y > 65535) return VCB_ERR_UNSUPPORTED;
    if (dtype == VCB_F32)
        vcb_launch(headwise_linear_kernel<float>, grid, 256, 0, s, (const float*)x, (const float*)w, (float*)out,
                   (const float*)gate, M, N, K, ldx, ldo, ldg, gate_per_head);
    else if (dtype == VCB_BF16)
        vcb_launch(headwise_linear_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                   (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, M, N, K, ldx, ldo, ldg, gate_per_head);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// out[t, i] *= sigmoid(gate[t, i / group]) in place (rows ldo and ldg apart; group 1: a gate per element, group N:
// one per run of N outputs, a head): the gate where the product before it was the library's.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ gate, int n, int cols, int ldo, int ldg, int group) {
    pdl_start();
    const size_t total = (size_t)n * cols;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / cols, i = idx - t * cols;
        const float v = to_f32<T>(out[t * ldo + i]);
        out[t * ldo + i] = from_f32<T>(v * (1.0f / (1.0f + expf(-to_f32<T>(gate[t * ldg + i / group])))));
    }
}

// bfloat16 rows of a multiple of 8 columns, 16-byte aligned: eight elements a thread.
__global__ void sigmoid_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate, int n,
                                           int cols, int ldo, int ldg) {
    pdl_start();
    const int nvec = cols >> 3;
    const long long total = (long long)n * nvec;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / nvec;
        const int i = (int)(idx - t * nvec) * 8;
        uint4 ov = *reinterpret_cast<const uint4*>(out + t * ldo + i);
        const uint4 gv = *reinterpret_cast<const uint4*>(gate + t * ldg + i);
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 o = __bfloat1622float2(o2[e]), g = __bfloat1622float2(g2[e]);
            o2[e] = __floats2bfloat162_rn(o.x * (1.0f / (1.0f + expf(-g.x))), o.y * (1.0f / (1.0f + expf(-g.y))));
        }
        *reinterpret_cast<uint4*>(out + t * ldo + i) = ov;
    }
}

VCB_EXPORT int vcb_sigmoid_gate(void* out, const void* gate, int n, int cols, int ldo, int ldg, int group, int dtype, void* stream) {
    if (n <= 0 || cols <= 0) return 0;
    if (group <= 0 || cols % group || ldo < cols || ldg < cols / group) return VCB_ERR_BAD_ARG;
    const size_t total = (size_t)n * cols;
    const int blocks = (int)((total + 255) / 256 < (size_t)vcb_sm_count() * 8 ? (total + 255) / 256 : (size_t)vcb_sm_count() * 8);
    cudaStream_t s = (cudaStream_t)stream;
    if (group == 1 && dtype == VCB_BF16 && cols % 8 == 0 && ldo % 8 == 0 && ldg % 8 == 0 && !(((uintptr_t)out | (uintptr_t)gate) & 15)) {
        const long long want = ((long long)n * (cols / 8) + 255) / 256, cap = (long long)vcb_sm_count() * 16;
        vcb_launch(sigmoid_gate_bf16x8_kernel, (int)(want < cap ? want : cap), 256, 0, s, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gate, n, cols, ldo, ldg);
        return vcb_last_error();
    }
    if (dtype == VCB_F32)
        vcb_launch(sigmoid_gate_kernel<float>, blocks, 256, 0, s, (float*)out, (const float*)gate, n, cols, ldo, ldg, group);
    else if (dtype == VCB_BF16)
        vcb_launch(sigmoid_gate_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, n,
                   cols, ldo, ldg, group);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------ RMS norm of rows of the activations' type
// out[t, i] = x[t, i] / sqrt(mean_i x[t, i]^2 + eps) * gain[i]  (statistics and products float; rows ldx / ldo apart):
// the norm of a low-rank row between two products.  A warp per row.
template <typename T>
__global__ void rows_rmsnorm_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ gain, T* __restrict__ out,
                                    int ldo, int n, int width, float eps) {
    pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n) return;
    const T* row = x + (size_t)t * ldx;
    float ss = 0.0f;
    for (int i = lane; i < width; i += 32) {
        const float v = to_f32<T>(row[i]);
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
    T* dst = out + (size_t)t * ldo;
    for (int i = lane; i < width; i += 32) dst[i] = from_f32<T>((to_f32<T>(row[i]) * r) * gain[i]);
}

VCB_EXPORT int vcb_rows_rmsnorm(const void* x, int ldx, const float* gain, void* out, int ldo, int n, int width, float eps,
                                int dtype, void* stream) {
    if (n <= 0) return 0;
    if (!x || !gain || !out || width <= 0 || ldx < width || ldo < width) return VCB_ERR_BAD_ARG;
    const int warps = 4, blocks = (n + warps - 1) / warps;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        vcb_launch(rows_rmsnorm_kernel<float>, blocks, warps * 32, 0, s, (const float*)x, ldx, gain, (float*)out, ldo, n, width, eps);
    else if (dtype == VCB_BF16)
        vcb_launch(rows_rmsnorm_kernel<__nv_bfloat16>, blocks, warps * 32, 0, s, (const __nv_bfloat16*)x, ldx, gain,
                   (__nv_bfloat16*)out, ldo, n, width, eps);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------- latent + one rotated key part that all heads share
// A token's cached row is [c | kr]: c the RMS-normed latent (rank wide, as latent_cache_write_kernel makes it) and kr a
// key part of `rot` coordinates, turned by the token's position, that every head scores against the rotated part of
// its query.  The same kernel turns the rotated part of every head's query in place: head h of q holds it at
// q[t, h * q_stride + q_off .. + rot).  Pair j of a rotated part is (2j, 2j + 1) (pairing 1) or (j, j + rot / 2)
// (pairing 0); its angle is position * inv_freq[j] in float; (u, v) -> (u cos - v sin, v cos + u sin).
// A CTA per token.
struct LatentRopeArgs {
    const void* raw;            // [n, ld]: the latent's columns, then the rot columns of the shared key part
    int ld;
    const float* gain;          // [rank]
    void* q;                    // [n, ldq], turned in place (null: no queries)
    int ldq, heads, q_stride, q_off;
    const float* inv_freq;      // [rot / 2]
    int rot, pairing;
    const int* positions;
    const int* req_of_token;
    const int* block_table;
    int bt_stride;
    void* cache;
    size_t page_stride;
    int n_tokens, rank, page, num_pages, write_kv;
    float eps;
    int* status;
};

template <typename T>
__global__ void latent_rope_cache_write_kernel(LatentRopeArgs a) {
    __shared__ float scratch[33];
    pdl_start();
    const int t = blockIdx.x;
    const int pos = a.positions[t];
    const int half = a.rot >> 1;
    const int row_w = a.rank + a.rot;
    // the queries' rotated parts, in place: a thread per (head, pair)
    if (a.q) {
        T* q = (T*)a.q + (size_t)t * a.ldq;
        for (int idx = threadIdx.x; idx < a.heads * half; idx += blockDim.x) {
            const int h = idx / half, j = idx - h * half;
            float sn, cs;
            sincosf((float)pos * a.inv_freq[j], &sn, &cs);
            T* part = q + (size_t)h * a.q_stride + a.q_off;
            const int iu = a.pairing ? 2 * j : j, iv = a.pairing ? 2 * j + 1 : j + half;
            const float u = to_f32<T>(part[iu]), v = to_f32<T>(part[iv]);
            part[iu] = from_f32<T>(u * cs - v * sn);
            part[iv] = from_f32<T>(v * cs + u * sn);
        }
    }
    if (!a.write_kv) return;
    const T* row = (const T*)a.raw + (size_t)t * a.ld;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)a.rank + a.eps);
    const int lp = pos / a.page, slot = pos - lp * a.page;
    const int pg = lp < a.bt_stride ? a.block_table[(size_t)a.req_of_token[t] * a.bt_stride + lp] : -1;
    if ((unsigned)pg >= (unsigned)a.num_pages) {
        if (a.status && threadIdx.x == 0) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
        return;
    }
    T* dst = (T*)a.cache + (size_t)pg * a.page_stride;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x)
        dst[kv_pos(i, slot, row_w, a.page, (int)sizeof(T))] = from_f32<T>((to_f32<T>(row[i]) * r) * a.gain[i]);
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * a.inv_freq[j], &sn, &cs);
        const int iu = a.pairing ? 2 * j : j, iv = a.pairing ? 2 * j + 1 : j + half;
        const float u = to_f32<T>(row[a.rank + iu]), v = to_f32<T>(row[a.rank + iv]);
        dst[kv_pos(a.rank + iu, slot, row_w, a.page, (int)sizeof(T))] = from_f32<T>(u * cs - v * sn);
        dst[kv_pos(a.rank + iv, slot, row_w, a.page, (int)sizeof(T))] = from_f32<T>(v * cs + u * sn);
    }
}

VCB_EXPORT int vcb_latent_rope_cache_write(const void* raw, int ld, const float* gain, void* q, int ldq, int heads, int q_stride,
                                           int q_off, const float* inv_freq, int rot, int pairing, const int* positions,
                                           const int* req_of_token, const int* block_table, int bt_stride, void* cache,
                                           long long page_stride, int n_tokens, int rank, int page, float eps, int num_pages,
                                           int write_kv, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rot < 0 || (rot & 1) || (rot && !inv_freq) || page <= 0 || ld < rank + rot ||
        page_stride < (long long)page * (rank + rot) || num_pages <= 0 || (pairing != 0 && pairing != 1))
        return VCB_ERR_BAD_ARG;
    if (q && (heads <= 0 || q_off < 0 || q_stride < q_off + rot || ldq < heads * q_stride)) return VCB_ERR_BAD_ARG;
    LatentRopeArgs a{raw, ld, gain, q, ldq, heads, q_stride, q_off, inv_freq, rot, pairing, positions, req_of_token, block_table,
                     bt_stride, cache, (size_t)page_stride, n_tokens, rank, page, num_pages, write_kv, eps, status};
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) vcb_launch(latent_rope_cache_write_kernel<float>, n_tokens, 128, 0, s, a);
    else if (dtype == VCB_BF16) vcb_launch(latent_rope_cache_write_kernel<__nv_bfloat16>, n_tokens, 128, 0, s, a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
