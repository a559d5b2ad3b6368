// A feed-forward of many small experts of which every token uses a few, without the host in the loop:
//
//   moe_router_*_kernel      logits = W_r h in float; scores by softmax over all router outputs or by a sigmoid each; the
//                            `top` outputs with the largest (score + correction) chosen, optionally only among the best
//                            groups of neighbouring outputs; their plain scores kept as weights, optionally divided by
//                            their sum and scaled (RouteRule)
//   moe_sort_kernel          the (token, choice) pairs grouped by expert: a row for each pair in a list sorted by
//                            expert, and the list's tiles of up to TM rows of one expert
//   moe_expert_gemm_kernel   one product per tile against that expert's matrix; the first product gathers the
//                            tokens' rows, computes gate and up together and applies the experts' activation
//                              g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(alpha * g) * (u + up_shift)
//                            (limit = inf, alpha = 1, up_shift = 0: silu(gate) * up)
//   moe_combine_kernel       out[t] = sum over the token's choices of weight * (the expert's row, or h[t] itself for a
//                            router output beyond the experts: an identity expert)
//
// Grids are sized for the most tiles a step can have; a block beyond the step's count leaves at once, so the
// same launches serve every routing (and a captured step).  Router, softmax, weights and all sums are float.
// The reference has no routed feed-forward (src/layers/mlp.cpp is dense).
#include "common.cuh"

// ------------------------------------------------------------------------------------------- router
// Two kernels.  Logits: a CTA takes RT_TOK tokens and eight router outputs, a warp per output: the tokens' rows pass
// through shared memory in slabs (as float), a row of the float32 router matrix is read once for the CTA's tokens
// with 16-byte loads.  Selection: a warp per token does the softmax over all outputs, adds the correction and
// picks the `top` largest (the lower index wins among equals); the plain scores of the chosen are the weights.
#define RT_TOK 4
#define RT_SLAB 2048

template <typename T>
__global__ void __launch_bounds__(256)
moe_router_logits_kernel(const T* __restrict__ h, long long ldh, const float* __restrict__ wr, float* __restrict__ logits,
                         int n_tokens, int width, int n_out) {
    __shared__ __align__(16) float rows[RT_TOK][RT_SLAB];
    pdl_start();
    const int t0 = blockIdx.x * RT_TOK, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.y * 8 + warp;
    const bool vec = (width & 3) == 0 && (((uintptr_t)wr) & 15) == 0;
    float acc[RT_TOK];
#pragma unroll
    for (int t = 0; t < RT_TOK; ++t) acc[t] = 0.0f;
    for (int s0 = 0; s0 < width; s0 += RT_SLAB) {
        const int len = min(RT_SLAB, width - s0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < RT_TOK * len; idx += 256) {
            const int t = idx / len, i = idx - t * len;
            rows[t][i] = t0 + t < n_tokens ? to_f32<T>(h[(size_t)(t0 + t) * ldh + s0 + i]) : 0.0f;
        }
        __syncthreads();
        if (e < n_out) {
            const float* w = wr + (size_t)e * width + s0;
            if (vec) {
                // four 16-byte pieces of the router's row in flight per lane before any is used
                for (int i = lane * 4; i < len; i += 512) {
                    float4 a[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        a[u] = i + u * 128 < len ? *reinterpret_cast<const float4*>(w + i + u * 128) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (i + u * 128 >= len) break;
#pragma unroll
                        for (int t = 0; t < RT_TOK; ++t) {
                            const float4 x = *reinterpret_cast<const float4*>(&rows[t][i + u * 128]);
                            acc[t] = fmaf(x.x, a[u].x, fmaf(x.y, a[u].y, fmaf(x.z, a[u].z, fmaf(x.w, a[u].w, acc[t]))));
                        }
                    }
                }
            } else {
                for (int i = lane; i < len; i += 32) {
                    const float a = w[i];
#pragma unroll
                    for (int t = 0; t < RT_TOK; ++t) acc[t] = fmaf(rows[t][i], a, acc[t]);
                }
            }
        }
    }
    if (e >= n_out) return;
#pragma unroll
    for (int t = 0; t < RT_TOK; ++t) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && t0 + t < n_tokens) logits[(size_t)(t0 + t) * n_out + e] = v;
    }
}

// How the scores are made and used (the fields a design does not have stay at their neutral values).
struct RouteRule {
    int score_fn;               // 0: softmax over all outputs; 1: sigmoid of each logit
    int n_groups, keep_groups;  // outputs form n_groups equal groups of neighbours, only those of the keep_groups best may be chosen
    int group_top;              // a group's score: the sum of its group_top largest (score + correction); at most 4
    int normalize;              // 1: the chosen weights are divided by (their sum + sum_eps)
    float sum_eps, scale;       // scale multiplies the weights
};

__global__ void __launch_bounds__(128)
moe_router_select_kernel(const float* __restrict__ logits, const float* __restrict__ logit_bias, const float* __restrict__ correction,
                         int* __restrict__ ids, float* __restrict__ wts, int n_tokens, int n_out, int top, RouteRule rule) {
    extern __shared__ float sm[];
    pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= n_tokens) return;
    float* score = sm + (size_t)warp * (2 * n_out + rule.n_groups);      // [n_out] scores
    float* choice = score + n_out;                     // [n_out] score + correction; -inf once taken or shut out
    float* gscore = choice + n_out;                    // [n_groups]
    const float* zr = logits + (size_t)t * n_out;
    auto z = [&](int e) { return logit_bias ? zr[e] + logit_bias[e] : zr[e]; };      // the router's bias joins the logits themselves (float)
    if (rule.score_fn == 0) {
        float m = -INFINITY;
        for (int e = lane; e < n_out; e += 32) m = fmaxf(m, z(e));
        m = warp_max(m);
        float sum = 0.0f;
        for (int e = lane; e < n_out; e += 32) { const float p = expf(z(e) - m); score[e] = p; sum += p; }
        sum = warp_sum(sum);
        for (int e = lane; e < n_out; e += 32) score[e] = score[e] / sum;
    } else {
        for (int e = lane; e < n_out; e += 32) score[e] = 1.0f / (1.0f + expf(-z(e)));
    }
    for (int e = lane; e < n_out; e += 32) choice[e] = score[e] + (correction ? correction[e] : 0.0f);
    __syncwarp();
    if (rule.n_groups > 1 && rule.keep_groups < rule.n_groups) {
        const int per = n_out / rule.n_groups;
        for (int g = lane; g < rule.n_groups; g += 32) {
            float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            for (int e = g * per; e < (g + 1) * per; ++e) {
                float v = choice[e];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (v > best[k]) { const float tmp = best[k]; best[k] = v; v = tmp; }
            }
            float sum = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (k < rule.group_top && k < per) sum += best[k];
            gscore[g] = sum;
        }
        __syncwarp();
        // the groups that stay: keep_groups times the best of those left (the lower index among equals); a group that
        // stays gets +inf, and what is not +inf afterwards is shut out
        for (int k = 0; k < rule.keep_groups; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < rule.n_groups; g += 32) {
                const float v = gscore[g];
                if (v != INFINITY && (v > best || at == 0x7fffffff)) { best = v; at = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (lane == 0 && at != 0x7fffffff) gscore[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < n_out; e += 32)
            if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_out; e += 32)
            if (choice[e] > best) { best = choice[e]; at = e; }        // the lowest index among equals of a lane
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0) {
            ids[(size_t)t * top + k] = at;
            wts[(size_t)t * top + k] = score[at];
            choice[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0 && (rule.normalize || rule.scale != 1.0f)) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) sum += wts[(size_t)t * top + k];
        const float f = rule.normalize ? rule.scale / (sum + rule.sum_eps) : rule.scale;
        for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] *= f;
    }
}

// logits: float scratch [n_tokens, n_out].
// logit_bias: float [n_out] added to the logits before the scores are made, or null.
VCB_EXPORT int vcb_moe_router_biased(const void* h, long long ldh, const float* wr, const float* logit_bias, const float* correction,
                                     float* logits, int* ids, float* wts, int n_tokens, int width, int n_out, int top, int score_fn,
                                     int n_groups, int keep_groups, int group_top, int normalize, float sum_eps, float scale,
                                     int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!h || !wr || !logits || !ids || !wts || width <= 0 || n_out <= 0 || top <= 0 || top > n_out) return VCB_ERR_BAD_ARG;
    if (n_groups <= 0 || n_out % n_groups || keep_groups <= 0 || keep_groups > n_groups || group_top <= 0 || group_top > 4 ||
        (score_fn != 0 && score_fn != 1) || top > (n_out / n_groups) * keep_groups)
        return VCB_ERR_BAD_ARG;
    const size_t smem = (size_t)4 * (2 * n_out + n_groups) * sizeof(float);
    if (smem > 48 * 1024 || (n_out + 7) / 8 > 65535) return VCB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((n_tokens + RT_TOK - 1) / RT_TOK, (n_out + 7) / 8);
    if (dtype == VCB_F32) vcb_launch(moe_router_logits_kernel<float>, grid, 256, 0, s, (const float*)h, ldh, wr, logits, n_tokens, width, n_out);
    else if (dtype == VCB_BF16)
        vcb_launch(moe_router_logits_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)h, ldh, wr, logits, n_tokens, width, n_out);
    else return VCB_ERR_BAD_ARG;
    RouteRule rule{score_fn, n_groups, keep_groups, group_top, normalize, sum_eps, scale};
    vcb_launch(moe_router_select_kernel, (n_tokens + 3) / 4, 128, smem, s, (const float*)logits, logit_bias, correction, ids, wts, n_tokens, n_out, top, rule);
    return vcb_last_error();
}

VCB_EXPORT int vcb_moe_router_ruled(const void* h, long long ldh, const float* wr, const float* correction, float* logits, int* ids,
                                    float* wts, int n_tokens, int width, int n_out, int top, int score_fn, int n_groups,
                                    int keep_groups, int group_top, int normalize, float sum_eps, float scale, int dtype,
                                    void* stream) {
    return vcb_moe_router_biased(h, ldh, wr, nullptr, correction, logits, ids, wts, n_tokens, width, n_out, top, score_fn, n_groups,
                                 keep_groups, group_top, normalize, sum_eps, scale, dtype, stream);
}

// Softmax scores, no groups, the plain scores as weights.
VCB_EXPORT int vcb_moe_router(const void* h, long long ldh, const float* wr, const float* correction, float* logits, int* ids,
                              float* wts, int n_tokens, int width, int n_out, int top, int dtype, void* stream) {
    return vcb_moe_router_ruled(h, ldh, wr, correction, logits, ids, wts, n_tokens, width, n_out, top, 0, 1, 1, 1, 0, 0.0f, 1.0f,
                                dtype, stream);
}

// --------------------------------------------------------------------------------------------- sort
// One CTA.  ids: [pairs] router outputs; outputs >= n_experts are identity experts and get no row (pos = -1).
// meta[0] = number of tiles.  Rows of one expert are in no particular order; every row is computed by itself.
__global__ void moe_sort_kernel(const int* __restrict__ ids, int pairs, int top, int n_experts, int tm,
                                int* __restrict__ sorted_token, int* __restrict__ pos, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int* __restrict__ tile_rows, int* __restrict__ meta) {
    extern __shared__ int smi[];
    int* count = smi;                   // [n_experts]
    int* cursor = smi + n_experts;      // [n_experts]
    pdl_start();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if ((unsigned)e < (unsigned)n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, nt = 0;
        for (int e = 0; e < n_experts; ++e) {
            cursor[e] = off;
            for (int r0 = 0; r0 < count[e]; r0 += tm) {
                tile_expert[nt] = e;
                tile_row0[nt] = off + r0;
                tile_rows[nt] = min(tm, count[e] - r0);
                ++nt;
            }
            off += count[e];
        }
        meta[0] = nt;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if ((unsigned)e < (unsigned)n_experts) {
            const int dst = atomicAdd(&cursor[e], 1);
            sorted_token[dst] = p / top;
            pos[p] = dst;
        } else {
            pos[p] = -1;
        }
    }
}

VCB_EXPORT int vcb_moe_sort(const int* ids, int pairs, int top, int n_experts, int tm, int* sorted_token, int* pos,
                            int* tile_expert, int* tile_row0, int* tile_rows, int* meta, void* stream) {
    if (pairs <= 0) return 0;
    if (n_experts <= 0 || top <= 0 || tm <= 0 || (size_t)n_experts * 2 * sizeof(int) > 48 * 1024) return VCB_ERR_BAD_ARG;
    vcb_launch(moe_sort_kernel, 1, 1024, (size_t)n_experts * 2 * sizeof(int), (cudaStream_t)stream, ids, pairs, top, n_experts,
               tm, sorted_token, pos, tile_expert, tile_row0, tile_rows, meta);
    return vcb_last_error();
}

// ------------------------------------------------------------------------------------ expert products
// C[row, n] = sum_k A[src(row), k] * W_e[n, k] for the rows of one tile, W_e the tile's expert's matrix.
// GATED: W_e = [gate rows; up rows] ([2 * N, K]), rows are gathered through sorted_token, and C (type T) receives
// the activation of (gate, up).  Otherwise A is the sorted list itself and C is float.
// 64 output columns per CTA, TM rows, 16-deep k slices in shared memory, float accumulation (FMA).
#define MG_N 64
#define MG_K 16

template <typename T, int TM, bool GATED>
__global__ void __launch_bounds__(256)
moe_expert_gemm_kernel(const T* __restrict__ A, long long lda, const T* __restrict__ W, void* __restrict__ Cv, long long ldc,
                       int N, int K, const int* __restrict__ sorted_token, const int* __restrict__ tile_expert,
                       const int* __restrict__ tile_row0, const int* __restrict__ tile_rows, const int* __restrict__ meta,
                       float limit, float alpha, float up_shift) {
    constexpr int RM = TM / 16;          // rows per thread
    __shared__ float As[MG_K][TM + 1];
    __shared__ float Ws[MG_K][MG_N + 1];
    __shared__ float Us[GATED ? MG_K : 1][MG_N + 1];
    __shared__ int src[TM];
    pdl_start();
    const int tile = blockIdx.y;
    if (tile >= meta[0]) return;
    const int e = tile_expert[tile], r0 = tile_row0[tile], rows = tile_rows[tile];
    const int n0 = blockIdx.x * MG_N;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int me = (int)threadIdx.x;
    if (me < TM) src[me] = me < rows ? (GATED ? sorted_token[r0 + me] : r0 + me) : -1;
    __syncthreads();
    const T* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    float acc[RM][4], accu[GATED ? RM : 1][4];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.0f; if (GATED) accu[i][j] = 0.0f; }

    for (int k0 = 0; k0 < K; k0 += MG_K) {
        for (int idx = threadIdx.x; idx < TM * MG_K; idx += 256) {
            const int r = idx / MG_K, kk = idx % MG_K, k = k0 + kk;
            As[kk][r] = (src[r] >= 0 && k < K) ? to_f32<T>(A[(size_t)src[r] * lda + k]) : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = threadIdx.x + q * 256;
            const int r = idx / MG_K, kk = idx % MG_K, k = k0 + kk;
            const bool ok = n0 + r < N && k < K;
            Ws[kk][r] = ok ? to_f32<T>(We[(size_t)(n0 + r) * K + k]) : 0.0f;
            if (GATED) Us[kk][r] = ok ? to_f32<T>(We[(size_t)(N + n0 + r) * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MG_K; ++kk) {
            float av[RM], wv[4], uv[4];
#pragma unroll
            for (int i = 0; i < RM; ++i) av[i] = As[kk][ty * RM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { wv[j] = Ws[kk][tx * 4 + j]; if (GATED) uv[j] = Us[kk][tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < RM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                    if (GATED) accu[i][j] = fmaf(av[i], uv[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int m = ty * RM + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GATED) {
                const float g = fminf(acc[i][j], limit);
                const float u = fminf(fmaxf(accu[i][j], -limit), limit);
                const float y = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + up_shift);
                ((T*)Cv)[(size_t)(r0 + m) * ldc + n] = from_f32<T>(y);
            } else {
                ((float*)Cv)[(size_t)(r0 + m) * ldc + n] = acc[i][j];
            }
        }
    }
}

// The same products for bfloat16 on the tensor cores (mma.sync m16n8k16, float accumulators): a CTA of four warps
// owns TM rows x 64 columns of a tile (and, gated, the 64 up columns beside the 64 gate columns); a ring of three
// 32-deep k slices is filled with cp.async (16-byte pieces; rows beyond the tile and k beyond K arrive as zeros),
// fragments come out of shared memory with ldmatrix (rows padded to 80 bytes: no bank conflicts).  K and the rows'
// strides must be multiples of 8 elements.
#define MM_BN 64
#define MM_BK 32
#define MM_LDS (MM_BK + 8)
#define MM_STAGES 3

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int TM, bool GATED>
__global__ void __launch_bounds__(128)
moe_expert_mma_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ W, void* __restrict__ Cv,
                      long long ldc, int N, int K, const int* __restrict__ sorted_token, const int* __restrict__ tile_expert,
                      const int* __restrict__ tile_row0, const int* __restrict__ tile_rows, const int* __restrict__ meta,
                      float limit, float alpha, float up_shift) {
    constexpr int WR = GATED ? 2 * MM_BN : MM_BN, MF = TM / 16;
    __shared__ __align__(16) __nv_bfloat16 As[MM_STAGES][TM][MM_LDS];
    __shared__ __align__(16) __nv_bfloat16 Ws[MM_STAGES][WR][MM_LDS];
    __shared__ int src[TM];
    pdl_start();
    const int tile = blockIdx.y;
    if (tile >= meta[0]) return;
    const int e = tile_expert[tile], r0 = tile_row0[tile], rows = tile_rows[tile];
    const int n0 = blockIdx.x * MM_BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < TM) src[tid] = tid < rows ? (GATED ? sorted_token[r0 + tid] : r0 + tid) : -1;
    __syncthreads();
    const __nv_bfloat16* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    const int KT = (K + MM_BK - 1) / MM_BK;

    auto load_stage = [&](int kt, int buf) {
        const int k0 = kt * MM_BK;
        for (int idx = tid; idx < TM * 4; idx += 128) {
            const int r = idx >> 2, k = k0 + (idx & 3) * 8;
            const bool ok = src[r] >= 0 && k < K;
            cp_async_16(&As[buf][r][(idx & 3) * 8], ok ? A + (size_t)src[r] * lda + k : A, ok);
        }
        for (int idx = tid; idx < WR * 4; idx += 128) {
            const int r = idx >> 2, k = k0 + (idx & 3) * 8;
            const int n = n0 + (r % MM_BN);
            const bool ok = n < N && k < K;
            const size_t wrow = (size_t)(GATED && r >= MM_BN ? N + n : n);
            cp_async_16(&Ws[buf][r][(idx & 3) * 8], ok ? We + wrow * K + k : We, ok);
        }
    };

    float acc[MF][2][4], accu[GATED ? MF : 1][2][4];
#pragma unroll
    for (int i = 0; i < MF; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) { acc[i][j][c] = 0.0f; if (GATED) accu[i][j][c] = 0.0f; }

#pragma unroll
    for (int st = 0; st < MM_STAGES - 1; ++st) {
        if (st < KT) load_stage(st, st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(MM_STAGES - 2) : "memory");
        __syncthreads();                                  // slice kt has landed for everyone; the slice before has been read
        if (kt + MM_STAGES - 1 < KT) load_stage(kt + MM_STAGES - 1, (kt + MM_STAGES - 1) % MM_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int buf = kt % MM_STAGES;
#pragma unroll
        for (int ks = 0; ks < MM_BK; ks += 16) {
            uint32_t b[4], bu[4];
            ldmatrix_x4(b, &Ws[buf][warp * 16 + (lane & 7) + (lane >> 4) * 8][ks + ((lane >> 3) & 1) * 8]);
            if (GATED) ldmatrix_x4(bu, &Ws[buf][MM_BN + warp * 16 + (lane & 7) + (lane >> 4) * 8][ks + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int mi = 0; mi < MF; ++mi) {
                uint32_t a[4];
                ldmatrix_x4(a, &As[buf][mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][ks + (lane >> 4) * 8]);
                mma_bf16(acc[mi][0], a, b[0], b[1]);
                mma_bf16(acc[mi][1], a, b[2], b[3]);
                if (GATED) {
                    mma_bf16(accu[mi][0], a, bu[0], bu[1]);
                    mma_bf16(accu[mi][1], a, bu[2], bu[3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int mi = 0; mi < MF; ++mi)
#pragma unroll
        for (int nf = 0; nf < 2; ++nf)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int m = mi * 16 + (lane >> 2) + (c >> 1) * 8;
                const int n = n0 + warp * 16 + nf * 8 + (lane & 3) * 2 + (c & 1);
                if (m >= rows || n >= N) continue;
                if (GATED) {
                    const float g = fminf(acc[mi][nf][c], limit);
                    const float u = fminf(fmaxf(accu[mi][nf][c], -limit), limit);
                    const float y = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + up_shift);
                    ((__nv_bfloat16*)Cv)[(size_t)(r0 + m) * ldc + n] = __float2bfloat16_rn(y);
                } else {
                    ((float*)Cv)[(size_t)(r0 + m) * ldc + n] = acc[mi][nf][c];
                }
            }
}

// gated 1: A = the tokens' rows [n, K] (T), W [E, 2 * N, K], C [pairs, N] (T).  gated 0: A [pairs, K] (T), W [E, N, K],
// C [pairs, N] float.  max_tiles: the grid's height; tm: 16 or 64, the tile height moe_sort was given.
VCB_EXPORT int vcb_moe_expert_gemm(const void* A, long long lda, const void* W, void* C, long long ldc, int N, int K,
                                   const int* sorted_token, const int* tile_expert, const int* tile_row0, const int* tile_rows,
                                   const int* meta, int max_tiles, int tm, int gated, float limit, float alpha, float up_shift,
                                   int dtype, void* stream) {
    if (max_tiles <= 0) return 0;
    if (!A || !W || !C || N <= 0 || K <= 0 || (tm != 16 && tm != 64) || max_tiles > 65535) return VCB_ERR_BAD_ARG;
    dim3 grid((N + MG_N - 1) / MG_N, max_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_BF16 && K % 8 == 0 && lda % 8 == 0 && !(((uintptr_t)A | (uintptr_t)W) & 15)) {
        // the tensor-core form
#define MOE_MMA(TMV, G) vcb_launch(moe_expert_mma_kernel<TMV, G>, grid, 128, 0, s, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, C, ldc, N, K, \
                                   sorted_token, tile_expert, tile_row0, tile_rows, meta, limit, alpha, up_shift)
        if (tm == 16) { if (gated) MOE_MMA(16, true); else MOE_MMA(16, false); }
        else { if (gated) MOE_MMA(64, true); else MOE_MMA(64, false); }
#undef MOE_MMA
        return vcb_last_error();
    }
#define MOE_GO(TT, TMV, G) vcb_launch(moe_expert_gemm_kernel<TT, TMV, G>, grid, 256, 0, s, (const TT*)A, lda, (const TT*)W, C, ldc, N, K, \
                                      sorted_token, tile_expert, tile_row0, tile_rows, meta, limit, alpha, up_shift)
    if (dtype == VCB_F32) {
        if (tm == 16) { if (gated) MOE_GO(float, 16, true); else MOE_GO(float, 16, false); }
        else { if (gated) MOE_GO(float, 64, true); else MOE_GO(float, 64, false); }
    } else if (dtype == VCB_BF16) {
        if (tm == 16) { if (gated) MOE_GO(__nv_bfloat16, 16, true); else MOE_GO(__nv_bfloat16, 16, false); }
        else { if (gated) MOE_GO(__nv_bfloat16, 64, true); else MOE_GO(__nv_bfloat16, 64, false); }
    } else return VCB_ERR_BAD_ARG;
#undef MOE_GO
    return vcb_last_error();
}

// ------------------------------------------------------------------------------------------ combine
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ h, long long ldh, const int* __restrict__ pos,
                                   const float* __restrict__ wts, T* __restrict__ out, int width, int top,
                                   const T* __restrict__ add, long long lda) {
    pdl_start();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float acc = add ? to_f32<T>(add[(size_t)t * lda + i]) : 0.0f;      // what every token takes beside its choices (a shared expert)
        for (int k = 0; k < top; ++k) {
            const int p = pos[(size_t)t * top + k];
            const float w = wts[(size_t)t * top + k];
            acc += w * (p >= 0 ? y[(size_t)p * width + i] : to_f32<T>(h[(size_t)t * ldh + i]));
        }
        out[(size_t)t * width + i] = from_f32<T>(acc);
    }
}

VCB_EXPORT int vcb_moe_combine_add(const float* y, const void* h, long long ldh, const int* pos, const float* wts, void* out,
                                   int n_tokens, int width, int top, const void* add, long long lda, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!y || !h || !pos || !wts || !out || width <= 0 || top <= 0) return VCB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == VCB_F32) vcb_launch(moe_combine_kernel<float>, n_tokens, threads, 0, s, y, (const float*)h, ldh, pos, wts, (float*)out, width, top, (const float*)add, lda);
    else if (dtype == VCB_BF16)
        vcb_launch(moe_combine_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, y, (const __nv_bfloat16*)h, ldh, pos, wts,
                   (__nv_bfloat16*)out, width, top, (const __nv_bfloat16*)add, lda);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

VCB_EXPORT int vcb_moe_combine(const float* y, const void* h, long long ldh, const int* pos, const float* wts, void* out,
                               int n_tokens, int width, int top, int dtype, void* stream) {
    return vcb_moe_combine_add(y, h, ldh, pos, wts, out, n_tokens, width, top, nullptr, 0, dtype, stream);
}
