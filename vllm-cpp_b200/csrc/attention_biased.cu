// Paged attention whose scores are capped and carry a learned bias by distance, with keys and values of
// different widths and no rotation:
//
//   qk_norm_cache_write_kernel   RMS norm of a token's whole query projection and of its whole key projection
//                                (all heads at once, one gain per channel), the normed keys and the values into
//                                the token's slot of the cache, the normed queries out
//   attention_biased_kernel      score(i, j) = cap * tanh(scale * (q_i . k_j) / cap) + bias[min(i - j, L - 1), head]
//                                over the keys j <= i (window > 0: i - j < window), softmax, sum of values, and a
//                                sigmoid gate on the result
//
// The cache block of a (page, k|v, kv head) holds `page` rows of `row` elements in the layout of kv_pos
// (common.cuh); keys fill the first dk elements of a row of the key plane, values the first dv of the value
// plane (row = max(dk, dv)).  Norm statistics, scores, the cap, the bias, softmax and the sums are float.
// One warp per (token, head), a key per lane: the plain form, for both storage types.  The reference's
// attention (src/attention/paged_attention.cu) has no cap, no bias and no gate.
#include "common.cuh"

struct QkNormArgs {
    const void* proj;           // [n, ...] rows that hold the token's q, k and v projections
    long long ld;
    int q_off, k_off, v_off;    // first element of each inside a row
    const float* wq;            // [H * dk] gain of the query norm (null: queries are not normed)
    const float* wk;            // [G * dk]
    void* q_out;                // [n, H * dk]
    void* cache;
    const int* positions;
    const int* req_of_token;
    const int* block_table;
    int bt_stride, H, G, dk, dv, row, page, num_pages, write_kv;
    float eps;
    int* status;
};

template <typename T>
__global__ void qk_norm_cache_write_kernel(QkNormArgs a) {
    __shared__ float scratch[33];
    pdl_start();
    const int t = blockIdx.x;
    const T* src = (const T*)a.proj + (size_t)t * a.ld;
    const int nq = a.H * a.dk, nk = a.G * a.dk, nv = a.G * a.dv;
    float rq = 1.0f, rk = 1.0f;
    if (a.wq) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float x = to_f32<T>(src[a.q_off + i]); ss += x * x; }
        rq = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nq + a.eps);
    }
    if (a.wk) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float x = to_f32<T>(src[a.k_off + i]); ss += x * x; }
        rk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nk + a.eps);
    }
    T* qo = (T*)a.q_out + (size_t)t * nq;
    for (int i = threadIdx.x; i < nq; i += blockDim.x)
        qo[i] = from_f32<T>(to_f32<T>(src[a.q_off + i]) * rq * (a.wq ? a.wq[i] : 1.0f));
    if (!a.write_kv) return;
    const int pos = a.positions[t];
    const int lp = pos / a.page, slot = pos - lp * a.page;
    const int pg = lp < a.bt_stride ? a.block_table[(size_t)a.req_of_token[t] * a.bt_stride + lp] : -1;
    if ((unsigned)pg >= (unsigned)a.num_pages) {
        if (a.status && threadIdx.x == 0) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
        return;
    }
    const size_t block = (size_t)a.page * a.row;
    T* kp = (T*)a.cache + (size_t)pg * 2 * a.G * block;
    T* vp = kp + (size_t)a.G * block;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int g = i / a.dk, c = i - g * a.dk;
        kp[g * block + kv_pos(c, slot, a.row, a.page, (int)sizeof(T))] =
            from_f32<T>(to_f32<T>(src[a.k_off + i]) * rk * (a.wk ? a.wk[i] : 1.0f));
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int g = i / a.dv, c = i - g * a.dv;
        vp[g * block + kv_pos(c, slot, a.row, a.page, (int)sizeof(T))] = src[a.v_off + i];
    }
}

// The same for bfloat16 with every size, offset and stride a multiple of 8 elements: 16-byte accesses (a 16-byte piece
// of a row stays whole in the cache's layout).
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(p[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
}

__global__ void qk_norm_cache_write_bf16x8_kernel(QkNormArgs a) {
    pdl_start();
    const int t = blockIdx.x;
    const __nv_bfloat16* src = (const __nv_bfloat16*)a.proj + (size_t)t * a.ld;
    const int nq8 = a.H * a.dk / 8, nk8 = a.G * a.dk / 8, nv8 = a.G * a.dv / 8;
    const uint4* qsrc = reinterpret_cast<const uint4*>(src + a.q_off);
    const uint4* ksrc = reinterpret_cast<const uint4*>(src + a.k_off);
    const uint4* vsrc = reinterpret_cast<const uint4*>(src + a.v_off);
    // both sums of squares in one pass and one reduction: the queries' in the low lanes' share, the keys' beside it
    float sq = 0.0f, sk = 0.0f;
    // a thread's first four pieces of the query row stay in registers for the second pass
    constexpr int KEEP = 4;
    uint4 kept[KEEP];
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        kept[j] = c < nq8 ? qsrc[c] : make_uint4(0, 0, 0, 0);
        if (a.wq) {
            float f[8];
            unpack8(kept[j], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += f[e] * f[e];
        }
    }
    if (a.wq)
        for (int c = threadIdx.x + KEEP * blockDim.x; c < nq8; c += blockDim.x) {
            float f[8];
            unpack8(qsrc[c], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += f[e] * f[e];
        }
    if (a.wk)
        for (int c = threadIdx.x; c < nk8; c += blockDim.x) {
            float f[8];
            unpack8(ksrc[c], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sk += f[e] * f[e];
        }
    __shared__ float both[2][33];
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { both[0][warp] = sq; both[1][warp] = sk; }
        __syncthreads();
        if (warp == 0) {
            const float tq = warp_sum(lane < nwarps ? both[0][lane] : 0.0f), tk = warp_sum(lane < nwarps ? both[1][lane] : 0.0f);
            if (lane == 0) { both[0][32] = tq; both[1][32] = tk; }
        }
        __syncthreads();
    }
    const float rq = a.wq ? 1.0f / sqrtf(both[0][32] / (float)(nq8 * 8) + a.eps) : 1.0f;
    const float rk = a.wk ? 1.0f / sqrtf(both[1][32] / (float)(nk8 * 8) + a.eps) : 1.0f;
    auto normed = [](const uint4& raw, float r, const float* w) {
        float f[8];
        unpack8(raw, f);
        uint4 out;
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&out);
        if (w) {
            const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
            const float g[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) p[e] = __floats2bfloat162_rn(f[2 * e] * r * g[2 * e], f[2 * e + 1] * r * g[2 * e + 1]);
        } else {
            out = raw;
        }
        return out;
    };
    uint4* qo = reinterpret_cast<uint4*>((__nv_bfloat16*)a.q_out + (size_t)t * nq8 * 8);
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nq8) qo[c] = normed(kept[j], rq, a.wq ? a.wq + c * 8 : nullptr);
    }
    for (int c = threadIdx.x + KEEP * blockDim.x; c < nq8; c += blockDim.x) qo[c] = normed(qsrc[c], rq, a.wq ? a.wq + c * 8 : nullptr);
    if (!a.write_kv) return;
    const int pos = a.positions[t];
    const int lp = pos / a.page, slot = pos - lp * a.page;
    const int pg = lp < a.bt_stride ? a.block_table[(size_t)a.req_of_token[t] * a.bt_stride + lp] : -1;
    if ((unsigned)pg >= (unsigned)a.num_pages) {
        if (a.status && threadIdx.x == 0) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
        return;
    }
    const size_t block = (size_t)a.page * a.row;
    __nv_bfloat16* kp = (__nv_bfloat16*)a.cache + (size_t)pg * 2 * a.G * block;
    __nv_bfloat16* vp = kp + (size_t)a.G * block;
    for (int c = threadIdx.x; c < nk8; c += blockDim.x) {
        const int i = c * 8, g = i / a.dk, e = i - g * a.dk;
        *reinterpret_cast<uint4*>(kp + g * block + kv_pos(e, slot, a.row, a.page, 2)) = normed(ksrc[c], rk, a.wk ? a.wk + i : nullptr);
    }
    for (int c = threadIdx.x; c < nv8; c += blockDim.x) {
        const int i = c * 8, g = i / a.dv, e = i - g * a.dv;
        *reinterpret_cast<uint4*>(vp + g * block + kv_pos(e, slot, a.row, a.page, 2)) = vsrc[c];
    }
}

VCB_EXPORT int vcb_qk_norm_cache_write(const void* proj, long long ld, int q_off, int k_off, int v_off, const float* wq,
                                       const float* wk, void* q_out, void* cache, const int* positions,
                                       const int* req_of_token, const int* block_table, int bt_stride, int n_tokens,
                                       int H, int G, int dk, int dv, int row, int page, int num_pages, int write_kv,
                                       float eps, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!proj || !q_out || !cache || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || row < dk || row < dv || page <= 0)
        return VCB_ERR_BAD_ARG;
    QkNormArgs a{proj, ld, q_off, k_off, v_off, wq, wk, q_out, cache, positions, req_of_token, block_table, bt_stride,
                 H, G, dk, dv, row, page, num_pages, write_kv, eps, status};
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H * dk >= 2048 ? 512 : 256;
    const uintptr_t addrs = (uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)wq | (uintptr_t)wk;
    if (dtype == VCB_BF16 && !((dk | dv | row | q_off | k_off | v_off) & 7) && !(ld & 7) && !(addrs & 15)) {
        const int chunks = H * dk / 8;
        vcb_launch(qk_norm_cache_write_bf16x8_kernel, n_tokens, chunks >= 512 ? 256 : 128, 0, s, a);
        return vcb_last_error();
    }
    if (dtype == VCB_F32) vcb_launch(qk_norm_cache_write_kernel<float>, n_tokens, threads, 0, s, a);
    else if (dtype == VCB_BF16) vcb_launch(qk_norm_cache_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------- norm per head, rotation, cache write
// Queries and keys RMS-normed head by head over dk with one gain vector that all heads share (wq, wk: float [dk] or
// null), then rotated on their first `rot` coordinates: coordinate i pairs with i + rot / 2, angle = position *
// inv_freq[i] in float.  Keys and values go into the token's slot of the cache, queries to q_out.  A warp per head.
struct QkHeadArgs {
    QkNormArgs base;
    const float* inv_freq;      // [rot / 2] or null
    int rot;
};

template <typename T>
__global__ void qk_head_rope_cache_write_kernel(QkHeadArgs h) {
    const QkNormArgs& a = h.base;
    pdl_start();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const T* src = (const T*)a.proj + (size_t)t * a.ld;
    const int pos = a.positions[t];
    const int half = h.rot >> 1;
    T* kp = nullptr;
    T* vp = nullptr;
    const size_t block = (size_t)a.page * a.row;
    int slot = 0;
    if (a.write_kv) {
        const int lp = pos / a.page;
        slot = pos - lp * a.page;
        const int pg = lp < a.bt_stride ? a.block_table[(size_t)a.req_of_token[t] * a.bt_stride + lp] : -1;
        if ((unsigned)pg >= (unsigned)a.num_pages) {
            if (a.status && threadIdx.x == 0) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
        } else {
            kp = (T*)a.cache + (size_t)pg * 2 * a.G * block;
            vp = kp + (size_t)a.G * block;
        }
    }
    // the angles depend on the position and the pair only: a lane keeps cosine and sine of its pairs for all the heads
    // its warp takes (pairs lane, lane + 32, ...; beyond ROPE_KEPT * 32 pairs they are made where they are used)
    constexpr int ROPE_KEPT = 4;
    float cs[ROPE_KEPT], sn[ROPE_KEPT];
#pragma unroll
    for (int k = 0; k < ROPE_KEPT; ++k) {
        const int j = lane + 32 * k;
        cs[k] = 1.0f;
        sn[k] = 0.0f;
        if (j < half) sincosf((float)pos * h.inv_freq[j], &sn[k], &cs[k]);
    }
    for (int head = warp; head < a.H + a.G; head += nwarps) {
        const bool is_q = head < a.H;
        const int g = is_q ? head : head - a.H;
        const T* x = src + (is_q ? a.q_off + g * a.dk : a.k_off + g * a.dk);
        const float* w = is_q ? a.wq : a.wk;
        float r = 1.0f;
        if (w) {
            float ss = 0.0f;
            for (int i = lane; i < a.dk; i += 32) { const float v = to_f32<T>(x[i]); ss = fmaf(v, v, ss); }
            r = 1.0f / sqrtf(warp_sum(ss) / (float)a.dk + a.eps);
        }
        if (!is_q && !kp) continue;
        T* qo = (T*)a.q_out + (size_t)t * a.H * a.dk + (size_t)g * a.dk;
        T* ko = is_q ? nullptr : kp + (size_t)g * block;
        auto put = [&](int i, float v) {
            if (is_q) qo[i] = from_f32<T>(v);
            else ko[kv_pos(i, slot, a.row, a.page, (int)sizeof(T))] = from_f32<T>(v);
        };
        // a pair (j, j + half) at a time, then the coordinates that no rotation turns
#pragma unroll
        for (int k = 0; k < ROPE_KEPT; ++k) {
            const int j = lane + 32 * k;
            if (j < half) {
                const float u = to_f32<T>(x[j]) * r * (w ? w[j] : 1.0f), v = to_f32<T>(x[j + half]) * r * (w ? w[j + half] : 1.0f);
                put(j, u * cs[k] - v * sn[k]);
                put(j + half, v * cs[k] + u * sn[k]);
            }
        }
        for (int j = lane + 32 * ROPE_KEPT; j < half; j += 32) {
            float s1, c1;
            sincosf((float)pos * h.inv_freq[j], &s1, &c1);
            const float u = to_f32<T>(x[j]) * r * (w ? w[j] : 1.0f), v = to_f32<T>(x[j + half]) * r * (w ? w[j + half] : 1.0f);
            put(j, u * c1 - v * s1);
            put(j + half, v * c1 + u * s1);
        }
        for (int i = h.rot + lane; i < a.dk; i += 32) put(i, to_f32<T>(x[i]) * r * (w ? w[i] : 1.0f));
    }
    if (!vp) return;
    const int nv = a.G * a.dv;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int g = i / a.dv, c = i - g * a.dv;
        vp[g * block + kv_pos(c, slot, a.row, a.page, (int)sizeof(T))] = src[a.v_off + i];
    }
}

VCB_EXPORT int vcb_qk_head_rope_cache_write(const void* proj, long long ld, int q_off, int k_off, int v_off, const float* wq,
                                            const float* wk, const float* inv_freq, int rot, void* q_out, void* cache,
                                            const int* positions, const int* req_of_token, const int* block_table,
                                            int bt_stride, int n_tokens, int H, int G, int dk, int dv, int row, int page,
                                            int num_pages, int write_kv, float eps, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!proj || !q_out || !cache || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || row < dk || row < dv || page <= 0 || rot < 0 ||
        rot > dk || (rot & 1) || (rot && !inv_freq))
        return VCB_ERR_BAD_ARG;
    QkHeadArgs a{{proj, ld, q_off, k_off, v_off, wq, wk, q_out, cache, positions, req_of_token, block_table, bt_stride,
                  H, G, dk, dv, row, page, num_pages, write_kv, eps, status}, inv_freq, rot};
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = (H + G) >= 8 ? 256 : 128;
    if (dtype == VCB_F32) vcb_launch(qk_head_rope_cache_write_kernel<float>, n_tokens, threads, 0, s, a);
    else if (dtype == VCB_BF16) vcb_launch(qk_head_rope_cache_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ---------------------------------------------------------------------------------------- attention
#define ATB_MAX_DV 256
#define ATB_WARPS 4

struct BiasedAttnArgs {
    const void* q;              // [n, nh * dk]
    const void* cache;
    void* out;                  // [n, nh * dv]
    const void* gate;           // [n, nh * dv] with row stride ldg, or null: out *= sigmoid(gate)
    long long ldg;
    const int* positions;
    const int* req_of_token;
    const int* block_table;
    const float* bias;          // [bias_len, nh] by distance, or null
    int bias_len;
    int bt_stride, n_tokens, nh, nkv, dk, dv, row, page, window;
    float scale, cap;           // cap <= 0: scores are not capped
    int num_pages;
    int* status;
    const float* sink;          // [nh] or null: a logit per head that joins the softmax's denominator and has no value
    int gate_per_head;          // 1: the gate holds one number per head ([n, nh]) instead of one per channel
};

template <typename T>
__global__ void attention_biased_kernel(BiasedAttnArgs a) {
    extern __shared__ float qs_all[];
    pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * ATB_WARPS + warp;
    if (item >= (long long)a.n_tokens * a.nh) return;
    const int t = (int)(item / a.nh), h = (int)(item % a.nh);
    const int g = h / (a.nh / a.nkv);
    const int pos = a.positions[t];
    const int* bt = a.block_table + (size_t)a.req_of_token[t] * a.bt_stride;
    float* qs = qs_all + warp * a.dk;
    const T* qrow = (const T*)a.q + ((size_t)t * a.nh + h) * a.dk;
    for (int i = lane; i < a.dk; i += 32) qs[i] = to_f32<T>(qrow[i]);
    __syncwarp();

    const size_t block = (size_t)a.page * a.row;
    const size_t page_elems = 2 * (size_t)a.nkv * block, v_off = (size_t)a.nkv * block;
    const T* cache = (const T*)a.cache;
    const float inv_cap = a.cap > 0.0f ? 1.0f / a.cap : 0.0f;

    float o[ATB_MAX_DV / 32];
#pragma unroll
    for (int k = 0; k < ATB_MAX_DV / 32; ++k) o[k] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const int kstart = a.window > 0 ? max(0, pos - a.window + 1) : 0;

    for (int kb = kstart; kb <= pos; kb += 32) {
        const int j = kb + lane;
        bool valid = j <= pos;
        float s = -INFINITY;
        unsigned long long koff = 0;
        if (valid) {
            const int lp = j / a.page;
            const int pg = lp < a.bt_stride ? bt[lp] : -1;
            if ((unsigned)pg >= (unsigned)a.num_pages) {
                if (a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
                valid = false;
            } else {
                koff = (unsigned long long)pg * page_elems + (size_t)g * block;
            }
        }
        if (valid) {
            const T* kr = cache + koff;
            const int slot = j % a.page;
            float acc = 0.0f;
            for (int i = 0; i < a.dk; ++i) acc += qs[i] * to_f32<T>(kr[kv_pos(i, slot, a.row, a.page, (int)sizeof(T))]);
            s = acc * a.scale;
            if (a.cap > 0.0f) s = a.cap * tanhf(s * inv_cap);
            if (a.bias) s += a.bias[(size_t)min(pos - j, a.bias_len - 1) * a.nh + h];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int k = 0; k < ATB_MAX_DV / 32; ++k) o[k] *= corr;
        const int nvalid = min(32, pos - kb + 1);
        for (int jj = 0; jj < nvalid; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long off = __shfl_sync(0xffffffffu, koff, jj);
            const T* vr = cache + off + v_off;
            const int slot = (kb + jj) % a.page;
#pragma unroll
            for (int k = 0; k < ATB_MAX_DV / 32; ++k) {
                const int dim = lane + 32 * k;
                if (dim < a.dv) o[k] += pj * to_f32<T>(vr[kv_pos(dim, slot, a.row, a.page, (int)sizeof(T))]);
            }
        }
        m = m_new;
    }
    T* orow = (T*)a.out + ((size_t)t * a.nh + h) * a.dv;
    const T* grow = a.gate ? (const T*)a.gate + (size_t)t * a.ldg + (a.gate_per_head ? (size_t)h : (size_t)h * a.dv) : nullptr;
    float keep = 1.0f;
    if (a.sink) {
        // the sink counts once in the denominator, unscaled; the reference of the exponents moves if it is the largest
        const float sk = a.sink[h], mf = fmaxf(m, sk);
        keep = expf(m - mf);
        l = l * keep + expf(sk - mf);
    }
    const float inv = keep / l;
    const float head_gate = (grow && a.gate_per_head) ? 1.0f / (1.0f + expf(-to_f32<T>(grow[0]))) : 1.0f;
#pragma unroll
    for (int k = 0; k < ATB_MAX_DV / 32; ++k) {
        const int dim = lane + 32 * k;
        if (dim < a.dv) {
            float y = o[k] * inv * head_gate;
            if (grow && !a.gate_per_head) y *= 1.0f / (1.0f + expf(-to_f32<T>(grow[dim])));
            orow[dim] = from_f32<T>(y);
        }
    }
}

VCB_EXPORT int vcb_attention_biased(const void* q, const void* cache, void* out, const void* gate, long long ldg,
                                    const int* positions, const int* req_of_token, const int* block_table, int bt_stride,
                                    const float* bias, int bias_len, int n_tokens, int nh, int nkv, int dk, int dv, int row,
                                    int page, int window, float scale, float cap, int num_pages, int* status,
                                    const float* sink, int gate_per_head, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (dk <= 0 || dv <= 0 || dv > ATB_MAX_DV || dk > 1024 || row < dk || row < dv || nh <= 0 || nkv <= 0 || nh % nkv ||
        page <= 0 || window < 0 || num_pages < 0 || (bias && bias_len <= 0))
        return VCB_ERR_BAD_ARG;
    BiasedAttnArgs a{q, cache, out, gate, ldg, positions, req_of_token, block_table, bias, bias_len, bt_stride, n_tokens,
                     nh, nkv, dk, dv, row, page, window, scale, cap, num_pages, status, sink, gate_per_head};
    const long long items = (long long)n_tokens * nh;
    const int blocks = (int)((items + ATB_WARPS - 1) / ATB_WARPS);
    const size_t smem = (size_t)ATB_WARPS * dk * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) vcb_launch(attention_biased_kernel<float>, blocks, ATB_WARPS * 32, smem, s, a);
    else if (dtype == VCB_BF16) vcb_launch(attention_biased_kernel<__nv_bfloat16>, blocks, ATB_WARPS * 32, smem, s, a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
