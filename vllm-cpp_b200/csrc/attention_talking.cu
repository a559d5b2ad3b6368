// Paged attention whose heads talk to one another before the softmax: the scaled scores of all H heads at a
// (query, key) pair, each less a bias that grows with the distance, are mixed by an H x H matrix, and every head
// takes its softmax over the mixed scores:
//
//   raw_g(i, j)  = scale * (q_i,g . k_j,kv(g)) - slope[g] * (i - j)              kv(g) = g / (H / G)
//   s_h(i, j)    = sum_g mix[h, g] * raw_g(i, j)                                   over the keys j <= i (window > 0: i - j < window)
//   out_i,h      = sum_j softmax_j(s_h(i, .)) v_j,kv(h),   times sigmoid(gate) when a gate is given
//
// The cache block of a (page, k|v, kv head) holds `page` rows of `row` elements in the layout of kv_pos (common.cuh).
// Scores, bias, mixing, softmax and the sums are float for both storage types.
//
//   attention_talking_kernel        the plain form: a CTA per token, a warp per head, a key per lane; the heads' raw
//                                   scores of 32 keys meet in shared memory, where every warp mixes its own row
//   attention_talking_mma_kernel    bfloat16 heads of 64 or 128 on tensor cores (mma.sync m16n8k16, float accumulation):
//                                   a CTA per work item (16 query rows of a request and a run of its keys), a warp per
//                                   head; per tile of 32 keys every warp takes its head's 16 x 32 raw scores, leaves them
//                                   in shared memory, mixes its own row of the heads' matrix from there in float, runs the
//                                   online softmax on its fragments and multiplies the weights, as two bfloat16 terms
//                                   (16 bits of mantissa), with the value tile.  A work item that holds only part of its
//                                   rows' keys leaves (o, m, l) partials; attention_talking_merge_rows_kernel joins them.
//   attention_talking_decode_kernel the same for requests that bring one token: the fragment's rows are the heads of a kv
//                                   head's group, a warp per (kv head, sixteen keys of a tile); the runs of a request's
//                                   keys leave partials that attention_talking_merge_kernel joins.
//
// The reference's attention (src/attention/paged_attention.cu) has independent heads.
#include "common.cuh"

#define ATT_MAX_DV 256
#define ATT_MAX_HEADS 32

struct TalkingAttnArgs {
    const void* q;              // [n, H * dk]
    const void* cache;
    void* out;                  // [n, H * dv]
    const void* gate;           // [n, H * dv] rows ldg apart, or null: out *= sigmoid(gate)
    long long ldg;
    const int* positions;
    const int* req_of_token;
    const int* block_table;
    const float* mix;           // [H, H] row h: the weights of head h's mixed score
    const float* slope;         // [H] or null
    int bt_stride, n_tokens, H, G, dk, dv, row, page, window;
    float scale;
    int num_pages;
    int* status;
};

template <typename T>
__global__ void attention_talking_kernel(TalkingAttnArgs a) {
    extern __shared__ float sm[];
    float* qs = sm;                                 // [H][dk]
    float* raw = qs + (size_t)a.H * a.dk;           // [H][32]
    float* mixs = raw + a.H * 32;                   // [H][H]
    pdl_start();
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int g = h / (a.H / a.G);
    const int pos = a.positions[t];
    const int* bt = a.block_table + (size_t)a.req_of_token[t] * a.bt_stride;
    const T* qrow = (const T*)a.q + (size_t)t * a.H * a.dk;
    for (int i = threadIdx.x; i < a.H * a.dk; i += blockDim.x) qs[i] = to_f32<T>(qrow[i]);
    for (int i = threadIdx.x; i < a.H * a.H; i += blockDim.x) mixs[i] = a.mix[i];
    __syncthreads();
    const float* qh = qs + (size_t)h * a.dk;
    const float slope = a.slope ? a.slope[h] : 0.0f;

    const size_t block = (size_t)a.page * a.row;
    const size_t page_elems = 2 * (size_t)a.G * block, v_off = (size_t)a.G * block;
    const T* cache = (const T*)a.cache;

    float o[ATT_MAX_DV / 32];
#pragma unroll
    for (int k = 0; k < ATT_MAX_DV / 32; ++k) o[k] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const int kstart = a.window > 0 ? max(0, pos - a.window + 1) : 0;

    for (int kb = kstart; kb <= pos; kb += 32) {
        const int j = kb + lane;
        bool valid = j <= pos;
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
        float r = 0.0f;                             // a key that is not seen contributes nothing to any head's mix
        if (valid) {
            const T* kr = cache + koff;
            const int slot = j % a.page;
            float acc = 0.0f;
            for (int i = 0; i < a.dk; ++i) acc = fmaf(qh[i], to_f32<T>(kr[kv_pos(i, slot, a.row, a.page, (int)sizeof(T))]), acc);
            r = acc * a.scale - slope * (float)(pos - j);
        }
        raw[h * 32 + lane] = r;
        __syncthreads();
        float s = -INFINITY;
        if (valid) {
            s = 0.0f;
            for (int gg = 0; gg < a.H; ++gg) s = fmaf(mixs[h * a.H + gg], raw[gg * 32 + lane], s);
        }
        __syncthreads();                            // raw is written again in the next round
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = m_new == -INFINITY ? 1.0f : expf(m - m_new);
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int k = 0; k < ATT_MAX_DV / 32; ++k) o[k] *= corr;
        const int nvalid = min(32, pos - kb + 1);
        for (int jj = 0; jj < nvalid; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long off = __shfl_sync(0xffffffffu, koff, jj);
            if (pj == 0.0f) continue;               // also the keys whose page was refused
            const T* vr = cache + off + v_off;
            const int slot = (kb + jj) % a.page;
#pragma unroll
            for (int k = 0; k < ATT_MAX_DV / 32; ++k) {
                const int dim = lane + 32 * k;
                if (dim < a.dv) o[k] = fmaf(pj, to_f32<T>(vr[kv_pos(dim, slot, a.row, a.page, (int)sizeof(T))]), o[k]);
            }
        }
        m = m_new;
    }
    T* orow = (T*)a.out + ((size_t)t * a.H + h) * a.dv;
    const T* grow = a.gate ? (const T*)a.gate + (size_t)t * a.ldg + (size_t)h * a.dv : nullptr;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int k = 0; k < ATT_MAX_DV / 32; ++k) {
        const int dim = lane + 32 * k;
        if (dim < a.dv) {
            float y = o[k] * inv;
            if (grow) y *= 1.0f / (1.0f + expf(-to_f32<T>(grow[dim])));
            orow[dim] = from_f32<T>(y);
        }
    }
}

VCB_EXPORT int vcb_attention_talking(const void* q, const void* cache, void* out, const void* gate, long long ldg,
                                     const int* positions, const int* req_of_token, const int* block_table, int bt_stride,
                                     const float* mix, const float* slope, int n_tokens, int H, int G, int dk, int dv, int row,
                                     int page, int window, float scale, int num_pages, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!q || !cache || !out || !mix || dk <= 0 || dv <= 0 || dv > ATT_MAX_DV || dk > 1024 || row < dk || row < dv || H <= 0 ||
        G <= 0 || H % G || page <= 0 || window < 0 || num_pages < 0)
        return VCB_ERR_BAD_ARG;
    if (H > ATT_MAX_HEADS) return VCB_ERR_UNSUPPORTED;
    TalkingAttnArgs a{q, cache, out, gate, ldg, positions, req_of_token, block_table, mix, slope, bt_stride, n_tokens, H, G, dk, dv,
                      row, page, window, scale, num_pages, status};
    const size_t smem = ((size_t)H * dk + (size_t)H * 32 + (size_t)H * H) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    static unsigned long long done_f = 0, done_b = 0;
    if (dtype == VCB_F32) {
        if (smem > 48 * 1024) { const int e = vcb_allow_dynamic_smem(attention_talking_kernel<float>, (int)smem, &done_f); if (e) return e; }
        vcb_launch(attention_talking_kernel<float>, n_tokens, H * 32, smem, s, a);
    } else if (dtype == VCB_BF16) {
        if (smem > 48 * 1024) { const int e = vcb_allow_dynamic_smem(attention_talking_kernel<__nv_bfloat16>, (int)smem, &done_b); if (e) return e; }
        vcb_launch(attention_talking_kernel<__nv_bfloat16>, n_tokens, H * 32, smem, s, a);
    } else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------------ tensor cores (bfloat16, heads of 64 or 128)
#define TKM_ROWS 16            // query rows of a work item
#define TKM_KEYS 32            // keys of a tile
#define TKM_MAX_HEADS 16       // a warp per head, and a head's fragments want more registers than 1024 threads leave
#define TKM_MAX_PARTS 8        // most items a portion's tile is cut into along its keys
#define TKM_ITEM_INTS 6        // request, first row within the request's rows of this step, rows, first key, end of keys, partial slot or -1

struct TalkingMmaArgs {
    const __nv_bfloat16* q;     // [n, H * D]
    const __nv_bfloat16* cache;
    __nv_bfloat16* out;         // [n, H * D]
    const __nv_bfloat16* gate;  // [n, H * D] rows ldg apart, or null
    long long ldg;
    const int* items;           // [n_items, TKM_ITEM_INTS]
    const int* q_start;         // [n_reqs + 1] first row of each request in this step
    const int* ctx_lens;        // [n_reqs] keys in the cache before this step
    const int* block_table;
    const float* mix;           // [H, H]
    const float* slope;         // [H] or null
    float* part_o;              // [slots, H, TKM_ROWS... see below] partial sums of a split item: [slot][h][D]
    float* part_ml;             // [slot][h][2]
    int bt_stride, H, G, page, window, num_pages;
    float scale;
    int* status;
    int page_shift;             // log2(page) when the page size is a power of two, else -1
    int wide;                   // 1: an item's partial sums are kept for all its 16 rows, [slot][head][row][D] (portions cut along the keys)
};

__device__ __forceinline__ uint32_t tkm_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void tkm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t tkm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Two weights (not negative) as two pairs of bfloat16: hi is the upper half of each float (cut off, so that what is left
// is exact), lo the rounding of what is left: hi + lo carries 16 bits of the weight's mantissa.
__device__ __forceinline__ void tkm_two_terms(float x, float y, uint32_t& hi, uint32_t& lo) {
    const uint32_t bx = __float_as_uint(x), by = __float_as_uint(y);
    hi = __byte_perm(bx, by, 0x7632);
    lo = tkm_pack(x - __uint_as_float(bx & 0xffff0000u), y - __uint_as_float(by & 0xffff0000u));
}

__device__ __forceinline__ float tkm_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int MAXT>
__global__ void __launch_bounds__(MAXT) attention_talking_mma_kernel(TalkingMmaArgs a) {
    constexpr int LDK = D + 8;                      // bfloat16 elements between two keys of a tile in shared memory
    extern __shared__ __align__(16) unsigned char tkm_smem[];
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(tkm_smem);                 // [2][G][TKM_KEYS][LDK] normed keys, two stages
    __nv_bfloat16* vs = ks + 2 * (size_t)a.G * TKM_KEYS * LDK;                      // [2][G][TKM_KEYS][LDK] values
    float* raw0 = reinterpret_cast<float*>(vs + 2 * (size_t)a.G * TKM_KEYS * LDK); // [2][H][key octet][lane] float4, taking turns
    float* mixs = raw0 + 2 * (size_t)a.H * TKM_ROWS * TKM_KEYS;                     // [H][H]
    pdl_start();
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gr = lane >> 2, tq = lane & 3;        // fragment row (and row + 8) and column pair of this lane
    const int* item = a.items + (size_t)blockIdx.x * TKM_ITEM_INTS;
    const int req = item[0], q0 = item[1], nq = item[2], k_lo = item[3], k_hi = item[4], slot_out = item[5];
    const int g = h / (a.H / a.G);
    const int row0 = a.q_start[req] + q0;           // first row of the item among the step's tokens
    const int pos0 = a.ctx_lens[req] + q0;          // its position in the request
    const int* bt = a.block_table + (size_t)req * a.bt_stride;
    for (int i = threadIdx.x; i < a.H * a.H; i += blockDim.x) mixs[i] = a.mix[i];
    const float slope = a.slope ? a.slope[h] : 0.0f;

    // the head's queries as A fragments: rows gr and gr + 8, D / 16 steps of 16 coordinates
    uint32_t qf[D / 16][4];
    {
        const __nv_bfloat16* qa = a.q + ((size_t)(row0 + gr) * a.H + h) * D + tq * 2;
        const __nv_bfloat16* qb = qa + (size_t)8 * a.H * D;
        const bool ra = gr < nq, rb = gr + 8 < nq;
#pragma unroll
        for (int s = 0; s < D / 16; ++s) {
            qf[s][0] = ra ? *reinterpret_cast<const uint32_t*>(qa + s * 16) : 0u;
            qf[s][1] = rb ? *reinterpret_cast<const uint32_t*>(qb + s * 16) : 0u;
            qf[s][2] = ra ? *reinterpret_cast<const uint32_t*>(qa + s * 16 + 8) : 0u;
            qf[s][3] = rb ? *reinterpret_cast<const uint32_t*>(qb + s * 16 + 8) : 0u;
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;     // rows gr and gr + 8
    const int pos_a = pos0 + gr, pos_b = pos0 + gr + 8;
    const bool row_a = gr < nq, row_b = gr + 8 < nq;

    const size_t block = (size_t)a.page * D;
    const size_t page_elems = 2 * (size_t)a.G * block;
    constexpr int CH = D / 8;                       // 16-byte chunks of a key
    constexpr int PER = CH / 4;                     // chunks a thread copies of a key: four threads share one
    const size_t stage_elems = (size_t)a.G * TKM_KEYS * LDK;
    const int n_pairs = a.G * TKM_KEYS;
    // a tile's keys and values of every kv head, out of their pages into rows of LDK elements of stage `st`: asynchronous
    // 16-byte copies, a page looked up once per (kv head, key) by the four threads that share the key
    auto fetch = [&](int st, int k0) {
        __nv_bfloat16* kd = ks + (size_t)st * stage_elems;
        __nv_bfloat16* vd = vs + (size_t)st * stage_elems;
        for (int p = threadIdx.x >> 2; p < n_pairs; p += blockDim.x >> 2) {
            const int gk = p / TKM_KEYS, key = p - gk * TKM_KEYS, j = k0 + key, sub = threadIdx.x & 3;
            const __nv_bfloat16* src = a.cache;
            uint32_t bytes = 0;
            int sl = 0;
            if (j < k_hi) {
                const int lp = a.page_shift >= 0 ? j >> a.page_shift : j / a.page;
                sl = j - lp * a.page;
                const int pg = lp < a.bt_stride ? bt[lp] : -1;
                if ((unsigned)pg >= (unsigned)a.num_pages) {
                    if (a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
                } else {
                    src = a.cache + (size_t)pg * page_elems + (size_t)gk * block;
                    bytes = 16;
                }
            }
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const int ch = sub * PER + e;
                const __nv_bfloat16* from = bytes ? src + kv_pos(ch * 8, sl, D, a.page, 2) : a.cache;
                const uint32_t to_k = cx_smem(kd + ((size_t)gk * TKM_KEYS + key) * LDK + ch * 8);
                const uint32_t to_v = cx_smem(vd + ((size_t)gk * TKM_KEYS + key) * LDK + ch * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(to_k), "l"(from), "r"(bytes) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(to_v), "l"(bytes ? from + (size_t)a.G * block : from), "r"(bytes)
                             : "memory");
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    float off[TKM_KEYS / 4];                        // slope * (a key's offset from this lane's first key of the tile)
#pragma unroll
    for (int n = 0; n < TKM_KEYS / 8; ++n) {
        off[2 * n] = slope * (float)(n * 8);
        off[2 * n + 1] = slope * (float)(n * 8 + 1);
    }
    if (k_lo < k_hi) fetch(0, k_lo);
    int it = 0;
    for (int k0 = k_lo; k0 < k_hi; k0 += TKM_KEYS, ++it) {
        const int st = it & 1;
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();                            // the tile has arrived; the round before is over for every warp (and mixs is in place)
        if (k0 + TKM_KEYS < k_hi) fetch(st ^ 1, k0 + TKM_KEYS);        // the next tile travels while this one is worked on
        const __nv_bfloat16* kst = ks + (size_t)st * stage_elems;
        const __nv_bfloat16* vst = vs + (size_t)st * stage_elems;
        float* raw = raw0 + (size_t)st * a.H * TKM_ROWS * TKM_KEYS;
        // raw scores of this warp's head: 16 rows x 32 keys
        float sc[TKM_KEYS / 8][4];
#pragma unroll
        for (int n = 0; n < TKM_KEYS / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
        const __nv_bfloat16* kh = kst + (size_t)g * TKM_KEYS * LDK;
#pragma unroll
        for (int s = 0; s < D / 16; ++s) {
#pragma unroll
            for (int n = 0; n < TKM_KEYS / 8; ++n) {
                const __nv_bfloat16* kp = kh + (size_t)(n * 8 + gr) * LDK + s * 16 + tq * 2;
                tkm_mma(sc[n], qf[s], *reinterpret_cast<const uint32_t*>(kp), *reinterpret_cast<const uint32_t*>(kp + 8));
            }
        }
        // scale, distance bias (slope * (position - key), the key's offset inside the tile taken from constants), and into
        // shared memory for the other heads, a lane's four values of a key octet side by side
        const float base_a = -slope * (float)(pos_a - k0 - tq * 2), base_b = base_a - slope * 8.0f;
        float4* mine = reinterpret_cast<float4*>(raw) + (size_t)h * (TKM_KEYS / 8) * 32 + lane;
#pragma unroll
        for (int n = 0; n < TKM_KEYS / 8; ++n)
            mine[n * 32] = make_float4(fmaf(sc[n][0], a.scale, base_a + off[2 * n]), fmaf(sc[n][1], a.scale, base_a + off[2 * n + 1]),
                                       fmaf(sc[n][2], a.scale, base_b + off[2 * n]), fmaf(sc[n][3], a.scale, base_b + off[2 * n + 1]));
        __syncthreads();
        // this head's mixed scores, in the fragments' places, in units of log 2 (the exponentials below are powers of two)
#pragma unroll
        for (int n = 0; n < TKM_KEYS / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
        for (int gg = 0; gg < a.H; ++gg) {
            const float w = mixs[h * a.H + gg] * 1.4426950408889634f;
            const float4* theirs = reinterpret_cast<const float4*>(raw) + (size_t)gg * (TKM_KEYS / 8) * 32 + lane;
#pragma unroll
            for (int n = 0; n < TKM_KEYS / 8; ++n) {
                const float4 r = theirs[n * 32];
                sc[n][0] = fmaf(w, r.x, sc[n][0]);
                sc[n][1] = fmaf(w, r.y, sc[n][1]);
                sc[n][2] = fmaf(w, r.z, sc[n][2]);
                sc[n][3] = fmaf(w, r.w, sc[n][3]);
            }
        }
        // (the next round writes the other copy of raw, and the round after that starts behind a barrier)
        // what a row may see: keys up to its own position (and inside its window), below the item's end.  A tile that lies
        // wholly before the item's first row, inside the item's keys, is seen by every row
        const bool all_seen = a.window <= 0 && k0 + TKM_KEYS - 1 <= pos0 && k0 + TKM_KEYS <= k_hi;
        float mx_a = -INFINITY, mx_b = -INFINITY;
        if (all_seen) {
#pragma unroll
            for (int n = 0; n < TKM_KEYS / 8; ++n) {
                mx_a = fmaxf(mx_a, fmaxf(sc[n][0], sc[n][1]));
                mx_b = fmaxf(mx_b, fmaxf(sc[n][2], sc[n][3]));
            }
        } else {
#pragma unroll
            for (int n = 0; n < TKM_KEYS / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = k0 + n * 8 + tq * 2 + e;
                    const bool in = j < k_hi;
                    const bool see_a = in && row_a && j <= pos_a && (a.window <= 0 || pos_a - j < a.window);
                    const bool see_b = in && row_b && j <= pos_b && (a.window <= 0 || pos_b - j < a.window);
                    if (!see_a) sc[n][e] = -INFINITY;
                    if (!see_b) sc[n][2 + e] = -INFINITY;
                    mx_a = fmaxf(mx_a, sc[n][e]);
                    mx_b = fmaxf(mx_b, sc[n][2 + e]);
                }
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        // a row that has seen nothing yet keeps the reference 0, so that no difference of infinities is taken
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ra = mn_a == -INFINITY ? 0.0f : mn_a, rb = mn_b == -INFINITY ? 0.0f : mn_b;
        const float ca = tkm_exp2(m_a - ra), cb = tkm_exp2(m_b - rb);            // 2^(-inf) = 0 for a row's first keys
        float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
        for (int n = 0; n < TKM_KEYS / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float pa = tkm_exp2(sc[n][e] - ra), pb = tkm_exp2(sc[n][2 + e] - rb);
                sc[n][e] = pa;
                sc[n][2 + e] = pb;
                sum_a += pa;
                sum_b += pb;
            }
        }
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
        l_a = l_a * ca + sum_a;
        l_b = l_b * cb + sum_b;
        m_a = mn_a;
        m_b = mn_b;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) { o[n][0] *= ca; o[n][1] *= ca; o[n][2] *= cb; o[n][3] *= cb; }
        // weights x values: the weights as A fragments in two bfloat16 terms (the upper half of the float, and what that
        // leaves, rounded), the values' tile read transposed
        const __nv_bfloat16* vh = vst + (size_t)g * TKM_KEYS * LDK;
#pragma unroll
        for (int s = 0; s < TKM_KEYS / 16; ++s) {
            uint32_t hi[4], lo[4];
            tkm_two_terms(sc[2 * s][0], sc[2 * s][1], hi[0], lo[0]);
            tkm_two_terms(sc[2 * s][2], sc[2 * s][3], hi[1], lo[1]);
            tkm_two_terms(sc[2 * s + 1][0], sc[2 * s + 1][1], hi[2], lo[2]);
            tkm_two_terms(sc[2 * s + 1][2], sc[2 * s + 1][3], hi[3], lo[3]);
            const uint32_t vrow = cx_smem(vh + (size_t)(s * 16 + (lane & 15)) * LDK);
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                uint32_t b0, b1;
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(vrow + n * 16));
                tkm_mma(o[n], hi, b0, b1);
                tkm_mma(o[n], lo, b0, b1);
            }
        }
    }
    if (slot_out >= 0 && a.wide) {
        // part of the keys of a portion's rows: every row's sums as they stand, with their references and weights
        float* po = a.part_o + ((size_t)slot_out * a.H + h) * TKM_ROWS * D;
        float* pm = a.part_ml + ((size_t)slot_out * a.H + h) * TKM_ROWS * 2;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            *reinterpret_cast<float2*>(po + (size_t)gr * D + n * 8 + tq * 2) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(po + (size_t)(gr + 8) * D + n * 8 + tq * 2) = make_float2(o[n][2], o[n][3]);
        }
        if (tq == 0) {
            pm[gr * 2] = m_a;
            pm[gr * 2 + 1] = l_a;
            pm[(gr + 8) * 2] = m_b;
            pm[(gr + 8) * 2 + 1] = l_b;
        }
        return;
    }
    if (slot_out >= 0) {
        // part of a row's keys (single rows only): the sums as they stand, with their reference and weight
        if (gr == 0) {
            float* po = a.part_o + ((size_t)slot_out * a.H + h) * D;
#pragma unroll
            for (int n = 0; n < D / 8; ++n) *reinterpret_cast<float2*>(po + n * 8 + tq * 2) = make_float2(o[n][0], o[n][1]);
            if (tq == 0) {
                a.part_ml[((size_t)slot_out * a.H + h) * 2] = m_a;
                a.part_ml[((size_t)slot_out * a.H + h) * 2 + 1] = l_a;
            }
        }
        return;
    }
    const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = gr + 8 * half;
        if (r >= nq) continue;
        const float inv = half ? inv_b : inv_a;
        __nv_bfloat16* orow = a.out + ((size_t)(row0 + r) * a.H + h) * D;
        const __nv_bfloat16* grow = a.gate ? a.gate + (size_t)(row0 + r) * a.ldg + (size_t)h * D : nullptr;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            float y0 = o[n][2 * half] * inv, y1 = o[n][2 * half + 1] * inv;
            if (grow) {
                const float2 gt = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(grow + n * 8 + tq * 2));
                y0 *= 1.0f / (1.0f + expf(-gt.x));
                y1 *= 1.0f / (1.0f + expf(-gt.y));
            }
            *reinterpret_cast<__nv_bfloat162*>(orow + n * 8 + tq * 2) = __floats2bfloat162_rn(y0, y1);
        }
    }
}

// ------------------------------------------------------------------ single tokens on tensor cores
// A request that brings one token: the fragment's 16 rows are the heads of one kv head's group instead of 16 tokens, so the
// keys of a kv head are multiplied once for all its heads.  A CTA per work item (a request and a run of its keys, as
// above), a warp per (kv head, sixteenth-of-a-tile): warp (g, ks) takes keys ks * 16 .. + 16 of every tile of 16 * KS keys
// for the heads of group g, with sums of its own that the CTA joins at the end.  Raw scores of all heads meet in shared
// memory as before; a warp mixes the rows of its own heads.
template <int D, int KS, int MAXT>
__global__ void __launch_bounds__(MAXT) attention_talking_decode_kernel(TalkingMmaArgs a) {
    constexpr int LDK = D + 8;
    extern __shared__ __align__(16) unsigned char tkm_smem[];
    constexpr int tile = 16 * KS;
    constexpr int RS = tile + 8;                    // floats between two heads' raw scores: eight heads' pairs fall into eight banks
    const int MS = a.H | 1;                         // floats between two rows of the mixing matrix: odd, so that rows fall into different banks
    const size_t stage_elems = (size_t)a.G * tile * LDK;
    __nv_bfloat16* ks_ = reinterpret_cast<__nv_bfloat16*>(tkm_smem);               // [2][G][tile][LDK]
    __nv_bfloat16* vs_ = ks_ + 2 * stage_elems;                                     // [2][G][tile][LDK]
    float* raw0 = reinterpret_cast<float*>(vs_ + 2 * stage_elems);                 // [2][H][RS]
    float* mixs = raw0 + 2 * (size_t)a.H * RS;                                      // [H][MS], times log2(e)
    pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = warp / KS, ks = warp - g * KS;
    const int gr = lane >> 2, tq = lane & 3;
    const int Hg = a.H / a.G;
    const int* item = a.items + (size_t)blockIdx.x * TKM_ITEM_INTS;
    const int req = item[0], k_lo = item[3], k_hi = item[4], slot_out = item[5];
    const int row = a.q_start[req] + item[1];
    const int pos = a.ctx_lens[req] + item[1];
    const int* bt = a.block_table + (size_t)req * a.bt_stride;
    for (int i = threadIdx.x; i < a.H * a.H; i += blockDim.x) mixs[(i / a.H) * MS + i % a.H] = a.mix[i] * 1.4426950408889634f;
    const bool row_a = gr < Hg, row_b = gr + 8 < Hg;
    const int head_a = g * Hg + gr, head_b = head_a + 8;
    const float slope_a = (a.slope && row_a) ? a.slope[head_a] : 0.0f, slope_b = (a.slope && row_b) ? a.slope[head_b] : 0.0f;

    uint32_t qf[D / 16][4];
    {
        const __nv_bfloat16* qa = a.q + ((size_t)row * a.H + head_a) * D + tq * 2;
        const __nv_bfloat16* qb = qa + (size_t)8 * D;
#pragma unroll
        for (int s = 0; s < D / 16; ++s) {
            qf[s][0] = row_a ? *reinterpret_cast<const uint32_t*>(qa + s * 16) : 0u;
            qf[s][1] = row_b ? *reinterpret_cast<const uint32_t*>(qb + s * 16) : 0u;
            qf[s][2] = row_a ? *reinterpret_cast<const uint32_t*>(qa + s * 16 + 8) : 0u;
            qf[s][3] = row_b ? *reinterpret_cast<const uint32_t*>(qb + s * 16 + 8) : 0u;
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;

    const size_t block = (size_t)a.page * D;
    const size_t page_elems = 2 * (size_t)a.G * block;
    constexpr int CH = D / 8, PER = CH / 4;
    const int n_pairs = a.G * tile;
    auto fetch = [&](int st, int k0) {
        __nv_bfloat16* kd = ks_ + (size_t)st * stage_elems;
        __nv_bfloat16* vd = vs_ + (size_t)st * stage_elems;
        for (int p = threadIdx.x >> 2; p < n_pairs; p += blockDim.x >> 2) {
            const int gk = p / tile, key = p - gk * tile, j = k0 + key, sub = threadIdx.x & 3;
            const __nv_bfloat16* src = a.cache;
            uint32_t bytes = 0;
            int sl = 0;
            if (j < k_hi) {
                const int lp = a.page_shift >= 0 ? j >> a.page_shift : j / a.page;
                sl = j - lp * a.page;
                const int pg = lp < a.bt_stride ? bt[lp] : -1;
                if ((unsigned)pg >= (unsigned)a.num_pages) {
                    if (a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
                } else {
                    src = a.cache + (size_t)pg * page_elems + (size_t)gk * block;
                    bytes = 16;
                }
            }
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const int ch = sub * PER + e;
                const __nv_bfloat16* from = bytes ? src + kv_pos(ch * 8, sl, D, a.page, 2) : a.cache;
                const uint32_t to_k = cx_smem(kd + ((size_t)gk * tile + key) * LDK + ch * 8);
                const uint32_t to_v = cx_smem(vd + ((size_t)gk * tile + key) * LDK + ch * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(to_k), "l"(from), "r"(bytes) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(to_v), "l"(bytes ? from + (size_t)a.G * block : from), "r"(bytes)
                             : "memory");
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    // this lane's places in a stage: its key row of the warp's sixteen for the scores' B fragments, its row for ldmatrix
    const uint32_t k_lane = cx_smem(ks_) + (uint32_t)((((g * tile + ks * 16) + gr) * LDK + tq * 2) * 2);
    const uint32_t v_lane = cx_smem(vs_) + (uint32_t)((((g * tile + ks * 16) + (lane & 15)) * LDK) * 2);
    if (k_lo < k_hi) fetch(0, k_lo);
    int it = 0;
    for (int k0 = k_lo; k0 < k_hi; k0 += tile, ++it) {
        const int st = it & 1;
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();
        if (k0 + tile < k_hi) fetch(st ^ 1, k0 + tile);
        const uint32_t stage_at = (uint32_t)st * (uint32_t)stage_elems * 2u;                 // bytes
        const uint32_t kaddr = k_lane + stage_at, vaddr = v_lane + stage_at;
        float* raw = raw0 + st * a.H * RS;
        float sc[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
        for (int s = 0; s < D / 16; ++s) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const uint32_t kp = kaddr + (uint32_t)((n * 8 * LDK + s * 16) * 2);
                tkm_mma(sc[n], qf[s], tkm_lds32(kp), tkm_lds32(kp + 16));
            }
        }
        // scale and distance bias; the rows of this group's heads into shared memory
        const int j0 = k0 + ks * 16 + tq * 2;           // this lane's first key of the tile
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const float da = (float)(pos - j0 - n * 8);
            if (row_a) *reinterpret_cast<float2*>(raw + head_a * RS + ks * 16 + n * 8 + tq * 2) =
                make_float2(fmaf(sc[n][0], a.scale, -slope_a * da), fmaf(sc[n][1], a.scale, -slope_a * (da - 1.0f)));
            if (row_b) *reinterpret_cast<float2*>(raw + head_b * RS + ks * 16 + n * 8 + tq * 2) =
                make_float2(fmaf(sc[n][2], a.scale, -slope_b * da), fmaf(sc[n][3], a.scale, -slope_b * (da - 1.0f)));
        }
        __syncthreads();
        // the mixed scores of this warp's heads at its sixteen keys, in units of log 2
#pragma unroll
        for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
        const float* wa = mixs + (row_a ? head_a : 0) * MS;
        const float* wb = mixs + (row_b ? head_b : 0) * MS;
        const float* theirs = raw + ks * 16 + tq * 2;
#pragma unroll 4
        for (int gg = 0; gg < a.H; ++gg, theirs += RS) {
            const float ua = wa[gg], ub = wb[gg];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const float2 r = *reinterpret_cast<const float2*>(theirs + n * 8);
                sc[n][0] = fmaf(ua, r.x, sc[n][0]);
                sc[n][1] = fmaf(ua, r.y, sc[n][1]);
                sc[n][2] = fmaf(ub, r.x, sc[n][2]);
                sc[n][3] = fmaf(ub, r.y, sc[n][3]);
            }
        }
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + n * 8 + e;
                const bool see = j < k_hi && j <= pos && (a.window <= 0 || pos - j < a.window);
                if (!(see && row_a)) sc[n][e] = -INFINITY;
                if (!(see && row_b)) sc[n][2 + e] = -INFINITY;
                mx_a = fmaxf(mx_a, sc[n][e]);
                mx_b = fmaxf(mx_b, sc[n][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ra = mn_a == -INFINITY ? 0.0f : mn_a, rb = mn_b == -INFINITY ? 0.0f : mn_b;
        const float ca = tkm_exp2(m_a - ra), cb = tkm_exp2(m_b - rb);
        float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float pa = tkm_exp2(sc[n][e] - ra), pb = tkm_exp2(sc[n][2 + e] - rb);
                sc[n][e] = pa;
                sc[n][2 + e] = pb;
                sum_a += pa;
                sum_b += pb;
            }
        }
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
        l_a = l_a * ca + sum_a;
        l_b = l_b * cb + sum_b;
        m_a = mn_a;
        m_b = mn_b;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) { o[n][0] *= ca; o[n][1] *= ca; o[n][2] *= cb; o[n][3] *= cb; }
        uint32_t hi[4], lo[4];
        tkm_two_terms(sc[0][0], sc[0][1], hi[0], lo[0]);
        tkm_two_terms(sc[0][2], sc[0][3], hi[1], lo[1]);
        tkm_two_terms(sc[1][0], sc[1][1], hi[2], lo[2]);
        tkm_two_terms(sc[1][2], sc[1][3], hi[3], lo[3]);
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            uint32_t b0, b1;
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(vaddr + n * 16));
            tkm_mma(o[n], hi, b0, b1);
            tkm_mma(o[n], lo, b0, b1);
        }
    }
    // the warps' sums meet in shared memory (where the tiles lay): [warp][16 rows][D] and [warp][16][2]
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    float* jo = reinterpret_cast<float*>(tkm_smem);
    float* jml = jo + (size_t)(blockDim.x >> 5) * 16 * D;
    {
        float* mine = jo + (size_t)warp * 16 * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            *reinterpret_cast<float2*>(mine + (size_t)gr * D + n * 8 + tq * 2) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(mine + (size_t)(gr + 8) * D + n * 8 + tq * 2) = make_float2(o[n][2], o[n][3]);
        }
        if (tq == 0) {
            jml[((size_t)warp * 16 + gr) * 2] = m_a;
            jml[((size_t)warp * 16 + gr) * 2 + 1] = l_a;
            jml[((size_t)warp * 16 + gr + 8) * 2] = m_b;
            jml[((size_t)warp * 16 + gr + 8) * 2 + 1] = l_b;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < a.H * D; idx += blockDim.x) {
        const int head = idx / D, i = idx - head * D;
        const int gh = head / Hg, r = head - gh * Hg;
        float m = -INFINITY;
        for (int s = 0; s < KS; ++s) m = fmaxf(m, jml[((size_t)(gh * KS + s) * 16 + r) * 2]);
        float l = 0.0f, acc = 0.0f;
        for (int s = 0; s < KS; ++s) {
            const size_t at = (size_t)(gh * KS + s) * 16 + r;
            const float ms = jml[at * 2];
            if (ms == -INFINITY) continue;
            const float f = tkm_exp2(ms - m);
            l = fmaf(jml[at * 2 + 1], f, l);
            acc = fmaf(jo[at * D + i], f, acc);
        }
        if (slot_out >= 0) {
            a.part_o[((size_t)slot_out * a.H + head) * D + i] = acc;
            if (i == 0) {
                a.part_ml[((size_t)slot_out * a.H + head) * 2] = m;
                a.part_ml[((size_t)slot_out * a.H + head) * 2 + 1] = l;
            }
        } else {
            float y = l > 0.0f ? acc / l : 0.0f;
            if (a.gate) y *= 1.0f / (1.0f + expf(-__bfloat162float(a.gate[(size_t)row * a.ldg + (size_t)head * D + i])));
            a.out[((size_t)row * a.H + head) * D + i] = __float2bfloat16_rn(y);
        }
    }
}

// Sixteenths of a tile that the single-token kernel's CTA takes at once (a warp each per kv head), 0: the sizes do not fit.
static int tkm_decode_split(int H, int G, int D, long long* smem_out) {
    if (H % G || H / G > 16 || (D != 64 && D != 128)) return 0;
    const int most_warps = D == 128 ? 8 : 16;
    for (int KS = 4; KS >= 1; KS >>= 1) {
        if (G * KS > most_warps) continue;
        const long long tiles = (long long)4 * G * 16 * KS * (D + 8) * 2, join = (long long)G * KS * 16 * (D + 2) * 4;
        const long long smem = (tiles > join ? tiles : join) + (long long)2 * H * (16 * KS + 8) * 4 + (long long)H * (H | 1) * 4;
        if (smem <= 200 * 1024) { *smem_out = smem; return KS; }
    }
    return 0;
}

VCB_EXPORT int vcb_attention_talking_decode_fits(int H, int G, int D) {
    long long smem = 0;
    return tkm_decode_split(H, G, D, &smem);
}

// Joins the partial sums of single-row items (their references are in units of log 2): request r's row was cut into `nsplit` runs of keys, whose partials lie
// in slots r * nsplit .. r * nsplit + nsplit - 1.  A CTA per request, a warp per head.
__global__ void attention_talking_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                               __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate, long long ldg,
                                               const int* __restrict__ q_start, int H, int D, int nsplit) {
    pdl_start();
    const int r = blockIdx.x, h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (h >= H) return;
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(((size_t)r * nsplit + s) * H + h) * 2]);
    float l = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float* ml = part_ml + (((size_t)r * nsplit + s) * H + h) * 2;
        if (ml[0] != -INFINITY) l += ml[1] * exp2f(ml[0] - m);
    }
    const int row = q_start[r];
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int i = lane; i < D; i += 32) {
        float acc = 0.0f;
        for (int s = 0; s < nsplit; ++s) {
            const size_t at = ((size_t)r * nsplit + s) * H + h;
            const float ms = part_ml[at * 2];
            if (ms != -INFINITY) acc = fmaf(part_o[at * D + i], exp2f(ms - m), acc);
        }
        float y = acc * inv;
        if (gate) y *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)row * ldg + (size_t)h * D + i])));
        out[((size_t)row * H + h) * D + i] = __float2bfloat16_rn(y);
    }
}

// Joins the partial sums of portions that were cut along the keys.  merge: [n, 5] = (request, first row within the request's
// rows of this step, rows, first slot, slots); partials as the kernel above leaves them with `wide`.  A CTA per entry, a
// warp per head.
__global__ void attention_talking_merge_rows_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                    __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate, long long ldg,
                                                    const int* __restrict__ q_start, const int* __restrict__ merge, int H, int D) {
    pdl_start();
    const int* e = merge + (size_t)blockIdx.x * 5;
    const int r = blockIdx.y;                       // a row of the entry a CTA, a warp per head
    if (r >= e[2]) return;
    const int row = q_start[e[0]] + e[1] + r, first = e[3], parts = min(e[4], TKM_MAX_PARTS);
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (h >= H) return;
    float ms[TKM_MAX_PARTS], ls[TKM_MAX_PARTS];
#pragma unroll
    for (int s = 0; s < TKM_MAX_PARTS; ++s) {       // every load in flight at once
        const float2 v = s < parts ? *reinterpret_cast<const float2*>(part_ml + (((size_t)(first + s) * H + h) * TKM_ROWS + r) * 2)
                                   : make_float2(-INFINITY, 0.0f);
        ms[s] = v.x;
        ls[s] = v.y;
    }
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < TKM_MAX_PARTS; ++s) m = fmaxf(m, ms[s]);
    float l = 0.0f;
#pragma unroll
    for (int s = 0; s < TKM_MAX_PARTS; ++s) {
        ms[s] = ms[s] == -INFINITY ? 0.0f : exp2f(ms[s] - m);        // from here on the part's factor
        l = fmaf(ls[s], ms[s], l);
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int i = lane; i < D; i += 32) {
        float acc = 0.0f;
#pragma unroll
        for (int s = 0; s < TKM_MAX_PARTS; ++s)
            if (s < parts) acc = fmaf(part_o[(((size_t)(first + s) * H + h) * TKM_ROWS + r) * D + i], ms[s], acc);
        float y = acc * inv;
        if (gate) y *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)row * ldg + (size_t)h * D + i])));
        out[((size_t)row * H + h) * D + i] = __float2bfloat16_rn(y);
    }
}

VCB_EXPORT long long vcb_attention_talking_mma_smem(int H, int G, int D) {
    return (long long)4 * G * TKM_KEYS * (D + 8) * 2 + (long long)2 * H * TKM_ROWS * TKM_KEYS * 4 + (long long)H * H * 4;
}

// items: [n_items, 6] as TalkingMmaArgs says.  nsplit > 1: every item is one row of a request cut into nsplit runs
// (slot = request * nsplit + run), and the merge kernel writes the n_reqs rows.  single_rows 1: every item is one row
// (a step of single tokens), which the kernel whose fragment rows are heads takes where its tiles fit.  merge (n_merge
// entries of 5, see attention_talking_merge_rows_kernel): portions whose keys were cut into several items, each with a slot.
VCB_EXPORT int vcb_attention_talking_mma(const void* q, const void* cache, void* out, const void* gate, long long ldg,
                                         const int* items, int n_items, const int* q_start, const int* ctx_lens,
                                         const int* block_table, int bt_stride, const float* mix, const float* slope,
                                         float* part_o, float* part_ml, int nsplit, int n_reqs, int H, int G, int D, int page,
                                         int window, float scale, int num_pages, int* status, int single_rows, const int* merge,
                                         int n_merge, void* stream) {
    if (n_items <= 0) return 0;
    if (!q || !cache || !out || !items || !mix || H <= 0 || G <= 0 || H % G || page <= 0 || window < 0 || num_pages < 0 || nsplit < 1)
        return VCB_ERR_BAD_ARG;
    if (H > TKM_MAX_HEADS || (D != 64 && D != 128)) return VCB_ERR_UNSUPPORTED;
    if (nsplit > 1 && (!part_o || !part_ml || n_items != n_reqs * nsplit)) return VCB_ERR_BAD_ARG;
    const long long smem = vcb_attention_talking_mma_smem(H, G, D);
    if (smem > 220 * 1024) return VCB_ERR_UNSUPPORTED;
    TalkingMmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, ldg, items,
                     q_start, ctx_lens, block_table, mix, slope, part_o, part_ml, bt_stride, H, G, page, window, num_pages, scale, status,
                     (page & (page - 1)) ? -1 : __builtin_ctz((unsigned)page), (merge && n_merge > 0) ? 1 : 0};
    if (a.wide && (nsplit > 1 || single_rows || !part_o || !part_ml)) return VCB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    long long dsmem = 0;
    const int KS = single_rows ? tkm_decode_split(H, G, D, &dsmem) : 0;
    if (KS) {
        static unsigned long long ddone[6] = {0, 0, 0, 0, 0, 0};
#define TKD_GO(DD, KK, TT, I)                                                                                       \
    do {                                                                                                            \
        const int e = vcb_allow_dynamic_smem(attention_talking_decode_kernel<DD, KK, TT>, 200 * 1024, &ddone[I]);   \
        if (e) return e;                                                                                            \
        vcb_launch(attention_talking_decode_kernel<DD, KK, TT>, n_items, G * KK * 32, (size_t)dsmem, s, a);         \
    } while (0)
        if (D == 64 && KS == 4) TKD_GO(64, 4, 512, 0);
        else if (D == 64 && KS == 2) TKD_GO(64, 2, 512, 1);
        else if (D == 64) TKD_GO(64, 1, 512, 2);
        else if (KS == 4) TKD_GO(128, 4, 256, 3);
        else if (KS == 2) TKD_GO(128, 2, 256, 4);
        else TKD_GO(128, 1, 256, 5);
#undef TKD_GO
        if (nsplit > 1)
            vcb_launch(attention_talking_merge_kernel, n_reqs, H * 32, 0, s, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out,
                       (const __nv_bfloat16*)gate, ldg, q_start, H, D, nsplit);
        return vcb_last_error();
    }
    static unsigned long long done[4] = {0, 0, 0, 0};
#define TKM_GO(DD, TT, I)                                                                                   \
    do {                                                                                                    \
        const int e = vcb_allow_dynamic_smem(attention_talking_mma_kernel<DD, TT>, 220 * 1024, &done[I]);   \
        if (e) return e;                                                                                    \
        vcb_launch(attention_talking_mma_kernel<DD, TT>, n_items, H * 32, (size_t)smem, s, a);              \
    } while (0)
    if (D == 64 && H <= 8) TKM_GO(64, 256, 0);
    else if (D == 64) TKM_GO(64, 512, 1);
    else if (H <= 8) TKM_GO(128, 256, 2);
    else TKM_GO(128, 512, 3);
#undef TKM_GO
    if (a.wide)
        vcb_launch(attention_talking_merge_rows_kernel, dim3(n_merge, TKM_ROWS), H * 32, 0, s, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gate, ldg, q_start, merge, H, D);
    if (nsplit > 1)
        vcb_launch(attention_talking_merge_kernel, n_reqs, H * 32, 0, s, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gate, ldg, q_start, H, D, nsplit);
    return vcb_last_error();
}
