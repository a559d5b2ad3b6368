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
