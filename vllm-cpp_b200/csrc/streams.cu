// A residual stream kept as several copies (hyper-connections) and the layer norm that reads it.
//
//   x: float [S, n, hidden], S streams of the step's rows.  A sublayer reads  u = sum_s in[s] x_s  through a layer norm
//   with gain and bias,  h = (u - mean(u)) / sqrt(var(u) + eps) * w + b,  and its result y joins all streams at once,
//   x_t <- sum_s mix[s, t] x_s + out[t] y.
//
//   stream_norm_kernel   h = layer_norm(sum_s coef[s] x_s) for the step's rows, or for gathered rows (the rows whose
//                        logits are wanted, with coef = 1: the model's output reads the sum of the streams)
//   stream_join_kernel   the join of a sublayer's result and, in the same pass, the read and the norm of the sublayer
//                        that follows (its in[], gain and bias), the row staying in shared memory between the two
//
// S = 1 with in = out = mix = 1 is the plain residual stream, x += y, with a layer norm.  Streams, sums, mean and
// variance (mean of the squared deviations, two passes) are float whatever the activations' type T is.
// The reference has one residual stream and an RMS norm (src/model/qwen.cpp:300-318, src/kernels/layernorm.cu).
#include "common.cuh"

#define STREAMS_MAX 8

struct StreamNormArgs {
    const float* x;             // [S, n, hidden]
    long long stream_stride;    // elements between two streams
    const float* coef;          // [S]
    const float* w;             // [hidden]
    const float* b;             // [hidden] or null
    void* out;                  // [rows, hidden] of T
    const int* row_index;       // [rows] or null: out row o reads x row row_index[o]
    int S, hidden;
    float eps, out_scale;       // out_scale multiplies the normed row (gain and bias alike)
};

// u (shared, [hidden]) holds the row; every thread gets mean and 1 / sqrt(var + eps)
__device__ __forceinline__ void row_statistics(const float* u, int hidden, float eps, float* scratch, float& mean, float& rstd) {
    float s = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) s += u[i];
    mean = block_sum(s, scratch) / (float)hidden;
    float v = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float d = u[i] - mean; v += d * d; }
    rstd = 1.0f / sqrtf(block_sum(v, scratch) / (float)hidden + eps);
}

template <typename T>
__global__ void stream_norm_kernel(StreamNormArgs a) {
    extern __shared__ float u[];
    __shared__ float scratch[33];
    pdl_start();
    const int o = blockIdx.x;
    const int row = a.row_index ? a.row_index[o] : o;
    float c[STREAMS_MAX];
#pragma unroll
    for (int s = 0; s < STREAMS_MAX; ++s) c[s] = s < a.S ? a.coef[s] : 0.0f;
    const float* x = a.x + (size_t)row * a.hidden;
    for (int i = threadIdx.x; i < a.hidden; i += blockDim.x) {
        float acc = 0.0f;
#pragma unroll
        for (int s = 0; s < STREAMS_MAX; ++s)
            if (s < a.S) acc = fmaf(c[s], x[(size_t)s * a.stream_stride + i], acc);
        u[i] = acc;
    }
    float mean, rstd;
    row_statistics(u, a.hidden, a.eps, scratch, mean, rstd);
    T* dst = (T*)a.out + (size_t)o * a.hidden;
    for (int i = threadIdx.x; i < a.hidden; i += blockDim.x) {
        const float y = (u[i] - mean) * rstd * a.w[i] + (a.b ? a.b[i] : 0.0f);
        dst[i] = from_f32<T>(y * a.out_scale);
    }
}

VCB_EXPORT int vcb_stream_norm(const float* x, long long stream_stride, const float* coef, const float* w, const float* b,
                               void* out, const int* row_index, int rows, int S, int hidden, float eps, float out_scale,
                               int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (!x || !coef || !w || !out || S <= 0 || S > STREAMS_MAX || hidden <= 0) return VCB_ERR_BAD_ARG;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return VCB_ERR_UNSUPPORTED;
    StreamNormArgs a{x, stream_stride, coef, w, b, out, row_index, S, hidden, eps, out_scale};
    const int threads = hidden >= 4096 ? 512 : hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    static unsigned long long done_f = 0, done_b = 0;
    if (dtype == VCB_F32) {
        if (smem > 48 * 1024) { const int e = vcb_allow_dynamic_smem(stream_norm_kernel<float>, (int)smem, &done_f); if (e) return e; }
        vcb_launch(stream_norm_kernel<float>, rows, threads, smem, s, a);
    } else if (dtype == VCB_BF16) {
        if (smem > 48 * 1024) { const int e = vcb_allow_dynamic_smem(stream_norm_kernel<__nv_bfloat16>, (int)smem, &done_b); if (e) return e; }
        vcb_launch(stream_norm_kernel<__nv_bfloat16>, rows, threads, smem, s, a);
    } else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

struct StreamJoinArgs {
    float* x;                   // [S, n, hidden], rewritten in place
    long long stream_stride;
    const void* y;              // [n, hidden] of T: the sublayer's result
    const float* mix;           // [S, S], indexed [from, to]
    const float* out_coef;      // [S]
    // the sublayer that follows (null next_out: none)
    const float* next_coef;     // [S]
    const float* next_w;
    const float* next_b;        // or null
    void* next_out;             // [n, hidden] of T
    int S, hidden;
    float eps;
};

template <typename T>
__global__ void stream_join_kernel(StreamJoinArgs a) {
    extern __shared__ float u[];
    __shared__ float scratch[33];
    __shared__ float coefs[STREAMS_MAX * STREAMS_MAX + 2 * STREAMS_MAX];
    const int S = a.S;
    // the coefficients are weights: read ahead of the kernel before
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) coefs[i] = a.mix[i];
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        coefs[STREAMS_MAX * STREAMS_MAX + i] = a.out_coef[i];
        coefs[STREAMS_MAX * STREAMS_MAX + STREAMS_MAX + i] = a.next_out ? a.next_coef[i] : 0.0f;
    }
    pdl_start();
    __syncthreads();
    const float* mix = coefs;
    const float* oc = coefs + STREAMS_MAX * STREAMS_MAX;
    const float* nc = oc + STREAMS_MAX;
    const size_t row = (size_t)blockIdx.x * a.hidden;
    float* x = a.x + row;
    const T* y = (const T*)a.y + row;
    for (int i = threadIdx.x; i < a.hidden; i += blockDim.x) {
        float old[STREAMS_MAX];
#pragma unroll
        for (int s = 0; s < STREAMS_MAX; ++s) old[s] = s < S ? x[(size_t)s * a.stream_stride + i] : 0.0f;
        const float yv = to_f32<T>(y[i]);
        float acc = 0.0f;
#pragma unroll
        for (int t = 0; t < STREAMS_MAX; ++t) {
            if (t >= S) break;
            float v = oc[t] * yv;
#pragma unroll
            for (int s = 0; s < STREAMS_MAX; ++s)
                if (s < S) v = fmaf(mix[s * S + t], old[s], v);
            x[(size_t)t * a.stream_stride + i] = v;
            acc = fmaf(nc[t], v, acc);
        }
        if (a.next_out) u[i] = acc;
    }
    if (!a.next_out) return;
    float mean, rstd;
    row_statistics(u, a.hidden, a.eps, scratch, mean, rstd);
    T* dst = (T*)a.next_out + row;
    for (int i = threadIdx.x; i < a.hidden; i += blockDim.x)
        dst[i] = from_f32<T>((u[i] - mean) * rstd * a.next_w[i] + (a.next_b ? a.next_b[i] : 0.0f));
}

VCB_EXPORT int vcb_stream_join(float* x, long long stream_stride, const void* y, const float* mix, const float* out_coef,
                               const float* next_coef, const float* next_w, const float* next_b, void* next_out, int n,
                               int S, int hidden, float eps, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (!x || !y || !mix || !out_coef || S <= 0 || S > STREAMS_MAX || hidden <= 0) return VCB_ERR_BAD_ARG;
    if (next_out && (!next_coef || !next_w)) return VCB_ERR_BAD_ARG;
    const size_t smem = next_out ? (size_t)hidden * sizeof(float) : 0;
    if (smem > 200 * 1024) return VCB_ERR_UNSUPPORTED;
    StreamJoinArgs a{x, stream_stride, y, mix, out_coef, next_coef, next_w, next_b, next_out, S, hidden, eps};
    const int threads = hidden >= 4096 ? 512 : hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    static unsigned long long done_f = 0, done_b = 0;
    if (dtype == VCB_F32) {
        if (smem > 48 * 1024) { const int e = vcb_allow_dynamic_smem(stream_join_kernel<float>, (int)smem, &done_f); if (e) return e; }
        vcb_launch(stream_join_kernel<float>, n, threads, smem, s, a);
    } else if (dtype == VCB_BF16) {
        if (smem > 48 * 1024) { const int e = vcb_allow_dynamic_smem(stream_join_kernel<__nv_bfloat16>, (int)smem, &done_b); if (e) return e; }
        vcb_launch(stream_join_kernel<__nv_bfloat16>, n, threads, smem, s, a);
    } else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
