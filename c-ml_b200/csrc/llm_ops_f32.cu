// fp32 device kernels behind the stand-alone C-ML entry points that sit next to the quantized
// path: cml_gqa_forward / cml_gqa_forward_cached with all of their mask options
// (src/nn/llm_ops.c:194-372), cml_rope_forward for every tensor rank it accepts (:702-805), and the
// fp32 linear of cml_column_parallel_forward / cml_row_parallel_forward
// (src/distributed/tensor_parallel.c: y = x . W^T + b). They follow C-ML's formulas literally
// (masked scores are -1e9, not -inf; a row whose keys are all masked therefore comes out as a
// uniform average) and are sized for correctness on arbitrary shapes, not for the decode hot
// path, which has its own kernels (llm_kernels.cu).
#include "common.cuh"

namespace {

constexpr int GQA_THREADS = 128;

// grid = (seq_q, heads, batch); dynamic shared memory: kv_len scores.
__global__ void __launch_bounds__(GQA_THREADS)
gqa_general_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const float* __restrict__ mask, int mask_per_batch, int seq_q, int kv_len, int heads, int kv_heads, int hd,
                   float scale, int causal, int window, float* __restrict__ out) {
    extern __shared__ float sc[];
    __shared__ float red[GQA_THREADS / 32];
    __shared__ float s_max, s_inv;
    const int sq = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (heads / kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* qv = q + ((size_t)b * seq_q + sq) * heads * hd + (size_t)h * hd;
    // scores, one key per thread and step
    for (int sk = threadIdx.x; sk < kv_len; sk += GQA_THREADS) {
        const float* kv = k + ((size_t)b * kv_len + sk) * kv_heads * hd + (size_t)kvh * hd;
        float dot = 0.f;
        for (int d = 0; d < hd; d++) dot += qv[d] * kv[d];
        float s = dot * scale;
        if (causal && sk > sq) s = -1e9f;
        if (window > 0 && sq - sk > window) s = -1e9f;
        if (mask) {
            const size_t mi = (mask_per_batch ? (size_t)b * seq_q * kv_len : 0) + (size_t)sq * kv_len + sk;
            if (mask[mi] == 0.0f) s = -1e9f;
        }
        sc[sk] = s;
    }
    __syncthreads();
    float m = -INFINITY;
    for (int sk = threadIdx.x; sk < kv_len; sk += GQA_THREADS) m = fmaxf(m, sc[sk]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int w = 1; w < GQA_THREADS / 32; w++) t = fmaxf(t, red[w]);
        s_max = t;
    }
    __syncthreads();
    float sum = 0.f;
    for (int sk = threadIdx.x; sk < kv_len; sk += GQA_THREADS) {
        const float e = expf(sc[sk] - s_max);
        sc[sk] = e;
        sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < GQA_THREADS / 32; w++) t += red[w];
        s_inv = t > 0.f ? 1.0f / t : 1.0f;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += GQA_THREADS) {
        float acc = 0.f;
        for (int sk = 0; sk < kv_len; sk++) acc += sc[sk] * s_inv * v[((size_t)b * kv_len + sk) * kv_heads * hd + (size_t)kvh * hd + d];
        out[((size_t)b * seq_q + sq) * heads * hd + (size_t)h * hd + d] = acc;
    }
}

// One thread per rotation pair of every vector. Vector v sits at position start_pos + (v / inner) % seq_len.
__global__ void rope_general_kernel(float* __restrict__ x, size_t nvec, int last_dim, int half_dim, int dim, float base,
                                    int start_pos, int seq_len, int inner) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nvec * (size_t)half_dim) return;
    const size_t vec = idx / half_dim;
    const int i = (int)(idx - vec * half_dim);
    const int pos = start_pos + (int)((vec / inner) % seq_len);
    const float freq = 1.0f / powf(base, (float)(2 * i) / (float)dim);
    const float th = (float)pos * freq;
    const float c = cosf(th), s = sinf(th);
    float* p = x + vec * last_dim + 2 * i;
    const float x0 = p[0], x1 = p[1];
    p[0] = x0 * c - x1 * s;
    p[1] = x0 * s + x1 * c;
}

// y[m][n] = sum_k x[m][k] * w[n][k] (+ b[n]); one warp per output element.
__global__ void __launch_bounds__(256)
linear_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, int N, int K,
                  float* __restrict__ y) {
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), m = blockIdx.y, lane = threadIdx.x & 31;
    if (n >= N) return;
    const float* xr = x + (size_t)m * K;
    const float* wr = w + (size_t)n * K;
    float acc = 0.f;
    for (int kk = lane; kk < K; kk += 32) acc = fmaf(xr[kk], wr[kk], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[(size_t)m * N + n] = acc + (bias ? bias[n] : 0.f);
}

}  // namespace

// softmax(Q K^T * scale + masks) V exactly as cml_gqa_forward lays it out: q [batch, seq_q, heads*hd],
// k, v [batch, kv_len, kv_heads*hd], mask NULL or [seq_q, kv_len] (mask_per_batch = 0) or
// [batch, seq_q, kv_len] (1) with 0 = masked, out [batch, seq_q, heads*hd].
extern "C" int cmlb200_gqa_f32(const float* d_q, const float* d_k, const float* d_v, const float* d_mask, int mask_per_batch, int batch,
                               int seq_q, int kv_len, int heads, int kv_heads, int head_dim, float scale, int causal, int window,
                               float* d_out, void* stream) {
    CMLB_REQUIRE(d_q && d_k && d_v && d_out, "cmlb200_gqa_f32: NULL argument");
    CMLB_REQUIRE(batch > 0 && seq_q > 0 && kv_len > 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && heads % kv_heads == 0,
                 "cmlb200_gqa_f32: bad shape");
    CMLB_REQUIRE(heads <= 65535 && batch <= 65535, "cmlb200_gqa_f32: more than 65535 heads or batches");
    const size_t smem = (size_t)kv_len * sizeof(float);
    CMLB_REQUIRE(smem <= 200 * 1024, "cmlb200_gqa_f32: kv_len %d exceeds the 51200 keys one CTA can hold", kv_len);
    if (smem > 48 * 1024) CMLB_CUDA(cudaFuncSetAttribute(gqa_general_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gqa_general_kernel<<<dim3(seq_q, heads, batch), GQA_THREADS, smem, as_stream(stream)>>>(
        d_q, d_k, d_v, d_mask, mask_per_batch, seq_q, kv_len, heads, kv_heads, head_dim, scale, causal, window, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

// In-place rotation of the first min(dim, last_dim) elements of every vector of x (pairs 2i, 2i+1,
// frequency base^(-2i/dim)); vector number v is at position start_pos + (v / inner) % seq_len.
extern "C" int cmlb200_rope_f32(float* d_x, size_t nvec, int last_dim, int dim, float base, int start_pos, int seq_len, int inner,
                                void* stream) {
    CMLB_REQUIRE(d_x && nvec > 0 && last_dim > 0 && dim > 0 && seq_len > 0 && inner > 0, "cmlb200_rope_f32: bad argument");
    if (base <= 0.f) base = 10000.0f;
    const int half = (dim < last_dim ? dim : last_dim) / 2;
    if (half == 0) return CMLB200_OK;
    const size_t total = nvec * (size_t)half;
    rope_general_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(d_x, nvec, last_dim, half, dim, base, start_pos,
                                                                                       seq_len, inner);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

// y[M, N] = x[M, K] . w[N, K]^T (+ bias[N]), all fp32.
extern "C" int cmlb200_linear_f32(const float* d_x, const float* d_w, const float* d_bias, int M, int N, int K, float* d_y, void* stream) {
    CMLB_REQUIRE(d_x && d_w && d_y && M > 0 && N > 0 && K > 0 && M <= 65535, "cmlb200_linear_f32: bad argument");
    linear_f32_kernel<<<dim3((N + 7) / 8, M), 256, 0, as_stream(stream)>>>(d_x, d_w, d_bias, N, K, d_y);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
