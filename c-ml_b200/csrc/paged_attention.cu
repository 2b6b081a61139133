// Attention of one sequence over a paged KV pool (src/nn/paged_attention.c:332-480): the keys and
// values of token t live in block ids[t / block_size], slot t % block_size, of one pool
// [blocks][block_size][kv_heads * head_dim] per K and V. Query row sq sits at absolute position
// kv_len - seq_q + sq; with `causal` later keys score -1e9 as in C-ML (their weight is exactly 0 in
// fp32). One CTA per (query row, head): scores with one warp per key (lanes across head_dim, so a
// key row is one coalesced read), softmax with max subtraction, then the weighted sum of V with
// the output elements across the threads.
#include "common.cuh"

namespace {

constexpr int PG_THREADS = 128;

__global__ void __launch_bounds__(PG_THREADS)
paged_gqa_kernel(const float* __restrict__ q, const float* __restrict__ kpool, const float* __restrict__ vpool,
                 const int* __restrict__ ids, int block_size, int seq_q, int kv_len, int heads, int kv_heads, int hd, float scale,
                 int causal, float* __restrict__ out) {
    extern __shared__ float sc[];                       // kv_len scores
    __shared__ float red[PG_THREADS / 32];
    __shared__ float s_max, s_inv;
    const int sq = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (heads / kv_heads), kvw = kv_heads * hd;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* qv = q + ((size_t)sq * heads + h) * hd;
    const int abs_pos = kv_len - seq_q + sq;
    for (int sk = warp; sk < kv_len; sk += PG_THREADS / 32) {
        const float* kr = kpool + ((size_t)ids[sk / block_size] * block_size + sk % block_size) * kvw + (size_t)kvh * hd;
        float dot = 0.f;
        for (int d = lane; d < hd; d += 32) dot = fmaf(qv[d], kr[d], dot);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) sc[sk] = (causal && sk > abs_pos) ? -1e9f : dot * scale;
    }
    __syncthreads();
    float m = -INFINITY;
    for (int sk = threadIdx.x; sk < kv_len; sk += PG_THREADS) m = fmaxf(m, sc[sk]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int w = 1; w < PG_THREADS / 32; w++) t = fmaxf(t, red[w]);
        s_max = t;
    }
    __syncthreads();
    float sum = 0.f;
    for (int sk = threadIdx.x; sk < kv_len; sk += PG_THREADS) {
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
        for (int w = 0; w < PG_THREADS / 32; w++) t += red[w];
        s_inv = t > 0.f ? 1.0f / t : 1.0f;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += PG_THREADS) {
        float acc = 0.f;
        for (int sk = 0; sk < kv_len; sk++) {
            if (sc[sk] == 0.f) continue;                 // masked keys (uniform across the threads)
            const float* vr = vpool + ((size_t)ids[sk / block_size] * block_size + sk % block_size) * kvw + (size_t)kvh * hd;
            acc = fmaf(sc[sk] * s_inv, vr[d], acc);
        }
        out[((size_t)sq * heads + h) * hd + d] = acc;
    }
}

}  // namespace

// d_q, d_out: [seq_q, heads * head_dim] fp32; d_kpool, d_vpool: [blocks][block_size][kv_heads * head_dim]
// fp32; d_block_ids: the sequence's block table (ceil(kv_len / block_size) entries).
extern "C" int cmlb200_paged_gqa_f32(const float* d_q, const float* d_kpool, const float* d_vpool, const int* d_block_ids, int block_size,
                                     int seq_q, int kv_len, int heads, int kv_heads, int head_dim, float scale, int causal, float* d_out,
                                     void* stream) {
    CMLB_REQUIRE(d_q && d_kpool && d_vpool && d_block_ids && d_out, "cmlb200_paged_gqa_f32: NULL argument");
    CMLB_REQUIRE(block_size > 0 && seq_q > 0 && kv_len > 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && heads % kv_heads == 0,
                 "cmlb200_paged_gqa_f32: bad shape");
    CMLB_REQUIRE(heads <= 65535, "cmlb200_paged_gqa_f32: more than 65535 heads");
    const size_t smem = (size_t)kv_len * sizeof(float);
    CMLB_REQUIRE(smem <= 200 * 1024, "cmlb200_paged_gqa_f32: kv_len %d exceeds the 51200 keys one CTA can hold", kv_len);
    static size_t attr_smem[kMaxDevices] = {};
    CMLB_CUDA(cmlb_ensure_smem(paged_gqa_kernel, smem, attr_smem));
    paged_gqa_kernel<<<dim3(seq_q, heads), PG_THREADS, smem, as_stream(stream)>>>(d_q, d_kpool, d_vpool, d_block_ids, block_size, seq_q, kv_len,
                                                                                  heads, kv_heads, head_dim, scale, causal, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
