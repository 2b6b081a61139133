// The non-matmul pieces of the LLaMA forward pass, on device: embedding gather, RMSNorm,
// RoPE, KV-cache append, grouped-query attention over the cache (split over the key range and
// merged), greedy argmax, and the small element-wise kernels of the bf16 prefill pipeline.
//
// "Rows" are the activation rows of one forward call: the positions of a prompt (prefill) or
// one token per sequence (batched decode). Every row r carries row_seq[r] (which sequence's
// cache it belongs to), row_pos[r] (absolute position) and row_limit[r] (last cache slot it may
// attend to), so one set of kernels serves prefill, decode and batching.
//
// C-ML equivalents: embed_tokens_lookup src/nn/llama.c:421-452, rms_norm :71-124,
// cml_rope_forward src/nn/llm_ops.c:702-805, cml_kv_cache_append :118-157,
// cml_gqa_forward :194-361, greedy branch of cml_llama_sample_token src/nn/llama.c:650-660.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- embedding gather: fp16 table -> fp32 rows; out-of-range ids read row 0 (llama.c:440-444)
__global__ void embed_kernel(const __half* __restrict__ table, const int* __restrict__ tokens, int hidden, int vocab,
                             float* __restrict__ out) {
    const int r = blockIdx.x;
    int t = tokens[r];
    if (t < 0 || t >= vocab) t = 0;
    const __half* src = table + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)r * hidden + i] = __half2float(src[i]);
}

// ---- RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w, fp16 weight, fp32 or bf16 output
template <bool BF16_OUT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const __half* __restrict__ w, int dim, float eps, void* out) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)r * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / (float)dim + eps);
    }
    __syncthreads();
    const float inv = red[0];
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = xr[i] * inv * __half2float(w[i]);
        if (BF16_OUT) reinterpret_cast<__nv_bfloat16*>(out)[(size_t)r * dim + i] = __float2bfloat16_rn(v);
        else reinterpret_cast<float*>(out)[(size_t)r * dim + i] = v;
    }
}

// ---- RoPE, interleaved pairs (2i, 2i+1), freq = 1 / powf(base, 2i / head_dim), in place.
// heads_to_rotate = 1 reproduces C-ML's behaviour on the 2-D [seq, heads*head_dim] tensors
// llama.c passes (only the first head_dim columns rotate); = heads rotates every head.
__global__ void rope_kernel(float* __restrict__ x, const int* __restrict__ row_pos, int width, int head_dim, float base,
                            int heads_to_rotate) {
    const int r = blockIdx.x;
    const float pos = (float)row_pos[r];
    const int half = head_dim / 2;
    for (int idx = threadIdx.x; idx < heads_to_rotate * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const float freq = 1.0f / powf(base, (float)(2 * i) / (float)head_dim);
        const float th = pos * freq;
        const float c = cosf(th), s = sinf(th);
        float* v = x + (size_t)r * width + (size_t)h * head_dim + 2 * i;
        const float a = v[0], b = v[1];
        v[0] = a * c - b * s;
        v[1] = a * s + b * c;
    }
}

// ---- KV append: rows of K and V go to slot row_pos[r] of sequence row_seq[r]
template <typename KV>
__global__ void kv_append_kernel(const float* __restrict__ k, const float* __restrict__ v, KV* __restrict__ kc,
                                 KV* __restrict__ vc, const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                 int kvw, int max_seq) {
    const int r = blockIdx.x;
    const size_t dst = ((size_t)row_seq[r] * max_seq + row_pos[r]) * kvw;
    for (int i = threadIdx.x; i < kvw; i += blockDim.x) {
        kc[dst + i] = (KV)k[(size_t)r * kvw + i];
        vc[dst + i] = (KV)v[(size_t)r * kvw + i];
    }
}

// ---- attention over the cache. grid = (heads, rows, splits). Each CTA covers keys
// [split*chunk, min((split+1)*chunk, limit+1)) of one (row, head): scores q.k/sqrt(d), running
// max / sum / weighted V per warp, merged in shared memory, written as an unnormalised partial
// (max, sum, acc[hd]); attention_merge_kernel combines the splits. Keys beyond row_limit are the
// causally masked ones: C-ML gives them -1e9 before the softmax, i.e. weight exp(-1e9 - max) = 0
// in fp32, so skipping them yields the same result.
constexpr int ATT_THREADS = 128;
template <typename KV, int HD>
__global__ void __launch_bounds__(ATT_THREADS)
attention_partial_kernel(const float* __restrict__ q, const KV* __restrict__ kc, const KV* __restrict__ vc,
                         const int* __restrict__ row_seq, const int* __restrict__ row_limit, int heads, int kv_heads,
                         int max_seq, int chunk, float* __restrict__ partial) {
    constexpr int PER = HD / 32;                       // head-dim elements per lane
    const int h = blockIdx.x, r = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = ATT_THREADS / 32;
    const int kvw = kv_heads * HD;
    const int kh = h / (heads / kv_heads);
    const int limit = row_limit[r];
    const int k_begin = split * chunk, k_end = min(limit + 1, k_begin + chunk);
    const size_t base = (size_t)row_seq[r] * max_seq * kvw + (size_t)kh * HD;
    const float scale = 1.0f / sqrtf((float)HD);
    float qv[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) qv[i] = q[((size_t)r * heads + h) * HD + lane + 32 * i];
    float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;
    for (int sk = k_begin + warp; sk < k_end; sk += NW) {
        const KV* kp = kc + base + (size_t)sk * kvw;
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < PER; i++) d = fmaf(qv[i], (float)kp[lane + 32 * i], d);
        d = warp_sum(d) * scale;
        const float mn = fmaxf(m, d);
        const float corr = expf(m - mn), p = expf(d - mn);
        const KV* vp = vc + base + (size_t)sk * kvw;
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < PER; i++) acc[i] = acc[i] * corr + p * (float)vp[lane + 32 * i];
        m = mn;
    }
    __shared__ float sm[NW], sl[NW], sacc[NW][HD];
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int i = 0; i < PER; i++) sacc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; w++) gm = fmaxf(gm, sm[w]);
    float* out = partial + (((size_t)r * heads + h) * nsplit + split) * (HD + 2);
    if (threadIdx.x < HD) {
        float a = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float c = (sm[w] == -INFINITY) ? 0.f : expf(sm[w] - gm);
            a = fmaf(sacc[w][threadIdx.x], c, a);
            lt = fmaf(sl[w], c, lt);
        }
        out[2 + threadIdx.x] = a;
        if (threadIdx.x == 0) { out[0] = gm; out[1] = lt; }
    }
}

template <int HD>
__global__ void attention_merge_kernel(const float* __restrict__ partial, int nsplit, float* __restrict__ out) {
    const size_t rh = blockIdx.x;                      // row * heads + head
    const float* p = partial + rh * nsplit * (HD + 2);
    float gm = -INFINITY;
    for (int s = 0; s < nsplit; s++) gm = fmaxf(gm, p[s * (HD + 2)]);
    float l = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ms = p[s * (HD + 2)];
        if (ms != -INFINITY) l += p[s * (HD + 2) + 1] * expf(ms - gm);
    }
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < nsplit; s++) {
            const float ms = p[s * (HD + 2)];
            if (ms != -INFINITY) a = fmaf(p[s * (HD + 2) + 2 + i], expf(ms - gm), a);
        }
        out[rh * HD + i] = a / l;
    }
}

// ---- greedy pick: first index holding the strict maximum of each row
__global__ void argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    }
}

// ---- row bookkeeping kept on the device so that a decode step can be replayed as a CUDA graph
// mode 0: sequence `seq`, `rows` consecutive positions starting at cur_len[seq] (prefill / single decode)
// mode 1: `rows` sequences, one token each at cur_len[b] (batched decode)
// relative_mask != 0 reproduces C-ML's causal mask on call-relative indices (llm_ops.c:290-298).
__global__ void prepare_rows_kernel(const int* __restrict__ cur_len, int rows, int mode, int relative_mask, int seq,
                                    int* row_seq, int* row_pos, int* row_limit) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    if (mode == 0) {
        row_seq[r] = seq;
        row_pos[r] = cur_len[seq] + r;
        row_limit[r] = relative_mask ? r : cur_len[seq] + r;
    } else {
        row_seq[r] = r;
        row_pos[r] = cur_len[r];
        row_limit[r] = relative_mask ? 0 : cur_len[r];
    }
}
__global__ void advance_rows_kernel(int* cur_len, int rows, int mode, int seq) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (mode == 0) { if (r == 0) cur_len[seq] += rows; }
    else if (r < rows) cur_len[r] += 1;
}

// ---- element-wise helpers of the bf16 prefill pipeline
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(in[i]);
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void add_bf16_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ in, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        acc[i] += __bfloat162float(in[i]);
}
__global__ void add_f32_kernel(float* __restrict__ acc, const float* __restrict__ in, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        acc[i] += in[i];
}
// silu(g) * u with silu(g) = g / (1 + expf(-g)) (src/ops/ir/execution.c:2980-2987)
__global__ void swiglu_bf16_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                   __nv_bfloat16* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float gv = __bfloat162float(g[i]);
        out[i] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * __bfloat162float(u[i]));
    }
}

__global__ void swiglu_f32_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float gv = g[i];
        out[i] = gv / (1.0f + expf(-gv)) * u[i];
    }
}

// LoRA low-rank term of the quantized Linear (src/nn/qlora.c:336-361):
// t[b][r] = sum_i x[b][i] * A[r][i]   then   y[b][o] += scaling * sum_r t[b][r] * B[o][r]
__global__ void lora_down_kernel(const float* __restrict__ x, const float* __restrict__ A, int K, int rank, float* __restrict__ t) {
    const int b = blockIdx.y, r = blockIdx.x;
    float s = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) s = fmaf(x[(size_t)b * K + i], A[(size_t)r * K + i], s);
    s = warp_sum(s);
    __shared__ float red[32];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) t[(size_t)b * rank + r] = v;
    }
}
__global__ void lora_up_kernel(const float* __restrict__ t, const float* __restrict__ B, int N, int rank, float scaling,
                               float* __restrict__ y) {
    const int b = blockIdx.y;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= N) return;
    float s = 0.f;
    for (int r = 0; r < rank; r++) s = fmaf(t[(size_t)b * rank + r], B[(size_t)o * rank + r], s);
    y[(size_t)b * N + o] += scaling * s;
}

inline int ew_grid(size_t n) {
    size_t g = (n + 255) / 256;
    const size_t cap = (size_t)cmlb_num_sms() * 8;
    return (int)(g > cap ? cap : (g ? g : 1));
}

}  // namespace

extern "C" int cmlb200_embed_f16(const uint16_t* d_table_f16, const int* d_tokens, int rows, int hidden, int vocab,
                                 float* d_out, void* stream) {
    CMLB_REQUIRE(d_table_f16 && d_tokens && d_out && rows > 0 && hidden > 0 && vocab > 0, "cmlb200_embed_f16: bad argument");
    embed_kernel<<<rows, 256, 0, as_stream(stream)>>>((const __half*)d_table_f16, d_tokens, hidden, vocab, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_rmsnorm(const float* d_x, const uint16_t* d_w_f16, int rows, int dim, float eps, float* d_out_f32,
                               uint16_t* d_out_bf16, void* stream) {
    CMLB_REQUIRE(d_x && d_w_f16 && (d_out_f32 || d_out_bf16) && rows > 0 && dim > 0, "cmlb200_rmsnorm: bad argument");
    if (d_out_bf16) rmsnorm_kernel<true><<<rows, 256, 0, as_stream(stream)>>>(d_x, (const __half*)d_w_f16, dim, eps, d_out_bf16);
    else rmsnorm_kernel<false><<<rows, 256, 0, as_stream(stream)>>>(d_x, (const __half*)d_w_f16, dim, eps, d_out_f32);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_rope(float* d_x, const int* d_row_pos, int rows, int width, int head_dim, float base, int all_heads,
                            void* stream) {
    CMLB_REQUIRE(d_x && d_row_pos && rows > 0 && head_dim > 0 && head_dim % 2 == 0 && width >= head_dim && width % head_dim == 0,
                 "cmlb200_rope: bad argument");
    if (base <= 0.f) base = 10000.0f;
    rope_kernel<<<rows, 256, 0, as_stream(stream)>>>(d_x, d_row_pos, width, head_dim, base, all_heads ? width / head_dim : 1);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_kv_append(const float* d_k, const float* d_v, void* d_kcache, void* d_vcache, const int* d_row_seq,
                                 const int* d_row_pos, int rows, int kvw, int max_seq, int kv_is_f32, void* stream) {
    CMLB_REQUIRE(d_k && d_v && d_kcache && d_vcache && d_row_seq && d_row_pos && rows > 0 && kvw > 0 && max_seq > 0,
                 "cmlb200_kv_append: bad argument");
    if (kv_is_f32)
        kv_append_kernel<float><<<rows, 256, 0, as_stream(stream)>>>(d_k, d_v, (float*)d_kcache, (float*)d_vcache, d_row_seq, d_row_pos, kvw, max_seq);
    else
        kv_append_kernel<__half><<<rows, 256, 0, as_stream(stream)>>>(d_k, d_v, (__half*)d_kcache, (__half*)d_vcache, d_row_seq, d_row_pos, kvw, max_seq);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

// Number of floats of scratch cmlb200_attention needs for `rows` rows and `splits` key splits.
extern "C" size_t cmlb200_attention_scratch_floats(int rows, int heads, int head_dim, int splits) {
    return (size_t)rows * heads * splits * (head_dim + 2);
}

extern "C" int cmlb200_attention(const float* d_q, const void* d_kcache, const void* d_vcache, const int* d_row_seq,
                                 const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq,
                                 int max_limit, int kv_is_f32, float* d_out, float* d_scratch, int splits, void* stream) {
    CMLB_REQUIRE(d_q && d_kcache && d_vcache && d_row_seq && d_row_limit && d_out && d_scratch, "cmlb200_attention: NULL argument");
    CMLB_REQUIRE(rows > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "cmlb200_attention: num_heads (%d) must be divisible by num_kv_heads (%d)", heads, kv_heads);
    CMLB_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 32, "cmlb200_attention: head_dim %d not in {32, 64, 128}", head_dim);
    CMLB_REQUIRE(splits >= 1 && max_limit >= 0 && max_limit < max_seq, "cmlb200_attention: bad splits/max_limit");
    const int chunk = (max_limit + 1 + splits - 1) / splits;
    dim3 grid(heads, rows, splits);
    cudaStream_t st = as_stream(stream);
#define ATT_LAUNCH(KV, HD)                                                                                            \
    attention_partial_kernel<KV, HD><<<grid, ATT_THREADS, 0, st>>>(d_q, (const KV*)d_kcache, (const KV*)d_vcache,   \
                                                                   d_row_seq, d_row_limit, heads, kv_heads, max_seq, \
                                                                   chunk, d_scratch);                                \
    attention_merge_kernel<HD><<<rows * heads, HD, 0, st>>>(d_scratch, splits, d_out)
    if (kv_is_f32) {
        if (head_dim == 128) { ATT_LAUNCH(float, 128); } else if (head_dim == 64) { ATT_LAUNCH(float, 64); } else { ATT_LAUNCH(float, 32); }
    } else {
        if (head_dim == 128) { ATT_LAUNCH(__half, 128); } else if (head_dim == 64) { ATT_LAUNCH(__half, 64); } else { ATT_LAUNCH(__half, 32); }
    }
#undef ATT_LAUNCH
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_argmax(const float* d_logits, int rows, int vocab, int* d_out, void* stream) {
    CMLB_REQUIRE(d_logits && d_out && rows > 0 && vocab > 0, "cmlb200_argmax: bad argument");
    argmax_kernel<<<rows, 1024, 0, as_stream(stream)>>>(d_logits, vocab, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_prepare_rows(const int* d_cur_len, int rows, int mode, int relative_mask, int seq, int* d_row_seq,
                                    int* d_row_pos, int* d_row_limit, void* stream) {
    CMLB_REQUIRE(d_cur_len && d_row_seq && d_row_pos && d_row_limit && rows > 0 && seq >= 0, "cmlb200_prepare_rows: bad argument");
    prepare_rows_kernel<<<(rows + 127) / 128, 128, 0, as_stream(stream)>>>(d_cur_len, rows, mode, relative_mask, seq, d_row_seq, d_row_pos, d_row_limit);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_advance_rows(int* d_cur_len, int rows, int mode, int seq, void* stream) {
    CMLB_REQUIRE(d_cur_len && rows > 0 && seq >= 0, "cmlb200_advance_rows: bad argument");
    advance_rows_kernel<<<(rows + 127) / 128, 128, 0, as_stream(stream)>>>(d_cur_len, rows, mode, seq);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_bf16_to_f32(const uint16_t* d_in, float* d_out, size_t n, void* stream) {
    CMLB_REQUIRE(d_in && d_out && n, "cmlb200_bf16_to_f32: bad argument");
    bf16_to_f32_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>((const __nv_bfloat16*)d_in, d_out, n);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
extern "C" int cmlb200_f32_to_bf16(const float* d_in, uint16_t* d_out, size_t n, void* stream) {
    CMLB_REQUIRE(d_in && d_out && n, "cmlb200_f32_to_bf16: bad argument");
    f32_to_bf16_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>(d_in, (__nv_bfloat16*)d_out, n);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
extern "C" int cmlb200_add_bf16(float* d_acc, const uint16_t* d_in, size_t n, void* stream) {
    CMLB_REQUIRE(d_acc && d_in && n, "cmlb200_add_bf16: bad argument");
    add_bf16_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>(d_acc, (const __nv_bfloat16*)d_in, n);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
extern "C" int cmlb200_add_f32(float* d_acc, const float* d_in, size_t n, void* stream) {
    CMLB_REQUIRE(d_acc && d_in && n, "cmlb200_add_f32: bad argument");
    add_f32_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>(d_acc, d_in, n);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
extern "C" int cmlb200_swiglu_bf16(const uint16_t* d_gate, const uint16_t* d_up, uint16_t* d_out, size_t n, void* stream) {
    CMLB_REQUIRE(d_gate && d_up && d_out && n, "cmlb200_swiglu_bf16: bad argument");
    swiglu_bf16_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>((const __nv_bfloat16*)d_gate, (const __nv_bfloat16*)d_up,
                                                               (__nv_bfloat16*)d_out, n);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
extern "C" int cmlb200_swiglu_f32(const float* d_gate, const float* d_up, float* d_out, size_t n, void* stream) {
    CMLB_REQUIRE(d_gate && d_up && d_out && n, "cmlb200_swiglu_f32: bad argument");
    swiglu_f32_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>(d_gate, d_up, d_out, n);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
extern "C" int cmlb200_lora_accum(const float* d_x, const float* d_A, const float* d_B, int M, int K, int N, int rank,
                                  float scaling, float* d_t, float* d_y, void* stream) {
    CMLB_REQUIRE(d_x && d_A && d_B && d_t && d_y && M > 0 && K > 0 && N > 0 && rank > 0, "cmlb200_lora_accum: bad argument");
    lora_down_kernel<<<dim3(rank, M), 256, 0, as_stream(stream)>>>(d_x, d_A, K, rank, d_t);
    CMLB_LAUNCH_CHECK();
    lora_up_kernel<<<dim3((N + 255) / 256, M), 256, 0, as_stream(stream)>>>(d_t, d_B, N, rank, scaling, d_y);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
