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
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int r = blockIdx.x;
    int t = tokens[r];
    if (t < 0 || t >= vocab) t = 0;
    const __half* src = table + (size_t)t * hidden;
    float* dst = out + (size_t)r * hidden;
    if ((hidden & 7) == 0) {                               // 16 bytes of fp16 in, 32 bytes of fp32 out per thread and pass
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < hidden; i += gridDim.y * blockDim.x * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + i);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&v.z)), d = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
            *reinterpret_cast<float4*>(dst + i) = make_float4(a.x, a.y, b.x, b.y);
            *reinterpret_cast<float4*>(dst + i + 4) = make_float4(c.x, c.y, d.x, d.y);
        }
    } else {
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) dst[i] = __half2float(src[i]);
    }
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

// The same for rows of up to 8192 elements with dim % 4 == 0 (every LLaMA width): the row is read
// once with 16-byte loads and stays in registers between the sum of squares and the scaling; bf16
// results leave as 8-byte stores.
template <bool BF16_OUT>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, const __half* __restrict__ w, int dim, float eps, void* out) {
    __shared__ float red[8];
    const int r = blockIdx.x, nv = dim >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * dim);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < nv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) tot += red[k];
    const float inv = 1.0f / sqrtf(tot / (float)dim + eps);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < nv) {
            const uint2 wv = reinterpret_cast<const uint2*>(w)[i];
            const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&wv.x)), w23 = __half22float2(*reinterpret_cast<const __half2*>(&wv.y));
            const float a = v[j].x * inv * w01.x, b = v[j].y * inv * w01.y, c = v[j].z * inv * w23.x, d = v[j].w * inv * w23.y;
            if (BF16_OUT) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                reinterpret_cast<uint2*>(out)[(size_t)r * nv + i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            } else {
                reinterpret_cast<float4*>(out)[(size_t)r * nv + i] = make_float4(a, b, c, d);
            }
        }
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
// Launch with programmatic stream serialization: the kernel may become resident while its
// predecessor drains; every kernel launched this way starts with griddepcontrol.wait.
template <typename Kern, typename... Args>
static cudaError_t launch_dep(Kern kern, dim3 grid, dim3 block, cudaStream_t st, Args... args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.stream = st; cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

constexpr int ATT_THREADS = 128;
template <typename KV, int HD>
__global__ void __launch_bounds__(ATT_THREADS)
attention_partial_kernel(const float* __restrict__ q, const KV* __restrict__ kc, const KV* __restrict__ vc,
                         const int* __restrict__ row_seq, const int* __restrict__ row_limit, int heads, int kv_heads,
                         int max_seq, int chunk, float* __restrict__ partial, int q_stride) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
    for (int i = 0; i < PER; i++) qv[i] = q[(size_t)r * q_stride + (size_t)h * HD + lane + 32 * i];
    float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;
    // A warp takes KB consecutive keys per step and requests all their K and V rows before it
    // consumes any, so one memory round trip serves KB keys.
    constexpr int KB = 8;
    for (int sk0 = k_begin + warp * KB; sk0 < k_end; sk0 += NW * KB) {
        float kr[KB][PER], vr[KB][PER];
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const int sk = min(sk0 + j, k_end - 1);
            const KV* kp = kc + base + (size_t)sk * kvw;
            const KV* vp = vc + base + (size_t)sk * kvw;
#pragma unroll
            for (int i = 0; i < PER; i++) { kr[j][i] = (float)kp[lane + 32 * i]; vr[j][i] = (float)vp[lane + 32 * i]; }
        }
        float d[KB];
        float bm = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB; j++) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++) t = fmaf(qv[i], kr[j][i], t);
            d[j] = (sk0 + j < k_end) ? warp_sum(t) * scale : -INFINITY;
            bm = fmaxf(bm, d[j]);
        }
        const float mn = fmaxf(m, bm);
        const float corr = expf(m - mn);
        l *= corr;
#pragma unroll
        for (int i = 0; i < PER; i++) acc[i] *= corr;
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const float p = expf(d[j] - mn);               // exp(-inf) = 0 for keys past the end
            l += p;
#pragma unroll
            for (int i = 0; i < PER; i++) acc[i] = fmaf(p, vr[j][i], acc[i]);
        }
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

// Combines the splits of one (row, head). blockDim = HD. With xq != NULL the head's HD outputs are
// also written as activation digits (HD/32 block records) for the output projection that follows.
template <int HD>
__global__ void attention_merge_kernel(const float* __restrict__ partial, int nsplit, float* __restrict__ out,
                                       uint32_t* __restrict__ xq, int heads) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t rh = blockIdx.x;                      // row * heads + head
    const float* p = partial + rh * nsplit * (HD + 2);
    float gm = -INFINITY;
    for (int s = 0; s < nsplit; s++) gm = fmaxf(gm, p[s * (HD + 2)]);
    float l = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ms = p[s * (HD + 2)];
        if (ms != -INFINITY) l += p[s * (HD + 2) + 1] * expf(ms - gm);
    }
    const int i = threadIdx.x;
    float a = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ms = p[s * (HD + 2)];
        if (ms != -INFINITY) a = fmaf(p[s * (HD + 2) + 2 + i], expf(ms - gm), a);
    }
    const float v = a / l;
    out[rh * HD + i] = v;
    if (xq) {
        const size_t row = rh / heads, h = rh % heads;
        const size_t blk = (row * heads + h) * (HD / 32) + (i >> 5);     // block index within [rows][heads*HD/32]
        xq_emit_warp(v, i & 31, xq + blk * kXqWords);
    }
}

// RoPE on the Q and K parts of a fused [rows][q|k|v] buffer, then K and V into the cache
// (cml_rope_forward src/nn/llm_ops.c:702-805 + cml_kv_cache_append :118-157 in one pass).
// rotate_heads = 1 rotates only head 0 of Q and of K (C-ML's behaviour), -1 rotates all.
template <typename KV>
__global__ void qkv_rope_append_kernel(float* __restrict__ qkv, int stride, const int* __restrict__ row_seq,
                                       const int* __restrict__ row_pos, int heads, int kv_heads, int hd, float base,
                                       int rotate_all, int rotate_any, KV* __restrict__ kc, KV* __restrict__ vc, int max_seq) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // grid = (rows, groups of 32 heads), block = (hd/2 pairs, 4): thread (i, y) owns pair i of heads
    // y, y+4, ... of its group (Q heads, then K heads, then V heads) and computes the rotation of
    // its pair once for all of them
    const int r = blockIdx.x, i = threadIdx.x;
    const int qw = heads * hd, kvw = kv_heads * hd, total = heads + 2 * kv_heads;
    float* row = qkv + (size_t)r * stride;
    const int pos = row_pos[r];
    const size_t dst = ((size_t)row_seq[r] * max_seq + pos) * kvw;
    float c = 1.f, sn = 0.f;
    if (rotate_any) {
        const float freq = 1.0f / powf(base, (float)(2 * i) / (float)hd);
        const float th = (float)pos * freq;
        c = cosf(th); sn = sinf(th);
    }
    for (int hh = blockIdx.y * 32 + threadIdx.y; hh < min(total, (int)blockIdx.y * 32 + 32); hh += 4) {
        if (hh >= heads + kv_heads) {                               // V head: straight copy into the cache
            const int h = hh - heads - kv_heads;
            const float* v = row + qw + kvw + (size_t)h * hd + 2 * i;
            vc[dst + (size_t)h * hd + 2 * i] = (KV)v[0];
            vc[dst + (size_t)h * hd + 2 * i + 1] = (KV)v[1];
            continue;
        }
        const bool is_k = hh >= heads;
        const int h = is_k ? hh - heads : hh;
        float* v = row + (is_k ? qw : 0) + (size_t)h * hd + 2 * i;
        float a = v[0], b = v[1];
        if (rotate_any && (rotate_all || h == 0)) {
            const float na = a * c - b * sn, nb = a * sn + b * c;
            a = na; b = nb;
            v[0] = a; v[1] = b;
        }
        if (is_k) {
            kc[dst + (size_t)h * hd + 2 * i] = (KV)a;
            kc[dst + (size_t)h * hd + 2 * i + 1] = (KV)b;
        }
    }
}

// ---- decode attention in one launch: RoPE of the new token's Q and K, cache append, split-KV
// attention and the merge of the splits (cml_rope_forward src/nn/llm_ops.c:702-805,
// cml_kv_cache_append :118-157, cml_gqa_forward :243-372 for one new token per sequence).
// grid = (heads, rows, splits), 128 threads. Every CTA rotates its own head of Q; the CTA whose
// key range holds the new token's position takes that key and value from the q|k|v buffer (rotated,
// rounded to the cache type) instead of the cache, and the first Q head of each KV group also
// writes them into the cache for later steps, so no CTA reads a cache row another CTA writes.
// Each CTA leaves an unnormalised partial (max, sum, acc[hd]); the last CTA of a (row, head) to
// arrive (atomic counter, reset for the next launch) merges the splits in split order.
// Requires that all other attended keys are in the cache already: one row per sequence.
// cos/sin of every rotation pair at each row's position: cs[row][i] = (cos, sin)(pos * base^(-2i/hd)),
// computed once per decode step and read by every layer's attention launch.
__global__ void rope_table_kernel(const int* __restrict__ row_pos, int hd, float base, float2* __restrict__ cs) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int r = blockIdx.x, i = threadIdx.x;
    if (i < hd / 2) {
        const float freq = 1.0f / powf(base, (float)(2 * i) / (float)hd);
        const float th = (float)row_pos[r] * freq;
        cs[(size_t)r * (hd / 2) + i] = make_float2(cosf(th), sinf(th));
    }
}

constexpr int ATTD_THREADS = 128;
constexpr int ATTD_MAX_SPLITS = 256;       // key splits per (row, head) the merge has room for
template <typename KV, int HD>
__global__ void __launch_bounds__(ATTD_THREADS)
attention_decode_kernel(const float* __restrict__ qkv, int stride, KV* __restrict__ kc, KV* __restrict__ vc,
                        const int* __restrict__ row_seq, const int* __restrict__ row_pos, const int* __restrict__ row_limit,
                        int heads, int kv_heads, int max_seq, int chunk, const float2* __restrict__ rope_cs,
                        float* __restrict__ partial, unsigned int* __restrict__ counters, float* __restrict__ out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int PER = HD / 32;                       // contiguous head-dim elements per lane
    constexpr int NW = ATTD_THREADS / 32;
    const int h = blockIdx.x, r = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qw = heads * HD, kvw = kv_heads * HD, group = heads / kv_heads;
    const int kh = h / group;
    const int limit = row_limit[r], pos = row_pos[r];
    const int k_begin = split * chunk, k_end = min(limit + 1, k_begin + chunk);
    const size_t base = (size_t)row_seq[r] * max_seq * kvw + (size_t)kh * HD;
    const float* row = qkv + (size_t)r * stride;
    const bool has_new = pos >= k_begin && pos < k_end;           // the new token's key belongs to this CTA

    __shared__ float qs[HD], knew[HD], vnew[HD];
    __shared__ float sm[NW], sl[NW], sacc[NW][HD];
    __shared__ unsigned int s_last;
    if (threadIdx.x < HD / 2) {
        const int i = threadIdx.x;
        const float2 cs = rope_cs[(size_t)r * (HD / 2) + i];
        const float c = cs.x, sn = cs.y;
        const float2 qp = *reinterpret_cast<const float2*>(row + (size_t)h * HD + 2 * i);
        const float scale = 1.0f / sqrtf((float)HD);
        qs[2 * i] = (qp.x * c - qp.y * sn) * scale;
        qs[2 * i + 1] = (qp.x * sn + qp.y * c) * scale;
        if (has_new) {
            const float2 kp = *reinterpret_cast<const float2*>(row + qw + (size_t)kh * HD + 2 * i);
            const float2 vp = *reinterpret_cast<const float2*>(row + qw + kvw + (size_t)kh * HD + 2 * i);
            const KV k0 = (KV)(kp.x * c - kp.y * sn), k1 = (KV)(kp.x * sn + kp.y * c);
            const KV v0 = (KV)vp.x, v1 = (KV)vp.y;
            knew[2 * i] = (float)k0; knew[2 * i + 1] = (float)k1;
            vnew[2 * i] = (float)v0; vnew[2 * i + 1] = (float)v1;
            if (h % group == 0) {
                const size_t dst = base + (size_t)pos * kvw;
                kc[dst + 2 * i] = k0; kc[dst + 2 * i + 1] = k1;
                vc[dst + 2 * i] = v0; vc[dst + 2 * i + 1] = v1;
            }
        }
    }
    __syncthreads();
    float qv[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) qv[i] = qs[lane * PER + i];
    float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;
    // A warp takes KB consecutive keys per step and requests all their K and V rows (one vector load
    // per lane and row) before it consumes any; with a chunk of 32 keys every warp makes one step.
    constexpr int KB = 8;
    for (int sk0 = k_begin + warp * KB; sk0 < k_end; sk0 += NW * KB) {
        float kr[KB][PER], vr[KB][PER];
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const int sk = min(sk0 + j, k_end - 1);
            const KV* kp = kc + base + (size_t)sk * kvw + lane * PER;
            const KV* vp = vc + base + (size_t)sk * kvw + lane * PER;
            if (sizeof(KV) == 2 && PER == 4) {
                const uint2 ku = *reinterpret_cast<const uint2*>(kp), vu = *reinterpret_cast<const uint2*>(vp);
                const float2 k01 = __half22float2(*reinterpret_cast<const __half2*>(&ku.x)), k23 = __half22float2(*reinterpret_cast<const __half2*>(&ku.y));
                const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&vu.x)), v23 = __half22float2(*reinterpret_cast<const __half2*>(&vu.y));
                kr[j][0] = k01.x; kr[j][1] = k01.y; kr[j][2 % PER] = k23.x; kr[j][3 % PER] = k23.y;
                vr[j][0] = v01.x; vr[j][1] = v01.y; vr[j][2 % PER] = v23.x; vr[j][3 % PER] = v23.y;
            } else {
#pragma unroll
                for (int i = 0; i < PER; i++) { kr[j][i] = (float)kp[i]; vr[j][i] = (float)vp[i]; }
            }
            if (sk == pos) {                            // the row being written by another CTA: take the values from the buffer
#pragma unroll
                for (int i = 0; i < PER; i++) { kr[j][i] = knew[lane * PER + i]; vr[j][i] = vnew[lane * PER + i]; }
            }
        }
        float d[KB];
        float bm = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB; j++) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++) t = fmaf(qv[i], kr[j][i], t);
            d[j] = (sk0 + j < k_end) ? warp_sum(t) : -INFINITY;
            bm = fmaxf(bm, d[j]);
        }
        const float mn = fmaxf(m, bm);
        const float corr = expf(m - mn);
        l *= corr;
#pragma unroll
        for (int i = 0; i < PER; i++) acc[i] *= corr;
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const float p = expf(d[j] - mn);               // exp(-inf) = 0 for keys past the end
            l += p;
#pragma unroll
            for (int i = 0; i < PER; i++) acc[i] = fmaf(p, vr[j][i], acc[i]);
        }
        m = mn;
    }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int i = 0; i < PER; i++) sacc[warp][lane * PER + i] = acc[i];
    __syncthreads();
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; w++) gm = fmaxf(gm, sm[w]);
    const size_t rh = (size_t)r * heads + h;
    float* mine = partial + (rh * nsplit + split) * (HD + 2);
    if (threadIdx.x < HD) {
        float a = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float c = (sm[w] == -INFINITY) ? 0.f : expf(sm[w] - gm);
            a = fmaf(sacc[w][threadIdx.x], c, a);
            lt = fmaf(sl[w], c, lt);
        }
        mine[2 + threadIdx.x] = a;
        if (threadIdx.x == 0) { mine[0] = gm; mine[1] = lt; }
    }
    // ---- the last split of this (row, head) to finish merges all of them. The barrier orders the
    // CTA's partial before thread 0's release-acquire increment, which publishes it (cumulativity) and,
    // in the last CTA, makes the other splits' partials visible to the threads behind the next barrier.
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counters + rh) : "memory");
        s_last = (old == (unsigned)nsplit - 1) ? 1u : 0u;
        if (s_last) counters[rh] = 0u;                  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    // Two rounds of loads, each issued as one batch: the splits' (max, sum) pairs by one thread each,
    // then every output element's share of all splits.
    const float* p = partial + rh * nsplit * (HD + 2);
    __shared__ float s_w[ATTD_MAX_SPLITS], s_l[ATTD_MAX_SPLITS];
    for (int s2 = threadIdx.x; s2 < nsplit; s2 += ATTD_THREADS) {
        s_w[s2] = __ldcg(p + s2 * (HD + 2));
        s_l[s2] = __ldcg(p + s2 * (HD + 2) + 1);
    }
    __syncthreads();
    float mg = -INFINITY;
    for (int s2 = 0; s2 < nsplit; s2++) mg = fmaxf(mg, s_w[s2]);
    __syncthreads();
    for (int s2 = threadIdx.x; s2 < nsplit; s2 += ATTD_THREADS) s_w[s2] = (s_w[s2] == -INFINITY) ? 0.f : expf(s_w[s2] - mg);
    __syncthreads();
    if (threadIdx.x < HD) {
        float a = 0.f, lg = 0.f;
        int s2 = 0;
        for (; s2 + 8 <= nsplit; s2 += 8) {
            float as[8];
#pragma unroll
            for (int k = 0; k < 8; k++) as[k] = __ldcg(p + (s2 + k) * (HD + 2) + 2 + threadIdx.x);
#pragma unroll
            for (int k = 0; k < 8; k++) { a = fmaf(as[k], s_w[s2 + k], a); lg = fmaf(s_l[s2 + k], s_w[s2 + k], lg); }
        }
        float as[8];
#pragma unroll
        for (int k = 0; k < 8; k++) as[k] = (s2 + k < nsplit) ? __ldcg(p + (s2 + k) * (HD + 2) + 2 + threadIdx.x) : 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (s2 + k < nsplit) { a = fmaf(as[k], s_w[s2 + k], a); lg = fmaf(s_l[s2 + k], s_w[s2 + k], lg); }
        out[rh * HD + threadIdx.x] = a / lg;
    }
}

// ---- greedy pick: first index holding the strict maximum of each row
__device__ __forceinline__ void argmax_take(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }          // first index of the strict maximum; NaN never wins
}
__device__ __forceinline__ void argmax_warp(float& bv, int& bi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(bv, bi, ov, oi);
    }
}
// One cluster of ARGMAX_CTAS CTAs per row: every CTA scans a contiguous slice of the row with
// 16-byte loads, the slice winners meet in the shared memory of the cluster's first CTA
// (distributed shared memory), which picks the row's winner. No global scratch, fixed order.
constexpr int ARGMAX_CTAS = 8, ARGMAX_THREADS = 256;
__global__ void __cluster_dims__(ARGMAX_CTAS, 1, 1) __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out, float2* __restrict__ out_pair, int index_offset) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float sv[ARGMAX_THREADS / 32];
    __shared__ int si[ARGMAX_THREADS / 32];
    __shared__ float cv[ARGMAX_CTAS];
    __shared__ int ci[ARGMAX_CTAS];
    const int part = blockIdx.x % ARGMAX_CTAS, r = blockIdx.x / ARGMAX_CTAS;
    const float* row = logits + (size_t)r * vocab;
    const int per = ((vocab + ARGMAX_CTAS - 1) / ARGMAX_CTAS + 3) & ~3;
    const int lo = min(vocab, part * per), hi = min(vocab, lo + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if ((vocab & 3) == 0 && ((uintptr_t)row & 15) == 0) {
        for (int i = lo + threadIdx.x * 4; i < hi; i += ARGMAX_THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            argmax_take(bv, bi, v.x, i); argmax_take(bv, bi, v.y, i + 1);
            argmax_take(bv, bi, v.z, i + 2); argmax_take(bv, bi, v.w, i + 3);
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) argmax_take(bv, bi, row[i], i);
    }
    argmax_warp(bv, bi);
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < ARGMAX_THREADS / 32 ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < ARGMAX_THREADS / 32 ? si[threadIdx.x] : 0x7fffffff;
        argmax_warp(bv, bi);
        if (threadIdx.x == 0) {                            // this slice's winner into slot `part` of CTA 0's arrays
            uint32_t dv, di;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dv) : "r"((uint32_t)__cvta_generic_to_shared(&cv[part])), "r"(0));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(di) : "r"((uint32_t)__cvta_generic_to_shared(&ci[part])), "r"(0));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dv), "f"(bv) : "memory");
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(di), "r"(bi) : "memory");
        }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (part == 0 && threadIdx.x < 32) {
        bv = threadIdx.x < ARGMAX_CTAS ? cv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < ARGMAX_CTAS ? ci[threadIdx.x] : 0x7fffffff;
        argmax_warp(bv, bi);
        if (threadIdx.x == 0) {
            if (out) out[r] = (bi == 0x7fffffff) ? 0 : bi;
            // (value, global index) of this slice of a vocabulary split over ranks; an empty result keeps -inf
            if (out_pair) out_pair[r] = make_float2(bv, __int_as_float(bi == 0x7fffffff ? 0x7fffffff : bi + index_offset));
        }
    }
}

// Winner per row among `parts` (value, index) candidates laid out [part][row]: greatest value, lowest
// index among equals (the candidates come from consecutive slices of one row, so this is the row's
// first strict maximum).
__global__ void argmax_merge_kernel(const float2* __restrict__ pairs, int parts, int rows, int* __restrict__ out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int q = 0; q < parts; q++) {
        const float2 c = pairs[(size_t)q * rows + r];
        argmax_take(bv, bi, c.x, __float_as_int(c.y));
    }
    out[r] = (bi == 0x7fffffff) ? 0 : bi;
}

// dst[row][part * w + j] = src[part][row][j]: the slices of a row gathered from all ranks, side by side.
__global__ void gather_columns_kernel(const float* __restrict__ src, int parts, int rows, int w, float* __restrict__ dst) {
    const size_t total = (size_t)parts * rows * w, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int j = (int)(i % w), row = (int)((i / w) % rows), part = (int)(i / ((size_t)w * rows));
        dst[((size_t)row * parts + part) * w + j] = src[i];
    }
}


// ---- row bookkeeping kept on the device so that a decode step can be replayed as a CUDA graph
// mode 0: sequence `seq`, `rows` consecutive positions starting at cur_len[seq] (prefill / single decode)
// mode 1: `rows` sequences, one token each at cur_len[b] (batched decode)
// relative_mask != 0 reproduces C-ML's causal mask on call-relative indices (llm_ops.c:290-298).
__global__ void prepare_rows_kernel(const int* __restrict__ cur_len, int rows, int mode, int relative_mask, int seq,
                                    int* row_seq, int* row_pos, int* row_limit) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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

// Merging a LoRA pair into an fp32 weight (src/nn/lora.c:263-273): W[o][i] += scaling * sum_r B[o][r] * A[r][i],
// one thread per weight, r ascending as in C-ML's loop.
__global__ void lora_merge_kernel(float* __restrict__ W, const float* __restrict__ A, const float* __restrict__ B, int out_f, int in_f,
                                  int rank, float scaling) {
    const size_t n = (size_t)out_f * in_f, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        const size_t o = e / in_f, i = e % in_f;
        float s = 0.f;
        for (int r = 0; r < rank; r++) s = fmaf(B[o * rank + r], A[(size_t)r * in_f + i], s);
        W[e] = fmaf(scaling, s, W[e]);
    }
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
    const int slices = hidden >= 4096 ? 2 : 1;             // two CTAs per row once a row is 8 KB of fp16
    CMLB_CUDA(launch_dep(embed_kernel, dim3(rows, slices), dim3(256), as_stream(stream), (const __half*)d_table_f16, d_tokens, hidden, vocab, d_out));
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_rmsnorm(const float* d_x, const uint16_t* d_w_f16, int rows, int dim, float eps, float* d_out_f32,
                               uint16_t* d_out_bf16, void* stream) {
    CMLB_REQUIRE(d_x && d_w_f16 && (d_out_f32 || d_out_bf16) && rows > 0 && dim > 0, "cmlb200_rmsnorm: bad argument");
    const bool vec = dim % 4 == 0 && dim <= 8192 && ((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_w_f16 & 7) == 0 &&
                     (d_out_bf16 ? ((uintptr_t)d_out_bf16 & 7) == 0 : ((uintptr_t)d_out_f32 & 15) == 0);
    if (vec && d_out_bf16) rmsnorm_vec_kernel<true><<<rows, 256, 0, as_stream(stream)>>>(d_x, (const __half*)d_w_f16, dim, eps, d_out_bf16);
    else if (vec) rmsnorm_vec_kernel<false><<<rows, 256, 0, as_stream(stream)>>>(d_x, (const __half*)d_w_f16, dim, eps, d_out_f32);
    else if (d_out_bf16) rmsnorm_kernel<true><<<rows, 256, 0, as_stream(stream)>>>(d_x, (const __half*)d_w_f16, dim, eps, d_out_bf16);
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

static int attention_impl(const float* d_q, int q_stride, const void* d_kcache, const void* d_vcache, const int* d_row_seq,
                          const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq,
                          int max_limit, int kv_is_f32, float* d_out, uint32_t* d_xq, float* d_scratch, int splits, void* stream) {
    CMLB_REQUIRE(d_q && d_kcache && d_vcache && d_row_seq && d_row_limit && d_out && d_scratch, "cmlb200_attention: NULL argument");
    CMLB_REQUIRE(rows > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "cmlb200_attention: num_heads (%d) must be divisible by num_kv_heads (%d)", heads, kv_heads);
    CMLB_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 32, "cmlb200_attention: head_dim %d not in {32, 64, 128}", head_dim);
    CMLB_REQUIRE(splits >= 1 && max_limit >= 0 && max_limit < max_seq, "cmlb200_attention: bad splits/max_limit");
    const int chunk = (max_limit + 1 + splits - 1) / splits;
    dim3 grid(heads, rows, splits);
    cudaStream_t st = as_stream(stream);
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t c1 = {}, c2 = {};
    c1.gridDim = grid; c1.blockDim = dim3(ATT_THREADS); c1.stream = st; c1.attrs = pdl; c1.numAttrs = 1;
    c2.gridDim = dim3(rows * heads); c2.blockDim = dim3(head_dim); c2.stream = st; c2.attrs = pdl; c2.numAttrs = 1;
#define ATT_LAUNCH(KV, HD)                                                                                               \
    CMLB_CUDA(cudaLaunchKernelEx(&c1, attention_partial_kernel<KV, HD>, d_q, (const KV*)d_kcache, (const KV*)d_vcache,  \
                                 d_row_seq, d_row_limit, heads, kv_heads, max_seq, chunk, d_scratch, q_stride));        \
    CMLB_CUDA(cudaLaunchKernelEx(&c2, attention_merge_kernel<HD>, (const float*)d_scratch, splits, d_out, d_xq, heads))
    if (kv_is_f32) {
        if (head_dim == 128) { ATT_LAUNCH(float, 128); } else if (head_dim == 64) { ATT_LAUNCH(float, 64); } else { ATT_LAUNCH(float, 32); }
    } else {
        if (head_dim == 128) { ATT_LAUNCH(__half, 128); } else if (head_dim == 64) { ATT_LAUNCH(__half, 64); } else { ATT_LAUNCH(__half, 32); }
    }
#undef ATT_LAUNCH
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_attention(const float* d_q, const void* d_kcache, const void* d_vcache, const int* d_row_seq,
                                 const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq,
                                 int max_limit, int kv_is_f32, float* d_out, float* d_scratch, int splits, void* stream) {
    return attention_impl(d_q, heads * head_dim, d_kcache, d_vcache, d_row_seq, d_row_limit, rows, heads, kv_heads, head_dim,
                          max_seq, max_limit, kv_is_f32, d_out, nullptr, d_scratch, splits, stream);
}

// Same with Q rows `q_stride` floats apart (Q inside a fused q|k|v buffer) and, when d_xq is not
// NULL, the attention output also written as activation digits for cmlb200_gemv_xq.
extern "C" int cmlb200_attention_ex(const float* d_q, int q_stride, const void* d_kcache, const void* d_vcache,
                                    const int* d_row_seq, const int* d_row_limit, int rows, int heads, int kv_heads,
                                    int head_dim, int max_seq, int max_limit, int kv_is_f32, float* d_out, void* d_xq,
                                    float* d_scratch, int splits, void* stream) {
    CMLB_REQUIRE(q_stride >= heads * head_dim, "cmlb200_attention_ex: q_stride %d smaller than a row of Q", q_stride);
    return attention_impl(d_q, q_stride, d_kcache, d_vcache, d_row_seq, d_row_limit, rows, heads, kv_heads, head_dim, max_seq,
                          max_limit, kv_is_f32, d_out, (uint32_t*)d_xq, d_scratch, splits, stream);
}

// Scratch of cmlb200_attention_decode: 16 KB of per-(row, head) arrival counters (rows*heads <= 4096),
// then the partials.
constexpr size_t kAttCounterBytes = 16384;
extern "C" size_t cmlb200_attention_decode_scratch_bytes(int rows, int heads, int head_dim, int splits) {
    return kAttCounterBytes + cmlb200_attention_scratch_floats(rows, heads, head_dim, splits) * sizeof(float);
}

// (cos, sin) of every rotation pair at each row's position: d_cs[rows][head_dim/2][2], for
// cmlb200_attention_decode. One launch per decode step serves all layers.
extern "C" int cmlb200_rope_table(const int* d_row_pos, int rows, int head_dim, float base, float* d_cs, void* stream) {
    CMLB_REQUIRE(d_row_pos && d_cs && rows > 0 && head_dim > 0 && head_dim % 2 == 0 && head_dim <= 2048, "cmlb200_rope_table: bad argument");
    if (base <= 0.f) base = 10000.0f;
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows); cfg.blockDim = dim3((head_dim / 2 + 31) / 32 * 32); cfg.stream = as_stream(stream); cfg.attrs = pdl; cfg.numAttrs = 1;
    CMLB_CUDA(cudaLaunchKernelEx(&cfg, rope_table_kernel, d_row_pos, head_dim, base, reinterpret_cast<float2*>(d_cs)));
    return CMLB200_OK;
}

// Decode attention for rows that are one new token per sequence: d_qkv holds [rows][q|k|v] as the
// projection left it (row_stride floats apart, nothing rotated yet). Rotates Q and K of every head
// with the (cos, sin) table of cmlb200_rope_table for the same row_pos, appends K and V to the cache, attends keys 0..row_limit (row_limit[r] >= row_pos[r]
// is not required, but the new key is only used when row_pos[r] <= row_limit[r]) and writes
// [rows][heads*head_dim] fp32. d_scratch: cmlb200_attention_decode_scratch_bytes bytes whose
// first 16 KB (the counters) are zero before the first call; the kernel leaves them zero.
extern "C" int cmlb200_attention_decode(const float* d_qkv, int row_stride, void* d_kcache, void* d_vcache, const int* d_row_seq,
                                        const int* d_row_pos, const int* d_row_limit, int rows, int heads, int kv_heads,
                                        int head_dim, int max_seq, int max_limit, int kv_is_f32, const float* d_rope_cs, float* d_out,
                                        void* d_scratch, int splits, void* stream) {
    CMLB_REQUIRE(d_qkv && d_kcache && d_vcache && d_row_seq && d_row_pos && d_row_limit && d_rope_cs && d_out && d_scratch, "cmlb200_attention_decode: NULL argument");
    CMLB_REQUIRE(rows > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "cmlb200_attention_decode: num_heads (%d) must be divisible by num_kv_heads (%d)", heads, kv_heads);
    CMLB_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 32, "cmlb200_attention_decode: head_dim %d not in {32, 64, 128}", head_dim);
    CMLB_REQUIRE(row_stride >= (heads + 2 * kv_heads) * head_dim, "cmlb200_attention_decode: row_stride %d smaller than a q|k|v row", row_stride);
    CMLB_REQUIRE(splits >= 1 && splits <= ATTD_MAX_SPLITS && max_limit >= 0 && max_limit < max_seq, "cmlb200_attention_decode: bad splits/max_limit (splits <= 256)");
    const int chunk = (max_limit + 1 + splits - 1) / splits;
    CMLB_REQUIRE((size_t)rows * heads * sizeof(unsigned int) <= kAttCounterBytes, "cmlb200_attention_decode: rows*heads = %d exceeds 4096", rows * heads);
    unsigned int* counters = static_cast<unsigned int*>(d_scratch);
    float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(d_scratch) + kAttCounterBytes);
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t c1 = {};
    c1.gridDim = dim3(heads, rows, splits); c1.blockDim = dim3(ATTD_THREADS); c1.stream = as_stream(stream); c1.attrs = pdl; c1.numAttrs = 1;
#define ATT_LAUNCH(KV, HD)                                                                                                    \
    CMLB_CUDA(cudaLaunchKernelEx(&c1, attention_decode_kernel<KV, HD>, d_qkv, row_stride, (KV*)d_kcache, (KV*)d_vcache, d_row_seq, \
                                 d_row_pos, d_row_limit, heads, kv_heads, max_seq, chunk, reinterpret_cast<const float2*>(d_rope_cs), partial, counters, d_out))
    if (kv_is_f32) {
        if (head_dim == 128) { ATT_LAUNCH(float, 128); } else if (head_dim == 64) { ATT_LAUNCH(float, 64); } else { ATT_LAUNCH(float, 32); }
    } else {
        if (head_dim == 128) { ATT_LAUNCH(__half, 128); } else if (head_dim == 64) { ATT_LAUNCH(__half, 64); } else { ATT_LAUNCH(__half, 32); }
    }
#undef ATT_LAUNCH
    return CMLB200_OK;
}

extern "C" int cmlb200_qkv_rope_append(float* d_qkv, int row_stride, const int* d_row_seq, const int* d_row_pos, int rows,
                                       int heads, int kv_heads, int head_dim, float base, int rotate_heads, void* d_kcache,
                                       void* d_vcache, int max_seq, int kv_is_f32, void* stream) {
    CMLB_REQUIRE(d_qkv && d_row_seq && d_row_pos && d_kcache && d_vcache, "cmlb200_qkv_rope_append: NULL argument");
    CMLB_REQUIRE(rows > 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && head_dim % 2 == 0 && max_seq > 0 &&
                     row_stride >= (heads + 2 * kv_heads) * head_dim,
                 "cmlb200_qkv_rope_append: bad shape");
    if (base <= 0.f) base = 10000.0f;
    cudaLaunchConfig_t cfg = {};
    CMLB_REQUIRE(head_dim <= 512, "cmlb200_qkv_rope_append: head_dim %d above 512", head_dim);
    cfg.gridDim = dim3(rows, (heads + 2 * kv_heads + 31) / 32);
    cfg.blockDim = dim3(head_dim / 2, 4);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int rotate_any = rotate_heads != 0, rotate_all = rotate_heads < 0;
    if (kv_is_f32)
        CMLB_CUDA(cudaLaunchKernelEx(&cfg, qkv_rope_append_kernel<float>, d_qkv, row_stride, d_row_seq, d_row_pos, heads, kv_heads,
                                     head_dim, base, rotate_all, rotate_any, (float*)d_kcache, (float*)d_vcache, max_seq));
    else
        CMLB_CUDA(cudaLaunchKernelEx(&cfg, qkv_rope_append_kernel<__half>, d_qkv, row_stride, d_row_seq, d_row_pos, heads, kv_heads,
                                     head_dim, base, rotate_all, rotate_any, (__half*)d_kcache, (__half*)d_vcache, max_seq));
    return CMLB200_OK;
}

extern "C" int cmlb200_argmax(const float* d_logits, int rows, int vocab, int* d_out, void* stream) {
    CMLB_REQUIRE(d_logits && d_out && rows > 0 && vocab > 0, "cmlb200_argmax: bad argument");
    CMLB_CUDA(launch_dep(argmax_kernel, dim3(rows * ARGMAX_CTAS), dim3(ARGMAX_THREADS), as_stream(stream), d_logits, vocab, d_out, (float2*)nullptr, 0));
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_argmax_slice(const float* d_logits, int rows, int width, int index_offset, float* d_pairs, void* stream) {
    CMLB_REQUIRE(d_logits && d_pairs && rows > 0 && width > 0 && index_offset >= 0, "cmlb200_argmax_slice: bad argument");
    CMLB_CUDA(launch_dep(argmax_kernel, dim3(rows * ARGMAX_CTAS), dim3(ARGMAX_THREADS), as_stream(stream), d_logits, width, (int*)nullptr,
                         reinterpret_cast<float2*>(d_pairs), index_offset));
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_argmax_merge(const float* d_pairs, int parts, int rows, int* d_out, void* stream) {
    CMLB_REQUIRE(d_pairs && d_out && parts > 0 && rows > 0, "cmlb200_argmax_merge: bad argument");
    CMLB_CUDA(launch_dep(argmax_merge_kernel, dim3((rows + 63) / 64), dim3(64), as_stream(stream), reinterpret_cast<const float2*>(d_pairs), parts, rows, d_out));
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_gather_columns(const float* d_src, int parts, int rows, int width, float* d_dst, void* stream) {
    CMLB_REQUIRE(d_src && d_dst && parts > 0 && rows > 0 && width > 0, "cmlb200_gather_columns: bad argument");
    const size_t total = (size_t)parts * rows * width;
    gather_columns_kernel<<<(unsigned)min((size_t)2368, (total + 255) / 256), 256, 0, as_stream(stream)>>>(d_src, parts, rows, width, d_dst);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_prepare_rows(const int* d_cur_len, int rows, int mode, int relative_mask, int seq, int* d_row_seq,
                                    int* d_row_pos, int* d_row_limit, void* stream) {
    CMLB_REQUIRE(d_cur_len && d_row_seq && d_row_pos && d_row_limit && rows > 0 && seq >= 0, "cmlb200_prepare_rows: bad argument");
    CMLB_CUDA(launch_dep(prepare_rows_kernel, dim3((rows + 127) / 128), dim3(128), as_stream(stream), d_cur_len, rows, mode, relative_mask, seq, d_row_seq, d_row_pos, d_row_limit));
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_advance_rows(int* d_cur_len, int rows, int mode, int seq, void* stream) {
    CMLB_REQUIRE(d_cur_len && rows > 0 && seq >= 0, "cmlb200_advance_rows: bad argument");
    CMLB_CUDA(launch_dep(advance_rows_kernel, dim3((rows + 127) / 128), dim3(128), as_stream(stream), d_cur_len, rows, mode, seq));
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
extern "C" int cmlb200_lora_merge(float* d_W, const float* d_A, const float* d_B, int out_features, int in_features, int rank, float scaling,
                                  void* stream) {
    CMLB_REQUIRE(d_W && d_A && d_B && out_features > 0 && in_features > 0 && rank > 0, "cmlb200_lora_merge: bad argument");
    lora_merge_kernel<<<ew_grid((size_t)out_features * in_features), 256, 0, as_stream(stream)>>>(d_W, d_A, d_B, out_features, in_features, rank, scaling);
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
