/*
 * cml_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C CPU restatement of the C-ML algorithms on the quantized-LLM path
 * (block dequantisation, NF4, the quantized Linear forward, the LLaMA forward
 * pass, paged attention, the LoRA layer and the per-tensor 8-bit quantisers). It exists only so that the CUDA path can be checked against
 * it; nothing shipped may call it. Every function cites the C-ML file:line it
 * restates (paths relative to the C-ML source tree).
 *
 * Parity status: PINNED. The test-suite compares every function here
 *   (a) with the compiled C-ML reference itself (oracle/_ref/libcml_ref.so,
 *       through oracle/ref_driver.c) whenever that library is present, and
 *   (b) with stored vectors in tests/golden/ that were produced by running
 *       that compiled reference (tests/golden/make_golden.py), and
 *   (c) with the single-block known answers of C-ML's tests/test_gguf_quant.c.
 *
 * All entry points take flat pointers so the tests can drive them via ctypes.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_Q4_0 2
#define ORC_Q8_0 7

/* ---- fp16 -> fp32 (src/core/gguf_quant.c:14-58) -------------------------
 * Widening of IEEE binary16 as C-ML does it: exact for normals, zeros, inf and
 * NaN (payload shifted into the fp32 mantissa). For subnormals C-ML shifts the
 * mantissa up to bit 10 and then counts one more shift (:35-36), which yields
 * exponent 112 - lz instead of the IEEE 113 - lz: a subnormal half widens to
 * exactly half its IEEE value. That behaviour is kept here on purpose. */
float orc_fp16_to_fp32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            int lz = 0;
            while (!(m & 0x400u)) { m <<= 1; lz++; }
            m &= 0x3FFu;
            bits = sign | ((uint32_t)(112 - lz) << 23) | (m << 13);
        }
    } else if (e == 31) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* fp32 -> fp16, round-to-nearest-even. The reference has no such routine on
 * this path (its test helper truncates, tests/test_gguf_quant.c:11-26); the
 * synthetic-model writer needs a correct one to create scales. */
uint16_t orc_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);        /* rounds to inf */
    if (ax < 0x33000001u) return (uint16_t)sign;                      /* rounds to 0 */
    int e = (int)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t half = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) half++;
    uint32_t out;
    if (e < -14) out = half;                       /* subnormal (may carry into normal) */
    else out = ((uint32_t)(e + 15) << 10) + (half - 0x400u);
    return (uint16_t)(sign | out);
}

/* ---- GGUF block dequantisation ------------------------------------------
 * Q8_0 block = fp16 d + 32 int8 (34 B); y = (float)q * d
 *   (include/core/gguf_quant.h:27-31, src/core/gguf_quant.c:114-125).
 * Q4_0 block = fp16 d + 16 B; byte j -> element j (low nibble) and j+16
 *   (high nibble); y = (float)(nib - 8) * d
 *   (include/core/gguf_quant.h:14-18, src/core/gguf_quant.c:66-82). */
void orc_dequant_q8_0(const uint8_t* blocks, float* dst, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t* p = blocks + b * 34;
        uint16_t dh;
        memcpy(&dh, p, 2);
        float d = orc_fp16_to_fp32(dh);
        const int8_t* q = (const int8_t*)(p + 2);
        for (int j = 0; j < 32; j++) dst[b * 32 + j] = (float)q[j] * d;
    }
}

void orc_dequant_q4_0(const uint8_t* blocks, float* dst, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t* p = blocks + b * 18;
        uint16_t dh;
        memcpy(&dh, p, 2);
        float d = orc_fp16_to_fp32(dh);
        for (int j = 0; j < 16; j++) {
            int lo = p[2 + j] & 15, hi = p[2 + j] >> 4;
            dst[b * 32 + j] = (float)(lo - 8) * d;
            dst[b * 32 + j + 16] = (float)(hi - 8) * d;
        }
    }
}

/* The block types beside Q4_0 / Q8_0 that the reference reads.
 * Q4_1 (include/core/gguf_quant.h:20-25, src/core/gguf_quant.c:90-112): fp16 d, fp16 m, 16 bytes
 *   packed like Q4_0; y = (float)nibble * d + m. */
static float orc_half_at(const uint8_t* p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return orc_fp16_to_fp32(h);
}

void orc_dequant_q4_1(const uint8_t* blocks, float* dst, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t* p = blocks + b * 20;
        const float d = orc_half_at(p), m = orc_half_at(p + 2);
        for (int j = 0; j < 16; j++) {
            dst[b * 32 + j] = (float)(p[4 + j] & 15) * d + m;
            dst[b * 32 + j + 16] = (float)(p[4 + j] >> 4) * d + m;
        }
    }
}

/* 6-bit scale and min of sub-block i of a Q4_K / Q5_K super-block from its 12 packed bytes
 * (src/core/gguf_quant.c:162-171): the first four pairs sit in the low 6 bits of bytes i and
 * i + 4; the last four take a nibble of byte i + 4 and the top two bits of bytes i - 4 and i. */
static void orc_k_scale_min(const uint8_t* s, int i, int* sc, int* mn) {
    if (i < 4) { *sc = s[i] & 63; *mn = s[i + 4] & 63; return; }
    *sc = (s[i + 4] & 15) | ((s[i - 4] >> 6) << 4);
    *mn = (s[i + 4] >> 4) | ((s[i] >> 6) << 4);
}

/* Q4_K (gguf_quant.h:34-39, gguf_quant.c:151-196) and Q5_K (gguf_quant.h:41-47,
 * gguf_quant.c:211-270): 256 elements = 8 sub-blocks of 32; sub-block i keeps its nibbles in
 * qs[16i .. 16i+15], element k in the low and k + 16 in the high nibble (the reference's own
 * order); Q5_K adds bit e of the 256-bit field qh as bit 4; y = q * (d * sc) - dmin * mn. */
static void orc_dequant_q45_k(const uint8_t* blocks, float* dst, size_t nblocks, int five) {
    const size_t bb = five ? 176 : 144;
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t* p = blocks + b * bb;
        const float d = orc_half_at(p), dmin = orc_half_at(p + 2);
        const uint8_t* qh = p + 16;
        const uint8_t* qs = p + (five ? 48 : 16);
        for (int e = 0; e < 256; e++) {
            const int i = e >> 5, k = e & 31;
            int sc, mn;
            orc_k_scale_min(p + 4, i, &sc, &mn);
            const uint8_t byte = qs[i * 16 + (k & 15)];
            int q = k < 16 ? (byte & 15) : (byte >> 4);
            if (five) q |= ((qh[e >> 3] >> (e & 7)) & 1) << 4;
            const float scale = d * (float)sc, minv = dmin * (float)mn;
            dst[b * 256 + e] = (float)q * scale - minv;
        }
    }
}

/* Q6_K (gguf_quant.h:49-54, gguf_quant.c:283-311): ql[128] low nibbles (even element in the low
 * half), qh[64] two high bits each, 16 int8 sub-block scales, fp16 d last;
 * y = d * scale[e / 16] * (q6 - 32). */
void orc_dequant_q6_k(const uint8_t* blocks, float* dst, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t* p = blocks + b * 210;
        const float d = orc_half_at(p + 208);
        for (int e = 0; e < 256; e++) {
            const int low4 = (e & 1) ? (p[e >> 1] >> 4) : (p[e >> 1] & 15);
            const int high2 = (p[128 + (e >> 2)] >> (2 * (e & 3))) & 3;
            const float sc = (float)(int8_t)p[192 + (e >> 4)];
            dst[b * 256 + e] = d * sc * (float)((low4 | (high2 << 4)) - 32);
        }
    }
}

/* Dispatcher with the reference's error contract (src/core/gguf_quant.c:351-391):
 * -1 for NULL pointers, numel == 0, a type without a block size, or numel not
 * a multiple of the block size (32; 256 for the K types). */
int orc_gguf_dequantize(int type, const void* src, float* dst, size_t numel) {
    if (!src || !dst || numel == 0) return -1;
    const uint8_t* s = (const uint8_t*)src;
    switch (type) {
        case ORC_Q4_0: if (numel % 32) return -1; orc_dequant_q4_0(s, dst, numel / 32); return 0;
        case ORC_Q8_0: if (numel % 32) return -1; orc_dequant_q8_0(s, dst, numel / 32); return 0;
        case 3: if (numel % 32) return -1; orc_dequant_q4_1(s, dst, numel / 32); return 0;
        case 12: if (numel % 256) return -1; orc_dequant_q45_k(s, dst, numel / 256, 0); return 0;
        case 13: if (numel % 256) return -1; orc_dequant_q45_k(s, dst, numel / 256, 1); return 0;
        case 14: if (numel % 256) return -1; orc_dequant_q6_k(s, dst, numel / 256); return 0;
        default: return -1;
    }
}

/* Q4_0 / Q8_0 quantisers. C-ML has none (its GGUF writer cannot emit
 * quantized tensors, src/core/gguf.c:47-56); these follow the public GGML
 * definition (absmax / -8 for Q4_0, absmax / 127 for Q8_0) and only serve to
 * make synthetic models. Parity is defined on dequantisation, not on these. */
void orc_quantize_q4_0(const float* x, uint8_t* blocks, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++) {
        float amax = 0.f, vmax = 0.f;
        for (int j = 0; j < 32; j++) {
            float v = x[b * 32 + j];
            if (fabsf(v) > amax) { amax = fabsf(v); vmax = v; }
        }
        float d = vmax / -8.0f;
        uint16_t dh = orc_fp32_to_fp16(d);
        float id = d != 0.f ? 1.0f / d : 0.f;
        uint8_t* p = blocks + b * 18;
        memcpy(p, &dh, 2);
        for (int j = 0; j < 16; j++) {
            int q0 = (int)(x[b * 32 + j] * id + 8.5f);
            int q1 = (int)(x[b * 32 + j + 16] * id + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            if (q0 < 0) q0 = 0;
            if (q1 < 0) q1 = 0;
            p[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

void orc_quantize_q8_0(const float* x, uint8_t* blocks, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++) {
        float amax = 0.f;
        for (int j = 0; j < 32; j++) if (fabsf(x[b * 32 + j]) > amax) amax = fabsf(x[b * 32 + j]);
        float d = amax / 127.0f;
        uint16_t dh = orc_fp32_to_fp16(d);
        float id = d != 0.f ? 1.0f / d : 0.f;
        uint8_t* p = blocks + b * 34;
        memcpy(p, &dh, 2);
        for (int j = 0; j < 32; j++) {
            float r = roundf(x[b * 32 + j] * id);
            if (r > 127.f) r = 127.f;
            if (r < -127.f) r = -127.f;
            p[2 + j] = (uint8_t)(int8_t)r;
        }
    }
}

/* ---- NF4 ------------------------------------------------------------------
 * Code book: the 16 four-decimal literals of src/core/quantization.c:195-198. */
const float ORC_NF4_TABLE[16] = {
    -1.0f, -0.6962f, -0.5251f, -0.3949f, -0.2844f, -0.1848f, -0.0911f, 0.0f,
    0.0796f, 0.1609f, 0.2461f, 0.3379f, 0.4407f, 0.5626f, 0.7230f, 1.0f};

/* src/core/quantization.c:213-312: per-block absmax (floored at 1e-10),
 * x/absmax clamped to [-1,1], nearest code by linear scan where the first
 * minimum wins (:200-211), even element in the HIGH nibble (:303-305).
 * packed has (numel+1)/2 bytes, scales has ceil(numel/block) floats. */
int orc_nf4_quantize(const float* x, size_t numel, int block, uint8_t* packed, float* scales) {
    if (!x || !packed || !scales || numel == 0 || block <= 0) return -1;
    size_t nb = (numel + (size_t)block - 1) / (size_t)block;
    for (size_t b = 0; b < nb; b++) {
        size_t s = b * (size_t)block, e = s + (size_t)block;
        if (e > numel) e = numel;
        float amax = 0.f;
        for (size_t i = s; i < e; i++) if (fabsf(x[i]) > amax) amax = fabsf(x[i]);
        scales[b] = amax < 1e-10f ? 1e-10f : amax;
    }
    size_t nbytes = (numel + 1) / 2;
    memset(packed, 0, nbytes);
    for (size_t i = 0; i < numel; i++) {
        float v = x[i] / scales[i / (size_t)block];
        if (v > 1.f) v = 1.f;
        if (v < -1.f) v = -1.f;
        int best = 0;
        float bd = fabsf(v - ORC_NF4_TABLE[0]);
        for (int c = 1; c < 16; c++) {
            float dd = fabsf(v - ORC_NF4_TABLE[c]);
            if (dd < bd) { bd = dd; best = c; }
        }
        if (i & 1) packed[i / 2] |= (uint8_t)best;
        else packed[i / 2] |= (uint8_t)(best << 4);
    }
    return (int)nb;
}

/* src/core/quantization.c:314-370: out[e] = TABLE[idx] * scales[min(e/block,
 * num_scales-1)]; element 2i is the high nibble of byte i. */
int orc_nf4_dequantize(const uint8_t* packed, const float* scales, int num_scales, int block,
                       size_t numel, float* out) {
    if (!packed || !scales || !out || num_scales <= 0 || block <= 0 || numel == 0) return -1;
    for (size_t e = 0; e < numel; e++) {
        uint8_t byte = packed[e / 2];
        int idx = (e & 1) ? (byte & 15) : (byte >> 4);
        size_t bi = e / (size_t)block;
        if (bi >= (size_t)num_scales) bi = (size_t)num_scales - 1;
        out[e] = ORC_NF4_TABLE[idx] * scales[bi];
    }
    return 0;
}

/* ---- y = x . W^T with W stored [N,K], fp32, k summed in order -------------
 * src/nn/qlora.c:309-317, src/distributed/tensor_parallel.c:9-22,
 * src/ops/ir/execution.c:3109-3122 (scalar UOP_LINEAR). */
void orc_linear_nt(const float* x, const float* W, int M, int N, int K, float* y) {
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            float s = 0.f;
            const float* xr = x + (size_t)i * K;
            const float* wr = W + (size_t)j * K;
            for (int k = 0; k < K; k++) s += xr[k] * wr[k];
            y[(size_t)i * N + j] = s;
        }
}

/* y = x . W with W stored [K,N] (the llama.c orientation, src/nn/llama.c:464-466;
 * scalar UOP_MATMUL src/ops/ir/execution.c:1030-1051 sums k in order within
 * 32-wide tiles, which for one output element is still ascending k). */
void orc_matmul_nn(const float* x, const float* W, int M, int K, int N, float* y) {
    for (int i = 0; i < M; i++) {
        float* yr = y + (size_t)i * N;
        for (int j = 0; j < N; j++) yr[j] = 0.f;
        for (int k = 0; k < K; k++) {
            float xv = x[(size_t)i * K + k];
            const float* wr = W + (size_t)k * N;
            for (int j = 0; j < N; j++) yr[j] += xv * wr[j];
        }
    }
}

/* ---- quantized Linear forward (src/nn/qlora.c:240-365) --------------------
 * y = x . dequant(W)^T + scaling * (x . A^T) . B^T, all fp32, k in order.
 * W is NF4 over the flat [out,in] index. lora_A/lora_B may be NULL (rank 0). */
int orc_qlora_forward(const float* x, int M, int in_f, int out_f, const uint8_t* packed,
                      const float* scales, int num_scales, int block, const float* A,
                      const float* B, int rank, float scaling, float* y) {
    size_t numel = (size_t)in_f * out_f;
    float* W = (float*)malloc(numel * sizeof(float));
    if (!W) return -1;
    if (orc_nf4_dequantize(packed, scales, num_scales, block, numel, W)) { free(W); return -1; }
    orc_linear_nt(x, W, M, out_f, in_f, y);
    free(W);
    if (A && B && rank > 0) {
        float* t = (float*)malloc((size_t)M * rank * sizeof(float));
        if (!t) return -1;
        orc_linear_nt(x, A, M, rank, in_f, t);
        for (int b = 0; b < M; b++)
            for (int o = 0; o < out_f; o++) {
                float s = 0.f;
                for (int r = 0; r < rank; r++) s += t[b * rank + r] * B[o * rank + r];
                y[(size_t)b * out_f + o] += scaling * s;
            }
        free(t);
    }
    return 0;
}

/* ---- LLaMA pieces ----------------------------------------------------------
 * RMSNorm: x * (1/sqrt(mean(x^2)+eps)) * w, eps added before the sqrt
 * (src/nn/llama.c:71-124). */
void orc_rmsnorm(const float* x, const float* w, int rows, int dim, float eps, float* out) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * dim;
        float ss = 0.f;
        for (int i = 0; i < dim; i++) ss += xr[i] * xr[i];
        float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int i = 0; i < dim; i++) out[(size_t)r * dim + i] = xr[i] * inv * w[i];
    }
}

/* RoPE on a 2-D [seq, width] tensor (src/nn/llm_ops.c:702-805, 2-D branch
 * :785-802): interleaved pairs (2i,2i+1), freq = 1/powf(base, 2i/dim),
 * theta = (start_pos+s)*freq. all_heads == 0 reproduces what llama.c gets by
 * passing [seq, heads*head_dim] (src/nn/llama.c:483-484): only the first
 * head_dim columns of each row rotate. all_heads != 0 rotates every head. */
void orc_rope(float* x, int seq, int width, int head_dim, int start_pos, float base,
              int all_heads) {
    if (base <= 0.f) base = 10000.0f;
    int heads = all_heads ? width / head_dim : 1;
    for (int s = 0; s < seq; s++)
        for (int h = 0; h < heads; h++) {
            float* v = x + (size_t)s * width + (size_t)h * head_dim;
            for (int i = 0; i < head_dim / 2; i++) {
                float freq = 1.0f / powf(base, (float)(2 * i) / (float)head_dim);
                float th = (float)(start_pos + s) * freq;
                float c = cosf(th), sn = sinf(th);
                float a = v[2 * i], b = v[2 * i + 1];
                v[2 * i] = a * c - b * sn;
                v[2 * i + 1] = a * sn + b * c;
            }
        }
}

/* Grouped-query attention over a dense cache (src/nn/llm_ops.c:194-361):
 * scores = q.k * 1/sqrt(head_dim); causal mask -1e9 where sk > sq + mask_off;
 * softmax with max subtraction (:9-28); out = P.V.  mask_off = 0 reproduces
 * the reference's relative-index mask (:290-298); mask_off = start_pos is the
 * position-correct mask. K/V: [kv_len, kv_heads*head_dim]; Q: [seq, heads*hd]. */
int orc_gqa(const float* q, const float* k, const float* v, int seq, int kv_len, int heads,
            int kv_heads, int hd, int mask_off, float* out) {
    if (heads <= 0 || kv_heads <= 0 || hd <= 0 || heads % kv_heads) return -1;
    int groups = heads / kv_heads;
    float scale = 1.0f / sqrtf((float)hd);
    float* sc = (float*)malloc((size_t)kv_len * sizeof(float));
    if (!sc) return -1;
    for (int h = 0; h < heads; h++) {
        int kh = h / groups;
        for (int sq = 0; sq < seq; sq++) {
            const float* qv = q + ((size_t)sq * heads + h) * hd;
            for (int sk = 0; sk < kv_len; sk++) {
                const float* kv = k + ((size_t)sk * kv_heads + kh) * hd;
                float d = 0.f;
                for (int i = 0; i < hd; i++) d += qv[i] * kv[i];
                sc[sk] = (sk > sq + mask_off) ? -1e9f : d * scale;
            }
            float mx = sc[0];
            for (int sk = 1; sk < kv_len; sk++) if (sc[sk] > mx) mx = sc[sk];
            float sum = 0.f;
            for (int sk = 0; sk < kv_len; sk++) { sc[sk] = expf(sc[sk] - mx); sum += sc[sk]; }
            if (sum > 0.f) {
                float inv = 1.0f / sum;
                for (int sk = 0; sk < kv_len; sk++) sc[sk] *= inv;
            }
            float* o = out + ((size_t)sq * heads + h) * hd;
            for (int i = 0; i < hd; i++) {
                float a = 0.f;
                for (int sk = 0; sk < kv_len; sk++) a += sc[sk] * v[((size_t)sk * kv_heads + kh) * hd + i];
                o[i] = a;
            }
        }
    }
    free(sc);
    return 0;
}

/* Paged attention of one sequence (src/nn/paged_attention.c:332-480): the keys and values of the
 * sequence's blocks, walked in block-table order, are its tokens 0..kv_len-1 (here already
 * gathered: K/V [kv_len, kv_heads*hd]); query row sq sits at absolute position
 * kv_len - seq_q + sq (:425-433); score = dot * scale, masked ones become -1e9 (:418-436), softmax
 * with max subtraction (:9-29), out += p * v in token order (:441-460). scale <= 0 means
 * 1/sqrt(hd) (:381-384). */
int orc_paged_gqa(const float* q, const float* k, const float* v, int seq_q, int kv_len, int heads,
                  int kv_heads, int hd, float scale, int causal, float* out) {
    if (heads <= 0 || kv_heads <= 0 || hd <= 0 || heads % kv_heads || kv_len <= 0 || seq_q <= 0) return -1;
    int groups = heads / kv_heads;
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)hd);
    float* sc = (float*)malloc((size_t)kv_len * sizeof(float));
    if (!sc) return -1;
    for (int h = 0; h < heads; h++) {
        int kh = h / groups;
        for (int sq = 0; sq < seq_q; sq++) {
            const float* qv = q + ((size_t)sq * heads + h) * hd;
            int abs_pos = kv_len - seq_q + sq;
            for (int sk = 0; sk < kv_len; sk++) {
                const float* kv = k + ((size_t)sk * kv_heads + kh) * hd;
                float d = 0.f;
                for (int i = 0; i < hd; i++) d += qv[i] * kv[i];
                sc[sk] = (causal && sk > abs_pos) ? -1e9f : d * scale;
            }
            float mx = sc[0];
            for (int sk = 1; sk < kv_len; sk++) if (sc[sk] > mx) mx = sc[sk];
            float sum = 0.f;
            for (int sk = 0; sk < kv_len; sk++) { sc[sk] = expf(sc[sk] - mx); sum += sc[sk]; }
            if (sum > 0.f) {
                float inv = 1.0f / sum;
                for (int sk = 0; sk < kv_len; sk++) sc[sk] *= inv;
            }
            float* o = out + ((size_t)sq * heads + h) * hd;
            for (int i = 0; i < hd; i++) o[i] = 0.f;
            for (int sk = 0; sk < kv_len; sk++)
                for (int i = 0; i < hd; i++) o[i] += sc[sk] * v[((size_t)sk * kv_heads + kh) * hd + i];
        }
    }
    free(sc);
    return 0;
}

static float orc_silu(float g) { return g / (1.0f + expf(-g)); } /* src/ops/ir/execution.c:2980-2987 */

/* A LLaMA model as flat fp32 arrays, in the reference's orientation: every
 * projection is [in, out] and is applied as x . W (include/nn/llama.h:31-69). */
typedef struct {
    int vocab, hidden, inter, layers, heads, kv_heads, max_seq;
    float rope_theta, eps;
    const float* embed;             /* [vocab, hidden] */
    const float* final_norm;        /* [hidden] */
    const float* lm_head;           /* [hidden, vocab] */
    const float* const* wq;         /* per layer [hidden, heads*hd] */
    const float* const* wk;         /* [hidden, kv_heads*hd] */
    const float* const* wv;
    const float* const* wo;         /* [heads*hd, hidden] */
    const float* const* wgate;      /* [hidden, inter] */
    const float* const* wup;
    const float* const* wdown;      /* [inter, hidden] */
    const float* const* norm1;      /* [hidden] */
    const float* const* norm2;
    float* kcache;                  /* [layers, max_seq, kv_heads*hd] */
    float* vcache;
    int cur_len;
    int rope_all_heads;             /* 0 = reference behaviour, 1 = every head */
    int mask_absolute;              /* 0 = reference behaviour, 1 = offset by start_pos */
} OrcLlama;

/* cml_llama_forward (src/nn/llama.c:550-612) with cml_llama_layer_forward
 * (:454-548) and swiglu_ffn (:126-155) inlined. Writes logits [seq, vocab];
 * returns 0, or -1 on bad arguments / cache overflow (src/nn/llm_ops.c:133-137). */
int orc_llama_forward(OrcLlama* m, const int* tokens, int seq, float* logits) {
    if (!m || !tokens || seq <= 0 || !m->embed) return -1;
    int H = m->hidden, hd = H / m->heads, qw = m->heads * hd, kvw = m->kv_heads * hd, I = m->inter;
    int start = m->cur_len;
    if (start + seq > m->max_seq) return -1;
    size_t sH = (size_t)seq * H;
    float* h = (float*)malloc(sH * 4);
    float* nrm = (float*)malloc(sH * 4);
    float* q = (float*)malloc((size_t)seq * qw * 4);
    float* kk = (float*)malloc((size_t)seq * kvw * 4);
    float* vv = (float*)malloc((size_t)seq * kvw * 4);
    float* att = (float*)malloc((size_t)seq * qw * 4);
    float* prj = (float*)malloc(sH * 4);
    float* g = (float*)malloc((size_t)seq * I * 4);
    float* u = (float*)malloc((size_t)seq * I * 4);
    if (!h || !nrm || !q || !kk || !vv || !att || !prj || !g || !u) return -1;
    for (int s = 0; s < seq; s++) {
        int t = tokens[s];
        if (t < 0 || t >= m->vocab) t = 0;           /* src/nn/llama.c:440-444 */
        memcpy(h + (size_t)s * H, m->embed + (size_t)t * H, (size_t)H * 4);
    }
    for (int l = 0; l < m->layers; l++) {
        orc_rmsnorm(h, m->norm1[l], seq, H, m->eps, nrm);
        orc_matmul_nn(nrm, m->wq[l], seq, H, qw, q);
        orc_matmul_nn(nrm, m->wk[l], seq, H, kvw, kk);
        orc_matmul_nn(nrm, m->wv[l], seq, H, kvw, vv);
        orc_rope(q, seq, qw, hd, start, m->rope_theta, m->rope_all_heads);
        orc_rope(kk, seq, kvw, hd, start, m->rope_theta, m->rope_all_heads);
        float* kc = m->kcache + (size_t)l * m->max_seq * kvw;
        float* vc = m->vcache + (size_t)l * m->max_seq * kvw;
        memcpy(kc + (size_t)start * kvw, kk, (size_t)seq * kvw * 4);
        memcpy(vc + (size_t)start * kvw, vv, (size_t)seq * kvw * 4);
        if (orc_gqa(q, kc, vc, seq, start + seq, m->heads, m->kv_heads, hd,
                    m->mask_absolute ? start : 0, att)) return -1;
        orc_matmul_nn(att, m->wo[l], seq, qw, H, prj);
        for (size_t i = 0; i < sH; i++) h[i] += prj[i];
        orc_rmsnorm(h, m->norm2[l], seq, H, m->eps, nrm);
        orc_matmul_nn(nrm, m->wgate[l], seq, H, I, g);
        orc_matmul_nn(nrm, m->wup[l], seq, H, I, u);
        for (size_t i = 0; i < (size_t)seq * I; i++) g[i] = orc_silu(g[i]) * u[i];
        orc_matmul_nn(g, m->wdown[l], seq, I, H, prj);
        for (size_t i = 0; i < sH; i++) h[i] += prj[i];
    }
    if (m->final_norm) { orc_rmsnorm(h, m->final_norm, seq, H, m->eps, nrm); memcpy(h, nrm, sH * 4); }
    orc_matmul_nn(h, m->lm_head, seq, H, m->vocab, logits);
    m->cur_len = start + seq;
    free(h); free(nrm); free(q); free(kk); free(vv); free(att); free(prj); free(g); free(u);
    return 0;
}

/* Greedy pick: first index holding the strict maximum (src/nn/llama.c:650-660). */
int orc_argmax_first(const float* v, int n) {
    int best = 0;
    for (int i = 1; i < n; i++) if (v[i] > v[best]) best = i;
    return best;
}

/* ---- tensor parallel (src/distributed/tensor_parallel.c) -------------------
 * column shard = rows [r*N/tp,(r+1)*N/tp) of W[N,K] (:65-79); row shard =
 * columns [r*K/tp,(r+1)*K/tp) (:80-101); reduce = sum of partials in rank
 * order (:468-479). Returns -1 when the split is not even (:46-53). */
int orc_tp_shard(const float* W, int rows, int cols, int dim, int tp, int rank, float* out) {
    if (!W || !out || tp <= 0 || rank < 0 || rank >= tp || (dim != 0 && dim != 1)) return -1;
    if (dim == 0) {
        if (rows % tp) return -1;
        int sr = rows / tp;
        memcpy(out, W + (size_t)rank * sr * cols, (size_t)sr * cols * 4);
    } else {
        if (cols % tp) return -1;
        int sc = cols / tp;
        for (int r = 0; r < rows; r++)
            memcpy(out + (size_t)r * sc, W + (size_t)r * cols + (size_t)rank * sc, (size_t)sc * 4);
    }
    return 0;
}

void orc_tp_allreduce_sum(const float* const* parts, int nparts, size_t numel, float* out) {
    for (size_t i = 0; i < numel; i++) out[i] = 0.f;
    for (int p = 0; p < nparts; p++)
        for (size_t i = 0; i < numel; i++) out[i] += parts[p][i];
}

/* ---- LoRA over an fp32 weight (src/nn/lora.c:105-273) ----------------------
 * y[b][o] = sum_i x[b][i] W[o][i]  (+ scaling * sum_r (sum_i x[b][i] A[r][i]) B[o][r] unless merged),
 * every sum in fp32, ascending index, as C-ML's loops. t: M * rank floats of scratch. */
void orc_lora_forward(const float* x, int M, int K, int N, const float* W, const float* A, const float* B, int rank,
                      float scaling, int merged, float* t, float* y) {
    for (int b = 0; b < M; b++)
        for (int o = 0; o < N; o++) {
            float s = 0.0f;
            for (int i = 0; i < K; i++) s += x[(size_t)b * K + i] * W[(size_t)o * K + i];
            y[(size_t)b * N + o] = s;
        }
    if (merged) return;
    for (int b = 0; b < M; b++)
        for (int r = 0; r < rank; r++) {
            float s = 0.0f;
            for (int i = 0; i < K; i++) s += x[(size_t)b * K + i] * A[(size_t)r * K + i];
            t[(size_t)b * rank + r] = s;
        }
    for (int b = 0; b < M; b++)
        for (int o = 0; o < N; o++) {
            float s = 0.0f;
            for (int r = 0; r < rank; r++) s += t[(size_t)b * rank + r] * B[(size_t)o * rank + r];
            y[(size_t)b * N + o] += scaling * s;
        }
}
/* src/nn/lora.c:263-273: W[o][i] += scaling * sum_r B[o][r] A[r][i] */
void orc_lora_merge(float* W, const float* A, const float* B, int N, int K, int rank, float scaling) {
    for (int o = 0; o < N; o++)
        for (int i = 0; i < K; i++) {
            float s = 0.0f;
            for (int r = 0; r < rank; r++) s += B[(size_t)o * rank + r] * A[(size_t)r * K + i];
            W[(size_t)o * K + i] += scaling * s;
        }
}

/* ---- per-tensor affine 8-bit quantisation (src/core/quantization.c:8-192) ----
 * params_out = {scale bits, zero_point}. mode 0: symmetric int8 parameters, 1: asymmetric int8
 * (zero point shifted by -128), 2: the uint8 mapping of [min, max] onto 0..255. */
void orc_quant_params(const float* x, size_t n, int mode, int32_t* params_out) {
    float lo = 3.402823466e+38f, hi = -3.402823466e+38f, scale;
    int32_t zp = 0;
    for (size_t i = 0; i < n; i++) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
    }
    if (mode == 0) {
        scale = fmaxf(fabsf(lo), fabsf(hi)) / 127.0f;
    } else {
        scale = (hi - lo) / 255.0f;
        if (scale < 1e-10f) scale = 1e-10f;
        zp = (int32_t)roundf(-lo / scale) - (mode == 1 ? 128 : 0);
    }
    if (scale < 1e-10f) scale = 1e-10f;
    memcpy(&params_out[0], &scale, 4);
    params_out[1] = zp;
}
/* q = clamp(round(v / scale) + zero_point). Where the quotient leaves the int32 range C-ML's cast is
 * undefined; the compiled x86 reference yields INT_MIN there and wraps the addition, restated here
 * without undefined behaviour. */
void orc_quantize8(const float* x, size_t n, float scale, int32_t zero_point, int is_unsigned, uint8_t* q) {
    const int32_t lo = is_unsigned ? 0 : -128, hi = is_unsigned ? 255 : 127;
    for (size_t i = 0; i < n; i++) {
        const float r = roundf(x[i] / scale);
        const int32_t c = (r >= -2147483648.0f && r < 2147483648.0f) ? (int32_t)r : INT32_MIN;
        int32_t v = (int32_t)((uint32_t)c + (uint32_t)zero_point);
        v = v < lo ? lo : (v > hi ? hi : v);
        q[i] = (uint8_t)v;
    }
}
void orc_dequantize8(const uint8_t* q, size_t n, float scale, int32_t zero_point, int is_unsigned, float* out) {
    for (size_t i = 0; i < n; i++) {
        const float v = is_unsigned ? (float)q[i] : (float)(int8_t)q[i];
        out[i] = (v - (float)zero_point) * scale;
    }
}
