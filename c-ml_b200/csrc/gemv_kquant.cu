// Decode GEMV over the GGUF block types C-ML reads besides Q4_0 / Q8_0: Q4_1, Q4_K, Q5_K, Q6_K
// (src/core/gguf_quant.c:90-112, 151-196, 211-270, 283-311), straight from the file's bytes:
// y[M, N] (= | +=) x[M, K] . dequant(W[N, K])^T with fp32 accumulation. Replaces "dequantise the
// tensor to fp32 (src/core/gguf.c:271-295), then multiply" for weights of those types.
//
// The weight is the tensor's block stream unchanged, row n at byte n * (K / BS) * BB. One warp owns
// one output row; a lane takes 8 consecutive elements per step ("octet"), so the 32 lanes of a step
// cover exactly one 256-element K-block (or eight Q4_1 blocks): its header is one broadcast load,
// its quants one coalesced load. Q4_K / Q5_K follow C-ML's own nibble order (each 32-element
// sub-block in 16 consecutive bytes, src/core/gguf_quant.c:174-187), not ggml's. CUDA cores, bound by
// instruction issue (about 8 + M instructions per weight element against 0.56-0.82 bytes).
#include "common.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1 };
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kSegMaxFloats = 12288;   // activation floats staged per K segment (48 KB)

template <int GTYPE> struct KQ;
template <> struct KQ<3> { static constexpr int BS = 32, BB = 20; };
template <> struct KQ<12> { static constexpr int BS = 256, BB = 144; };
template <> struct KQ<13> { static constexpr int BS = 256, BB = 176; };
template <> struct KQ<14> { static constexpr int BS = 256, BB = 210; };

__device__ __forceinline__ float h2f(uint32_t bits) { return cml_half_to_float((uint16_t)(bits & 0xFFFFu)); }

// 6-bit scale and minimum of sub-block i from the 12 packed bytes in (s0, s1, s2) = bytes 0-3, 4-7, 8-11
// (get_scale_min_k4, src/core/gguf_quant.c:131-149)
__device__ __forceinline__ void scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int i, int& sc, int& mn) {
    const int sh = 8 * (i & 3);
    const uint32_t a = (s0 >> sh) & 255u, b = (s1 >> sh) & 255u, c = (s2 >> sh) & 255u;
    if (i < 4) { sc = (int)(a & 63u); mn = (int)(b & 63u); }
    else { sc = (int)((c & 15u) | ((a >> 6) << 4)); mn = (int)((c >> 4) | ((b >> 6) << 4)); }
}

// The 8 weights of octet o of a row: elements 8o .. 8o+7.
template <int GTYPE>
__device__ __forceinline__ void decode8(const uint8_t* __restrict__ row, int o, float (&w)[8]) {
    if (GTYPE == 3) {                                        // d, m, 16 bytes: byte j = element j (low) and j + 16 (high)
        const uint8_t* p = row + (size_t)(o >> 2) * 20;
        const int t = o & 3, sh = (t >> 1) * 4;
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(p);
        const float d = h2f(dm), m = h2f(dm >> 16);
        const uint32_t q0 = *reinterpret_cast<const uint32_t*>(p + 4 + 8 * (t & 1)), q1 = *reinterpret_cast<const uint32_t*>(p + 8 + 8 * (t & 1));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            w[j] = (float)((q0 >> (8 * j + sh)) & 15u) * d + m;
            w[4 + j] = (float)((q1 >> (8 * j + sh)) & 15u) * d + m;
        }
    } else if (GTYPE == 12 || GTYPE == 13) {                 // d, dmin, scales[12], (qh[32],) qs[128]
        const uint8_t* p = row + (size_t)(o >> 5) * KQ<GTYPE>::BB;
        const int l = o & 31, i = l >> 2, t = l & 3, sh = (t >> 1) * 4;
        const uint4 hdr = *reinterpret_cast<const uint4*>(p);
        int sc, mn;
        scale_min(hdr.y, hdr.z, hdr.w, i, sc, mn);
        const float scale = h2f(hdr.x) * (float)sc, mnv = h2f(hdr.x >> 16) * (float)mn;
        const uint2 qv = *reinterpret_cast<const uint2*>(p + (GTYPE == 12 ? 16 : 48) + i * 16 + 8 * (t & 1));
        const uint32_t hb = GTYPE == 13 ? (uint32_t)p[16 + l] : 0u;   // bit j = fifth bit of element 8l + j
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t qa = (qv.x >> (8 * j + sh)) & 15u, qb = (qv.y >> (8 * j + sh)) & 15u;
            if (GTYPE == 13) { qa |= ((hb >> j) & 1u) << 4; qb |= ((hb >> (4 + j)) & 1u) << 4; }
            w[j] = (float)qa * scale - mnv;
            w[4 + j] = (float)qb * scale - mnv;
        }
    } else {                                                 // ql[128], qh[64], scales[16] (int8), d; blocks are only 2-byte aligned
        const uint8_t* p = row + (size_t)(o >> 5) * 210;
        const int l = o & 31;
        const uint16_t* ql16 = reinterpret_cast<const uint16_t*>(p + 4 * l);
        const uint32_t ql = (uint32_t)ql16[0] | ((uint32_t)ql16[1] << 16);                 // nibble j = low 4 bits of element 8l + j
        const uint32_t qh = *reinterpret_cast<const uint16_t*>(p + 128 + 2 * l);            // 2 bits per element
        const float ds = h2f(*reinterpret_cast<const uint16_t*>(p + 208)) * (float)(int)(int8_t)p[192 + (l >> 1)];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int q = (int)(((ql >> (4 * j)) & 15u) | (((qh >> (2 * j)) & 3u) << 4));
            w[j] = ds * (float)(q - 32);
        }
    }
}

template <int GTYPE, int MT, int EPI>
__global__ void __launch_bounds__(kThreads)
gemv_kq_kernel(const uint8_t* __restrict__ blocks, const float* __restrict__ x, float* __restrict__ y, int N, int K, int kseg) {
    extern __shared__ __align__(16) float xs[];   // [MT][kseg]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row_bytes = (size_t)(K / KQ<GTYPE>::BS) * KQ<GTYPE>::BB;
    for (int g0 = blockIdx.x * kWarps; g0 < N; g0 += gridDim.x * kWarps) {
        const int n = g0 + warp;
        const uint8_t* row = blocks + (size_t)min(n, N - 1) * row_bytes;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.f;
        for (int k0 = 0; k0 < K; k0 += kseg) {
            const int klen = min(kseg, K - k0);
            __syncthreads();
            for (int m = 0; m < MT; m++)
                for (int i = threadIdx.x * 4; i < klen; i += kThreads * 4)
                    *reinterpret_cast<float4*>(xs + m * kseg + i) = *reinterpret_cast<const float4*>(x + (size_t)m * K + k0 + i);
            __syncthreads();
            if (n < N) {
#pragma unroll 2
                for (int o = lane; o < klen / 8; o += 32) {
                    float w[8];
                    decode8<GTYPE>(row, k0 / 8 + o, w);
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float4 xa = *reinterpret_cast<const float4*>(xs + m * kseg + 8 * o);
                        const float4 xb = *reinterpret_cast<const float4*>(xs + m * kseg + 8 * o + 4);
                        float s = acc[m];
                        s = fmaf(w[0], xa.x, s); s = fmaf(w[1], xa.y, s); s = fmaf(w[2], xa.z, s); s = fmaf(w[3], xa.w, s);
                        s = fmaf(w[4], xb.x, s); s = fmaf(w[5], xb.y, s); s = fmaf(w[6], xb.z, s); s = fmaf(w[7], xb.w, s);
                        acc[m] = s;
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && n < N) {
                float* out = y + (size_t)m * N + n;
                if (EPI == EPI_ACCUM) *out += v; else *out = v;
            }
        }
    }
}

template <int GTYPE, int MT, int EPI>
int launch_kq(const cmlb200_qmat* W, const float* x, float* y, cudaStream_t st) {
    const int N = W->rows, K = W->cols;
    int kseg = K;
    if ((size_t)kseg * MT > (size_t)kSegMaxFloats) kseg = (kSegMaxFloats / MT) / 256 * 256;
    auto kern = gemv_kq_kernel<GTYPE, MT, EPI>;
    static size_t attr_smem[kMaxDevices] = {};
    CMLB_CUDA(cmlb_ensure_smem(kern, (size_t)kSegMaxFloats * 4, attr_smem));
    int grid = (N + kWarps - 1) / kWarps;
    const int cap = cmlb_num_sms() * 4;
    if (grid > cap) grid = cap;
    kern<<<grid, kThreads, (size_t)kseg * MT * sizeof(float), st>>>((const uint8_t*)W->qs, x, y, N, K, kseg);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

template <int GTYPE, int EPI>
int run_kq(const cmlb200_qmat* W, const float* x, float* y, int M, cudaStream_t st) {
    int m0 = 0, rc = 0;
    while (m0 < M && rc == 0) {
        const int left = M - m0;
        const float* xm = x + (size_t)m0 * W->cols;
        float* ym = y + (size_t)m0 * W->rows;
        if (left >= 8) { rc = launch_kq<GTYPE, 8, EPI>(W, xm, ym, st); m0 += 8; }
        else if (left >= 4) { rc = launch_kq<GTYPE, 4, EPI>(W, xm, ym, st); m0 += 4; }
        else if (left >= 2) { rc = launch_kq<GTYPE, 2, EPI>(W, xm, ym, st); m0 += 2; }
        else { rc = launch_kq<GTYPE, 1, EPI>(W, xm, ym, st); m0 += 1; }
    }
    return rc;
}

}  // namespace

bool cmlb200_is_kquant_type_(int type) { return type == CMLB200_Q4_1 || type == CMLB200_Q4_K || type == CMLB200_Q5_K || type == CMLB200_Q6_K; }

// y[M, rows] (= | +=) for a weight of GGUF type 3, 12, 13 or 14 whose `qs` is the tensor's block
// stream, 16-byte aligned; `cols` a whole number of blocks. accumulate: add onto y.
int cmlb200_gemv_kquant_(const cmlb200_qmat* W, const float* x, float* y, int M, int accumulate, cudaStream_t st) {
    const int bs = W->type == CMLB200_Q4_1 ? 32 : 256;
    CMLB_REQUIRE(W->cols % bs == 0, "cmlb200_gemv: cols=%d is not a whole number of %d-element blocks (GGUF type %d)", W->cols, bs, W->type);
    CMLB_REQUIRE(((uintptr_t)W->qs & 15) == 0, "cmlb200_gemv: the block stream must be 16-byte aligned");
#define KQ_RUN(T) (accumulate ? run_kq<T, EPI_ACCUM>(W, x, y, M, st) : run_kq<T, EPI_STORE>(W, x, y, M, st))
    switch (W->type) {
        case CMLB200_Q4_1: return KQ_RUN(3);
        case CMLB200_Q4_K: return KQ_RUN(12);
        case CMLB200_Q5_K: return KQ_RUN(13);
        default: return KQ_RUN(14);
    }
#undef KQ_RUN
}
