// Decode GEMV over the GGUF block types C-ML reads besides Q4_0 / Q8_0: Q4_1, Q4_K, Q5_K, Q6_K
// (src/core/gguf_quant.c:90-112, 151-196, 211-270, 283-311), straight from the file's bytes:
// y[M, N] (= | +=) x[M, K] . dequant(W[N, K])^T with fp32 accumulation. Replaces "dequantise the
// tensor to fp32 (src/core/gguf.c:271-295), then multiply" for weights of those types.
//
// The weight is the tensor's block stream unchanged, row n at byte n * (K / BS) * BB. The quants
// stay small integers: x is turned into three planes of signed 8-bit digits per 32-element block
// (24-bit fixed point relative to the block's maximum, exact to 2^-24 of it) and every 32-element
// sub-block costs 24 dp4a per row of x; the fp16 / 6-bit / int8 scales, minima and offsets of the
// formats are applied once per sub-block in fp32. Q4_K / Q5_K follow C-ML's own nibble order (each
// 32-element sub-block in 16 consecutive bytes, src/core/gguf_quant.c:174-187), not ggml's.
#include "common.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1 };
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

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

// ---- activation digits: per 32-element block of x a record of kXqWords words (three planes of
// signed 8-bit digits of the block's 24-bit fixed-point form, the block scale, and in word 25 the
// fp32 sum of the block's elements, which the minimum / offset terms of Q4_1, Q4_K and Q5_K need).
__global__ void __launch_bounds__(256) kq_digits_kernel(const float* __restrict__ x, int items, uint32_t* __restrict__ rec) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMV may start fetching weights
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int sub = threadIdx.x & 7;                  // 8 lanes share a block, 4 elements each
    const int item = (blockIdx.x * 256 + threadIdx.x) >> 3;
    if (item < items) {                               // whole groups of 8 lanes enter or skip together
        const unsigned gmask = 0xffu << (threadIdx.x & 24);
        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)item * 32 + sub * 4);
        const float e[4] = {v.x, v.y, v.z, v.w};
        uint32_t* dst = rec + (size_t)item * kXqWords;
        xq_emit_oct(e, sub, gmask, dst);
        float s = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) s += __shfl_xor_sync(gmask, s, o);
        if (sub == 0) dst[25] = __float_as_uint(s);
    }
}

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {     // unsigned bytes of a times signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 32-bit word at a 2-byte aligned address, from the two aligned words around it
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~(uintptr_t)3);
    return (a & 2) ? __funnelshift_r(q[0], q[1], 16) : q[0];
}

// The weights of one 32-element sub-block as 8 words of 4 small integers each (word w = elements
// 4w .. 4w+3, matching the digit planes), plus what turns the integer dot products into the result:
//   Q4_1: y += d * S + m * sum(x)                 Q4_K / Q5_K: y += d*sc * S - dmin*mn * sum(x)
//   Q6_K: y += d * (sc_lo * S(words 0-3) + sc_hi * S(words 4-7)), weights already minus 32 (signed)
struct Sub { uint32_t w[8]; float s0, s1; };

template <int GTYPE>
__device__ __forceinline__ void load_sub(const uint8_t* __restrict__ row, int blk, Sub& s) {
    if (GTYPE == 3) {                                        // 20-byte block: d, m, 16 bytes (byte j = element j low, j + 16 high)
        const uint8_t* p = row + (size_t)blk * 20;
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(p);
        s.s0 = h2f(dm); s.s1 = h2f(dm >> 16);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t q = *reinterpret_cast<const uint32_t*>(p + 4 + 4 * k);
            s.w[k] = q & 0x0F0F0F0Fu; s.w[4 + k] = (q >> 4) & 0x0F0F0F0Fu;
        }
    } else if (GTYPE == 12 || GTYPE == 13) {                 // d, dmin, scales[12], (qh[32],) qs[128]: sub-block i in 16 consecutive bytes
        const uint8_t* p = row + (size_t)(blk >> 3) * KQ<GTYPE>::BB;
        const int i = blk & 7;
        const uint4 hdr = *reinterpret_cast<const uint4*>(p);
        const uint4 qv = *reinterpret_cast<const uint4*>(p + (GTYPE == 12 ? 16 : 48) + i * 16);
        int sc, mn;
        scale_min(hdr.y, hdr.z, hdr.w, i, sc, mn);
        s.s0 = h2f(hdr.x) * (float)sc; s.s1 = h2f(hdr.x >> 16) * (float)mn;
        const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int k = 0; k < 4; k++) { s.w[k] = q[k] & 0x0F0F0F0Fu; s.w[4 + k] = (q[k] >> 4) & 0x0F0F0F0Fu; }
        if (GTYPE == 13) {                                   // bit e of the sub-block's 32 high bits belongs to element e
            const uint32_t hb = *reinterpret_cast<const uint32_t*>(p + 16 + 4 * i);
#pragma unroll
            for (int k = 0; k < 8; k++) s.w[k] |= ((((hb >> (4 * k)) & 15u) * 0x00204081u) & 0x01010101u) << 4;
        }
    } else {                                                 // ql[128], qh[64], scales[16] (int8), d; 2-byte aligned blocks
        const uint8_t* p = row + (size_t)(blk >> 3) * 210;
        const int i = blk & 7;
        const uint32_t sd = *reinterpret_cast<const uint16_t*>(p + 192 + 2 * i);   // two int8 scales of this sub-block's halves
        const float d = h2f(*reinterpret_cast<const uint16_t*>(p + 208));        // (16-bit loads: nothing is read past the block)
        s.s0 = d * (float)(int)(int8_t)(sd & 0xFFu); s.s1 = d * (float)(int)(int8_t)(sd >> 8);
#pragma unroll
        for (int k = 0; k < 4; k++) {                        // word k of ql: bytes = element pairs (8k, 8k+1) .. (8k+6, 8k+7)
            const uint32_t q = ld_u32_a2(p + 16 * i + 4 * k);
            const uint32_t lo = q & 0x0F0F0F0Fu, hi = (q >> 4) & 0x0F0F0F0Fu;
            s.w[2 * k] = __byte_perm(lo, hi, 0x5140);        // elements 8k .. 8k+3
            s.w[2 * k + 1] = __byte_perm(lo, hi, 0x7362);    // elements 8k+4 .. 8k+7
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {                        // byte b of qh: two high bits of elements 4b .. 4b+3
            const uint32_t h = ld_u32_a2(p + 128 + 8 * i + 4 * k);
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const uint32_t f = (h >> (8 * b)) & 0xFFu;
                const uint32_t spread = ((f & 0x03u) | ((f & 0x0Cu) << 6) | ((f & 0x30u) << 12) | ((f & 0xC0u) << 18)) << 4;
                const uint32_t t6 = (s.w[4 * k + b] | spread) ^ 0x20202020u;       // q - 32 as signed bytes: flip bit 5, extend it
                s.w[4 * k + b] = t6 | ((t6 & 0x20202020u) * 6u);
            }
        }
    }
}

// Adds this sub-block's share of y for one row of x, whose digit planes dg and (block scale, block
// sum) `tail` the caller has loaded from the record.
template <int GTYPE>
__device__ __forceinline__ float dot_sub(const Sub& s, const uint32_t (&dg)[3][8], float2 tail, float acc) {
    int c[3][2];
#pragma unroll
    for (int pl = 0; pl < 3; pl++) {
        int lo = 0, hi = 0;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            lo = GTYPE == 14 ? dp4a_ss(s.w[k], dg[pl][k], lo) : dp4a_us(s.w[k], dg[pl][k], lo);
            hi = GTYPE == 14 ? dp4a_ss(s.w[4 + k], dg[pl][4 + k], hi) : dp4a_us(s.w[4 + k], dg[pl][4 + k], hi);
        }
        c[pl][0] = lo; c[pl][1] = hi;
    }
    if (GTYPE == 14) {
        const float slo = fmaf((float)c[0][0], 65536.f, (float)(c[1][0] * 256 + c[2][0]));
        const float shi = fmaf((float)c[0][1], 65536.f, (float)(c[1][1] * 256 + c[2][1]));
        return fmaf(tail.x, fmaf(s.s0, slo, s.s1 * shi), acc);
    }
    const float S = fmaf((float)(c[0][0] + c[0][1]), 65536.f, (float)((c[1][0] + c[1][1]) * 256 + (c[2][0] + c[2][1])));
    const float off = s.s1 * tail.y;
    return fmaf(s.s0 * tail.x, S, GTYPE == 3 ? acc + off : acc - off);
}

// One warp per R consecutive output rows (R = 2 from four rows of x up, so that a digit record
// read from L1 serves two weight rows); a lane takes one 32-element sub-block per step (a step =
// 1024 elements of K), so a 16-byte quant load per lane is 512 contiguous bytes per warp. The
// weight loads of UN steps are issued before the first is consumed, the very first ones before the
// wait for the digits kernel.
template <int GTYPE, int MT, int R, int EPI>
__global__ void __launch_bounds__(kThreads)
gemv_kq_kernel(const uint8_t* __restrict__ blocks, const uint32_t* __restrict__ rec, float* __restrict__ y, int N, int K) {
    constexpr int UN = R == 1 ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * kWarps + (threadIdx.x >> 5)) * R;
    const bool live = n0 < N;
    const int nblk = K / 32;
    const size_t row_bytes = (size_t)(K / KQ<GTYPE>::BS) * KQ<GTYPE>::BB;
    const uint8_t* row[R];
#pragma unroll
    for (int r = 0; r < R; r++) row[r] = blocks + (size_t)min(n0 + r, N - 1) * row_bytes;
    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < MT; m++) acc[r][m] = 0.f;
    Sub s[UN][R];
    auto fetch = [&](int b0) {
#pragma unroll
        for (int u = 0; u < UN; u++)
#pragma unroll
            for (int r = 0; r < R; r++) load_sub<GTYPE>(row[r], min(b0 + 32 * u, nblk - 1), s[u][r]);
    };
    if (live) fetch(lane);                                   // weights do not depend on the digits kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!live) return;
    for (int b0 = lane; b0 < nblk; b0 += 32 * UN) {
        if (b0 != lane) fetch(b0);
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int blk = b0 + 32 * u;
            if (blk < nblk) {
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    const uint32_t* rp = rec + ((size_t)m * nblk + blk) * kXqWords;
                    const uint4* r4 = reinterpret_cast<const uint4*>(rp);
                    uint32_t dg[3][8];
#pragma unroll
                    for (int pl = 0; pl < 3; pl++) {
                        const uint4 a = __ldg(r4 + 2 * pl), b = __ldg(r4 + 2 * pl + 1);
                        dg[pl][0] = a.x; dg[pl][1] = a.y; dg[pl][2] = a.z; dg[pl][3] = a.w;
                        dg[pl][4] = b.x; dg[pl][5] = b.y; dg[pl][6] = b.z; dg[pl][7] = b.w;
                    }
                    const float2 tail = __ldg(reinterpret_cast<const float2*>(rp + 24));   // block scale of x, sum of the block's x
#pragma unroll
                    for (int r = 0; r < R; r++) acc[r][m] = dot_sub<GTYPE>(s[u][r], dg, tail, acc[r][m]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && n0 + r < N) {
                float* out = y + (size_t)m * N + n0 + r;
                if (EPI == EPI_ACCUM) *out += v; else *out = v;
            }
        }
}

// Per-device scratch for the digit records of up to 32 rows of x: allocated once, never moved (so
// captured CUDA graphs stay valid). Calls that use it must be ordered on one stream per device.
constexpr size_t kRecBytes = 16u << 20;                     // M * K <= 4,793,490 elements
uint32_t* g_rec[kMaxDevices] = {};

int get_rec(uint32_t** out) {
    const int dev = cmlb_device_index();
    if (!g_rec[dev]) CMLB_CUDA(cudaMalloc((void**)&g_rec[dev], kRecBytes));
    *out = g_rec[dev];
    return CMLB200_OK;
}

template <typename Kern, typename... Args>
int launch_dep(Kern kern, dim3 grid, dim3 block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CMLB_CUDA(cudaLaunchKernelEx(&cfg, kern, args...));
    return CMLB200_OK;
}

template <int GTYPE, int MT, int EPI>
int launch_kq(const cmlb200_qmat* W, const uint32_t* rec, float* y, cudaStream_t st) {
    constexpr int R = MT >= 4 ? 2 : 1;
    const int N = W->rows, K = W->cols;
    return launch_dep(gemv_kq_kernel<GTYPE, MT, R, EPI>, dim3((N + kWarps * R - 1) / (kWarps * R)), dim3(kThreads), st, (const uint8_t*)W->qs, rec, y, N, K);
}

template <int GTYPE, int EPI>
int run_kq(const cmlb200_qmat* W, const float* x, float* y, int M, cudaStream_t st) {
    const int nblk = W->cols / 32;
    CMLB_REQUIRE((size_t)M * nblk * kXqWords * 4 <= kRecBytes, "cmlb200_gemv: M*cols = %d*%d too large for the activation scratch", M, W->cols);
    uint32_t* rec = nullptr;
    int rc = get_rec(&rec);
    if (rc) return rc;
    const int items = M * nblk;
    rc = launch_dep(kq_digits_kernel, dim3((items * 8 + 255) / 256), dim3(256), st, x, items, rec);
    int m0 = 0;
    while (m0 < M && rc == 0) {
        const int left = M - m0;
        const uint32_t* rm = rec + (size_t)m0 * nblk * kXqWords;
        float* ym = y + (size_t)m0 * W->rows;
        if (left >= 8) { rc = launch_kq<GTYPE, 8, EPI>(W, rm, ym, st); m0 += 8; }
        else if (left >= 4) { rc = launch_kq<GTYPE, 4, EPI>(W, rm, ym, st); m0 += 4; }
        else if (left >= 2) { rc = launch_kq<GTYPE, 2, EPI>(W, rm, ym, st); m0 += 2; }
        else { rc = launch_kq<GTYPE, 1, EPI>(W, rm, ym, st); m0 += 1; }
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
