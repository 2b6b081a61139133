// Decode GEMV for Q4_0 / Q8_0 at M <= 2 per launch on the integer tensor cores (mma.sync
// m16n8k32 s8 x s8 -> s32), built around the instruction budget of a B200 SM.
//
// At HBM speed an SM receives a 32-weight block every ~0.8 clocks. dp4a shares the 64-lane
// integer pipe with the nibble unpacking, so three exact 8-bit digit planes of x cost about as
// many integer-pipe cycles as the memory system leaves (measured: the dp4a kernels issue ~125
// thread instructions per block and stall on that pipe). One MMA does 16 rows x 32 weights x 8
// columns; with the digit planes of x as columns (3 digits + a zero column per row of x, so two
// rows of x fit) the whole dot-product work is one tensor instruction per 512 weights, and the
// integer pipe only unpacks nibbles.
//
//   * A operand straight from the file format: thread (g, t) of the MMA needs k = 4t..4t+3 and
//     k = 16+4t..16+4t+3 of rows g and g+8. Word t of a Q4_0 block holds exactly those elements
//     (low nibbles 4t..4t+3, high nibbles 16+4t..), so one ldmatrix over 16-byte block rows in
//     shared memory delivers each thread its word, and three logic operations turn it into the
//     two int8x4 registers 16*(q-8). Q8_0 bytes are used as they are.
//   * B operand = digit planes of the block-fixed-point form of x (common.cuh), kept in
//     registers for the whole kernel when every warp owns a single 8-block slice of K.
//   * The accumulator comes back as int32; started at 0x4B400000 its bit pattern read as fp32 is
//     12582912 + sum, so one subtraction converts it exactly, and a fused multiply-add applies
//     the fp16 block scale times the block scale of x. Digit columns are combined at the end.
//
// Work split: item = 16 consecutive weight rows over all of K; the 16 warps of a CTA split K in
// slices of 8 blocks, each warp streaming its slice of successive items through its own ring of
// cp.async buffers (issued before griddepcontrol.wait: weights do not depend on the previous
// kernel), and the CTA sums the 16 partial results of an item in a fixed order. One CTA per SM,
// items dealt round-robin. Replaces C-ML's dequantize-then-fp32-matmul (src/core/gguf.c:271-295
// + src/ops/ir/execution.c:989-1052, 3090-3134) like the other GEMV kernels.
#include "common.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };
constexpr int SW = 16;                 // warps per CTA
constexpr int KU = 8;                  // blocks per unit (one warp, one item, one ring buffer)
constexpr int XW = kXqWords;
constexpr uint32_t MAGIC = 0x4B400000u;
constexpr float MAGICF = 12582912.0f;

template <int TYPE, int NW>
struct Cfg {
    static constexpr int QB = (TYPE == CMLB200_Q8_0) ? 32 : 16;     // quant bytes per block
    static constexpr int PPR = KU * QB / 16;                         // 16-byte pieces per row of a unit
    static constexpr int ROW_STRIDE = KU * QB + 16;                  // padded: 8 rows hit 8 different bank groups
    static constexpr int QS_BYTES = 16 * ROW_STRIDE;
    static constexpr int SC_STRIDE = 48;                             // 8 fp16 scales + pad, conflict-free for 128-bit reads
    static constexpr int MAT_BYTES = QS_BYTES + 16 * SC_STRIDE;
    static constexpr int UNIT_BYTES = NW * MAT_BYTES;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
// D = A(16x32 s8, row) * B(32x8 s8, col) + MAGIC in every lane of the accumulator
__device__ __forceinline__ void mma_s8(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                       int& d0, int& d1, int& d2, int& d3) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(MAGIC));
}
__device__ __forceinline__ float unmagic(int c) { return __int_as_float(c) - MAGICF; }

template <bool QUIRK>
__device__ __forceinline__ float scale_of(uint32_t packed, int odd) {
    const uint16_t h = (uint16_t)(odd ? (packed >> 16) : (packed & 0xFFFFu));
    return QUIRK ? cml_half_to_float(h) : __half2float(__ushort_as_half(h));
}

// xin: digit records [MT][K/32][XW] (XMODE 0), fp32 activations [MT][K] (XMODE 1), or fp32
// activations RMS-normalised with the fp16 weight nw first (XMODE 2; src/nn/llama.c:71-124).
// y: [MT][N]. K % 256 == 0. BREG: K/256 <= SW, every warp keeps its B fragments in registers.
// NW = 2: SwiGLU of two weights (gate, up); NW = 1: epi selects store or accumulate.
template <int TYPE, int MT, int NW, bool QUIRK, bool BREG, int NBUF>
__global__ void __launch_bounds__(SW * 32, 1)
gemv_mma_kernel(const uint8_t* __restrict__ qs, const uint16_t* __restrict__ scales,
                const uint8_t* __restrict__ qs2, const uint16_t* __restrict__ scales2,
                const void* __restrict__ xin, const __half* __restrict__ nw, float eps, float* __restrict__ y, int N, int K,
                int XMODE, int epi) {
    using C = Cfg<TYPE, NW>;
    constexpr int QB = C::QB, NC = 4 * MT;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[SW][MT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nblk = K / 32, nocts = nblk / KU;
    // shared memory: B table [nblk][NC][8 words] | xs [MT][nblk] | partials [2][SW][NW][MT][16] | rings
    uint32_t* table = reinterpret_cast<uint32_t*>(smem);
    float* xs_all = reinterpret_cast<float*>(smem + (size_t)nblk * NC * 32);
    float* partial = xs_all + (((size_t)MT * nblk + 31) & ~(size_t)31);
    uint8_t* ring = reinterpret_cast<uint8_t*>(partial + 2 * SW * NW * MT * 16) + (size_t)warp * NBUF * C::UNIT_BYTES;
    const uint32_t ring0 = smem_u32(ring);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this warp's slice of K (in units of KU blocks) and this CTA's items
    const int q = nocts / SW, rem = nocts % SW;
    const int my_noct = q + (warp < rem ? 1 : 0);
    const int oct0 = warp * q + min(warp, rem);
    const int items = (N + 15) / 16;
    const int my_items = ((int)blockIdx.x < items) ? (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int n_units = my_items * my_noct;
    const size_t row_bytes = (size_t)nblk * QB;

    auto issue = [&](int u, int buf) {
        const int it = u / my_noct, oct = oct0 + (u - it * my_noct);
        const int row0 = ((int)blockIdx.x + it * (int)gridDim.x) * 16;
        const uint32_t dst = ring0 + buf * C::UNIT_BYTES;
#pragma unroll
        for (int a = 0; a < NW; a++) {
            const uint8_t* wq = a ? qs2 : qs;
            const uint16_t* ws = a ? scales2 : scales;
#pragma unroll
            for (int p = lane; p < 16 * C::PPR; p += 32) {
                const int row = p / C::PPR, off = p - row * C::PPR;
                const int srow = min(row0 + row, N - 1);             // rows past N repeat the last row; never written
                cp_async16(dst + a * C::MAT_BYTES + row * C::ROW_STRIDE + off * 16,
                           wq + (size_t)srow * row_bytes + (size_t)oct * (KU * QB) + off * 16);
            }
            if (lane < 16) {
                const int srow = min(row0 + lane, N - 1);
                cp_async16(dst + a * C::MAT_BYTES + C::QS_BYTES + lane * C::SC_STRIDE, ws + (size_t)srow * nblk + (size_t)oct * KU);
            }
        }
    };

    // Weights do not depend on the preceding kernel: fill the ring before the dependency wait.
#pragma unroll
    for (int i = 0; i < NBUF; i++) {
        if (i < n_units) issue(i, i);
        cp_async_commit();
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- digits of x into the B table
    {
        const int sub = threadIdx.x & 7;
        const unsigned gmask = 0xffu << (threadIdx.x & 24);
        if (XMODE != 0) {
            const float* x = static_cast<const float*>(xin);
            float inv[MT];
#pragma unroll
            for (int m = 0; m < MT; m++) inv[m] = 1.f;
            if (XMODE == 2) {
                
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    float ss = 0.f;
                    for (int i = threadIdx.x * 4; i < K; i += SW * 128) {
                        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + i);
                        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0) red[warp][m] = ss;
                }
                __syncthreads();
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    float tot = 0.f;
#pragma unroll
                    for (int w = 0; w < SW; w++) tot += red[w][m];
                    inv[m] = 1.0f / sqrtf(tot / (float)K + eps);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; m++)
                for (int b = threadIdx.x >> 3; b < nblk; b += SW * 4) {
                    const int i = b * 32 + sub * 4;
                    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + i);
                    float e[4] = {v.x, v.y, v.z, v.w};
                    if (XMODE == 2) {
                        const uint2 wr = *reinterpret_cast<const uint2*>(nw + i);
                        const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&wr.x));
                        const float2 w23 = __half22float2(*reinterpret_cast<const __half2*>(&wr.y));
                        e[0] = e[0] * inv[m] * w01.x; e[1] = e[1] * inv[m] * w01.y;
                        e[2] = e[2] * inv[m] * w23.x; e[3] = e[3] * inv[m] * w23.y;
                    }
                    float amax = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
                    const float sc = amax > 0.f ? (float)kXqFull / amax : 0.f;
                    uint32_t w[3] = {0, 0, 0};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        int X = __float2int_rn(e[k] * sc);
                        X = max(-kXqFull, min(kXqFull, X));
                        int d0, d1, d2;
                        xq_split(X, d0, d1, d2);
                        w[0] |= (uint32_t)(d0 & 0xFF) << (8 * k);
                        w[1] |= (uint32_t)(d1 & 0xFF) << (8 * k);
                        w[2] |= (uint32_t)(d2 & 0xFF) << (8 * k);
                    }
                    uint32_t* dst = table + ((size_t)b * NC + m * 4) * 8 + (sub & 3) * 2 + (sub >> 2);
                    dst[0] = w[0]; dst[8] = w[1]; dst[16] = w[2]; dst[24] = 0u;
                    if (sub == 0) xs_all[m * nblk + b] = amax / (float)kXqFull;
                }
        } else {
            const uint32_t* xq = static_cast<const uint32_t*>(xin);
            for (int idx = threadIdx.x; idx < MT * nblk * 8; idx += SW * 32) {
                const int s8 = idx & 7, mb = idx >> 3, m = mb / nblk, b = mb - m * nblk;
                const uint32_t* rec = xq + (size_t)mb * XW;
                uint32_t* dst = table + ((size_t)b * NC + m * 4) * 8 + (s8 & 3) * 2 + (s8 >> 2);
                dst[0] = rec[s8]; dst[8] = rec[8 + s8]; dst[16] = rec[16 + s8]; dst[24] = 0u;
                if (s8 == 0) xs_all[m * nblk + b] = __uint_as_float(rec[24]);
            }
        }
    }
    __syncthreads();

    // B fragment of block b for this thread: column g (n index), words t and 4+t of the plane
    auto load_b = [&](int b, uint32_t& b0, uint32_t& b1) {
        if (g < NC) {
            const uint2 v = *reinterpret_cast<const uint2*>(table + ((size_t)b * NC + g) * 8 + t * 2);
            b0 = v.x; b1 = v.y;
        } else { b0 = 0u; b1 = 0u; }
    };
    const int xm = (MT == 2) ? (t >> 1) : 0;                 // row of x this thread's accumulator columns belong to

    uint32_t breg[BREG ? KU : 1][2];
    float xsr[BREG ? KU : 1];
    if (BREG && my_noct > 0) {
#pragma unroll
        for (int i = 0; i < (BREG ? KU : 1); i++) {
            load_b(oct0 * KU + i, breg[i][0], breg[i][1]);
            xsr[i] = xs_all[xm * nblk + oct0 * KU + i];
        }
    }

    const uint32_t ld_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * C::ROW_STRIDE + (lane >> 4) * 16);
    int u = 0;
    for (int it = 0; it < my_items; it++) {
        float acc[NW][4];
#pragma unroll
        for (int a = 0; a < NW; a++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[a][k] = 0.f;

        for (int o = 0; o < my_noct; o++, u++) {
            const int buf = u % NBUF;
            cp_async_wait<NBUF - 1>();
            __syncwarp();
            const uint32_t ub = ring0 + buf * C::UNIT_BYTES;
            const int blk0 = (oct0 + o) * KU;
#pragma unroll
            for (int a = 0; a < NW; a++) {
                const uint32_t mb = ub + a * C::MAT_BYTES;
                uint4 sg, sg8;       // fp16 scales of rows g and g+8, 8 blocks each
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(sg.x), "=r"(sg.y), "=r"(sg.z), "=r"(sg.w) : "r"(mb + C::QS_BYTES + g * C::SC_STRIDE));
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(sg8.x), "=r"(sg8.y), "=r"(sg8.z), "=r"(sg8.w) : "r"(mb + C::QS_BYTES + (g + 8) * C::SC_STRIDE));
                const uint32_t sgw[4] = {sg.x, sg.y, sg.z, sg.w}, sg8w[4] = {sg8.x, sg8.y, sg8.z, sg8.w};
                auto one_block = [&](int i, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
                    uint32_t b0, b1;
                    float xs;
                    if (BREG) { b0 = breg[BREG ? i : 0][0]; b1 = breg[BREG ? i : 0][1]; xs = xsr[BREG ? i : 0]; }
                    else { load_b(blk0 + i, b0, b1); xs = xs_all[xm * nblk + blk0 + i]; }
                    int c0, c1, c2, c3;
                    mma_s8(a0, a1, a2, a3, b0, b1, c0, c1, c2, c3);
                    const float s_lo = scale_of<QUIRK>(sgw[i >> 1], i & 1) * xs;
                    const float s_hi = scale_of<QUIRK>(sg8w[i >> 1], i & 1) * xs;
                    acc[a][0] = fmaf(unmagic(c0), s_lo, acc[a][0]);
                    acc[a][1] = fmaf(unmagic(c1), s_lo, acc[a][1]);
                    acc[a][2] = fmaf(unmagic(c2), s_hi, acc[a][2]);
                    acc[a][3] = fmaf(unmagic(c3), s_hi, acc[a][3]);
                };
                if (TYPE == CMLB200_Q4_0) {
#pragma unroll
                    for (int p = 0; p < KU / 2; p++) {       // two blocks per ldmatrix: [rows 0-7 | 8-15] x [block 2p | 2p+1]
                        uint32_t r0, r1, r2, r3;
                        ldmatrix_x4(mb + ld_off + p * 32, r0, r1, r2, r3);
                        // nibble n in the top half of a byte, top bit flipped, reads as the int8 16*(n-8)
                        one_block(2 * p, ((r0 << 4) & 0xF0F0F0F0u) ^ 0x80808080u, ((r1 << 4) & 0xF0F0F0F0u) ^ 0x80808080u,
                                  (r0 & 0xF0F0F0F0u) ^ 0x80808080u, (r1 & 0xF0F0F0F0u) ^ 0x80808080u);
                        one_block(2 * p + 1, ((r2 << 4) & 0xF0F0F0F0u) ^ 0x80808080u, ((r3 << 4) & 0xF0F0F0F0u) ^ 0x80808080u,
                                  (r2 & 0xF0F0F0F0u) ^ 0x80808080u, (r3 & 0xF0F0F0F0u) ^ 0x80808080u);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < KU; i++) {           // one block per ldmatrix: [rows 0-7 | 8-15] x [bytes 0-15 | 16-31]
                        uint32_t r0, r1, r2, r3;
                        ldmatrix_x4(mb + ld_off + i * 32, r0, r1, r2, r3);
                        one_block(i, r0, r1, r2, r3);
                    }
                }
            }
            __syncwarp();                                    // every lane is done with this buffer
            if (u + NBUF < n_units) issue(u + NBUF, buf);
            cp_async_commit();
        }

        // ---- combine digit columns, then the 16 K-slices of the CTA
        const int par = it & 1;
#pragma unroll
        for (int a = 0; a < NW; a++) {
            float p_lo = (t & 1) ? acc[a][0] : fmaf(acc[a][0], 65536.0f, acc[a][1] * 256.0f);     // row g
            float p_hi = (t & 1) ? acc[a][2] : fmaf(acc[a][2], 65536.0f, acc[a][3] * 256.0f);     // row g + 8
            p_lo += __shfl_xor_sync(0xffffffffu, p_lo, 1);
            p_hi += __shfl_xor_sync(0xffffffffu, p_hi, 1);
            if ((t & 1) == 0 && (t >> 1) < MT) {
                float* dst = partial + ((((size_t)par * SW + warp) * NW + a) * MT + (t >> 1)) * 16;
                dst[g] = p_lo;
                dst[g + 8] = p_hi;
            }
        }
        __syncthreads();
        if (threadIdx.x < 16 * MT) {
            const int r = threadIdx.x & 15, m = threadIdx.x >> 4;
            const int row = ((int)blockIdx.x + it * (int)gridDim.x) * 16 + r;
            if (row < N) {
                float s[NW];
#pragma unroll
                for (int a = 0; a < NW; a++) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < SW; w++) v += partial[((((size_t)par * SW + w) * NW + a) * MT + m) * 16 + r];
                    s[a] = v * ((TYPE == CMLB200_Q4_0) ? 0.0625f : 1.0f);
                }
                float* out = y + (size_t)m * N + row;
                if (NW == 2) *out = (s[0] / (1.0f + expf(-s[0]))) * s[NW - 1];
                else if (epi == EPI_ACCUM) *out += s[0];
                else *out = s[0];
            }
        }
    }
    cp_async_wait<0>();
}

template <typename Kern, typename... Args>
int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CMLB_CUDA(cudaLaunchKernelEx(&cfg, kern, args...));
    return CMLB200_OK;
}

constexpr size_t kSmemLimit = 227 * 1024;

template <int TYPE, int NW>
size_t smem_bytes(int MT, int nblk, int nbuf) {
    return (size_t)nblk * 4 * MT * 32 + ((((size_t)MT * nblk + 31) & ~(size_t)31) + 2 * SW * NW * MT * 16) * sizeof(float) +
           (size_t)SW * nbuf * Cfg<TYPE, NW>::UNIT_BYTES;
}

template <int TYPE, int MT, int NW, bool QUIRK, bool BREG, int NBUF>
int launch_cfg(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, int xmode, int epi,
               cudaStream_t st) {
    const int N = W->rows, K = W->cols;
    const size_t smem = smem_bytes<TYPE, NW>(MT, K / 32, NBUF);
    auto kern = gemv_mma_kernel<TYPE, MT, NW, QUIRK, BREG, NBUF>;
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        CMLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
    const int grid = min(cmlb_num_sms(), (N + 15) / 16);
    return launch_pdl(kern, dim3(grid), dim3(SW * 32), smem, st, (const uint8_t*)W->qs, (const uint16_t*)W->scales,
                      W2 ? (const uint8_t*)W2->qs : (const uint8_t*)nullptr,
                      W2 ? (const uint16_t*)W2->scales : (const uint16_t*)nullptr, xin, nw, eps, y, N, K, xmode, epi);
}

template <int TYPE, int MT, int NW, bool QUIRK>
int launch(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, int xmode, int epi,
           cudaStream_t st) {
    const int nblk = W->cols / 32;
    const bool breg = nblk / KU <= SW;
    const int nbuf = smem_bytes<TYPE, NW>(MT, nblk, 4) <= kSmemLimit ? 4 : smem_bytes<TYPE, NW>(MT, nblk, 3) <= kSmemLimit ? 3 : 2;
    if (breg) {
        if (nbuf == 4) return launch_cfg<TYPE, MT, NW, QUIRK, true, 4>(W, W2, xin, nw, eps, y, xmode, epi, st);
        if (nbuf == 3) return launch_cfg<TYPE, MT, NW, QUIRK, true, 3>(W, W2, xin, nw, eps, y, xmode, epi, st);
        return launch_cfg<TYPE, MT, NW, QUIRK, true, 2>(W, W2, xin, nw, eps, y, xmode, epi, st);
    }
    if (nbuf == 4) return launch_cfg<TYPE, MT, NW, QUIRK, false, 4>(W, W2, xin, nw, eps, y, xmode, epi, st);
    if (nbuf == 3) return launch_cfg<TYPE, MT, NW, QUIRK, false, 3>(W, W2, xin, nw, eps, y, xmode, epi, st);
    return launch_cfg<TYPE, MT, NW, QUIRK, false, 2>(W, W2, xin, nw, eps, y, xmode, epi, st);
}

// Rows of x two at a time (one launch streams the weight once for both), then one.
template <int TYPE, int NW, bool QUIRK>
int run_m(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, size_t x_row_bytes, const __half* nw, float eps, float* y, int M,
          int xmode, int epi, cudaStream_t st) {
    int m0 = 0, rc = 0;
    while (m0 < M && rc == 0) {
        const void* xm = static_cast<const uint8_t*>(xin) + (size_t)m0 * x_row_bytes;
        float* ym = y + (size_t)m0 * W->rows;
        if (M - m0 >= 2) { rc = launch<TYPE, 2, NW, QUIRK>(W, W2, xm, nw, eps, ym, xmode, epi, st); m0 += 2; }
        else { rc = launch<TYPE, 1, NW, QUIRK>(W, W2, xm, nw, eps, ym, xmode, epi, st); m0 += 1; }
    }
    return rc;
}

template <int TYPE, bool QUIRK>
int run_x(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const __half* nw, float eps, const uint32_t* xq, float* y, int M,
          int epi, cudaStream_t st) {
    const int K = W->cols;
    const void* xin = xq ? (const void*)xq : (const void*)x;
    const size_t xrb = xq ? (size_t)(K / 32) * XW * 4 : (size_t)K * 4;
    const int xmode = xq ? 0 : (nw ? 2 : 1);
    if (epi == EPI_SWIGLU) return run_m<TYPE, 2, QUIRK>(W, W2, xin, xrb, nw, eps, y, M, xmode, epi, st);
    return run_m<TYPE, 1, QUIRK>(W, W2, xin, xrb, nw, eps, y, M, xmode, epi, st);
}

}  // namespace

// Shapes the tensor-core decode kernel takes: whole 8-block slices of K with 16-byte aligned
// scale rows, and room in shared memory for the digit table of two rows of x next to the rings.
bool cmlb200_gemv_mma_ok_(const cmlb200_qmat* W, int epi) {
    if (W->type != CMLB200_Q4_0 && W->type != CMLB200_Q8_0) return false;
    if (W->cols % 256 != 0 || ((uintptr_t)W->qs & 15) || ((uintptr_t)W->scales & 15)) return false;
    const int nblk = W->cols / 32;
    const bool q8 = W->type == CMLB200_Q8_0;
    const size_t need = epi == EPI_SWIGLU ? (q8 ? smem_bytes<CMLB200_Q8_0, 2>(2, nblk, 2) : smem_bytes<CMLB200_Q4_0, 2>(2, nblk, 2))
                                          : (q8 ? smem_bytes<CMLB200_Q8_0, 1>(2, nblk, 2) : smem_bytes<CMLB200_Q4_0, 1>(2, nblk, 2));
    return need <= kSmemLimit;
}

// y[M, rows] (= | += | swiglu) for M <= 4. Exactly one of xq (digit records) and x (fp32, with
// optional RMSNorm weight norm_w) is given. Arguments are validated by the callers.
int cmlb200_gemv_mma_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                      const uint32_t* xq, float* y, int M, int epi, cudaStream_t st) {
    const __half* nw = reinterpret_cast<const __half*>(norm_w);
    const bool quirk = (W->flags & CMLB200_QMAT_SUBNORMAL_SCALES) || (W2 && (W2->flags & CMLB200_QMAT_SUBNORMAL_SCALES));
    const bool q8 = W->type == CMLB200_Q8_0;
    if (quirk) return q8 ? run_x<CMLB200_Q8_0, true>(W, W2, x, nw, eps, xq, y, M, epi, st) : run_x<CMLB200_Q4_0, true>(W, W2, x, nw, eps, xq, y, M, epi, st);
    return q8 ? run_x<CMLB200_Q8_0, false>(W, W2, x, nw, eps, xq, y, M, epi, st) : run_x<CMLB200_Q4_0, false>(W, W2, x, nw, eps, xq, y, M, epi, st);
}
