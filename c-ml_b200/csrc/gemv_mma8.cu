// Decode GEMV for Q4_0 with 5 to 8 rows of x per launch on the integer tensor cores (mma.sync
// m16n8k32 s8 x s8 -> s32): the batched-decode sibling of gemv_mma.cu, which stops at 4 rows
// because its digit table (3 digit columns + 1 zero column per row of x, all of K) fills shared
// memory and every CTA rebuilds it.
//
// What is different here:
//   * Plane-major digit columns. An MMA has 8 columns; column n of MMA p is digit plane p of row n
//     of x, so 8 rows of x cost 3 MMAs per 32-weight block and 16 weight rows, with no zero
//     column. A thread's accumulators (rows g, g+8 x columns 2t, 2t+1) of the three MMAs belong
//     to the same two rows of x, so X . w = c0 * 65536 + (c1 << 8) + c2 is formed in the thread:
//     one shift-add, two conversions and two fused multiply-adds with the fp16 block scale.
//   * The digits are made once, not per CTA: x_planes_kernel (one CTA per row of x and 16 units
//     of K, RMSNorm of src/nn/llama.c:71-124 included when a norm weight is given) writes them to
//     a device scratch in the register layout of the MMA's B operand. Measured with eight rows made
//     inside every GEMV CTA instead: 5.5 us of a 13.4 us launch (10.5 of 18.4 with the RMSNorm).
//   * K in phases of 16 units (one unit of 8 blocks per warp). A warp keeps the B fragments of its
//     unit in registers (48) for a whole phase, so no digit table sits in shared memory and the
//     per-warp rings can be four units deep; with more than one phase a CTA walks its items once
//     per phase and keeps their sums in shared memory in between. Every weight byte is read once.
//   * SwiGLU pairs are two items (gate rows, up rows) of one row group instead of two matrices
//     per ring buffer, so the rings stay as small as for a single weight.
// The rest is the scheme of gemv_mma.cu: item = 16 weight rows, per-warp cp.async rings that start
// before griddepcontrol.wait, x as 24-bit fixed point of its 256-element slice maximum in three
// balanced int8 digits, partial sums of four items parked per CTA barrier and added in warp order,
// grid = one CTA per SM. Replaces C-ML's dequantize-then-fp32-matmul
// (src/core/gguf.c:271-295 + src/ops/ir/execution.c:989-1052, 3090-3134) for batched decode.
#include "common.cuh"
#include "mma_util.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };
constexpr int SW = 16;                          // warps per CTA = units per phase
constexpr int KU = 8;                           // blocks per unit
constexpr int MR = 8;                           // rows of x = columns of an MMA
constexpr int FB = 4;                           // items per CTA barrier (even: SwiGLU pairs stay together)
constexpr int NBUF = 4;                         // ring depth per warp
constexpr int NPRE = 4;                         // of which requested before the dependency wait (measured 11.9 us
                                                // per launch on 11008 x 4096 with 4, 12.2-12.9 with 2, 13.1 with 1)
constexpr int QB = 16;                          // quant bytes per Q4_0 block
constexpr int ROW_STRIDE = KU * QB + 16;        // padded: 8 rows hit 8 different bank groups
constexpr int QS_BYTES = 16 * ROW_STRIDE;
constexpr int UNIT_BYTES = QS_BYTES + 16 * 16;  // + 8 fp16 scales per row
constexpr int BLK_WORDS = 3 * MR * 8;           // digit words per block: [plane][row of x][8 words = 32 k]
constexpr int XFULL = kXqFull - 1;
constexpr size_t kSmemLimit = 227 * 1024;

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Digit planes of M <= 8 rows of x for the kernel below. grid = (M, ceil(units / 16)); CTA (m, c)
// handles units 16c .. 16c+15 of row m, one warp each. planes: [unit][block 8][plane 3][row 8][8 words],
// word 2t of a (plane, row) = k 4t..4t+3, word 2t+1 = k 16+4t..: thread (g, t) of the MMA reads its B
// registers of plane p as the uint2 at [p][g][2t]. xs: [unit][row 8] = slice scale of x.
template <bool NORM>
__global__ void __launch_bounds__(SW * 32)
x_planes_kernel(const float* __restrict__ x, const __half* __restrict__ nw, float eps, int K, uint32_t* __restrict__ planes,
                float* __restrict__ xs) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float red[SW];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 7;
    const int m = blockIdx.x, nun = K / (32 * KU);
    const float* xr = x + (size_t)m * K;
    const int un = blockIdx.y * SW + warp;
    float e[2][4];
    uint2 wv[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
    if (un < nun) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t i = (size_t)(un * KU + (lane >> 3) + 4 * h) * 32 + sub * 4;
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            e[h][0] = v.x; e[h][1] = v.y; e[h][2] = v.z; e[h][3] = v.w;
            if (NORM) wv[h] = *reinterpret_cast<const uint2*>(nw + i);
        }
    }
    if (NORM) {                                   // 1 / sqrt(mean(x^2) + eps) over the whole row
        float ss = 0.f;
        for (int i = threadIdx.x * 4; i < K; i += SW * 32 * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < SW; w++) tot += red[w];
        const float inv = 1.0f / sqrtf(tot / (float)K + eps);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&wv[h].x));
            const float2 w23 = __half22float2(*reinterpret_cast<const __half2*>(&wv[h].y));
            e[h][0] = e[h][0] * inv * w01.x; e[h][1] = e[h][1] * inv * w01.y;
            e[h][2] = e[h][2] * inv * w23.x; e[h][3] = e[h][3] * inv * w23.y;
        }
    }
    if (un >= nun) return;
    float amax = 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int k = 0; k < 4; k++) amax = fmaxf(amax, fabsf(e[h][k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax > 0.f ? (float)XFULL / amax : 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        // Z = (X + 0x8080) ^ 0x8080: its bytes 0, 1, 2 are the balanced digits d2, d1, d0 of X
        uint32_t Z[4];
#pragma unroll
        for (int k = 0; k < 4; k++) Z[k] = (uint32_t)(__float2int_rn(e[h][k] * sc) + 0x8080) ^ 0x8080u;
        const uint32_t t01 = __byte_perm(Z[0], Z[1], 0x5140), t23 = __byte_perm(Z[2], Z[3], 0x5140);
        const uint32_t u01 = __byte_perm(Z[0], Z[1], 0x0062), u23 = __byte_perm(Z[2], Z[3], 0x0062);
        uint32_t* dst = planes + ((size_t)(un * KU + (lane >> 3) + 4 * h) * 3 * MR + m) * 8 + (sub & 3) * 2 + (sub >> 2);
        dst[0] = __byte_perm(u01, u23, 0x5410);            // plane 0: d0
        dst[MR * 8] = __byte_perm(t01, t23, 0x7632);       // plane 1: d1
        dst[2 * MR * 8] = __byte_perm(t01, t23, 0x5410);   // plane 2: d2
    }
    if (lane == 0) xs[un * MR + m] = amax / (float)XFULL;
}

// planes, xs: digit planes and slice scales of x from x_planes_kernel; y: [M][N]. K % 256 == 0.
// nwi = 1, or 2 for SwiGLU (qs = gate, qs2 = up). acc_items: items per CTA whose sums are kept
// between phases (0 when K is a single phase).
template <bool QUIRK>
__global__ void __launch_bounds__(SW * 32, 1)
gemv_mma8_kernel(const uint8_t* __restrict__ qs, const uint16_t* __restrict__ scales, const uint8_t* __restrict__ qs2,
                 const uint16_t* __restrict__ scales2, const uint2* __restrict__ planes, const float* __restrict__ xs,
                 float* __restrict__ y, int N, int K, int M, int nwi, int epi, int acc_items) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nblk = K / 32, nun = nblk / KU, nph = (nun + SW - 1) / SW;
    // shared memory: partials [FB][SW][MR][16] | item sums [acc_items][MR][16] | rings [SW][NBUF][UNIT_BYTES]
    float* partial = reinterpret_cast<float*>(smem);
    float* itemacc = partial + FB * SW * MR * 16;
    uint8_t* ring = reinterpret_cast<uint8_t*>(itemacc + (size_t)acc_items * MR * 16) + (size_t)warp * NBUF * UNIT_BYTES;
    const uint32_t ring0 = smem_u32(ring);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int rgs = (N + 15) / 16;                                   // row groups of 16 weight rows
    const int my_rgs = ((int)blockIdx.x < rgs) ? (rgs - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int my_items = my_rgs * nwi;
    const int nun_last = nun - (nph - 1) * SW;                       // units of the last phase
    const int my_nph = (nph - 1) + (warp < nun_last ? 1 : 0);        // phases in which this warp has a unit
    const int my_tasks = my_items * my_nph;
    const size_t row_bytes = (size_t)nblk * QB;

    // ---- ring: task number iss = (phase iss_ph, item iss_li) of this warp
    int iss = 0, iss_ph = 0, iss_li = 0;
    const uint32_t dst_off_l = (uint32_t)((lane >> 3) * ROW_STRIDE + (lane & 7) * 16);
    auto issue_next = [&](int buf) {
        if (iss < my_tasks) {
            const int a = iss_li & (nwi - 1);
            const int row0 = ((int)blockIdx.x + (iss_li >> (nwi - 1)) * (int)gridDim.x) * 16;
            const int un = iss_ph * SW + warp;
            const uint8_t* wq = (a ? qs2 : qs) + (size_t)un * (KU * QB) + (size_t)(lane & 7) * 16;
            const uint16_t* ws = (a ? scales2 : scales) + (size_t)un * KU;
            const uint32_t dst = ring0 + buf * UNIT_BYTES;
#pragma unroll
            for (int k = 0; k < 4; k++) {                            // rows past N repeat row N-1; never written
                const int srow = min(row0 + k * 4 + (lane >> 3), N - 1);
                cp_async16(dst + dst_off_l + k * (4 * ROW_STRIDE), wq + (size_t)srow * row_bytes);
            }
            if (lane < 16) cp_async16(dst + QS_BYTES + lane * 16, ws + (size_t)min(row0 + lane, N - 1) * nblk);
            iss++;
            if (++iss_li == my_items) { iss_li = 0; iss_ph++; }
        }
        cp_async_commit();
    };

    // B fragments of this warp's unit of phase ph and the slice scales of its two rows of x
    uint2 breg[KU][3];
    float xs0 = 0.f, xs1 = 0.f;
    auto load_b = [&](int ph) {
        const int un = ph * SW + warp;
        const uint2* src = planes + (size_t)un * (KU * BLK_WORDS / 2) + lane;
#pragma unroll
        for (int i = 0; i < KU; i++)
#pragma unroll
            for (int p = 0; p < 3; p++) breg[i][p] = __ldcg(src + (i * 3 + p) * 32);
        xs0 = __ldcg(xs + un * MR + 2 * t) * 0.0625f;                // 1/16: the nibble form is 16*(q-8)
        xs1 = __ldcg(xs + un * MR + 2 * t + 1) * 0.0625f;
    };

#pragma unroll
    for (int i = 0; i < NPRE; i++) issue_next(i);                    // weights do not depend on the previous kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (warp < min(nun, SW)) load_b(0);                              // the loads everything waits for go first
#pragma unroll
    for (int i = NPRE; i < NBUF; i++) issue_next(i);

    const uint32_t ld_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * ROW_STRIDE + (lane >> 4) * 16);
    const uint32_t nib_mask = 0xF0F0F0F0u, nib_flip = 0x80808080u;
    // One unit: 8 blocks x 3 MMAs; au = sums for (row g | g+8, row of x 2t | 2t+1) before the scale of x
    auto unit_mmas = [&](uint32_t mb, float (&au)[4]) {
        auto one_block = [&](int i, float d_lo, float d_hi, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
            int c[3][4];
#pragma unroll
            for (int p = 0; p < 3; p++) {
                mma_s8(a0, a1, a2, a3, breg[i][p].x, breg[i][p].y, c[p][0], c[p][1], c[p][2], c[p][3]);
            }
            const float d_lo16 = d_lo * 65536.0f, d_hi16 = d_hi * 65536.0f;
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const float d = v < 2 ? d_lo : d_hi, d16 = v < 2 ? d_lo16 : d_hi16;
                au[v] = fmaf((float)c[0][v], d16, au[v]);
                au[v] = fmaf((float)((c[1][v] << 8) + c[2][v]), d, au[v]);
            }
        };
#pragma unroll
        for (int p = 0; p < KU / 2; p++) {
            const float2 dlo = scales_of<QUIRK>(lds32(mb + QS_BYTES + g * 16 + p * 4)), dhi = scales_of<QUIRK>(lds32(mb + QS_BYTES + (g + 8) * 16 + p * 4));
            uint32_t r0, r1, r2, r3;                 // one ldmatrix: [rows 0-7 | 8-15] x [block 2p | 2p+1]
            ldmatrix_x4(mb + ld_off + p * 32, r0, r1, r2, r3);
            // nibble n in the top half of a byte, top bit flipped, reads as the int8 16*(n-8)
            one_block(2 * p, dlo.x, dhi.x, and_xor(r0 << 4, nib_mask, nib_flip), and_xor(r1 << 4, nib_mask, nib_flip),
                      and_xor(r0, nib_mask, nib_flip), and_xor(r1, nib_mask, nib_flip));
            one_block(2 * p + 1, dlo.y, dhi.y, and_xor(r2 << 4, nib_mask, nib_flip), and_xor(r3 << 4, nib_mask, nib_flip),
                      and_xor(r2, nib_mask, nib_flip), and_xor(r3, nib_mask, nib_flip));
        }
    };

    // Items li_first .. li_first+count-1 of phase ph sit in slots 0..count-1: add the warps' partial
    // sums in warp order, carry them to the next phase or, in the last one, write y.
    auto flush = [&](int li_first, int count, int ph) {
        __syncthreads();
        const int nact = min(SW, nun - ph * SW);
        const int groups = count >> (nwi - 1);
        for (int idx = threadIdx.x; idx < groups * MR * 16; idx += SW * 32) {
            const int r = idx & 15, m = (idx >> 4) & (MR - 1), gi = idx >> 7;
            const int li0 = li_first + gi * nwi;
            const int row = ((int)blockIdx.x + (li0 >> (nwi - 1)) * (int)gridDim.x) * 16 + r;
            if (m < M && row < N) {
                auto item_sum = [&](int a) {
                    const float* src = partial + (size_t)(gi * nwi + a) * (SW * MR * 16) + m * 16 + r;
                    float v = 0.f;
                    for (int w = 0; w < nact; w++) v += src[w * (MR * 16)];
                    if (nph > 1) {
                        float* keep = itemacc + (size_t)(li0 + a) * (MR * 16) + m * 16 + r;
                        if (ph > 0) v += *keep;
                        if (ph < nph - 1) *keep = v;
                    }
                    return v;
                };
                const float sum0 = item_sum(0);
                const float sum1 = nwi == 2 ? item_sum(1) : 0.f;
                if (ph == nph - 1) {
                    float* out = y + (size_t)m * N + row;
                    if (nwi == 2) *out = (sum0 / (1.0f + expf(-sum0))) * sum1;
                    else if (epi == EPI_ACCUM) *out += sum0;
                    else *out = sum0;
                }
            }
        }
        __syncthreads();
    };

    int u = 0;
    for (int ph = 0; ph < nph; ph++) {
        const bool active = ph * SW + warp < nun;
        if (active && ph > 0) load_b(ph);
        for (int li = 0; li < my_items; li++) {
            const int slot = li % FB;
            if (active) {
                const int buf = u % NBUF;
                cp_async_wait<NBUF - 1>();
                __syncwarp();
                float au[4] = {0.f, 0.f, 0.f, 0.f};
                unit_mmas(ring0 + buf * UNIT_BYTES, au);
                __syncwarp();                                    // every lane is done with this buffer
                issue_next(buf);
                u++;
                float* dst = partial + ((size_t)slot * SW + warp) * (MR * 16) + (2 * t) * 16 + g;
                dst[0] = au[0] * xs0;
                dst[16] = au[1] * xs1;
                dst[8] = au[2] * xs0;
                dst[24] = au[3] * xs1;
            }
            if (slot == FB - 1 || li == my_items - 1) flush(li - slot, slot + 1, ph);
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

struct Plan { int grid, acc_items; size_t smem; };

Plan plan_of(const cmlb200_qmat* W, int nwi) {
    Plan p;
    const int rgs = (W->rows + 15) / 16, nun = W->cols / (32 * KU);
    p.grid = min(cmlb_num_sms(), rgs);
    p.acc_items = nun > SW ? (rgs + p.grid - 1) / p.grid * nwi : 0;
    p.smem = (size_t)(FB * SW * MR * 16 + (size_t)p.acc_items * MR * 16) * sizeof(float) + (size_t)SW * NBUF * UNIT_BYTES;
    return p;
}

// Per-device scratch for the digit planes and slice scales of x: allocated once, never moved (so
// captured CUDA graphs stay valid), zero-filled (rows of x beyond M read as zero digits). Calls
// that use it must be ordered on one stream per device.
constexpr int kMaxUnits = 512;                                       // K <= 131072
struct Scratch { uint32_t* planes; float* xs; };
Scratch g_scratch[16] = {};

int get_scratch(Scratch** out) {
    int dev = 0;
    CMLB_CUDA(cudaGetDevice(&dev));
    CMLB_REQUIRE(dev >= 0 && dev < 16, "device index %d out of range", dev);
    Scratch& s = g_scratch[dev];
    if (!s.planes) {
        const size_t pb = (size_t)kMaxUnits * KU * BLK_WORDS * 4, xb = (size_t)kMaxUnits * MR * 4;
        uint8_t* base = nullptr;
        CMLB_CUDA(cudaMalloc((void**)&base, pb + xb));
        CMLB_CUDA(cudaMemset(base, 0, pb + xb));
        s.planes = reinterpret_cast<uint32_t*>(base);
        s.xs = reinterpret_cast<float*>(base + pb);
    }
    *out = &s;
    return CMLB200_OK;
}

template <bool QUIRK>
int launch8(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const __half* nw, float eps, float* y, int M, int epi,
            cudaStream_t st) {
    const int nwi = epi == EPI_SWIGLU ? 2 : 1;
    const int K = W->cols, nun = K / (32 * KU);
    Scratch* sc = nullptr;
    int rc = get_scratch(&sc);
    if (rc) return rc;
    const dim3 pgrid(M, (nun + SW - 1) / SW);
    rc = nw ? launch_pdl(x_planes_kernel<true>, pgrid, dim3(SW * 32), 0, st, x, nw, eps, K, sc->planes, sc->xs)
            : launch_pdl(x_planes_kernel<false>, pgrid, dim3(SW * 32), 0, st, x, nw, eps, K, sc->planes, sc->xs);
    if (rc) return rc;
    const Plan p = plan_of(W, nwi);
    auto kern = gemv_mma8_kernel<QUIRK>;
    static size_t attr_smem[kMaxDevices] = {};
    CMLB_CUDA(cmlb_ensure_smem(kern, p.smem, attr_smem));
    return launch_pdl(kern, dim3(p.grid), dim3(SW * 32), p.smem, st, (const uint8_t*)W->qs, (const uint16_t*)W->scales,
                      W2 ? (const uint8_t*)W2->qs : (const uint8_t*)nullptr, W2 ? (const uint16_t*)W2->scales : (const uint16_t*)nullptr,
                      (const uint2*)sc->planes, (const float*)sc->xs, y, W->rows, K, M, nwi, epi, p.acc_items);
}

}  // namespace

// Shapes the 8-row kernel takes: Q4_0, whole 8-block slices of K with 16-byte aligned scale rows,
// and (for K of more than one phase) few enough items per CTA for their sums to fit in shared
// memory next to the rings.
bool cmlb200_gemv_mma8_ok_(const cmlb200_qmat* W, int epi) {
    if (W->type != CMLB200_Q4_0 || W->cols % 256 != 0 || W->cols / 256 > kMaxUnits || ((uintptr_t)W->qs & 15) || ((uintptr_t)W->scales & 15)) return false;
    return plan_of(W, epi == EPI_SWIGLU ? 2 : 1).smem <= kSmemLimit;
}

// y[M, rows] (= | += | swiglu) for M <= 8 from fp32 x, RMS-normalised with norm_w first when it is
// given: one launch for the digit planes of x, one for the GEMV. Arguments are validated by the
// callers.
int cmlb200_gemv_mma8_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps, float* y, int M,
                       int epi, cudaStream_t st) {
    const __half* nw = reinterpret_cast<const __half*>(norm_w);
    const bool quirk = (W->flags & CMLB200_QMAT_SUBNORMAL_SCALES) || (W2 && (W2->flags & CMLB200_QMAT_SUBNORMAL_SCALES));
    return quirk ? launch8<true>(W, W2, x, nw, eps, y, M, epi, st) : launch8<false>(W, W2, x, nw, eps, y, M, epi, st);
}

extern "C" int cmlb200_gemv_batched_from_planes(const cmlb200_qmat* W) {
    return W && W->qs && W->scales && W->rows > 0 && W->cols > 0 && cmlb200_gemv_mma8_ok_(W, EPI_STORE) && cmlb200_gemv_mma8_ok_(W, EPI_SWIGLU) ? 1 : 0;
}
