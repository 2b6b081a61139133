// Decode GEMV for Q4_0 / Q8_0 at M <= 2 per launch on the integer tensor cores (mma.sync
// m16n8k32 s8 x s8 -> s32), built around the instruction budget of a B200 SM.
//
// At HBM speed an SM receives a 32-weight block every ~0.8 clocks. dp4a shares the 64-lane
// integer pipe with the nibble unpacking, so three exact 8-bit digit planes of x cost about as
// many integer-pipe cycles as the memory system leaves (measured: the dp4a kernels execute ~125
// thread instructions per block and stall on that pipe). One MMA does 16 rows x 32 weights x 8
// columns; with the digit planes of x as columns (3 digits + a zero column per row of x, so two
// rows of x fit) the whole dot-product work is one tensor instruction per 512 weights, and the
// integer pipe only unpacks nibbles.
//
//   * A operand straight from the file format: thread (g, t) of the MMA needs k = 4t..4t+3 and
//     k = 16+4t..16+4t+3 of rows g and g+8. Word t of a Q4_0 block holds exactly those elements
//     (low nibbles 4t..4t+3, high nibbles 16+4t..), so one ldmatrix over 16-byte block rows in
//     shared memory delivers each thread its word, and one shift plus two 3-input logic
//     operations turn it into the two int8x4 registers 16*(q-8). Q8_0 bytes are used as they are.
//   * B operand = digit planes of a fixed-point form of x: every warp takes its own slice of K
//     (8 blocks), finds the slice maximum, writes x_k ~= s * X_k with X_k a signed 24-bit integer
//     split in three balanced 8-bit digits, and keeps the fragments in registers for the whole
//     kernel when the slice is its only one. No CTA-wide barrier is involved (except the sum of
//     squares when the RMSNorm is applied here). The rounding of x to 24 bits of its slice maximum
//     is of the order of the rounding an fp32 accumulation commits.
//   * A thread's two accumulator columns are neighbouring digits, so (c_even << 8) + c_odd is
//     their exact int32 combination; one conversion and one fused multiply-add apply the fp16
//     block scale, the slice scale of x is applied once per unit, and the two column pairs of a
//     row of x are combined at the end of an item.
//
// Work split: item = 16 consecutive weight rows over all of K; the 16 warps of a CTA split K in
// units of 8 blocks, each warp streaming its units of successive items through its own ring of
// cp.async buffers (issued before griddepcontrol.wait: weights do not depend on the previous
// kernel), and the CTA sums the partial results of an item in a fixed order. Grid = one CTA per
// SM, items dealt round-robin. Replaces C-ML's dequantize-then-fp32-matmul
// (src/core/gguf.c:271-295 + src/ops/ir/execution.c:989-1052, 3090-3134) like the other GEMV
// kernels.
#include "common.cuh"
#include "mma_util.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };
constexpr int SW = 16;                 // warps per CTA
constexpr int KU = 8;                  // blocks per unit: what one warp takes from one item at a time
constexpr int XW = kXqWords;
// items whose partial results wait in shared memory for one CTA barrier
__host__ __device__ constexpr int flush_batch(int nw, int mt) { return (void)nw, (void)mt, 4; }
constexpr int XFULL = kXqFull - 1;     // |X| <= XFULL + 1 after rounding, which still splits into int8 digits

// One unit = 16 rows x KU blocks of one weight.
template <int TYPE, int NW>
struct Cfg {
    static constexpr int QB = (TYPE == CMLB200_Q8_0) ? 32 : 16;     // quant bytes per block
    static constexpr int PPR = KU * QB / 16;                         // 16-byte pieces per row
    static constexpr int RPP = 32 / PPR;                             // rows one warp-wide copy covers
    static constexpr int PASSES = 16 / RPP;
    static constexpr int ROW_STRIDE = KU * QB + 16;                  // padded: 8 rows hit 8 different bank groups
    static constexpr int QS_BYTES = 16 * ROW_STRIDE;
    static constexpr int MAT_BYTES = QS_BYTES + 16 * 16;             // + 8 fp16 scales per row
    static constexpr int UNIT_BYTES = NW * MAT_BYTES;
};

// xin: digit records [MT][K/32][XW] (xmode 0), fp32 activations [MT][K] (xmode 1), or fp32
// activations RMS-normalised with the fp16 weight nw first (xmode 2; src/nn/llama.c:71-124).
// y: [MT][N]. K % 256 == 0. BREG: K/256 <= SW, every warp owns at most one unit per item and
// keeps its B fragments in registers. NW = 2: SwiGLU of two weights (gate, up); NW = 1: epi
// selects store or accumulate.
template <int TYPE, int MT, int NW, bool QUIRK, bool BREG, int NBUF, int NPRE, bool TP>
__global__ void __launch_bounds__(SW * 32, 1)
gemv_mma_kernel(const uint8_t* __restrict__ qs, const uint16_t* __restrict__ scales,
                const uint8_t* __restrict__ qs2, const uint16_t* __restrict__ scales2,
                const void* __restrict__ xin, const __half* __restrict__ nw, float eps, float* __restrict__ y, int N, int K,
                int xmode, int epi, TpPeers tpa) {
    using C = Cfg<TYPE, NW>;
    constexpr int QB = C::QB, NC = 4 * MT, FB = flush_batch(NW, MT);
    constexpr int NM = (MT + 1) / 2;          // MMAs per block: two rows of x (8 digit columns) each
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[SW][MT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nblk = K / 32, nun = nblk / KU;
    // shared memory: B table [nblk][NC][8 words] | unit scales [MT][nun] | partials [FB][SW][NW][MT][16] | rings
    uint32_t* table = reinterpret_cast<uint32_t*>(smem);
    float* xs_all = reinterpret_cast<float*>(smem + (size_t)nblk * NC * 32);
    float* partial = xs_all + (((size_t)MT * nun + 31) & ~(size_t)31);                 // [FB][SW][NW][MT][16]
    uint8_t* ring = reinterpret_cast<uint8_t*>(partial + FB * SW * NW * MT * 16) + (size_t)warp * NBUF * C::UNIT_BYTES;
    const uint32_t ring0 = smem_u32(ring);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this warp's units of K and this CTA's items
    const int q = nun / SW, rem = nun % SW;
    const int my_nun = q + (warp < rem ? 1 : 0);
    const int un0 = warp * q + min(warp, rem);
    const int items = (N + 15) / 16;
    const int my_items = ((int)blockIdx.x < items) ? (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const size_t row_bytes = (size_t)nblk * QB;

    // per-lane constants of the copy pattern: pass k moves rows k*RPP .. k*RPP+RPP-1 of the unit
    const size_t src_off_l = (size_t)(lane / C::PPR) * row_bytes + (size_t)(lane % C::PPR) * 16;
    const uint32_t dst_off_l = (uint32_t)((lane / C::PPR) * C::ROW_STRIDE + (lane % C::PPR) * 16);
    const size_t src_step = (size_t)C::RPP * row_bytes;

    // The next unit to request: item counter, unit counter within the item, and this lane's
    // source addresses for it (quants: first pass; scales: row `lane`, lanes 0..15).
    int iss_it = 0, iss_o = 0;
    const size_t item_step_q = (size_t)gridDim.x * 16 * row_bytes, item_step_s = (size_t)gridDim.x * 16 * nblk;
    const uint8_t* qptr[NW];
    const uint16_t* sptr[NW];
#pragma unroll
    for (int a = 0; a < NW; a++) {
        qptr[a] = (a ? qs2 : qs) + (size_t)blockIdx.x * 16 * row_bytes + (size_t)un0 * (KU * QB) + src_off_l;
        sptr[a] = (a ? scales2 : scales) + ((size_t)blockIdx.x * 16 + (lane & 15)) * nblk + (size_t)un0 * KU;
    }
    auto issue_next = [&](int buf) {
        if (iss_it < my_items && my_nun > 0) {
            const int row0 = ((int)blockIdx.x + iss_it * (int)gridDim.x) * 16;
            const uint32_t dst = ring0 + buf * C::UNIT_BYTES;
            if (row0 + 16 <= N) {
#pragma unroll
                for (int a = 0; a < NW; a++) {
#pragma unroll
                    for (int k = 0; k < C::PASSES; k++)
                        cp_async16(dst + a * C::MAT_BYTES + dst_off_l + k * (C::RPP * C::ROW_STRIDE), qptr[a] + k * src_step);
                    if (lane < 16) cp_async16(dst + a * C::MAT_BYTES + C::QS_BYTES + lane * 16, sptr[a]);
                }
            } else {                                                  // last item: rows past N repeat row N-1; never written
                const int un = un0 + iss_o;
#pragma unroll
                for (int a = 0; a < NW; a++) {
                    const uint8_t* wq = (a ? qs2 : qs) + (size_t)un * (KU * QB);
                    const uint16_t* ws = (a ? scales2 : scales) + (size_t)un * KU;
#pragma unroll
                    for (int k = 0; k < C::PASSES; k++) {
                        const int srow = min(row0 + k * C::RPP + lane / C::PPR, N - 1);
                        cp_async16(dst + a * C::MAT_BYTES + dst_off_l + k * (C::RPP * C::ROW_STRIDE),
                                   wq + (size_t)srow * row_bytes + (size_t)(lane % C::PPR) * 16);
                    }
                    if (lane < 16) cp_async16(dst + a * C::MAT_BYTES + C::QS_BYTES + lane * 16, ws + (size_t)min(row0 + lane, N - 1) * nblk);
                }
            }
            if (BREG || ++iss_o == my_nun) {
                iss_o = 0;
                iss_it++;
#pragma unroll
                for (int a = 0; a < NW; a++) {
                    qptr[a] += item_step_q - (size_t)(my_nun - 1) * (KU * QB);
                    sptr[a] += item_step_s - (size_t)(my_nun - 1) * KU;
                }
            } else {
#pragma unroll
                for (int a = 0; a < NW; a++) { qptr[a] += KU * QB; sptr[a] += KU; }
            }
        }
        cp_async_commit();
    };

    // Weights do not depend on the preceding kernel: the first NPRE units are requested before the
    // dependency wait. The rest of the ring follows right after this warp's loads of x, so that
    // those loads, which everything else waits for, do not queue behind a ring-full of copies.
#pragma unroll
    for (int i = 0; i < NPRE; i++) issue_next(i);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // tensor-parallel epilogue: sequence number of this all-reduce and the inbox buffer it uses
    const uint32_t tp_seq = TP ? tpws_seq(tpa.ws[tpa.rank], 1)[blockIdx.x] + 1 : 0u;
    const int tp_par = (int)(tp_seq & 1u);

    // ---- digits of this warp's units of x into the B table. Lane = (block lane>>3 (+4), elements
    // 4*(lane&7)..+3); a unit is 8 blocks = two such passes, loaded together.
    const int sub = lane & 7;
    // values of unit `un` this lane owns: fp32 x (raw; xmode 1, 2) with the norm weights, or rebuilt
    // from block-scaled digit records (xmode 0)
    auto load_unit = [&](int un, float (&e)[MT][2][4], uint2 (&wv)[2]) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int b = un * KU + (lane >> 3) + 4 * h;
            const int i = b * 32 + sub * 4;
            if (xmode == 2) wv[h] = *reinterpret_cast<const uint2*>(nw + i);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (xmode == 0) {
                    const uint32_t* rec = static_cast<const uint32_t*>(xin) + ((size_t)m * nblk + b) * XW;
                    const uint32_t w0 = rec[sub], w1 = rec[8 + sub], w2 = rec[16 + sub];
                    const float bs = __uint_as_float(rec[24]);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int X = ((int)(int8_t)(w0 >> (8 * k))) * 65536 + ((int)(int8_t)(w1 >> (8 * k))) * 256 + (int)(int8_t)(w2 >> (8 * k));
                        e[m][h][k] = (float)X * bs;
                    }
                } else {
                    const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(xin) + (size_t)m * K + i);
                    e[m][h][0] = v.x; e[m][h][1] = v.y; e[m][h][2] = v.z; e[m][h][3] = v.w;
                }
            }
        }
    };
    auto digits_unit = [&](int un, float (&e)[MT][2][4], const uint2 (&wv)[2], const float (&inv)[MT]) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (xmode == 2) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&wv[h].x));
                    const float2 w23 = __half22float2(*reinterpret_cast<const __half2*>(&wv[h].y));
                    e[m][h][0] = e[m][h][0] * inv[m] * w01.x; e[m][h][1] = e[m][h][1] * inv[m] * w01.y;
                    e[m][h][2] = e[m][h][2] * inv[m] * w23.x; e[m][h][3] = e[m][h][3] * inv[m] * w23.y;
                }
            }
            float amax = 0.f;
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int k = 0; k < 4; k++) amax = fmaxf(amax, fabsf(e[m][h][k]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float sc = amax > 0.f ? (float)XFULL / amax : 0.f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int b = un * KU + (lane >> 3) + 4 * h;
                // Z = (X + 0x8080) ^ 0x8080: its bytes 0, 1, 2 are the balanced digits d2, d1, d0 of X
                uint32_t Z[4];
#pragma unroll
                for (int k = 0; k < 4; k++) Z[k] = (uint32_t)(__float2int_rn(e[m][h][k] * sc) + 0x8080) ^ 0x8080u;
                const uint32_t t01 = __byte_perm(Z[0], Z[1], 0x5140), t23 = __byte_perm(Z[2], Z[3], 0x5140);
                const uint32_t u01 = __byte_perm(Z[0], Z[1], 0x0062), u23 = __byte_perm(Z[2], Z[3], 0x0062);
                uint32_t* dst = table + ((size_t)b * NC + m * 4) * 8 + (sub & 3) * 2 + (sub >> 2);
                dst[0] = __byte_perm(u01, u23, 0x5410);
                dst[8] = __byte_perm(t01, t23, 0x7632);
                dst[16] = __byte_perm(t01, t23, 0x5410);
                dst[24] = 0u;
            }
            if (lane == 0) xs_all[m * nun + un] = amax / (float)XFULL;
        }
    };

    float e0[MT][2][4];
    uint2 wv0[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
    if (my_nun > 0) load_unit(un0, e0, wv0);          // the loads everything waits for go first
#pragma unroll
    for (int i = NPRE; i < NBUF; i++) issue_next(i);
    {
        float inv[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) inv[m] = 1.f;
        if (xmode == 2) {                                            // sum of squares: every warp its units, then all
            const float* x = static_cast<const float*>(xin);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float ss = 0.f;
                if (my_nun > 0) {
#pragma unroll
                    for (int h = 0; h < 2; h++)
#pragma unroll
                        for (int k = 0; k < 4; k++) ss = fmaf(e0[m][h][k], e0[m][h][k], ss);
                }
                for (int i = KU * 32 + lane * 4; i < my_nun * KU * 32; i += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)un0 * KU * 32 + i);
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
        if (my_nun > 0) digits_unit(un0, e0, wv0, inv);
        for (int uo = 1; uo < my_nun; uo++) {
            float e[MT][2][4];
            uint2 wv[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
            load_unit(un0 + uo, e, wv);
            digits_unit(un0 + uo, e, wv, inv);
        }
    }
    __syncwarp();

    // B fragment of block b for MMA j and this thread: column 8j+g (n index), words t and 4+t of the plane
    auto load_b = [&](int b, int j, uint32_t& b0, uint32_t& b1) {
        if (8 * j + g < NC) {
            const uint2 v = *reinterpret_cast<const uint2*>(table + ((size_t)b * NC + 8 * j + g) * 8 + t * 2);
            b0 = v.x; b1 = v.y;
        } else { b0 = 0u; b1 = 0u; }
    };
    // row of x the accumulator columns of this thread belong to in MMA j: 2j + (t >> 1)
    const int xm0 = (MT >= 2) ? (t >> 1) : 0;

    uint32_t breg[BREG ? KU : 1][NM][2];
    float xs_reg[NM];
#pragma unroll
    for (int j = 0; j < NM; j++) xs_reg[j] = 0.f;
    if (BREG && my_nun > 0) {
#pragma unroll
        for (int i = 0; i < (BREG ? KU : 1); i++)
#pragma unroll
            for (int j = 0; j < NM; j++) load_b(un0 * KU + i, j, breg[i][j][0], breg[i][j][1]);
#pragma unroll
        for (int j = 0; j < NM; j++) xs_reg[j] = xs_all[min(2 * j + xm0, MT - 1) * nun + un0];
    }

    const uint32_t ld_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * C::ROW_STRIDE + (lane >> 4) * 16);
    const uint32_t nib_mask = 0xF0F0F0F0u, nib_flip = 0x80808080u;
    // One unit: 8 blocks x NM MMAs per weight; au[j][0/1] = the unit's sums of MMA j for rows g and g+8
    // before the scale of x.
    auto unit_mmas = [&](uint32_t mb, int blk0, float (&au)[NM][2]) {
        const uint4 sv = lds128(mb + C::QS_BYTES + g * 16), sw = lds128(mb + C::QS_BYTES + (g + 8) * 16);
        const uint32_t sgw[4] = {sv.x, sv.y, sv.z, sv.w}, sg8w[4] = {sw.x, sw.y, sw.z, sw.w};
        auto one_block = [&](int i, float d_lo, float d_hi, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
#pragma unroll
            for (int j = 0; j < NM; j++) {
                uint32_t b0, b1;
                if (BREG) { b0 = breg[BREG ? i : 0][j][0]; b1 = breg[BREG ? i : 0][j][1]; }
                else load_b(blk0 + i, j, b0, b1);
                int c0, c1, c2, c3;
                mma_s8(a0, a1, a2, a3, b0, b1, c0, c1, c2, c3);
                au[j][0] = fmaf((float)((c0 << 8) + c1), d_lo, au[j][0]);
                au[j][1] = fmaf((float)((c2 << 8) + c3), d_hi, au[j][1]);
            }
        };
#pragma unroll
        for (int p = 0; p < KU / 2; p++) {
            const float2 dlo = scales_of<QUIRK>(sgw[p]), dhi = scales_of<QUIRK>(sg8w[p]);
            uint32_t r0, r1, r2, r3;
            if (TYPE == CMLB200_Q4_0) {          // one ldmatrix: [rows 0-7 | 8-15] x [block 2p | 2p+1]
                ldmatrix_x4(mb + ld_off + p * 32, r0, r1, r2, r3);
                // nibble n in the top half of a byte, top bit flipped, reads as the int8 16*(n-8)
                one_block(2 * p, dlo.x, dhi.x, and_xor(r0 << 4, nib_mask, nib_flip), and_xor(r1 << 4, nib_mask, nib_flip),
                          and_xor(r0, nib_mask, nib_flip), and_xor(r1, nib_mask, nib_flip));
                one_block(2 * p + 1, dlo.y, dhi.y, and_xor(r2 << 4, nib_mask, nib_flip), and_xor(r3 << 4, nib_mask, nib_flip),
                          and_xor(r2, nib_mask, nib_flip), and_xor(r3, nib_mask, nib_flip));
            } else {                             // one ldmatrix per block: [rows 0-7 | 8-15] x [bytes 0-15 | 16-31]
                ldmatrix_x4(mb + ld_off + (2 * p) * 32, r0, r1, r2, r3);
                one_block(2 * p, dlo.x, dhi.x, r0, r1, r2, r3);
                ldmatrix_x4(mb + ld_off + (2 * p + 1) * 32, r0, r1, r2, r3);
                one_block(2 * p + 1, dlo.y, dhi.y, r0, r1, r2, r3);
            }
        }
    };

    // Results of FB items are parked in shared memory and the CTA meets once per FB items: the
    // threads of the first warps then add the 16 K-slices of every row in warp order and write y.
    const float wgt = ((t & 1) ? (1.0f / 256.0f) : 256.0f) * ((TYPE == CMLB200_Q4_0) ? 0.0625f : 1.0f);
    float* my_part = partial + (size_t)warp * (NW * MT * 16) + xm0 * 16 + g;     // + slot * SW*NW*MT*16 + a * MT*16 + 2j * 16
    const bool even_t = (t & 1) == 0;
    auto flush = [&](int it_first, int count) {              // items it_first .. it_first+count-1 sit in slots 0..count-1
        __syncthreads();
        for (int idx = threadIdx.x; idx < count * MT * 16; idx += SW * 32) {
            const int r = idx & 15, m = (idx >> 4) % MT, slot = idx / (16 * MT);
            const int row = ((int)blockIdx.x + (it_first + slot) * (int)gridDim.x) * 16 + r;
            if (row < N) {
                float sum[NW];
#pragma unroll
                for (int a = 0; a < NW; a++) {
                    const float* src = partial + (size_t)slot * (SW * NW * MT * 16) + a * (MT * 16) + m * 16 + r;
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < SW; w++) v += src[w * (NW * MT * 16)];
                    sum[a] = v;
                }
                float* out = y + (size_t)m * N + row;
                if (NW == 2) *out = (sum[0] / (1.0f + expf(-sum[0]))) * sum[NW - 1];
                else if (TP) {                               // this rank's share goes to every rank's inbox, its own included
                    for (int qr = 0; qr < tpa.tp; qr++)
                        st_packet_sys(reinterpret_cast<uint2*>(tpws_inbox(tpa.ws[qr], 1, tp_par, tpa.rank, tpa.max_floats)) + (size_t)m * N + row, sum[0], tp_seq);
                } else if (epi == EPI_ACCUM) *out += sum[0];
                else *out = sum[0];
            }
        }
        __syncthreads();
    };

    int u = 0;
    for (int it = 0; it < my_items; it++) {
        float acc[NW][NM][2];        // rows g and g+8 of MMA j: sum over blocks of scales * (c_even * 256 + c_odd)
#pragma unroll
        for (int a = 0; a < NW; a++)
#pragma unroll
            for (int j = 0; j < NM; j++) { acc[a][j][0] = 0.f; acc[a][j][1] = 0.f; }

        for (int o = 0; o < (BREG ? min(my_nun, 1) : my_nun); o++, u++) {
            const int buf = u % NBUF;
            cp_async_wait<NBUF - 1>();
            __syncwarp();
            const uint32_t ub = ring0 + buf * C::UNIT_BYTES;
            float xs[NM];
#pragma unroll
            for (int j = 0; j < NM; j++) xs[j] = BREG ? xs_reg[j] : xs_all[min(2 * j + xm0, MT - 1) * nun + un0 + o];
            {
#pragma unroll
                for (int a = 0; a < NW; a++) {
                    float au[NM][2];
#pragma unroll
                    for (int j = 0; j < NM; j++) { au[j][0] = 0.f; au[j][1] = 0.f; }
                    unit_mmas(ub + a * C::MAT_BYTES, (un0 + o) * KU, au);
#pragma unroll
                    for (int j = 0; j < NM; j++) {
                        acc[a][j][0] = fmaf(au[j][0], xs[j], acc[a][j][0]);
                        acc[a][j][1] = fmaf(au[j][1], xs[j], acc[a][j][1]);
                    }
                }
            }
            __syncwarp();                                    // every lane is done with this buffer
            issue_next(buf);
        }

        // ---- combine the column pairs (t even: d0*256 + d1, t odd: d2*256) and park the item
        const int slot = it % FB;
#pragma unroll
        for (int a = 0; a < NW; a++)
#pragma unroll
            for (int j = 0; j < NM; j++) {
                float p_lo = acc[a][j][0] * wgt, p_hi = acc[a][j][1] * wgt;
                p_lo += __shfl_xor_sync(0xffffffffu, p_lo, 1);
                p_hi += __shfl_xor_sync(0xffffffffu, p_hi, 1);
                if (even_t && 2 * j + xm0 < MT) {
                    float* dst = my_part + (size_t)slot * (SW * NW * MT * 16) + a * (MT * 16) + 2 * j * 16;
                    dst[0] = p_lo;
                    dst[8] = p_hi;
                }
            }
        if (slot == FB - 1 || it == my_items - 1) flush(it - slot, slot + 1);
    }
    cp_async_wait<0>();
    if (TP) {
        // All rows of this CTA are on their way to every rank as (value, sequence) packets. Collect
        // the packets of all ranks for the same rows (they carry this all-reduce's sequence number
        // once they have landed) and add them in rank order onto the residual.
        uint8_t* mine = tpa.ws[tpa.rank];
        for (int idx = threadIdx.x; idx < my_items * MT * 16; idx += SW * 32) {
            const int r = idx & 15, m = (idx >> 4) % MT, it = idx / (16 * MT);
            const int row = ((int)blockIdx.x + it * (int)gridDim.x) * 16 + r;
            if (row < N) {
                const size_t at = (size_t)m * N + row;
                float v = 0.f;
                bool ok = true;
                for (int qr = 0; qr < tpa.tp && ok; qr++) {
                    const uint2* src = reinterpret_cast<const uint2*>(tpws_inbox(mine, 1, tp_par, qr, tpa.max_floats)) + at;
                    uint2 pkt = ld_packet_sys(src);
                    for (int i = 0; pkt.y != tp_seq && i < tpa.spin_limit; i++) pkt = ld_packet_sys(src);
                    if (pkt.y != tp_seq) { ok = false; atomicExch(tpws_status(mine), 1u + qr); }
                    v += __uint_as_float(pkt.x);
                }
                if (ok) tpa.h[at] += v;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) tpws_seq(mine, 1)[blockIdx.x] = tp_seq;
    }
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
    return (size_t)nblk * 4 * MT * 32 + ((((size_t)MT * (nblk / KU) + 31) & ~(size_t)31) + flush_batch(NW, MT) * SW * NW * MT * 16) * sizeof(float) +
           (size_t)SW * nbuf * Cfg<TYPE, NW>::UNIT_BYTES;
}

template <int TYPE, int MT, int NW, bool QUIRK, bool BREG, int NBUF, int NPRE, bool TP>
int launch_cfg(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, int xmode, int epi,
               const TpPeers& tpa, cudaStream_t st) {
    const int N = W->rows, K = W->cols;
    const size_t smem = smem_bytes<TYPE, NW>(MT, K / 32, NBUF);
    auto kern = gemv_mma_kernel<TYPE, MT, NW, QUIRK, BREG, NBUF, NPRE, TP>;
    static size_t attr_smem[kMaxDevices] = {};
    CMLB_CUDA(cmlb_ensure_smem(kern, smem, attr_smem));
    const int grid = min(cmlb_num_sms(), (N + 15) / 16);
    return launch_pdl(kern, dim3(grid), dim3(SW * 32), smem, st, (const uint8_t*)W->qs, (const uint16_t*)W->scales,
                      W2 ? (const uint8_t*)W2->qs : (const uint8_t*)nullptr,
                      W2 ? (const uint16_t*)W2->scales : (const uint16_t*)nullptr, xin, nw, eps, y, N, K, xmode, epi, tpa);
}

// Ring depth 2, one unit of it requested before the dependency wait. Measured on the 11008 x 4096
// case: (2 buffers, 1 before the wait) 6.43 us, (2, 2) 6.52, (3, 1) 6.56, (4, 1) 7.01: more copies in
// flight do not help a loop that is issue-bound, and they get in the way of the loads of x.
constexpr int kNbuf = 2, kNpre = 1;

template <int TYPE, int NW>
bool fits_smem(int MT, int nblk) { return smem_bytes<TYPE, NW>(MT, nblk, kNbuf) <= kSmemLimit; }

template <int TYPE, int MT, int NW, bool QUIRK, bool BREG, bool TP>
int launch_ring(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, int xmode, int epi,
                const TpPeers& tpa, cudaStream_t st) {
    return launch_cfg<TYPE, MT, NW, QUIRK, BREG, kNbuf, kNpre, TP>(W, W2, xin, nw, eps, y, xmode, epi, tpa, st);
}

template <int TYPE, int MT, int NW, bool QUIRK, bool BREG>
int launch_b(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, int xmode, int epi,
             const TpPeers& tpa, cudaStream_t st) {
    CMLB_REQUIRE((fits_smem<TYPE, NW>(MT, W->cols / 32)), "cmlb200_gemv: K=%d does not fit the tensor-core decode kernel", W->cols);
    if (NW == 1 && tpa.tp) return launch_ring<TYPE, MT, 1, QUIRK, BREG, true>(W, W2, xin, nw, eps, y, xmode, epi, tpa, st);
    return launch_ring<TYPE, MT, NW, QUIRK, BREG, false>(W, W2, xin, nw, eps, y, xmode, epi, tpa, st);
}

template <int TYPE, int MT, int NW, bool QUIRK>
int launch(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, int xmode, int epi,
           const TpPeers& tpa, cudaStream_t st) {
    if (W->cols / (32 * KU) <= SW) return launch_b<TYPE, MT, NW, QUIRK, true>(W, W2, xin, nw, eps, y, xmode, epi, tpa, st);
    return launch_b<TYPE, MT, NW, QUIRK, false>(W, W2, xin, nw, eps, y, xmode, epi, tpa, st);
}

// Rows of x four at a time when the digit table fits (one launch streams the weight once for
// all of them), then two, then one.
template <int TYPE, int NW, bool QUIRK>
int run_m(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, size_t x_row_bytes, const __half* nw, float eps, float* y, int M,
          int xmode, int epi, const TpPeers& tp0, cudaStream_t st) {
    int m0 = 0, rc = 0;
    while (m0 < M && rc == 0) {
        const void* xm = static_cast<const uint8_t*>(xin) + (size_t)m0 * x_row_bytes;
        float* ym = y + (size_t)m0 * W->rows;
        TpPeers tpa = tp0;
        if (tpa.tp) tpa.h = tp0.h + (size_t)m0 * W->rows;
        const int nblk = W->cols / 32, left = M - m0;
        if (left >= 4 && fits_smem<TYPE, NW>(4, nblk)) { rc = launch<TYPE, 4, NW, QUIRK>(W, W2, xm, nw, eps, ym, xmode, epi, tpa, st); m0 += 4; }
        else if (left >= 2 && fits_smem<TYPE, NW>(2, nblk)) { rc = launch<TYPE, 2, NW, QUIRK>(W, W2, xm, nw, eps, ym, xmode, epi, tpa, st); m0 += 2; }
        else { rc = launch<TYPE, 1, NW, QUIRK>(W, W2, xm, nw, eps, ym, xmode, epi, tpa, st); m0 += 1; }
    }
    return rc;
}

template <int TYPE, bool QUIRK>
int run_x(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const __half* nw, float eps, const uint32_t* xq, float* y, int M,
          int epi, const TpPeers& tpa, cudaStream_t st) {
    const int K = W->cols;
    const void* xin = xq ? (const void*)xq : (const void*)x;
    const size_t xrb = xq ? (size_t)(K / 32) * XW * 4 : (size_t)K * 4;
    const int xmode = xq ? 0 : (nw ? 2 : 1);
    if (epi == EPI_SWIGLU) return run_m<TYPE, 2, QUIRK>(W, W2, xin, xrb, nw, eps, y, M, xmode, epi, tpa, st);
    return run_m<TYPE, 1, QUIRK>(W, W2, xin, xrb, nw, eps, y, M, xmode, epi, tpa, st);
}

template <int TYPE>
bool fits(int nblk, int epi, int mt) {
    return epi == EPI_SWIGLU ? fits_smem<TYPE, 2>(mt, nblk) : fits_smem<TYPE, 1>(mt, nblk);
}

}  // namespace

// Shapes the tensor-core decode kernel takes: whole 8-block slices of K with 16-byte aligned
// scale rows, and room in shared memory for the digit table of two rows of x next to the rings.
bool cmlb200_gemv_mma_ok_(const cmlb200_qmat* W, int epi, int M) {
    if (W->type != CMLB200_Q4_0 && W->type != CMLB200_Q8_0) return false;
    if (W->cols % 256 != 0 || ((uintptr_t)W->qs & 15) || ((uintptr_t)W->scales & 15)) return false;
    const int nblk = W->cols / 32;
    (void)M;                                   // rows of x go four, two or one per launch, whatever fits
    return W->type == CMLB200_Q8_0 ? fits<CMLB200_Q8_0>(nblk, epi, 1) : fits<CMLB200_Q4_0>(nblk, epi, 1);
}

// Rows of x one launch of the tensor-core decode kernel takes for this weight: 4, 2, 1, or 0 when
// the shape is outside the kernel.
int cmlb200_gemv_mma_rows_(const cmlb200_qmat* W, int epi) {
    if (!cmlb200_gemv_mma_ok_(W, epi, 1)) return 0;
    const int nblk = W->cols / 32;
    const bool q8 = W->type == CMLB200_Q8_0;
    for (int mt = 4; mt >= 2; mt >>= 1)
        if (q8 ? fits<CMLB200_Q8_0>(nblk, epi, mt) : fits<CMLB200_Q4_0>(nblk, epi, mt)) return mt;
    return 1;
}

// y[M, rows] (= | += | swiglu) for M <= 4. Exactly one of xq (digit records) and x (fp32, with
// optional RMSNorm weight norm_w) is given. Arguments are validated by the callers.
static int run_all(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                   const uint32_t* xq, float* y, int M, int epi, const TpPeers& tpa, cudaStream_t st) {
    const __half* nw = reinterpret_cast<const __half*>(norm_w);
    const bool quirk = (W->flags & CMLB200_QMAT_SUBNORMAL_SCALES) || (W2 && (W2->flags & CMLB200_QMAT_SUBNORMAL_SCALES));
    const bool q8 = W->type == CMLB200_Q8_0;
    if (quirk) return q8 ? run_x<CMLB200_Q8_0, true>(W, W2, x, nw, eps, xq, y, M, epi, tpa, st) : run_x<CMLB200_Q4_0, true>(W, W2, x, nw, eps, xq, y, M, epi, tpa, st);
    return q8 ? run_x<CMLB200_Q8_0, false>(W, W2, x, nw, eps, xq, y, M, epi, tpa, st) : run_x<CMLB200_Q4_0, false>(W, W2, x, nw, eps, xq, y, M, epi, tpa, st);
}

int cmlb200_gemv_mma_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                      const uint32_t* xq, float* y, int M, int epi, cudaStream_t st) {
    return run_all(W, W2, x, norm_w, eps, xq, y, M, epi, TpPeers{}, st);
}

// Row-parallel projection of a tensor-parallel layer with the all-reduce in its epilogue:
// h[M, rows] += sum over ranks of x_rank . dequant(W_rank)^T (src/nn/llama.c:523-530, 538-543 with
// src/distributed/tensor_parallel.c:195-260 in between). One launch per rank: every CTA sends
// the rows it finishes to all ranks' inboxes as (value, sequence) packets and, once its items
// are done, adds the packets of all ranks for its rows in rank order. All projections that use one workspace must have the same `rows`, since
// the flags are kept per CTA and the CTA-to-rows mapping depends on rows alone.
extern "C" int cmlb200_gemv_tp_allreduce(const cmlb200_qmat* W, const float* d_x, float* d_h, int M, int tp, int rank, void* const* ws,
                                         size_t max_floats, void* stream) {
    CMLB_REQUIRE(W && W->qs && W->scales && d_x && d_h && ws, "cmlb200_gemv_tp_allreduce: NULL argument");
    CMLB_REQUIRE(M >= 1 && M <= 4, "cmlb200_gemv_tp_allreduce: M=%d outside 1..4", M);
    CMLB_REQUIRE(tp >= 2 && tp <= kTpMaxRanks && rank >= 0 && rank < tp, "cmlb200_gemv_tp_allreduce: tp=%d rank=%d (tp must be 2..8)", tp, rank);
    CMLB_REQUIRE(cmlb200_gemv_mma_ok_(W, EPI_STORE, M), "cmlb200_gemv_tp_allreduce: weight %dx%d type %d is outside the tensor-core decode kernel", W->rows, W->cols, W->type);
    CMLB_REQUIRE((size_t)M * W->rows * 2 <= max_floats, "cmlb200_gemv_tp_allreduce: M*rows = %zu exceeds the workspace (max_floats / 2)", (size_t)M * W->rows);
    CMLB_REQUIRE(cmlb_num_sms() <= kTpGemvSlices, "cmlb200_gemv_tp_allreduce: more than %d SMs", kTpGemvSlices);
    CMLB_REQUIRE(((uintptr_t)d_x & 15) == 0, "cmlb200_gemv_tp_allreduce: x must be 16-byte aligned");
    TpPeers p = {};
    for (int r = 0; r < tp; r++) {
        CMLB_REQUIRE(ws[r], "cmlb200_gemv_tp_allreduce: workspace of rank %d missing", r);
        p.ws[r] = static_cast<uint8_t*>(ws[r]);
    }
    p.tp = tp; p.rank = rank; p.max_floats = max_floats; p.h = d_h;
    p.spin_limit = cmlb_tp_spin_limit();
    return run_all(W, nullptr, d_x, nullptr, 0.f, nullptr, d_h, M, EPI_STORE, p, as_stream(stream));
}

extern "C" int cmlb200_gemv_tp_fused_ok(const cmlb200_qmat* W, int M) {
    return W && W->qs && W->scales && M >= 1 && M <= 4 && cmlb200_gemv_mma_ok_(W, EPI_STORE, M) && cmlb_num_sms() <= kTpGemvSlices ? 1 : 0;
}
