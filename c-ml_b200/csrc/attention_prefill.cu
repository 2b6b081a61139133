// Causal grouped-query attention for prompt-sized calls (many query rows of ONE sequence against
// that sequence's fp16 KV cache): softmax(Q K^T / sqrt(d) + mask) V, the computation of C-ML's
// cml_gqa_forward (src/nn/llm_ops.c:243-372) as llama.c drives it (src/nn/llama.c:490-521), tiled so
// that every key and value is read once per 64 query rows instead of once per row.
//
// One CTA = 64 query rows of one head (4 warps x 16 rows); keys in tiles of 64 staged in shared
// memory with cp.async. Per tile and warp: S = Q K^T on mma.sync m16n8k16 (fp16 operands, fp32
// accumulators; Q is pre-scaled by log2(e)/sqrt(d) so the softmax uses exp2), the mask from each
// row's own limit (the last cache slot it may attend, so absolute or call-relative masking is the
// caller's choice), running row maximum and sum, P rounded to fp16 and fed straight from the
// accumulator registers as the A operand of O += P V, V fragments through ldmatrix.trans.
// Output: fp32 [rows, heads*d] and / or bf16 (the next GEMM's operand). Tolerance of this path is
// that of the bf16 prefill pipeline (1e-2 of the largest logit): Q, K, V, P enter the MMAs as fp16.
#include <cuda_fp16.h>
#include "common.cuh"

namespace {

constexpr int QT = 64;            // query rows per CTA
constexpr int KT = 64;            // keys per tile
constexpr int THREADS_P = 128;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(THREADS_P)
attention_prefill_kernel(const float* __restrict__ q, int q_stride, const __half* __restrict__ kc, const __half* __restrict__ vc,
                         const int* __restrict__ row_limit, int rows, int heads, int kv_heads, int max_seq,
                         float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
    constexpr int LD = HD + 8;                         // padded row: fragment loads and ldmatrix rows spread over the banks
    __shared__ __align__(16) __half Ks[KT][LD];
    __shared__ __align__(16) __half Vs[KT][LD];
    __shared__ int s_kmax;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y, kh = h / (heads / kv_heads), kvw = kv_heads * HD;
    const int r0 = blockIdx.x * QT + warp * 16 + g, r1 = r0 + 8;
    const int lim0 = r0 < rows ? row_limit[r0] : -1, lim1 = r1 < rows ? row_limit[r1] : -1;
    if (threadIdx.x == 0) s_kmax = -1;
    __syncthreads();
    atomicMax(&s_kmax, max(lim0, lim1));

    // Q fragments of this warp's 16 rows, scaled so that exp2 of a score is exp of the true score
    const float qs = 1.4426950408889634f / sqrtf((float)HD);
    uint32_t qa[HD / 16][4];
    {
        const float* q0 = q + (size_t)min(r0, rows - 1) * q_stride + (size_t)h * HD;
        const float* q1 = q + (size_t)min(r1, rows - 1) * q_stride + (size_t)h * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
            const float2 a = *reinterpret_cast<const float2*>(q0 + 16 * kk + 2 * t), b = *reinterpret_cast<const float2*>(q1 + 16 * kk + 2 * t);
            const float2 c = *reinterpret_cast<const float2*>(q0 + 16 * kk + 2 * t + 8), d = *reinterpret_cast<const float2*>(q1 + 16 * kk + 2 * t + 8);
            qa[kk][0] = pack_h2(a.x * qs, a.y * qs);
            qa[kk][1] = pack_h2(b.x * qs, b.y * qs);
            qa[kk][2] = pack_h2(c.x * qs, c.y * qs);
            qa[kk][3] = pack_h2(d.x * qs, d.y * qs);
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    __syncthreads();
    const int kmax = min(s_kmax, max_seq - 1);
    const size_t head_off = (size_t)kh * HD;

    for (int kt = 0; kt <= kmax; kt += KT) {
        __syncthreads();                                    // the previous tile is no longer read
        for (int i = threadIdx.x; i < KT * (HD / 8); i += THREADS_P) {
            const int row = i / (HD / 8), ch = i % (HD / 8);
            const size_t src = (size_t)min(kt + row, max_seq - 1) * kvw + head_off + ch * 8;
            cp16(smem_addr(&Ks[row][ch * 8]), kc + src);
            cp16(smem_addr(&Vs[row][ch * 8]), vc + src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (__all_sync(0xffffffffu, kt > max(lim0, lim1))) continue;     // nothing in this tile is visible to this warp's rows

        // ---- S = Q K^T for 16 rows x 64 keys
        float s[KT / 8][4];
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++) {
            s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&Ks[nt * 8 + g][16 * kk + 2 * t]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&Ks[nt * 8 + g][16 * kk + 2 * t + 8]);
                mma_f16(s[nt], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
            }
        }
        // ---- mask by each row's limit, running maximum and sum
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++) {
            const int key = kt + nt * 8 + 2 * t;
            if (key > lim0) s[nt][0] = -INFINITY;
            if (key + 1 > lim0) s[nt][1] = -INFINITY;
            if (key > lim1) s[nt][2] = -INFINITY;
            if (key + 1 > lim1) s[nt][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;    // a row with nothing visible yet
        const float c0 = exp2f(m0 - u0), c1 = exp2f(m1 - u1);
        m0 = n0; m1 = n1;
        l0 *= c0; l1 *= c1;
#pragma unroll
        for (int i = 0; i < HD / 8; i++) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        uint32_t pa[KT / 16][4];
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++) {
            const float p0 = exp2f(s[nt][0] - u0), p1 = exp2f(s[nt][1] - u0), p2 = exp2f(s[nt][2] - u1), p3 = exp2f(s[nt][3] - u1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            pa[nt >> 1][(nt & 1) * 2] = pack_h2(p0, p1);          // keys 2t, 2t+1 (+8 for the odd tile): A registers 0 / 2 (row g)
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(p2, p3);      // A registers 1 / 3 (row g + 8)
        }
        // ---- O += P V: V fragments transposed by ldmatrix from the [key][d] tile
#pragma unroll
        for (int j = 0; j < KT / 16; j++) {
#pragma unroll
            for (int nt2 = 0; nt2 < HD / 8; nt2 += 2) {
                uint32_t v0, v1, v2, v3;
                const uint32_t addr = smem_addr(&Vs[16 * j + (lane & 15)][(nt2 + (lane >> 4)) * 8]);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(addr) : "memory");
                mma_f16(o[nt2], pa[j][0], pa[j][1], pa[j][2], pa[j][3], v0, v1);
                mma_f16(o[nt2 + 1], pa[j][0], pa[j][1], pa[j][2], pa[j][3], v2, v3);
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    const size_t ow = (size_t)heads * HD;
#pragma unroll
    for (int nt2 = 0; nt2 < HD / 8; nt2++) {
        const int col = h * HD + nt2 * 8 + 2 * t;
        if (r0 < rows) {
            if (out_f32) *reinterpret_cast<float2*>(out_f32 + (size_t)r0 * ow + col) = make_float2(o[nt2][0] * i0, o[nt2][1] * i0);
            if (out_bf16) *reinterpret_cast<__nv_bfloat162*>(out_bf16 + (size_t)r0 * ow + col) = __floats2bfloat162_rn(o[nt2][0] * i0, o[nt2][1] * i0);
        }
        if (r1 < rows) {
            if (out_f32) *reinterpret_cast<float2*>(out_f32 + (size_t)r1 * ow + col) = make_float2(o[nt2][2] * i1, o[nt2][3] * i1);
            if (out_bf16) *reinterpret_cast<__nv_bfloat162*>(out_bf16 + (size_t)r1 * ow + col) = __floats2bfloat162_rn(o[nt2][2] * i1, o[nt2][3] * i1);
        }
    }
}

}  // namespace

// rows query rows of sequence `seq` (Q rows q_stride floats apart, already rotated) against that
// sequence's fp16 cache [n_seq, max_seq, kv_heads*head_dim]; row r attends cache slots 0..d_row_limit[r].
// head_dim 64 or 128. Writes fp32 and / or bf16 [rows, heads*head_dim] (either pointer may be NULL).
extern "C" int cmlb200_attention_prefill(const float* d_q, int q_stride, const void* d_kcache_f16, const void* d_vcache_f16, int seq,
                                         const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq,
                                         float* d_out_f32, uint16_t* d_out_bf16, void* stream) {
    CMLB_REQUIRE(d_q && d_kcache_f16 && d_vcache_f16 && d_row_limit && (d_out_f32 || d_out_bf16), "cmlb200_attention_prefill: NULL argument");
    CMLB_REQUIRE(rows > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && seq >= 0 && max_seq > 0,
                 "cmlb200_attention_prefill: num_heads (%d) must be divisible by num_kv_heads (%d)", heads, kv_heads);
    CMLB_REQUIRE(head_dim == 64 || head_dim == 128, "cmlb200_attention_prefill: head_dim %d not in {64, 128}", head_dim);
    CMLB_REQUIRE(q_stride >= heads * head_dim && q_stride % 2 == 0 && ((uintptr_t)d_q & 7) == 0, "cmlb200_attention_prefill: q_stride %d / alignment of Q", q_stride);
    CMLB_REQUIRE(((uintptr_t)d_kcache_f16 & 15) == 0 && ((uintptr_t)d_vcache_f16 & 15) == 0, "cmlb200_attention_prefill: the caches must be 16-byte aligned");
    const size_t seq_off = (size_t)seq * max_seq * kv_heads * head_dim;
    const __half* kc = static_cast<const __half*>(d_kcache_f16) + seq_off;
    const __half* vc = static_cast<const __half*>(d_vcache_f16) + seq_off;
    const dim3 grid((rows + QT - 1) / QT, heads);
    cudaStream_t st = as_stream(stream);
    if (head_dim == 128)
        attention_prefill_kernel<128><<<grid, THREADS_P, 0, st>>>(d_q, q_stride, kc, vc, d_row_limit, rows, heads, kv_heads, max_seq, d_out_f32, (__nv_bfloat16*)d_out_bf16);
    else
        attention_prefill_kernel<64><<<grid, THREADS_P, 0, st>>>(d_q, q_stride, kc, vc, d_row_limit, rows, heads, kv_heads, max_seq, d_out_f32, (__nv_bfloat16*)d_out_bf16);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
