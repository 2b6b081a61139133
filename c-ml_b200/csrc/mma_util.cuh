// Small wrappers around the instructions the mma.sync decode kernels are built from: 16-byte
// cp.async copies, ldmatrix over 16-byte block rows, the one-instruction nibble-to-int8 logic
// operation, the int8 m16n8k32 MMA and the widening of packed fp16 block scales.
#pragma once
#include "common.cuh"

namespace {

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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// (a & m) ^ c in one logic instruction
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t m, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(m), "r"(c));
    return d;
}
// D = A(16x32 s8, row) * B(32x8 s8, col)
__device__ __forceinline__ void mma_s8(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                       int& d0, int& d1, int& d2, int& d3) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}

// The two fp16 scales packed in one word, widened (with C-ML's subnormal rule when QUIRK).
template <bool QUIRK>
__device__ __forceinline__ float2 scales_of(uint32_t packed) {
    if (QUIRK) return make_float2(cml_half_to_float((uint16_t)(packed & 0xFFFFu)), cml_half_to_float((uint16_t)(packed >> 16)));
    return __half22float2(*reinterpret_cast<const __half2*>(&packed));
}

}  // namespace
