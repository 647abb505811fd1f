// Building blocks of the integer warp-MMA mat-vec kernels (jq_qgemv_pint.cu, jq_qgemv_stream.cu):
// the u8 x s8 -> s32 m16n8k32 MMA wrappers, small cp.async forms and the shift-free unpack of 2-, 4- and
// 8-bit codes into byte operands.
//
// Shift-free unpack: a code stays at its bit position p inside its byte, A = word & (mask << p) = 2^p * q,
// and the activation that meets it is scaled by 2^-p before it is cut into limbs (exact: a power of two).
// A 32-bit word of codes costs one AND per operand register.
#pragma once

#include "jq_mma.cuh"

namespace jq {
namespace imma_ops {

__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// same with a zero accumulator input (starts a new sum without clearing registers)
__device__ __forceinline__ void imma0(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                      uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// The lane's 16 codes of a 64-code block (u[], code j at bit j*BITS) -> 4 registers of 4 bytes, without
// shifts.  Register i, byte t holds code elem(i, t) times 2^code_shift(elem(i, t)).
template <int BITS>
__device__ __forceinline__ void to_bytes(const uint32_t (&u)[Unit<BITS>::WORDS], uint32_t (&r)[4]) {
    if constexpr (BITS == 8) {
        r[0] = u[0]; r[1] = u[1]; r[2] = u[2]; r[3] = u[3];
    } else if constexpr (BITS == 4) {
        r[0] = u[0] & 0x0F0F0F0Fu; r[1] = u[0] & 0xF0F0F0F0u;
        r[2] = u[1] & 0x0F0F0F0Fu; r[3] = u[1] & 0xF0F0F0F0u;
    } else if constexpr (BITS == 6) {
        // 16 codes = 96 bits = four groups of 24 bits (4 codes each).  A group g = c0 | c1 << 6 | c2 << 12 |
        // c3 << 18 becomes the bytes (c0, c1, c2, c3) in two steps: the upper pair moves to the high half,
        // then the odd code of each half moves up by two bits.  Bits above the group's 24 fall out in the masks.
        const uint32_t grp[4] = {u[0], funnel_r(u[0], u[1], 24), funnel_r(u[1], u[2], 16), u[2] >> 8};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t h = (grp[i] & 0x0000FFFFu) | ((grp[i] << 4) & 0xFFFF0000u);
            r[i] = (h & 0x003F003Fu) | ((h << 2) & 0x3F003F00u);
        }
    } else {
        static_assert(BITS == 2, "widths of the integer kernels: 2, 4, 6, 8");
        r[0] = u[0] & 0x03030303u; r[1] = u[0] & 0x0C0C0C0Cu;
        r[2] = u[0] & 0x30303030u; r[3] = u[0] & 0xC0C0C0C0u;
    }
}
// 3-bit codes: the lane's 16 codes are two units of 8 codes = 24 bits.  Inside a unit six codes sit whole inside
// one of its three bytes (c0, c1 in byte 0; c3, c4 in byte 1; c6, c7 in byte 2) and are taken with one AND each
// way; the two that straddle a byte boundary (c2, c5) need one shift of the unit.  A unit thus becomes three
// operand registers with the bytes (c0, 2 c3, 4 c6, 0), (8 c1, 16 c4, 32 c7, 0), (c2, 2 c5, 0, 0): 8 codes on 12 byte
// positions, so a 64-code block takes three MMAs instead of two; the activation limbs leave the same gaps.
__device__ __forceinline__ void to_bytes3(const uint32_t (&u)[2], uint32_t (&r)[6]) {
    const uint32_t g0 = u[0], g1 = funnel_r(u[0], u[1], 24);
    r[0] = g0 & 0x001C0E07u; r[1] = g0 & 0x00E07038u; r[2] = (g0 >> 6) & 0x00000E07u;
    r[3] = g1 & 0x001C0E07u; r[4] = g1 & 0x00E07038u; r[5] = (g1 >> 6) & 0x00000E07u;
}
template <int BITS> __host__ __device__ constexpr int elem(int i, int t) {
    return BITS == 2 ? i + 4 * t : BITS == 4 ? 8 * (i >> 1) + (i & 1) + 2 * t : 4 * i + t;
}
// log2 of the factor the code of element j carries inside its byte
template <int BITS> __host__ __device__ constexpr int code_shift(int j) {
    return BITS == 2 ? 2 * (j & 3) : BITS == 4 ? 4 * (j & 1)
         : BITS == 3 ? ((j & 7) == 1 ? 3 : (j & 7) == 3 ? 1 : (j & 7) == 4 ? 4 : (j & 7) == 5 ? 1 : (j & 7) == 6 ? 2
                        : (j & 7) == 7 ? 5 : 0)
         : 0;
}

}  // namespace imma_ops
}  // namespace jq
