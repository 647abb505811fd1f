// Warp-level building blocks shared by the mat-vec (K2) and MoE-decode kernels:
// mbarrier + bulk-copy wrappers with bounded waits, the register dequantizer
// that turns packed codes into bf16/f16 tensor-core operands, and the
// m16n8k16 MMA wrappers.
//
// Register dequantization.  A code q of BITS bits is placed, still inside the
// packed word, at the top of the 16-bit float's mantissa and OR-ed with the
// exponent of 2^MANT (MANT = 7 for bf16, 10 for f16):
//     value = 2^MANT + q * 2^(MANT-FB) = 2^(MANT-FB) * (2^FB + q)        (exact)
// One shift plus one LOP3 converts two codes (the two halves of a register).
// The constant 2^FB term is removed after the MMA with sum(x) of the group, so
// no per-weight subtract or int->float conversion is issued.  8-bit codes do
// not fit a bf16 mantissa and are split into two 4-bit fields (two MMAs).
#pragma once

#include "jq_common.cuh"

namespace jq {

// ---- shared-memory address / mbarrier / bulk copy -----------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ unsigned long long wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// A wait gives up only when BOTH its poll budget is spent AND this much wall time has passed since its first
// clock reading: a poll count alone runs out under a profiler or time-slicing although nothing is wrong.
constexpr unsigned long long MBAR_WAIT_NS = 1000000000ull;

// Bounded wait on a phase parity.  Returns false when the limit ran out (the
// caller records an error and leaves instead of spinning for ever).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t max_polls = (1u << 20)) {
    const uint32_t addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((i & 1023u) == 1023u) {
            const unsigned long long now = wall_ns();
            if (t0 == 0) t0 = now;
            else if (i >= max_polls && now - t0 > MBAR_WAIT_NS) return false;
        }
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// The bit-manipulation helpers below also compile for the host so that the
// fragment mapping can be checked by emulation without a GPU.
// 16-byte asynchronous copy global -> shared (L2-only caching: streamed once)
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__host__ __device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#ifdef __CUDA_ARCH__
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
#else
    const unsigned long long ab = ((unsigned long long)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) r |= (uint32_t)((ab >> (8 * ((sel >> (4 * i)) & 7))) & 0xFFu) << (8 * i);
    return r;
#endif
}

// (a & b) | c
__host__ __device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
#ifdef __CUDA_ARCH__
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
#else
    return (a & b) | c;
#endif
}

// low 32 bits of (hi:lo) >> s, 0 <= s < 32
__host__ __device__ __forceinline__ uint32_t funnel_r(uint32_t lo, uint32_t hi, int s) {
#ifdef __CUDA_ARCH__
    return __funnelshift_r(lo, hi, s);
#else
    return s == 0 ? lo : (lo >> s) | (hi << (32 - s));
#endif
}

// ---- activation-type traits ------------------------------------------------------
template <typename AT> struct Act;

template <> struct Act<__nv_bfloat16> {
    static constexpr int MANT = 7;
    static constexpr uint32_t MAGIC = 0x43004300u;   // 2^7 in both halves
    static constexpr uint32_t ONES = 0x3F803F80u;    // 1.0, 1.0
    __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    // same with a zero accumulator input (starts a new sum without clearing registers)
    __device__ static __forceinline__ void mma0(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%10,%10,%10,%10};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
    __device__ static __forceinline__ uint32_t pack_hi(float a, float b) {   // round to nearest
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __device__ static __forceinline__ float lo_f32(uint32_t v) { return __uint_as_float(v << 16); }
    __device__ static __forceinline__ float hi_f32(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
    __device__ static __forceinline__ float to_f32(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
    __device__ static __forceinline__ uint16_t from_f32(float v) {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        return *reinterpret_cast<uint16_t*>(&h);
    }
};

template <> struct Act<__half> {
    static constexpr int MANT = 10;
    static constexpr uint32_t MAGIC = 0x64006400u;   // 2^10 in both halves
    static constexpr uint32_t ONES = 0x3C003C00u;
    __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ void mma0(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%10,%10,%10,%10};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
    __device__ static __forceinline__ uint32_t pack_hi(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __device__ static __forceinline__ float lo_f32(uint32_t v) {
        return __half2float(__ushort_as_half((unsigned short)(v & 0xFFFFu)));
    }
    __device__ static __forceinline__ float hi_f32(uint32_t v) {
        return __half2float(__ushort_as_half((unsigned short)(v >> 16)));
    }
    __device__ static __forceinline__ float to_f32(uint16_t v) { return __half2float(__ushort_as_half(v)); }
    __device__ static __forceinline__ uint16_t from_f32(float v) { return __half_as_ushort(__float2half_rn(v)); }
};

// ---- code layout of one lane's 16-code unit ------------------------------------------
// The 64 codes of a k-block are split over the 4 lanes that share a row in the
// MMA A fragment: lane `tig` owns codes [16*tig, 16*tig+16) of the block, i.e.
// 16*BITS bits of the row's stream.
// WORDS = 32-bit words a lane reads: BITS/2 for even widths; 3-bit: 2 (48 bits at bit
// offset 0 or 16); 5-bit: 3 (80 bits at offset 0 or 16).
template <int BITS> struct Unit;
template <> struct Unit<2> { static constexpr int WORDS = 1; };
template <> struct Unit<3> { static constexpr int WORDS = 2; };
template <> struct Unit<4> { static constexpr int WORDS = 2; };
template <> struct Unit<5> { static constexpr int WORDS = 3; };
template <> struct Unit<6> { static constexpr int WORDS = 3; };
template <> struct Unit<8> { static constexpr int WORDS = 4; };

// Read lane `tig`'s unit of k-block `blk` from a row segment in shared memory and
// normalise it so that code j starts at bit j*BITS of u[].
template <int BITS>
__host__ __device__ __forceinline__ void load_unit(const uint32_t* __restrict__ row, int blk, int tig,
                                          uint32_t (&u)[Unit<BITS>::WORDS]) {
    const uint32_t* p = row + blk * (2 * BITS);
    if constexpr (BITS == 2) {
        u[0] = p[tig];
    } else if constexpr (BITS == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p + 2 * tig);
        u[0] = v.x; u[1] = v.y;
    } else if constexpr (BITS == 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(p + 4 * tig);
        u[0] = v.x; u[1] = v.y; u[2] = v.z; u[3] = v.w;
    } else if constexpr (BITS == 6) {
        u[0] = p[3 * tig]; u[1] = p[3 * tig + 1]; u[2] = p[3 * tig + 2];
    } else if constexpr (BITS == 3) {
        const int w = (3 * tig) >> 1, off = (tig & 1) * 16;
        const uint32_t a = p[w], b = p[w + 1];
        u[0] = funnel_r(a, b, off);
        u[1] = b >> off;
    } else {  // 5
        const int w = (5 * tig) >> 1, off = (tig & 1) * 16;
        const uint32_t a = p[w], b = p[w + 1], c = p[w + 2];
        u[0] = funnel_r(a, b, off);
        u[1] = funnel_r(b, c, off);
        u[2] = c >> off;
    }
}

// Number of MMA passes per k16 step and the field each pass converts.
template <typename AT, int BITS> struct Fields {
    static constexpr bool SPLIT = BITS > Act<AT>::MANT;                          // bf16 + 8-bit
    static constexpr int PASSES = SPLIT ? 2 : 1;
    static constexpr int FB = SPLIT ? 4 : BITS;                                // field bits
    // after the MMA: sum(q*x) = POST * (combined C) - OFFSET * sum(x)
    //   single pass: C = 2^(MANT-FB) * (2^FB * X + sum q x)
    //   split:       16*C_hi + C_lo = 2^(MANT-4) * (272 * X + sum q x)
    static constexpr float POST = 1.0f / (float)(1 << (Act<AT>::MANT - FB));
    static constexpr float OFFSET = SPLIT ? 272.0f : (float)(1 << FB);
};

// Code indices (within the lane's 16-code unit) that MMA step t (0..3) consumes:
// register h (0 -> a0a1/a2a3, 1 -> a4a5/a6a7) holds codes (lo(t,h), hi(t,h)) in its
// low/high half.  Aligned widths pair codes 16 bits apart in one word so that one
// shift + LOP3 converts both; other widths pair neighbours.
template <int BITS> struct Pairing {
    static constexpr bool ALIGNED = (BITS == 2 || BITS == 4 || BITS == 8);
    static constexpr int PER_WORD = 32 / BITS;            // aligned widths only
    __host__ __device__ static constexpr int lo(int t, int h) {
        if (ALIGNED) {
            const int p = 2 * t + h;                       // pair index 0..7
            const int half = PER_WORD / 2;                 // pairs per word
            return (p / half) * PER_WORD + (p % half);
        }
        return 2 * (2 * t + h);
    }
    __host__ __device__ static constexpr int hi(int t, int h) {
        if (ALIGNED) return lo(t, h) + PER_WORD / 2;
        return 2 * (2 * t + h) + 1;
    }
};

// 32 bits of the unit's stream starting at bit A (A may be negative: zero-filled).
template <int BITS, int A>
__host__ __device__ __forceinline__ uint32_t field_at(const uint32_t (&u)[Unit<BITS>::WORDS]) {
    if constexpr (A < 0) return u[0] << (-A);
    else if constexpr (A % 32 == 0) return u[A / 32];
    else if constexpr (A / 32 + 1 < Unit<BITS>::WORDS) return funnel_r(u[A / 32], u[A / 32 + 1], A % 32);
    else return u[A / 32] >> (A % 32);
}

// Convert the pair (lo(t,h), hi(t,h)) of pass `pass` into one MMA A register.
template <typename AT, int BITS, int T, int H, int PASS>
__host__ __device__ __forceinline__ uint32_t make_a(const uint32_t (&u)[Unit<BITS>::WORDS]) {
    using F = Fields<AT, BITS>;
    constexpr int FB = F::FB;
    constexpr int TGT = Act<AT>::MANT - FB;                 // field lands at bits [TGT, TGT+FB)
    constexpr uint32_t MASK = (((1u << FB) - 1u) << TGT) * 0x00010001u;
    constexpr int FPOS = PASS * 4;                          // split: pass 0 = low nibble, 1 = high
    constexpr int JL = Pairing<BITS>::lo(T, H), JH = Pairing<BITS>::hi(T, H);
    if constexpr (Pairing<BITS>::ALIGNED) {
        constexpr int POS = JL * BITS + FPOS;               // bit of the low code's field
        constexpr int W = POS / 32, B = POS % 32;
        static_assert((JH * BITS + FPOS) == POS + 16, "aligned pairs are 16 bits apart");
        uint32_t r;
        if constexpr (B >= TGT) r = u[W] >> (B - TGT); else r = u[W] << (TGT - B);
        return and_or(r, MASK, Act<AT>::MAGIC);
    } else {
        const uint32_t lo = field_at<BITS, JL * BITS + FPOS - TGT>(u);
        const uint32_t hi = field_at<BITS, JH * BITS + FPOS - TGT>(u);
        const uint32_t r = prmt(lo, hi, 0x5410);             // (lo.low16, hi.low16)
        return and_or(r, MASK, Act<AT>::MAGIC);
    }
}

// Build the B register matching make_a<.., T, H, ..>: activations (x[lo], x[hi]) of
// the lane's 16 x values, held as 8 registers xr[i] = (x[2i], x[2i+1]).
template <int BITS, int T, int H>
__host__ __device__ __forceinline__ uint32_t make_b(const uint32_t (&xr)[8]) {
    constexpr int JL = Pairing<BITS>::lo(T, H), JH = Pairing<BITS>::hi(T, H);
    constexpr uint32_t SEL = ((JL & 1) ? 0x32u : 0x10u) | (((JH & 1) ? 0x76u : 0x54u) << 8);
    if constexpr (JL / 2 == JH / 2 && (JL & 1) == 0 && (JH & 1) == 1) return xr[JL / 2];
    return prmt(xr[JL / 2], xr[JH / 2], SEL);
}

// ---- activation limbs for the integer mat-vec kernels ---------------------------------------------
// A fixed-point activation xi (|xi| <= 2^22) is fed to the integer MMAs as three signed 8-bit digits,
// xi = l0 + 256*l1 + 65536*l2 with l in [-128, 127].  With u = xi + 0x8080 the bytes of u ^ 0x8080 are
// the two's-complement digits: adding 128 at every digit position turns the signed digits into plain
// base-256 digits, the xor takes the 128 off again.
// store_limbs8 writes the digits of 8 consecutive activations (half `hf` of a 16-code unit) into the
// unit's 16 bytes of the three limb rows, in the byte order the kernels unpack codes in:
//   8-bit: natural;  4-bit: per 8 codes the even ones, then the odd ones;
//   2-bit: code j of the unit is byte j >> 2 of word j & 3.
template <int BITS>
__device__ __forceinline__ void store_limbs8(uint8_t* d0, uint8_t* d1, uint8_t* d2, int hf, const int (&xi)[8]) {
    uint32_t t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = ((uint32_t)xi[j] + 0x8080u) ^ 0x8080u;
    uint8_t* const d[3] = {d0, d1, d2};
#pragma unroll
    for (int L = 0; L < 3; ++L) {
        const uint32_t sel = (uint32_t)(((4 + L) << 4) | L);          // (x.byteL, y.byteL) -> result bytes 0, 1
        if constexpr (BITS == 2) {
            uint16_t* d16 = reinterpret_cast<uint16_t*>(d[L]) + hf;
            d16[0] = (uint16_t)prmt(t[0], t[4], sel);
            d16[2] = (uint16_t)prmt(t[1], t[5], sel);
            d16[4] = (uint16_t)prmt(t[2], t[6], sel);
            d16[6] = (uint16_t)prmt(t[3], t[7], sel);
        } else if constexpr (BITS == 4) {
            const uint32_t w0 = prmt(prmt(t[0], t[2], sel), prmt(t[4], t[6], sel), 0x5410);
            const uint32_t w1 = prmt(prmt(t[1], t[3], sel), prmt(t[5], t[7], sel), 0x5410);
            *reinterpret_cast<uint2*>(d[L] + 8 * hf) = make_uint2(w0, w1);
        } else {
            const uint32_t w0 = prmt(prmt(t[0], t[1], sel), prmt(t[2], t[3], sel), 0x5410);
            const uint32_t w1 = prmt(prmt(t[4], t[5], sel), prmt(t[6], t[7], sel), 0x5410);
            *reinterpret_cast<uint2*>(d[L] + 8 * hf) = make_uint2(w0, w1);
        }
    }
}

// The same for a unit of 8 three-bit codes: 12 bytes per limb row, (x0, x3, x6, 0), (x1, x4, x7, 0), (x2, x5, 0, 0)
// -- the byte positions the 3-bit unpack of the integer kernels leaves its codes at.
__device__ __forceinline__ void store_limbs3(uint8_t* d0, uint8_t* d1, uint8_t* d2, const int (&xi)[8]) {
    uint32_t t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = ((uint32_t)xi[j] + 0x8080u) ^ 0x8080u;
    uint8_t* const d[3] = {d0, d1, d2};
#pragma unroll
    for (int L = 0; L < 3; ++L) {
        const uint32_t sel = (uint32_t)(((4 + L) << 4) | L);
        uint32_t* o = reinterpret_cast<uint32_t*>(d[L]);
        o[0] = prmt(prmt(t[0], t[3], sel), prmt(t[6], 0u, sel), 0x5410);
        o[1] = prmt(prmt(t[1], t[4], sel), prmt(t[7], 0u, sel), 0x5410);
        o[2] = prmt(prmt(t[2], t[5], sel), 0u, 0x5410);
    }
}

}  // namespace jq
