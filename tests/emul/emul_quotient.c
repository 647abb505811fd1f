/* Host check of the arithmetic identities the quantizer kernels rest on, with the host's IEEE operations:
 *   1. RN(t / s) == fma(fma(-y0, s, t), r, y0) with r = RN(1 / s), y0 = RN(t * r)     (float and double);
 *   2. the bit pattern of RN(y * 2^-149) is rint(y) (ties to even) for 0 <= y < 2^22, and negative as an
 *      integer for y < 0;
 *   3. (0x4B400000 + q) >> k == (0x4B400000 >> k) + (q >> k) for q < 256, k <= 22.
 * Inputs: uniformly random bit patterns in the ranges the kernels see, and the structured case that makes
 * exact rounding ties common: weights and group edge on a coarse (bf16) grid, scale = edge / q0.
 * Prints one "name: ok" line per check; exit status 1 on the first mismatch. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static uint64_t rng_state = 0x9E3779B97F4A7C15ull;
static uint64_t rnd(void) {
    rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
    return rng_state;
}
static float f_from_bits(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static uint32_t bits_of(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }
static float to_bf16(float f) { return f_from_bits((bits_of(f) + 0x7FFFu + ((bits_of(f) >> 16) & 1u)) & 0xFFFF0000u); }

static int check_f32(float t, float s) {
    const float r = 1.0f / s;
    const float y0 = t * r;
    const float y = fmaf(fmaf(-y0, s, t), r, y0);
    const float q = t / s;
    if (bits_of(y) != bits_of(q) && !(y == 0.0f && q == 0.0f)) {
        printf("float quotient differs: t=%a s=%a  got %a want %a\n", t, s, y, q);
        return 1;
    }
    return 0;
}
static int check_f64(double t, double s) {
    const double r = 1.0 / s;
    const double y0 = t * r;
    const double y = fma(fma(-y0, s, t), r, y0);
    const double q = t / s;
    if (y != q) {
        printf("double quotient differs: t=%a s=%a  got %a want %a\n", t, s, y, q);
        return 1;
    }
    return 0;
}

int main(void) {
    /* 1a. random floats: |s| in [2^-83, 2^83] (the kernels divide per weight outside [1e-25, 1e25]); quotients from
     * 2^-2 up are compared bit for bit, smaller ones (where a residual may underflow) only through rint, which is all
     * the kernels take from them */
    for (int i = 0; i < 20000000; ++i) {
        const uint32_t eb = 44u + (uint32_t)(rnd() % 167u);                   /* exponent of s: 2^-83 .. 2^83 */
        const float s = f_from_bits(((uint32_t)(rnd() & 1u) << 31) | (eb << 23) | (uint32_t)(rnd() & 0x7FFFFFu));
        const int de = (int)(rnd() % 12u) - 2;                                /* |t / s| from 2^-2 to 2^10 */
        float t = f_from_bits((uint32_t)(rnd() & 0x7FFFFFu) | (127u << 23));
        t = ldexpf(t, (int)eb - 127 + de) * ((rnd() & 1u) ? -1.0f : 1.0f);
        if (check_f32(t, s)) return 1;
        const float tiny = ldexpf(t, -(int)(rnd() % 60u) - 3);               /* may be subnormal */
        const float r = 1.0f / s, y0 = tiny * r;
        if (rintf(fmaf(fmaf(-y0, s, tiny), r, y0)) != rintf(tiny / s)) { printf("small quotient rounds differently\n"); return 1; }
    }
    printf("float quotient, random: ok\n");
    /* 1b. the quantizer's own shape on a bf16 grid: scale = edge / q0, t = w - edge */
    for (int i = 0; i < 20000000; ++i) {
        const float edge = to_bf16(ldexpf(1.0f + (float)(rnd() % 128u) / 128.0f, (int)(rnd() % 40u) - 30)) *
                           ((rnd() & 1u) ? -1.0f : 1.0f);
        const int bins = (1 << (2 + (int)(rnd() % 7u))) - 1;                  /* 3 .. 255 */
        const float q0 = -(float)(1 + (int)(rnd() % (uint32_t)bins));
        const float s = edge / q0;
        const float w = to_bf16(edge * ((float)(rnd() % 4096u) / 4096.0f) * ((rnd() & 3u) ? 1.0f : -0.3f));
        if (check_f32(w - edge, s)) return 1;
    }
    printf("float quotient, bf16 grid: ok\n");
    /* 1c. doubles: scale = range * ratio / levels, x a float */
    for (int i = 0; i < 20000000; ++i) {
        const double range = ldexp(1.0 + (double)(rnd() >> 12) * 0x1p-52, (int)(rnd() % 120u) - 80);
        const double s = range * (0.7 + 0.3 * (double)(rnd() % 20u) / 19.0) / (double)((1 << (2 + (int)(rnd() % 3u))) - 1);
        const double x = (double)f_from_bits((uint32_t)rnd() & 0x7FFFFFu | (127u << 23)) * range *
                         ((rnd() & 1u) ? -1.0 : 1.0) * ldexp(1.0, (int)(rnd() % 12u) - 8);
        if (check_f64(x, s)) return 1;
    }
    printf("double quotient: ok\n");
    /* 2. subnormal rint */
    for (int i = 0; i < 20000000; ++i) {
        float y;
        const uint32_t k = (uint32_t)(rnd() % 3u);
        if (k == 0) y = (float)(rnd() % 600u) * 0.5f;                         /* integers and exact ties */
        else if (k == 1) y = ldexpf((float)(rnd() & 0xFFFFFFu), (int)(rnd() % 24u) - 24);
        else y = (float)(rnd() % 4000000u) + (float)(rnd() & 0xFFu) / 256.0f;
        if (y >= 4194304.0f) continue;
        const int32_t got = (int32_t)bits_of(y * 0x1p-149f);
        const int32_t want = (int32_t)rintf(y);
        if (got != want) { printf("subnormal rint differs: y=%a got %d want %d\n", y, got, want); return 1; }
        if (y > 0.3f && (int32_t)bits_of(-y * 0x1p-149f) >= 0 && rintf(y) != 0.0f) {
            printf("negative input does not read as a negative integer: y=%a\n", -y);
            return 1;
        }
    }
    printf("subnormal rint: ok\n");
    /* 3. shifted magic constant */
    for (uint32_t q = 0; q < 256u; ++q)
        for (uint32_t k = 0; k <= 22u; ++k)
            if (((0x4B400000u + q) >> k) != ((0x4B400000u >> k) + (q >> k))) { printf("shift identity fails\n"); return 1; }
    printf("shift identity: ok\n");
    return 0;
}
