// Host-side emulation of one warp of the mat-vec kernel's inner step: builds
// the MMA A/B registers with the very functions the kernel uses (jq_mma.cuh),
// applies the m16n8k16 fragment layout of the PTX ISA, and checks the result
// against a direct sum.  Runs without a GPU; built and run by
// tests/test_fragment_emulation.py.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../jangq_b200/csrc/jq_mma.cuh"

using namespace jq;

static float bf16_to_f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static uint16_t f_to_bf16(float f) { uint32_t u; memcpy(&u, &f, 4); return (uint16_t)(u >> 16); }  // exact for small ints
static float f16_to_f(uint16_t h) {
    const int e = (h >> 10) & 31, m = h & 1023;
    float v = e == 0 ? m * (1.0f / (1 << 24)) : (1.0f + m / 1024.0f) * (e >= 15 ? (float)(1u << (e - 15)) : 1.0f / (float)(1u << (15 - e)));
    return (h & 0x8000) ? -v : v;
}
static uint16_t small_int_to_f16(int v) {   // |v| <= 8
    if (v == 0) return 0;
    const uint16_t s = v < 0 ? 0x8000 : 0;
    int a = v < 0 ? -v : v, e = 0;
    while ((1 << (e + 1)) <= a) ++e;
    const int mant = ((a << 10) >> e) & 1023;
    return s | (uint16_t)((e + 15) << 10) | (uint16_t)mant;
}

template <typename AT> struct H;
template <> struct H<__nv_bfloat16> {
    static float dec(uint16_t v) { return bf16_to_f(v); }
    static uint16_t enc(int v) { return f_to_bf16((float)v); }
};
template <> struct H<__half> {
    static float dec(uint16_t v) { return f16_to_f(v); }
    static uint16_t enc(int v) { return small_int_to_f16(v); }
};

template <typename AT, int BITS, int T>
static void step(const uint32_t (&ulo)[Unit<BITS>::WORDS], const uint32_t (&uhi)[Unit<BITS>::WORDS],
                 const uint32_t (&xr)[8], uint32_t (&a)[Fields<AT, BITS>::PASSES][4], uint32_t (&b)[2]) {
    b[0] = make_b<BITS, T, 0>(xr);
    b[1] = make_b<BITS, T, 1>(xr);
    a[0][0] = make_a<AT, BITS, T, 0, 0>(ulo); a[0][1] = make_a<AT, BITS, T, 0, 0>(uhi);
    a[0][2] = make_a<AT, BITS, T, 1, 0>(ulo); a[0][3] = make_a<AT, BITS, T, 1, 0>(uhi);
    if constexpr (Fields<AT, BITS>::PASSES == 2) {
        a[1][0] = make_a<AT, BITS, T, 0, 1>(ulo); a[1][1] = make_a<AT, BITS, T, 0, 1>(uhi);
        a[1][2] = make_a<AT, BITS, T, 1, 1>(ulo); a[1][3] = make_a<AT, BITS, T, 1, 1>(uhi);
    }
}

template <typename AT, int BITS>
static int run(const char* name) {
    using F = Fields<AT, BITS>;
    constexpr int NBLK = 3;                       // a row segment of 3 k-blocks, use the middle one too
    constexpr int SEGW = NBLK * 2 * BITS;         // words per row segment
    int bad = 0;
    for (int trial = 0; trial < 20; ++trial) {
        std::vector<int> q(16 * 64 * NBLK);
        for (auto& v : q) v = rand() & ((1 << BITS) - 1);
        std::vector<uint32_t> seg(16 * (SEGW + 1), 0u);
        for (int r = 0; r < 16; ++r)
            for (int j = 0; j < 64 * NBLK; ++j) {
                const int pos = j * BITS, w = pos / 32, s = pos % 32;
                const unsigned long long v = (unsigned long long)q[r * 64 * NBLK + j] << s;
                seg[r * (SEGW + 1) + w] |= (uint32_t)v;
                if (s + BITS > 32) seg[r * (SEGW + 1) + w + 1] |= (uint32_t)(v >> 32);
            }
        std::vector<int> x(8 * 64 * NBLK);
        for (auto& v : x) v = (rand() % 9) - 4;
        for (int blk = 0; blk < NBLK; ++blk) {
            double C[F::PASSES][16][8] = {};
            for (int t = 0; t < 4; ++t) {
                float Am[F::PASSES][16][16] = {}, Bm[16][8] = {};
                for (int lane = 0; lane < 32; ++lane) {
                    const int g = lane >> 2, tig = lane & 3;
                    uint32_t ulo[Unit<BITS>::WORDS], uhi[Unit<BITS>::WORDS], xr[8];
                    load_unit<BITS>(&seg[g * (SEGW + 1)], blk, tig, ulo);
                    load_unit<BITS>(&seg[(g + 8) * (SEGW + 1)], blk, tig, uhi);
                    for (int i = 0; i < 8; ++i) {
                        const int k = blk * 64 + tig * 16 + 2 * i;
                        xr[i] = (uint32_t)H<AT>::enc(x[g * 64 * NBLK + k]) | ((uint32_t)H<AT>::enc(x[g * 64 * NBLK + k + 1]) << 16);
                    }
                    uint32_t a[F::PASSES][4], b[2];
                    switch (t) {
                        case 0: step<AT, BITS, 0>(ulo, uhi, xr, a, b); break;
                        case 1: step<AT, BITS, 1>(ulo, uhi, xr, a, b); break;
                        case 2: step<AT, BITS, 2>(ulo, uhi, xr, a, b); break;
                        default: step<AT, BITS, 3>(ulo, uhi, xr, a, b); break;
                    }
                    // PTX m16n8k16 fragment layout (A row-major 16x16, B 16x8, 16-bit types)
                    for (int p = 0; p < F::PASSES; ++p) {
                        Am[p][g][2 * tig] = H<AT>::dec(a[p][0] & 0xFFFF);       Am[p][g][2 * tig + 1] = H<AT>::dec(a[p][0] >> 16);
                        Am[p][g + 8][2 * tig] = H<AT>::dec(a[p][1] & 0xFFFF);   Am[p][g + 8][2 * tig + 1] = H<AT>::dec(a[p][1] >> 16);
                        Am[p][g][2 * tig + 8] = H<AT>::dec(a[p][2] & 0xFFFF);   Am[p][g][2 * tig + 9] = H<AT>::dec(a[p][2] >> 16);
                        Am[p][g + 8][2 * tig + 8] = H<AT>::dec(a[p][3] & 0xFFFF); Am[p][g + 8][2 * tig + 9] = H<AT>::dec(a[p][3] >> 16);
                    }
                    Bm[2 * tig][g] = H<AT>::dec(b[0] & 0xFFFF);     Bm[2 * tig + 1][g] = H<AT>::dec(b[0] >> 16);
                    Bm[2 * tig + 8][g] = H<AT>::dec(b[1] & 0xFFFF); Bm[2 * tig + 9][g] = H<AT>::dec(b[1] >> 16);
                }
                for (int p = 0; p < F::PASSES; ++p)
                    for (int r = 0; r < 16; ++r)
                        for (int m = 0; m < 8; ++m)
                            for (int k = 0; k < 16; ++k) C[p][r][m] += (double)Am[p][r][k] * Bm[k][m];
            }
            for (int r = 0; r < 16; ++r)
                for (int m = 0; m < 8; ++m) {
                    double qx = 0, X = 0;
                    for (int k = 0; k < 64; ++k) {
                        qx += (double)q[r * 64 * NBLK + blk * 64 + k] * x[m * 64 * NBLK + blk * 64 + k];
                        X += x[m * 64 * NBLK + blk * 64 + k];
                    }
                    double comb = C[0][r][m];
                    if (F::PASSES == 2) comb = 16.0 * C[F::PASSES - 1][r][m] + C[0][r][m];
                    const double got = comb * F::POST - F::OFFSET * X;
                    if (got != qx) {
                        if (bad < 5) printf("%s: mismatch blk %d row %d m %d: got %g want %g\n", name, blk, r, m, got, qx);
                        ++bad;
                    }
                }
        }
    }
    printf("%s: %s\n", name, bad ? "FAIL" : "ok");
    return bad;
}

int main() {
    int bad = 0;
#define RUN(AT, B) bad += run<AT, B>(#AT " bits=" #B);
    RUN(__nv_bfloat16, 2) RUN(__nv_bfloat16, 3) RUN(__nv_bfloat16, 4) RUN(__nv_bfloat16, 5) RUN(__nv_bfloat16, 6) RUN(__nv_bfloat16, 8)
    RUN(__half, 2) RUN(__half, 3) RUN(__half, 4) RUN(__half, 5) RUN(__half, 6) RUN(__half, 8)
    return bad ? 1 : 0;
}
