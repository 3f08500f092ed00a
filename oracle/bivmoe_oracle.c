/*
 * CPU oracle for the qwen35moe mixture-of-experts FFN path of vincenthz/biv.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is a C restatement of the
 * reference's CPU arithmetic (the reference is Rust and cannot be compiled in
 * this environment) and exists only as the checker for the CUDA path and as
 * the timed CPU baseline.  Nothing in the shipped library links or calls it.
 *
 * Parity status: pinned against the reference's four known-answer tests for
 * this path (engine/src/quant.rs:1566-1614, 1652-1712, 1715-1738 and
 * engine/src/model.rs:1461-1474, restated in tests/).  The reference holds no
 * test for the whole layer, the activation quantiser's integers, the
 * permutation or the combine: for those the parity is PINNED BY SOURCE ONLY
 * ("parity unpinned" by any reference golden vector).
 *
 * Every function cites the reference lines it follows (paths inside the
 * reference project).  Two kernel levels exist, as in the reference
 * (quant.rs:527-559): level 0 follows `scalar::*` (quant.rs:563-687), level 1
 * follows `x86::avx2::*` and level 2 `x86::vnni::*` (quant.rs:1283-1544); the
 * int32 block dots of all levels are the same integers, only the order of the
 * f32 accumulation differs.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no -ffast-math).
 * Explicit fmaf()/_mm256_fmadd_ps calls are kept where the reference fuses.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__x86_64__)
#include <cpuid.h>
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ggml type ids, quant.rs:30-48 */
enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q8_0 = 8, T_Q4K = 12, T_Q5K = 13, T_Q6K = 14, T_BF16 = 30 };

/* ------------------------------------------------------------------------ */
/* scalars                                                                   */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* quant.rs:114-131, the branch-free form the x86 build uses */
ORC_API float orc_f16_to_f32(uint16_t h) {
    uint32_t w = (uint32_t)h << 16;
    uint32_t sign = w & 0x80000000u;
    uint32_t two_w = w + w;
    uint32_t exp_offset = 0xE0u << 23;
    float normalized = bits_f32((two_w >> 4) + exp_offset) * bits_f32(0x07800000u);
    uint32_t magic_mask = 126u << 23;
    float denormalized = bits_f32((two_w >> 17) | magic_mask) - 0.5f;
    uint32_t bits = two_w < (1u << 27) ? f32_bits(denormalized) : f32_bits(normalized);
    return bits_f32(sign | bits);
}

/* quant.rs:134-136 */
ORC_API float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

static inline uint16_t rd16(const uint8_t* b, size_t off) {
    return (uint16_t)(b[off] | ((uint16_t)b[off + 1] << 8));
}

/* quant.rs:51-72 */
ORC_API long orc_row_size(int ty, long n) {
    switch (ty) {
        case T_F32: return n * 4;
        case T_F16: case T_BF16: return n * 2;
        case T_Q4_0: return n % 32 ? -1 : n / 32 * 18;
        case T_Q4_1: return n % 32 ? -1 : n / 32 * 20;
        case T_Q8_0: return n % 32 ? -1 : n / 32 * 34;
        case T_Q4K: return n % 256 ? -1 : n / 256 * 144;
        case T_Q5K: return n % 256 ? -1 : n / 256 * 176;
        case T_Q6K: return n % 256 ? -1 : n / 256 * 210;
        default: return -1;
    }
}

/* quant.rs:75-77 */
static int uses_f32_act(int ty) { return ty == T_F32 || ty == T_F16 || ty == T_BF16; }

/* quant.rs:144-153 */
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* quant.rs:156-349 (the types on this path only) */
ORC_API int orc_dequantize_row(int ty, const uint8_t* src, float* dst, long n) {
    switch (ty) {
        case T_F32:
            memcpy(dst, src, (size_t)n * 4);
            return 0;
        case T_F16:
            for (long i = 0; i < n; i++) dst[i] = orc_f16_to_f32(rd16(src, 2 * i));
            return 0;
        case T_BF16:
            for (long i = 0; i < n; i++) dst[i] = orc_bf16_to_f32(rd16(src, 2 * i));
            return 0;
        case T_Q4_0: /* quant.rs:174-182 */
            for (long b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + 18 * b;
                float d = orc_f16_to_f32(rd16(blk, 0));
                for (int j = 0; j < 16; j++) {
                    dst[32 * b + j] = (float)((int)(blk[2 + j] & 0xF) - 8) * d;
                    dst[32 * b + j + 16] = (float)((int)(blk[2 + j] >> 4) - 8) * d;
                }
            }
            return 0;
        case T_Q4_1: /* quant.rs:183-192 */
            for (long b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + 20 * b;
                float d = orc_f16_to_f32(rd16(blk, 0)), m = orc_f16_to_f32(rd16(blk, 2));
                for (int j = 0; j < 16; j++) {
                    dst[32 * b + j] = (float)(blk[4 + j] & 0xF) * d + m;
                    dst[32 * b + j + 16] = (float)(blk[4 + j] >> 4) * d + m;
                }
            }
            return 0;
        case T_Q8_0:
            for (long b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + 34 * b;
                float d = orc_f16_to_f32(rd16(blk, 0));
                for (int j = 0; j < 32; j++) dst[32 * b + j] = (float)(int8_t)blk[2 + j] * d;
            }
            return 0;
        case T_Q4K:
            for (long b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + 144 * b;
                float* y = dst + 256 * b;
                float d = orc_f16_to_f32(rd16(blk, 0)), min = orc_f16_to_f32(rd16(blk, 2));
                const uint8_t *scales = blk + 4, *qs = blk + 16;
                for (int j = 0; j < 4; j++) {
                    uint8_t s1, m1, s2, m2;
                    scale_min_k4(2 * j, scales, &s1, &m1);
                    scale_min_k4(2 * j + 1, scales, &s2, &m2);
                    float d1 = d * (float)s1, mm1 = min * (float)m1;
                    float d2 = d * (float)s2, mm2 = min * (float)m2;
                    const uint8_t* q = qs + 32 * j;
                    for (int l = 0; l < 32; l++) {
                        y[64 * j + l] = d1 * (float)(q[l] & 0xF) - mm1;
                        y[64 * j + 32 + l] = d2 * (float)(q[l] >> 4) - mm2;
                    }
                }
            }
            return 0;
        case T_Q5K:
            for (long b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + 176 * b;
                float* y = dst + 256 * b;
                float d = orc_f16_to_f32(rd16(blk, 0)), min = orc_f16_to_f32(rd16(blk, 2));
                const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
                for (int j = 0; j < 4; j++) {
                    uint8_t s1, m1, s2, m2;
                    scale_min_k4(2 * j, scales, &s1, &m1);
                    scale_min_k4(2 * j + 1, scales, &s2, &m2);
                    float d1 = d * (float)s1, mm1 = min * (float)m1;
                    float d2 = d * (float)s2, mm2 = min * (float)m2;
                    uint8_t u1 = (uint8_t)(1u << (2 * j)), u2 = (uint8_t)(2u << (2 * j));
                    const uint8_t* q = qs + 32 * j;
                    for (int l = 0; l < 32; l++) {
                        int h1 = (qh[l] & u1) ? 16 : 0, h2 = (qh[l] & u2) ? 16 : 0;
                        y[64 * j + l] = d1 * (float)((q[l] & 0xF) + h1) - mm1;
                        y[64 * j + 32 + l] = d2 * (float)((q[l] >> 4) + h2) - mm2;
                    }
                }
            }
            return 0;
        case T_Q6K:
            for (long b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + 210 * b;
                float d = orc_f16_to_f32(rd16(blk, 208));
                for (int h = 0; h < 2; h++) {
                    const uint8_t* ql = blk + 64 * h;
                    const uint8_t* qh = blk + 128 + 32 * h;
                    const int8_t* sc = (const int8_t*)blk + 192 + 8 * h;
                    float* y = dst + 256 * b + 128 * h;
                    for (int l = 0; l < 32; l++) {
                        int is = l / 16;
                        int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
                        int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        y[l] = d * (float)sc[is] * (float)q1;
                        y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                        y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                        y[l + 96] = d * (float)sc[is + 6] * (float)q4;
                    }
                }
            }
            return 0;
        default:
            return -1;
    }
}

/* ------------------------------------------------------------------------ */
/* Q8 activation quantiser, quant.rs:368-394.  f32::round = roundf           */

ORC_API void orc_q8_quantize(const float* x, long n, int8_t* qs, float* d, float* s) {
    for (long b = 0; b < n / 32; b++) {
        const float* xb = x + 32 * b;
        float amax = 0.0f;
        for (int j = 0; j < 32; j++) {
            float a = fabsf(xb[j]);
            amax = amax > a ? amax : a; /* f32::max */
        }
        float dd = amax / 127.0f;
        float id = dd != 0.0f ? 1.0f / dd : 0.0f;
        int32_t sum = 0;
        for (int j = 0; j < 32; j++) {
            int32_t r = (int32_t)roundf(xb[j] * id);
            qs[32 * b + j] = (int8_t)r;
            sum += r;
        }
        d[b] = dd;
        s[b] = dd * (float)sum;
    }
}

/* ------------------------------------------------------------------------ */
/* unpacking one 32-element block of a weight row into int32, shared by the
 * scalar dots and the int32 block-dot tap.  For k-quants `sb` is the
 * sub-block (0..8) of super-block `i`.                                      */

/* quant.rs:574-577 (Q4_0: nibble - 8) and 589-592 (Q4_1: the nibble): byte j holds
 * element j in its low half and element j + 16 in its high half */
static void unpack_q4_01(int ty, const uint8_t* blk, int32_t* q) {
    const uint8_t* qs = blk + (ty == T_Q4_0 ? 2 : 4);
    const int off = ty == T_Q4_0 ? 8 : 0;
    for (int j = 0; j < 16; j++) {
        q[j] = (int32_t)(qs[j] & 0xF) - off;
        q[j + 16] = (int32_t)(qs[j] >> 4) - off;
    }
}
static void unpack_q4k(const uint8_t* blk, int sb, int32_t* q) { /* quant.rs:616-620 */
    const uint8_t* q4 = blk + 16 + 32 * (sb / 2);
    for (int l = 0; l < 32; l++) q[l] = (q4[l] >> (4 * (sb % 2))) & 0xF;
}
static void unpack_q5k(const uint8_t* blk, int sb, int32_t* q) { /* quant.rs:636-642 */
    const uint8_t *qh = blk + 16, *q4 = blk + 48 + 32 * (sb / 2);
    for (int l = 0; l < 32; l++)
        q[l] = ((q4[l] >> (4 * (sb % 2))) & 0xF) | (((qh[l] >> sb) & 1) << 4);
}
static void unpack_q6k(const uint8_t* blk, int32_t* q, int32_t* sc16) { /* quant.rs:656-672 */
    for (int n = 0; n < 2; n++) {
        const uint8_t* ql = blk + 64 * n;
        const uint8_t* qh = blk + 128 + 32 * n;
        const int8_t* sc = (const int8_t*)blk + 192 + 8 * n;
        for (int l = 0; l < 32; l++) {
            q[128 * n + l] = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
            q[128 * n + l + 32] = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            q[128 * n + l + 64] = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            q[128 * n + l + 96] = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        }
        for (int k = 0; k < 8; k++) sc16[8 * n + k] = sc[k];
    }
}
static int32_t idot(const int32_t* a, const int8_t* b, int n) { /* quant.rs:566-568 */
    int32_t s = 0;
    for (int i = 0; i < n; i++) s += a[i] * (int32_t)b[i];
    return s;
}

/* The int32 dot of every 32-element block of one weight row against one
 * quantised activation row: the integers every kernel level of the reference
 * produces before its f32 scaling (quant.rs:599-686).  For Q6_K the value is
 * `isum`, which includes the int8 sub-block scales (quant.rs:674-683).      */
ORC_API int orc_block_dots(int ty, const uint8_t* w, const int8_t* xq, long n, int32_t* out) {
    int32_t q[256], sc16[16];
    switch (ty) {
        case T_Q4_0:
        case T_Q4_1:
            for (long i = 0; i < n / 32; i++) {
                unpack_q4_01(ty, w + (ty == T_Q4_0 ? 18 : 20) * i, q);
                out[i] = idot(q, xq + 32 * i, 32);
            }
            return 0;
        case T_Q8_0:
            for (long i = 0; i < n / 32; i++) {
                const uint8_t* b = w + 34 * i;
                for (int j = 0; j < 32; j++) q[j] = (int8_t)b[2 + j];
                out[i] = idot(q, xq + 32 * i, 32);
            }
            return 0;
        case T_Q4K:
        case T_Q5K:
            for (long i = 0; i < n / 256; i++) {
                const uint8_t* b = w + (ty == T_Q4K ? 144 : 176) * i;
                for (int sb = 0; sb < 8; sb++) {
                    if (ty == T_Q4K) unpack_q4k(b, sb, q); else unpack_q5k(b, sb, q);
                    out[8 * i + sb] = idot(q, xq + 256 * i + 32 * sb, 32);
                }
            }
            return 0;
        case T_Q6K:
            for (long i = 0; i < n / 256; i++) {
                unpack_q6k(w + 210 * i, q, sc16);
                for (int xb = 0; xb < 8; xb++) {
                    int32_t isum = 0;
                    for (int half = 0; half < 2; half++) {
                        int g = 2 * xb + half, off = 16 * g;
                        isum += sc16[g] * idot(q + off, xq + 256 * i + off, 16);
                    }
                    out[8 * i + xb] = isum;
                }
            }
            return 0;
        default:
            return -1;
    }
}

/* ------------------------------------------------------------------------ */
/* level 0: scalar kernels, quant.rs:563-687 and the iterator sums of
 * quant.rs:459-521 (sequential left folds)                                  */

static float dot_f32_seq(const float* a, const float* b, long n) { /* quant.rs:467 */
    float s = 0.0f;
    for (long i = 0; i < n; i++) s += a[i] * b[i];
    return s;
}
static float dot_bf16_seq(const uint8_t* w, const float* x, long n) { /* quant.rs:517-520 */
    float s = 0.0f;
    for (long i = 0; i < n; i++) s += orc_bf16_to_f32(rd16(w, 2 * i)) * x[i];
    return s;
}
static float dot_f16_seq(const uint8_t* w, const float* x, long n) { /* quant.rs:502-505 */
    float s = 0.0f;
    for (long i = 0; i < n; i++) s += orc_f16_to_f32(rd16(w, 2 * i)) * x[i];
    return s;
}

static float sc_dot_q4_0(const uint8_t* w, const int8_t* qs, const float* xd, long nb) {
    float sum = 0.0f; /* quant.rs:570-582 */
    int32_t q[32];
    for (long i = 0; i < nb; i++) {
        const uint8_t* b = w + 18 * i;
        float d = orc_f16_to_f32(rd16(b, 0));
        unpack_q4_01(T_Q4_0, b, q);
        sum += d * xd[i] * (float)idot(q, qs + 32 * i, 32);
    }
    return sum;
}
static float sc_dot_q4_1(const uint8_t* w, const int8_t* qs, const float* xd, const float* xs,
                         long nb) {
    float sum = 0.0f; /* quant.rs:584-597 */
    int32_t q[32];
    for (long i = 0; i < nb; i++) {
        const uint8_t* b = w + 20 * i;
        float d = orc_f16_to_f32(rd16(b, 0)), m = orc_f16_to_f32(rd16(b, 2));
        unpack_q4_01(T_Q4_1, b, q);
        sum += d * xd[i] * (float)idot(q, qs + 32 * i, 32) + m * xs[i];
    }
    return sum;
}
static float sc_dot_q8_0(const uint8_t* w, const int8_t* qs, const float* xd, long nb) {
    float sum = 0.0f; /* quant.rs:599-607 */
    int32_t q[32];
    for (long i = 0; i < nb; i++) {
        const uint8_t* b = w + 34 * i;
        float d = orc_f16_to_f32(rd16(b, 0));
        for (int j = 0; j < 32; j++) q[j] = (int8_t)b[2 + j];
        sum += d * xd[i] * (float)idot(q, qs + 32 * i, 32);
    }
    return sum;
}
static float sc_dot_q45k(int ty, const uint8_t* w, const int8_t* qs, const float* xd,
                         const float* xs, long nb) {
    float sum = 0.0f; /* quant.rs:609-649 */
    int32_t q[32];
    long bs = ty == T_Q4K ? 144 : 176;
    for (long i = 0; i < nb / 8; i++) {
        const uint8_t* b = w + bs * i;
        float d = orc_f16_to_f32(rd16(b, 0)), min = orc_f16_to_f32(rd16(b, 2));
        for (int sb = 0; sb < 8; sb++) {
            uint8_t sc, m;
            scale_min_k4(sb, b + 4, &sc, &m);
            if (ty == T_Q4K) unpack_q4k(b, sb, q); else unpack_q5k(b, sb, q);
            long xb = 8 * i + sb;
            sum += d * (float)sc * xd[xb] * (float)idot(q, qs + 32 * xb, 32)
                   - min * (float)m * xs[xb];
        }
    }
    return sum;
}
static float sc_dot_q6k(const uint8_t* w, const int8_t* qs, const float* xd, long nb) {
    float sum = 0.0f; /* quant.rs:651-686 */
    int32_t q[256], sc16[16];
    for (long i = 0; i < nb / 8; i++) {
        const uint8_t* b = w + 210 * i;
        float d = orc_f16_to_f32(rd16(b, 208));
        unpack_q6k(b, q, sc16);
        for (int xb = 0; xb < 8; xb++) {
            int32_t isum = 0;
            for (int half = 0; half < 2; half++) {
                int g = 2 * xb + half, off = 16 * g;
                isum += sc16[g] * idot(q + off, qs + 256 * i + off, 16);
            }
            sum += d * xd[8 * i + xb] * (float)isum;
        }
    }
    return sum;
}

/* ------------------------------------------------------------------------ */
/* levels 1 and 2: AVX2 (maddubs+madd) and AVX-VNNI (vpdpbusd) kernels,
 * quant.rs:1135-1544                                                        */
#if defined(__x86_64__)
#define AVX2 __attribute__((target("avx2,fma,f16c")))
#define VNNI __attribute__((target("avx2,fma,f16c,avxvnni")))

/* quant.rs:1048-1123: cpuid leaf 1 (fma, osxsave, avx, f16c), xcr0 ymm state,
 * leaf 7.0 ebx bit 5 (avx2), leaf 7.1 eax bit 4 (avx-vnni) */
static int detect_level(void) {
    unsigned a, b, c, d;
    if (!__get_cpuid(1, &a, &b, &c, &d)) return 0;
    int fma = (c >> 12) & 1, osxsave = (c >> 27) & 1, avx = (c >> 28) & 1, f16c = (c >> 29) & 1;
    if (!(fma && osxsave && avx && f16c) || __get_cpuid_max(0, 0) < 7) return 0;
    unsigned lo, hi;
    __asm__ volatile("xgetbv" : "=a"(lo), "=d"(hi) : "c"(0));
    if ((lo & 6) != 6) return 0;
    __cpuid_count(7, 0, a, b, c, d);
    if (!((b >> 5) & 1)) return 0;
    __cpuid_count(7, 1, a, b, c, d);
    return ((a >> 4) & 1) ? 2 : 1;
}

AVX2 static inline float hsum8(__m256 v) { /* quant.rs:1148-1152 */
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    return _mm_cvtss_f32(_mm_add_ss(s, _mm_movehdup_ps(s)));
}
AVX2 static inline float f16_hw(const uint8_t* p) { /* quant.rs:1125-1132 */
    uint16_t h;
    memcpy(&h, p, 2);
    return _mm_cvtss_f32(_mm_cvtph_ps(_mm_cvtsi32_si128((int)h)));
}
AVX2 static inline __m256 fma_i32(__m256 acc, __m256i p, float d) { /* quant.rs:1155-1159 */
    return _mm256_fmadd_ps(_mm256_cvtepi32_ps(p), _mm256_set1_ps(d), acc);
}
AVX2 static inline __m256i ld256(const void* p) { return _mm256_loadu_si256((const __m256i*)p); }
/* quant.rs:1165-1175: 16 bytes of nibbles as 32 bytes, the low halves in the low lane */
AVX2 static inline __m256i q4_nibbles(const uint8_t* p) {
    __m128i v = _mm_loadu_si128((const __m128i*)p);
    __m128i m4 = _mm_set1_epi8(0x0F);
    return _mm256_set_m128i(_mm_and_si128(_mm_srli_epi16(v, 4), m4), _mm_and_si128(v, m4));
}

/* quant.rs:1177-1206 */
AVX2 static float dot_f32_avx2(const float* a, const float* b, long n) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                     _mm256_setzero_ps()};
    long i = 0;
    for (; i + 32 <= n; i += 32)
        for (int k = 0; k < 4; k++)
            acc[k] = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8 * k),
                                     _mm256_loadu_ps(b + i + 8 * k), acc[k]);
    for (; i + 8 <= n; i += 8)
        acc[0] = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc[0]);
    float s = hsum8(_mm256_add_ps(_mm256_add_ps(acc[0], acc[1]), _mm256_add_ps(acc[2], acc[3])));
    for (; i < n; i++) s += a[i] * b[i];
    return s;
}
/* quant.rs:1209-1226 */
AVX2 static void axpy_avx2(float* y, float a, const float* x, long n) {
    __m256 va = _mm256_set1_ps(a);
    long i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(y + i, _mm256_fmadd_ps(va, _mm256_loadu_ps(x + i), _mm256_loadu_ps(y + i)));
    for (; i < n; i++) y[i] += a * x[i];
}
/* quant.rs:1229-1256 */
AVX2 static inline __m256 widen_bf16(const uint16_t* p) {
    return _mm256_castsi256_ps(
        _mm256_slli_epi32(_mm256_cvtepu16_epi32(_mm_loadu_si128((const __m128i*)p)), 16));
}
AVX2 static float dot_bf16_avx2(const uint8_t* wb, const float* x, long n) {
    const uint16_t* w = (const uint16_t*)wb;
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    long i = 0;
    for (; i + 16 <= n; i += 16) {
        acc0 = _mm256_fmadd_ps(widen_bf16(w + i), _mm256_loadu_ps(x + i), acc0);
        acc1 = _mm256_fmadd_ps(widen_bf16(w + i + 8), _mm256_loadu_ps(x + i + 8), acc1);
    }
    if (i + 8 <= n) {
        acc0 = _mm256_fmadd_ps(widen_bf16(w + i), _mm256_loadu_ps(x + i), acc0);
        i += 8;
    }
    float s = hsum8(_mm256_add_ps(acc0, acc1));
    for (; i < n; i++) s += orc_bf16_to_f32(w[i]) * x[i];
    return s;
}
/* quant.rs:1259-1278 */
AVX2 static float dot_f16_avx2(const uint8_t* w, const float* x, long n) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    long i = 0;
    for (; i + 16 <= n; i += 16) {
        __m256 h0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(w + 2 * i)));
        __m256 h1 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(w + 2 * i + 16)));
        acc0 = _mm256_fmadd_ps(h0, _mm256_loadu_ps(x + i), acc0);
        acc1 = _mm256_fmadd_ps(h1, _mm256_loadu_ps(x + i + 8), acc1);
    }
    float s = hsum8(_mm256_add_ps(acc0, acc1));
    for (; i < n; i++) s += f16_hw(w + 2 * i) * x[i];
    return s;
}

/* The int8 kernels are written once over `DOT_U8_I8`, the sum of products of
 * unsigned bytes u and signed bytes s into 8 i32 (quant.rs:1283-1299,
 * 1536-1544). */
#define INT8_KERNELS(SUF, ATTR, DOT_U8_I8)                                                      \
    ATTR static inline __m256i dot_u8_i8_##SUF(__m256i u, __m256i s) { return DOT_U8_I8; }      \
    ATTR static inline __m256i dot_i8_i8_##SUF(__m256i a, __m256i s) {                          \
        return dot_u8_i8_##SUF(_mm256_sign_epi8(a, a), _mm256_sign_epi8(s, a));                 \
    }                                                                                           \
    /* quant.rs:1302-1321: nibbles of 16 bytes as 32 bytes (low halves first), minus 8 */       \
    ATTR static float dot_q4_0_##SUF(const uint8_t* w, const int8_t* xq, const float* xd,       \
                                     long nb) {                                                 \
        const __m256i s8 = _mm256_set1_epi8(8);                                                 \
        __m256 acc[2] = {_mm256_setzero_ps(), _mm256_setzero_ps()};                             \
        for (long i = 0; i < nb; i++) {                                                         \
            const uint8_t* b = w + 18 * i;                                                      \
            __m256i q = _mm256_sub_epi8(q4_nibbles(b + 2), s8);                                 \
            acc[i & 1] = fma_i32(acc[i & 1], dot_i8_i8_##SUF(q, ld256(xq + 32 * i)),            \
                                 f16_hw(b) * xd[i]);                                            \
        }                                                                                       \
        return hsum8(_mm256_add_ps(acc[0], acc[1]));                                            \
    }                                                                                           \
    /* quant.rs:1323-1339: the min terms are summed apart, in block order */                    \
    ATTR static float dot_q4_1_##SUF(const uint8_t* w, const int8_t* xq, const float* xd,       \
                                     const float* xs, long nb) {                                \
        __m256 acc[2] = {_mm256_setzero_ps(), _mm256_setzero_ps()};                             \
        float summs = 0.0f;                                                                     \
        for (long i = 0; i < nb; i++) {                                                         \
            const uint8_t* b = w + 20 * i;                                                      \
            __m256i p = dot_u8_i8_##SUF(q4_nibbles(b + 4), ld256(xq + 32 * i));                 \
            acc[i & 1] = fma_i32(acc[i & 1], p, f16_hw(b) * xd[i]);                             \
            summs += f16_hw(b + 2) * xs[i];                                                     \
        }                                                                                       \
        return hsum8(_mm256_add_ps(acc[0], acc[1])) + summs;                                    \
    }                                                                                           \
    /* quant.rs:1369-1382 */                                                                    \
    ATTR static float dot_q8_0_##SUF(const uint8_t* w, const int8_t* xq, const float* xd,       \
                                     long nb) {                                                 \
        __m256 acc[2] = {_mm256_setzero_ps(), _mm256_setzero_ps()};                             \
        for (long i = 0; i < nb; i++) {                                                         \
            const uint8_t* b = w + 34 * i;                                                      \
            __m256i p = dot_i8_i8_##SUF(ld256(b + 2), ld256(xq + 32 * i));                      \
            acc[i & 1] = fma_i32(acc[i & 1], p, f16_hw(b) * xd[i]);                             \
        }                                                                                       \
        return hsum8(_mm256_add_ps(acc[0], acc[1]));                                            \
    }                                                                                           \
    /* quant.rs:1385-1473; Q5_K adds 16 where the sub-block's bit of qh is set */               \
    ATTR static float dot_q45k_##SUF(int ty, const uint8_t* w, const int8_t* xqs,               \
                                     const float* xd, const float* xs, long nb) {               \
        const __m256i m4 = _mm256_set1_epi8(0x0F), b16 = _mm256_set1_epi8(16);                  \
        __m256 acc_lo = _mm256_setzero_ps(), acc_hi = _mm256_setzero_ps();                      \
        float mins = 0.0f;                                                                      \
        long bs = ty == T_Q4K ? 144 : 176, qoff = ty == T_Q4K ? 16 : 48;                        \
        for (long i = 0; i < nb / 8; i++) {                                                     \
            const uint8_t* b = w + bs * i;                                                      \
            float d = f16_hw(b), dmin = f16_hw(b + 2);                                          \
            const uint8_t* scales = b + 4;                                                      \
            __m256i qh = ty == T_Q5K ? ld256(b + 16) : _mm256_setzero_si256();                  \
            const int8_t* xq = xqs + 256 * i;                                                   \
            for (int j = 0; j < 4; j++) {                                                       \
                __m256i v = ld256(b + qoff + 32 * j);                                           \
                __m256i lo = _mm256_and_si256(v, m4);                                           \
                __m256i hi = _mm256_and_si256(_mm256_srli_epi16(v, 4), m4);                     \
                if (ty == T_Q5K) {                                                              \
                    __m256i ma = _mm256_set1_epi8((char)(1u << (2 * j)));                       \
                    __m256i mb = _mm256_set1_epi8((char)(1u << (2 * j + 1)));                   \
                    lo = _mm256_or_si256(                                                       \
                        lo, _mm256_and_si256(_mm256_cmpeq_epi8(_mm256_and_si256(qh, ma), ma),   \
                                             b16));                                             \
                    hi = _mm256_or_si256(                                                       \
                        hi, _mm256_and_si256(_mm256_cmpeq_epi8(_mm256_and_si256(qh, mb), mb),   \
                                             b16));                                             \
                }                                                                               \
                uint8_t s1, m1, s2, m2;                                                         \
                scale_min_k4(2 * j, scales, &s1, &m1);                                          \
                scale_min_k4(2 * j + 1, scales, &s2, &m2);                                      \
                long xa = 8 * i + 2 * j, xb = xa + 1;                                           \
                acc_lo = fma_i32(acc_lo, dot_u8_i8_##SUF(lo, ld256(xq + 64 * j)),               \
                                 d * (float)s1 * xd[xa]);                                       \
                acc_hi = fma_i32(acc_hi, dot_u8_i8_##SUF(hi, ld256(xq + 64 * j + 32)),          \
                                 d * (float)s2 * xd[xb]);                                       \
                mins += dmin * ((float)m1 * xs[xa] + (float)m2 * xs[xb]);                       \
            }                                                                                   \
        }                                                                                       \
        return hsum8(_mm256_add_ps(acc_lo, acc_hi)) - mins;                                     \
    }

INT8_KERNELS(avx2, AVX2, _mm256_madd_epi16(_mm256_maddubs_epi16(u, s), _mm256_set1_epi16(1)))
INT8_KERNELS(vnni, VNNI, _mm256_dpbusd_avx_epi32(_mm256_setzero_si256(), u, s))

/* quant.rs:1476-1533: both levels use maddubs/madd here, so one body serves */
AVX2 static float dot_q6k_avx2(const uint8_t* w, const int8_t* xqs, const float* xd, long nb) {
    const __m256i m4 = _mm256_set1_epi8(0x0F), m3 = _mm256_set1_epi8(0x03),
                  s32 = _mm256_set1_epi8(32);
    __m256 acc[2] = {_mm256_setzero_ps(), _mm256_setzero_ps()};
    for (long i = 0; i < nb / 8; i++) {
        const uint8_t* b = w + 210 * i;
        float d = f16_hw(b + 208);
        const int8_t* xq = xqs + 256 * i;
        for (int n = 0; n < 2; n++) {
            __m256i ql0 = ld256(b + 64 * n), ql1 = ld256(b + 64 * n + 32);
            __m256i qh = ld256(b + 128 + 32 * n);
            const int8_t* sc = (const int8_t*)b + 192 + 8 * n;
            __m256i q[4];
            q[0] = _mm256_or_si256(_mm256_and_si256(ql0, m4),
                                   _mm256_slli_epi16(_mm256_and_si256(qh, m3), 4));
            q[1] = _mm256_or_si256(
                _mm256_and_si256(ql1, m4),
                _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2), m3), 4));
            q[2] = _mm256_or_si256(
                _mm256_and_si256(_mm256_srli_epi16(ql0, 4), m4),
                _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 4), m3), 4));
            q[3] = _mm256_or_si256(
                _mm256_and_si256(_mm256_srli_epi16(ql1, 4), m4),
                _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 6), m3), 4));
            for (int k = 0; k < 4; k++) {
                __m256i xv = ld256(xq + 128 * n + 32 * k);
                __m256i p = _mm256_sub_epi16(_mm256_maddubs_epi16(q[k], xv),
                                             _mm256_maddubs_epi16(s32, xv));
                __m256i scl = _mm256_set_m128i(_mm_set1_epi16(sc[2 * k + 1]),
                                               _mm_set1_epi16(sc[2 * k]));
                acc[k & 1] = fma_i32(acc[k & 1], _mm256_madd_epi16(p, scl),
                                     d * xd[8 * i + 4 * n + k]);
            }
        }
    }
    return hsum8(_mm256_add_ps(acc[0], acc[1]));
}
#else
static int detect_level(void) { return 0; }
#endif

/* The level `quant::kernels()` (quant.rs:548-559) would report on this host:
 * 0 scalar, 1 avx2, 2 avxvnni. */
ORC_API int orc_host_level(void) {
    static int cached = -1;
    if (cached < 0) cached = detect_level();
    return cached;
}

/* ------------------------------------------------------------------------ */
/* dot dispatch, quant.rs:415-433 and 527-544                                */

typedef struct {
    const float* xf;  /* float activations (types with uses_f32_act) */
    const int8_t* qs; /* Q8Act of the same row */
    const float* d;
    const float* s;
} act_row;

static float dot_level(int level, int ty, const uint8_t* w, act_row x, long n) {
    long nb = n / 32;
#if defined(__x86_64__)
    if (level >= 1) {
        switch (ty) {
            case T_F32: return dot_f32_avx2((const float*)w, x.xf, n);
            case T_F16: return dot_f16_avx2(w, x.xf, n);
            case T_BF16: return dot_bf16_avx2(w, x.xf, n);
            case T_Q4_0:
                return level == 2 ? dot_q4_0_vnni(w, x.qs, x.d, nb) : dot_q4_0_avx2(w, x.qs, x.d, nb);
            case T_Q4_1:
                return level == 2 ? dot_q4_1_vnni(w, x.qs, x.d, x.s, nb)
                                  : dot_q4_1_avx2(w, x.qs, x.d, x.s, nb);
            case T_Q8_0:
                return level == 2 ? dot_q8_0_vnni(w, x.qs, x.d, nb) : dot_q8_0_avx2(w, x.qs, x.d, nb);
            case T_Q4K: case T_Q5K:
                return level == 2 ? dot_q45k_vnni(ty, w, x.qs, x.d, x.s, nb)
                                  : dot_q45k_avx2(ty, w, x.qs, x.d, x.s, nb);
            case T_Q6K: return dot_q6k_avx2(w, x.qs, x.d, nb);
        }
    }
#endif
    switch (ty) {
        case T_F32: return dot_f32_seq((const float*)w, x.xf, n);
        case T_F16: return dot_f16_seq(w, x.xf, n);
        case T_BF16: return dot_bf16_seq(w, x.xf, n);
        case T_Q4_0: return sc_dot_q4_0(w, x.qs, x.d, nb);
        case T_Q4_1: return sc_dot_q4_1(w, x.qs, x.d, x.s, nb);
        case T_Q8_0: return sc_dot_q8_0(w, x.qs, x.d, nb);
        case T_Q4K: case T_Q5K: return sc_dot_q45k(ty, w, x.qs, x.d, x.s, nb);
        case T_Q6K: return sc_dot_q6k(w, x.qs, x.d, nb);
    }
    return NAN;
}

/* One weight row against one activation row (the reference's `dot`).  `xf` is
 * used by float types, `qs/d/s` by quantised ones. */
ORC_API float orc_dot(int level, int ty, const uint8_t* w, const float* xf, const int8_t* qs,
                      const float* d, const float* s, long n) {
    act_row x = {xf, qs, d, s};
    return dot_level(level, ty, w, x, n);
}

ORC_API float orc_dot_f32(int level, const float* a, const float* b, long n) {
#if defined(__x86_64__)
    if (level >= 1) return dot_f32_avx2(a, b, n);
#endif
    return dot_f32_seq(a, b, n);
}

ORC_API void orc_axpy(int level, float* y, float a, const float* x, long n) { /* quant.rs:471-481 */
#if defined(__x86_64__)
    if (level >= 1) { axpy_avx2(y, a, x, n); return; }
#endif
    for (long i = 0; i < n; i++) y[i] += a * x[i];
}

/* ------------------------------------------------------------------------ */
/* matmul, ops.rs:84-127: out[t*rows + r] = dot(w.row(r), x[t]); tasks are runs
 * of clamp(rows / (threads*8), 1, 256) rows.  Each output is computed whole
 * by one thread, so the thread count does not change the bits.              */

typedef struct {
    int8_t* qs;
    float* d;
    float* s;
} q8act;

static int q8act_make(q8act* q, const float* x, long n, long k, int threads) {
    q->qs = (int8_t*)malloc((size_t)(n * k));
    q->d = (float*)malloc(sizeof(float) * (size_t)(n * k / 32));
    q->s = (float*)malloc(sizeof(float) * (size_t)(n * k / 32));
    if (!q->qs || !q->d || !q->s) return -1;
    /* ops.rs:63-76: rows quantised in parallel, each row block-aligned */
#pragma omp parallel for num_threads(threads) schedule(static) if (threads > 1 && n > 1)
    for (long t = 0; t < n; t++)
        orc_q8_quantize(x + t * k, k, q->qs + t * k, q->d + t * k / 32, q->s + t * k / 32);
    return 0;
}
static void q8act_free(q8act* q) { free(q->qs); free(q->d); free(q->s); }

static void matmul_rows(int level, int ty, const uint8_t* w, long rows, long cols, const float* x,
                        const q8act* xq, long n, float* out, int threads) {
    long row_bytes = orc_row_size(ty, cols);
    long chunk = rows / ((long)threads * 8);
    if (chunk < 1) chunk = 1;
    if (chunk > 256) chunk = 256;
    long n_chunks = (rows + chunk - 1) / chunk;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1) if (threads > 1)
    for (long c = 0; c < n_chunks; c++) {
        long r0 = c * chunk, r1 = r0 + chunk < rows ? r0 + chunk : rows;
        for (long r = r0; r < r1; r++) {
            const uint8_t* wr = w + r * row_bytes;
            for (long t = 0; t < n; t++) {
                act_row a = {x + t * cols, xq ? xq->qs + t * cols : NULL,
                             xq ? xq->d + t * cols / 32 : NULL, xq ? xq->s + t * cols / 32 : NULL};
                out[t * rows + r] = dot_level(level, ty, wr, a, cols);
            }
        }
    }
}

ORC_API int orc_matmul(int level, int ty, const uint8_t* w, long rows, long cols, const float* x,
                       long n, float* out, int threads) {
    if (orc_row_size(ty, cols) < 0) return -1;
    if (threads < 1) threads = 1;
    q8act q = {0};
    int quant = !uses_f32_act(ty);
    if (quant && q8act_make(&q, x, n, cols, threads)) return -2;
    matmul_rows(level, ty, w, rows, cols, x, quant ? &q : NULL, n, out, threads);
    if (quant) q8act_free(&q);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* small ops, ops.rs:136-201                                                 */

ORC_API void orc_rms_norm(int level, float* x, long n_rows, const float* w, long e, float eps) {
    for (long r = 0; r < n_rows; r++) { /* ops.rs:136-144 */
        float* g = x + r * e;
        float ss = orc_dot_f32(level, g, g, e) / (float)e;
        float scale = 1.0f / sqrtf(ss + eps);
        for (long i = 0; i < e; i++) g[i] *= scale * w[i];
    }
}
ORC_API float orc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); } /* ops.rs:160-162 */
ORC_API float orc_silu(float x) { return x * orc_sigmoid(x); }           /* ops.rs:165-167 */

ORC_API void orc_softmax(float* x, long n) { /* ops.rs:192-201 */
    float max = -INFINITY;
    for (long i = 0; i < n; i++) max = x[i] > max ? x[i] : max;
    float sum = 0.0f;
    for (long i = 0; i < n; i++) {
        x[i] = expf(x[i] - max);
        sum += x[i];
    }
    float inv = 1.0f / sum;
    for (long i = 0; i < n; i++) x[i] *= inv;
}

/* f32::total_cmp as the reference's sort uses it (model.rs:263): the bits, with the
 * magnitude inverted for negative values, compared as signed integers.  A total order:
 * NaNs sort too (positive ones above +inf), so a row of NaN probabilities still yields
 * k distinct experts - the first k, every key being equal. */
static int32_t total_key(float v) {
    int32_t b;
    memcpy(&b, &v, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

/* model.rs:259-268: softmax, the k experts of highest probability with the
 * lowest index first among equals, weights = p / max(sum of the k, 2^-14).
 * `scratch` holds n_expert floats. */
ORC_API void orc_route(const float* logits, long n_expert, int k, int32_t* ids, float* w,
                       float* scratch) {
    memcpy(scratch, logits, sizeof(float) * (size_t)n_expert);
    orc_softmax(scratch, n_expert);
    /* selection of the k best by (p descending under total_cmp, id ascending): the
     * first k of the reference's full sort */
    for (int j = 0; j < k; j++) {
        long best = -1;
        for (long e = 0; e < n_expert; e++) {
            int taken = 0;
            for (int i = 0; i < j; i++) taken |= ids[i] == e;
            if (taken) continue;
            if (best < 0 || total_key(scratch[e]) > total_key(scratch[best])) best = e; /* strict: lower id wins ties */
        }
        ids[j] = (int32_t)best;
    }
    float sum = 0.0f;
    for (int j = 0; j < k; j++) sum += scratch[ids[j]];
    if (!(sum > 1.0f / 16384.0f)) sum = 1.0f / 16384.0f; /* f32::max: a NaN sum gives the floor */
    for (int j = 0; j < k; j++) w[j] = scratch[ids[j]] / sum;
}

/* ------------------------------------------------------------------------ */
/* the layer, model.rs:861-898 and 1119-1126                                 */

typedef struct {
    int32_t ty;
    int32_t _pad;
    int64_t cols, rows, n;
    const uint8_t* data;
    int64_t stride; /* bytes from one expert's matrix to the next */
    int64_t offset; /* bytes from the start of an expert's matrix to these rows */
} orc_experts;      /* model.rs:190-204 */

typedef struct {
    int32_t n_embd, n_expert, n_expert_used, n_ff_exp, n_ff_shexp, has_shared;
    const float* router; /* [n_expert][n_embd] f32 */
    orc_experts gate, up, down;
    orc_experts sh_gate, sh_up, sh_down; /* n = 1 */
    const float* sh_gate_inp;            /* [n_embd] f32 */
} orc_moe;

typedef struct {
    float* logits;     /* [n][n_expert] */
    int32_t* ids;      /* [n][k] in order of probability */
    float* weights;    /* [n][k] */
    int32_t* counts;   /* [n_expert] pairs per expert */
    int32_t* order;    /* [n*k] pair indices t*k+j grouped by expert ascending,
                          ascending pair index inside an expert */
    float* pair_out;   /* [n*k][n_embd] expert output of each pair, by pair index */
    float* shared_out; /* [n][n_embd] */
    float* shared_gate;/* [n] the logit before the sigmoid */
    int8_t* act_q;     /* [n][n_embd] Q8 rows of h */
    float* act_d;      /* [n][n_embd/32] */
    float* act_s;      /* [n][n_embd/32] */
    int8_t* mid_q;     /* [n*k][n_ff_exp] Q8 rows of silu(gate)*up, by pair index */
    float* mid_d;      /* [n*k][n_ff_exp/32] */
    float* mid;        /* [n*k][n_ff_exp] f32 silu(gate)*up, by pair index */
} orc_taps;            /* any pointer may be NULL */

static const uint8_t* expert_ptr(const orc_experts* e, long i) { /* model.rs:212-216 */
    return e->data + i * e->stride + e->offset;
}

/* model.rs:1119-1126.  y [n][down.rows]; mid (optional) [n][gate.rows];
 * midq (optional) receives the Q8 rows the down product consumed. */
static int dense_ffn(int level, const orc_experts* gate, const orc_experts* up,
                     const orc_experts* down, long ei, const float* x, long n, float* y,
                     float* mid_tap, int8_t* midq_tap, float* midd_tap, int threads) {
    long e = gate->cols, ff = gate->rows;
    float* g = (float*)malloc(sizeof(float) * (size_t)(n * ff));
    float* u = (float*)malloc(sizeof(float) * (size_t)(n * ff));
    if (!g || !u) { free(g); free(u); return -2; }
    q8act xq = {0};
    int need_q = !uses_f32_act(gate->ty) || !uses_f32_act(up->ty);
    if (need_q && q8act_make(&xq, x, n, e, threads)) return -2;
    matmul_rows(level, gate->ty, expert_ptr(gate, ei), ff, e, x,
                uses_f32_act(gate->ty) ? NULL : &xq, n, g, threads);
    matmul_rows(level, up->ty, expert_ptr(up, ei), ff, e, x, uses_f32_act(up->ty) ? NULL : &xq, n,
                u, threads);
    if (need_q) q8act_free(&xq);
    for (long i = 0; i < n * ff; i++) g[i] = orc_silu(g[i]) * u[i];
    if (mid_tap) memcpy(mid_tap, g, sizeof(float) * (size_t)(n * ff));
    q8act gq = {0};
    int down_q = !uses_f32_act(down->ty);
    if (down_q) {
        if (q8act_make(&gq, g, n, ff, threads)) return -2;
        if (midq_tap) memcpy(midq_tap, gq.qs, (size_t)(n * ff));
        if (midd_tap) memcpy(midd_tap, gq.d, sizeof(float) * (size_t)(n * ff / 32));
    }
    matmul_rows(level, down->ty, expert_ptr(down, ei), down->rows, ff, g, down_q ? &gq : NULL, n, y,
                threads);
    if (down_q) q8act_free(&gq);
    free(g);
    free(u);
    return 0;
}

ORC_API int orc_moe_forward(const orc_moe* m, const float* h, long n, float* out, int level,
                            int threads, const orc_taps* taps) {
    static const orc_taps none;
    if (!taps) taps = &none;
    if (threads < 1) threads = 1;
    long e = m->n_embd, ne = m->n_expert, k = m->n_expert_used, ff = m->n_ff_exp;
    float* logits = (float*)malloc(sizeof(float) * (size_t)(n * ne));
    int32_t* ids = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n * k));
    float* wts = (float*)malloc(sizeof(float) * (size_t)(n * k));
    int32_t* counts = (int32_t*)calloc((size_t)ne, sizeof(int32_t));
    int32_t* order = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n * k));
    float* scratch = (float*)malloc(sizeof(float) * (size_t)ne);
    if (!logits || !ids || !wts || !counts || !order || !scratch) return -2;

    /* model.rs:864-865: router product, f32 weights against f32 rows */
    matmul_rows(level, T_F32, (const uint8_t*)m->router, ne, e, h, NULL, n, logits, threads);
    /* model.rs:867-873 */
    for (long t = 0; t < n; t++) {
        orc_route(logits + t * ne, ne, (int)k, ids + t * k, wts + t * k, scratch);
        for (long j = 0; j < k; j++) counts[ids[t * k + j]]++;
    }
    /* the per-expert lists, in push order: ascending token, hence ascending pair index */
    long* start = (long*)malloc(sizeof(long) * (size_t)(ne + 1));
    long* fill = (long*)malloc(sizeof(long) * (size_t)ne);
    start[0] = 0;
    for (long i = 0; i < ne; i++) { start[i + 1] = start[i] + counts[i]; fill[i] = start[i]; }
    for (long p = 0; p < n * k; p++) order[fill[ids[p]]++] = (int32_t)p;

    if (taps->logits) memcpy(taps->logits, logits, sizeof(float) * (size_t)(n * ne));
    if (taps->ids) memcpy(taps->ids, ids, sizeof(int32_t) * (size_t)(n * k));
    if (taps->weights) memcpy(taps->weights, wts, sizeof(float) * (size_t)(n * k));
    if (taps->counts) memcpy(taps->counts, counts, sizeof(int32_t) * (size_t)ne);
    if (taps->order) memcpy(taps->order, order, sizeof(int32_t) * (size_t)(n * k));
    if (taps->act_q && taps->act_d && taps->act_s)
        for (long t = 0; t < n; t++)
            orc_q8_quantize(h + t * e, e, taps->act_q + t * e, taps->act_d + t * e / 32,
                            taps->act_s + t * e / 32);

    memset(out, 0, sizeof(float) * (size_t)(n * e));
    int rc = 0;
    /* model.rs:875-889: experts ascending, gather, dense_ffn, weighted add */
    for (long i = 0; i < ne && !rc; i++) {
        long len = counts[i];
        if (!len) continue;
        float* x = (float*)malloc(sizeof(float) * (size_t)(len * e));
        float* y = (float*)malloc(sizeof(float) * (size_t)(len * e));
        float* mid = taps->mid ? (float*)malloc(sizeof(float) * (size_t)(len * ff)) : NULL;
        int8_t* mq = taps->mid_q ? (int8_t*)malloc((size_t)(len * ff)) : NULL;
        float* md = taps->mid_d ? (float*)malloc(sizeof(float) * (size_t)(len * ff / 32)) : NULL;
        if (!x || !y) return -2;
        for (long a = 0; a < len; a++) {
            long t = order[start[i] + a] / k;
            memcpy(x + a * e, h + t * e, sizeof(float) * (size_t)e);
        }
        rc = dense_ffn(level, &m->gate, &m->up, &m->down, i, x, len, y, mid, mq, md, threads);
        for (long a = 0; a < len && !rc; a++) {
            long p = order[start[i] + a], t = p / k;
            orc_axpy(level, out + t * e, wts[p], y + a * e, e);
            if (taps->pair_out) memcpy(taps->pair_out + p * e, y + a * e, sizeof(float) * (size_t)e);
            if (mid) memcpy(taps->mid + p * ff, mid + a * ff, sizeof(float) * (size_t)ff);
            if (mq) memcpy(taps->mid_q + p * ff, mq + a * ff, (size_t)ff);
            if (md) memcpy(taps->mid_d + p * ff / 32, md + a * ff / 32, sizeof(float) * (size_t)(ff / 32));
        }
        free(x); free(y); free(mid); free(mq); free(md);
    }
    /* model.rs:890-896: shared expert last, scaled by sigmoid(gate_inp . h) */
    if (m->has_shared && !rc) {
        float* y = (float*)malloc(sizeof(float) * (size_t)(n * e));
        float* g = (float*)malloc(sizeof(float) * (size_t)n);
        if (!y || !g) return -2;
        rc = dense_ffn(level, &m->sh_gate, &m->sh_up, &m->sh_down, 0, h, n, y, NULL, NULL, NULL,
                       threads);
        matmul_rows(level, T_F32, (const uint8_t*)m->sh_gate_inp, 1, e, h, NULL, n, g, threads);
        for (long t = 0; t < n && !rc; t++)
            orc_axpy(level, out + t * e, orc_sigmoid(g[t]), y + t * e, e);
        if (taps->shared_out) memcpy(taps->shared_out, y, sizeof(float) * (size_t)(n * e));
        if (taps->shared_gate) memcpy(taps->shared_gate, g, sizeof(float) * (size_t)n);
        free(y); free(g);
    }
    free(logits); free(ids); free(wts); free(counts); free(order); free(scratch);
    free(start); free(fill);
    return rc;
}

/* A stack of layers with the residual carried over (model.rs:761-791, FFN half
 * only): per layer h = rms_norm(x, norm_w[l], eps); x += moe_l(h). */
ORC_API int orc_moe_stack(const orc_moe* layers, int n_layers, const float* const* norm_w,
                          float eps, float* x, long n, int level, int threads) {
    long e = layers[0].n_embd;
    float* h = (float*)malloc(sizeof(float) * (size_t)(n * e));
    float* y = (float*)malloc(sizeof(float) * (size_t)(n * e));
    if (!h || !y) return -2;
    int rc = 0;
    for (int l = 0; l < n_layers && !rc; l++) {
        memcpy(h, x, sizeof(float) * (size_t)(n * e)); /* ops.rs:146-149 */
        orc_rms_norm(level, h, n, norm_w[l], e, eps);
        rc = orc_moe_forward(&layers[l], h, n, y, level, threads, NULL);
        for (long i = 0; i < n * e; i++) x[i] += y[i]; /* ops.rs:175-177 */
    }
    free(h); free(y);
    return rc;
}

/* the host's usable cores; every parallel loop here names its thread count, so this
 * holds under a launcher that sets OMP_NUM_THREADS=1 for its workers */
ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}
