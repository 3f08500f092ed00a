// Grouped expert products for decode-sized groups: gate+up with the SwiGLU and
// the Q8 re-quantisation of its output fused, then down.
// Reference: dense_ffn (engine/src/model.rs:1119-1126) over matmul
// (engine/src/ops.rs:84-127) and the per-type dots (engine/src/quant.rs:
// 599-686 scalar, 1369-1533 AVX2), for each expert's token list
// (model.rs:875-889) and for the shared expert (model.rs:890-896).
//
// Design.  Blocks of four warps (several per SM) pull work items - a tile of
// up to 8 tokens of one group times a chunk of weight rows (64 gate rows with
// their 64 up rows, or 128 down rows) - from a counter.  The device layout
// (common.cuh) stores what one pipeline stage needs, one K-slice of the
// chunk's 128 rows, contiguously: a stage arrives as one bulk copy of weights
// plus one of the tile's activation record (cp.async.bulk on an mbarrier),
// double-buffered, and the stream of stages runs on across item boundaries.  Each 32-element block dot is an int8 tensor-core product
// (mma.sync m16n8k32, 16 weight rows x 8 tokens): its int32 results are the
// reference's block dots, scaled in f32 by the weight block scale and the
// activation block scale.  The measured __dp4a rate of this GPU (64 lanes per
// clock per SM) cannot keep up with HBM beyond two tokens per expert, which is
// why the block dots are on the tensor cores even at decode sizes.  No atomics
// on data: results are run-to-run identical.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "formats.cuh"
#include "tcgen05.cuh"
#include "launch.cuh"

namespace bivmoe {

constexpr int EX_TT = 8;                       // tokens per tile
constexpr uint32_t EX_WAIT_LIMIT = 1u << 16;   // bounded mbarrier wait: tries that may sleep wait_hint_ns each

enum { MODE_GATEUP = 0, MODE_DOWN = 1 };

struct ExpertArgs {
    DevTiles w, sh;        // the routed experts' and the shared expert's tiles for this product
    // activations by position, slice-major (common.cuh): rows of h for GATEUP, of mid for DOWN
    const float* x_f32;    // float-activation types
    const uint8_t* x_t;    // quantised types: the Q8 records, [K/256][R/8]
    int act_rows;          // R
    float* out;            // GATEUP: mid f32, slice-major; DOWN: pair_out [R][rows]
    uint8_t* out_t;        // GATEUP with a quantised down type: the Q8 records of mid
    const int32_t* grp_expert;
    const int32_t* grp_start;
    const int32_t* grp_count;
    const int4* tile_desc;    // {expert (n_expert: shared), first position, tokens, 0}
    const int32_t* n_tiles;   // [0] all tiles, [1] tiles of the shared group (they come first)
    uint32_t* work_ctr;
    int32_t* status;
    int n, k, n_expert;
    int tiles_mode;        // 0: every tile, 1: skip the shared group's, 2: only the shared group's
    int chunks;            // row chunks per group in this launch
    uint32_t wait_hint_ns; // how long one mbarrier try may sleep
};

// ---------------------------------------------------------------------------
// PTX helpers: mbarrier, bulk copy (TMA, untiled form), warp-level int8 MMA
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)   // may sleep up to hint_ns per try
        : "memory");
    return ok != 0;
}
// One look, without blocking: has the phase of parity `parity` completed?
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for a phase with an iteration limit; false when it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    for (uint32_t i = 0; i < EX_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity, hint_ns)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// D[16x8] = A[16x32] * B[32x8], s8 x s8 -> s32.  Lane (g = lane/4, c = lane%4) holds
// A: a0 (row g, k 4c..4c+3), a1 (row g+8, same k), a2 (row g, k 16+4c..), a3 (row g+8, k 16+4c..)
// B: b0 (k 4c..4c+3, column g), b1 (k 16+4c.., column g)
// D: d0 (row g, col 2c), d1 (row g, col 2c+1), d2 (row g+8, col 2c), d3 (row g+8, col 2c+1)
__device__ __forceinline__ void mma_s8_k32(int (&d)[4], const int (&a)[4], int b0, int b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
// The same with unsigned A bytes (u8 x s8), returning the sums as floats: the
// accumulator starts at the bit pattern of 1.5 * 2^23, so the int32 result read as
// an f32 is 12582912 + sum exactly (|sum| < 2^22), and one f32 subtraction - on the
// multiply-add pipe instead of a conversion on the integer pipe - gives float(sum).
__device__ __forceinline__ void mma_u8s8_k32_f(float (&f)[4], const int (&a)[4], int b0, int b1) {
    int d[4];
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0x4B400000));
#pragma unroll
    for (int i = 0; i < 4; i++) f[i] = __fsub_rn(__int_as_float(d[i]), 12582912.0f);
}
// The same, returning the results two tokens at a time (f32x2): lo = row g, hi = row g+8.
__device__ __forceinline__ void mma_u8s8_k32_f2(f32x2& lo, f32x2& hi, const int (&a)[4], int b0, int b1) {
    int d[4];
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0x4B400000));
    const f32x2 neg = pk(-12582912.0f, -12582912.0f);
    lo = add2(pk(__int_as_float(d[0]), __int_as_float(d[1])), neg);
    hi = add2(pk(__int_as_float(d[2]), __int_as_float(d[3])), neg);
}
// the k = 16 form: a0 (row g, k 4c..4c+3), a1 (row g+8), b0 (k 4c..4c+3, column g)
__device__ __forceinline__ void mma_s8_k16(int (&d)[4], int a0, int a1, int b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
        "{%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// D[16x8] += A[16x8] * B[8x8] in tf32 with f32 accumulation.  a0 (row g, k c), a1 (row g+8, k c),
// a2 (row g, k c+4), a3 (row g+8, k c+4); b0 (k c, column g), b1 (k c+4, column g); D as above.
__device__ __forceinline__ void mma_tf32_k8(float (&d)[4], const float (&a)[4], float b0, float b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])),
          "r"(__float_as_uint(a[3])), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// ---------------------------------------------------------------------------
// Per-type arithmetic of one staged K-slice for one warp.
//   rowp[mt][r]  this lane's two rows (g, g+8) of the warp's two 16-row MMA tiles:
//                slice + row*16; unit u of the row is 2048*u further (128 rows x 16
//                bytes), so byte `off` of the row's slice is WU(p, off)
//   act          the tile's Q8 record (common.cuh): q as [16 units][8 tokens][16 bytes],
//                then dx, s_hi, s_lo as [8 blocks][8 tokens] f32
//   XQ(act,u)    this lane's B-fragment word of unit u: token g, bytes 4c..4c+3
//   acc[mt][i]   i = 2*r + tt: row g+8r, token 2c+tt
// All of these take 32-bit shared-memory addresses and load with ld.shared: no
// generic-address arithmetic, constant offsets fold into the instruction.
#define WU(w, off) ((w) + ((((off)) >> 4) << 11) + ((off) & 15))
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float ldsf(uint32_t a) { return __uint_as_float(lds32(a)); }
__device__ __forceinline__ f32x2 lds64(uint32_t a) {
    f32x2 v;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
#define LDS32(a) lds32(a)
#define XQ(xlane, u) ((int)lds32((xlane) + (u) * 128))

struct NoSide {};

template <int TY> struct Fmt;

// ---- Q8_0 (quant.rs:599-607): term = d_w * d_x * sum(q_w * q_x) ------------
template <> struct Fmt<BIVMOE_Q8_0> {
    static constexpr int ELEMS = 256, SL = 272, MINB = 2;   // consumer groups per block: 2 x 2 stages of 37.7 KB
    static constexpr bool F32ACT = false;
    using Side = NoSide;
    __device__ static void compute(const uint32_t (&rowp)[2][2], Side, uint32_t act,
                                   float (&acc)[2][4], int g, int c) {
        const uint32_t dxp = act + kActOffDx;
        uint4 dwv[2][2];   // the 8 f16 scales of each row's slice (unit 16)
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int r = 0; r < 2; r++) dwv[mt][r] = lds128(WU(rowp[mt][r], 256));
        const uint32_t xlane = act + g * 16 + 4 * c;
#pragma unroll
        for (int j = 0; j < 4; j++) {       // blocks 2j and 2j+1
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int b = 2 * j + h;
                const int b0 = XQ(xlane, 2 * b), b1 = XQ(xlane, 2 * b + 1);
                const f32x2 dxv = lds64(dxp + 4 * (b * 8 + 2 * c));   // tokens 2c, 2c+1
                const float dx[2] = {lo_of(dxv), hi_of(dxv)};
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    int a[4], I[4];
                    a[0] = (int)LDS32(WU(rowp[mt][0], 32 * b) + 4 * c);
                    a[1] = (int)LDS32(WU(rowp[mt][1], 32 * b) + 4 * c);
                    a[2] = (int)LDS32(WU(rowp[mt][0], 32 * b + 16) + 4 * c);
                    a[3] = (int)LDS32(WU(rowp[mt][1], 32 * b + 16) + 4 * c);
                    mma_s8_k32(I, a, b0, b1);
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const uint32_t wv = (&dwv[mt][r].x)[b >> 1];
                        const float dw = __half2float(__ushort_as_half((unsigned short)(wv >> (16 * (b & 1)))));
#pragma unroll
                        for (int tt = 0; tt < 2; tt++)
                            acc[mt][2 * r + tt] = fmaf(dw, dx[tt] * (float)I[2 * r + tt], acc[mt][2 * r + tt]);
                    }
                }
            }
        }
    }
};

// ---- Q4_0 / Q4_1 (quant.rs:570-597): per 32-element block
//      Q4_0: d * d_x * sum((q - 8) * q_x)        Q4_1: d * d_x * sum(q * q_x) + m * s_x
//      A block's 16 bytes hold element j in the low half of byte j and element j + 16
//      in the high half: one word per row and block gives both halves of the MMA's K.
//      The nibbles go to the high half of their byte - Q4_0 with bit 3 flipped, which
//      makes the byte the int8 value 16 * (q - 8); Q4_1 as unsigned 16 * q - and the
//      exact factor 1/16 goes into the scale.
template <int TY> struct FmtQ4 {
    static constexpr int ELEMS = 256, SL = TY == BIVMOE_Q4_0 ? 144 : 160, MINB = 4;
    static constexpr bool F32ACT = false;
    using Side = NoSide;
    __device__ static void mma_f2(f32x2& lo, f32x2& hi, const int (&a)[4], int b0, int b1) {
        if (TY == BIVMOE_Q4_1) {
            mma_u8s8_k32_f2(lo, hi, a, b0, b1);
        } else {
            int d[4];
            asm volatile(
                "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                "{%10,%10,%10,%10};"
                : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0x4B400000));
            const f32x2 neg = pk(-12582912.0f, -12582912.0f);
            lo = add2(pk(__int_as_float(d[0]), __int_as_float(d[1])), neg);
            hi = add2(pk(__int_as_float(d[2]), __int_as_float(d[3])), neg);
        }
    }
    __device__ static float half_at(const uint4& v, int b) {
        const uint32_t w = (&v.x)[b >> 1];
        return __half2float(__ushort_as_half((unsigned short)(w >> (16 * (b & 1)))));
    }
    // half i (0..3, not known at compile time) of the four in the words w0, w1
    __device__ static float half_sel(uint32_t w0, uint32_t w1, int i) {
        const uint32_t w = (i & 2) ? w1 : w0;
        return __half2float(__ushort_as_half((unsigned short)((i & 1) ? w >> 16 : w)));
    }
    __device__ static void compute(const uint32_t (&rowp)[2][2], Side, uint32_t act,
                                   float (&acc)[2][4], int g, int c) {
        const uint32_t dxp = act + kActOffDx, shi = act + kActOffSHi, slo = act + kActOffSLo;
        uint4 dwv[2][2], mv[2][2];   // the 8 f16 scales (unit 8) and minimums (unit 9) of each row's slice
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int r = 0; r < 2; r++) {
                dwv[mt][r] = lds128(WU(rowp[mt][r], 128));
                if (TY == BIVMOE_Q4_1) mv[mt][r] = lds128(WU(rowp[mt][r], 144));
            }
        // Q4_1's term sum_b m[r][b] * s[t][b] is a 16x8x8 product: tf32 on the tensor core,
        // exact products because m is an f16 and s comes split in two tf32-exact parts.
        float tM[2][4] = {};
        if (TY == BIVMOE_Q4_1) {
            const float bh0 = ldsf(shi + 4 * (c * 8 + g)), bh1 = ldsf(shi + 4 * ((c + 4) * 8 + g));
            const float bl0 = ldsf(slo + 4 * (c * 8 + g)), bl1 = ldsf(slo + 4 * ((c + 4) * 8 + g));
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                float a[4];
                a[0] = half_sel(mv[mt][0].x, mv[mt][0].y, c);
                a[1] = half_sel(mv[mt][1].x, mv[mt][1].y, c);
                a[2] = half_sel(mv[mt][0].z, mv[mt][0].w, c);
                a[3] = half_sel(mv[mt][1].z, mv[mt][1].w, c);
                mma_tf32_k8(tM[mt], a, bh0, bh1);
                mma_tf32_k8(tM[mt], a, bl0, bl1);
            }
        }
        f32x2 tS[2][2] = {};   // [mt][r]: tokens 2c, 2c+1 of row g + 8r
        const uint32_t xlane = act + g * 16 + 4 * c;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const int b0 = XQ(xlane, 2 * b), b1 = XQ(xlane, 2 * b + 1);
            const f32x2 dxv = lds64(dxp + 4 * (b * 8 + 2 * c));   // d of tokens 2c, 2c+1
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const uint32_t w0 = LDS32(WU(rowp[mt][0], 16 * b) + 4 * c);
                const uint32_t w1 = LDS32(WU(rowp[mt][1], 16 * b) + 4 * c);
                const uint32_t flip = TY == BIVMOE_Q4_0 ? 0x80808080u : 0u;
                int a[4];
                a[0] = (int)(((w0 << 4) & 0xF0F0F0F0u) ^ flip);
                a[1] = (int)(((w1 << 4) & 0xF0F0F0F0u) ^ flip);
                a[2] = (int)((w0 & 0xF0F0F0F0u) ^ flip);
                a[3] = (int)((w1 & 0xF0F0F0F0u) ^ flip);
                f32x2 I[2];   // 16 x the int32 block dots, exactly, as floats
                mma_f2(I[0], I[1], a, b0, b1);
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const float dw = half_at(dwv[mt][r], b) * 0.0625f;
                    tS[mt][r] = fma2(pk(dw, dw), mul2(dxv, I[r]), tS[mt][r]);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float ts = (i & 1) ? hi_of(tS[mt][i >> 1]) : lo_of(tS[mt][i >> 1]);
                acc[mt][i] += ts + tM[mt][i];
            }
    }
};
template <> struct Fmt<BIVMOE_Q4_0> : FmtQ4<BIVMOE_Q4_0> {};
template <> struct Fmt<BIVMOE_Q4_1> : FmtQ4<BIVMOE_Q4_1> {};

// ---- Q4_K / Q5_K (quant.rs:609-649): per sub-block
//      d*sc*d_x*sum(q*q_x) - dmin*m*s_x ; Q5_K adds bit sb of qh[l] as value bit 4.
//      A stage is one super-block, so d and dmin are applied once per stage.
template <int TY> struct FmtK45 {
    static constexpr int QOFF = TY == BIVMOE_Q4_K ? 16 : 48;
    static constexpr int ELEMS = 256, SL = TY == BIVMOE_Q4_K ? 144 : 176, MINB = 4;
    static constexpr bool F32ACT = false;
    using Side = NoSide;
    __device__ static void compute(const uint32_t (&rowp)[2][2], Side, uint32_t act,
                                   float (&acc)[2][4], int g, int c) {
        const uint32_t dxp = act + kActOffDx, shi = act + kActOffSHi, slo = act + kActOffSLo;
        float d[2][2], dmin[2][2];
        K4Scales sc[2][2];
        uint32_t qh[2][2][2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint4 v = lds128(rowp[mt][r]);
                const __half2 dd = *(const __half2*)&v.x;
                d[mt][r] = __low2float(dd);
                dmin[mt][r] = __high2float(dd);
                sc[mt][r] = unpack_k4_scales(v.y, v.z, v.w);
                if (TY == BIVMOE_Q5_K) {   // the high bits of elements 4c..4c+3 and 16+4c..
                    qh[mt][r][0] = LDS32(WU(rowp[mt][r], 16) + 4 * c);
                    qh[mt][r][1] = LDS32(WU(rowp[mt][r], 32) + 4 * c);
                }
            }
        // The min term sum_b m[r][b] * s[t][b] of the stage is a 16x8x8 product: on the
        // tensor core in tf32, exact because m is a 6-bit integer and s comes split in
        // two tf32-exact parts.  Lane (g, c) supplies m of blocks c, c+4 and s of token g.
        float tM[2][4] = {};
        {
            const float bh0 = ldsf(shi + 4 * (c * 8 + g)), bh1 = ldsf(shi + 4 * ((c + 4) * 8 + g));
            const float bl0 = ldsf(slo + 4 * (c * 8 + g)), bl1 = ldsf(slo + 4 * ((c + 4) * 8 + g));
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                float a[4];
                a[0] = (float)((sc[mt][0].m_lo >> (8 * c)) & 0xFF);
                a[1] = (float)((sc[mt][1].m_lo >> (8 * c)) & 0xFF);
                a[2] = (float)((sc[mt][0].m_hi >> (8 * c)) & 0xFF);
                a[3] = (float)((sc[mt][1].m_hi >> (8 * c)) & 0xFF);
                mma_tf32_k8(tM[mt], a, bh0, bh1);
                mma_tf32_k8(tM[mt], a, bl0, bl1);
            }
        }
        f32x2 tS[2][2] = {};   // [mt][r]: tokens 2c, 2c+1 of row g + 8r
        const uint32_t xlane = act + g * 16 + 4 * c;
#pragma unroll
        for (int j = 0; j < 4; j++) {       // sub-blocks 2j (low nibbles) and 2j+1 (high nibbles)
            const f32x2 xa = lds64(dxp + 4 * ((2 * j) * 8 + 2 * c));             // d of tokens 2c, 2c+1
            const f32x2 xb = lds64(dxp + 4 * ((2 * j + 1) * 8 + 2 * c));
            const int blo0 = XQ(xlane, 4 * j), blo1 = XQ(xlane, 4 * j + 1);
            const int bhi0 = XQ(xlane, 4 * j + 2), bhi1 = XQ(xlane, 4 * j + 3);
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                uint32_t w[4];
                w[0] = LDS32(WU(rowp[mt][0], QOFF + 32 * j) + 4 * c);
                w[1] = LDS32(WU(rowp[mt][1], QOFF + 32 * j) + 4 * c);
                w[2] = LDS32(WU(rowp[mt][0], QOFF + 32 * j + 16) + 4 * c);
                w[3] = LDS32(WU(rowp[mt][1], QOFF + 32 * j + 16) + 4 * c);
                int alo[4], ahi[4];
                f32x2 I[2];   // the int32 block dots, exactly, as floats: [r] tokens 2c, 2c+1
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    alo[i] = (int)(w[i] & 0x0F0F0F0Fu);
                    if (TY == BIVMOE_Q4_K) {
                        // the high nibbles stay in place: unsigned bytes worth 16x the value,
                        // the exact factor 1/16 goes into the scale
                        ahi[i] = (int)(w[i] & 0xF0F0F0F0u);
                    } else {
                        ahi[i] = (int)((w[i] >> 4) & 0x0F0F0F0Fu);
                        const uint32_t hb = qh[mt][i & 1][i >> 1];
                        alo[i] |= (int)(((hb >> (2 * j)) & 0x01010101u) << 4);
                        ahi[i] |= (int)(((hb >> (2 * j + 1)) & 0x01010101u) << 4);
                    }
                }
                mma_u8s8_k32_f2(I[0], I[1], alo, blo0, blo1);
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const float scf = (float)k4_scale(sc[mt][r], 2 * j);
                    tS[mt][r] = fma2(pk(scf, scf), mul2(xa, I[r]), tS[mt][r]);
                }
                mma_u8s8_k32_f2(I[0], I[1], ahi, bhi0, bhi1);
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const float scf = (float)k4_scale(sc[mt][r], 2 * j + 1) * (TY == BIVMOE_Q4_K ? 0.0625f : 1.0f);
                    tS[mt][r] = fma2(pk(scf, scf), mul2(xb, I[r]), tS[mt][r]);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float ts = (i & 1) ? hi_of(tS[mt][i >> 1]) : lo_of(tS[mt][i >> 1]);
                acc[mt][i] += d[mt][i >> 1] * ts - dmin[mt][i >> 1] * tM[mt][i];
            }
    }
};
template <> struct Fmt<BIVMOE_Q4_K> : FmtK45<BIVMOE_Q4_K> {};
template <> struct Fmt<BIVMOE_Q5_K> : FmtK45<BIVMOE_Q5_K> {};

// ---- Q6_K (quant.rs:651-686), slice = ql[128] qh[64] scales[16], d aside: per
//      32-block d * d_x * (sc[2g]*sum16 + sc[2g+1]*sum16), 6-bit values minus 32.
//      The int8 scales apply to 16 elements, so the products are k = 16 MMAs.
template <> struct Fmt<BIVMOE_Q6_K> {
    static constexpr int ELEMS = 256, SL = 208, MINB = 3;
    static constexpr bool F32ACT = false;
    struct Side { float d[2][2]; };     // the super-block's f16 scale of the lane's four rows
    // 6-bit values 0..63 in the four bytes of v, minus 32, as int8: v^0x20 when
    // v >= 32, else v | 0xE0
    __device__ static int sub32(uint32_t v) {
        const uint32_t t = v ^ 0x20202020u;
        return (int)(t | ((t & 0x20202020u) * 7u));
    }
    __device__ static void compute(const uint32_t (&rowp)[2][2], Side sd, uint32_t act,
                                   float (&acc)[2][4], int g, int c) {
        const uint32_t dxp = act + kActOffDx;
        uint4 scv[2][2];   // the 16 int8 scales of each row's super-block (unit 12)
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int r = 0; r < 2; r++) scv[mt][r] = lds128(WU(rowp[mt][r], 192));
        const uint32_t xlane = act + g * 16 + 4 * c;
#pragma unroll
        for (int n = 0; n < 2; n++) {
            uint32_t qh[2][2][2];   // [mt][r][lhalf]
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int lh = 0; lh < 2; lh++)
                        qh[mt][r][lh] = LDS32(WU(rowp[mt][r], 128 + 32 * n + 16 * lh) + 4 * c);
#pragma unroll
            for (int par = 0; par < 2; par++) {   // kq = par (low nibbles) and par + 2 (high nibbles)
                uint32_t ql[2][2][2];
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int r = 0; r < 2; r++)
#pragma unroll
                        for (int lh = 0; lh < 2; lh++)
                            ql[mt][r][lh] = LDS32(WU(rowp[mt][r], 64 * n + 32 * par + 16 * lh) + 4 * c);
#pragma unroll
                for (int hi = 0; hi < 2; hi++) {
                    const int kq = par + 2 * hi, xb = 4 * n + kq;
                    const f32x2 dxv = lds64(dxp + 4 * (xb * 8 + 2 * c));
                    const float dx0 = lo_of(dxv), dx1 = hi_of(dxv);
                    const int b0 = XQ(xlane, 2 * xb), b1 = XQ(xlane, 2 * xb + 1);
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        int a[2][2];   // [lhalf][r]
#pragma unroll
                        for (int r = 0; r < 2; r++)
#pragma unroll
                            for (int lh = 0; lh < 2; lh++) {
                                const uint32_t nib = (hi ? ql[mt][r][lh] >> 4 : ql[mt][r][lh]) & 0x0F0F0F0Fu;
                                const uint32_t hb = ((qh[mt][r][lh] >> (2 * kq)) & 0x03030303u) << 4;
                                a[lh][r] = sub32(nib | hb);
                            }
                        int Ia[4], Ib[4];
                        mma_s8_k16(Ia, a[0][0], a[0][1], b0);
                        mma_s8_k16(Ib, a[1][0], a[1][1], b1);
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const uint32_t sw = (&scv[mt][r].x)[(8 * n + 2 * kq) >> 2];
                            const int sh = 8 * ((8 * n + 2 * kq) & 3);
                            const int sca = (int)(int8_t)(sw >> sh), scb = (int)(int8_t)(sw >> (sh + 8));
                            const float dr = sd.d[mt][r];
                            const int i0 = sca * Ia[2 * r] + scb * Ib[2 * r];
                            const int i1 = sca * Ia[2 * r + 1] + scb * Ib[2 * r + 1];
                            acc[mt][2 * r] = fmaf(dr, dx0 * (float)i0, acc[mt][2 * r]);
                            acc[mt][2 * r + 1] = fmaf(dr, dx1 * (float)i1, acc[mt][2 * r + 1]);
                        }
                    }
                }
            }
        }
    }
};

// ---- BF16, F16 and F32 weights meet f32 activations (quant.rs:483-521, 1229-1281):
//      f32 multiply-adds, a lane per weight row, activations read as broadcasts ----
template <int TY> struct FmtFloat {
    static constexpr int ELEMS = 64, SL = TY == BIVMOE_F32 ? 256 : 128, MINB = TY == BIVMOE_F32 ? 3 : 4;
    static constexpr bool F32ACT = true;
    static constexpr int PER_UNIT = TY == BIVMOE_F32 ? 4 : 8;   // values in a 16-byte unit
    using Side = NoSide;
    __device__ static void widen(const uint4& v, float (&w)[8]) {
        if (TY == BIVMOE_BF16) {
            w[0] = __uint_as_float(v.x << 16); w[1] = __uint_as_float(v.x & 0xFFFF0000u);
            w[2] = __uint_as_float(v.y << 16); w[3] = __uint_as_float(v.y & 0xFFFF0000u);
            w[4] = __uint_as_float(v.z << 16); w[5] = __uint_as_float(v.z & 0xFFFF0000u);
            w[6] = __uint_as_float(v.w << 16); w[7] = __uint_as_float(v.w & 0xFFFF0000u);
        } else if (TY == BIVMOE_F16) {
            const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(*(const __half2*)&p[i]);
                w[2 * i] = f.x;
                w[2 * i + 1] = f.y;
            }
        } else {
            w[0] = __uint_as_float(v.x); w[1] = __uint_as_float(v.y);
            w[2] = __uint_as_float(v.z); w[3] = __uint_as_float(v.w);
            w[4] = w[5] = w[6] = w[7] = 0.0f;
        }
    }
    // `wrow`: this lane's row (tile + row*16); acc[t] += dot(row slice, token t)
    __device__ static void compute_f32(const uint8_t* wrow, const float* xf, int cnt,
                                       float (&acc)[EX_TT]) {
#pragma unroll 2
        for (int u = 0; u < SL / 16; u++) {
            float w[8];
            widen(*(const uint4*)(wrow + 2048 * u), w);
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cnt) {
                    const float4* xp = (const float4*)(xf + t * ELEMS + PER_UNIT * u);
                    const float4 x0 = xp[0];
                    float s = acc[t];
                    s = fmaf(w[0], x0.x, s); s = fmaf(w[1], x0.y, s); s = fmaf(w[2], x0.z, s);
                    s = fmaf(w[3], x0.w, s);
                    if (PER_UNIT == 8) {
                        const float4 x1 = xp[1];
                        s = fmaf(w[4], x1.x, s); s = fmaf(w[5], x1.y, s);
                        s = fmaf(w[6], x1.z, s); s = fmaf(w[7], x1.w, s);
                    }
                    acc[t] = s;
                }
            }
        }
    }
};
template <> struct Fmt<BIVMOE_BF16> : FmtFloat<BIVMOE_BF16> {};
template <> struct Fmt<BIVMOE_F16> : FmtFloat<BIVMOE_F16> {};
template <> struct Fmt<BIVMOE_F32> : FmtFloat<BIVMOE_F32> {};

// ---------------------------------------------------------------------------
// The kernel.  One block per SM: G consumer groups of four warps and one producer
// warp.  A group works on its own items - a tile of up to 8 tokens times one chunk
// (gate+up) or two chunks (down) - and owns a two-slot ring of stages (one K-slice of a
// chunk's 128 rows plus the tile's activation record) that lane g of the producer warp
// keeps full: the lane takes the group's next item from the block's own list - item i of
// a launch belongs to block i mod gridDim.x, so every SM gets the same number of (equal)
// items give or take one, and the groups of a block share its list through a counter in
// shared memory - and issues its stages as slots come free.  (Claiming from one global
// counter instead left the SMs unevenly loaded at the end: measured 33 k to 69 k active
// cycles per SM, because an SM's groups share its issue slots and an SM that happened to
// claim four late items took twice as long over them as one that claimed two.)  A consumer warp waits for a slot,
// computes its 32 rows of the stage, and hands the slot back with one mbarrier arrive:
// the consumer warps never meet per stage and carry no pipeline state - everything a
// stage needs to know (tile, chunk, whether it opens or closes an accumulation) comes in
// a small descriptor the producer writes beside it.  The groups of a block share nothing
// but the producer warp, so one group's epilogue overlaps the others' products.
// The producer lanes never block: they stay together and poll their groups' slots in turn,
// so no lane's wait holds up the lanes of the other groups.
// Every wait is bounded; a wait that gives up records BIVMOE_ERR_TIMEOUT (and which wait
// it was) in the status words and raises a block-wide flag on which every role leaves its
// loop (the producer first waits, bounded again, for its copies still in flight).
template <int TY>
__host__ __device__ constexpr int act_stage_bytes() {
    return Fmt<TY>::F32ACT ? EX_TT * Fmt<TY>::ELEMS * 4 : kActCopyBytes;
}
template <int TY>
__host__ __device__ constexpr int stage_bytes() {
    return kChunkRows * Fmt<TY>::SL + act_stage_bytes<TY>();
}
constexpr int EX_SLOTS = 2;               // ring slots per group
constexpr int EX_HEAD = 1024;             // barriers, abort flag, stage descriptors
constexpr int EX_SMEM_MAX = 227 * 1024;
template <int TY>
__host__ __device__ constexpr int smem_bytes() {
    constexpr int G = Fmt<TY>::MINB;
    return EX_HEAD + G * EX_TT * 64 * 4 + G * EX_SLOTS * stage_bytes<TY>();
}

struct StageDesc {      // what the producer tells a group about a stage
    int pos0, tc;       // the tile: first position, tokens
    int chunk, slice;   // the weights: chunk of the expert's matrix, K-slice
    int expert;         // expert id (n_expert: the shared expert)
    int rows;           // rows of the expert's matrix (down: the stride of the output rows)
    int flags;          // SD_*
    int pad;
};
enum { SD_FIRST = 1, SD_LAST = 2, SD_END = 4 };
// which bounded wait gave up (status word 2, for the error text)
enum { SITE_PRODUCER_SLOT = 1, SITE_CONSUMER_STAGE = 2, SITE_END_MARKER = 3 };

struct Item {           // a decoded work item: a token tile x a run of chunks
    int shared;         // the shared expert's group
    int expert;
    int chunk0;         // first chunk
    int nch;            // chunks of the item present in this matrix
    int nsl;            // K-slices per chunk
    int pos0;           // first position of the tile
    int tc;             // tokens in the tile
    int rows;
    const uint8_t* src; // K-slice 0 of chunk0; slice s of chunk chunk0 + j is (j * nsl + s) * 128 * SL further
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void group_sync(int grp) {   // the 128 threads of one consumer group
    asm volatile("bar.sync %0, 128;" ::"r"(grp + 1) : "memory");
}
template <int TY, int MODE>
__global__ void __launch_bounds__(32 * (4 * Fmt<TY>::MINB + 1), 1)
experts_kernel(const ExpertArgs A) {
    using F = Fmt<TY>;
    using Side = typename F::Side;
    constexpr int G = F::MINB;
    constexpr int SB = stage_bytes<TY>();
    constexpr uint32_t W_BYTES = kChunkRows * F::SL, ACT_BYTES = act_stage_bytes<TY>();
    constexpr int CH = MODE == MODE_GATEUP ? 64 : 128;   // output rows per chunk
    pdl_launch_dependents();
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;                 // [G][2] a stage has landed
    uint64_t* empty = full + G * EX_SLOTS;            // [G][2] its four warps are done with it
    int* s_abort = (int*)(smem + 256);
    int* s_next = (int*)(smem + 260);                 // the block's next unclaimed item (index in its list)
    StageDesc* s_desc = (StageDesc*)(smem + 512);     // [G][2]
    float* s_mid_all = (float*)(smem + EX_HEAD);      // [G][EX_TT][64] SwiGLU staging
    uint8_t* ring = (uint8_t*)(s_mid_all + G * EX_TT * 64);   // [G][2][SB]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t hint = A.wait_hint_ns;

    if (tid == 0) {
        for (int i = 0; i < G * EX_SLOTS; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 4);
        }
        *s_abort = 0;
        *s_next = G;   // the first G items of the list are the groups' first items
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();   // the tile lists and the activation records are the previous kernels'

    // bounded wait that also gives up when another role has
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < EX_WAIT_LIMIT; i++) {
            if (mbar_try_wait(bar, parity, hint)) return true;
            if ((i & 31) == 31 && *(volatile int*)s_abort) return false;
        }
        return false;
    };
    auto give_up = [&](int site) {
        if (atomicExch(A.status, BIVMOE_ERR_TIMEOUT) == 0) atomicExch(A.status + 2, site);
        atomicExch(s_abort, 1);
    };

    if (warp == 4 * G) {
        // ------------------------------------------------------------ producer warp
        // lane g feeds group g
        if (lane >= G) return;
        const int tiles_all = A.n_tiles[0], tiles_sh = A.n_tiles[1];
        const int tile_lo = A.tiles_mode == 1 ? tiles_sh : 0;
        const int tile_hi = A.tiles_mode == 2 ? tiles_sh : tiles_all;
        // an item is a tile times one chunk: 8 stages (gate+up), 2 stages (down) at the qwen35moe shapes
        const int units = (tile_hi - tile_lo) * A.chunks;
        // The lanes stay together: every turn of the loop each lane looks once (without
        // blocking) whether its group has a free slot and, if so, issues its next stage, so
        // no group waits for another lane's wait to end.  A turn without progress in any
        // lane sleeps 64 ns; 2^20 such turns in a row (about 70 ms) end the kernel.
        constexpr uint32_t LANES = (1u << G) - 1u;
        uint32_t issued = 0;      // stages this lane has given its group
        Item it;
        it.nsl = 0;
        int slice = 0, s1 = 0;    // next K-slice of the lane's item, and its end
        int first = 1, ending = 0, done = 0;
        uint32_t idle = 0;
        while (true) {
            int progressed = 0;
            if (!done && !ending && slice >= s1) {
                // the block's list: items blockIdx.x, blockIdx.x + gridDim.x, ...; group g
                // starts with entry g, later entries go to whichever group is ready first
                const int entry = first ? lane : atomicAdd(s_next, 1);
                first = 0;
                const int idx = (int)blockIdx.x + entry * (int)gridDim.x;
                if (idx >= units) {
                    ending = 1;
                } else {
                    const int tile = tile_lo + idx / A.chunks;
                    it.chunk0 = idx % A.chunks;
                    const int4 td = A.tile_desc[tile];
                    it.expert = td.x;
                    it.shared = it.expert == A.n_expert;
                    it.pos0 = td.y;
                    it.tc = td.z;
                    const DevTiles& m = it.shared ? A.sh : A.w;
                    it.nsl = m.nslices;
                    it.nch = it.chunk0 < m.chunks ? 1 : 0;
                    it.rows = m.rows;
                    it.src = m.stage(it.shared ? 0 : it.expert, min(it.chunk0, max(m.chunks - 1, 0)), 0);
                    slice = 0;
                    s1 = it.nch ? it.nsl : 0;
                }
                progressed = 1;
            }
            if (!done && (ending || slice < s1)) {
                const int bi = lane * EX_SLOTS + (int)(issued & 1);
                if (mbar_test_wait(&empty[bi], ((issued >> 1) & 1) ^ 1)) {
                    if (ending) {   // the end marker: a stage without data
                        StageDesc d{};
                        d.flags = SD_END;
                        s_desc[bi] = d;
                        mbar_arrive(&full[bi]);
                        done = 1;
                    } else {
                        StageDesc d;
                        d.pos0 = it.pos0; d.tc = it.tc; d.chunk = it.chunk0; d.slice = slice;
                        d.expert = it.shared ? A.n_expert : it.expert; d.rows = it.rows;
                        d.flags = (slice == 0 ? SD_FIRST : 0) | (slice == s1 - 1 ? SD_LAST : 0);
                        d.pad = 0;
                        s_desc[bi] = d;
                        uint8_t* dst = ring + (size_t)bi * SB;
                        fence_proxy_async();   // the slot was last read through the generic proxy
                        mbar_expect_tx(&full[bi], W_BYTES + ACT_BYTES);
                        bulk_g2s(dst, it.src + (size_t)slice * W_BYTES, W_BYTES, &full[bi]);
                        uint8_t* adst = dst + W_BYTES;
                        if (F::F32ACT) {
                            const size_t row = (size_t)slice * A.act_rows + it.pos0;
                            bulk_g2s(adst, A.x_f32 + row * F::ELEMS, EX_TT * F::ELEMS * 4, &full[bi]);
                        } else {   // the tile's Q8 record of this K-slice (pos0 is a multiple of 8)
                            bulk_g2s(adst, A.x_t + ((size_t)slice * (A.act_rows / 8) + it.pos0 / 8) * kActTileBytes,
                                     kActCopyBytes, &full[bi]);
                        }
                        issued++;
                        slice++;
                    }
                    progressed = 1;
                }
            }
            if (__all_sync(LANES, done)) break;
            if (*(volatile int*)s_abort) break;
            if (__any_sync(LANES, progressed)) {
                idle = 0;
            } else if (++idle > (1u << 20)) {
                if (lane == 0) give_up(SITE_PRODUCER_SLOT);
                break;
            } else {
                __nanosleep(64);
            }
        }
        if (!done) {   // leave no copy in flight behind: the last two stages this lane issued
            for (uint32_t q = issued > 2 ? issued - 2 : 0; q < issued; q++)
                mbar_wait_bounded(&full[lane * EX_SLOTS + (q & 1)], (q >> 1) & 1, hint);
        }
        return;
    }

    // ---------------------------------------------------------------- consumer groups
    const int grp = warp >> 2, wig = warp & 3;
    const int g = lane >> 2, c = lane & 3;
    const uint32_t ring_a = smem_u32(ring);
    float* s_mid = s_mid_all + grp * EX_TT * 64;
    // the first chunk row of this warp's two 16-row MMA tiles
    int row_of[2];
    if (MODE == MODE_GATEUP) {   // warp w: gate rows 16w..16w+15 and the same up rows (64 further)
        row_of[0] = 16 * wig;
        row_of[1] = 64 + 16 * wig;
    } else {                     // warp w: down rows 32w..32w+31
        row_of[0] = 32 * wig;
        row_of[1] = 32 * wig + 16;
    }
    float acc[8];   // MMA path: [mt][i] = acc[4 * mt + i], i = 2 * r + tt: row g + 8r, token 2c + tt;
                    // float path: token t of this lane's row
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.0f;
    for (uint32_t q = 0;; q++) {
        const int bi = grp * EX_SLOTS + (int)(q & 1);
        if (!wait(&full[bi], (q >> 1) & 1)) {
            give_up(SITE_CONSUMER_STAGE);
            return;
        }
        const StageDesc d = s_desc[bi];
        if (d.flags & SD_END) return;
        if (d.flags & SD_FIRST) {
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] = 0.0f;
        }
        const bool shared = d.expert == A.n_expert;
        const uint32_t sta = ring_a + (uint32_t)bi * SB;
        if constexpr (F::F32ACT) {
            // a lane per weight row: GATEUP lanes 0-15 gate rows, 16-31 up rows
            const uint8_t* st = ring + (size_t)bi * SB;
            const uint8_t* wrow;
            if (MODE == MODE_GATEUP) wrow = st + (row_of[lane >> 4] + (lane & 15)) * 16;
            else wrow = st + (32 * wig + lane) * 16;
            F::compute_f32(wrow, (const float*)(st + W_BYTES), d.tc, acc);
        } else {
            Side side{};
            if constexpr (TY == BIVMOE_Q6_K) {
                const DevTiles& m = shared ? A.sh : A.w;
                const size_t base = ((size_t)(shared ? 0 : d.expert) * m.chunks + d.chunk) * kChunkRows;
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int r = 0; r < 2; r++)
                        side.d[mt][r] = __half2float(__ushort_as_half(
                            m.side[(base + row_of[mt] + g + 8 * r) * m.nslices + d.slice]));
            }
            uint32_t rowp[2][2];
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int r = 0; r < 2; r++) rowp[mt][r] = sta + (row_of[mt] + g + 8 * r) * 16;
            F::compute(rowp, side, sta + W_BYTES, *(float(*)[2][4])acc, g, c);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[bi]);   // this warp is done with the slot
        if (!(d.flags & SD_LAST)) continue;

        // ---- the chunk is complete
        if (MODE == MODE_GATEUP) {
            // SwiGLU into the staging tile [token][64 rows of the chunk]
            if constexpr (F::F32ACT) {
#pragma unroll
                for (int t = 0; t < EX_TT; t++) {
                    const float u = __shfl_down_sync(0xffffffffu, acc[t], 16);
                    if (lane < 16) {
                        const float gt = acc[t];
                        s_mid[t * 64 + 16 * wig + lane] = (gt * __fdiv_rn(1.0f, 1.0f + expf(-gt))) * u;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // ops.rs:160-167: silu(x) = x * (1 / (1 + exp(-x)))
                    const float gt = acc[i], u = acc[4 + i];
                    s_mid[(2 * c + (i & 1)) * 64 + 16 * wig + g + 8 * (i >> 1)] =
                        (gt * __fdiv_rn(1.0f, 1.0f + expf(-gt))) * u;
                }
            }
            group_sync(grp);
            // rows of mid: f32 (slice-major by 64) and, for quantised down types, the
            // Q8Act of each 32-row block (quant.rs:368-394); one warp per (token, block)
            for (int p = wig; p < 2 * d.tc; p += 4) {
                const int t = p >> 1, blk = p & 1;
                const float v = s_mid[t * 64 + 32 * blk + lane];
                const int r = d.chunk * CH + 32 * blk + lane;
                const size_t pos = d.pos0 + t;
                A.out[((size_t)(r / 64) * A.act_rows + pos) * 64 + r % 64] = v;
                if (A.out_t) {
                    float dd, ss;
                    const int qv = q8_quantize_lane(v, dd, ss);
                    uint8_t* rec = A.out_t + ((size_t)(r / 256) * (A.act_rows / 8) + pos / 8) * kActTileBytes;
                    rec[act_q_off((int)(pos % 8), r % 256)] = (uint8_t)(int8_t)qv;
                    if (lane < 4) {
                        float shi, slo;
                        split_tf32(ss, &shi, &slo);
                        const float val = lane == 0 ? dd : lane == 1 ? shi : lane == 2 ? slo : ss;
                        *(float*)(rec + kActOffDx + 256 * lane + (((r % 256) / 32) * 8 + pos % 8) * 4) = val;
                    }
                }
            }
            group_sync(grp);   // the staging tile is free for the group's next chunk
        } else {
            if constexpr (F::F32ACT) {
#pragma unroll
                for (int t = 0; t < EX_TT; t++)
                    if (t < d.tc)
                        A.out[(size_t)(d.pos0 + t) * d.rows + d.chunk * CH + 32 * wig + lane] = acc[t];
            } else {
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int t = 2 * c + (i & 1);
                        if (t < d.tc)
                            A.out[(size_t)(d.pos0 + t) * d.rows + d.chunk * CH + 32 * wig + 16 * mt + g +
                                  8 * (i >> 1)] = acc[4 * mt + i];
                    }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// host side

bool experts_supported(int ty, int cols, int rows, bool is_down) {
    // every type the reference has a dot kernel for (quant.rs:80-93)
    if (ty != BIVMOE_Q8_0 && ty != BIVMOE_Q4_K && ty != BIVMOE_Q5_K && ty != BIVMOE_Q6_K &&
        ty != BIVMOE_BF16 && ty != BIVMOE_F16 && ty != BIVMOE_F32 && ty != BIVMOE_Q4_0 &&
        ty != BIVMOE_Q4_1)
        return false;
    return cols > 0 && cols % 256 == 0 && rows > 0 && rows % (is_down ? 128 : 64) == 0;
}

template <int TY, int MODE>
static cudaError_t launch_one(const LaunchCfg& c, ExpertArgs A) {
    A.chunks = std::max(A.w.chunks, A.sh.chunks);
    constexpr int smem = smem_bytes<TY>();
    static_assert(smem <= EX_SMEM_MAX, "the block must fit in shared memory");
    static std::atomic<uint64_t> attr_set{0};
    if (cudaError_t e = ensure_dynamic_smem(experts_kernel<TY, MODE>, smem, attr_set)) return e;
    constexpr int threads = 32 * (4 * Fmt<TY>::MINB + 1);
    cudaError_t e = launch_after(c.stream, experts_kernel<TY, MODE>, dim3(c.sm_count), dim3(threads), smem, A);
    count_launch();
    return e;
}

template <int MODE>
static cudaError_t launch_typed(int ty, const LaunchCfg& c, const ExpertArgs& A) {
    switch (ty) {
        case BIVMOE_Q8_0: return launch_one<BIVMOE_Q8_0, MODE>(c, A);
        case BIVMOE_Q4_K: return launch_one<BIVMOE_Q4_K, MODE>(c, A);
        case BIVMOE_Q5_K: return launch_one<BIVMOE_Q5_K, MODE>(c, A);
        case BIVMOE_Q6_K: return launch_one<BIVMOE_Q6_K, MODE>(c, A);
        case BIVMOE_BF16: return launch_one<BIVMOE_BF16, MODE>(c, A);
        case BIVMOE_F16: return launch_one<BIVMOE_F16, MODE>(c, A);
        case BIVMOE_F32: return launch_one<BIVMOE_F32, MODE>(c, A);
        case BIVMOE_Q4_0: return launch_one<BIVMOE_Q4_0, MODE>(c, A);
        case BIVMOE_Q4_1: return launch_one<BIVMOE_Q4_1, MODE>(c, A);
        default: return cudaErrorInvalidValue;
    }
}

// gate+up then down, for the routed experts and the shared expert.  When the
// shared expert's matrices have the routed experts' types it rides in the same
// launches (its tiles come first in the tile list); otherwise it gets its own.
cudaError_t launch_experts(const LaunchCfg& c, const DevTiles& gate_up, const DevTiles& down,
                           const DevTiles& sh_gate_up, const DevTiles& sh_down, const Workspace& ws) {
    ExpertArgs A{};
    A.grp_expert = ws.grp_expert; A.grp_start = ws.grp_start; A.grp_count = ws.grp_count;
    A.tile_desc = ws.tile_desc; A.n_tiles = ws.n_tiles;
    A.status = ws.status;
    A.n = c.n; A.k = c.k; A.n_expert = c.n_expert;
    A.act_rows = ws.act_rows;
    {
        // read once; the initialisation of a function-local static is safe between host threads
        static const int hint = [] { const char* e = getenv("BIVMOE_WAIT_HINT"); return e ? atoi(e) : 1000; }();
        A.wait_hint_ns = (uint32_t)hint;
    }
    const bool fused = c.has_shared && sh_gate_up.ty == gate_up.ty && sh_down.ty == down.ty;
    cudaError_t err;
    // ---- gate + up (SwiGLU and the Q8 rows of its output in the epilogue)
    auto gateup = [&](int mode, int ctr, int ty, int down_ty) {
        ExpertArgs G = A;
        G.w = gate_up; G.sh = sh_gate_up;
        if (mode == 1) G.sh = DevTiles{};
        if (mode == 2) G.w = DevTiles{};
        G.x_f32 = ws.act_f; G.x_t = ws.act_t;
        G.out = ws.mid;
        G.out_t = type_uses_f32_act(down_ty) ? nullptr : ws.mid_t;
        G.work_ctr = ws.work_ctr + ctr;
        G.tiles_mode = mode;
        return launch_typed<MODE_GATEUP>(ty, c, G);
    };
    if (c.only_shared) {
        err = gateup(2, 1, sh_gate_up.ty, sh_down.ty);
    } else if (fused || !c.has_shared) {
        err = gateup(0, 0, gate_up.ty, down.ty);
    } else {
        err = gateup(1, 0, gate_up.ty, down.ty);
        if (err == cudaSuccess) err = gateup(2, 1, sh_gate_up.ty, sh_down.ty);
    }
    if (err != cudaSuccess) return err;
    mark(c, EV_GATEUP);
    // ---- down
    auto downp = [&](int mode, int ctr, int ty) {
        ExpertArgs D = A;
        D.w = down; D.sh = sh_down;
        if (mode == 1) D.sh = DevTiles{};
        if (mode == 2) D.w = DevTiles{};
        D.x_f32 = ws.mid; D.x_t = ws.mid_t;
        D.out = ws.pair_out;
        D.work_ctr = ws.work_ctr + ctr;
        D.tiles_mode = mode;
        return launch_typed<MODE_DOWN>(ty, c, D);
    };
    if (c.only_shared) {
        err = downp(2, 3, sh_down.ty);
    } else if (fused || !c.has_shared) {
        err = downp(0, 2, down.ty);
    } else {
        err = downp(1, 2, down.ty);
        if (err == cudaSuccess) err = downp(2, 3, sh_down.ty);
    }
    return err;
}

}  // namespace bivmoe
