// Grouped expert products for decode-sized groups: gate+up with the SwiGLU and
// the Q8 re-quantisation of its output fused, then down.
// Reference: dense_ffn (engine/src/model.rs:1119-1126) over matmul
// (engine/src/ops.rs:84-127) and the per-type dots (engine/src/quant.rs:
// 599-686 scalar, 1369-1533 AVX2), for each expert's token list
// (model.rs:875-889) and for the shared expert (model.rs:890-896).
//
// Design.  The kernel is a grid of independent warps, one block per SM.  A
// warp pulls work items (tile of <= 8 tokens of one group, chunk of weight
// rows) from a counter and streams the chunk's rows from HBM through its own
// two-slot ring in shared memory: per stage one K-slice of 64 rows (two 32-row
// tiles, each contiguous in the device layout of common.cuh) and the matching
// K-slice of the tile's 8 activation rows arrive by four bulk copies
// (cp.async.bulk) on the warp's own mbarrier, so warps never synchronise with
// each other and the copies of one stage overlap the arithmetic of the other,
// across item boundaries too.  A lane owns two weight rows (gate row r and up
// row r; or down rows r and r+32) and reads the activations as warp-wide
// broadcasts, so each weight word is unpacked once and meets every token from
// registers, and both rows share one activation load.  Each lane forms whole
// 32-element block dots with __dp4a (the reference's int32 values) and applies
// the block scales in f32.  No atomics on data: results are run-to-run identical.
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "formats.cuh"

namespace bivmoe {

constexpr int EX_TT = 8;                       // tokens per tile
constexpr int EX_ROWS = 64;                    // weight rows per stage (two per lane)
constexpr uint32_t EX_WAIT_LIMIT = 1u << 20;   // bounded mbarrier spin

enum { MODE_GATEUP = 0, MODE_DOWN = 1 };

struct ExpertArgs {
    DevStack w0, w1;       // routed stacks: gate, up (MODE_GATEUP) or down, - (MODE_DOWN)
    DevStack s0, s1;       // the shared expert's
    // activations by position, slice-major (common.cuh): rows of h for GATEUP, of mid for DOWN
    const float* x_f32;    // float-activation types
    const int8_t* x_q;     // quantised types
    const float2* x_ds;
    int act_rows;          // R
    float* out;            // GATEUP: mid f32, slice-major; DOWN: pair_out [P+n][rows]
    int8_t* out_q;         // GATEUP with a quantised down type: Q8 rows of mid, slice-major
    float2* out_ds;
    const int32_t* grp_expert;
    const int32_t* grp_start;
    const int32_t* grp_count;
    const int32_t* tile_group;
    const int32_t* tile_t0;
    const int32_t* n_tiles;   // [0] all tiles, [1] tiles of the shared group (they come first)
    uint32_t* work_ctr;
    int32_t* status;
    int n, k, n_expert;
    int tiles_mode;        // 0: every tile, 1: skip the shared group's, 2: only the shared group's
    int chunks;            // row chunks per group
};

// ---------------------------------------------------------------------------
// PTX helpers: mbarrier + bulk copy (TMA, untiled form)
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
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for a phase with an iteration limit; false when it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < EX_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
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

// ---------------------------------------------------------------------------
// Per-type arithmetic of one staged K-slice.  `wa` / `wb` point at this lane's
// row inside the two staged tiles (tile + lane*16); unit u of the row is 512*u
// further (unit-major tiles), so byte `off` of the row's slice is WU(w, off).
//   ELEMS   columns per stage,  SL  bytes per row per stage
//   WARPS   warps per block that fit two stages each in 227 KB
//   Side    per-row words kept outside the tiles (Q6_K's f16 d), fetched with a
//           plain load when the stage is issued
#define WU(w, off) ((w) + ((((off)) >> 4) << 9) + ((off) & 15))
#define LO4(v) ((int)((v) & 0x0F0F0F0Fu))
#define HI4(v) ((int)(((v) >> 4) & 0x0F0F0F0Fu))

__device__ __forceinline__ int dot8(const int (&w)[8], const int4& a0, const int4& a1) {
    int s = dp4a_s8(w[0], a0.x, 0);
    s = dp4a_s8(w[1], a0.y, s);
    s = dp4a_s8(w[2], a0.z, s);
    s = dp4a_s8(w[3], a0.w, s);
    s = dp4a_s8(w[4], a1.x, s);
    s = dp4a_s8(w[5], a1.y, s);
    s = dp4a_s8(w[6], a1.z, s);
    s = dp4a_s8(w[7], a1.w, s);
    return s;
}
// the 32 bytes at offset `off` (a multiple of 16) of this lane's row slice
__device__ __forceinline__ void load8(const uint8_t* w, int off, uint32_t (&v)[8]) {
    const uint4 a = *(const uint4*)WU(w, off), b = *(const uint4*)WU(w, off + 16);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

struct NoSide {};

template <int TY> struct Fmt;

// ---- Q8_0 (quant.rs:599-607): term = d_w * d_x * sum(q_w * q_x) ------------
template <> struct Fmt<BIVMOE_Q8_0> {
    static constexpr int ELEMS = 256, SL = 272, WARPS = 5;
    static constexpr bool F32ACT = false;
    using Side = NoSide;
    __device__ static Side side(const uint16_t*, int) { return {}; }
    __device__ static void accum2(const uint8_t* wa, const uint8_t* wb, Side, Side,
                                  const int8_t* xq, const float2* xds, int cnt,
                                  float (&accA)[EX_TT], float (&accB)[EX_TT]) {
#pragma unroll 2
        for (int b = 0; b < 8; b++) {
            uint32_t ua[8], ub[8];
            load8(wa, 32 * b, ua);
            load8(wb, 32 * b, ub);
            int qa[8], qb[8];
#pragma unroll
            for (int i = 0; i < 8; i++) { qa[i] = (int)ua[i]; qb[i] = (int)ub[i]; }
            const float da = __half2float(*(const __half*)WU(wa, 256 + 2 * b));
            const float db = __half2float(*(const __half*)WU(wb, 256 + 2 * b));
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cnt) {
                    const int4* ap = (const int4*)(xq + t * ELEMS + 32 * b);
                    const int4 a0 = ap[0], a1 = ap[1];
                    const float dx = xds[t * (ELEMS / 32) + b].x;
                    accA[t] += (da * dx) * (float)dot8(qa, a0, a1);
                    accB[t] += (db * dx) * (float)dot8(qb, a0, a1);
                }
            }
        }
    }
};

// ---- Q4_K / Q5_K (quant.rs:609-649): per sub-block
//      d*sc*d_x*sum(q*q_x) - dmin*m*s_x ; Q5_K adds bit sb of qh[l] as value bit 4
template <int TY> struct FmtK45 {
    static constexpr int QOFF = TY == BIVMOE_Q4_K ? 16 : 48;
    static constexpr int ELEMS = 256, SL = TY == BIVMOE_Q4_K ? 144 : 176, WARPS = 8;
    static constexpr bool F32ACT = false;
    using Side = NoSide;
    __device__ static Side side(const uint16_t*, int) { return {}; }
    struct Hdr { float d, dmin; K4Scales sc; uint32_t qh[8]; };
    __device__ static Hdr header(const uint8_t* w) {
        Hdr h;
        const uint4 v = *(const uint4*)w;
        const __half2 dd = *(const __half2*)&v.x;
        h.d = __low2float(dd);
        h.dmin = __high2float(dd);
        h.sc = unpack_k4_scales(v.y, v.z, v.w);
        if (TY == BIVMOE_Q5_K) load8(w, 16, h.qh);
        return h;
    }
    __device__ static void unpack(const uint8_t* w, const Hdr& h, int j, int (&lo)[8], int (&hi)[8]) {
        uint32_t qv[8];
        load8(w, QOFF + 32 * j, qv);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            lo[i] = LO4(qv[i]);
            hi[i] = HI4(qv[i]);
            if (TY == BIVMOE_Q5_K) {
                lo[i] |= (int)(((h.qh[i] >> (2 * j)) & 0x01010101u) << 4);
                hi[i] |= (int)(((h.qh[i] >> (2 * j + 1)) & 0x01010101u) << 4);
            }
        }
    }
    __device__ static void accum2(const uint8_t* wa, const uint8_t* wb, Side, Side,
                                  const int8_t* xq, const float2* xds, int cnt,
                                  float (&accA)[EX_TT], float (&accB)[EX_TT]) {
        const Hdr ha = header(wa), hb = header(wb);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int alo[8], ahi[8], blo[8], bhi[8];
            unpack(wa, ha, j, alo, ahi);
            unpack(wb, hb, j, blo, bhi);
            const float a_s0 = ha.d * (float)k4_scale(ha.sc, 2 * j);
            const float a_m0 = ha.dmin * (float)k4_min(ha.sc, 2 * j);
            const float a_s1 = ha.d * (float)k4_scale(ha.sc, 2 * j + 1);
            const float a_m1 = ha.dmin * (float)k4_min(ha.sc, 2 * j + 1);
            const float b_s0 = hb.d * (float)k4_scale(hb.sc, 2 * j);
            const float b_m0 = hb.dmin * (float)k4_min(hb.sc, 2 * j);
            const float b_s1 = hb.d * (float)k4_scale(hb.sc, 2 * j + 1);
            const float b_m1 = hb.dmin * (float)k4_min(hb.sc, 2 * j + 1);
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cnt) {
                    const int4* ap = (const int4*)(xq + t * ELEMS + 64 * j);
                    const int4 x0 = ap[0], x1 = ap[1], x2 = ap[2], x3 = ap[3];
                    const float4 dx = *(const float4*)(xds + t * (ELEMS / 32) + 2 * j);  // d0 s0 d1 s1
                    accA[t] += (a_s0 * dx.x) * (float)dot8(alo, x0, x1) - a_m0 * dx.y;
                    accA[t] += (a_s1 * dx.z) * (float)dot8(ahi, x2, x3) - a_m1 * dx.w;
                    accB[t] += (b_s0 * dx.x) * (float)dot8(blo, x0, x1) - b_m0 * dx.y;
                    accB[t] += (b_s1 * dx.z) * (float)dot8(bhi, x2, x3) - b_m1 * dx.w;
                }
            }
        }
    }
};
template <> struct Fmt<BIVMOE_Q4_K> : FmtK45<BIVMOE_Q4_K> {};
template <> struct Fmt<BIVMOE_Q5_K> : FmtK45<BIVMOE_Q5_K> {};

// ---- Q6_K (quant.rs:651-686), slice = ql[128] qh[64] scales[16], d aside: per
//      32-block d * d_x * (sc[2g]*sum16 + sc[2g+1]*sum16), 6-bit values minus 32
template <> struct Fmt<BIVMOE_Q6_K> {
    static constexpr int ELEMS = 256, SL = 208, WARPS = 7;
    static constexpr bool F32ACT = false;
    struct Side { float d; };     // the super-block's f16 scale
    __device__ static Side side(const uint16_t* row_side, int s) {
        return {__half2float(__ushort_as_half(row_side[s]))};
    }
    __device__ static void unpack(const uint32_t (&l0)[8], const uint32_t (&l1)[8],
                                  const uint32_t (&hh)[8], int kq, int (&q)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t base = (kq & 1) ? l1[i] : l0[i];
            const uint32_t nib = (kq >= 2 ? base >> 4 : base) & 0x0F0F0F0Fu;
            const uint32_t hb = ((hh[i] >> (2 * kq)) & 0x03030303u) << 4;
            q[i] = (int)__vsub4(nib | hb, 0x20202020u);
        }
    }
    __device__ static int isum(const int (&q)[8], const int4& a0, const int4& a1, uint32_t sw, int kq) {
        const int sca = (int)(int8_t)((sw >> (16 * (kq & 1))) & 0xFF);
        const int scb = (int)(int8_t)((sw >> (16 * (kq & 1) + 8)) & 0xFF);
        int ia = dp4a_s8(q[0], a0.x, 0);
        ia = dp4a_s8(q[1], a0.y, ia);
        ia = dp4a_s8(q[2], a0.z, ia);
        ia = dp4a_s8(q[3], a0.w, ia);
        int ib = dp4a_s8(q[4], a1.x, 0);
        ib = dp4a_s8(q[5], a1.y, ib);
        ib = dp4a_s8(q[6], a1.z, ib);
        ib = dp4a_s8(q[7], a1.w, ib);
        return sca * ia + scb * ib;
    }
    __device__ static void accum2(const uint8_t* wa, const uint8_t* wb, Side sa, Side sb,
                                  const int8_t* xq, const float2* xds, int cnt,
                                  float (&accA)[EX_TT], float (&accB)[EX_TT]) {
#pragma unroll
        for (int n = 0; n < 2; n++) {
            uint32_t al0[8], al1[8], ah[8], bl0[8], bl1[8], bh[8];
            load8(wa, 64 * n, al0); load8(wa, 64 * n + 32, al1); load8(wa, 128 + 32 * n, ah);
            load8(wb, 64 * n, bl0); load8(wb, 64 * n + 32, bl1); load8(wb, 128 + 32 * n, bh);
            const uint2 asc = *(const uint2*)WU(wa, 192 + 8 * n), bsc = *(const uint2*)WU(wb, 192 + 8 * n);
#pragma unroll
            for (int kq = 0; kq < 4; kq++) {
                int qa[8], qb[8];
                unpack(al0, al1, ah, kq, qa);
                unpack(bl0, bl1, bh, kq, qb);
                const uint32_t aw = kq < 2 ? asc.x : asc.y, bw = kq < 2 ? bsc.x : bsc.y;
                const int xb = 4 * n + kq;
#pragma unroll
                for (int t = 0; t < EX_TT; t++) {
                    if (t < cnt) {
                        const int4* ap = (const int4*)(xq + t * ELEMS + 32 * xb);
                        const int4 a0 = ap[0], a1 = ap[1];
                        const float dx = xds[t * (ELEMS / 32) + xb].x;
                        accA[t] += (sa.d * dx) * (float)isum(qa, a0, a1, aw, kq);
                        accB[t] += (sb.d * dx) * (float)isum(qb, a0, a1, bw, kq);
                    }
                }
            }
        }
    }
};

// ---- BF16 weights meet f32 activations (quant.rs:509-521, 1229-1256) -------
template <> struct Fmt<BIVMOE_BF16> {
    static constexpr int ELEMS = 64, SL = 128, WARPS = 8;
    static constexpr bool F32ACT = true;
    using Side = NoSide;
    __device__ static Side side(const uint16_t*, int) { return {}; }
    __device__ static void widen(const uint4& v, float (&w)[8]) {
        w[0] = __uint_as_float(v.x << 16); w[1] = __uint_as_float(v.x & 0xFFFF0000u);
        w[2] = __uint_as_float(v.y << 16); w[3] = __uint_as_float(v.y & 0xFFFF0000u);
        w[4] = __uint_as_float(v.z << 16); w[5] = __uint_as_float(v.z & 0xFFFF0000u);
        w[6] = __uint_as_float(v.w << 16); w[7] = __uint_as_float(v.w & 0xFFFF0000u);
    }
    __device__ static float fma8(const float (&w)[8], const float4& x0, const float4& x1, float s) {
        s = fmaf(w[0], x0.x, s); s = fmaf(w[1], x0.y, s); s = fmaf(w[2], x0.z, s);
        s = fmaf(w[3], x0.w, s); s = fmaf(w[4], x1.x, s); s = fmaf(w[5], x1.y, s);
        s = fmaf(w[6], x1.z, s); s = fmaf(w[7], x1.w, s);
        return s;
    }
    __device__ static void accum2f(const uint8_t* wa, const uint8_t* wb, const float* xf, int cnt,
                                   float (&accA)[EX_TT], float (&accB)[EX_TT]) {
#pragma unroll 2
        for (int u = 0; u < 8; u++) {
            float fa[8], fb[8];
            widen(*(const uint4*)(wa + 512 * u), fa);
            widen(*(const uint4*)(wb + 512 * u), fb);
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cnt) {
                    const float4* xp = (const float4*)(xf + t * ELEMS + 8 * u);
                    const float4 x0 = xp[0], x1 = xp[1];
                    accA[t] = fma8(fa, x0, x1, accA[t]);
                    accB[t] = fma8(fb, x0, x1, accB[t]);
                }
            }
        }
    }
};

// ---------------------------------------------------------------------------
template <int TY>
__host__ __device__ constexpr int act_stage_bytes() {
    return Fmt<TY>::F32ACT ? EX_TT * Fmt<TY>::ELEMS * 4
                           : EX_TT * Fmt<TY>::ELEMS + EX_TT * (Fmt<TY>::ELEMS / 32) * 8;
}
template <int TY>
__host__ __device__ constexpr int stage_bytes() {
    return EX_ROWS * Fmt<TY>::SL + act_stage_bytes<TY>();
}
template <int TY>
__host__ __device__ constexpr int smem_bytes() {
    return 128 + Fmt<TY>::WARPS * 2 * stage_bytes<TY>();
}

struct Item {           // a decoded work item (warp-uniform except sa, sb)
    int valid;
    int shared;         // the shared expert's group
    int expert;
    int pos0;           // first position of the tile
    int tc;             // tokens in the tile
    int r0;             // first output row of the chunk
    int nst;            // stages: slices of the inner dimension
    const uint8_t* ta;  // slice 0 of the two 32-row weight tiles; slice s is s*32*SL further
    const uint8_t* tb;
    const uint16_t* sa; // this lane's rows in the side plane (Q6_K)
    const uint16_t* sb;
};

template <int TY, int MODE>
__global__ void __launch_bounds__(Fmt<TY>::WARPS * 32, 1)
experts_kernel(const ExpertArgs A) {
    using F = Fmt<TY>;
    using Side = typename F::Side;
    constexpr int SB = stage_bytes<TY>();
    constexpr int CH = MODE == MODE_GATEUP ? 32 : 64;   // output rows per chunk
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t* mbar = (uint64_t*)smem + 2 * warp;                 // this warp's two barriers
    uint8_t* ring = smem + 128 + (size_t)warp * 2 * SB;
    const int P = A.n * A.k;

    if (lane == 0) {
        mbar_init(&mbar[0], 1);
        mbar_init(&mbar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const int tiles_all = A.n_tiles[0], tiles_sh = A.n_tiles[1];
    const int tile_lo = A.tiles_mode == 1 ? tiles_sh : 0;
    const int tile_hi = A.tiles_mode == 2 ? tiles_sh : tiles_all;
    const int total = (tile_hi - tile_lo) * A.chunks;

    // pulls the next item off the counter and decodes it
    auto fetch = [&]() -> Item {
        Item it;
        int idx = 0;
        if (lane == 0) idx = (int)atomicAdd(A.work_ctr, 1u);
        idx = __shfl_sync(0xffffffffu, idx, 0);
        it.valid = idx < total;
        if (!it.valid) return it;
        const int tile = tile_lo + idx / A.chunks, chunk = idx % A.chunks;
        const int g = A.tile_group[tile], t0 = A.tile_t0[tile];
        it.expert = A.grp_expert[g];
        it.shared = it.expert == A.n_expert;
        const int start = A.grp_start[g], cnt = A.grp_count[g];
        it.pos0 = start + t0;
        it.tc = min(EX_TT, cnt - t0);
        it.r0 = chunk * CH;
        const DevStack& m0 = it.shared ? A.s0 : A.w0;
        const DevStack& m1 = MODE == MODE_GATEUP ? (it.shared ? A.s1 : A.w1) : m0;
        const int64_t e = it.shared ? 0 : it.expert;
        // row tiles: gate and up rows r0..r0+31 (GATEUP), down rows r0..r0+31 and r0+32..r0+63
        const int rta = min(it.r0 / 32, m0.rows / 32 - 1);
        const int rtb = MODE == MODE_GATEUP ? rta : min(it.r0 / 32 + 1, m0.rows / 32 - 1);
        it.ta = m0.tile(e, rta);
        it.tb = m1.tile(e, rtb);
        it.nst = m0.nslices;
        it.sa = m0.side + ((size_t)e * m0.rows + rta * 32 + lane) * m0.nslices;
        it.sb = m1.side + ((size_t)e * m1.rows + rtb * 32 + lane) * m1.nslices;
        return it;
    };
    // issues stage `s` of an item into ring slot `slot`: four contiguous copies
    constexpr uint32_t TILE_BYTES = 32 * F::SL;
    constexpr uint32_t ACT_BYTES = act_stage_bytes<TY>();
    auto issue = [&](const Item& it, int s, int slot) {
        uint8_t* dst = ring + (size_t)slot * SB;
        fence_proxy_async();   // the slot was last read through the generic proxy
        __syncwarp();
        if (lane == 0) {
            mbar_expect_tx(&mbar[slot], 2 * TILE_BYTES + ACT_BYTES);
            bulk_g2s(dst, it.ta + (size_t)s * TILE_BYTES, TILE_BYTES, &mbar[slot]);
            bulk_g2s(dst + TILE_BYTES, it.tb + (size_t)s * TILE_BYTES, TILE_BYTES, &mbar[slot]);
            uint8_t* adst = dst + 2 * TILE_BYTES;
            const size_t row = (size_t)s * A.act_rows + it.pos0;
            if (F::F32ACT) {
                bulk_g2s(adst, A.x_f32 + row * F::ELEMS, EX_TT * F::ELEMS * 4, &mbar[slot]);
            } else {
                bulk_g2s(adst, A.x_q + row * F::ELEMS, EX_TT * F::ELEMS, &mbar[slot]);
                bulk_g2s(adst + EX_TT * F::ELEMS, A.x_ds + row * (F::ELEMS / 32),
                         EX_TT * (F::ELEMS / 32) * 8, &mbar[slot]);
            }
        }
        __syncwarp();
    };

    Item cur = fetch();
    if (!cur.valid) return;
    Item nxt;
    nxt.valid = 0;
    // The stages of successive items form one stream; stream stage q lives in
    // slot q & 1.  `issued` runs at most two ahead of `consumed`; the producer
    // cursor (p_in_next, p_stage) names the next stage to issue.
    int issued = 0, consumed = 0, p_in_next = 0, p_stage = 0;
    Side sideA0{}, sideA1{}, sideB0{}, sideB1{};
    auto pump = [&]() {
        while (issued < consumed + 2) {
            if (!p_in_next && p_stage >= cur.nst) {
                p_in_next = 1;
                p_stage = 0;
            }
            if (p_in_next && (!nxt.valid || p_stage >= nxt.nst)) break;
            const Item& it = p_in_next ? nxt : cur;
            const int slot = issued & 1;
            const Side sa = F::side(it.sa, p_stage), sb = F::side(it.sb, p_stage);
            if (slot) { sideA1 = sa; sideB1 = sb; } else { sideA0 = sa; sideB0 = sb; }
            issue(it, p_stage, slot);
            p_stage++;
            issued++;
        }
    };
    pump();
    nxt = fetch();
    pump();

    while (true) {
        float accA[EX_TT], accB[EX_TT];
#pragma unroll
        for (int t = 0; t < EX_TT; t++) accA[t] = accB[t] = 0.0f;
        const int nst = cur.nst;
        for (int s = 0; s < nst; s++) {
            const int slot = consumed & 1;
            if (!mbar_wait_bounded(&mbar[slot], (consumed >> 1) & 1)) {
                // give up: flag it, give the other slot's copies the same bounded wait, leave
                if (lane == 0) atomicExch(A.status, BIVMOE_ERR_TIMEOUT);
                if (issued > consumed + 1)
                    mbar_wait_bounded(&mbar[slot ^ 1], ((consumed + 1) >> 1) & 1);
                return;
            }
            const uint8_t* st = ring + (size_t)slot * SB;
            const uint8_t* wa = st + lane * 16;
            const uint8_t* wb = st + TILE_BYTES + lane * 16;
            const uint8_t* act = st + 2 * TILE_BYTES;
            if constexpr (F::F32ACT) {
                F::accum2f(wa, wb, (const float*)act, cur.tc, accA, accB);
            } else {
                F::accum2(wa, wb, slot ? sideA1 : sideA0, slot ? sideB1 : sideB0, (const int8_t*)act,
                          (const float2*)(act + EX_TT * F::ELEMS), cur.tc, accA, accB);
            }
            __syncwarp();
            consumed++;
            pump();
        }
        // ---- epilogue
        const int rows = (cur.shared ? A.s0 : A.w0).rows;
        if (MODE == MODE_GATEUP) {
            // rows r0..r0+31 of mid: one Q8 block, half a 64-wide f32 slice
            const bool row_ok = cur.r0 < rows;
            const int r = cur.r0 + lane;
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cur.tc && row_ok) {
                    // ops.rs:160-167: silu(x) = x * (1 / (1 + exp(-x)))
                    const float g = accA[t], u = accB[t];
                    const float sg = __fdiv_rn(1.0f, 1.0f + expf(-g));
                    const float v = (g * sg) * u;
                    const size_t pos = cur.pos0 + t;
                    A.out[((size_t)(r / 64) * A.act_rows + pos) * 64 + r % 64] = v;
                    if (A.out_q) {   // Q8Act of the mid row (quant.rs:368-394)
                        float dd, ss;
                        const int q = q8_quantize_lane(v, dd, ss);
                        const size_t srow = (size_t)(r / 256) * A.act_rows + pos;
                        A.out_q[srow * 256 + r % 256] = (int8_t)q;
                        if (lane == 0) A.out_ds[srow * 8 + (cur.r0 % 256) / 32] = make_float2(dd, ss);
                    }
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cur.tc) {
                    float* o = A.out + (size_t)(cur.pos0 + t) * rows + cur.r0;
                    if (cur.r0 + lane < rows) o[lane] = accA[t];
                    if (cur.r0 + 32 + lane < rows) o[32 + lane] = accB[t];
                }
            }
        }
        if (!nxt.valid) break;
        // the stream may already run inside `nxt`: it becomes the current item
        cur = nxt;
        if (p_in_next) p_in_next = 0;
        else p_stage = 0;   // (not reached: a finished item has all its stages issued)
        nxt = fetch();
        pump();
    }
}

// ---------------------------------------------------------------------------
// host side

bool experts_supported(int ty, int cols, int rows, bool is_down) {
    if (ty != BIVMOE_Q8_0 && ty != BIVMOE_Q4_K && ty != BIVMOE_Q5_K && ty != BIVMOE_Q6_K &&
        ty != BIVMOE_BF16)
        return false;
    (void)is_down;
    return cols > 0 && cols % 256 == 0 && rows > 0 && rows % 32 == 0;
}

template <int TY, int MODE>
static cudaError_t launch_one(const LaunchCfg& c, ExpertArgs A, int rows_max) {
    constexpr int CH = MODE == MODE_GATEUP ? 32 : 64;
    A.chunks = (rows_max + CH - 1) / CH;
    constexpr int smem = smem_bytes<TY>();
    static_assert(smem <= 227 * 1024, "two stages per warp must fit in shared memory");
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(experts_kernel<TY, MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    experts_kernel<TY, MODE><<<c.sm_count, Fmt<TY>::WARPS * 32, smem, c.stream>>>(A);
    count_launch();
    return cudaGetLastError();
}

template <int MODE>
static cudaError_t launch_typed(int ty, const LaunchCfg& c, const ExpertArgs& A, int rows_max) {
    switch (ty) {
        case BIVMOE_Q8_0: return launch_one<BIVMOE_Q8_0, MODE>(c, A, rows_max);
        case BIVMOE_Q4_K: return launch_one<BIVMOE_Q4_K, MODE>(c, A, rows_max);
        case BIVMOE_Q5_K: return launch_one<BIVMOE_Q5_K, MODE>(c, A, rows_max);
        case BIVMOE_Q6_K: return launch_one<BIVMOE_Q6_K, MODE>(c, A, rows_max);
        case BIVMOE_BF16: return launch_one<BIVMOE_BF16, MODE>(c, A, rows_max);
        default: return cudaErrorInvalidValue;
    }
}

// gate+up then down, for the routed experts and the shared expert.  When the
// shared expert's matrices have the routed experts' types it rides in the same
// launches (its tiles come first in the tile list); otherwise it gets its own.
cudaError_t launch_experts(const LaunchCfg& c, const float* /*h: dispatched already*/, const DevStack& gate,
                           const DevStack& up, const DevStack& down, const DevStack& sh_gate,
                           const DevStack& sh_up, const DevStack& sh_down, const Workspace& ws) {
    if (gate.ty != up.ty || (c.has_shared && sh_gate.ty != sh_up.ty)) return cudaErrorInvalidValue;
    ExpertArgs A{};
    A.grp_expert = ws.grp_expert; A.grp_start = ws.grp_start; A.grp_count = ws.grp_count;
    A.tile_group = ws.tile_group; A.tile_t0 = ws.tile_t0; A.n_tiles = ws.n_tiles;
    A.status = ws.status;
    A.n = c.n; A.k = c.k; A.n_expert = c.n_expert;
    A.act_rows = ws.act_rows;
    const bool fused = c.has_shared && sh_gate.ty == gate.ty && sh_down.ty == down.ty;
    cudaError_t err;
    // ---- gate + up (SwiGLU and the Q8 rows of its output in the epilogue)
    auto gateup = [&](int mode, int rows, int ctr, int ty, int down_ty) {
        ExpertArgs G = A;
        G.w0 = gate; G.w1 = up; G.s0 = sh_gate; G.s1 = sh_up;
        G.x_f32 = ws.act_f; G.x_q = ws.act_q; G.x_ds = ws.act_ds;
        G.out = ws.mid;
        const bool qdown = !type_uses_f32_act(down_ty);
        G.out_q = qdown ? ws.mid_q : nullptr;
        G.out_ds = qdown ? ws.mid_ds : nullptr;
        G.work_ctr = ws.work_ctr + ctr;
        G.tiles_mode = mode;
        return launch_typed<MODE_GATEUP>(ty, c, G, rows);
    };
    if (fused || !c.has_shared) {
        err = gateup(0, std::max(c.ff, c.ff_sh), 0, gate.ty, down.ty);
    } else {
        err = gateup(1, c.ff, 0, gate.ty, down.ty);
        if (err == cudaSuccess) err = gateup(2, c.ff_sh, 1, sh_gate.ty, sh_down.ty);
    }
    if (err != cudaSuccess) return err;
    mark(c, EV_GATEUP);
    // ---- down
    auto downp = [&](int mode, int ctr, int ty) {
        ExpertArgs D = A;
        D.w0 = down; D.s0 = sh_down;
        D.x_f32 = ws.mid; D.x_q = ws.mid_q; D.x_ds = ws.mid_ds;
        D.out = ws.pair_out;
        D.work_ctr = ws.work_ctr + ctr;
        D.tiles_mode = mode;
        return launch_typed<MODE_DOWN>(ty, c, D, c.e);
    };
    if (fused || !c.has_shared) {
        err = downp(0, 2, down.ty);
    } else {
        err = downp(1, 2, down.ty);
        if (err == cudaSuccess) err = downp(2, 3, sh_down.ty);
    }
    return err;
}

}  // namespace bivmoe
