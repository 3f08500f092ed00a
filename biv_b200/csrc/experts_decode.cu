// Grouped expert products for decode-sized groups: gate+up with the SwiGLU
// fused, and down with the Q8 re-quantisation of its input fused.
// Reference: dense_ffn (engine/src/model.rs:1119-1126) over matmul
// (engine/src/ops.rs:84-127) and the per-type dots (engine/src/quant.rs:
// 599-686 scalar, 1369-1533 AVX2), for each expert's token list
// (model.rs:875-889) and for the shared expert (model.rs:890-896).
//
// Design.  A work item is (group, slab of weight rows); persistent blocks pull
// items from a counter.  The slab's rows are streamed from HBM exactly once
// with per-row bulk copies (cp.async.bulk + mbarrier) into padded shared-memory
// rows, double-buffered against the previous item's arithmetic.  A lane owns
// one weight row, a warp owns a 256-column slice of it; the group's
// activations are staged in shared memory eight tokens at a time and read as
// warp-wide broadcasts, so each weight word is unpacked once and meets every
// token from registers.  Each lane forms whole 32-element block dots with
// __dp4a (the same int32 values as the reference) and applies the block
// scales in f32.  Slices are summed across warps through shared memory in a
// fixed order: no atomics, results are run-to-run identical.
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "formats.cuh"

namespace bivmoe {

constexpr int EX_THREADS = 256;   // 8 warps
constexpr int EX_TT = 8;          // tokens per activation tile
constexpr uint32_t EX_WAIT_LIMIT = 1u << 20;   // bounded mbarrier spin

enum { MODE_GATEUP = 0, MODE_DOWN = 1 };

struct ExpertArgs {
    DevStack w0, w1;     // routed stacks: gate, up (MODE_GATEUP) or down (MODE_DOWN)
    DevStack s0, s1;     // the shared expert's
    const float* x_f32;  // GATEUP: h [n][K]; DOWN: mid [P+n][mid_stride]
    const int8_t* act_q; // GATEUP, quantised types: Q8 rows of h by token
    const float* act_d;
    const float* act_s;
    float* out;          // GATEUP: mid [P+n][mid_stride]; DOWN: pair_out [P+n][e]
    const int32_t* order;
    const int32_t* grp_expert;
    const int32_t* grp_start;
    const int32_t* grp_count;
    const int32_t* n_groups;
    uint32_t* work_ctr;
    int32_t* status;
    int n, k, n_expert;
    int mid_stride;
    int g_lo;            // first group this launch serves
    int g_only_one;      // serve exactly one group (the shared expert's)
    int slabs;           // row slabs per group
    int row_stride;      // shared-memory bytes per staged weight row
    int k_max;           // largest inner dimension among the stacks served
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
// The activation tile in shared memory.
struct ActTile {
    const int8_t* qs;   // [EX_TT][K] (quantised types)
    const float2* ds;   // [EX_TT][K/32] (d, s) per block
    const float* xf;    // [EX_TT][K] (float-activation types)
    int K;
};

// acc[t] += dot(row, activation t) over super-block `sb` (256 columns) for the
// first `cnt` tokens of the tile.  `wrow` is this lane's weight row in shared memory.
template <int TY>
__device__ __forceinline__ void accum_sb(const uint8_t* wrow, int sb, const ActTile& a, int cnt,
                                         float (&acc)[EX_TT]);

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

// Q8_0 (quant.rs:599-607): term = d_w * d_x * sum(q_w * q_x)
template <>
__device__ __forceinline__ void accum_sb<BIVMOE_Q8_0>(const uint8_t* wrow, int sb, const ActTile& a,
                                                      int cnt, float (&acc)[EX_TT]) {
    const int K = a.K;
#pragma unroll 2
    for (int bb = 0; bb < 8; bb++) {
        const int b = sb * 8 + bb;
        const uint4 q0 = *(const uint4*)(wrow + 32 * b), q1 = *(const uint4*)(wrow + 32 * b + 16);
        const int w[8] = {(int)q0.x, (int)q0.y, (int)q0.z, (int)q0.w,
                          (int)q1.x, (int)q1.y, (int)q1.z, (int)q1.w};
        const float dw = __half2float(*(const __half*)(wrow + K + 2 * b));
#pragma unroll
        for (int t = 0; t < EX_TT; t++) {
            if (t < cnt) {
                const int4* ap = (const int4*)(a.qs + (size_t)t * K + 32 * b);
                const int i0 = dot8(w, ap[0], ap[1]);
                const float dx = a.ds[t * (K / 32) + b].x;
                acc[t] += (dw * dx) * (float)i0;
            }
        }
    }
}

// Q4_K / Q5_K (quant.rs:609-649): per sub-block
//   d*sc*d_x*sum(q*q_x) - dmin*m*s_x ; Q5_K adds bit sb of qh[l] as value bit 4
template <int TY>
__device__ __forceinline__ void accum_k45(const uint8_t* wrow, int sb, const ActTile& a, int cnt,
                                          float (&acc)[EX_TT]) {
    constexpr int BS = TY == BIVMOE_Q4_K ? 144 : 176;
    constexpr int QOFF = TY == BIVMOE_Q4_K ? 16 : 48;
    const int K = a.K;
    const uint8_t* blk = wrow + (size_t)sb * BS;
    const uint4 hdr = *(const uint4*)blk;
    const __half2 dd = *(const __half2*)&hdr.x;
    const float d = __low2float(dd), dmin = __high2float(dd);
    const K4Scales sc = unpack_k4_scales(hdr.y, hdr.z, hdr.w);
    uint32_t qh[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (TY == BIVMOE_Q5_K) {
        const uint4 h0 = *(const uint4*)(blk + 16), h1 = *(const uint4*)(blk + 32);
        qh[0] = h0.x; qh[1] = h0.y; qh[2] = h0.z; qh[3] = h0.w;
        qh[4] = h1.x; qh[5] = h1.y; qh[6] = h1.z; qh[7] = h1.w;
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint4 qa = *(const uint4*)(blk + QOFF + 32 * j);
        const uint4 qb = *(const uint4*)(blk + QOFF + 32 * j + 16);
        const uint32_t qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        int lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            lo[i] = LO4(qv[i]);
            hi[i] = HI4(qv[i]);
            if (TY == BIVMOE_Q5_K) {
                lo[i] |= (int)(((qh[i] >> (2 * j)) & 0x01010101u) << 4);
                hi[i] |= (int)(((qh[i] >> (2 * j + 1)) & 0x01010101u) << 4);
            }
        }
        const float dsc0 = d * (float)k4_scale(sc, 2 * j), dm0 = dmin * (float)k4_min(sc, 2 * j);
        const float dsc1 = d * (float)k4_scale(sc, 2 * j + 1),
                    dm1 = dmin * (float)k4_min(sc, 2 * j + 1);
        const int xb = sb * 8 + 2 * j;
#pragma unroll
        for (int t = 0; t < EX_TT; t++) {
            if (t < cnt) {
                const int4* ap = (const int4*)(a.qs + (size_t)t * K + 32 * xb);
                const int i0 = dot8(lo, ap[0], ap[1]);
                const int i1 = dot8(hi, ap[2], ap[3]);
                const float4 dx = *(const float4*)(a.ds + t * (K / 32) + xb);  // d0 s0 d1 s1
                acc[t] += (dsc0 * dx.x) * (float)i0 - dm0 * dx.y;
                acc[t] += (dsc1 * dx.z) * (float)i1 - dm1 * dx.w;
            }
        }
    }
}
template <>
__device__ __forceinline__ void accum_sb<BIVMOE_Q4_K>(const uint8_t* wrow, int sb, const ActTile& a,
                                                      int cnt, float (&acc)[EX_TT]) {
    accum_k45<BIVMOE_Q4_K>(wrow, sb, a, cnt, acc);
}
template <>
__device__ __forceinline__ void accum_sb<BIVMOE_Q5_K>(const uint8_t* wrow, int sb, const ActTile& a,
                                                      int cnt, float (&acc)[EX_TT]) {
    accum_k45<BIVMOE_Q5_K>(wrow, sb, a, cnt, acc);
}

// Q6_K (quant.rs:651-686), device row planes [ql][qh][scales][d]: per 32-block
//   d * d_x * (sc[2g]*sum16 + sc[2g+1]*sum16), 6-bit values minus 32
template <>
__device__ __forceinline__ void accum_sb<BIVMOE_Q6_K>(const uint8_t* wrow, int sb, const ActTile& a,
                                                      int cnt, float (&acc)[EX_TT]) {
    const int K = a.K, nb = K / 256;
    const uint8_t* ql = wrow + (size_t)sb * 128;
    const uint8_t* qhp = wrow + (size_t)nb * 128 + (size_t)sb * 64;
    const int8_t* scp = (const int8_t*)wrow + (size_t)nb * 192 + (size_t)sb * 16;
    const float d = __half2float(*(const __half*)(wrow + (size_t)nb * 208 + 2 * sb));
#pragma unroll
    for (int n = 0; n < 2; n++) {
        uint32_t l0[8], l1[8], hh[8];
        {
            const uint4 a0 = *(const uint4*)(ql + 64 * n), a1 = *(const uint4*)(ql + 64 * n + 16);
            const uint4 b0 = *(const uint4*)(ql + 64 * n + 32), b1 = *(const uint4*)(ql + 64 * n + 48);
            const uint4 h0 = *(const uint4*)(qhp + 32 * n), h1 = *(const uint4*)(qhp + 32 * n + 16);
            l0[0] = a0.x; l0[1] = a0.y; l0[2] = a0.z; l0[3] = a0.w;
            l0[4] = a1.x; l0[5] = a1.y; l0[6] = a1.z; l0[7] = a1.w;
            l1[0] = b0.x; l1[1] = b0.y; l1[2] = b0.z; l1[3] = b0.w;
            l1[4] = b1.x; l1[5] = b1.y; l1[6] = b1.z; l1[7] = b1.w;
            hh[0] = h0.x; hh[1] = h0.y; hh[2] = h0.z; hh[3] = h0.w;
            hh[4] = h1.x; hh[5] = h1.y; hh[6] = h1.z; hh[7] = h1.w;
        }
        const uint2 scw = *(const uint2*)(scp + 8 * n);
#pragma unroll
        for (int kq = 0; kq < 4; kq++) {
            int q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t base = (kq & 1) ? l1[i] : l0[i];
                const uint32_t nib = (kq >= 2 ? base >> 4 : base) & 0x0F0F0F0Fu;
                const uint32_t hb = ((hh[i] >> (2 * kq)) & 0x03030303u) << 4;
                q[i] = (int)__vsub4(nib | hb, 0x20202020u);
            }
            const uint32_t sw = kq < 2 ? scw.x : scw.y;
            const int sca = (int)(int8_t)((sw >> (16 * (kq & 1))) & 0xFF);
            const int scb = (int)(int8_t)((sw >> (16 * (kq & 1) + 8)) & 0xFF);
            const int xb = sb * 8 + 4 * n + kq;
#pragma unroll
            for (int t = 0; t < EX_TT; t++) {
                if (t < cnt) {
                    const int4* ap = (const int4*)(a.qs + (size_t)t * K + 32 * xb);
                    const int4 a0 = ap[0], a1 = ap[1];
                    int ia = dp4a_s8(q[0], a0.x, 0);
                    ia = dp4a_s8(q[1], a0.y, ia);
                    ia = dp4a_s8(q[2], a0.z, ia);
                    ia = dp4a_s8(q[3], a0.w, ia);
                    int ib = dp4a_s8(q[4], a1.x, 0);
                    ib = dp4a_s8(q[5], a1.y, ib);
                    ib = dp4a_s8(q[6], a1.z, ib);
                    ib = dp4a_s8(q[7], a1.w, ib);
                    const int isum = sca * ia + scb * ib;
                    const float dx = a.ds[t * (K / 32) + xb].x;
                    acc[t] += (d * dx) * (float)isum;
                }
            }
        }
    }
}

// BF16 weights meet f32 activations (quant.rs:509-521, 1229-1256)
template <>
__device__ __forceinline__ void accum_sb<BIVMOE_BF16>(const uint8_t* wrow, int sb, const ActTile& a,
                                                      int cnt, float (&acc)[EX_TT]) {
    const int K = a.K;
#pragma unroll 4
    for (int u = 0; u < 32; u++) {
        const uint4 wv = *(const uint4*)(wrow + (size_t)sb * 512 + 16 * u);
        const float w[8] = {__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xFFFF0000u),
                            __uint_as_float(wv.y << 16), __uint_as_float(wv.y & 0xFFFF0000u),
                            __uint_as_float(wv.z << 16), __uint_as_float(wv.z & 0xFFFF0000u),
                            __uint_as_float(wv.w << 16), __uint_as_float(wv.w & 0xFFFF0000u)};
#pragma unroll
        for (int t = 0; t < EX_TT; t++) {
            if (t < cnt) {
                const float4* xp = (const float4*)(a.xf + (size_t)t * K + sb * 256 + 8 * u);
                const float4 x0 = xp[0], x1 = xp[1];
                float s = acc[t];
                s = fmaf(w[0], x0.x, s); s = fmaf(w[1], x0.y, s);
                s = fmaf(w[2], x0.z, s); s = fmaf(w[3], x0.w, s);
                s = fmaf(w[4], x1.x, s); s = fmaf(w[5], x1.y, s);
                s = fmaf(w[6], x1.z, s); s = fmaf(w[7], x1.w, s);
                acc[t] = s;
            }
        }
    }
}

// ---------------------------------------------------------------------------
template <int MODE> struct Shape;
template <> struct Shape<MODE_GATEUP> {   // 16 gate rows + the 16 matching up rows
    static constexpr int WARPS_ROW = 1, WARPS_K = 8, ROWS = 32, OUT_ROWS = 16;
};
template <> struct Shape<MODE_DOWN> {
    static constexpr int WARPS_ROW = 4, WARPS_K = 2, ROWS = 128, OUT_ROWS = 128;
};

template <int TY> struct TypeCfg { static constexpr int NSTAGE = 2; };
template <> struct TypeCfg<BIVMOE_BF16> { static constexpr int NSTAGE = 1; };

__host__ __device__ inline int padded_row_stride(int64_t row_bytes) {
    // an odd number of 16-byte units: lanes that own consecutive rows then hit
    // distinct bank groups on 128-bit loads
    int units = (int)(row_bytes / 16);
    return (units | 1) * 16;
}

struct SmemPlan {
    int stage_off, act_off, ds_off, part_off, total;
};
template <int TY, int MODE>
__host__ __device__ inline SmemPlan smem_plan(int row_stride, int k_max) {
    using S = Shape<MODE>;
    SmemPlan p;
    p.stage_off = 64;
    int off = p.stage_off + TypeCfg<TY>::NSTAGE * S::ROWS * row_stride;
    p.act_off = off;
    if (type_uses_f32_act(TY)) {
        off += EX_TT * k_max * 4;
        p.ds_off = off;
    } else {
        off += EX_TT * k_max;
        p.ds_off = off;
        off += EX_TT * (k_max / 32) * 8;
    }
    p.part_off = off;
    off += S::WARPS_K * S::ROWS * EX_TT * 4;
    p.total = off;
    return p;
}

template <int TY, int MODE>
__global__ void __launch_bounds__(EX_THREADS)
experts_kernel(const ExpertArgs A) {
    using S = Shape<MODE>;
    constexpr int NSTAGE = TypeCfg<TY>::NSTAGE;
    constexpr bool F32ACT = TY == BIVMOE_BF16 || TY == BIVMOE_F32;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* mbar = (uint64_t*)smem;            // [NSTAGE]
    int* s_item = (int*)(smem + 32);
    const SmemPlan plan = smem_plan<TY, MODE>(A.row_stride, A.k_max);
    uint8_t* stage_base = smem + plan.stage_off;
    int8_t* s_qs = (int8_t*)(smem + plan.act_off);
    float* s_xf = (float*)(smem + plan.act_off);
    float2* s_ds = (float2*)(smem + plan.ds_off);
    float* s_part = (float*)(smem + plan.part_off);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wr = warp % S::WARPS_ROW, wk = warp / S::WARPS_ROW;
    const int P = A.n * A.k;
    const int n_groups = A.g_only_one ? 1 : *A.n_groups - A.g_lo;
    const int total = n_groups * A.slabs;

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; s++) mbar_init(&mbar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // streams the rows of one item into a stage (warp 0)
    auto issue = [&](int item, int stage) {
        const int g = A.g_lo + item / A.slabs, slab = item % A.slabs;
        const int ex = A.grp_expert[g];
        const bool shared = ex == A.n_expert;
        const DevStack& m0 = shared ? A.s0 : A.w0;
        const DevStack& m1 = shared ? A.s1 : A.w1;
        const int e_idx = shared ? 0 : ex;
        const int r0 = slab * S::OUT_ROWS;
        const int valid = max(0, min(S::OUT_ROWS, m0.rows - r0));
        uint8_t* dst = stage_base + (size_t)stage * S::ROWS * A.row_stride;
        const uint32_t rb = (uint32_t)m0.row_bytes;
        // the stage was last read through the generic proxy (before a block barrier)
        fence_proxy_async();
        if (lane == 0) mbar_expect_tx(&mbar[stage], rb * valid * (MODE == MODE_GATEUP ? 2 : 1));
        __syncwarp();
        const uint8_t* src0 = m0.data + (size_t)e_idx * m0.expert_bytes + (size_t)r0 * rb;
        for (int r = lane; r < valid; r += 32)
            bulk_g2s(dst + (size_t)r * A.row_stride, src0 + (size_t)r * rb, rb, &mbar[stage]);
        if (MODE == MODE_GATEUP) {
            const uint8_t* src1 = m1.data + (size_t)e_idx * m1.expert_bytes + (size_t)r0 * rb;
            for (int r = lane; r < valid; r += 32)
                bulk_g2s(dst + (size_t)(S::OUT_ROWS + r) * A.row_stride, src1 + (size_t)r * rb, rb,
                         &mbar[stage]);
        }
    };
    auto fetch = [&]() -> int {
        if (tid == 0) *s_item = (int)atomicAdd(A.work_ctr, 1u);
        __syncthreads();
        const int it = *s_item;
        __syncthreads();
        return it;
    };

    int item = fetch();
    if (item >= total) return;
    if (warp == 0) issue(item, 0);
    uint32_t phase[2] = {0, 0};
    int stage = 0;

    while (true) {
        const int next = fetch();
        if (NSTAGE == 2 && next < total && warp == 0) issue(next, stage ^ 1);
        if (!mbar_wait_bounded(&mbar[stage], phase[stage])) {
            // every thread waits on the same barrier, so all give up together; the
            // copies already issued for the next item get the same bounded wait
            if (tid == 0) atomicExch(A.status, BIVMOE_ERR_TIMEOUT);
            if (NSTAGE == 2 && next < total) mbar_wait_bounded(&mbar[stage ^ 1], phase[stage ^ 1]);
            return;
        }
        phase[stage] ^= 1;

        const int g = A.g_lo + item / A.slabs, slab = item % A.slabs;
        const int ex = A.grp_expert[g], start = A.grp_start[g], cnt = A.grp_count[g];
        const bool shared = ex == A.n_expert;
        const DevStack& m0 = shared ? A.s0 : A.w0;
        const int K = m0.cols, nsb = K / 256;
        const int r0 = slab * S::OUT_ROWS;
        const uint8_t* wrow =
            stage_base + ((size_t)stage * S::ROWS + wr * 32 + lane) * A.row_stride;
        ActTile at;
        at.qs = s_qs; at.ds = s_ds; at.xf = s_xf; at.K = K;

        for (int t0 = 0; t0 < cnt; t0 += EX_TT) {
            const int tc = min(EX_TT, cnt - t0);
            // ---- stage the activations of tokens t0..t0+tc
            if (MODE == MODE_GATEUP) {
                if (F32ACT) {
                    for (int i = tid; i < tc * (K / 4); i += EX_THREADS) {
                        const int t = i / (K / 4), c = i % (K / 4);
                        const int pos = start + t0 + t;
                        const int tok = shared ? pos - P : A.order[pos] / A.k;
                        ((float4*)s_xf)[t * (K / 4) + c] =
                            ((const float4*)(A.x_f32 + (size_t)tok * K))[c];
                    }
                } else {
                    for (int i = tid; i < tc * (K / 16); i += EX_THREADS) {
                        const int t = i / (K / 16), c = i % (K / 16);
                        const int pos = start + t0 + t;
                        const int tok = shared ? pos - P : A.order[pos] / A.k;
                        ((int4*)s_qs)[t * (K / 16) + c] =
                            ((const int4*)(A.act_q + (size_t)tok * K))[c];
                    }
                    for (int i = tid; i < tc * (K / 32); i += EX_THREADS) {
                        const int t = i / (K / 32), b = i % (K / 32);
                        const int pos = start + t0 + t;
                        const int tok = shared ? pos - P : A.order[pos] / A.k;
                        s_ds[t * (K / 32) + b] = make_float2(A.act_d[(size_t)tok * (K / 32) + b],
                                                             A.act_s[(size_t)tok * (K / 32) + b]);
                    }
                }
            } else {
                if (F32ACT) {
                    for (int i = tid; i < tc * (K / 4); i += EX_THREADS) {
                        const int t = i / (K / 4), c = i % (K / 4);
                        ((float4*)s_xf)[t * (K / 4) + c] =
                            ((const float4*)(A.x_f32 + (size_t)(start + t0 + t) * A.mid_stride))[c];
                    }
                } else {
                    // Q8Act of the mid rows, quantised here (quant.rs:368-394)
                    for (int i = warp; i < tc * (K / 32); i += EX_THREADS / 32) {
                        const int t = i / (K / 32), b = i % (K / 32);
                        const float v =
                            A.x_f32[(size_t)(start + t0 + t) * A.mid_stride + 32 * b + lane];
                        float dd, ss;
                        const int q = q8_quantize_lane(v, dd, ss);
                        s_qs[(size_t)t * K + 32 * b + lane] = (int8_t)q;
                        if (lane == 0) s_ds[t * (K / 32) + b] = make_float2(dd, ss);
                    }
                }
            }
            __syncthreads();
            // ---- this warp's slice of the dots
            float acc[EX_TT];
#pragma unroll
            for (int t = 0; t < EX_TT; t++) acc[t] = 0.0f;
            for (int sb = wk; sb < nsb; sb += S::WARPS_K) accum_sb<TY>(wrow, sb, at, tc, acc);
#pragma unroll
            for (int t = 0; t < EX_TT; t++)
                s_part[(wk * S::ROWS + wr * 32 + lane) * EX_TT + t] = acc[t];
            __syncthreads();
            // ---- sum the slices in a fixed order, epilogue
            if (MODE == MODE_GATEUP) {
                if (tid < S::OUT_ROWS * EX_TT) {
                    const int r = tid % S::OUT_ROWS, t = tid / S::OUT_ROWS;
                    float gsum = 0.0f, usum = 0.0f;
#pragma unroll
                    for (int w = 0; w < S::WARPS_K; w++) {
                        gsum += s_part[(w * S::ROWS + r) * EX_TT + t];
                        usum += s_part[(w * S::ROWS + S::OUT_ROWS + r) * EX_TT + t];
                    }
                    if (t < tc && r0 + r < m0.rows) {
                        // ops.rs:160-167: silu(x) = x * (1 / (1 + exp(-x)))
                        const float sg = __fdiv_rn(1.0f, 1.0f + expf(-gsum));
                        A.out[(size_t)(start + t0 + t) * A.mid_stride + r0 + r] = (gsum * sg) * usum;
                    }
                }
            } else {
                for (int i = tid; i < S::OUT_ROWS * EX_TT; i += EX_THREADS) {
                    const int r = i % S::OUT_ROWS, t = i / S::OUT_ROWS;
                    float sum = 0.0f;
#pragma unroll
                    for (int w = 0; w < S::WARPS_K; w++) sum += s_part[(w * S::ROWS + r) * EX_TT + t];
                    if (t < tc && r0 + r < m0.rows)
                        A.out[(size_t)(start + t0 + t) * m0.rows + r0 + r] = sum;
                }
            }
            // the next tile's staging overwrites the activations only after every
            // warp passed the barrier above; s_part is rewritten after the next one
        }
        __syncthreads();
        if (next >= total) break;
        if (NSTAGE == 1 && warp == 0) issue(next, 0);
        item = next;
        if (NSTAGE == 2) stage ^= 1;
    }
}

// ---------------------------------------------------------------------------
// host side

bool experts_supported(int ty, int cols, int rows, bool is_down) {
    if (ty != BIVMOE_Q8_0 && ty != BIVMOE_Q4_K && ty != BIVMOE_Q5_K && ty != BIVMOE_Q6_K &&
        ty != BIVMOE_BF16)
        return false;
    if (cols <= 0 || cols % 256) return false;
    if (rows <= 0 || (!is_down && rows % 16)) return false;
    return dev_row_bytes(ty, cols) % 16 == 0;
}

template <int TY, int MODE>
static cudaError_t launch_one(const LaunchCfg& c, ExpertArgs A, int rows_max, bool only_shared) {
    using S = Shape<MODE>;
    A.row_stride = padded_row_stride(std::max(A.w0.row_bytes, A.s0.row_bytes));
    A.slabs = (rows_max + S::OUT_ROWS - 1) / S::OUT_ROWS;
    const SmemPlan plan = smem_plan<TY, MODE>(A.row_stride, A.k_max);
    if (plan.total > 227 * 1024) return cudaErrorInvalidConfiguration;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(experts_kernel<TY, MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    int per_sm = std::max(1, std::min(4, (227 * 1024) / (plan.total + 1024)));
    int max_items = (only_shared ? 1 : c.n_expert + 1) * A.slabs;
    int grid = std::min(c.sm_count * per_sm, max_items);
    experts_kernel<TY, MODE><<<grid, EX_THREADS, plan.total, c.stream>>>(A);
    count_launch();
    return cudaGetLastError();
}

template <int MODE>
static cudaError_t launch_typed(int ty, const LaunchCfg& c, const ExpertArgs& A, int rows_max,
                                bool only_shared) {
    switch (ty) {
        case BIVMOE_Q8_0: return launch_one<BIVMOE_Q8_0, MODE>(c, A, rows_max, only_shared);
        case BIVMOE_Q4_K: return launch_one<BIVMOE_Q4_K, MODE>(c, A, rows_max, only_shared);
        case BIVMOE_Q5_K: return launch_one<BIVMOE_Q5_K, MODE>(c, A, rows_max, only_shared);
        case BIVMOE_Q6_K: return launch_one<BIVMOE_Q6_K, MODE>(c, A, rows_max, only_shared);
        case BIVMOE_BF16: return launch_one<BIVMOE_BF16, MODE>(c, A, rows_max, only_shared);
        default: return cudaErrorInvalidValue;
    }
}

// gate+up then down, for the routed experts and the shared expert.  When the
// shared expert's matrices have the routed experts' types (and the same
// gate/up type) it rides in the same launches as group 0.
cudaError_t launch_experts(const LaunchCfg& c, const float* h, const DevStack& gate,
                           const DevStack& up, const DevStack& down, const DevStack& sh_gate,
                           const DevStack& sh_up, const DevStack& sh_down, const Workspace& ws) {
    if (gate.ty != up.ty || (c.has_shared && sh_gate.ty != sh_up.ty)) return cudaErrorInvalidValue;
    ExpertArgs A{};
    A.order = ws.order;
    A.grp_expert = ws.grp_expert; A.grp_start = ws.grp_start; A.grp_count = ws.grp_count;
    A.n_groups = ws.n_groups;
    A.status = ws.status;
    A.n = c.n; A.k = c.k; A.n_expert = c.n_expert;
    A.mid_stride = std::max(c.ff, c.ff_sh);
    A.act_q = ws.act_q; A.act_d = ws.act_d; A.act_s = ws.act_s;
    const bool fuse_gu = c.has_shared && sh_gate.ty == gate.ty;
    const bool fuse_dn = c.has_shared && sh_down.ty == down.ty;
    cudaError_t err;
    // ---- gate + up
    {
        ExpertArgs G = A;
        G.w0 = gate; G.w1 = up; G.s0 = sh_gate; G.s1 = sh_up;
        G.x_f32 = h; G.out = ws.mid;
        G.k_max = c.e;
        G.work_ctr = ws.work_ctr + 0;
        G.g_lo = c.has_shared && !fuse_gu ? 1 : 0;
        G.g_only_one = 0;
        if (!fuse_gu) G.s0 = DevStack{}, G.s1 = DevStack{};
        err = launch_typed<MODE_GATEUP>(gate.ty, c, G, std::max(c.ff, fuse_gu ? c.ff_sh : 0), false);
        if (err != cudaSuccess) return err;
        if (c.has_shared && !fuse_gu) {
            ExpertArgs H = A;
            H.s0 = sh_gate; H.s1 = sh_up; H.w0 = sh_gate; H.w1 = sh_up;
            H.x_f32 = h; H.out = ws.mid; H.k_max = c.e;
            H.work_ctr = ws.work_ctr + 1;
            H.g_lo = 0; H.g_only_one = 1;
            err = launch_typed<MODE_GATEUP>(sh_gate.ty, c, H, c.ff_sh, true);
            if (err != cudaSuccess) return err;
        }
    }
    mark(c, EV_GATEUP);
    // ---- down
    {
        ExpertArgs D = A;
        D.w0 = down; D.s0 = sh_down;
        D.x_f32 = ws.mid; D.out = ws.pair_out;
        D.k_max = std::max(c.ff, fuse_dn ? c.ff_sh : 0);
        D.work_ctr = ws.work_ctr + 2;
        D.g_lo = c.has_shared && !fuse_dn ? 1 : 0;
        D.g_only_one = 0;
        if (!fuse_dn) D.s0 = DevStack{};
        err = launch_typed<MODE_DOWN>(down.ty, c, D, c.e, false);
        if (err != cudaSuccess) return err;
        if (c.has_shared && !fuse_dn) {
            ExpertArgs H = A;
            H.s0 = sh_down; H.w0 = sh_down;
            H.x_f32 = ws.mid; H.out = ws.pair_out; H.k_max = c.ff_sh;
            H.work_ctr = ws.work_ctr + 3;
            H.g_lo = 0; H.g_only_one = 1;
            err = launch_typed<MODE_DOWN>(sh_down.ty, c, H, c.e, true);
            if (err != cudaSuccess) return err;
        }
    }
    return cudaSuccess;
}

}  // namespace bivmoe
