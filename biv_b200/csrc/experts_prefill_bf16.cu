// Grouped expert products for prefill-sized groups with BF16 weights on the 5th
// generation tensor cores: tcgen05.mma kind::f16 (bf16 x bf16 -> f32) with the
// accumulator in tensor memory.
// Reference: dense_ffn (engine/src/model.rs:1119-1126) over the bf16 dot
// (engine/src/quant.rs:509-521: bf16 weights widened to f32, times f32
// activations, f32 accumulation), for experts whose token list is long
// (model.rs:875-889).
//
// The reference multiplies bf16 weights by f32 activations.  The tensor core
// takes bf16 on both sides, so an activation row is fed as two bf16 terms,
// x = hi + lo (hi = bf16(x), lo = bf16(x - hi)), which represents x to 2^-17 |x|;
// every weight K-step is multiplied by both and the products - exact in f32 -
// accumulate in tensor memory.  That doubles the MMA count and keeps the result
// within a few f32 roundings of the reference's, far inside the layer tolerance.
//
// Design.  One block per SM: one thread of warp 0 issues the copies, one thread of a
// warp of its own the MMAs; four epilogue warps own the 128 tensor-memory lanes.  A work item is
// a tile of 128 tokens of one group times TWO chunks of 128 weight rows (a chunk:
// 64 gate rows with their 64 up rows, or 128 down rows).  A pipeline stage is one
// K-slice of 64 values: 128 rows x 128 bytes of weights per chunk and the tile's
// 16 activation records (hi and lo), all in the tensor core's canonical K-major
// layout (common.cuh).  The weights and, for the down product, the records of mid
// (written in that layout by the gate+up epilogue) arrive by bulk copies.  For the
// gate+up product four more warps gather the tile's rows by token from the
// token-ordered bf16 terms (rowops.cu, split_rows_kernel) with 16-byte asynchronous
// copies that complete on the stage's barrier: a row is split once and never
// written per position.  The kernel is
// bound by what an SM can pull from L2, and the activation records are two
// thirds of a one-chunk stage: sharing them between two chunks cuts the bytes per
// multiply-add by a third.  Per stage the MMA thread issues, per chunk, 2 terms x
// 4 K-steps (M = 128, N = 128, K = 16) accumulating into that chunk's half of
// one of two tensor-memory buffers; unlike the Q8_0 kernel nothing is scaled per
// block, so the epilogue runs once per item, while the next item's MMAs fill the
// other buffer.  Every wait is bounded; a wait that gives up records
// BIVMOE_ERR_TIMEOUT, the block leaves its loops, frees its tensor memory and
// returns.
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "tcgen05.cuh"
#include "launch.cuh"

namespace bivmoe {

constexpr int BF_NT = kPrefillTileBf16;                         // tokens per tile = MMA N
constexpr int BF_CG = 4;                                        // epilogue warps per tensor-memory lane quadrant
constexpr int BF_EPI_WARPS = 4 * BF_CG, BF_GATHER_WARPS = 4;
constexpr int BF_MMA_WARP = 1 + BF_EPI_WARPS;                            // a warp of its own (see the kernel)
constexpr int BF_THREADS = 32 * (2 + BF_EPI_WARPS);                      // the down product
constexpr int BF_THREADS_GATHER = BF_THREADS + 32 * BF_GATHER_WARPS;     // gate+up
constexpr uint32_t BF_W_BYTES = kChunkRows * 128;               // 16384: one K-slice of a chunk
constexpr uint32_t BF_X_BYTES = (BF_NT / 8) * kActBRec;         // 32768
constexpr uint32_t BF_X_TERM = BF_NT * 128;                     // gathered rows: the lo tile follows the hi tile
constexpr int BF_MC = 2;                                        // chunks per item
constexpr uint32_t BF_STAGE = BF_MC * BF_W_BYTES + BF_X_BYTES;  // 65536
constexpr int BF_NSTAGE = 3;
constexpr uint32_t BF_HEAD = 1024;
constexpr uint32_t BF_XCHG = BF_CG * 64 * 16 * 4;               // SwiGLU exchange: 16 tokens per column group
constexpr uint32_t BF_SMEM = BF_HEAD + BF_NSTAGE * BF_STAGE + BF_XCHG;   // 214016
constexpr uint32_t BF_TMEM_COLS = 512;                          // two buffers of 2 x 128 columns
constexpr uint32_t BF_TBUF = BF_MC * BF_NT;                     // columns of one buffer

enum { BF_GATEUP = 0, BF_DOWN = 1 };

struct Bf16Args {
    DevTiles w, sh;
    const uint8_t* x_b;    // DOWN: bf16 hi/lo records of mid by position, [K/64][R/8]
    const uint8_t* tok_b;  // GATEUP: bf16 hi/lo terms of the rows by token, [N][K/64][kTokBRec]
    const int32_t* order;  // GATEUP: order[pos] / k is the token at a routed group's position
    int k;
    int act_rows;          // R
    float* out;            // GATEUP: mid f32 slice-major; DOWN: pair_out [R][rows]
    uint8_t* out_b;        // GATEUP: bf16 hi/lo records of mid
    const int32_t* grp_expert;
    const int32_t* grp_start;
    const int32_t* grp_count;
    const int32_t* ptile_group;
    const int32_t* ptile_t0;
    const int32_t* n_ptiles;
    int32_t* status;
    int n_expert;
    int tiles_mode;        // 0: every tile, 1: skip the shared group's, 2: only the shared group's
    int chunks;
};

struct BfItem {
    int shared, expert, chunk, nch, pos0, tc, nst;   // chunks chunk .. chunk + nch - 1
    int n_mma;             // tc rounded up to the MMA's N granularity of 16: a ragged last
                           // tile costs MMA time and activation bytes for its own tokens only
    const uint8_t* wsrc;   // stage 0 of the first chunk's weights; stage s is s * BF_W_BYTES
    size_t wstep;          // further, the next chunk wstep further
};

__device__ __forceinline__ void bf_cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// one arrival on `bar` once this thread's copies so far have landed (counted in the
// barrier's expected arrivals)
__device__ __forceinline__ void bf_cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(pf_smem(bar)) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(MODE == 0 ? BF_THREADS_GATHER : BF_THREADS, 1)
experts_prefill_bf16_kernel(const Bf16Args A) {
    pdl_launch_dependents();
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;            // [3] copies landed
    uint64_t* empty = full + 4;                  // [3] stage free: its MMAs are done
    uint64_t* tfull = full + 8;                  // [2] an item's products are in tensor memory
    uint64_t* tempty = full + 10;                // [2] drained by the epilogue warps
    uint64_t* xbar = full + 12;                  // [BF_CG] meeting points of the epilogue warps of a column group
    uint32_t* s_tmem = (uint32_t*)(smem + 256);
    int* s_abort = (int*)(smem + 260);
    uint8_t* stages = smem + BF_HEAD;
    float* s_xchg = (float*)(smem + BF_HEAD + BF_NSTAGE * BF_STAGE);   // [BF_CG][16 tokens][64 rows]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int CH = MODE == BF_GATEUP ? 64 : 128;   // output rows per chunk

    if (tid == 0) {
        for (int i = 0; i < BF_NSTAGE; i++) {
            // the copy thread's arrival with the bulk copies' bytes + every gathering thread
            pf_bar_init(&full[i], MODE == BF_GATEUP ? 1 + 32 * BF_GATHER_WARPS : 1);
            pf_bar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            pf_bar_init(&tfull[i], 1);
            pf_bar_init(&tempty[i], BF_EPI_WARPS);
        }
        for (int i = 0; i < BF_CG; i++) pf_bar_init(&xbar[i], 4);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         pf_smem(s_tmem)),
                     "r"(BF_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pf_fence_before();
    __syncthreads();
    pf_fence_after();
    const uint32_t tmem = *s_tmem;
    pdl_wait();   // the tile lists and the activation records are the previous kernels'

    const int tiles_all = A.n_ptiles[0], tiles_sh = A.n_ptiles[1];
    const int tile_lo = A.tiles_mode == 1 ? tiles_sh : 0;
    const int tile_hi = A.tiles_mode == 2 ? tiles_sh : tiles_all;
    const int cpairs = (A.chunks + BF_MC - 1) / BF_MC;
    const int total = (tile_hi - tile_lo) * cpairs;

    // items are dealt round-robin; every role walks the same sequence on its own
    auto decode = [&](int idx) -> BfItem {
        BfItem it;
        const int tile = tile_lo + idx / cpairs;
        it.chunk = (idx % cpairs) * BF_MC;
        const int gi = A.ptile_group[tile], t0 = A.ptile_t0[tile];
        it.expert = A.grp_expert[gi];
        it.shared = it.expert == A.n_expert;
        it.pos0 = A.grp_start[gi] + t0;
        it.tc = min(BF_NT, A.grp_count[gi] - t0);
        it.n_mma = (it.tc + 15) & ~15;
        const DevTiles& m = it.shared ? A.sh : A.w;
        it.nch = max(0, min(BF_MC, m.chunks - it.chunk));
        it.nst = it.nch > 0 ? m.nslices : 0;
        it.wsrc = m.stage(it.shared ? 0 : it.expert, min(it.chunk, max(m.chunks - 1, 0)), 0);
        it.wstep = (size_t)m.nslices * BF_W_BYTES;
        return it;
    };
    auto give_up = [&]() {
        atomicExch(A.status, BIVMOE_ERR_TIMEOUT);
        atomicExch(s_abort, 1);
    };

    if (warp == 0 && lane == 0) {
        // ---------------- copy thread: two bulk copies per stage
        uint32_t q = 0;
        bool dead = false;
        for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            for (int s = 0; s < it.nst && !dead; s++, q++) {
                const uint32_t slot = q % BF_NSTAGE;
                if (!pf_bar_wait(&empty[slot], ((q / BF_NSTAGE) & 1) ^ 1)) { give_up(); dead = true; break; }
                uint8_t* dst = stages + slot * BF_STAGE;
                const uint32_t x_bytes = MODE == BF_GATEUP ? 0u : (uint32_t)(it.n_mma / 8) * kActBRec;
                pf_bar_expect_tx(&full[slot], it.nch * BF_W_BYTES + x_bytes);
                for (int ch = 0; ch < it.nch; ch++)
                    pf_bulk_g2s(dst + ch * BF_W_BYTES, it.wsrc + ch * it.wstep + (size_t)s * BF_W_BYTES,
                                BF_W_BYTES, &full[slot]);
                if (MODE == BF_DOWN)
                    pf_bulk_g2s(dst + BF_MC * BF_W_BYTES,
                                A.x_b + ((size_t)s * (A.act_rows / 8) + it.pos0 / 8) * kActBRec, x_bytes,
                                &full[slot]);
            }
        }
    } else if (warp == BF_MMA_WARP && lane == 0) {
        // ---------------- MMA thread: 2 terms x 4 K-steps per stage.  In a warp of its own:
        // as a second lane of the copy thread's warp it ran only when that lane's waits
        // let the warp switch paths, and the tensor pipe idled in between.
        uint32_t q = 0, item = 0;
        bool dead = false;
        for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            if (it.nst == 0) continue;
            const uint32_t buf = item & 1;
            const uint32_t idesc = pf_idesc_bf16(kChunkRows, it.n_mma);
            if (!pf_bar_wait(&tempty[buf], ((item >> 1) & 1) ^ 1)) { give_up(); break; }
            pf_fence_after();
            for (int s = 0; s < it.nst && !dead; s++, q++) {
                const uint32_t slot = q % BF_NSTAGE;
                if (!pf_bar_wait(&full[slot], (q / BF_NSTAGE) & 1)) { give_up(); dead = true; break; }
                if (MODE == BF_GATEUP)   // the gathered rows were written by ordinary asynchronous copies
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                pf_fence_after();
                const uint32_t wa = pf_smem(stages + slot * BF_STAGE);
                const uint32_t xa = wa + BF_MC * BF_W_BYTES;
                for (int ch = 0; ch < it.nch; ch++)
#pragma unroll
                    for (int term = 0; term < 2; term++)
#pragma unroll
                        for (int ks = 0; ks < 4; ks++) {
                            // A: the chunk's rows, units 2ks and 2ks+1 (16 bf16 of K): 8-row groups
                            //    128 B apart, the two units 2048 B apart.  B: the tokens' hi or lo
                            //    term, the same units of each record: 8-token groups one record
                            //    apart, the two units 128 B apart (down); the gathered rows of
                            //    gate+up are swizzled tiles, a K-step 32 B further in the row.
                            const uint64_t ad = pf_desc(wa + ch * BF_W_BYTES + 2 * ks * (kChunkRows * 16),
                                                        kChunkRows * 16, 128);
                            const uint64_t bd = MODE == BF_GATEUP
                                                    ? pf_desc_sw128(xa + term * BF_X_TERM + ks * 32)
                                                    : pf_desc(xa + term * kActBLo + 2 * ks * 128, 128, kActBRec);
                            pf_mma_bf16(tmem + buf * BF_TBUF + ch * BF_NT, ad, bd, idesc, (s | term | ks) != 0);
                        }
                pf_commit(&empty[slot]);   // the stage's operands are no longer read
            }
            if (!dead) pf_commit(&tfull[buf]);
            item++;
        }
    } else if (MODE == BF_GATEUP && warp > BF_MMA_WARP) {
        // ---------------- gathering warps: the tile's rows, by token, into the stage.
        // The gathered operand uses the 128-byte swizzle (tcgen05.cuh): one tile of 128 rows
        // x 128 bytes per term.  Warp w owns rows 32w .. 32w+31; eight lanes copy the eight
        // 16-byte pieces of one row and term, so a warp-wide copy reads 128 contiguous
        // bytes of each of four token rows (whole 128-byte requests: 16-byte pieces from
        // eight different rows per request measured half the speed, bound by the L2 tag
        // rate) and writes 512 contiguous bytes of shared memory, the pieces of a row
        // permuted by the swizzle.
        const int gw = warp - (1 + BF_MMA_WARP), r4 = lane >> 3, pc = lane & 7;
        const size_t tok_stride = (size_t)max(A.w.nslices, A.sh.nslices) * kTokBRec;
        uint32_t q = 0;
        bool dead = false;
        for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            if (it.nst == 0) continue;
            const uint8_t* src[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int j = 32 * gw + 4 * i + r4;      // row of the tile
                src[i] = nullptr;
                if (j < it.tc) {
                    const int tok = it.shared ? it.pos0 + j : A.order[it.pos0 + j] / A.k;
                    src[i] = A.tok_b + (size_t)tok * tok_stride + pc * 16;
                }
            }
            for (int s = 0; s < it.nst && !dead; s++, q++) {
                const uint32_t slot = q % BF_NSTAGE;
                if (!pf_bar_wait(&empty[slot], ((q / BF_NSTAGE) & 1) ^ 1)) { give_up(); dead = true; break; }
                const uint32_t xa = pf_smem(stages + slot * BF_STAGE + BF_MC * BF_W_BYTES) + (uint32_t)(32 * gw) * 128;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (!src[i]) continue;
                    const int r = 4 * i + r4;            // row within the warp's 32; r % 8 = row of its atom
                    const uint32_t dp = xa + (uint32_t)r * 128 + (uint32_t)((pc ^ (r & 7)) * 16);
                    const uint8_t* sp = src[i] + (size_t)s * kTokBRec;
                    bf_cp_async16(dp, sp);                               // hi
                    bf_cp_async16(dp + BF_X_TERM, sp + kTokBLo);         // lo
                }
                bf_cp_async_arrive(&full[slot]);
            }
        }
    } else if (warp > 0 && warp <= BF_EPI_WARPS) {
        // ---------------- epilogue warps: once per item.  Warp (quad, cg) reads the 32
        // tensor-memory lanes of its quadrant and, of each chunk's four 32-token column
        // pieces, the pieces cg, cg + BF_CG, ...: with one warp per quadrant each scheduler
        // had a single epilogue warp and nothing to hide its latencies behind, and the
        // epilogue, not the tensor pipe, set the kernel's time.
        const int quad = warp & 3;               // the tensor-memory lanes this warp may read
        const int cg = (warp - 1) >> 2;
        const int row = 32 * quad + lane;        // chunk row = tensor-memory lane
        const uint32_t tlane = tmem + ((uint32_t)(32 * quad) << 16);
        float* xch = s_xchg + cg * (16 * 64);    // [16 tokens][64 rows] of this column group
        uint64_t* xb = xbar + cg;
        uint32_t item = 0, xphase = 0;
        auto meet = [&]() -> bool {   // the four warps of a column group meet (bounded)
            __syncwarp();
            if (lane == 0) pf_bar_arrive(xb);
            const bool ok = pf_bar_wait(xb, xphase);
            xphase ^= 1;
            return ok;
        };
        bool ok = true;
        for (int idx = blockIdx.x; idx < total && ok && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            if (it.nst == 0) continue;
            const uint32_t buf = item & 1;
            if (!pf_bar_wait(&tfull[buf], (item >> 1) & 1)) { ok = false; break; }
            pf_fence_after();
            const int rows = MODE == BF_DOWN ? (it.shared ? A.sh : A.w).rows : 0;
#pragma unroll 1
            for (int ch = 0; ch < it.nch && ok; ch++) {
#pragma unroll 1
                for (int c = cg; c < BF_NT / 32 && ok; c += BF_CG) {
                    const int chunk = it.chunk + ch;
                    int v[32];
                    pf_tmem_ld32(tlane + buf * BF_TBUF + ch * BF_NT + c * 32, v);
                    pf_tmem_wait_ld();
                    if (ch == it.nch - 1 && c + BF_CG >= BF_NT / 32) {   // this warp's last piece is in registers
                        pf_fence_before();
                        __syncwarp();
                        if (lane == 0) pf_bar_arrive(&tempty[buf]);
                    }
                    const int tok0 = c * 32;
                    if (tok0 >= it.tc) continue;     // uniform; the loads above still ran for the hand-back
                    if (MODE == BF_GATEUP) {
                        // Thread `row` of quadrants 0-1 holds gate row `row`, its partner in
                        // quadrants 2-3 the up row of the same output.  The gate thread finishes
                        // tokens 0..15 of the piece, the up thread tokens 16..31, in two rounds
                        // of 8: each hands the other the 8 values it needs through the tile.
                        const int half = quad >> 1;
                        const int orow = row & 63;
                        const int r = chunk * CH + orow;      // row of mid
#pragma unroll
                        for (int rd = 0; rd < 2 && ok; rd++) {
#pragma unroll
                            for (int i = 0; i < 8; i++)
                                xch[(half ? i : 8 + i) * 64 + orow] =
                                    __int_as_float(half ? v[8 * rd + i] : v[16 + 8 * rd + i]);
                            if (!meet()) { ok = false; break; }
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const int tl = 16 * half + 8 * rd + i, tok = tok0 + tl;
                                if (tok >= it.tc) break;          // uniform across the warp
                                const float other = xch[(half ? 8 + i : i) * 64 + orow];
                                const float gt = half ? other : __int_as_float(v[8 * rd + i]);
                                const float u = half ? __int_as_float(v[16 + 8 * rd + i]) : other;
                                // ops.rs:160-167: silu(x) = x * (1 / (1 + exp(-x))); the hardware's
                                // approximate exp2 and reciprocal (about 2^-21 relative) - the
                                // bf16 terms of the operands are ten times coarser
                                const float y = (gt * __fdividef(1.0f, 1.0f + __expf(-gt))) * u;
                                const size_t pos = (size_t)it.pos0 + tok;
                                A.out[((size_t)(r / 64) * A.act_rows + pos) * 64 + r % 64] = y;
                                const __nv_bfloat16 hi = __float2bfloat16_rn(y);
                                const __nv_bfloat16 lo = __float2bfloat16_rn(y - __bfloat162float(hi));
                                uint8_t* rec = A.out_b + ((size_t)(r / 64) * (A.act_rows / 8) + pos / 8) * kActBRec +
                                               act_b_off((int)(pos % 8), r % 64);
                                *(__nv_bfloat16*)rec = hi;
                                *(__nv_bfloat16*)(rec + kActBLo) = lo;
                            }
                            if (!meet()) { ok = false; break; }   // the exchange tile is free again
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            const int tok = tok0 + i;
                            if (tok >= it.tc) break;
                            A.out[((size_t)it.pos0 + tok) * rows + chunk * CH + row] = __int_as_float(v[i]);
                        }
                    }
                }
            }
            item++;
        }
        if (!ok && lane == 0) give_up();
    }
    pf_fence_before();
    __syncthreads();
    pf_fence_after();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                     "r"(BF_TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// host side

template <int MODE>
static cudaError_t launch_bf16_one(const LaunchCfg& c, Bf16Args A) {
    A.chunks = std::max(A.w.chunks, A.sh.chunks);
    static std::atomic<uint64_t> attr_set{0};
    if (cudaError_t e = ensure_dynamic_smem(experts_prefill_bf16_kernel<MODE>, (int)BF_SMEM, attr_set)) return e;
    count_launch();
    return launch_after(c.stream, experts_prefill_bf16_kernel<MODE>, dim3(c.sm_count),
                        dim3(MODE == BF_GATEUP ? BF_THREADS_GATHER : BF_THREADS), BF_SMEM, A);
}

// gate+up then down for the groups the sort put on the prefill tile list
cudaError_t launch_experts_prefill_bf16(const LaunchCfg& c, const DevTiles& gate_up, const DevTiles& down,
                                        const DevTiles& sh_gate_up, const DevTiles& sh_down,
                                        const Workspace& ws) {
    Bf16Args A{};
    A.grp_expert = ws.grp_expert; A.grp_start = ws.grp_start; A.grp_count = ws.grp_count;
    A.ptile_group = ws.ptile_group; A.ptile_t0 = ws.ptile_t0; A.n_ptiles = ws.n_ptiles;
    A.status = ws.status;
    A.n_expert = c.n_expert;
    A.act_rows = ws.act_rows;
    A.tiles_mode = c.only_shared ? 2 : 0;
    Bf16Args G = A;
    G.w = gate_up; G.sh = sh_gate_up;
    G.tok_b = ws.tok_b; G.order = ws.order; G.k = std::max(c.k, 1);
    G.out = ws.mid; G.out_b = ws.mid_b;
    cudaError_t err = launch_bf16_one<BF_GATEUP>(c, G);
    if (err != cudaSuccess) return err;
    Bf16Args D = A;
    D.w = down; D.sh = sh_down;
    D.x_b = ws.mid_b; D.out = ws.pair_out; D.out_b = nullptr;
    return launch_bf16_one<BF_DOWN>(c, D);
}

}  // namespace bivmoe
