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
// Design.  Two kernels, one block per SM each: one thread of warp 0 issues the bulk
// copies, one thread of a warp of its own the MMAs, sixteen epilogue warps (four per
// tensor-memory lane quadrant) drain the accumulators.  A work item is a tile of up
// to 128 tokens of one group times TWO chunks of 128 weight rows (a chunk: 64 gate
// rows with their 64 up rows, or 128 down rows); a pipeline stage is one K-slice of
// 64 values of both chunks' weights (32 KB) and of the tile's two activation terms
// (32 KB), three stages in flight; the products of an item accumulate across the
// whole K in one of two 256-column tensor-memory buffers, so that the epilogue of an
// item - which runs once per item, nothing being scaled per block - overlaps the
// MMAs of the next.
//   down     the chunk's 128 rows are the MMA's M, the tile's tokens its N (sized to
//            the tile, a multiple of 16); the records of mid, written by the gate+up
//            epilogue in the canonical K-major layout (common.cuh), and the weights
//            arrive by bulk copies; a thread of the epilogue owns an output row and
//            a warp stores 32 consecutive rows of one token.
//   gate+up  the tile's tokens are M, the 256 rows of both chunks N: one MMA per term
//            and K-step reads 4 KB + 8 KB of shared memory where two MMAs with the
//            rows as M read 16 KB.  Four more warps gather the tile's rows by token
//            from the token-ordered bf16 terms (rowops.cu, split_rows_kernel) with
//            16-byte asynchronous copies that complete on the stage's barrier: a row is
//            split once and never written per position.  A thread of the epilogue owns
//            a token and finds gate and up of an output row in its own lane.
// What bounds them (measured with loads, MMAs or epilogue switched off in throw-away
// builds): all three at once - a stage's 64 KB is what an SM pulls from L2 in the
// 1024 cycles its MMAs take, the fills and the MMAs' operand reads share the
// shared-memory bandwidth, and the epilogue's stores share the SM with both.  Every
// wait is bounded; a wait that gives up records BIVMOE_ERR_TIMEOUT, the block leaves
// its loops, frees its tensor memory and returns.
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
constexpr uint32_t BF_W_BYTES = kChunkRows * 128;               // 16384: one K-slice of a chunk
constexpr uint32_t BF_X_BYTES = (BF_NT / 8) * kActBRec;         // 32768
constexpr uint32_t BF_X_TERM = BF_NT * 128;                     // gathered rows: the lo tile follows the hi tile
constexpr int BF_MC = 2;                                        // chunks per item
constexpr uint32_t BF_STAGE = BF_MC * BF_W_BYTES + BF_X_BYTES;  // 65536
constexpr int BF_NSTAGE = 3;
constexpr uint32_t BF_HEAD = 1024;
constexpr uint32_t BF_SMEM = BF_HEAD + BF_NSTAGE * BF_STAGE;    // 197632
constexpr uint32_t BF_TMEM_COLS = 512;                          // two buffers of 2 x 128 columns
constexpr uint32_t BF_TBUF = BF_MC * BF_NT;                     // columns of one buffer

struct Bf16Args {
    DevTiles w, sh;
    const uint8_t* x_b;    // DOWN: bf16 hi/lo records of mid by position, [K/64][R/8]
    const uint8_t* tok_b;  // GATEUP: bf16 hi/lo terms of the rows by token, [N][K/64][kTokBRec]
    const int32_t* order;  // GATEUP: order[pos] / k is the token at a routed group's position
    int k;
    int act_rows;          // R
    float* out;            // DOWN: pair_out [R][rows]
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

// ---------------------------------------------------------------------------
// down: the 128 rows of a chunk are the MMA's M (tensor-memory lanes), the tile's tokens
// its N, sized to the tile; both operands arrive by bulk copies
__global__ void __launch_bounds__(BF_THREADS, 1)
experts_prefill_bf16_down_kernel(const Bf16Args A) {
    pdl_launch_dependents();
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;            // [3] copies landed
    uint64_t* empty = full + 4;                  // [3] stage free: its MMAs are done
    uint64_t* tfull = full + 8;                  // [2] an item's products are in tensor memory
    uint64_t* tempty = full + 10;                // [2] drained by the epilogue warps
    uint32_t* s_tmem = (uint32_t*)(smem + 256);
    int* s_abort = (int*)(smem + 260);
    uint8_t* stages = smem + BF_HEAD;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int CH = kChunkRows;               // output rows per chunk

    if (tid == 0) {
        for (int i = 0; i < BF_NSTAGE; i++) {
            pf_bar_init(&full[i], 1);
            pf_bar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            pf_bar_init(&tfull[i], 1);
            pf_bar_init(&tempty[i], BF_EPI_WARPS);
        }
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
                const uint32_t x_bytes = (uint32_t)(it.n_mma / 8) * kActBRec;
                pf_bar_expect_tx(&full[slot], it.nch * BF_W_BYTES + x_bytes);
                for (int ch = 0; ch < it.nch; ch++)
                    pf_bulk_g2s(dst + ch * BF_W_BYTES, it.wsrc + ch * it.wstep + (size_t)s * BF_W_BYTES,
                                BF_W_BYTES, &full[slot]);
                pf_bulk_g2s(dst + BF_MC * BF_W_BYTES,
                            A.x_b + ((size_t)s * (A.act_rows / 8) + it.pos0 / 8) * kActBRec, x_bytes, &full[slot]);
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
                            //    apart, the two units 128 B apart.
                            const uint64_t ad = pf_desc(wa + ch * BF_W_BYTES + 2 * ks * (kChunkRows * 16),
                                                        kChunkRows * 16, 128);
                            const uint64_t bd = pf_desc(xa + term * kActBLo + 2 * ks * 128, 128, kActBRec);
                            pf_mma_bf16(tmem + buf * BF_TBUF + ch * BF_NT, ad, bd, idesc, (s | term | ks) != 0);
                        }
                pf_commit(&empty[slot]);   // the stage's operands are no longer read
            }
            if (!dead) pf_commit(&tfull[buf]);
            item++;
        }
    } else if (warp > 0 && warp <= BF_EPI_WARPS) {
        // ---------------- epilogue warps: once per item.  Warp (quad, cg) reads the 32
        // tensor-memory lanes of its quadrant and, of each chunk's four 32-token column
        // pieces, the pieces cg, cg + BF_CG, ...: with one warp per quadrant each scheduler
        // had a single epilogue warp and nothing to hide its latencies behind.
        const int quad = warp & 3;               // the tensor-memory lanes this warp may read
        const int cg = (warp - 1) >> 2;
        const int row = 32 * quad + lane;        // chunk row = tensor-memory lane
        const uint32_t tlane = tmem + ((uint32_t)(32 * quad) << 16);
        uint32_t item = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < total && ok && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            if (it.nst == 0) continue;
            const uint32_t buf = item & 1;
            if (!pf_bar_wait(&tfull[buf], (item >> 1) & 1)) { ok = false; break; }
            pf_fence_after();
            const int rows = (it.shared ? A.sh : A.w).rows;
#pragma unroll 1
            for (int ch = 0; ch < it.nch; ch++) {
#pragma unroll 1
                for (int c = cg; c < BF_NT / 32; c += BF_CG) {
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
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int tok = tok0 + i;
                        if (tok >= it.tc) break;
                        A.out[((size_t)it.pos0 + tok) * rows + chunk * CH + row] = __int_as_float(v[i]);
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
// gate+up with the operands' roles exchanged: the tile's 128 tokens are the MMA's M
// (tensor-memory lanes), the 256 weight rows of two chunks its N (columns).  One MMA per
// term and K-step then reads 4 KB of tokens + 8 KB of weights for 128 cycles of the
// tensor pipe, where two MMAs with the rows as M read 16 KB: the kernel is bound by
// shared-memory bandwidth (operand reads + the stage fills), not by the pipe.  A thread of
// the epilogue owns a token and finds gate and up of an output row in its own lane, so
// SwiGLU needs no exchange, and it stores 16 consecutive rows of its token at a time.
constexpr int GU_EPI_WARPS = 16;                                  // 4 per lane quadrant: 16 output rows of a chunk each
constexpr int GU_MMA_WARP = 1 + GU_EPI_WARPS;
constexpr int GU_THREADS = 32 * (2 + GU_EPI_WARPS + BF_GATHER_WARPS);
constexpr uint32_t GU_UNIT = BF_MC * kChunkRows * 16;             // 4096: one 16-byte K unit of the 256 rows
constexpr uint32_t GU_SMEM = BF_HEAD + BF_NSTAGE * BF_STAGE;      // 197632

__global__ void __launch_bounds__(GU_THREADS, 1)
experts_prefill_bf16_gateup_kernel(const Bf16Args A) {
    pdl_launch_dependents();
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;            // [3] copies landed
    uint64_t* empty = full + 4;                  // [3] stage free: its MMAs are done
    uint64_t* tfull = full + 8;                  // [2] an item's products are in tensor memory
    uint64_t* tempty = full + 10;                // [2] drained by the epilogue warps
    uint32_t* s_tmem = (uint32_t*)(smem + 256);
    int* s_abort = (int*)(smem + 260);
    uint8_t* stages = smem + BF_HEAD;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int i = 0; i < BF_NSTAGE; i++) {
            // the copy thread's arrival with the bulk copies' bytes + every gathering thread
            pf_bar_init(&full[i], 1 + 32 * BF_GATHER_WARPS);
            pf_bar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            pf_bar_init(&tfull[i], 1);
            pf_bar_init(&tempty[i], GU_EPI_WARPS);
        }
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
    pdl_wait();   // the tile lists and the token terms are the previous kernels'

    const int tiles_all = A.n_ptiles[0], tiles_sh = A.n_ptiles[1];
    const int tile_lo = A.tiles_mode == 1 ? tiles_sh : 0;
    const int tile_hi = A.tiles_mode == 2 ? tiles_sh : tiles_all;
    const int cpairs = (A.chunks + BF_MC - 1) / BF_MC;
    const int total = (tile_hi - tile_lo) * cpairs;

    auto decode = [&](int idx) -> BfItem {
        BfItem it;
        const int tile = tile_lo + idx / cpairs;
        it.chunk = (idx % cpairs) * BF_MC;
        const int gi = A.ptile_group[tile], t0 = A.ptile_t0[tile];
        it.expert = A.grp_expert[gi];
        it.shared = it.expert == A.n_expert;
        it.pos0 = A.grp_start[gi] + t0;
        it.tc = min(BF_NT, A.grp_count[gi] - t0);
        it.n_mma = BF_NT;
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
        // ---------------- copy thread: the K-slice of each chunk, its eight 16-byte K units
        // placed so that the 256 rows of a unit are contiguous (the MMA's N runs over both chunks)
        uint32_t q = 0;
        bool dead = false;
        for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            for (int s = 0; s < it.nst && !dead; s++, q++) {
                const uint32_t slot = q % BF_NSTAGE;
                if (!pf_bar_wait(&empty[slot], ((q / BF_NSTAGE) & 1) ^ 1)) { give_up(); dead = true; break; }
                uint8_t* dst = stages + slot * BF_STAGE;
                pf_bar_expect_tx(&full[slot], it.nch * BF_W_BYTES);
                for (int ch = 0; ch < it.nch; ch++) {
                    const uint8_t* src = it.wsrc + ch * it.wstep + (size_t)s * BF_W_BYTES;
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        pf_bulk_g2s(dst + u * GU_UNIT + ch * (kChunkRows * 16), src + u * (kChunkRows * 16),
                                    kChunkRows * 16, &full[slot]);
                }
            }
        }
    } else if (warp == GU_MMA_WARP && lane == 0) {
        // ---------------- MMA thread: 2 terms x 4 K-steps per stage
        uint32_t q = 0, item = 0;
        bool dead = false;
        for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            if (it.nst == 0) continue;
            const uint32_t buf = item & 1;
            const uint32_t idesc = pf_idesc_bf16(BF_NT, it.nch * kChunkRows);
            if (!pf_bar_wait(&tempty[buf], ((item >> 1) & 1) ^ 1)) { give_up(); break; }
            pf_fence_after();
            for (int s = 0; s < it.nst && !dead; s++, q++) {
                const uint32_t slot = q % BF_NSTAGE;
                if (!pf_bar_wait(&full[slot], (q / BF_NSTAGE) & 1)) { give_up(); dead = true; break; }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the gathered rows
                pf_fence_after();
                const uint32_t wb = pf_smem(stages + slot * BF_STAGE);
                const uint32_t xa = wb + BF_MC * BF_W_BYTES;
#pragma unroll
                for (int term = 0; term < 2; term++)
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        // A: the tokens' hi or lo term, a swizzled tile, a K-step 32 B further in
                        //    the row.  B: the rows of both chunks, units 2ks and 2ks+1: 8-row
                        //    groups 128 B apart, the two units GU_UNIT apart.
                        const uint64_t ad = pf_desc_sw128(xa + term * BF_X_TERM + ks * 32);
                        const uint64_t bd = pf_desc(wb + 2 * ks * GU_UNIT, GU_UNIT, 128);
                        pf_mma_bf16(tmem + buf * BF_TBUF, ad, bd, idesc, (s | term | ks) != 0);
                    }
                pf_commit(&empty[slot]);   // the stage's operands are no longer read
            }
            if (!dead) pf_commit(&tfull[buf]);
            item++;
        }
    } else if (warp > GU_MMA_WARP) {
        // ---------------- gathering warps: the tile's rows, by token, into the stage: one
        // tile of 128 rows x 128 bytes per term in the 128-byte swizzle (tcgen05.cuh).  Warp w
        // owns rows 32w .. 32w+31; eight lanes copy the eight 16-byte pieces of one row and
        // term, so a warp-wide copy reads 128 contiguous bytes of each of four token rows
        // (whole 128-byte requests: 16-byte pieces from eight different rows per request
        // measured half the speed, bound by the L2 tag rate) and writes 512 contiguous bytes
        // of shared memory, the pieces of a row permuted by the swizzle.
        const int gw = warp - (1 + GU_MMA_WARP), r4 = lane >> 3, pc = lane & 7;
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
    } else if (warp > 0 && warp <= GU_EPI_WARPS) {
        // ---------------- epilogue warps: once per item.  Warp (quad, cg): the 32 tokens of
        // its lane quadrant, output rows 16cg .. 16cg+15 of each chunk - their gate products
        // in columns 16cg.. of the chunk's 128, their up products 64 columns further.
        const int quad = warp & 3;               // the tensor-memory lanes this warp may read
        const int cg = (warp - 1) >> 2;
        const int j = 32 * quad + lane;          // the thread's token: row of the tile = tensor-memory lane
        const uint32_t tlane = tmem + ((uint32_t)(32 * quad) << 16);
        uint32_t item = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < total && ok && !*(volatile int*)s_abort; idx += gridDim.x) {
            const BfItem it = decode(idx);
            if (it.nst == 0) continue;
            const uint32_t buf = item & 1;
            if (!pf_bar_wait(&tfull[buf], (item >> 1) & 1)) { ok = false; break; }
            pf_fence_after();
            const size_t pos = (size_t)it.pos0 + j;
#pragma unroll 1
            for (int ch = 0; ch < it.nch; ch++) {
                int g[16], u[16];
                pf_tmem_ld16(tlane + buf * BF_TBUF + ch * kChunkRows + 16 * cg, g);
                pf_tmem_ld16(tlane + buf * BF_TBUF + ch * kChunkRows + 64 + 16 * cg, u);
                pf_tmem_wait_ld();
                if (ch == it.nch - 1) {          // this warp's last columns are in registers
                    pf_fence_before();
                    __syncwarp();
                    if (lane == 0) pf_bar_arrive(&tempty[buf]);
                }
                if (j >= it.tc) continue;
                float y[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float gt = __int_as_float(g[i]);
                    // ops.rs:160-167: silu(x) = x * (1 / (1 + exp(-x))); the hardware's
                    // approximate exp2 and reciprocal (about 2^-21 relative) - the bf16 terms
                    // of the operands are ten times coarser
                    y[i] = (gt * __fdividef(1.0f, 1.0f + __expf(-gt))) * __int_as_float(u[i]);
                }
                const int chunk = it.chunk + ch;   // rows 64 chunk + 16cg .. of mid: K-slice `chunk` of the down product
                // (no f32 copy of mid for these groups: the down product reads the two terms,
                //  and the tap of mid adds them up)
                uint8_t* rec = A.out_b + ((size_t)chunk * (A.act_rows / 8) + pos / 8) * kActBRec +
                               act_b_off((int)(pos % 8), 16 * cg);
#pragma unroll
                for (int un = 0; un < 2; un++) {   // two 16-byte units of 8 rows, 128 bytes apart
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const float a = y[8 * un + 2 * p], b = y[8 * un + 2 * p + 1];
                        const __nv_bfloat16 h0 = __float2bfloat16_rn(a), h1 = __float2bfloat16_rn(b);
                        const __nv_bfloat16 l0 = __float2bfloat16_rn(a - __bfloat162float(h0));
                        const __nv_bfloat16 l1 = __float2bfloat16_rn(b - __bfloat162float(h1));
                        hi[p] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
                        lo[p] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
                    }
                    *(uint4*)(rec + un * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *(uint4*)(rec + un * 128 + kActBLo) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
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
    G.chunks = std::max(G.w.chunks, G.sh.chunks);
    static std::atomic<uint64_t> gu_attr{0}, down_attr{0};
    if (cudaError_t e = ensure_dynamic_smem(experts_prefill_bf16_gateup_kernel, (int)GU_SMEM, gu_attr)) return e;
    count_launch();
    if (cudaError_t e = launch_after(c.stream, experts_prefill_bf16_gateup_kernel, dim3(c.sm_count), dim3(GU_THREADS),
                                     GU_SMEM, G))
        return e;
    Bf16Args D = A;
    D.w = down; D.sh = sh_down;
    D.x_b = ws.mid_b; D.out = ws.pair_out; D.out_b = nullptr;
    D.chunks = std::max(D.w.chunks, D.sh.chunks);
    if (cudaError_t e = ensure_dynamic_smem(experts_prefill_bf16_down_kernel, (int)BF_SMEM, down_attr)) return e;
    count_launch();
    return launch_after(c.stream, experts_prefill_bf16_down_kernel, dim3(c.sm_count), dim3(BF_THREADS), BF_SMEM, D);
}

}  // namespace bivmoe
