// Grouped expert products for prefill-sized groups (Q8_0 weights) on the 5th
// generation tensor cores: tcgen05.mma kind::i8 with the accumulator in tensor
// memory, operands staged in shared memory by bulk copies.
// Reference: the same functions as experts_decode.cu (dense_ffn,
// engine/src/model.rs:1119-1126, over the Q8_0 dot, engine/src/quant.rs:599-607),
// for experts whose token list is long (model.rs:875-889).
//
// Design.  One block per SM, eighteen warps: a warp whose lane 0 issues the copies,
// a warp whose lane 0 issues the MMAs (two lanes of one warp take turns: the MMA
// lane then runs only when the copy lane's waits let the warp switch paths), and
// sixteen epilogue warps (four per tensor-memory lane quadrant, 32 token columns
// each: a thread's accumulators and one drained block fit in 96 registers, and four
// warps per scheduler hide the tensor-memory load latency better than three).  A
// work item is a tile of 128 tokens of one group times a chunk of 128 weight rows
// (64 gate rows with their 64 up rows, or 128 down rows).  The device layouts of common.cuh are already the tensor core's
// canonical K-major operand layouts, so a stage - one K-slice of 256 columns:
// 128 rows x 272 bytes of weights and the 16 activation records of the tile -
// is two bulk copies (cp.async.bulk) and no shuffling.  The reference scales
// every 32-element block dot by its own pair of scales, so the products cannot
// accumulate across blocks inside the tensor core: each block is one MMA
// (M = 128 rows, N = 128 tokens, K = 32) into one of four tensor-memory buffers,
// which the epilogue warps drain (tcgen05.ld), scale by d_w * d_x and add to f32
// accumulators in registers while the next MMA runs.  The int32 values in tensor
// memory are the reference's block dots exactly.  The epilogue is the bottleneck
// by construction - per 32 multiply-adds of the tensor core it converts one
// int32 and does two f32 operations - so it is kept short: the conversion runs
// on the conversion pipe, the scaling two tokens at a time (f32x2) on the FMA
// pipe, and a buffer is handed back to the MMA thread as soon as it is in
// registers.  (Letting the MMA accumulate onto a buffer pre-set to the bits of
// 1.5 * 2^23, so that the int32 read as f32 needs a subtraction instead of a
// conversion, measured slower: re-arming the buffer with tcgen05.st moves
// 177 B/clk/SM at most, which costs more than the conversions.)
// Every wait is bounded; a wait that gives up records BIVMOE_ERR_TIMEOUT, the
// block leaves its loops, frees its tensor memory and returns.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "formats.cuh"
#include "tcgen05.cuh"
#include "launch.cuh"

namespace bivmoe {

constexpr int PF_NT = kPrefillTile;                  // tokens per tile = MMA N
constexpr int PF_EPI_WARPS = 16;                     // four per tensor-memory lane quadrant
constexpr int PF_COLS = PF_NT / (PF_EPI_WARPS / 4);  // token columns per epilogue thread
static_assert(PF_COLS == 32, "an epilogue thread drains one 32-column load per block dot");
constexpr int PF_MMA_WARP = 1 + PF_EPI_WARPS;        // the MMA thread's own warp
constexpr int PF_THREADS = 32 * (2 + PF_EPI_WARPS);  // warp 0: lane 0 copies; the last warp: lane 0 issues MMAs
constexpr int PF_SL = 272;                           // Q8_0: bytes per row per K-slice
constexpr uint32_t PF_W_BYTES = kChunkRows * PF_SL;                // 34816
constexpr uint32_t PF_X_BYTES = (PF_NT / 8) * kActTileBytes;       // 49152
constexpr uint32_t PF_STAGE = PF_W_BYTES + PF_X_BYTES;             // 83968
constexpr uint32_t PF_HEAD = 1024;
constexpr uint32_t PF_XCHG = 64 * PF_NT * 4;                        // SwiGLU exchange, 32 KiB
constexpr uint32_t PF_SMEM = PF_HEAD + 2 * PF_STAGE + PF_XCHG;      // 201728
constexpr uint32_t PF_TMEM_COLS = 512;                              // four buffers, 128 columns apart
constexpr uint32_t PF_TBUF = 4;
constexpr uint32_t PF_TSTRIDE = PF_TMEM_COLS / PF_TBUF;

enum { PF_GATEUP = 0, PF_DOWN = 1 };

struct PrefillArgs {
    DevTiles w, sh;
    const uint8_t* x_t;    // Q8 records of the inputs by position, [K/256][R/8]
    int act_rows;          // R
    float* out;            // GATEUP: mid f32 slice-major; DOWN: pair_out [R][rows]
    uint8_t* out_t;        // GATEUP: Q8 records of mid
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

struct PfItem {
    int shared, expert, chunk, pos0, tc, nst;
    int n_mma;             // tc rounded up to the MMA's N granularity of 16 (ragged last tiles)
    const uint8_t* wsrc;   // stage 0 of the chunk's weights; stage s is s * PF_W_BYTES further
};

template <int MODE>
__global__ void __launch_bounds__(PF_THREADS, 1)
experts_prefill_kernel(const PrefillArgs A) {
    pdl_launch_dependents();
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;            // [2] copies landed
    uint64_t* empty = full + 2;                  // [2] stage free: MMAs done + the epilogue warps
    uint64_t* tfull = full + 16;                 // [4] a block dot is in tensor memory
    uint64_t* tempty = full + 20;                // [4] drained by the epilogue warps
    uint64_t* xbar = full + 8;                   // [1] meeting point of the epilogue warps
    uint32_t* s_tmem = (uint32_t*)(smem + 256);
    int* s_abort = (int*)(smem + 260);
    uint8_t* stages = smem + PF_HEAD;
    float* s_xchg = (float*)(smem + PF_HEAD + 2 * PF_STAGE);   // [128 tokens][64 rows]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int CH = MODE == PF_GATEUP ? 64 : 128;   // output rows per chunk

    if (tid == 0) {
        for (int i = 0; i < 2; i++) {
            pf_bar_init(&full[i], 1);
            pf_bar_init(&empty[i], 1 + PF_EPI_WARPS);
        }
        for (int i = 0; i < (int)PF_TBUF; i++) {
            pf_bar_init(&tfull[i], 1);
            pf_bar_init(&tempty[i], PF_EPI_WARPS);
        }
        pf_bar_init(xbar, PF_EPI_WARPS);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {   // tensor memory: all 512 columns for the whole kernel
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         pf_smem(s_tmem)),
                     "r"(PF_TMEM_COLS)
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
    const int total = (tile_hi - tile_lo) * A.chunks;

    // items are dealt round-robin: every role walks the same sequence on its own
    auto decode = [&](int idx) -> PfItem {
        PfItem it;
        const int tile = tile_lo + idx / A.chunks;
        it.chunk = idx % A.chunks;
        const int gi = A.ptile_group[tile], t0 = A.ptile_t0[tile];
        it.expert = A.grp_expert[gi];
        it.shared = it.expert == A.n_expert;
        it.pos0 = A.grp_start[gi] + t0;
        it.tc = min(PF_NT, A.grp_count[gi] - t0);
        it.n_mma = (it.tc + 15) & ~15;
        const DevTiles& m = it.shared ? A.sh : A.w;
        it.nst = it.chunk < m.chunks ? m.nslices : 0;
        it.wsrc = m.stage(it.shared ? 0 : it.expert, min(it.chunk, max(m.chunks - 1, 0)), 0);
        return it;
    };
    auto give_up = [&]() {
        atomicExch(A.status, BIVMOE_ERR_TIMEOUT);
        atomicExch(s_abort, 1);
    };

    if (warp == 0) {
        // ---------------- copy thread: two bulk copies per stage
        if (lane == 0) {
            uint32_t q = 0;
            bool dead = false;
            for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
                const PfItem it = decode(idx);
                for (int s = 0; s < it.nst && !dead; s++, q++) {
                    const uint32_t slot = q & 1;
                    if (!pf_bar_wait(&empty[slot], ((q >> 1) & 1) ^ 1)) { give_up(); dead = true; break; }
                    uint8_t* dst = stages + slot * PF_STAGE;
                    const uint32_t x_bytes = (uint32_t)(it.n_mma / 8) * kActTileBytes;
                    pf_bar_expect_tx(&full[slot], PF_W_BYTES + x_bytes);
                    pf_bulk_g2s(dst, it.wsrc + (size_t)s * PF_W_BYTES, PF_W_BYTES, &full[slot]);
                    pf_bulk_g2s(dst + PF_W_BYTES,
                                A.x_t + ((size_t)s * (A.act_rows / 8) + it.pos0 / 8) * kActTileBytes,
                                x_bytes, &full[slot]);
                }
            }
        }
    } else if (warp == PF_MMA_WARP) {
        // ---------------- MMA thread: one MMA per 32-column block.  In a warp of its own:
        // as a second lane of the copy thread's warp it ran only when that lane's waits
        // let the warp switch paths.
        if (lane == 0) {
            uint32_t q = 0, kb = 0;
            bool dead = false;
            for (int idx = blockIdx.x; idx < total && !dead && !*(volatile int*)s_abort; idx += gridDim.x) {
                const PfItem it = decode(idx);
                const uint32_t idesc = pf_idesc(kChunkRows, it.n_mma);
                for (int s = 0; s < it.nst && !dead; s++, q++) {
                    const uint32_t slot = q & 1;
                    if (!pf_bar_wait(&full[slot], (q >> 1) & 1)) { give_up(); dead = true; break; }
                    const uint32_t wa = pf_smem(stages + slot * PF_STAGE);
                    const uint32_t xa = wa + PF_W_BYTES;
                    for (int b = 0; b < 8 && !dead; b++, kb++) {
                        const uint32_t buf = kb % PF_TBUF;
                        if (!pf_bar_wait(&tempty[buf], ((kb / PF_TBUF) & 1) ^ 1)) { give_up(); dead = true; break; }
                        pf_fence_after();
                        // A: rows of the chunk, units 2b and 2b+1: 8-row groups 128 B apart,
                        //    K steps 2048 B apart.  B: tokens, units 2b, 2b+1 of each record:
                        //    8-token groups one record apart, K steps 128 B apart.
                        const uint64_t ad = pf_desc(wa + 2 * b * (kChunkRows * 16), kChunkRows * 16, 128);
                        const uint64_t bd = pf_desc(xa + 2 * b * 128, 128, kActTileBytes);
                        pf_mma_i8(tmem + buf * PF_TSTRIDE, ad, bd, idesc);
                        pf_commit(&tfull[buf]);
                    }
                    if (!dead) pf_commit(&empty[slot]);   // the stage's operands are no longer read
                }
            }
        }
    } else {
        // ---------------- epilogue warps
        const int ew = warp - 1;                 // 0..11
        const int quad = warp & 3;               // the tensor-memory lanes this warp may read
        const int cg = ew >> 2;                  // which 32 of the 128 token columns
        const int row = 32 * quad + lane;        // chunk row = tensor-memory lane
        const uint32_t tlane = tmem + ((uint32_t)(32 * quad) << 16) + cg * PF_COLS;
        uint32_t q = 0, kb = 0, xphase = 0;
        // the epilogue warps meet (bounded): false when the wait gave up
        auto meet = [&]() -> bool {
            __syncwarp();
            if (lane == 0) pf_bar_arrive(xbar);
            const bool ok = pf_bar_wait(xbar, xphase);
            xphase ^= 1;
            return ok;
        };
        for (int idx = blockIdx.x; idx < total && !*(volatile int*)s_abort; idx += gridDim.x) {
            const PfItem it = decode(idx);
            f32x2 acc[PF_COLS / 2];   // tokens cg*32 + 2i, 2i+1
#pragma unroll
            for (int i = 0; i < PF_COLS / 2; i++) acc[i] = 0ull;
            bool ok = true;
            for (int s = 0; s < it.nst && ok; s++, q++) {
                const uint32_t slot = q & 1;
                if (!pf_bar_wait(&full[slot], (q >> 1) & 1)) { ok = false; break; }
                const uint8_t* wst = stages + slot * PF_STAGE;
                const uint8_t* xst = wst + PF_W_BYTES + (cg * (PF_COLS / 8)) * kActTileBytes + kActOffDx;
                const uint4 dwv = *(const uint4*)(wst + 16 * (kChunkRows * 16) + row * 16);   // 8 f16 scales
                for (int b = 0; b < 8 && ok; b++, kb++) {
                    const uint32_t buf = kb % PF_TBUF;
                    if (!pf_bar_wait(&tfull[buf], (kb / PF_TBUF) & 1)) { ok = false; break; }
                    pf_fence_after();
                    // drain this warp's 32 columns and hand the buffer back (a warp whose
                    // columns lie past the end of a ragged tile only hands back)
                    int v[32];
                    pf_tmem_ld32(tlane + buf * PF_TSTRIDE, v);
                    pf_tmem_wait_ld();
                    pf_fence_before();
                    __syncwarp();
                    if (lane == 0) pf_bar_arrive(&tempty[buf]);
                    const uint32_t wv = (b & 4) ? ((b & 2) ? dwv.w : dwv.z) : ((b & 2) ? dwv.y : dwv.x);
                    const float dw = __half2float(__ushort_as_half((unsigned short)(wv >> (16 * (b & 1)))));
                    const f32x2 dw2 = pk(dw, dw);
#pragma unroll
                    for (int j = 0; j < 4; j++) {   // a record: 8 tokens, their d_x of block b
                        const ulonglong2* dxp = (const ulonglong2*)(xst + j * kActTileBytes + b * 32);
                        const ulonglong2 d01 = dxp[0], d23 = dxp[1];
                        const f32x2 dxs[4] = {d01.x, d01.y, d23.x, d23.y};
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            const int i = j * 4 + t;
                            // the int32 block dots, exact as floats (below 2^24)
                            const f32x2 f = pk(__int2float_rn(v[2 * i]), __int2float_rn(v[2 * i + 1]));
                            acc[i] = fma2(dw2, mul2(dxs[t], f), acc[i]);
                        }
                    }
                }
                if (ok) {
                    __syncwarp();
                    if (lane == 0) pf_bar_arrive(&empty[slot]);   // done with the stage's scales
                }
            }
            if (!ok) { if (lane == 0) give_up(); break; }
            if (it.nst == 0) continue;
            // ---- the item's outputs: column i of this thread is token cg*32 + i
            auto accf = [&](int i) -> float {   // column i of this thread
                const f32x2 p = acc[i >> 1];
                return __uint_as_float((uint32_t)((i & 1) ? p >> 32 : p));
            };
            if (MODE == PF_GATEUP) {
                // Thread (row, cg) of quadrants 0-1 holds gate row `row`, its partner in
                // quadrants 2-3 the up row of the same output, for the same 32 tokens.
                // Each finishes half of the tokens: the gate thread hands over its gate
                // values of tokens 16..31, the up thread its up values of tokens 0..15.
                const int half = quad >> 1;              // 0: gate rows, finishes tokens 0..15
                const int orow = row & 63;               // output row within the chunk
#pragma unroll
                for (int i = 0; i < 16; i++)
                    s_xchg[(cg * PF_COLS + (half ? i : 16 + i)) * 64 + orow] = accf(half ? i : 16 + i);
                if (!meet()) { if (lane == 0) give_up(); break; }
                {
                    const int r = it.chunk * CH + orow;   // row of mid
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int tok = cg * PF_COLS + 16 * half + i;
                        if (tok >= it.tc) break;          // uniform across the warp
                        const float other = s_xchg[tok * 64 + orow];
                        const float gt = half ? other : accf(i);
                        const float u = half ? accf(16 + i) : other;
                        // ops.rs:160-167: silu(x) = x * (1 / (1 + exp(-x)))
                        const float v = (gt * __fdiv_rn(1.0f, 1.0f + expf(-gt))) * u;
                        const size_t pos = (size_t)it.pos0 + tok;
                        A.out[((size_t)(r / 64) * A.act_rows + pos) * 64 + r % 64] = v;
                        // Q8Act of the mid row (quant.rs:368-394): the warp's 32 rows are one block
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
                if (!meet()) { if (lane == 0) give_up(); break; }   // the exchange tile is free again
            } else {
                const int rows = (it.shared ? A.sh : A.w).rows;
#pragma unroll
                for (int i = 0; i < PF_COLS; i++) {
                    const int tok = cg * PF_COLS + i;
                    if (tok >= it.tc) break;
                    A.out[((size_t)it.pos0 + tok) * rows + it.chunk * CH + row] = accf(i);
                }
            }
        }
    }
    pf_fence_before();
    __syncthreads();
    pf_fence_after();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                     "r"(PF_TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// host side

bool prefill_supported(int gate_up_ty, int down_ty) {
    return (gate_up_ty == BIVMOE_Q8_0 && down_ty == BIVMOE_Q8_0) ||
           (gate_up_ty == BIVMOE_BF16 && down_ty == BIVMOE_BF16);
}

template <int MODE>
static cudaError_t launch_prefill_one(const LaunchCfg& c, PrefillArgs A) {
    A.chunks = std::max(A.w.chunks, A.sh.chunks);
    static std::atomic<uint64_t> attr_set{0};
    if (cudaError_t e = ensure_dynamic_smem(experts_prefill_kernel<MODE>, (int)PF_SMEM, attr_set)) return e;
    count_launch();
    return launch_after(c.stream, experts_prefill_kernel<MODE>, dim3(c.sm_count), dim3(PF_THREADS), PF_SMEM, A);
}

// gate+up then down for the groups the sort put on the prefill tile list
cudaError_t launch_experts_prefill(const LaunchCfg& c, const DevTiles& gate_up, const DevTiles& down,
                                   const DevTiles& sh_gate_up, const DevTiles& sh_down,
                                   const Workspace& ws) {
    const int ty = c.only_shared ? sh_gate_up.ty : gate_up.ty;
    if (ty == BIVMOE_BF16) return launch_experts_prefill_bf16(c, gate_up, down, sh_gate_up, sh_down, ws);
    PrefillArgs A{};
    A.grp_expert = ws.grp_expert; A.grp_start = ws.grp_start; A.grp_count = ws.grp_count;
    A.ptile_group = ws.ptile_group; A.ptile_t0 = ws.ptile_t0; A.n_ptiles = ws.n_ptiles;
    A.status = ws.status;
    A.n_expert = c.n_expert;
    A.act_rows = ws.act_rows;
    A.tiles_mode = c.only_shared ? 2 : 0;
    PrefillArgs G = A;
    G.w = gate_up; G.sh = sh_gate_up;
    G.x_t = ws.act_t; G.out = ws.mid; G.out_t = ws.mid_t;
    cudaError_t err = launch_prefill_one<PF_GATEUP>(c, G);
    if (err != cudaSuccess) return err;
    PrefillArgs D = A;
    D.w = down; D.sh = sh_down;
    D.x_t = ws.mid_t; D.out = ws.pair_out; D.out_t = nullptr;
    return launch_prefill_one<PF_DOWN>(c, D);
}

}  // namespace bivmoe

// ---------------------------------------------------------------------------
// The int8 tensor-pipe peak of this GPU, measured: no int8 figure comes with the
// machine's measured peaks, so the Q8_0 kernel's roofline denominator is taken here.
// One block per SM issues back-to-back tcgen05.mma kind::i8 (M 128, N 256, K 32) from
// one thread, alternating between two tensor-memory accumulators, on operands that stay
// in shared memory; nothing is loaded or drained, so this is the pipe alone.
namespace bivmoe {

constexpr uint32_t PEAK_SMEM = 1024 + 128 * 32 + 256 * 32;   // descriptors' operands: A 4 KiB, B 8 KiB

__global__ void __launch_bounds__(128, 1) int8_peak_kernel(int mmas, int32_t* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* done = (uint64_t*)smem;
    uint32_t* s_tmem = (uint32_t*)(smem + 64);
    const int tid = threadIdx.x, warp = tid >> 5;
    for (uint32_t i = tid; i < (PEAK_SMEM - 1024) / 4; i += blockDim.x) ((uint32_t*)(smem + 1024))[i] = 0x01010101u;
    if (tid == 0) {
        pf_bar_init(done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the operands, for the tensor core
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         pf_smem(s_tmem)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pf_fence_before();
    __syncthreads();
    pf_fence_after();
    const uint32_t tmem = *s_tmem;
    if (tid == 0) {
        const uint32_t a = pf_smem(smem + 1024), b = a + 128 * 32;
        // K-major, two 16-byte K units: rows 16 bytes apart inside an 8-row group
        const uint64_t ad = pf_desc(a, 128 * 16, 128), bd = pf_desc(b, 256 * 16, 128);
        const uint32_t idesc = pf_idesc(128, 256);
        for (int i = 0; i < mmas; i++) pf_mma_i8(tmem + (i & 1) * 256, ad, bd, idesc);
        pf_commit(done);
        if (!pf_bar_wait(done, 0)) atomicExch(status, BIVMOE_ERR_TIMEOUT);
    }
    pf_fence_before();
    __syncthreads();
    pf_fence_after();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u)
                     : "memory");
    }
}

// tera-operations per second (2 per multiply-add) over all SMs; `status_dev`: a device
// word that a bounded wait flags
cudaError_t measure_int8_peak(int sm_count, int32_t* status_dev, cudaStream_t stream, double* tops) {
    static std::atomic<uint64_t> attr_set{0};
    if (cudaError_t e = ensure_dynamic_smem(int8_peak_kernel, (int)PEAK_SMEM, attr_set)) return e;
    const int mmas = 1 << 15;
    cudaEvent_t e0, e1;
    cudaError_t err = cudaEventCreate(&e0);
    if (err != cudaSuccess) return err;
    err = cudaEventCreate(&e1);
    if (err != cudaSuccess) { cudaEventDestroy(e0); return err; }
    int8_peak_kernel<<<sm_count, 128, PEAK_SMEM, stream>>>(1 << 10, status_dev);   // warm-up
    cudaEventRecord(e0, stream);
    int8_peak_kernel<<<sm_count, 128, PEAK_SMEM, stream>>>(mmas, status_dev);
    cudaEventRecord(e1, stream);
    err = cudaEventSynchronize(e1);
    float ms = 0.0f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (err != cudaSuccess) return err;
    *tops = 2.0 * 128 * 256 * 32 * (double)mmas * sm_count / (ms * 1e-3) / 1e12;
    return cudaGetLastError();
}

}  // namespace bivmoe
