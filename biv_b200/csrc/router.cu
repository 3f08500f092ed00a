// Router product, softmax / top-k / renormalisation, and the stable
// token-to-expert sort.  Reference: engine/src/model.rs:259-268 (route),
// 864-873 (logits and per-expert lists), engine/src/ops.rs:192-201 (softmax),
// engine/src/quant.rs:1177-1206 (the AVX2 f32 dot whose summation order the
// logits kernel reproduces bit for bit).
#include "common.cuh"
#include "launch.cuh"
#include "tcgen05.cuh"

namespace bivmoe {

// ---------------------------------------------------------------------------
// logits[t][r] = dot(W[r], h[t]) for the n_expert router rows plus, as row
// n_expert, the shared expert's gate vector.
//
// The reference's x86 dot keeps 4 accumulators of 8 lanes: element i goes to
// lane (i mod 32) of a 32-wide accumulator set, with one fused multiply-add per
// element in ascending i, and the 32 lanes are then summed as
// (k0+k1)+(k2+k3) per lane j (lane = 8k+j), then j with j+4, j+2, j+1.  A warp
// lane per accumulator lane and the butterfly 8,16,4,2,1 give the same bits.
constexpr int RT_ROWS = 4, RT_TOKS = 4;          // register tile of one warp
constexpr int RT_BROWS = 8, RT_BTOKS = 16;       // rows and tokens of one block (8 warps)
constexpr int RT_THREADS = 256;
constexpr uint32_t RT_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t rt_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// The block's 8 weight rows and 16 activation rows are brought into shared memory
// with one bulk copy each, all in flight together, so the kernel pays one memory
// round trip instead of one per step of the dot.
__global__ void __launch_bounds__(RT_THREADS, 1)
router_logits_kernel(const float* __restrict__ W, const float* __restrict__ h,
                     float* __restrict__ logits, int n, int e, int n_rows, int* status,
                     const float* __restrict__ norm_w, float norm_eps, float* __restrict__ row_scale) {
    pdl_enter();
    extern __shared__ __align__(128) uint8_t rt_smem[];
    uint64_t* bar = (uint64_t*)rt_smem;
    float* s_w = (float*)(rt_smem + 128);              // [RT_BROWS][e]
    float* s_x = s_w + (size_t)RT_BROWS * e;           // [RT_BTOKS][e]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int br0 = blockIdx.x * RT_BROWS, bt0 = blockIdx.y * RT_BTOKS;
    const uint32_t row_bytes = (uint32_t)e * 4;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rt_smem_u32(bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rt_smem_u32(bar)),
                         "r"(row_bytes * (RT_BROWS + RT_BTOKS))
                         : "memory");
        __syncwarp();
        if (lane < RT_BROWS + RT_BTOKS) {   // rows past the end repeat the last one; never stored
            const float* src = lane < RT_BROWS ? W + (size_t)min(br0 + lane, n_rows - 1) * e
                                               : h + (size_t)min(bt0 + lane - RT_BROWS, n - 1) * e;
            float* dst = lane < RT_BROWS ? s_w + (size_t)lane * e : s_x + (size_t)(lane - RT_BROWS) * e;
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                    "r"(rt_smem_u32(dst)),
                "l"(src), "r"(row_bytes), "r"(rt_smem_u32(bar))
                : "memory");
        }
    }
    bool ok = false;
    for (uint32_t i = 0; i < RT_WAIT_LIMIT && !ok; i++) {
        uint32_t p;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(p)
            : "r"(rt_smem_u32(bar))
            : "memory");
        ok = p != 0;
    }
    if (!ok) {   // bounded wait gave up: every thread waits on the same barrier
        if (threadIdx.x == 0) atomicExch(status, BIVMOE_ERR_TIMEOUT);
        return;
    }
    if (norm_w) {
        // The rows are the residual x: the layer's input is rms_norm(x) (ops.rs:136-149),
        // h = x * (scale * w) with scale = 1 / sqrt(dot(x, x) / e + eps), the dot in the
        // lane order of the reference's AVX2 kernel.  Normalised in place in shared
        // memory, so the normed rows never travel through HBM; the block of the first
        // router rows publishes the scales for the kernels that read x after this one.
        for (int tr = warp; tr < RT_BTOKS; tr += RT_THREADS / 32) {
            float* xr = s_x + (size_t)tr * e;
            float ss = 0.0f;
            for (int i = lane; i < e; i += 32) ss = fmaf(xr[i], xr[i], ss);
            ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 8));
            ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 16));
            ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 4));
            ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 2));
            ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 1));
            const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)e), norm_eps)));
            for (int i = lane; i < e; i += 32) xr[i] = __fmul_rn(xr[i], __fmul_rn(scale, norm_w[i]));
            if (lane == 0 && blockIdx.x == 0 && bt0 + tr < n) row_scale[bt0 + tr] = scale;
        }
        __syncthreads();
    }
    const int r0 = (warp & 1) * RT_ROWS, t0 = (warp >> 1) * RT_TOKS;   // inside the block
    float acc[RT_ROWS][RT_TOKS] = {};
#pragma unroll 4
    for (int i = lane; i < e; i += 32) {
        float w[RT_ROWS], x[RT_TOKS];
#pragma unroll
        for (int r = 0; r < RT_ROWS; r++) w[r] = s_w[(size_t)(r0 + r) * e + i];
#pragma unroll
        for (int t = 0; t < RT_TOKS; t++) x[t] = s_x[(size_t)(t0 + t) * e + i];
#pragma unroll
        for (int r = 0; r < RT_ROWS; r++)
#pragma unroll
            for (int t = 0; t < RT_TOKS; t++) acc[r][t] = fmaf(w[r], x[t], acc[r][t]);
    }
#pragma unroll
    for (int r = 0; r < RT_ROWS; r++)
#pragma unroll
        for (int t = 0; t < RT_TOKS; t++) {
            float v = acc[r][t];
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            const int row = br0 + r0 + r, tok = bt0 + t0 + t;
            if (lane == 0 && row < n_rows && tok < n) logits[(size_t)tok * n_rows + row] = v;
        }
}

// The same product for many tokens: a block of 8 warps computes 16 rows x 64
// tokens, a warp 8 rows x 16 tokens (128 accumulators per lane, so 24 shared-
// memory loads feed 128 multiply-adds), over K in chunks of 128 values that a
// three-stage ring of 16-byte asynchronous copies keeps in flight (a chunk of
// one row is 512 bytes: too small for bulk copies to pay).  The multiply-adds are issued
// two tokens at a time (fma.rn.f32x2; measured 0.64 -> 0.56 ms at 16 384 tokens).  The per-lane order of the
// multiply-adds and the order of the final lane sums are those of the small
// kernel above, so the logits are the same bits.
constexpr int RL_ROWS = 8, RL_TOKS = 16;              // register tile of one warp
constexpr int RL_BROWS = 16, RL_BTOKS = 64;           // rows and tokens of one block
constexpr int RL_KC = 128, RL_STAGES = 3;
constexpr int RL_STAGE_FLOATS = (RL_BROWS + RL_BTOKS) * RL_KC;
constexpr int RL_SMEM = 128 + RL_STAGES * RL_STAGE_FLOATS * 4;   // 123008

// one step of the lane sums: the lanes of a pair (lane ^ M) split the 2 * HALF values
template <int HALF, int M>
__device__ __forceinline__ void rl_reduce_step(float (&acc)[RL_ROWS * RL_TOKS], int lane, int& base) {
    const bool up = (lane & M) != 0;
#pragma unroll
    for (int j = 0; j < HALF; j++) {
        const float a = acc[j], b = acc[j + HALF];
        const float send = up ? a : b, keep = up ? b : a;
        acc[j] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, M));
    }
    if (up) base += HALF;
}

__global__ void __launch_bounds__(RT_THREADS, 1)
router_logits_tiled_kernel(const float* __restrict__ W, const float* __restrict__ h,
                           float* __restrict__ logits, int n, int e, int n_rows) {
    pdl_enter();
    extern __shared__ __align__(128) uint8_t rt_smem[];
    float* ring = (float*)(rt_smem + 128);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int br0 = blockIdx.x * RL_BROWS, bt0 = blockIdx.y * RL_BTOKS;
    const int nchunk = e / RL_KC;
    // every thread copies ten 16-byte pieces of chunk c into stage `c % RL_STAGES`: piece j of
    // the thread lies in row `warp + 8j` of the stage (rows 0-15 router rows, 16-79 token
    // rows), 16-byte column `lane`; the rows' addresses are worked out once (rows past the
    // end repeat the last one)
    constexpr int RL_PIECES = (RL_BROWS + RL_BTOKS) * (RL_KC / 4) / RT_THREADS;   // 10
    static_assert(RL_KC / 4 == 32 && RT_THREADS == 256, "a warp copies one row of a chunk");
    const float* rowp[RL_PIECES];
#pragma unroll
    for (int j = 0; j < RL_PIECES; j++) {
        const int r = warp + 8 * j;
        rowp[j] = (r < RL_BROWS ? W + (size_t)min(br0 + r, n_rows - 1) * e
                                : h + (size_t)min(bt0 + r - RL_BROWS, n - 1) * e) + lane * 4;
    }
    const uint32_t ring_u32 = rt_smem_u32(ring) + (uint32_t)(warp * RL_KC + lane * 4) * 4;
    auto fill = [&](int c) {
        const uint32_t st = ring_u32 + (uint32_t)(c % RL_STAGES) * (RL_STAGE_FLOATS * 4);
#pragma unroll
        for (int j = 0; j < RL_PIECES; j++)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(st + j * 8 * RL_KC * 4),
                         "l"(rowp[j] + (size_t)c * RL_KC)
                         : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int c = 0; c < RL_STAGES - 1; c++) {
        if (c < nchunk) fill(c);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int r0 = (warp & 1) * RL_ROWS, t0 = (warp >> 1) * RL_TOKS;   // inside the block
    // two tokens per multiply-add (fma.rn.f32x2: each half rounds as the scalar form does,
    // so the logits keep their bits): acc2[r][j] = tokens 2j, 2j+1 of row r
    f32x2 acc2[RL_ROWS * RL_TOKS / 2];
#pragma unroll
    for (int i = 0; i < RL_ROWS * RL_TOKS / 2; i++) acc2[i] = 0ull;
    for (int c = 0; c < nchunk; c++) {
        // chunk c has landed (one younger group may still be in flight); after the barrier
        // everyone is also done with chunk c - 1, whose stage chunk c + RL_STAGES - 1 reuses
        asm volatile("cp.async.wait_group %0;" ::"n"(RL_STAGES - 2) : "memory");
        __syncthreads();
        if (c + RL_STAGES - 1 < nchunk) fill(c + RL_STAGES - 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const float* sw = ring + (size_t)(c % RL_STAGES) * RL_STAGE_FLOATS + (size_t)r0 * RL_KC;
        const float* sx = ring + (size_t)(c % RL_STAGES) * RL_STAGE_FLOATS +
                          (size_t)(RL_BROWS + t0) * RL_KC;
#pragma unroll
        for (int kk = 0; kk < RL_KC / 32; kk++) {
            const int i = kk * 32 + lane;
            float w[RL_ROWS];
            f32x2 x2[RL_TOKS / 2];
#pragma unroll
            for (int r = 0; r < RL_ROWS; r++) w[r] = sw[r * RL_KC + i];
#pragma unroll
            for (int t = 0; t < RL_TOKS / 2; t++) x2[t] = pk(sx[(2 * t) * RL_KC + i], sx[(2 * t + 1) * RL_KC + i]);
#pragma unroll
            for (int r = 0; r < RL_ROWS; r++) {
                const f32x2 w2 = pk(w[r], w[r]);
#pragma unroll
                for (int t = 0; t < RL_TOKS / 2; t++)
                    acc2[r * (RL_TOKS / 2) + t] = fma2(w2, x2[t], acc2[r * (RL_TOKS / 2) + t]);
            }
        }
    }
    float acc[RL_ROWS * RL_TOKS];
#pragma unroll
    for (int i = 0; i < RL_ROWS * RL_TOKS / 2; i++) {
        acc[2 * i] = lo_of(acc2[i]);
        acc[2 * i + 1] = hi_of(acc2[i]);
    }
    // Lane sums in the order 8, 16, 4, 2, 1.  Each step halves the values a lane
    // carries: a lane keeps the half chosen by its bit of the step and gives the
    // other half to its partner, which adds the same two numbers as a full
    // butterfly would.  A lane ends with 4 of the warp's 128 outputs.
    int base = 0;
    rl_reduce_step<64, 8>(acc, lane, base);
    rl_reduce_step<32, 16>(acc, lane, base);
    rl_reduce_step<16, 4>(acc, lane, base);
    rl_reduce_step<8, 2>(acc, lane, base);
    rl_reduce_step<4, 1>(acc, lane, base);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int o = base + j;
        const int row = br0 + r0 + o / RL_TOKS, tok = bt0 + t0 + o % RL_TOKS;
        if (row < n_rows && tok < n) logits[(size_t)tok * n_rows + row] = acc[j];
    }
}

constexpr int RL_MIN_TOKENS = 256;   // from here on the tiled kernel is the faster one

// whether the kernel that stages whole rows serves this call: few tokens, and 8 router
// rows + 16 token rows fit in shared memory (n_embd <= 2304)
static bool router_stages_rows(int n, int e) {
    return n < RL_MIN_TOKENS && 128 + (RT_BROWS + RT_BTOKS) * (size_t)e * 4 <= 227 * 1024;
}
bool router_fuses_norm(int n, int e) { return router_stages_rows(n, e); }

cudaError_t launch_router(const LaunchCfg& c, const float* router_dev, const float* h,
                          const Workspace& ws, const RowNorm* norm) {
    int n_rows = c.n_expert + 1;
    if (!router_stages_rows(c.n, c.e)) {
        // many tokens, or rows too wide to stage whole: K travels in chunks of 128 values
        if (c.e % RL_KC || norm) return cudaErrorInvalidValue;
        static std::atomic<uint64_t> attr_set{0};
        if (cudaError_t err = ensure_dynamic_smem(router_logits_tiled_kernel, RL_SMEM, attr_set)) return err;
        dim3 grid((n_rows + RL_BROWS - 1) / RL_BROWS, (c.n + RL_BTOKS - 1) / RL_BTOKS);
        count_launch();
        return launch_after(c.stream, router_logits_tiled_kernel, grid, dim3(RT_THREADS), RL_SMEM, router_dev, h,
                            ws.logits, c.n, c.e, n_rows);
    }
    const int smem = 128 + (RT_BROWS + RT_BTOKS) * c.e * 4;
    static std::atomic<uint64_t> attr_set{0};
    if (cudaError_t err = ensure_dynamic_smem(router_logits_kernel, 227 * 1024, attr_set)) return err;
    dim3 grid((n_rows + RT_BROWS - 1) / RT_BROWS, (c.n + RT_BTOKS - 1) / RT_BTOKS);
    count_launch();
    return launch_after(c.stream, router_logits_kernel, grid, dim3(RT_THREADS), smem, router_dev, h, ws.logits, c.n,
                        c.e, n_rows, ws.status, norm ? norm->w : (const float*)nullptr,
                        norm ? norm->eps : 0.0f, ws.row_scale);
}

// ---------------------------------------------------------------------------
// One warp per token: softmax in the reference's order (max, exp, sequential
// sum, multiply by 1/sum), the k best by (probability descending, expert id
// ascending), weights p / max(sum of the k in rank order, 2^-14).
// The order of the probabilities is f32::total_cmp's, as in the reference's sort
// (model.rs:263): a total order, so a row with NaN or Inf activations - whose
// probabilities are all NaN - still selects k distinct, valid experts (the first k,
// all keys being equal) and only that token's weights and output are NaN.
constexpr int TK_WARPS = 4, TK_MAX_EXPERTS = 1024, TK_MAX_K = 32;

// total_cmp's key: the bits with the magnitude inverted for negative values, compared
// as signed integers; the mapping is its own inverse
__device__ __forceinline__ int tk_total_key(int bits) { return bits ^ (int)(((uint32_t)(bits >> 31)) >> 1); }

__global__ void __launch_bounds__(TK_WARPS * 32)
route_topk_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids,
                  float* __restrict__ weights, int n, int n_expert, int k) {
    pdl_enter();
    extern __shared__ float tk_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * TK_WARPS + warp;
    if (t >= n) return;
    float* p = tk_smem + (size_t)warp * n_expert;
    const float* l = logits + (size_t)t * (n_expert + 1);
    float mx = -INFINITY;
    for (int i = lane; i < n_expert; i += 32) mx = fmaxf(mx, l[i]);   // f32::max: a NaN is passed over
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int i = lane; i < n_expert; i += 32) p[i] = expf(__fsub_rn(l[i], mx));
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0) {   // the order of the adds is the reference's; the loads are batched
        int i = 0;
        for (; i + 8 <= n_expert; i += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = p[i + u];
#pragma unroll
            for (int u = 0; u < 8; u++) sum = __fadd_rn(sum, v[u]);
        }
        for (; i < n_expert; i++) sum = __fadd_rn(sum, p[i]);
    }
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inv = __fdiv_rn(1.0f, sum);
    int* key = (int*)p;   // the probabilities are replaced by their keys
    for (int i = lane; i < n_expert; i += 32) key[i] = tk_total_key(__float_as_int(__fmul_rn(p[i], inv)));
    __syncwarp();
    float sel_p = 0.0f;   // lane j keeps the j-th selection
    int sel_id = 0;
    uint32_t taken = 0;   // bit m: this lane's entry lane + 32 m is selected already
    constexpr int NONE = 0x7fffffff;
    for (int j = 0; j < k; j++) {
        int bk = 0, bi = NONE;
        for (int i = lane, m = 0; i < n_expert; i += 32, m++) {
            if ((taken >> m) & 1u) continue;
            const int kv = key[i];
            if (bi == NONE || kv > bk) { bk = kv; bi = i; }   // ascending i: the lower id wins ties
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const int ok = __shfl_xor_sync(0xffffffffu, bk, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != NONE && (bi == NONE || ok > bk || (ok == bk && oi < bi))) { bk = ok; bi = oi; }
        }
        // k <= n_expert, so some lane always had a candidate and bi is a valid id
        if (lane == j) { sel_p = __int_as_float(tk_total_key(bk)); sel_id = bi; }
        if (bi < n_expert && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    }
    float tot = 0.0f;
    for (int j = 0; j < k; j++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, sel_p, j));
    tot = fmaxf(tot, 1.0f / 16384.0f);   // f32::max: a NaN sum gives the floor
    if (lane < k) {
        ids[(size_t)t * k + lane] = min(sel_id, n_expert - 1);
        weights[(size_t)t * k + lane] = __fdiv_rn(sel_p, tot);
    }
}

cudaError_t launch_route_topk(const LaunchCfg& c, const Workspace& ws) {
    if (c.n_expert > TK_MAX_EXPERTS || c.k > TK_MAX_K) return cudaErrorInvalidValue;
    size_t smem = (size_t)TK_WARPS * c.n_expert * sizeof(float);
    count_launch();
    return launch_after(c.stream, route_topk_kernel, dim3((c.n + TK_WARPS - 1) / TK_WARPS), dim3(TK_WARPS * 32),
                        smem, (const float*)ws.logits, ws.ids, ws.weights, c.n, c.n_expert, c.k);
}

// ---------------------------------------------------------------------------
// Stable grouping of the n*k (token, expert) pairs by expert: inside an expert
// pairs keep ascending pair index t*k+j, which is the order the reference
// pushes them in (model.rs:867-873; Metal moe_sort, kernels.metal:1723-1729).
// A block owns SORT_TOKENS consecutive tokens.  Phase 1 counts per (block,
// expert); phase 2 turns the counts into bases (exclusive over blocks, then
// over experts) and builds the list of non-empty groups; phase 3 lets one
// thread per expert walk its block's pairs in order.  With one block the three
// phases run in a single launch.
constexpr int SORT_TOKENS = 256, SORT_THREADS = 256;
constexpr uint16_t kNoExpert = 0xFFFF;
constexpr int SORT_TILE = 8;   // tokens per tile of the expert kernels

__device__ void sort_load_ids(const int32_t* ids, int pair0, int npairs, uint16_t* s_ids) {
    // a negative id marks an empty slot (a row with fewer than k experts: expert parallelism)
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int id = ids[pair0 + i];
        s_ids[i] = id < 0 ? kNoExpert : (uint16_t)id;
    }
}
__device__ void sort_hist(const uint16_t* s_ids, int npairs, int n_expert, int* s_cnt) {
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) s_cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < npairs; i += blockDim.x)
        if (s_ids[i] != kNoExpert) atomicAdd(&s_cnt[s_ids[i]], 1);
    __syncthreads();
}
// exclusive scan over the block of one int per thread slot; `n_items` slots,
// ITEMS consecutive slots per thread.  Returns the total in *total.
template <int ITEMS>
__device__ void block_exclusive_scan(int (&v)[ITEMS], int* s_warp, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int local = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) { int t = v[i]; v[i] = local; local += t; }
    int inc = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nwarp ? s_warp[lane] : 0, winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        if (lane < nwarp) s_warp[lane] = winc - w;
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    const int base = s_warp[warp] + inc - local;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) v[i] += base;
    __syncthreads();
}

// One block: bases over blocks and experts, the list of non-empty groups, the
// list of token tiles, counters reset.  Positions: the shared expert's group
// (the tokens, in order) comes first at position 0; every routed group starts
// at a multiple of 8 so that a tile of 8 positions never straddles two groups.
// `s_cnt` (shared memory) holds the per-expert counts when one block sorts
// everything; otherwise they are summed from the per-block counts.
constexpr int SORT_EPT = 4;   // experts per thread in the scans (n_expert <= 1024)
__device__ void sort_scan(const Workspace& ws, int n_expert, int nblk, int n, int k,
                          int has_shared, int prefill_min, int ptile, const int* s_cnt, int* s_off) {
    __shared__ int s_warp[32];
    __shared__ int s_total[4];
    int cnt[SORT_EPT], off[SORT_EPT], act[SORT_EPT], til[SORT_EPT], ptl[SORT_EPT];
    const int e0 = threadIdx.x * SORT_EPT;
#pragma unroll
    for (int i = 0; i < SORT_EPT; i++) {
        const int e = e0 + i;
        int run = 0;
        if (e < n_expert) {
            if (s_cnt) {
                run = s_cnt[e];
            } else {
                for (int b = 0; b < nblk; b++) {
                    int c = ws.blk_counts[(size_t)b * n_expert + e];
                    ws.blk_counts[(size_t)b * n_expert + e] = run;
                    run += c;
                }
            }
        }
        // a group of at least prefill_min tokens is cut into tiles of `ptile` for the
        // tcgen05 kernels, a smaller one into tiles of 8 for the decode kernels
        const bool big = prefill_min > 0 && run >= prefill_min;
        cnt[i] = run;
        off[i] = (run + SORT_TILE - 1) / SORT_TILE * SORT_TILE;
        til[i] = big ? 0 : off[i] / SORT_TILE;
        ptl[i] = big ? (run + ptile - 1) / ptile : 0;
        act[i] = run > 0;
    }
    __syncthreads();   // s_cnt is read; s_off may alias it
    block_exclusive_scan<SORT_EPT>(off, s_warp, &s_total[0]);
    block_exclusive_scan<SORT_EPT>(act, s_warp, &s_total[1]);
    block_exclusive_scan<SORT_EPT>(til, s_warp, &s_total[2]);
    block_exclusive_scan<SORT_EPT>(ptl, s_warp, &s_total[3]);
    const int g_sh = has_shared ? 1 : 0;
    const bool big_sh = has_shared && prefill_min > 0 && n >= prefill_min;
    const int p_sh = has_shared ? (n + SORT_TILE - 1) / SORT_TILE * SORT_TILE : 0;
    const int t_sh = has_shared && !big_sh ? p_sh / SORT_TILE : 0;
    const int pt_sh = big_sh ? (n + ptile - 1) / ptile : 0;
#pragma unroll
    for (int i = 0; i < SORT_EPT; i++) {
        const int e = e0 + i;
        if (e >= n_expert) continue;
        const int start = p_sh + off[i];
        ws.counts[e] = cnt[i];
        ws.offsets[e] = start;
        if (s_off) s_off[e] = start;
        if (cnt[i]) {
            const int g = g_sh + act[i];
            ws.grp_expert[g] = e;
            ws.grp_start[g] = start;
            ws.grp_count[g] = cnt[i];
            const bool big = prefill_min > 0 && cnt[i] >= prefill_min;
            const int nt = big ? 0 : (cnt[i] + SORT_TILE - 1) / SORT_TILE;
            for (int j = 0; j < nt; j++) {
                ws.tile_desc[t_sh + til[i] + j] =
                    make_int4(e, start + j * SORT_TILE, min(SORT_TILE, cnt[i] - j * SORT_TILE), 0);
            }
            const int npt = big ? (cnt[i] + ptile - 1) / ptile : 0;
            for (int j = 0; j < npt; j++) {
                ws.ptile_group[pt_sh + ptl[i] + j] = g;
                ws.ptile_t0[pt_sh + ptl[i] + j] = j * ptile;
            }
        }
    }
    for (int j = threadIdx.x; j < t_sh; j += blockDim.x) {
        ws.tile_desc[j] = make_int4(n_expert, j * SORT_TILE, min(SORT_TILE, n - j * SORT_TILE), 0);
    }
    for (int j = threadIdx.x; j < pt_sh; j += blockDim.x) {
        ws.ptile_group[j] = 0;
        ws.ptile_t0[j] = j * ptile;
    }
    if (threadIdx.x == 0) {
        if (has_shared) {
            ws.grp_expert[0] = n_expert;
            ws.grp_start[0] = 0;
            ws.grp_count[0] = n;
        }
        ws.offsets[n_expert] = p_sh + s_total[0];
        *ws.n_groups = g_sh + s_total[1];
        ws.n_tiles[0] = t_sh + s_total[2];
        ws.n_tiles[1] = t_sh;
        ws.n_ptiles[0] = pt_sh + s_total[3];
        ws.n_ptiles[1] = pt_sh;
        for (int i = 0; i < 8; i++) ws.work_ctr[i] = 0;
    }
    __syncthreads();
}
// A token selects an expert at most once, so the rank of pair (t, j) inside its
// expert is the number of earlier tokens of the block that selected the expert:
// a popcount over the expert's token bitmask.
__device__ void sort_build_masks(const uint16_t* s_ids, int npairs, int k, int n_expert,
                                 uint32_t* s_mask) {
    for (int i = threadIdx.x; i < n_expert * (SORT_TOKENS / 32); i += blockDim.x) s_mask[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int t = i / k;
        if (s_ids[i] == kNoExpert) continue;
        atomicOr(&s_mask[s_ids[i] * (SORT_TOKENS / 32) + (t >> 5)], 1u << (t & 31));
    }
    __syncthreads();
}
__device__ void sort_scatter(const Workspace& ws, const uint16_t* s_ids, const uint32_t* s_mask,
                             int pair0, int npairs, int k, int n_expert, int blk, const int* s_off) {
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int e = s_ids[i], t = i / k;
        if (e == kNoExpert) {
            ws.pos_of[pair0 + i] = -1;
            continue;
        }
        const uint32_t* m = s_mask + e * (SORT_TOKENS / 32);
        int rank = __popc(m[t >> 5] & ((1u << (t & 31)) - 1u));
        for (int w = 0; w < (t >> 5); w++) rank += __popc(m[w]);
        const int pos = (s_off ? s_off[e] : ws.offsets[e] + ws.blk_counts[(size_t)blk * n_expert + e]) + rank;
        ws.order[pos] = pair0 + i;
        ws.pos_of[pair0 + i] = pos;
    }
}

__global__ void __launch_bounds__(SORT_THREADS)
sort_kernel(Workspace ws, int n, int k, int n_expert, int has_shared, int prefill_min, int ptile,
            int phase) {
    pdl_enter();
    extern __shared__ uint8_t sort_smem[];
    uint16_t* s_ids = (uint16_t*)sort_smem;
    int* s_cnt = (int*)(sort_smem + (((size_t)SORT_TOKENS * k * 2 + 15) & ~(size_t)15));
    uint32_t* s_mask = (uint32_t*)(s_cnt + n_expert);
    const int nblk = (n + SORT_TOKENS - 1) / SORT_TOKENS;
    const int blk = blockIdx.x;
    const int tok0 = blk * SORT_TOKENS, ntok = min(SORT_TOKENS, n - tok0);
    const int pair0 = tok0 * k, npairs = ntok * k;
    if (phase == 0) {   // one block does everything, counts and bases stay in shared memory
        sort_load_ids(ws.ids, pair0, npairs, s_ids);
        __syncthreads();
        sort_hist(s_ids, npairs, n_expert, s_cnt);
        sort_build_masks(s_ids, npairs, k, n_expert, s_mask);
        sort_scan(ws, n_expert, 1, n, k, has_shared, prefill_min, ptile, s_cnt, s_cnt);
        sort_scatter(ws, s_ids, s_mask, pair0, npairs, k, n_expert, 0, s_cnt);
        return;
    }
    if (phase == 1) {
        sort_load_ids(ws.ids, pair0, npairs, s_ids);
        __syncthreads();
        sort_hist(s_ids, npairs, n_expert, s_cnt);
        for (int e = threadIdx.x; e < n_expert; e += blockDim.x)
            ws.blk_counts[(size_t)blk * n_expert + e] = s_cnt[e];
    }
    if (phase == 2) sort_scan(ws, n_expert, nblk, n, k, has_shared, prefill_min, ptile, nullptr, nullptr);
    if (phase == 3) {
        sort_load_ids(ws.ids, pair0, npairs, s_ids);
        __syncthreads();
        sort_build_masks(s_ids, npairs, k, n_expert, s_mask);
        sort_scatter(ws, s_ids, s_mask, pair0, npairs, k, n_expert, blk, nullptr);
    }
}

// The lists of the shared expert's group alone (its positions are the tokens, in order):
// what sort_kernel writes for that group, for a rank of an expert-parallel layer, whose
// routed pairs are sorted where their experts live.
__global__ void __launch_bounds__(SORT_THREADS)
shared_lists_kernel(Workspace ws, int n, int n_expert, int prefill_min, int ptile) {
    pdl_enter();
    const bool big_sh = prefill_min > 0 && n >= prefill_min;
    const int p_sh = (n + SORT_TILE - 1) / SORT_TILE * SORT_TILE;
    const int t_sh = big_sh ? 0 : p_sh / SORT_TILE;
    const int pt_sh = big_sh ? (n + ptile - 1) / ptile : 0;
    for (int j = threadIdx.x; j < t_sh; j += blockDim.x)
        ws.tile_desc[j] = make_int4(n_expert, j * SORT_TILE, min(SORT_TILE, n - j * SORT_TILE), 0);
    for (int j = threadIdx.x; j < pt_sh; j += blockDim.x) {
        ws.ptile_group[j] = 0;
        ws.ptile_t0[j] = j * ptile;
    }
    if (threadIdx.x == 0) {
        ws.grp_expert[0] = n_expert;
        ws.grp_start[0] = 0;
        ws.grp_count[0] = n;
        ws.offsets[n_expert] = p_sh;
        *ws.n_groups = 1;
        ws.n_tiles[0] = t_sh;
        ws.n_tiles[1] = t_sh;
        ws.n_ptiles[0] = pt_sh;
        ws.n_ptiles[1] = pt_sh;
        for (int i = 0; i < 8; i++) ws.work_ctr[i] = 0;
    }
}

cudaError_t launch_shared_lists(const LaunchCfg& c, const Workspace& ws) {
    count_launch();
    return launch_after(c.stream, shared_lists_kernel, dim3(1), dim3(SORT_THREADS), 0, ws, c.n, c.n_expert,
                        c.prefill_min, c.prefill_tile);
}

cudaError_t launch_sort(const LaunchCfg& c, const Workspace& ws) {
    const int nblk = (c.n + SORT_TOKENS - 1) / SORT_TOKENS;
    size_t smem = (((size_t)SORT_TOKENS * c.k * 2 + 15) & ~(size_t)15) + (size_t)c.n_expert * 4 +
                  (size_t)c.n_expert * (SORT_TOKENS / 32) * 4;   // <= 16 + 4 + 32 KiB
    static std::atomic<uint64_t> attr_set{0};
    if (cudaError_t err = ensure_dynamic_smem(sort_kernel, 64 * 1024, attr_set)) return err;
    auto phase = [&](int blocks, int ph) {
        return launch_after(c.stream, sort_kernel, dim3(blocks), dim3(SORT_THREADS), smem, ws, c.n, c.k, c.n_expert,
                            c.has_shared, c.prefill_min, c.prefill_tile, ph);
    };
    if (nblk == 1) {
        count_launch();
        return phase(1, 0);
    }
    count_launch(3);
    if (cudaError_t err = phase(nblk, 1)) return err;
    if (cudaError_t err = phase(1, 2)) return err;
    return phase(nblk, 3);
}

}  // namespace bivmoe
