// Row-wise helpers around the expert products: the Q8 activation quantiser,
// rms_norm, the weighted gather-combine, and the upload-time repack of GGUF
// rows into the device row layout.
#include <cuda_bf16.h>

#include "common.cuh"
#include "formats.cuh"
#include "launch.cuh"

namespace bivmoe {

// ---------------------------------------------------------------------------
// Dispatch: the rows the expert kernels consume, laid out by position
// (slice-major, see common.cuh).  Token t's row goes to position t (the
// shared expert's group) and to the position of each of its k pairs.  For
// quantised weight types the row is quantised once, Q8Act::quantize_into
// (quant.rs:368-394) - the reference quantises it again for every expert it is
// routed to (model.rs:876-884), with the same result, the quantiser being a
// function of the row alone.  One block per token.
constexpr int DP_THREADS = 256, DP_MAX_K = 32;

// s_pos[j]: the position of pair j (j < k) and, as entry k, the token's position in the
// shared expert's group; s_big[j]: whether that position's group is large enough for
// the tcgen05 kernels.  Without a shared expert entry k repeats the first pair.
__device__ __forceinline__ void dispatch_positions(const Workspace& ws, int t, int n, int k, int n_expert,
                                                   int has_shared, int prefill_min, int* s_pos,
                                                   int* s_big) {
    if (threadIdx.x < k) {   // a negative position: an empty slot, nothing is written for it
        const int id = ws.ids[(size_t)t * k + threadIdx.x];
        s_pos[threadIdx.x] = id < 0 ? -1 : ws.pos_of[(size_t)t * k + threadIdx.x];
        s_big[threadIdx.x] = id >= 0 && prefill_min > 0 && ws.counts[id] >= prefill_min;
    }
    if (threadIdx.x == k) {
        s_pos[k] = has_shared ? t : -1;
        s_big[k] = has_shared && prefill_min > 0 && n >= prefill_min;
    }
    __syncthreads();
}

// Quantised rows.  A thread owns 8 consecutive values, four threads a 32-value block:
// the block's amax and sum(q) take two shuffle steps, two neighbouring threads make one
// 16-byte unit of int8, and one thread of the four stores the block's scales.  (One lane
// per value - a warp per block, five shuffle steps per reduction - cost eight times the
// instructions and took 0.18 ms for 4096 rows.)  The quantiser's arithmetic is
// q8_quantize_lane's: max and the integer sum do not depend on the order.
__global__ void __launch_bounds__(DP_THREADS)
dispatch_q8_kernel(const float* __restrict__ h, Workspace ws, int n, int k, int e, int has_shared,
                   const float* __restrict__ norm_w) {
    __shared__ int s_pos[DP_MAX_K + 1], s_big[DP_MAX_K + 1];
    pdl_enter();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int R = ws.act_rows;
    dispatch_positions(ws, t, n, k, 0, has_shared, 0, s_pos, s_big);
    const float* x = h + (size_t)t * e;
    // with norm_w the rows are the residual and h = x * (scale * w), rms_norm on the fly
    const float nscale = norm_w ? ws.row_scale[t] : 1.0f;
    for (int i0 = threadIdx.x * 8; i0 < e; i0 += DP_THREADS * 8) {   // e % 256 == 0: whole warps
        float4 a = *(const float4*)(x + i0), b = *(const float4*)(x + i0 + 4);
        if (norm_w) {
            const float4 wa = *(const float4*)(norm_w + i0), wb = *(const float4*)(norm_w + i0 + 4);
            a.x = __fmul_rn(a.x, __fmul_rn(nscale, wa.x)); a.y = __fmul_rn(a.y, __fmul_rn(nscale, wa.y));
            a.z = __fmul_rn(a.z, __fmul_rn(nscale, wa.z)); a.w = __fmul_rn(a.w, __fmul_rn(nscale, wa.w));
            b.x = __fmul_rn(b.x, __fmul_rn(nscale, wb.x)); b.y = __fmul_rn(b.y, __fmul_rn(nscale, wb.y));
            b.z = __fmul_rn(b.z, __fmul_rn(nscale, wb.z)); b.w = __fmul_rn(b.w, __fmul_rn(nscale, wb.w));
        }
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        // quant.rs:380-393: d = amax/127, id = 1/d (0 when d is 0), q = round(v*id) with
        // halves away from zero, s = d * (float)sum
        float amax = fabsf(v[0]);
#pragma unroll
        for (int j = 1; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float dd = __fdiv_rn(amax, 127.0f);
        const float id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
        int sum = 0;
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int q = (int)roundf(__fmul_rn(v[j], id));
            sum += q;
            if (j < 4) w0 |= ((uint32_t)q & 0xffu) << (8 * j);
            else w1 |= ((uint32_t)q & 0xffu) << (8 * (j - 4));
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float ss = __fmul_rn(dd, (float)sum);
        // the neighbour's 8 bytes: an even thread holds the low half of a 16-byte unit
        const uint32_t p0 = __shfl_down_sync(0xffffffffu, w0, 1), p1 = __shfl_down_sync(0xffffffffu, w1, 1);
        const uint4 unit = make_uint4(w0, w1, p0, p1);
        float shi, slo;
        split_tf32(ss, &shi, &slo);
        const int sl = i0 / 256, el = i0 % 256;      // K-slice, element within it
        const int bb = el / 32;                       // block of the slice
        const int which = lane & 3;                   // of the block's four threads: d, s_hi, s_lo, s
        const float val = which == 0 ? dd : which == 1 ? shi : which == 2 ? slo : ss;
        for (int j = 0; j <= k; j++) {
            const int pos = s_pos[j];
            if (pos < 0) continue;
            uint8_t* rec = ws.act_t + ((size_t)sl * (R / 8) + pos / 8) * kActTileBytes;
            if (!(lane & 1)) *(uint4*)(rec + act_q_off(pos % 8, el)) = unit;
            *(float*)(rec + kActOffDx + 256 * which + (bb * 8 + pos % 8) * 4) = val;
        }
    }
}

// Float rows (BF16 weights).  A thread owns 8 consecutive values: two float4 stores
// per position of a decode-sized group (slice-major f32 rows).  Positions of groups the
// tcgen05 kernel takes get nothing: that kernel gathers its rows by token from the
// bf16 terms split_rows_kernel writes.
__global__ void __launch_bounds__(DP_THREADS)
dispatch_f32_kernel(const float* __restrict__ h, Workspace ws, int n, int k, int e, int has_shared,
                    int prefill_min, const float* __restrict__ norm_w) {
    __shared__ int s_pos[DP_MAX_K + 1], s_big[DP_MAX_K + 1];
    pdl_enter();
    const int t = blockIdx.x;
    const int R = ws.act_rows;
    dispatch_positions(ws, t, n, k, 0, has_shared, ws.tok_b ? prefill_min : 0, s_pos, s_big);
    const float* x = h + (size_t)t * e;
    const float nscale = norm_w ? ws.row_scale[t] : 1.0f;
    for (int i0 = threadIdx.x * 8; i0 < e; i0 += DP_THREADS * 8) {
        float4 a = *(const float4*)(x + i0), b = *(const float4*)(x + i0 + 4);
        if (norm_w) {   // rms_norm on the fly: h = x * (scale * w)
            const float4 wa = *(const float4*)(norm_w + i0), wb = *(const float4*)(norm_w + i0 + 4);
            a.x = __fmul_rn(a.x, __fmul_rn(nscale, wa.x)); a.y = __fmul_rn(a.y, __fmul_rn(nscale, wa.y));
            a.z = __fmul_rn(a.z, __fmul_rn(nscale, wa.z)); a.w = __fmul_rn(a.w, __fmul_rn(nscale, wa.w));
            b.x = __fmul_rn(b.x, __fmul_rn(nscale, wb.x)); b.y = __fmul_rn(b.y, __fmul_rn(nscale, wb.y));
            b.z = __fmul_rn(b.z, __fmul_rn(nscale, wb.z)); b.w = __fmul_rn(b.w, __fmul_rn(nscale, wb.w));
        }
        const int sl = i0 / 64, off = i0 % 64;
        for (int j = 0; j <= k; j++) {
            const int pos = s_pos[j];
            if (pos < 0 || s_big[j]) continue;
            float* dst = ws.act_f + ((size_t)sl * R + pos) * 64 + off;
            *(float4*)dst = a;
            *(float4*)(dst + 4) = b;
        }
    }
}

// The rows as two bf16 terms, x = hi + lo, by token: [token][K / 64][hi 64 | lo 64], 256
// bytes per token and K-slice.  The tcgen05 kernel gathers a tile's rows from here in
// 16-byte units (experts_prefill_bf16.cu), so a row is split once, not once per position
// it occupies.  A row no group wants (an expert-parallel receive slot that is empty) is
// skipped.
__global__ void __launch_bounds__(DP_THREADS)
split_rows_kernel(const float* __restrict__ h, Workspace ws, int n, int k, int e, int has_shared,
                  const float* __restrict__ norm_w) {
    pdl_enter();
    const int t = blockIdx.x;
    if (!has_shared) {
        bool any = false;
        for (int j = 0; j < k; j++) any |= ws.ids[(size_t)t * k + j] >= 0;
        if (!any) return;
    }
    const float* x = h + (size_t)t * e;
    const float nscale = norm_w ? ws.row_scale[t] : 1.0f;
    for (int i0 = threadIdx.x * 8; i0 < e; i0 += DP_THREADS * 8) {
        float4 a = *(const float4*)(x + i0), b = *(const float4*)(x + i0 + 4);
        if (norm_w) {
            const float4 wa = *(const float4*)(norm_w + i0), wb = *(const float4*)(norm_w + i0 + 4);
            a.x = __fmul_rn(a.x, __fmul_rn(nscale, wa.x)); a.y = __fmul_rn(a.y, __fmul_rn(nscale, wa.y));
            a.z = __fmul_rn(a.z, __fmul_rn(nscale, wa.z)); a.w = __fmul_rn(a.w, __fmul_rn(nscale, wa.w));
            b.x = __fmul_rn(b.x, __fmul_rn(nscale, wb.x)); b.y = __fmul_rn(b.y, __fmul_rn(nscale, wb.y));
            b.z = __fmul_rn(b.z, __fmul_rn(nscale, wb.z)); b.w = __fmul_rn(b.w, __fmul_rn(nscale, wb.w));
        }
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const __nv_bfloat16 h0 = __float2bfloat16_rn(v[2 * p]), h1 = __float2bfloat16_rn(v[2 * p + 1]);
            const __nv_bfloat16 l0 = __float2bfloat16_rn(v[2 * p] - __bfloat162float(h0));
            const __nv_bfloat16 l1 = __float2bfloat16_rn(v[2 * p + 1] - __bfloat162float(h1));
            hi[p] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
            lo[p] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
        }
        uint8_t* rec = ws.tok_b + ((size_t)t * (e / 64) + i0 / 64) * kTokBRec + (i0 % 64) * 2;
        *(uint4*)rec = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *(uint4*)(rec + kTokBLo) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// Float rows by position, for many tokens: a block per tile of 8 positions of a
// decode-sized group, taken from the sort's tile list (groups the tcgen05 kernel takes
// have no tiles there).  It reads the tile's 8 source rows and writes them slice-major.
// (For quantised rows the same arrangement measured slower than the by-token kernel:
// it quantises a row once per position.)
constexpr int DP_MIN_TOKENS = 256;   // from here on the by-position kernel is the faster one

__global__ void __launch_bounds__(DP_THREADS)
dispatch_pos_f32_kernel(const float* __restrict__ h, Workspace ws, int k, int e, int n_expert,
                        int only_shared) {
    pdl_enter();
    const int n_tiles = ws.n_tiles[only_shared ? 1 : 0];   // the shared group's tiles come first
    // thread (tk, u): 8 consecutive values of token tk
    const int tk = threadIdx.x & 7, u0 = threadIdx.x >> 3;
    const int R = ws.act_rows;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int4 td = ws.tile_desc[tile];   // {expert (n_expert: shared), first position, tokens, 0}
        if (tk >= td.z) continue;
        const int pos = td.y + tk;
        const int tok = td.x == n_expert ? pos : ws.order[pos] / k;
        const float* x = h + (size_t)tok * e;
        for (int i0 = u0 * 8; i0 < e; i0 += (DP_THREADS / 8) * 8) {
            const float4 a = *(const float4*)(x + i0), b = *(const float4*)(x + i0 + 4);
            const int sl = i0 / 64, off = i0 % 64;
            float* dst = ws.act_f + ((size_t)sl * R + pos) * 64 + off;
            *(float4*)dst = a;
            *(float4*)(dst + 4) = b;
        }
    }
}

cudaError_t launch_dispatch(const LaunchCfg& c, const float* h, const Workspace& ws, bool quant,
                            bool f32, const RowNorm* norm) {
    if (c.k > DP_MAX_K || c.e % 256) return cudaErrorInvalidValue;
    if (norm && c.n >= DP_MIN_TOKENS) return cudaErrorInvalidValue;   // the by-position kernel reads normed rows
    const float* nw = norm ? norm->w : nullptr;
    if (quant) {
        if (cudaError_t err = launch_after(c.stream, dispatch_q8_kernel, dim3(c.n), dim3(DP_THREADS), 0, h, ws,
                                           c.n, c.k, c.e, c.has_shared, nw))
            return err;
        count_launch();
    }
    if (f32 && ws.tok_b && c.prefill_min > 0) {
        if (cudaError_t err = launch_after(c.stream, split_rows_kernel, dim3(c.n), dim3(DP_THREADS), 0, h, ws, c.n,
                                           c.k, c.e, c.has_shared, nw))
            return err;
        count_launch();
    }
    if (f32 && c.n >= DP_MIN_TOKENS) {
        // the tiles in use are known on the device only: blocks stride over the list
        const int shared_tiles = c.has_shared ? (c.n + 7) / 8 : 0;
        const int tiles = c.k == 0 ? shared_tiles : shared_tiles + (c.n * c.k) / 8 + c.n_expert;
        if (cudaError_t err = launch_after(c.stream, dispatch_pos_f32_kernel, dim3(min(tiles, 16 * c.sm_count)),
                                           dim3(DP_THREADS), 0, h, ws, max(c.k, 1), c.e, c.n_expert,
                                           c.only_shared || c.k == 0 ? 1 : 0))
            return err;
        count_launch();
    } else if (f32) {
        if (cudaError_t err = launch_after(c.stream, dispatch_f32_kernel, dim3(c.n), dim3(DP_THREADS), 0, h, ws, c.n,
                                           c.k, c.e, c.has_shared, c.prefill_min, nw))
            return err;
        count_launch();
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// ops.rs:136-149: out = x * (1/sqrt(dot(x,x)/e + eps)) * w, one warp per row.
// The sum of squares uses the reference's AVX2 dot order (see router.cu).
__global__ void __launch_bounds__(128)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                float* __restrict__ out, int n, int e) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const float* xr = x + (size_t)row * e;
    float acc = 0.0f;
    for (int i = lane; i < e; i += 32) acc = fmaf(xr[i], xr[i], acc);
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 16));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    const float ss = __fdiv_rn(acc, (float)e);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, eps)));
    for (int i = lane; i < e; i += 32)
        out[(size_t)row * e + i] = __fmul_rn(xr[i], __fmul_rn(scale, w[i]));
}

cudaError_t launch_rms_norm(const LaunchCfg& c, const float* x, const float* w, float eps,
                            float* out) {
    count_launch();
    return launch_after(c.stream, rms_norm_kernel, dim3((c.n + 3) / 4), dim3(128), 0, x, w, eps, out, c.n, c.e);
}

// ---------------------------------------------------------------------------
// Weighted gather-combine (model.rs:886-896; Metal moe_combine,
// kernels.metal:1885-1908): out[t] (+)= sum over the token's experts in
// ascending expert id of w * y, then sigmoid(gate) * shared, each step one
// fused multiply-add as the reference's axpy.  No atomics: run-to-run identical.
constexpr int CB_THREADS = 256, CB_MAX_K = 32;

// PEER: the rows are an owner rank's receive regions (expert parallelism by peer stores,
// ep.cu); row t = region t / cap, slot t % cap; a slot past the region's count has no row,
// and the sum of a row goes straight into region `me`, same slot, of the return buffer of
// the rank the row came from - the weighted sum and its way home are one kernel.
struct PeerDest {
    PeerTable peers;
    PeerLayout lay;
    const int32_t* counts;
    int me;
};

template <bool PEER>
__global__ void __launch_bounds__(CB_THREADS)
combine_kernel(const int32_t* __restrict__ ids, const float* __restrict__ weights,
               const float* __restrict__ routed_rows, const int32_t* __restrict__ routed_pos,
               const float* __restrict__ shared_rows, const float* __restrict__ logits,
               float* __restrict__ out, int n, int k, int e, int n_expert, int has_shared, int accumulate,
               PeerDest pd) {
    __shared__ int s_pos[CB_MAX_K];
    __shared__ float s_w[CB_MAX_K];
    __shared__ float s_gate;
    __shared__ int s_valid;
    pdl_enter();
    const int t = blockIdx.x;
    if (PEER && t % pd.lay.cap >= pd.counts[t / pd.lay.cap]) return;   // the whole block
    if (threadIdx.x == 0) s_valid = 0;
    __syncthreads();
    if (threadIdx.x < k) {
        // rank of this pair among the token's pairs by expert id (ids are distinct; a
        // negative id is an empty slot and takes no rank)
        const int my = ids[(size_t)t * k + threadIdx.x];
        if (my >= 0) {
            int rank = 0;
            for (int j = 0; j < k; j++) {
                const int o = ids[(size_t)t * k + j];
                rank += o >= 0 && o < my;
            }
            s_pos[rank] = routed_pos[(size_t)t * k + threadIdx.x];
            s_w[rank] = weights[(size_t)t * k + threadIdx.x];
            atomicAdd(&s_valid, 1);
        }
    }
    if (threadIdx.x == 32 && has_shared) {
        const float g = logits[(size_t)t * (n_expert + 1) + n_expert];
        s_gate = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));   // ops.rs:160-162
    }
    __syncthreads();
    const int kv = s_valid;
    const int c4 = blockIdx.y * CB_THREADS + threadIdx.x;     // float4 column
    if (c4 * 4 >= e) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < kv; j++) {
        const float4 y = *(const float4*)(routed_rows + (size_t)s_pos[j] * e + c4 * 4);
        const float w = s_w[j];
        acc.x = fmaf(w, y.x, acc.x); acc.y = fmaf(w, y.y, acc.y);
        acc.z = fmaf(w, y.z, acc.z); acc.w = fmaf(w, y.w, acc.w);
    }
    if (has_shared) {
        const float4 y = *(const float4*)(shared_rows + (size_t)t * e + c4 * 4);
        const float w = s_gate;
        acc.x = fmaf(w, y.x, acc.x); acc.y = fmaf(w, y.y, acc.y);
        acc.z = fmaf(w, y.z, acc.z); acc.w = fmaf(w, y.w, acc.w);
    }
    float4* o = (float4*)(out + (size_t)t * e + c4 * 4);
    if (PEER)
        o = (float4*)(pd.peers.base[t / pd.lay.cap] + pd.lay.returned) +
            ((size_t)pd.me * pd.lay.cap + t % pd.lay.cap) * (e / 4) + c4;
    if (accumulate) {
        float4 r = *o;
        acc.x += r.x; acc.y += r.y; acc.z += r.z; acc.w += r.w;
    }
    *o = acc;
}

cudaError_t launch_combine(const LaunchCfg& c, const CombineSrc& src, float* out, int accumulate) {
    if (c.k > CB_MAX_K || c.e % 4) return cudaErrorInvalidValue;
    dim3 grid(c.n, (c.e / 4 + CB_THREADS - 1) / CB_THREADS);
    count_launch();
    return launch_after(c.stream, combine_kernel<false>, grid, dim3(CB_THREADS), 0, src.ids, src.weights,
                        src.routed_rows, src.routed_pos, src.shared_rows, src.logits, out, c.n, c.k, c.e,
                        c.n_expert, c.has_shared, accumulate, PeerDest{});
}

cudaError_t launch_combine_to_peers(const LaunchCfg& c, const CombineSrc& src, const uint8_t* block, int me,
                                    const PeerTable& peers, const PeerLayout& lay) {
    if (c.k > CB_MAX_K || c.e % 4) return cudaErrorInvalidValue;
    dim3 grid(c.n, (c.e / 4 + CB_THREADS - 1) / CB_THREADS);
    const PeerDest pd{peers, lay, (const int32_t*)(block + lay.counts), me};
    count_launch();
    return launch_after(c.stream, combine_kernel<true>, grid, dim3(CB_THREADS), 0, src.ids, src.weights,
                        src.routed_rows, src.routed_pos, src.shared_rows, src.logits, (float*)nullptr, c.n, c.k,
                        c.e, c.n_expert, c.has_shared, 0, pd);
}

// ---------------------------------------------------------------------------
// Upload-time repack: GGUF rows -> tiled device layout (common.cuh).  One
// thread per 16-byte unit of the destination.  `tile_base` places the source
// matrix inside the chunk: 0 for gate and for down, 2 for up (chunk rows 64..127).
__global__ void repack_kernel(DevTiles dt, const uint8_t* __restrict__ src, int tile_base) {
    const int units = dt.slice_bytes / 16;
    const int64_t n_rows = (int64_t)dt.n * dt.rows;
    const int64_t total = n_rows * dt.nslices * units;
    const int64_t grb = gguf_row_bytes(dt.ty, dt.cols);
    const int64_t slice_tile_bytes = kChunkRows * (int64_t)dt.slice_bytes;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int u = (int)(i % units);
        const int s = (int)((i / units) % dt.nslices);
        const int64_t rg = i / ((int64_t)units * dt.nslices);   // row over all experts
        const int64_t e = rg / dt.rows;
        const int r = (int)(rg % dt.rows);
        const int chunk = r / dt.chunk_rows, vrow = tile_base * 32 + r % dt.chunk_rows;
        const uint8_t* row = src + rg * grb;
        uint8_t* dst = dt.data + e * dt.expert_bytes +
                       ((int64_t)chunk * dt.nslices + s) * slice_tile_bytes +
                       ((int64_t)u * kChunkRows + vrow) * 16;
        const uint8_t* from = nullptr;
        switch (dt.ty) {
            case BIVMOE_Q4_K: from = row + 144 * (int64_t)s + 16 * u; break;
            case BIVMOE_Q5_K: from = row + 176 * (int64_t)s + 16 * u; break;
            case BIVMOE_BF16:
            case BIVMOE_F16: from = row + 128 * (int64_t)s + 16 * u; break;
            case BIVMOE_F32: from = row + 256 * (int64_t)s + 16 * u; break;
            case BIVMOE_Q4_0:
                if (u < 8) from = row + 18 * (int64_t)(8 * s + u) + 2;
                break;
            case BIVMOE_Q4_1:
                if (u < 8) from = row + 20 * (int64_t)(8 * s + u) + 4;
                break;
            case BIVMOE_Q6_K: from = row + 210 * (int64_t)s + 16 * u; break;   // ql, qh, scales in order
            case BIVMOE_Q8_0:
                if (u < 16) from = row + 34 * (int64_t)(8 * s + u / 2) + 2 + 16 * (u % 2);
                break;
        }
        if (from) {
            for (int j = 0; j < 16; j++) dst[j] = from[j];
        } else {   // the eight f16 scales of the slice (Q4_1 unit 9: its eight f16 minimums)
            const int bb = dt.ty == BIVMOE_Q8_0 ? 34 : dt.ty == BIVMOE_Q4_0 ? 18 : 20;
            const int at = dt.ty == BIVMOE_Q4_1 && u == 9 ? 2 : 0;
            for (int b = 0; b < 8; b++) {
                dst[2 * b] = row[bb * (int64_t)(8 * s + b) + at];
                dst[2 * b + 1] = row[bb * (int64_t)(8 * s + b) + at + 1];
            }
        }
        if (dt.ty == BIVMOE_Q6_K && u == 0) {
            const uint8_t* d = row + 210 * (int64_t)s + 208;
            dt.side[(((int64_t)e * dt.chunks + chunk) * kChunkRows + vrow) * dt.nslices + s] =
                (uint16_t)(d[0] | (d[1] << 8));
        }
    }
}

cudaError_t launch_repack(const DevTiles& dst, const uint8_t* gguf_rows, int tile_base,
                          cudaStream_t stream) {
    repack_kernel<<<2048, 256, 0, stream>>>(dst, gguf_rows, tile_base);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Parity tap: the int32 dot of each 32-element block of one weight row with one
// Q8 activation row, decoded byte by byte as the reference's scalar kernels
// define the values (quant.rs:599-686).  One thread per block; not on the
// timed path.
__device__ inline uint8_t tile_byte(const DevTiles& t, const uint8_t* chunk0, int vrow, int s, int off) {
    // chunk0: K-slice 0 of the row's chunk; byte `off` of the row's slice s
    return chunk0[(int64_t)s * kChunkRows * t.slice_bytes + ((off >> 4) * kChunkRows + vrow) * 16 + (off & 15)];
}

__global__ void block_dots_kernel(DevTiles t, int tile_base, int expert, int row,
                                  const uint8_t* __restrict__ act_t, int act_rows, int pos,
                                  int32_t* __restrict__ out) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;   // 32-element block of the row
    if (b >= t.cols / 32) return;
    const int chunk = row / t.chunk_rows, rr = tile_base * 32 + row % t.chunk_rows;
    const uint8_t* t0 = t.stage(expert, chunk, 0);
    const int s = b / 8, sb = b % 8;
    const int8_t* rec = (const int8_t*)act_t + ((size_t)s * (act_rows / 8) + pos / 8) * kActTileBytes;
    int8_t x[32];
    for (int l = 0; l < 32; l++) x[l] = rec[act_q_off(pos % 8, 32 * sb + l)];
    int32_t sum = 0;
    if (t.ty == BIVMOE_Q8_0) {
        for (int l = 0; l < 32; l++) sum += (int)(int8_t)tile_byte(t, t0, rr, s, 32 * sb + l) * x[l];
    } else if (t.ty == BIVMOE_Q4_0 || t.ty == BIVMOE_Q4_1) {
        // quant.rs:574-577, 589-592: byte j = element j (low half) and j + 16 (high half)
        for (int l = 0; l < 32; l++) {
            const int q = (tile_byte(t, t0, rr, s, 16 * sb + (l & 15)) >> (4 * (l >> 4))) & 0xF;
            sum += (t.ty == BIVMOE_Q4_0 ? q - 8 : q) * x[l];
        }
    } else if (t.ty == BIVMOE_Q4_K || t.ty == BIVMOE_Q5_K) {
        const int qoff = (t.ty == BIVMOE_Q4_K ? 16 : 48) + 32 * (sb / 2);
        for (int l = 0; l < 32; l++) {
            int q = (tile_byte(t, t0, rr, s, qoff + l) >> (4 * (sb % 2))) & 0xF;
            if (t.ty == BIVMOE_Q5_K) q |= ((tile_byte(t, t0, rr, s, 16 + l) >> sb) & 1) << 4;
            sum += q * x[l];
        }
    } else if (t.ty == BIVMOE_Q6_K) {
        const int n = sb / 4, kq = sb % 4;
        for (int half = 0; half < 2; half++) {
            int32_t part = 0;
            for (int l = 16 * half; l < 16 * half + 16; l++) {
                const int ql = tile_byte(t, t0, rr, s, 64 * n + 32 * (kq & 1) + l);
                const int qh = tile_byte(t, t0, rr, s, 128 + 32 * n + l);
                const int nib = kq >= 2 ? ql >> 4 : ql & 0xF;
                part += ((nib | (((qh >> (2 * kq)) & 3) << 4)) - 32) * x[l];
            }
            sum += (int)(int8_t)tile_byte(t, t0, rr, s, 192 + 8 * n + 2 * kq + half) * part;
        }
    }
    out[b] = sum;
}

cudaError_t launch_block_dots(const DevTiles& t, int tile_base, int expert, int row,
                              const uint8_t* act_t, int act_rows, int pos, int32_t* out,
                              cudaStream_t stream) {
    const int nb = t.cols / 32;
    block_dots_kernel<<<(nb + 63) / 64, 64, 0, stream>>>(t, tile_base, expert, row, act_t, act_rows,
                                                         pos, out);
    return cudaGetLastError();
}

}  // namespace bivmoe
