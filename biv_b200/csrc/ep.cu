// Expert parallelism: the two small kernels either side of the all-to-all
// exchanges.  The reference has no multi-device path (one MTLDevice,
// engine/src/metal/mod.rs:450-462; one thread pool on the CPU), so these have no
// counterpart there.  Rank r of W owns experts [r * n_expert / W, (r + 1) *
// n_expert / W) - a contiguous byte range of each ffn_*_exps tensor, experts
// being outermost (engine/src/model.rs:353) - and is the home rank of its own
// tokens.
//
//   home rank    route + sort by expert (router.cu)  ->  ep_gather: the token
//                rows in expert order, compact, which is also destination-rank
//                order since a rank's experts are contiguous
//   exchange 1   rows to the owners (the caller's all-to-all)
//   owner rank   ep_expand: the local expert id of every received row from the
//                count matrix, then the ordinary sort / dispatch / expert kernels
//   exchange 2   the rows' outputs back, same layout
//   home rank    combine (rowops.cu) with the returned rows as the routed source
#include <algorithm>

#include "common.cuh"

namespace bivmoe {

// ---------------------------------------------------------------------------
// compact_start[x] = number of pairs of experts below x; also hands the counts
// to the caller.  One block of 1024 threads (n_expert <= 1024).
__global__ void __launch_bounds__(1024)
ep_compact_starts_kernel(const int32_t* __restrict__ counts, int n_expert,
                         int32_t* __restrict__ compact_start, int32_t* __restrict__ counts_out) {
    __shared__ int s_warp[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = threadIdx.x < n_expert ? counts[threadIdx.x] : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = s_warp[lane], winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        s_warp[lane] = winc - w;
    }
    __syncthreads();
    if (threadIdx.x < n_expert) {
        compact_start[threadIdx.x] = s_warp[warp] + inc - c;
        if (counts_out) counts_out[threadIdx.x] = c;
        if (threadIdx.x == n_expert - 1) compact_start[n_expert] = s_warp[warp] + inc;
    }
}

// One block per pair: its token's row goes to the pair's compact slot.
constexpr int EPG_THREADS = 256;
__global__ void __launch_bounds__(EPG_THREADS)
ep_gather_kernel(const float* __restrict__ h, Workspace ws, const int32_t* __restrict__ compact_start,
                 int k, int e, float* __restrict__ send_rows, int32_t* __restrict__ compact_pos) {
    const int p = blockIdx.x;
    const int x = ws.ids[p];
    const int slot = compact_start[x] + (ws.pos_of[p] - ws.offsets[x]);
    if (threadIdx.x == 0) compact_pos[p] = slot;
    const float4* src = (const float4*)(h + (size_t)(p / k) * e);
    float4* dst = (float4*)(send_rows + (size_t)slot * e);
    for (int i = threadIdx.x; i < e / 4; i += EPG_THREADS) dst[i] = src[i];
}

cudaError_t launch_ep_gather(const LaunchCfg& c, const float* h, const Workspace& ws,
                             int32_t* compact_start, int32_t* compact_pos, float* send_rows,
                             int32_t* counts_out) {
    if (c.n_expert > 1024 || c.e % 4) return cudaErrorInvalidValue;
    ep_compact_starts_kernel<<<1, 1024, 0, c.stream>>>(ws.counts, c.n_expert, compact_start, counts_out);
    ep_gather_kernel<<<c.n * c.k, EPG_THREADS, 0, c.stream>>>(h, ws, compact_start, c.k, c.e, send_rows,
                                                            compact_pos);
    count_launch(2);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// The owner's view of what it received: rows ordered by source rank, then by
// expert, `recv_counts[s][x]` of them for local expert x from source s.  Writes
// the local expert id of every row (and a weight of one) as a k = 1 routing
// result, which the ordinary sort then groups.  Every block redoes the small
// scan and fills a slice of the rows.
__global__ void __launch_bounds__(1024)
ep_expand_kernel(const int32_t* __restrict__ recv_counts, int cells /* world * n_local */,
                 int n_local, int m, int32_t* __restrict__ ids, float* __restrict__ weights,
                 int32_t* __restrict__ status) {
    __shared__ int s_warp[32];
    __shared__ int s_start[1025];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = threadIdx.x < cells ? recv_counts[threadIdx.x] : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = s_warp[lane], winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        s_warp[lane] = winc - w;
    }
    __syncthreads();
    s_start[threadIdx.x] = threadIdx.x < cells ? s_warp[warp] + inc - c : 0x7fffffff;
    if (threadIdx.x == cells - 1) {
        s_start[cells] = s_warp[warp] + inc;
        // the caller's row count must be the sum of the matrix
        if (blockIdx.x == 0 && s_warp[warp] + inc != m) atomicExch(status, BIVMOE_ERR_ARGUMENT);
    }
    __syncthreads();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m; i += gridDim.x * blockDim.x) {
        int lo = 0, hi = cells;   // the last cell whose start is <= i (empty cells share a start)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_start[mid] <= i) lo = mid; else hi = mid;
        }
        ids[i] = lo % n_local;
        weights[i] = 1.0f;
    }
}

cudaError_t launch_ep_expand(const LaunchCfg& c, const int32_t* recv_counts, int world,
                             const Workspace& ws) {
    const int cells = world * c.n_expert;   // c.n_expert: the rank's local experts
    if (cells > 1024 || cells <= 0) return cudaErrorInvalidValue;
    const int blocks = std::max(1, std::min(c.sm_count, (c.n + 1023) / 1024));
    ep_expand_kernel<<<blocks, 1024, 0, c.stream>>>(recv_counts, cells, c.n_expert, c.n, ws.ids, ws.weights,
                                                    ws.status);
    count_launch();
    return cudaGetLastError();
}

}  // namespace bivmoe
