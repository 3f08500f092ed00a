// Expert parallelism: the small kernels either side of the all-to-all exchanges.
// The reference has no multi-device path (one MTLDevice,
// engine/src/metal/mod.rs:450-462; one thread pool on the CPU), so these have no
// counterpart there.  Rank r of W owns experts [r * n_expert / W, (r + 1) *
// n_expert / W) - a contiguous byte range of each ffn_*_exps tensor, experts
// being outermost (engine/src/model.rs:353) - and is the home rank of its own
// tokens.
//
//   home rank    route (router.cu), then ep_rank_slots / ep_rank_gather: a token's
//                row goes ONCE to every rank that owns at least one of its experts,
//                with the token's k expert ids and weights as a tag
//   exchange 1   rows and tags to the owners (the caller's all-to-all)
//   owner rank   ep_localize: the tag becomes a routing result over the local
//                experts with empty slots for the others; then the ordinary sort /
//                dispatch / expert kernels, and the ordinary combine, which leaves
//                per row the weighted sum over the local experts
//   exchange 2   one partial sum per row back, same layout
//   home rank    combine (rowops.cu) with the ranks as "experts" of weight one and
//                the partial sums as the routed rows, then the shared expert
//
// The exchanges come in two forms.  With the caller's all-to-all the rows are packed
// by destination and the row counts cross the host.  With peer stores (the ep_peer_*
// kernels) every rank maps one block of every other rank's memory (NVLink peer access)
// and the kernels write where the rows are needed: the home rank's scatter kernel puts
// a row straight into region [home rank] of the owner's receive buffer, the owner's
// combine kernel puts the partial sum straight into region [owner] of the home rank's
// return buffer (that kernel is the owner's combine itself, rowops.cu: the weighted sum
// over the local experts is stored where the home rank reads it).  A region holds `cap` rows (the most a rank can send to one peer), so
// no offsets depend on other ranks' counts, the counts travel as peer stores too, and
// the host never waits; the owner treats a region's unused rows as rows without experts.
// Two stream-ordered barriers of the caller's communicator per pass order the stores
// against their readers.  Plain stores only: no multicast, no waiting inside a kernel.
#include <algorithm>

#include "common.cuh"

namespace bivmoe {

// ---------------------------------------------------------------------------
// Block d: which tokens have an expert on rank d, and the rank-d slot of each (its
// index among them, in token order).  slot[t * world + d] = slot or -1;
// counts[d] = rows for rank d.
__global__ void __launch_bounds__(1024)
ep_rank_slots_kernel(const int32_t* __restrict__ ids, int n, int k, int n_local, int world,
                     int32_t* __restrict__ slot, int32_t* __restrict__ counts,
                     int32_t* __restrict__ counts_out) {
    __shared__ int s_warp[32];
    __shared__ int s_base;
    const int d = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    for (int t0 = 0; t0 < n; t0 += 1024) {
        const int t = t0 + threadIdx.x;
        int flag = 0;
        if (t < n)
            for (int j = 0; j < k; j++) {
                const int id = ids[(size_t)t * k + j];
                flag |= id >= 0 && id / n_local == d;
            }
        int inc = flag;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        if (lane == 31) s_warp[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            int w = s_warp[lane], winc = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, winc, o);
                if (lane >= o) winc += v;
            }
            s_warp[lane] = winc - w;
        }
        __syncthreads();
        const int base = s_base;
        if (t < n) slot[(size_t)t * world + d] = flag ? base + s_warp[warp] + inc - flag : -1;
        __syncthreads();
        if (threadIdx.x == 1023) s_base = base + s_warp[31] + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        counts[d] = s_base;
        counts_out[d] = s_base;
    }
}

// One block per token: its row, ids and weights go to the slot of every rank it uses;
// also the home combine's view of the pass: rank_ids[t][d] = d or -1, rank_pos[t][d] =
// the row's index in the send (= return) buffer.
constexpr int EPG_THREADS = 256;
__global__ void __launch_bounds__(EPG_THREADS)
ep_rank_gather_kernel(const float* __restrict__ h, const int32_t* __restrict__ ids,
                      const float* __restrict__ weights, const int32_t* __restrict__ slot,
                      const int32_t* __restrict__ counts, int k, int e, int world,
                      float* __restrict__ send_rows, int32_t* __restrict__ send_tags,
                      int32_t* __restrict__ rank_ids, int32_t* __restrict__ rank_pos) {
    __shared__ int s_dst[32];
    const int t = blockIdx.x;
    if (threadIdx.x < world) {
        const int d = threadIdx.x, sl = slot[(size_t)t * world + d];
        int base = 0;
        for (int x = 0; x < d; x++) base += counts[x];
        s_dst[d] = sl < 0 ? -1 : base + sl;
        rank_ids[(size_t)t * world + d] = sl < 0 ? -1 : d;
        rank_pos[(size_t)t * world + d] = sl < 0 ? 0 : base + sl;
    }
    __syncthreads();
    const float4* src = (const float4*)(h + (size_t)t * e);
    for (int d = 0; d < world; d++) {
        const int dst = s_dst[d];
        if (dst < 0) continue;
        float4* drow = (float4*)(send_rows + (size_t)dst * e);
        for (int i = threadIdx.x; i < e / 4; i += EPG_THREADS) drow[i] = src[i];
        if (threadIdx.x < k) {   // the tag: k ids, then the k weights' bits
            send_tags[(size_t)dst * 2 * k + threadIdx.x] = ids[(size_t)t * k + threadIdx.x];
            send_tags[(size_t)dst * 2 * k + k + threadIdx.x] =
                __float_as_int(weights[(size_t)t * k + threadIdx.x]);
        }
    }
}

cudaError_t launch_ep_gather(const LaunchCfg& c, const float* h, const Workspace& ws, int world,
                             int n_local, int32_t* slot, int32_t* counts, int32_t* rank_ids,
                             int32_t* rank_pos, float* send_rows, int32_t* send_tags,
                             int32_t* counts_out) {
    if (world > 32 || c.k > 32 || c.e % 4) return cudaErrorInvalidValue;
    ep_rank_slots_kernel<<<world, 1024, 0, c.stream>>>(ws.ids, c.n, c.k, n_local, world, slot, counts,
                                                      counts_out);
    ep_rank_gather_kernel<<<c.n, EPG_THREADS, 0, c.stream>>>(h, ws.ids, ws.weights, slot, counts, c.k, c.e,
                                                           world, send_rows, send_tags, rank_ids, rank_pos);
    count_launch(2);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// The owner's routing result from the received tags: the ids this rank owns, made
// local; every other slot empty.
__global__ void ep_localize_kernel(const int32_t* __restrict__ tags, int m, int k, int first, int n_local,
                                   int32_t* __restrict__ ids, float* __restrict__ weights) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * k) return;
    const int row = i / k, j = i % k;
    const int id = tags[(size_t)row * 2 * k + j];
    ids[i] = id >= first && id < first + n_local ? id - first : -1;
    weights[i] = __int_as_float(tags[(size_t)row * 2 * k + k + j]);
}

cudaError_t launch_ep_localize(const LaunchCfg& c, const int32_t* tags, int first, const Workspace& ws) {
    const int total = c.n * c.k;
    ep_localize_kernel<<<(total + 255) / 256, 256, 0, c.stream>>>(tags, c.n, c.k, first, c.n_expert, ws.ids,
                                                                ws.weights);
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Peer stores.  PeerLayout::rows etc. are byte offsets into every rank's block.

// Block d: the count of rows for rank d goes to rank d's recv_counts[me].
__global__ void ep_peer_counts_kernel(const int32_t* __restrict__ counts, PeerTable peers,
                                      PeerLayout lay, int me, int world) {
    const int d = threadIdx.x;
    if (d < world) ((int32_t*)(peers.base[d] + lay.counts))[me] = counts[d];
}

// One block per token, as ep_rank_gather_kernel, but the row and its tag go into region
// `me` of each owner's receive buffer; rank_pos is the row's index in this rank's own
// return buffer (region d, same slot).
__global__ void __launch_bounds__(EPG_THREADS)
ep_peer_scatter_kernel(const float* __restrict__ h, const int32_t* __restrict__ ids,
                       const float* __restrict__ weights, const int32_t* __restrict__ slot, int k, int e,
                       int world, int me, PeerTable peers, PeerLayout lay,
                       int32_t* __restrict__ rank_ids, int32_t* __restrict__ rank_pos) {
    __shared__ int s_slot[32];
    const int t = blockIdx.x;
    if (threadIdx.x < world) {
        const int d = threadIdx.x, sl = slot[(size_t)t * world + d];
        s_slot[d] = sl;
        rank_ids[(size_t)t * world + d] = sl < 0 ? -1 : d;
        rank_pos[(size_t)t * world + d] = sl < 0 ? 0 : d * lay.cap + sl;
    }
    __syncthreads();
    const float4* src = (const float4*)(h + (size_t)t * e);
    for (int d = 0; d < world; d++) {
        const int sl = s_slot[d];
        if (sl < 0) continue;
        const size_t row = (size_t)me * lay.cap + sl;
        float4* drow = (float4*)(peers.base[d] + lay.rows) + row * (e / 4);
        for (int i = threadIdx.x; i < e / 4; i += EPG_THREADS) drow[i] = src[i];
        if (threadIdx.x < k) {
            int32_t* tag = (int32_t*)(peers.base[d] + lay.tags) + row * 2 * k;
            tag[threadIdx.x] = ids[(size_t)t * k + threadIdx.x];
            tag[k + threadIdx.x] = __float_as_int(weights[(size_t)t * k + threadIdx.x]);
        }
    }
}

cudaError_t launch_ep_peer_scatter(const LaunchCfg& c, const float* h, const Workspace& ws, int world,
                                   int me, int n_local, int32_t* slot, int32_t* counts,
                                   int32_t* rank_ids, int32_t* rank_pos, const PeerTable& peers,
                                   const PeerLayout& lay) {
    if (world > 32 || c.k > 32 || c.e % 4) return cudaErrorInvalidValue;
    // c.n = 0 still publishes the (zero) counts: the owners read them every pass
    ep_rank_slots_kernel<<<world, 1024, 0, c.stream>>>(ws.ids, c.n, c.k, n_local, world, slot, counts,
                                                      counts);
    ep_peer_counts_kernel<<<1, 32, 0, c.stream>>>(counts, peers, lay, me, world);
    count_launch(2);
    if (c.n > 0) {
        ep_peer_scatter_kernel<<<c.n, EPG_THREADS, 0, c.stream>>>(h, ws.ids, ws.weights, slot, c.k, c.e,
                                                                world, me, peers, lay, rank_ids, rank_pos);
        count_launch();
    }
    return cudaGetLastError();
}

// The owner's routing result from its receive buffer: row r = region r / cap, slot
// r % cap; slots past the region's count are rows without experts.
__global__ void ep_peer_localize_kernel(const int32_t* __restrict__ tags, const int32_t* __restrict__ counts,
                                        int cap, int m, int k, int first, int n_local,
                                        int32_t* __restrict__ ids, float* __restrict__ weights) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * k) return;
    const int row = i / k, j = i % k;
    const bool used = row % cap < counts[row / cap];
    const int id = used ? tags[(size_t)row * 2 * k + j] : -1;
    ids[i] = id >= first && id < first + n_local ? id - first : -1;
    weights[i] = used ? __int_as_float(tags[(size_t)row * 2 * k + k + j]) : 0.0f;
}

cudaError_t launch_ep_peer_localize(const LaunchCfg& c, const uint8_t* block, const PeerLayout& lay,
                                    int first, const Workspace& ws) {
    const int total = c.n * c.k;
    ep_peer_localize_kernel<<<(total + 255) / 256, 256, 0, c.stream>>>(
        (const int32_t*)(block + lay.tags), (const int32_t*)(block + lay.counts), lay.cap, c.n, c.k, first,
        c.n_expert, ws.ids, ws.weights);
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// A stream-ordered barrier over the ranks' blocks, in two halves.  Barrier number e
// (every rank runs the same sequence of barriers, so the numbers agree without being
// exchanged): a rank SIGNALS by storing e into word [its rank] of every rank's flag
// array - a peer store like the rows' - and WAITS until every word of its own array
// has reached e.  Kernels earlier in the signalling stream have completed, so their
// peer stores are in place before the flag is; the waiting side reads the flags with
// acquire loads from its own memory.  The wait is bounded by a time limit, after which
// the kernel records BIVMOE_ERR_TIMEOUT in the layer's status word and returns: a rank
// that never arrives costs its peers the limit, not the GPU.  The barrier numbers live
// in device memory (the two counters behind the flags), so a captured graph replays
// the barrier with fresh numbers.
__device__ __forceinline__ unsigned long long ep_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__global__ void ep_peer_signal_kernel(uint8_t* block, PeerTable peers, PeerLayout lay, int me, int world) {
    __shared__ uint32_t s_epoch;
    uint32_t* ctr = (uint32_t*)(block + lay.flags) + kPeerFlagCounters;
    if (threadIdx.x == 0) {
        s_epoch = ctr[0] + 1;   // only this rank's own kernels touch the counters, in stream order
        ctr[0] = s_epoch;
    }
    __syncwarp();
    __threadfence_system();
    if ((int)threadIdx.x < world) {
        uint32_t* flag = (uint32_t*)(peers.base[threadIdx.x] + lay.flags) + me;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(s_epoch) : "memory");
    }
}

__global__ void ep_peer_wait_kernel(uint8_t* block, PeerLayout lay, int world, unsigned long long limit_ns,
                                    int32_t* status) {
    uint32_t* flags = (uint32_t*)(block + lay.flags);
    uint32_t* ctr = flags + kPeerFlagCounters;
    const uint32_t epoch = ctr[1] + 1;
    bool late = false;
    if ((int)threadIdx.x < world) {
        const unsigned long long t0 = ep_now_ns();
        while (true) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
            if ((int32_t)(v - epoch) >= 0) break;
            if (ep_now_ns() - t0 > limit_ns) { late = true; break; }
            __nanosleep(200);
        }
    }
    late = __any_sync(0xffffffffu, late);
    if (threadIdx.x == 0) {
        ctr[1] = epoch;   // the barrier is spent either way: the sequence stays in step
        if (late) atomicExch(status, BIVMOE_ERR_TIMEOUT);
    }
    __threadfence_system();
}

cudaError_t launch_ep_peer_signal(cudaStream_t stream, uint8_t* block, int me, int world,
                                  const PeerTable& peers, const PeerLayout& lay) {
    if (world > 32) return cudaErrorInvalidValue;
    ep_peer_signal_kernel<<<1, 32, 0, stream>>>(block, peers, lay, me, world);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_ep_peer_wait(cudaStream_t stream, uint8_t* block, int world, const PeerLayout& lay,
                                unsigned long long limit_ns, int32_t* status) {
    if (world > 32) return cudaErrorInvalidValue;
    ep_peer_wait_kernel<<<1, 32, 0, stream>>>(block, lay, world, limit_ns, status);
    count_launch();
    return cudaGetLastError();
}

}  // namespace bivmoe
