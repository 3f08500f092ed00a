// Internal declarations shared by the kernels and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/bivmoe.h"

namespace bivmoe {

// ---------------------------------------------------------------------------
// Device layout of the weights.  The expert kernels work on chunks of 128 rows:
// 64 gate rows (chunk rows 0-63) together with the same 64 up rows (64-127), or
// 128 down rows.  What one pipeline stage consumes - one K-slice of a chunk - is
// stored contiguously (128 * SL bytes, one bulk copy), the K-slices of a chunk
// and then the chunks of an expert following each other:
//     [expert][chunk][K-slice][SL/16 units][128 rows][16 bytes]
// The bytes of a slice are unit-major: row r's 16-byte unit u sits at
// (u*128 + r)*16.  Lanes that own consecutive rows therefore read consecutive
// 16-byte pieces (no shared-memory bank conflicts), and for int8 and bf16 data
// two consecutive units are exactly the canonical K-major, unswizzled operand
// layout of the tensor core: 8 rows x 16 bytes contiguous, 128 bytes from one
// 8-row group to the next, 2048 bytes from one 16-byte K step to the next.
// The repack is a permutation of the GGUF bytes (nothing is widened):
//   type   K-slice   SL   the slice's bytes of one row
//   Q8_0   256       272  8 blocks' int8 quants (256) then their 8 f16 scales (16)
//   Q4_K   256       144  the 144-byte super-block {d, dmin, scales[12], qs[128]}
//   Q5_K   256       176  the 176-byte super-block {d, dmin, scales[12], qh[32], qs[128]}
//   Q6_K   256       208  ql[128], qh[64], scales[16]; the f16 d goes to a side plane
//   BF16   64        128  64 values
//   F16    64        128  64 values
//   F32    64        256  64 values
//   Q4_0   256       144  8 blocks' nibbles (8 x 16 bytes) then their 8 f16 scales (16)
//   Q4_1   256       160  8 blocks' nibbles, their 8 f16 scales, their 8 f16 minimums
constexpr int kRepackVersion = 4;
constexpr int kChunkRows = 128;
constexpr int kPrefillTile = 128;   // tokens per tile of the tcgen05 kernel for Q8_0
constexpr int kPrefillTileBf16 = 128;   // and for BF16
constexpr int kPrefillPad = 128;    // positions a tile's copy may run past the last group

struct SliceGeom { int elems, sl; };
__host__ __device__ inline SliceGeom slice_geom(int ty) {
    switch (ty) {
        case BIVMOE_Q8_0: return {256, 272};
        case BIVMOE_Q4_K: return {256, 144};
        case BIVMOE_Q5_K: return {256, 176};
        case BIVMOE_Q6_K: return {256, 208};
        case BIVMOE_BF16: return {64, 128};
        case BIVMOE_F16: return {64, 128};
        case BIVMOE_F32: return {64, 256};
        case BIVMOE_Q4_0: return {256, 144};
        case BIVMOE_Q4_1: return {256, 160};
        default: return {0, 0};
    }
}
__host__ __device__ inline int64_t gguf_row_bytes(int ty, int64_t cols) {
    switch (ty) {
        case BIVMOE_F32: return cols * 4;
        case BIVMOE_BF16: case BIVMOE_F16: return cols * 2;
        case BIVMOE_Q4_0: return cols / 32 * 18;
        case BIVMOE_Q4_1: return cols / 32 * 20;
        case BIVMOE_Q8_0: return cols / 32 * 34;
        case BIVMOE_Q4_K: return cols / 256 * 144;
        case BIVMOE_Q5_K: return cols / 256 * 176;
        case BIVMOE_Q6_K: return cols / 256 * 210;
        default: return -1;
    }
}
__host__ __device__ inline bool type_uses_f32_act(int ty) {  // quant.rs:75-77
    return ty == BIVMOE_F32 || ty == BIVMOE_F16 || ty == BIVMOE_BF16;
}

struct DevTiles {          // the tiles of one product (gate+up, or down) of a stack of experts
    int ty = 0;
    int cols = 0;              // inner dimension K
    int rows = 0;              // rows of one source matrix (ff for gate and up, n_embd for down)
    int n = 0;                 // experts
    int chunks = 0;            // chunks per expert: rows/64 (gate+up) or rows/128 (down)
    int chunk_rows = 0;        // source rows per chunk: 64 or 128
    int slice_bytes = 0;       // SL
    int nslices = 0;           // cols / slice elems
    uint8_t* data = nullptr;
    uint16_t* side = nullptr;  // Q6_K: f16 d, [expert][chunk][128 rows][nslices]
    int64_t expert_bytes = 0;  // chunks * nslices * 128 * SL
    // first byte of K-slice s of a chunk
    __host__ __device__ const uint8_t* stage(int64_t e, int chunk, int s) const {
        return data + e * expert_bytes + ((int64_t)chunk * nslices + s) * kChunkRows * slice_bytes;
    }
};

// Activation rows live in a position space in which every group starts at a
// multiple of 8, so a tile of 8 positions belongs to one group.  Quantised rows
// (Q8Act, quant.rs:352-394) are stored as one record per (K-slice of 256, tile):
//     q     [16 units][8 tokens][16] int8: unit-major like the weights, so that 8
//                            tokens x 16 bytes are contiguous (bank-conflict free
//                            fragment loads; the tensor core's canonical K-major layout)
//     dx    [8 blocks][8 tokens] f32: the block scales d
//     s_hi  [8 blocks][8 tokens] f32: s = d*sum(q) split in two tf32-exact parts
//     s_lo                            (11 + 11 mantissa bits), for the tensor-core min term
//     s     [8 blocks][8 tokens] f32: s itself (read by the taps only)
// which is what one pipeline stage of the expert kernels copies (all but `s`).
// Float rows (BF16 weights) are [K/64][R][64] f32.  R = ceil8(n) + n*k + 8*n_expert + 8.
// For the BF16 tensor-core kernel the float rows are also kept as two bf16
// terms, x = hi + lo up to 2^-17 |x| (hi = bf16(x), lo = bf16(x - hi)), one
// record per (K-slice of 64, tile of 8 positions):
//     hi    [8 units][8 tokens][8 bf16]   the canonical K-major operand layout
//     lo    the same, 1024 bytes further
constexpr int kActBRec = 2048, kActBLo = 1024;
// the same two terms of one token and K-slice before they are gathered into records:
// hi[64] then lo[64]
constexpr int kTokBRec = 256, kTokBLo = 128;
// byte offset inside a record of element i (0..63) of token tk (0..7), hi term
__host__ __device__ inline int act_b_off(int tk, int i) { return ((i >> 3) * 8 + tk) * 16 + (i & 7) * 2; }
constexpr int kActOffDx = 2048, kActOffSHi = kActOffDx + 256, kActOffSLo = kActOffSHi + 256,
              kActOffS = kActOffSLo + 256;
constexpr int kActCopyBytes = kActOffS;        // 2816: what a stage copies
constexpr int kActTileBytes = kActOffS + 256;  // 3072
// byte offset inside a record of element i (0..255) of token tk (0..7)
__host__ __device__ inline int act_q_off(int tk, int i) { return ((i >> 4) * 8 + tk) * 16 + (i & 15); }
// the two tf32-exact parts of an f32 (the tensor core ignores the low 13 mantissa bits)
__host__ __device__ inline void split_tf32(float v, float* hi, float* lo) {
    union { float f; uint32_t u; } a, b;
    a.f = v;
    a.u &= 0xFFFFE000u;
    b.f = v - a.f;
    b.u &= 0xFFFFE000u;
    *hi = a.f;
    *lo = b.f;
}
// Per-forward scratch.  P = n * k routed pairs; "positions" 0..P are the pairs
// in expert-sorted order, positions P..P+n are the tokens of the shared expert.
struct Workspace {
    float* logits;       // [n][n_expert + 1]; the last column is the shared-gate logit
    int32_t* ids;        // [n][k]
    float* weights;      // [n][k]
    int32_t* counts;     // [n_expert]
    int32_t* offsets;    // [n_expert + 1]
    int32_t* order;      // [P] position -> pair index
    int32_t* pos_of;     // [P] pair index -> position
    int32_t* blk_counts; // [sort blocks][n_expert]
    int32_t* grp_expert; // [n_expert + 1] group -> expert id (n_expert = shared)
    int32_t* grp_start;  // [n_expert + 1] first position
    int32_t* grp_count;  // [n_expert + 1]
    int32_t* n_groups;   // [1]
    int4* tile_desc;     // [tiles] a tile is <= 8 consecutive positions of a group:
                         // {expert id (n_expert = shared), first position, tokens, 0}
    int32_t* n_tiles;    // [2] all tiles; the shared group's tiles (they come first)
    int32_t* ptile_group;// [ptiles] tiles of 128 positions of the prefill-sized groups
    int32_t* ptile_t0;
    int32_t* n_ptiles;   // [2] all prefill tiles; the shared group's (they come first)
    uint32_t* work_ctr;  // [8] dynamic work counters, zeroed by the sort
    int32_t* status;     // [4] device-side error flags (0 = ok)
    int act_rows;        // R: positions
    uint8_t* act_t;      // Q8 records of h, [n_embd/256][R/8] tiles (quantised gate/up types)
    float* act_f;        // f32 rows of h by position, slice-major (float-activation types)
    uint8_t* tok_b;      // bf16 hi/lo terms of h by token, [N][n_embd/64][kTokBRec] (BF16 layers with the tcgen05 kernels)
    uint8_t* mid_b;      // the same of silu(gate)*up, [ff/64][R/8]
    float* mid;          // silu(gate)*up by position, slice-major f32 [ff/64][R][64]
    uint8_t* mid_t;      // its Q8 records, [ff/256][R/8] tiles (quantised down types)
    float* pair_out;     // [P + n][e], by position
    float* h_norm;       // [n][e] rms-normed rows (forward_stack with many tokens)
    float* row_scale;    // [n] rms_norm scales of the rows (forward_stack, norm fused into the router)
};

// The rms_norm that precedes the layer (ops.rs:136-149), applied on the fly by the
// kernels that read the rows: h[t][i] = x[t][i] * (scale[t] * w[i]).
struct RowNorm {
    const float* w;       // [e] post_norm weights
    float eps;
    const float* scale;   // [n] written by the router kernel, read by the dispatch kernels
};

struct LaunchCfg {
    cudaStream_t stream;
    int n, k, e, n_expert, ff, ff_sh, has_shared;
    int sm_count;
    int prefill_min = 0;         // groups with at least this many tokens go to the tcgen05 kernels (0: none)
    int prefill_tile = kPrefillTile;   // positions per tile of the tcgen05 kernel in use
    int only_shared = 0;         // expert launches cover the shared expert's group alone (expert parallelism)
    cudaEvent_t* ev = nullptr;   // optional: events recorded between the stages (profiling call)
};
enum { EV_START = 0, EV_ROUTER, EV_TOPK, EV_SORT, EV_QUANT, EV_GATEUP, EV_DOWN, EV_COMBINE, EV_COUNT };
inline void mark(const LaunchCfg& c, int which) {
    if (c.ev) cudaEventRecord(c.ev[which], c.stream);
}

// Raises a kernel's dynamic shared-memory limit once per device (the attribute is per
// device; `done` is the caller's static bit mask, one bit per device ordinal).
template <class K>
inline cudaError_t ensure_dynamic_smem(K kernel, int bytes, std::atomic<uint64_t>& done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return e;
}

// kernels (one translation unit each)
// `norm`: the rows are the residual x and the router kernel normalises them itself
// (only where router_fuses_norm says so; it also fills ws.row_scale)
cudaError_t launch_router(const LaunchCfg& c, const float* router_dev /*[n_expert+1][e]*/,
                          const float* h, const Workspace& ws, const RowNorm* norm = nullptr);
bool router_fuses_norm(int n, int e);
cudaError_t launch_route_topk(const LaunchCfg& c, const Workspace& ws);
cudaError_t launch_sort(const LaunchCfg& c, const Workspace& ws);
cudaError_t launch_shared_lists(const LaunchCfg& c, const Workspace& ws);
cudaError_t launch_dispatch(const LaunchCfg& c, const float* h, const Workspace& ws, bool quant,
                            bool f32, const RowNorm* norm = nullptr);
cudaError_t launch_experts(const LaunchCfg& c, const DevTiles& gate_up, const DevTiles& down,
                           const DevTiles& sh_gate_up, const DevTiles& sh_down, const Workspace& ws);
// What the combine sums for token t: for each of its k slots j with ids[t*k+j] >= 0, in
// ascending id, weights[t*k+j] * routed_rows[routed_pos[t*k+j]]; then, with a shared
// expert, sigmoid(logits[t][n_expert]) * shared_rows[t].  One layer: the workspace's
// routing result, pair_out and pos_of.  Expert parallelism: the ranks as "experts" and
// the partial sums they returned as the routed rows.
struct CombineSrc {
    const int32_t* ids;
    const float* weights;
    const float* routed_rows;
    const int32_t* routed_pos;
    const float* shared_rows;
    const float* logits;
};
inline CombineSrc combine_src(const Workspace& ws) {
    return CombineSrc{ws.ids, ws.weights, ws.pair_out, ws.pos_of, ws.pair_out, ws.logits};
}
cudaError_t launch_combine(const LaunchCfg& c, const CombineSrc& src, float* out, int accumulate);
cudaError_t launch_ep_gather(const LaunchCfg& c, const float* h, const Workspace& ws, int world,
                             int n_local, int32_t* slot, int32_t* counts, int32_t* rank_ids,
                             int32_t* rank_pos, float* send_rows, int32_t* send_tags,
                             int32_t* counts_out);
cudaError_t launch_ep_localize(const LaunchCfg& c, const int32_t* tags, int first, const Workspace& ws);
// Peer-store exchange (ep.cu): every rank owns one block of this layout and maps the others'.
struct PeerTable { uint8_t* base[32]; };          // rank -> its block, as seen from this device
struct PeerLayout {
    int cap;                                       // rows per region = the layer's max_tokens
    size_t rows, returned, tags, counts, bytes;   // byte offsets: [W][cap][e] f32 received rows,
                                                   // [W][cap][e] f32 returned sums, [W][cap][2k] i32
                                                   // tags, [W] i32 counts; the block's size
    size_t flags;                                  // [W] u32 barrier epochs, word r written by rank r;
                                                   // then (64 words on) this rank's own two counters:
                                                   // barriers signalled, barriers waited for
};
constexpr int kPeerFlagCounters = 64;              // word offset of the two counters after `flags`
cudaError_t launch_ep_peer_scatter(const LaunchCfg& c, const float* h, const Workspace& ws, int world,
                                   int me, int n_local, int32_t* slot, int32_t* counts,
                                   int32_t* rank_ids, int32_t* rank_pos, const PeerTable& peers,
                                   const PeerLayout& lay);
cudaError_t launch_ep_peer_localize(const LaunchCfg& c, const uint8_t* block, const PeerLayout& lay,
                                    int first, const Workspace& ws);
// the two halves of a stream-ordered barrier over the ranks' blocks (ep.cu)
cudaError_t launch_ep_peer_signal(cudaStream_t stream, uint8_t* block, int me, int world,
                                  const PeerTable& peers, const PeerLayout& lay);
cudaError_t launch_ep_peer_wait(cudaStream_t stream, uint8_t* block, int world, const PeerLayout& lay,
                                unsigned long long limit_ns, int32_t* status);
// the combine over an owner's receive regions, each row's sum stored into the return
// buffer of the rank it came from (rowops.cu)
cudaError_t launch_combine_to_peers(const LaunchCfg& c, const CombineSrc& src, const uint8_t* block, int me,
                                    const PeerTable& peers, const PeerLayout& lay);
cudaError_t launch_rms_norm(const LaunchCfg& c, const float* x, const float* w, float eps,
                            float* out);
cudaError_t launch_repack(const DevTiles& dst, const uint8_t* gguf_rows, int tile_base,
                          cudaStream_t stream);
cudaError_t launch_block_dots(const DevTiles& t, int tile_base, int expert, int row,
                              const uint8_t* act_t, int act_rows, int pos, int32_t* out,
                              cudaStream_t stream);
bool experts_supported(int ty, int cols, int rows, bool is_down);
bool prefill_supported(int gate_up_ty, int down_ty);
cudaError_t measure_int8_peak(int sm_count, int32_t* status_dev, cudaStream_t stream, double* tops);
cudaError_t launch_experts_prefill_bf16(const LaunchCfg& c, const DevTiles& gate_up, const DevTiles& down,
                                        const DevTiles& sh_gate_up, const DevTiles& sh_down,
                                        const Workspace& ws);
cudaError_t launch_experts_prefill(const LaunchCfg& c, const DevTiles& gate_up, const DevTiles& down,
                                   const DevTiles& sh_gate_up, const DevTiles& sh_down,
                                   const Workspace& ws);

void count_launch(int n = 1);

// Makes a device current for the duration of an entry point and puts the caller's
// back afterwards (a caller with several GPUs in one process need not switch).
struct DeviceScope {
    int prev = -1;
    bool switched = false;
    explicit DeviceScope(int device) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != device)
            switched = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceScope() {
        if (switched) cudaSetDevice(prev);
    }
    DeviceScope(const DeviceScope&) = delete;
    DeviceScope& operator=(const DeviceScope&) = delete;
};

// what the routing step needs to know about a layer (filled by api.cu)
struct RouteView {
    int device, sm_count, e, n_expert, k, has_shared;
    const float* router;   // device, [n_expert + 1][e]
    int32_t* status;       // the layer's device status word
};
int layer_route_view(bivmoe_layer* layer, RouteView* out, const char* error_or_null);

}  // namespace bivmoe
