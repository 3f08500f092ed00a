// Internal declarations shared by the kernels and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bivmoe.h"

namespace bivmoe {

// ---------------------------------------------------------------------------
// Device layout of weight rows.  GGUF blocks whose size is not a multiple of
// 16 bytes are split into planes per row at upload so that every row starts on
// a 16-byte boundary and bulk copies and 128-bit loads apply:
//   Q8_0  [qs: K int8][d: K/32 f16]                       K + K/16 bytes (= 34*K/32)
//   Q4_K  native 144-byte blocks {d, dmin, scales[12], qs[128]}
//   Q5_K  native 176-byte blocks {d, dmin, scales[12], qh[32], qs[128]}
//   Q6_K  [ql: nb*128][qh: nb*64][scales: nb*16][d: nb f16, padded to 16]
//         (nb = K/256; 1680 bytes at K=2048 as in GGUF, 432 instead of 420 at K=512)
//   BF16, F32 native
constexpr int kRepackVersion = 1;

__host__ __device__ inline int64_t dev_row_bytes(int ty, int64_t cols) {
    switch (ty) {
        case BIVMOE_F32: return cols * 4;
        case BIVMOE_BF16: return cols * 2;
        case BIVMOE_Q8_0: return cols + cols / 16;
        case BIVMOE_Q4_K: return cols / 256 * 144;
        case BIVMOE_Q5_K: return cols / 256 * 176;
        case BIVMOE_Q6_K: {
            int64_t nb = cols / 256;
            return nb * 208 + ((nb * 2 + 15) / 16) * 16;
        }
        default: return -1;
    }
}
__host__ __device__ inline int64_t gguf_row_bytes(int ty, int64_t cols) {
    switch (ty) {
        case BIVMOE_F32: return cols * 4;
        case BIVMOE_BF16: return cols * 2;
        case BIVMOE_Q8_0: return cols / 32 * 34;
        case BIVMOE_Q4_K: return cols / 256 * 144;
        case BIVMOE_Q5_K: return cols / 256 * 176;
        case BIVMOE_Q6_K: return cols / 256 * 210;
        default: return -1;
    }
}
__host__ __device__ inline bool type_uses_f32_act(int ty) {  // quant.rs:75-77
    return ty == BIVMOE_F32 || ty == BIVMOE_BF16;
}

struct DevStack {          // one stack of expert matrices on the device
    int ty = 0;
    int cols = 0, rows = 0, n = 0;
    uint8_t* data = nullptr;
    int64_t row_bytes = 0;     // dev_row_bytes
    int64_t expert_bytes = 0;  // rows * row_bytes
};

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
    int32_t* tile_group; // [tiles] tile -> group; a tile is <= 8 consecutive positions of a group
    int32_t* tile_t0;    // [tiles] first token of the tile inside its group
    int32_t* n_tiles;    // [2] all tiles; the shared group's tiles (they come first)
    uint32_t* work_ctr;  // [4] dynamic work counters, zeroed by the sort
    int32_t* status;     // [4] device-side error flags (0 = ok)
    int8_t* act_q;       // [n][e]
    float2* act_ds;      // [n][e/32] (d, s) per block
    float* mid;          // [P + n][ff] silu(gate)*up, by position
    int8_t* mid_q;       // [P + n][ff] its Q8 rows (quantised down types)
    float2* mid_ds;      // [P + n][ff/32]
    float* pair_out;     // [P + n][e], by position
    float* h_norm;       // [n][e] rms-normed rows (forward_stack)
};

struct LaunchCfg {
    cudaStream_t stream;
    int n, k, e, n_expert, ff, ff_sh, has_shared;
    int sm_count;
    cudaEvent_t* ev = nullptr;   // optional: events recorded between the stages (profiling call)
};
enum { EV_START = 0, EV_ROUTER, EV_TOPK, EV_SORT, EV_QUANT, EV_GATEUP, EV_DOWN, EV_COMBINE, EV_COUNT };
inline void mark(const LaunchCfg& c, int which) {
    if (c.ev) cudaEventRecord(c.ev[which], c.stream);
}

// kernels (one translation unit each)
cudaError_t launch_router(const LaunchCfg& c, const float* router_dev /*[n_expert+1][e]*/,
                          const float* h, const Workspace& ws);
cudaError_t launch_route_topk(const LaunchCfg& c, const Workspace& ws);
cudaError_t launch_sort(const LaunchCfg& c, const Workspace& ws);
cudaError_t launch_quantize_rows(const LaunchCfg& c, const float* x, int rows, int cols,
                                 int8_t* q, float2* ds);
cudaError_t launch_experts(const LaunchCfg& c, const float* h, const DevStack& gate,
                           const DevStack& up, const DevStack& down, const DevStack& sh_gate,
                           const DevStack& sh_up, const DevStack& sh_down, const Workspace& ws);
cudaError_t launch_combine(const LaunchCfg& c, const Workspace& ws, float* out, int accumulate);
cudaError_t launch_rms_norm(const LaunchCfg& c, const float* x, const float* w, float eps,
                            float* out);
cudaError_t launch_repack(int ty, const uint8_t* gguf_rows, uint8_t* dev_rows, int64_t n_rows,
                          int64_t cols, cudaStream_t stream);
cudaError_t launch_block_dots(int ty, const uint8_t* dev_row, int64_t cols, const int8_t* xq,
                              int32_t* out, cudaStream_t stream);
bool experts_supported(int ty, int cols, int rows, bool is_down);

void count_launch(int n = 1);

}  // namespace bivmoe
