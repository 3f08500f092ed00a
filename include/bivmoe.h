/*
 * bivmoe: the qwen35moe mixture-of-experts feed-forward layer of the biv
 * inference engine as hand-written CUDA for NVIDIA B200 (sm_100a), behind a C ABI.
 *
 * The reference engine (vincenthz/biv) has no per-operator plugin point: its
 * only backend seam is the whole-model trait set `Engine` / `Session` / `Batch`
 * (engine/src/engine.rs:15-60, 120-170, 282-323), implemented by the CPU
 * graph (`Model`) and by `MetalEngine`.  A CUDA backend is a third
 * implementation of those traits whose feed-forward step - the point where
 * the CPU backend calls `Model::moe` (engine/src/model.rs:788-790, 861-898)
 * and the Metal backend calls `encode_moe` (engine/src/metal/mod.rs:2095-2109,
 * 2140-2266) - calls this library once per layer.  Every entry point below
 * names the reference interface it stands in for.
 *
 * Conventions: every function returns a status (0 = ok); nothing aborts,
 * throws across the boundary or traps the device.  Calls that only enqueue work
 * on a stream return before it runs: what the device finds out later (a bounded
 * wait that gave up) is reported by `bivmoe_status`, which waits for the stream
 * (`bivmoe_host_wait` for the host-buffer calls).  A layer handle is not
 * thread-safe; distinct handles may be driven from distinct host threads.
 * Host pointers passed to `bivmoe_create` stay owned by the caller and may be
 * freed after it returns (the engine's GGUF mmap, src/lib.rs:74-84).
 */
#ifndef BIVMOE_H
#define BIVMOE_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BIVMOE_API __attribute__((visibility("default")))
#else
#define BIVMOE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  The Rust side maps them onto the reference's error enum
 * (engine/src/error.rs:36-40 NoKernel, 53-56 OutOfMemory, 67-68 Backend). */
enum {
    BIVMOE_OK = 0,
    BIVMOE_ERR_ARGUMENT = 1,    /* null pointer, size mismatch, n > max_tokens: Error::Backend */
    BIVMOE_ERR_UNSUPPORTED = 2, /* a ggml type or shape without a kernel: Error::NoKernel */
    BIVMOE_ERR_OOM = 3,         /* device allocation failed: Error::OutOfMemory{bytes} */
    BIVMOE_ERR_CUDA = 4,        /* a CUDA runtime call failed: Error::Backend */
    BIVMOE_ERR_NCCL = 5,        /* reserved: the library calls no collective (the exchanges are the
                                   caller's, or the library's own peer stores and barrier) */
    BIVMOE_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up: Error::Backend */
};

/* ggml type ids as stored in GGUF files (engine/src/quant.rs:30-48). */
enum {
    BIVMOE_F32 = 0,
    BIVMOE_F16 = 1,
    BIVMOE_Q4_0 = 2,
    BIVMOE_Q4_1 = 3,
    BIVMOE_Q8_0 = 8,
    BIVMOE_Q4_K = 12,
    BIVMOE_Q5_K = 13,
    BIVMOE_Q6_K = 14,
    BIVMOE_BF16 = 30,
};

/* A stack of same-shaped weight matrices, one per expert, inside one GGUF
 * tensor.  Field for field the reference's `Experts` (engine/src/model.rs:
 * 190-204): expert `i` starts at `data + i*stride_bytes + offset_bytes`
 * (model.rs:212-216), so the up half of a fused `ffn_gate_up_exps` tensor
 * (model.rs:389-399) is addressed without a copy.  `stride_bytes` 0 means
 * tightly packed (`rows * row_size(cols)`). */
typedef struct bivmoe_experts {
    int32_t ggml_type;
    int32_t reserved;
    int64_t cols;         /* elements per row (the product's inner dimension) */
    int64_t rows;         /* rows per expert */
    int64_t n;            /* experts in the stack (1 for the shared expert) */
    const void* data;     /* host memory, GGUF block layout */
    int64_t stride_bytes;
    int64_t offset_bytes;
} bivmoe_experts;

/* Everything `Loader::ffn` hands to the CPU and Metal backends for one layer
 * (engine/src/model.rs:377-421; `Moe` 230-237, `SharedExpert` 221-227,
 * `MoeConfig` 57-66; Metal's `gpu_layer`, engine/src/metal/mod.rs:584-605). */
typedef struct bivmoe_desc {
    int32_t n_embd;
    int32_t n_expert;
    int32_t n_expert_used;
    int32_t n_ff_exp;
    int32_t n_ff_shexp;   /* 0: no shared expert */
    int32_t max_tokens;   /* the largest n any forward call will pass */
    int32_t device;       /* CUDA device ordinal */
    int32_t reserved;
    const float* router;  /* host f32 [n_expert][n_embd], `ffn_gate_inp` */
    bivmoe_experts gate, up, down;
    bivmoe_experts sh_gate, sh_up, sh_down; /* ignored when n_ff_shexp == 0 */
    const float* sh_gate_inp;               /* host f32 [n_embd], `ffn_gate_inp_shexp` */
} bivmoe_desc;

typedef struct bivmoe_layer bivmoe_layer;

/* Upload one layer's tensors (repacked where a GGUF block is not 16-byte
 * sized) and allocate its workspace.  Stands in for `Loader::ffn` +
 * `gpu_layer` (model.rs:377-421; metal/mod.rs:584-605).  On failure *out is
 * NULL and `bivmoe_global_error` describes why. */
BIVMOE_API int bivmoe_create(const bivmoe_desc* desc, bivmoe_layer** out);
BIVMOE_API void bivmoe_destroy(bivmoe_layer* layer);

/* The dense feed-forward block of the qwen35 layers, `Ffn::Dense` (engine/src/model.rs:
 * 853-858; `dense_ffn`, 1119-1126): out = down(silu(gate h) * up h), the step the
 * mixture-of-experts layer replaces in the same place of the graph.  `gate` and `up` are
 * [n_ff x n_embd], `down` is [n_embd x n_ff], each with n = 1.  The layer object is a
 * mixture with one expert that every row selects with weight exactly 1 (a softmax over
 * one logit), so every other call of this header - forward, host forms, stack, taps -
 * takes it unchanged. */
BIVMOE_API int bivmoe_dense_create(int32_t device, int32_t n_embd, int32_t n_ff, int32_t max_tokens,
                                   const bivmoe_experts* gate, const bivmoe_experts* up,
                                   const bivmoe_experts* down, bivmoe_layer** out);

/* The layer on device rows: out[n][n_embd] = (accumulate ? out : 0) + moe(h).
 * `accumulate` 0 is `Model::moe`'s return value (model.rs:861-898);
 * 1 is Metal's `moe_combine`, which adds into the residual
 * (metal/kernels.metal:1885-1908), i.e. `moe` followed by the `add_inplace`
 * of model.rs:790.  Asynchronous on `stream` (a cudaStream_t); no host sync. */
BIVMOE_API int bivmoe_forward(bivmoe_layer* layer, const float* h_dev, float* out_dev, int32_t n,
                   int32_t accumulate, void* stream);

/* Waits for `stream` and reports what the layer's kernels recorded on the device since
 * the last report: BIVMOE_ERR_TIMEOUT when a bounded device-side wait (a copy that never
 * landed, a peer that never reached a barrier) gave up, in which case the outputs of the
 * passes since then are not to be used; BIVMOE_OK otherwise.  The flag is cleared by the
 * report.  For any layer, sharded or not.  Stands in for the `Result` a Metal command
 * buffer's completion yields (engine/src/metal/mod.rs:1535-1541, which panics instead). */
BIVMOE_API int bivmoe_status(bivmoe_layer* layer, void* stream);

/* The same call for an engine that keeps activations on the host (the CPU
 * backend's calling convention, `fn moe(&self, m, h: &[f32], n) -> Vec<f32>`,
 * model.rs:861): copies h in, runs the layer, copies the delta out and
 * waits for it.  Pinned host buffers make the copies asynchronous.  From 4096 rows on
 * the call works in sections of at least 2048 rows (up to five; from three on the first
 * and the last are half as long as the others, their copies being the ones nothing
 * overlaps): the copy-in of the next section and the copy-out of the last one run on
 * streams of their own beside the section at work (rows are independent, so the result
 * is the same; the taps then describe the last section).  BIVMOE_HOST_SECTIONS=1 in the
 * environment keeps one. */
BIVMOE_API int bivmoe_forward_host(bivmoe_layer* layer, const float* h_host, float* out_host, int32_t n);

/* The same in two halves, for a host that keeps several passes in flight (layers
 * of different micro-batches, each layer object with its own buffers): the first
 * enqueues copy-in, the layer, copy-out on the layer's own stream and returns;
 * the second waits for it and reports a device-side failure.  `out_host` is
 * complete, and `h_host` reusable, only after bivmoe_host_wait.  One pass per layer
 * object may be outstanding; page-locked buffers are needed for the copies to
 * overlap anything. */
BIVMOE_API int bivmoe_forward_host_async(bivmoe_layer* layer, const float* h_host, float* out_host,
                                         int32_t n);
BIVMOE_API int bivmoe_host_wait(bivmoe_layer* layer);

/* `bivmoe_forward` (accumulate 0) with CUDA events between its stages, for
 * benchmarks: waits for the pass and writes the device time of each stage in
 * milliseconds to ms[7] = {router product, softmax/top-k, sort, activation
 * quantiser, gate+up experts, down experts, combine}.  The reference times
 * this path only with wall clocks (examples/bench.rs:22-35). */
BIVMOE_API int bivmoe_forward_profile(bivmoe_layer* layer, const float* h_dev, float* out_dev,
                                      int32_t n, void* stream, float* ms);

/* The norm that precedes the layer in the graph (`post_norm`, model.rs:788;
 * ops.rs:136-149), needed by `bivmoe_forward_stack`.  `w` is host f32 [n_embd]. */
BIVMOE_API int bivmoe_set_post_norm(bivmoe_layer* layer, const float* w, float eps);

/* A run of layers with the residual carried on the device, FFN half of
 * `Model::layer` only (model.rs:788-790): per layer h = rms_norm(x, post_norm),
 * x += moe(h).  `x_dev` [n][n_embd] is updated in place.  Like `bivmoe_forward`, the
 * call replays its launches - of all layers - as one CUDA graph from the second call with
 * the same layers, buffer, n and (non-default) stream on. */
BIVMOE_API int bivmoe_forward_stack(bivmoe_layer* const* layers, int32_t n_layers, float* x_dev, int32_t n,
                         void* stream);

/* Intermediates of the last forward call, copied to host memory after a
 * stream sync: test-only, not on the timed path.  The reference has no such
 * hook; the oracle exposes the same quantities. */
enum {
    BIVMOE_TAP_LOGITS = 0,     /* f32 [n][n_expert] router logits */
    BIVMOE_TAP_IDS = 1,        /* i32 [n][k] experts in order of probability (model.rs:259-268) */
    BIVMOE_TAP_WEIGHTS = 2,    /* f32 [n][k] */
    BIVMOE_TAP_COUNTS = 3,     /* i32 [n_expert] pairs per expert */
    BIVMOE_TAP_ORDER = 4,      /* i32 [n*k] pair indices t*k+j grouped by expert, ascending */
    BIVMOE_TAP_ACT_Q = 5,      /* i8  [n][n_embd] Q8 rows of h (quant.rs:368-394) */
    BIVMOE_TAP_ACT_D = 6,      /* f32 [n][n_embd/32] */
    BIVMOE_TAP_ACT_S = 7,      /* f32 [n][n_embd/32] */
    BIVMOE_TAP_MID = 8,        /* f32 [n*k][n_ff_exp] silu(gate)*up by pair index */
    BIVMOE_TAP_PAIR_OUT = 9,   /* f32 [n*k][n_embd] expert outputs by pair index */
    BIVMOE_TAP_SHARED_OUT = 10,/* f32 [n][n_embd] */
    BIVMOE_TAP_SHARED_GATE = 11/* f32 [n] logit before the sigmoid */
};
BIVMOE_API int bivmoe_tap(bivmoe_layer* layer, int32_t which, void* host_dst, size_t bytes);

/* The int32 dot of every 32-element block of one weight row against one
 * quantised activation row of the last forward call - the integers the
 * reference's kernels produce before scaling (quant.rs:599-686; for Q6_K the
 * value includes the int8 sub-block scales).  matrix: 0 gate, 1 up, 2 down,
 * 3..5 the shared expert's; gate/up rows meet token `act_row`'s Q8 row of h,
 * down rows meet the Q8 row of pair `act_row`'s mid vector (pair index
 * t*k+j; for the shared expert, token t).  `out` is host i32 [cols/32]. */
BIVMOE_API int bivmoe_tap_block_dots(bivmoe_layer* layer, int32_t matrix, int32_t expert, int32_t row,
                          int32_t act_row, int32_t* out);

/* The routing step alone - router product, softmax, the k best experts and their
 * renormalised weights (what `route` computes per token, model.rs:259-268) - for
 * callers that cannot allocate device memory: code running under a stream capture,
 * inside another framework's memory pool, or in a latency-critical loop where a
 * cudaMalloc (which synchronises the device) is not acceptable.  It has no
 * counterpart in the reference; it exists because every other entry point relies
 * on the workspace `bivmoe_create` allocated.
 *
 * The call allocates nothing.  Its scratch (the router logits) is a fixed array
 * built into the library, `BIVMOE_ROUTE_NOALLOC_MAX_LOGITS` floats, which every GPU
 * that loads the library holds until the process exits; a call with
 * n * (n_expert + 1) beyond that limit is rejected with BIVMOE_ERR_ARGUMENT.
 * `h_dev` [n][n_embd] f32, `ids_dev` [n][n_expert_used] i32 and `weights_dev`
 * [n][n_expert_used] f32 are the caller's device buffers; results equal the
 * BIVMOE_TAP_IDS / BIVMOE_TAP_WEIGHTS of `bivmoe_forward` on the same rows.
 *
 * The first call on a device looks up the array's device address (a host-side
 * set-up step): make that first call before starting any stream capture.  All
 * calls share the one array, which keeps the previous call's logits; each call
 * overwrites every entry it reads, so nothing needs clearing, but two calls that
 * overlap on the GPU (different streams) race on it - serialise them. */
#define BIVMOE_ROUTE_NOALLOC_MAX_LOGITS (512 * 257)
BIVMOE_API int bivmoe_route_noalloc(bivmoe_layer* layer, const float* h_dev, int32_t n,
                                    int32_t* ids_dev, float* weights_dev, void* stream);

/* ---------------------------------------------------------------------------
 * Expert parallelism.  The reference runs on one device (one MTLDevice,
 * engine/src/metal/mod.rs:450-462; the CPU backend loops over the experts in
 * one process, engine/src/model.rs:875), so these entry points replace nothing
 * there: they split `Model::moe` (model.rs:861-898) into the steps either side
 * of two all-to-all exchanges that the CALLER performs (NCCL grouped
 * send/receive, or any transport that moves device rows), one process per GPU.
 *
 * Rank r of W holds experts [r * n_expert / W, (r + 1) * n_expert / W): `gate`,
 * `up`, `down` of the descriptor describe those n_expert / W experts only (for
 * a GGUF tensor: the same `data` and `stride_bytes`, `offset_bytes` advanced to
 * the rank's first expert, `n` = n_expert / W); `n_expert`, the router, the
 * shared expert and its gate vector are the whole layer's, on every rank.  Each
 * rank is the home of its own token rows.  A token's row travels once to every
 * rank that owns at least one of its k experts, and one partial sum per row
 * comes back.  One pass:
 *
 *   1. bivmoe_ep_route    home: router and top-k; writes, grouped by destination
 *                         rank and in token order inside a rank, the rows to
 *                         `send_rows_dev` [.][n_embd], their tags - the token's k
 *                         expert ids (i32) followed by its k weights (f32 bits) -
 *                         to `send_tags_dev` [.][2 * k], and the number of rows
 *                         for each rank to `send_counts_dev` [W].  At most
 *                         n * min(W, k) rows.
 *   2. caller             exchanges the counts (an all-gather), then rows and
 *                         tags: rank d receives, from every source in rank order,
 *                         that source's rows for d.
 *      bivmoe_ep_shared   home, any time after step 1 (e.g. on a second stream,
 *                         during the exchange): the shared expert over the rank's
 *                         own rows.
 *   3. bivmoe_ep_experts  owner: m received rows with their tags.  Writes to
 *                         `out_rows_dev` [m][n_embd], row for row, the weighted sum
 *                         over the experts THIS rank owns among the row's k:
 *                         sum_j w_j * down_j(silu(gate_j x) * (up_j x)), in
 *                         ascending expert id.
 *   4. caller             sends every row's partial sum back where the row came
 *                         from (the exchange of step 2 reversed).
 *   5. bivmoe_ep_combine  home: out[t] (+)= the partial sums of token t in ascending
 *                         rank (= ascending expert id), + sigmoid(gate) * shared[t].
 *
 * The result differs from bivmoe_forward on the same rows only in the association
 * of the f32 sum over a token's experts (by rank first).  All steps are
 * asynchronous on `stream`; the caller orders them against its exchanges.
 * `max_tokens` bounds n (a rank's own rows), `max_recv_rows` bounds m (W *
 * max_tokens is always enough).  bivmoe_ep_status synchronises the stream and
 * is bivmoe_status for a sharded layer.  With W = 1 bivmoe_ep_create is bivmoe_create
 * and bivmoe_forward applies. */
BIVMOE_API int bivmoe_ep_create(const bivmoe_desc* desc, int32_t ep_rank, int32_t ep_world,
                                int32_t max_recv_rows, bivmoe_layer** out);
BIVMOE_API int bivmoe_ep_route(bivmoe_layer* layer, const float* h_dev, int32_t n,
                               float* send_rows_dev, int32_t* send_tags_dev,
                               int32_t* send_counts_dev, void* stream);
BIVMOE_API int bivmoe_ep_shared(bivmoe_layer* layer, const float* h_dev, void* stream);
BIVMOE_API int bivmoe_ep_experts(bivmoe_layer* layer, const float* recv_rows_dev,
                                 const int32_t* recv_tags_dev, int32_t m, float* out_rows_dev,
                                 void* stream);
BIVMOE_API int bivmoe_ep_combine(bivmoe_layer* layer, const float* returned_rows_dev, float* out_dev,
                                 int32_t n, int32_t accumulate, void* stream);
BIVMOE_API int bivmoe_ep_status(bivmoe_layer* layer, void* stream);

/* The same pass with the exchanges done by the library's own kernels as stores into
 * the other ranks' memory (NVLink peer access), for ranks on the GPUs of one node.
 * Every rank owns one block holding a receive buffer, a return buffer, the tags and
 * the counts, each split in W regions of `max_tokens` rows, one per peer; a rank maps
 * the blocks of all ranks.  Steps 1-2 become one call whose kernels write each row
 * into region [home rank] of its owner's receive buffer; steps 3-4 one call whose last
 * kernel writes each partial sum into region [owner] of the home rank's return
 * buffer; a region's unused rows count as rows without experts.  No size depends on
 * another rank's counts, so the host never waits.  Two barriers order the stores against
 * their readers - the library's own (bivmoe_ep_peer_barrier, below) or any stream-ordered
 * barrier of the caller's communicator:
 *
 *   setup   bivmoe_ep_peer_info on every rank, the W results gathered to every rank (any
 *           transport), bivmoe_ep_peer_attach.  Ranks may be processes (the block is
 *           opened through its CUDA IPC handle) or threads of one process (the pointer
 *           is used as it is, peer access enabled between distinct devices).
 *   pass    bivmoe_ep_peer_dispatch(h, n)                    home: route, stores to owners
 *           barrier A (bivmoe_ep_peer_barrier, or e.g. a one-element all-reduce)
 *           bivmoe_ep_shared(h)            [may run beside the next call on another stream]
 *           bivmoe_ep_peer_experts()                         owner: experts, stores to homes
 *           barrier B
 *           bivmoe_ep_peer_combine(out, n, accumulate)       home
 *
 * Barrier A orders every rank's stores before the owners' reads; barrier B orders the
 * returned sums before the combine, and - every rank having finished its experts step -
 * the receive buffers against the next pass's stores.  All ranks pass the same
 * max_tokens, and max_recv_rows >= W * max_tokens.  The kernels only store to peers:
 * none waits on another GPU. */
typedef struct bivmoe_peer_info {
    uint8_t ipc_handle[64];   /* cudaIpcMemHandle_t of the rank's block */
    void* base;               /* the block in the owning process */
    int64_t pid;              /* the owning process */
    int64_t bytes;            /* the block's size: equal on all ranks */
    int32_t device;           /* the owning process's device ordinal */
    int32_t reserved;
} bivmoe_peer_info;
BIVMOE_API int bivmoe_ep_peer_info(bivmoe_layer* layer, bivmoe_peer_info* info);
BIVMOE_API int bivmoe_ep_peer_attach(bivmoe_layer* layer, const bivmoe_peer_info* all_ranks);
BIVMOE_API int bivmoe_ep_peer_dispatch(bivmoe_layer* layer, const float* h_dev, int32_t n, void* stream);
BIVMOE_API int bivmoe_ep_peer_experts(bivmoe_layer* layer, void* stream);
BIVMOE_API int bivmoe_ep_peer_combine(bivmoe_layer* layer, float* out_dev, int32_t n, int32_t accumulate,
                                      void* stream);

/* The barrier of the peer-store pass, inside the library: no communicator, no host step.
 * Every rank runs the same sequence of barriers.  `signal` stores this rank's next barrier
 * number into a word of every rank's block (after the stream's earlier stores);
 * `wait` holds the stream until every rank's number for this barrier is in this rank's
 * own block, or until the wait limit (2 s unless bivmoe_ep_peer_wait_limit says otherwise)
 * has passed - then the kernel records BIVMOE_ERR_TIMEOUT, which bivmoe_status reports,
 * and the stream goes on.  `barrier` is signal followed by wait.  The ranks must sit on
 * different GPUs for a wait to run beside the signals it waits for; where ranks share a
 * GPU (tests), enqueue every rank's signal before any rank's wait.  With these a whole
 * pass is five calls per rank and nothing else: dispatch, barrier, (shared,) experts,
 * barrier, combine.  The reference has no counterpart (one device). */
BIVMOE_API int bivmoe_ep_peer_signal(bivmoe_layer* layer, void* stream);
BIVMOE_API int bivmoe_ep_peer_wait(bivmoe_layer* layer, void* stream);
BIVMOE_API int bivmoe_ep_peer_barrier(bivmoe_layer* layer, void* stream);
BIVMOE_API int bivmoe_ep_peer_wait_limit(bivmoe_layer* layer, uint64_t microseconds);

/* The int8 tensor-pipe peak of the layer's GPU in tera-operations per second (two per
 * multiply-add), measured with back-to-back tcgen05.mma kind::i8 on resident operands
 * (about 10 ms).  A benchmark hook with no reference counterpart: the roofline
 * denominator of the Q8_0 tensor-core kernel. */
BIVMOE_API int bivmoe_int8_peak(bivmoe_layer* layer, double* tops);

/* What decides the numbers besides code and weights, as `Engine::numerics`
 * reports (engine.rs:42-46): device, kernel variants, repack version. */
BIVMOE_API int bivmoe_numerics(const bivmoe_layer* layer, char* buf, size_t len);

/* Bytes held on the device by this layer: weights and workspace
 * (`Engine::model_memory`, engine.rs:30; memory.rs:189-194). */
BIVMOE_API int bivmoe_memory(const bivmoe_layer* layer, uint64_t* weight_bytes, uint64_t* workspace_bytes);

/* Kernels this library launched since load, for benchmark accounting. */
BIVMOE_API uint64_t bivmoe_launch_count(void);

/* The size of the device allocation whose failure made the calling thread's last
 * BIVMOE_ERR_OOM: the `bytes` of `Error::OutOfMemory` (engine/src/error.rs:53-56). */
BIVMOE_API uint64_t bivmoe_last_oom_bytes(void);

BIVMOE_API const char* bivmoe_last_error(const bivmoe_layer* layer);
BIVMOE_API const char* bivmoe_global_error(void);

#ifdef __cplusplus
}
#endif
#endif /* BIVMOE_H */
