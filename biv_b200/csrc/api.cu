// The C ABI of include/bivmoe.h: layer objects, weight upload and repack,
// workspace, the forward sequence and the parity taps.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace bivmoe {

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

static thread_local std::string g_error;
static thread_local uint64_t g_oom_bytes = 0;   // size of the device allocation that failed last

// cudaMalloc that remembers the size of a failed request (Error::OutOfMemory{bytes})
static cudaError_t dev_alloc(void** p, size_t bytes) {
    const cudaError_t e = cudaMalloc(p, bytes);
    if (e == cudaErrorMemoryAllocation) g_oom_bytes = bytes;
    return e;
}

static int set_err(std::string* dst, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    (dst ? *dst : g_error) = buf;
    return code;
}

struct Arena {   // carves 256-byte aligned pieces out of one allocation
    size_t off = 0;
    uint8_t* base = nullptr;
    template <class T> T* take(size_t count) {
        size_t bytes = (count * sizeof(T) + 255) & ~(size_t)255;
        T* p = base && count ? (T*)(base + off) : nullptr;
        off += bytes;
        return p;
    }
};

}  // namespace bivmoe

using namespace bivmoe;

// bivmoe_forward_host: rows per section and the most sections of one call
constexpr int kHostSectionRows = 2048, kHostSectionsDefault = 4, kHostSectionsMax = 8;

struct bivmoe_layer {
    int device = 0, sm_count = 0;
    int e = 0, n_expert = 0, k = 0, ff = 0, ff_sh = 0, max_tokens = 0;
    bool has_shared = false;
    DevTiles gate_up, down, sh_gate_up, sh_down;
    float* router = nullptr;      // [n_expert + 1][e]; the last row is the shared-gate vector
    float* post_norm = nullptr;   // [e]
    float norm_eps = 0.0f;
    uint8_t* ws_mem = nullptr;
    size_t ws_bytes = 0, weight_bytes = 0;
    Workspace ws{};
    cudaStream_t own_stream = nullptr;   // bivmoe_forward_host
    // a host-buffer call over many rows runs in sections: the copy-in of the next section
    // and the copy-out of the last one (streams of their own) overlap the section at work
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    cudaEvent_t host_ev[2 * (kHostSectionsMax + 1) + 2] = {};
    float* host_in = nullptr;            // device staging of forward_host
    float* host_out = nullptr;
    int last_n = 0, host_last_n = 0;
    // the launch sequence of the last forward call, replayed as a CUDA graph while the
    // call's arguments stay the same (an engine passes the same scratch buffers each pass)
    struct {
        cudaGraphExec_t exec = nullptr;
        const float* h = nullptr;
        float* out = nullptr;
        int n = -1, accumulate = -1;
        cudaStream_t stream = nullptr;
        int seen = 0;            // identical calls seen; the graph is built on the second
    } graph;
    // bivmoe_forward_host with page-locked buffers: both copies, the launches and the
    // status read are one graph, replayed while the call's arguments stay the same
    struct {
        cudaGraphExec_t exec = nullptr;
        const float* h = nullptr;
        float* out = nullptr;
        int n = -1, seen = 0;
    } host_graph;
    // bivmoe_forward_stack, kept by the stack's first layer: the launches of all layers as
    // one graph, replayed while the same layers, rows and stream come back
    struct {
        cudaGraphExec_t exec = nullptr;
        std::vector<bivmoe_layer*> layers;
        float* x = nullptr;
        int n = -1, seen = 0;
        cudaStream_t stream = nullptr;
    } stack_graph;
    int32_t* status_host = nullptr;   // page-locked copy of the device status words
    int prefill_min = 0;   // set at create when the tcgen05 kernels support the layer's types
    int prefill_tile = kPrefillTile;
    // expert parallelism (bivmoe_ep_create): this rank's experts are global ids
    // ep_rank * n_local .. +n_local; `ws` serves the rank's own tokens (routing over all
    // experts, the shared expert), `ws_owner` the rows received for the local experts
    int ep_rank = 0, ep_world = 1, n_local = 0, max_recv = 0, ep_n = 0;
    Workspace ws_owner{};
    int32_t* ep_slot = nullptr;       // [max_tokens][world] a token's slot among a rank's rows, or -1
    int32_t* ep_counts = nullptr;     // [world] rows for each rank
    int32_t* ep_rank_ids = nullptr;   // [max_tokens][world] the rank, or -1: the home combine's "ids"
    int32_t* ep_rank_pos = nullptr;   // [max_tokens][world] the row's index among the sent rows
    float* ep_ones = nullptr;         // [max_tokens][world] the home combine's weights
    // the peer-store exchange (bivmoe_ep_peer_*): this rank's block, the ranks' blocks as
    // mapped into this process
    uint8_t* peer_block = nullptr;
    PeerLayout peer_lay{};
    PeerTable peers{};
    bool peers_attached = false;
    unsigned long long barrier_limit_ns = 2000000000ull;   // how long bivmoe_ep_peer_wait waits
    std::vector<void*> ipc_opened;
    bool use_graph = true;
    int launches_per_forward = 0;
    std::string error, device_name;
    std::vector<void*> allocs;
};

// One workspace: `N` rows of `k` pairs over `ne` experts.  `routed_rows` false: only
// the shared group's positions get activation buffers (the home side of expert
// parallelism, whose routed rows are computed elsewhere).
static void layout_one(bivmoe_layer* L, Arena& a, Workspace& w, size_t N, size_t k, size_t ne,
                       bool routed_rows) {
    const size_t P = N * k, e = L->e;
    const size_t mid = std::max(L->ff, L->ff_sh);
    w.logits = a.take<float>(N * (ne + 1));
    w.ids = a.take<int32_t>(P);
    w.weights = a.take<float>(P);
    w.counts = a.take<int32_t>(ne);
    w.offsets = a.take<int32_t>(ne + 1);
    w.order = a.take<int32_t>(((N + 7) / 8) * 8 + P + 8 * ne + 8 + kPrefillPad);
    w.pos_of = a.take<int32_t>(P);
    w.blk_counts = a.take<int32_t>(((N + 255) / 256) * ne);
    w.grp_expert = a.take<int32_t>(ne + 1);
    w.grp_start = a.take<int32_t>(ne + 1);
    w.grp_count = a.take<int32_t>(ne + 1);
    w.n_groups = a.take<int32_t>(1);
    const size_t tiles = P / 8 + N / 8 + ne + 2;
    w.tile_desc = a.take<int4>(tiles);
    w.n_tiles = a.take<int32_t>(2);
    const size_t ptiles = (P + N) / kPrefillTile + ne + 2;
    w.ptile_group = a.take<int32_t>(ptiles);
    w.ptile_t0 = a.take<int32_t>(ptiles);
    w.n_ptiles = a.take<int32_t>(2);
    w.work_ctr = a.take<uint32_t>(8);
    w.status = a.take<int32_t>(4);
    // positions: the tokens (shared group), then the routed groups, each padded to 8
    // (+kPrefillPad: a tile of the tcgen05 kernels copies up to that many positions from its first one)
    const size_t R = ((N + 7) / 8) * 8 + (routed_rows ? P + 8 * ne : 0) + 8 + kPrefillPad;
    w.act_rows = (int)R;
    const bool qact = !type_uses_f32_act(L->gate_up.ty) || (L->has_shared && !type_uses_f32_act(L->sh_gate_up.ty));
    const bool fact = type_uses_f32_act(L->gate_up.ty) || (L->has_shared && type_uses_f32_act(L->sh_gate_up.ty));
    const bool qmid = !type_uses_f32_act(L->down.ty) || (L->has_shared && !type_uses_f32_act(L->sh_down.ty));
    w.act_t = a.take<uint8_t>(qact ? (e / 256) * (R / 8) * kActTileBytes : 0);
    w.act_f = a.take<float>(fact ? R * e : 0);
    const bool brec = L->prefill_min > 0 && L->gate_up.ty == BIVMOE_BF16;   // bf16 hi/lo records
    w.tok_b = a.take<uint8_t>(brec ? N * (e / 64) * kTokBRec : 0);
    w.mid_b = a.take<uint8_t>(brec ? (mid / 64) * (R / 8) * kActBRec : 0);
    w.mid = a.take<float>(R * mid);
    w.mid_t = a.take<uint8_t>(qmid ? (mid / 256) * (R / 8) * kActTileBytes : 0);
    w.pair_out = a.take<float>(R * e);
    w.h_norm = a.take<float>(N * e);
    w.row_scale = a.take<float>(N);
}

static void layout_workspace(bivmoe_layer* L, Arena& a) {
    if (L->ep_world <= 1) {
        layout_one(L, a, L->ws, (size_t)L->max_tokens, (size_t)L->k, (size_t)L->n_expert, true);
        return;
    }
    layout_one(L, a, L->ws, (size_t)L->max_tokens, (size_t)L->k, (size_t)L->n_expert, false);
    layout_one(L, a, L->ws_owner, (size_t)L->max_recv, (size_t)L->k, (size_t)L->n_local, true);
    const size_t nw = (size_t)L->max_tokens * L->ep_world;
    L->ep_slot = a.take<int32_t>(nw);
    L->ep_counts = a.take<int32_t>((size_t)L->ep_world);
    L->ep_rank_ids = a.take<int32_t>(nw);
    L->ep_rank_pos = a.take<int32_t>(nw);
    L->ep_ones = a.take<float>(nw);
}

#define CU(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return set_err(errp, e_ == cudaErrorMemoryAllocation ? BIVMOE_ERR_OOM         \
                                                                 : BIVMOE_ERR_CUDA,       \
                           "%s: %s", #call, cudaGetErrorString(e_));                      \
    } while (0)

static int check_stack(std::string* errp, const char* name, const bivmoe_experts& s, int64_t cols,
                       int64_t rows, int64_t n, bool is_down) {
    if (!s.data) return set_err(errp, BIVMOE_ERR_ARGUMENT, "%s: null data", name);
    if (s.cols != cols || s.rows != rows || s.n != n)
        return set_err(errp, BIVMOE_ERR_ARGUMENT,
                       "%s: shape [%lld x %lld] x %lld, expected [%lld x %lld] x %lld", name,
                       (long long)s.rows, (long long)s.cols, (long long)s.n, (long long)rows,
                       (long long)cols, (long long)n);
    if (!experts_supported(s.ggml_type, (int)cols, (int)rows, is_down))
        return set_err(errp, BIVMOE_ERR_UNSUPPORTED,
                       "%s: no kernel for ggml type %d with %lld columns, %lld rows", name,
                       s.ggml_type, (long long)cols, (long long)rows);
    return BIVMOE_OK;
}

// Copies one product's stacks (gate and up, or down alone) to the device and
// repacks them into the tiled layout.
static int upload_tiles(bivmoe_layer* L, std::string* errp, const bivmoe_experts* a,
                        const bivmoe_experts* b, int chunk_rows, DevTiles* out) {
    const SliceGeom g = slice_geom(a->ggml_type);
    out->ty = a->ggml_type;
    out->cols = (int)a->cols; out->rows = (int)a->rows; out->n = (int)a->n;
    out->chunk_rows = chunk_rows;
    out->chunks = (int)(a->rows / chunk_rows);
    out->slice_bytes = g.sl;
    out->nslices = (int)(a->cols / g.elems);
    out->expert_bytes = (int64_t)out->chunks * out->nslices * kChunkRows * g.sl;
    const size_t dev_bytes = (size_t)(a->n * out->expert_bytes);
    void* p = nullptr;
    CU(dev_alloc(&p, dev_bytes));
    L->allocs.push_back(p);
    L->weight_bytes += dev_bytes;
    out->data = (uint8_t*)p;
    if (a->ggml_type == BIVMOE_Q6_K) {
        const size_t sb = (size_t)a->n * out->chunks * kChunkRows * out->nslices * 2;
        CU(dev_alloc(&p, sb));
        L->allocs.push_back(p);
        L->weight_bytes += sb;
        out->side = (uint16_t*)p;
    }
    const bivmoe_experts* srcs[2] = {a, b};
    for (int i = 0; i < 2; i++) {
        const bivmoe_experts* s = srcs[i];
        if (!s) continue;
        const int64_t mat = s->rows * gguf_row_bytes(s->ggml_type, s->cols);
        const int64_t stride = s->stride_bytes ? s->stride_bytes : mat;
        void* staging = nullptr;
        CU(dev_alloc(&staging, (size_t)(s->n * mat)));
        cudaError_t e1 = cudaMemcpy2D(staging, (size_t)mat, (const uint8_t*)s->data + s->offset_bytes,
                                      (size_t)stride, (size_t)mat, (size_t)s->n, cudaMemcpyHostToDevice);
        if (e1 == cudaSuccess) e1 = launch_repack(*out, (const uint8_t*)staging, 2 * i, 0);
        if (e1 == cudaSuccess) e1 = cudaDeviceSynchronize();
        cudaFree(staging);
        CU(e1);
    }
    return BIVMOE_OK;
}

namespace bivmoe {
// A read-only view of the routing tensors for entry points kept in other files;
// with `error_or_null` it instead records that text as the layer's last error.
int layer_route_view(bivmoe_layer* L, RouteView* out, const char* error_or_null) {
    if (!L) return BIVMOE_ERR_ARGUMENT;
    if (error_or_null) {
        L->error = error_or_null;
        return BIVMOE_OK;
    }
    *out = RouteView{L->device, L->sm_count, L->e, L->n_expert, L->k, L->has_shared ? 1 : 0,
                     L->router, L->ws.status};
    return BIVMOE_OK;
}
}  // namespace bivmoe

extern "C" {

const char* bivmoe_global_error(void) { return g_error.c_str(); }
const char* bivmoe_last_error(const bivmoe_layer* layer) {
    return layer ? layer->error.c_str() : g_error.c_str();
}
uint64_t bivmoe_launch_count(void) { return g_launches.load(); }
uint64_t bivmoe_last_oom_bytes(void) { return g_oom_bytes; }

void bivmoe_destroy(bivmoe_layer* L) {
    if (!L) return;
    DeviceScope on_device(L->device);
    if (L->graph.exec) cudaGraphExecDestroy(L->graph.exec);
    if (L->host_graph.exec) cudaGraphExecDestroy(L->host_graph.exec);
    if (L->stack_graph.exec) cudaGraphExecDestroy(L->stack_graph.exec);
    if (L->status_host) cudaFreeHost(L->status_host);
    for (void* p : L->ipc_opened) cudaIpcCloseMemHandle(p);
    for (void* p : L->allocs) cudaFree(p);
    if (L->own_stream) cudaStreamDestroy(L->own_stream);
    if (L->in_stream) cudaStreamDestroy(L->in_stream);
    if (L->out_stream) cudaStreamDestroy(L->out_stream);
    for (cudaEvent_t ev : L->host_ev)
        if (ev) cudaEventDestroy(ev);
    delete L;
}

static int create_impl(const bivmoe_desc* d, int ep_rank, int ep_world, int max_recv,
                       bivmoe_layer** out) {
    std::string* errp = nullptr;
    if (out) *out = nullptr;
    if (!d || !out) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null descriptor or output");
    if (ep_world < 1 || ep_rank < 0 || ep_rank >= ep_world)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "rank %d outside 0..%d", ep_rank, ep_world);
    if (ep_world > 1 && (d->n_expert % ep_world || max_recv <= 0 || ep_world > 32))
        return set_err(errp, BIVMOE_ERR_ARGUMENT,
                       "%d experts do not split over %d ranks (at most 32), or max_recv_rows %d is not positive",
                       d->n_expert, ep_world, max_recv);
    const int n_local = d->n_expert / ep_world;
    if (d->n_embd <= 0 || d->n_expert <= 0 || d->n_ff_exp <= 0 || d->max_tokens <= 0 || !d->router)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "non-positive dimension or null router");
    // model.rs:108-112: 1 <= n_expert_used <= n_expert
    if (d->n_expert_used < 1 || d->n_expert_used > d->n_expert || d->n_expert_used > 32)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "n_expert_used %d outside 1..min(%d, 32)",
                       d->n_expert_used, d->n_expert);
    if (d->n_expert > 1024)
        return set_err(errp, BIVMOE_ERR_UNSUPPORTED, "more than 1024 experts");
    if (d->n_embd % 256)
        return set_err(errp, BIVMOE_ERR_UNSUPPORTED, "n_embd %d is not a multiple of 256", d->n_embd);
    int rc;
    if ((rc = check_stack(errp, "ffn_gate_exps", d->gate, d->n_embd, d->n_ff_exp, n_local, false)) ||
        (rc = check_stack(errp, "ffn_up_exps", d->up, d->n_embd, d->n_ff_exp, n_local, false)) ||
        (rc = check_stack(errp, "ffn_down_exps", d->down, d->n_ff_exp, d->n_embd, n_local, true)))
        return rc;
    if (d->gate.ggml_type != d->up.ggml_type)
        return set_err(errp, BIVMOE_ERR_UNSUPPORTED, "gate and up of different types");
    const bool shared = d->n_ff_shexp > 0;
    if (shared) {
        if (!d->sh_gate_inp) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null ffn_gate_inp_shexp");
        if ((rc = check_stack(errp, "ffn_gate_shexp", d->sh_gate, d->n_embd, d->n_ff_shexp, 1, false)) ||
            (rc = check_stack(errp, "ffn_up_shexp", d->sh_up, d->n_embd, d->n_ff_shexp, 1, false)) ||
            (rc = check_stack(errp, "ffn_down_shexp", d->sh_down, d->n_ff_shexp, d->n_embd, 1, true)))
            return rc;
        if (d->sh_gate.ggml_type != d->sh_up.ggml_type)
            return set_err(errp, BIVMOE_ERR_UNSUPPORTED, "shared gate and up of different types");
    }
    DeviceScope on_device(d->device);   // the caller's device is current again on return
    {
        int cur = -1;
        CU(cudaGetDevice(&cur));
        if (cur != d->device) CU(cudaSetDevice(d->device));   // reports an invalid ordinal
    }
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, d->device));
    if (prop.major != 10)
        return set_err(errp, BIVMOE_ERR_UNSUPPORTED,
                       "device %d is sm_%d%d; this library is built for sm_100a only", d->device,
                       prop.major, prop.minor);
    bivmoe_layer* L = new (std::nothrow) bivmoe_layer();
    if (!L) return set_err(errp, BIVMOE_ERR_OOM, "host allocation failed");
    L->device = d->device;
    L->sm_count = prop.multiProcessorCount;
    L->device_name = prop.name;
    L->e = d->n_embd; L->n_expert = d->n_expert; L->k = d->n_expert_used;
    L->ff = d->n_ff_exp; L->ff_sh = d->n_ff_shexp; L->max_tokens = d->max_tokens;
    L->has_shared = shared;
    L->ep_rank = ep_rank; L->ep_world = ep_world; L->n_local = n_local; L->max_recv = max_recv;
    auto fail = [&](int code) { g_error = g_error.empty() ? L->error : g_error; bivmoe_destroy(L); return code; };
    if ((rc = upload_tiles(L, errp, &d->gate, &d->up, 64, &L->gate_up)) ||
        (rc = upload_tiles(L, errp, &d->down, nullptr, 128, &L->down)))
        return fail(rc);
    if (shared && ((rc = upload_tiles(L, errp, &d->sh_gate, &d->sh_up, 64, &L->sh_gate_up)) ||
                   (rc = upload_tiles(L, errp, &d->sh_down, nullptr, 128, &L->sh_down))))
        return fail(rc);
    auto cu_fail = [&](cudaError_t e, const char* what) {
        set_err(errp, e == cudaErrorMemoryAllocation ? BIVMOE_ERR_OOM : BIVMOE_ERR_CUDA, "%s: %s",
                what, cudaGetErrorString(e));
        return fail(e == cudaErrorMemoryAllocation ? BIVMOE_ERR_OOM : BIVMOE_ERR_CUDA);
    };
    cudaError_t ce;
    const size_t rbytes = (size_t)(L->n_expert + 1) * L->e * sizeof(float);
    if ((ce = dev_alloc((void**)&L->router, rbytes)) != cudaSuccess) return cu_fail(ce, "router");
    L->allocs.push_back(L->router);
    L->weight_bytes += rbytes;
    if ((ce = cudaMemset(L->router, 0, rbytes)) != cudaSuccess) return cu_fail(ce, "router");
    if ((ce = cudaMemcpy(L->router, d->router, (size_t)L->n_expert * L->e * 4,
                         cudaMemcpyHostToDevice)) != cudaSuccess)
        return cu_fail(ce, "router upload");
    if (shared && (ce = cudaMemcpy(L->router + (size_t)L->n_expert * L->e, d->sh_gate_inp,
                                   (size_t)L->e * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
        return cu_fail(ce, "shared gate upload");
    // groups of at least this many tokens run on the tcgen05 kernels, where they exist
    // for the layer's types (shared expert of the same types, or none).  Q8_0: the
    // warp-MMA kernels win below about 96 rows (0.25 / 0.41 ms against 0.29 / 0.44 ms per
    // pass of 512 / 1024 tokens).  BF16: the tcgen05 kernel sizes its MMA to the tile's rows
    // and reads the weights once per group, the float kernel once per 8 rows on the CUDA
    // cores: every group that needs more than one 8-row tile goes to the tensor core
    // (0.60 / 0.55 / 0.65 ms against 1.75 / 3.16 / 5.83 ms per pass of 512 / 1024 / 2048
    // tokens).
    if (prefill_supported(L->gate_up.ty, L->down.ty) &&
        (!shared || (L->sh_gate_up.ty == L->gate_up.ty && L->sh_down.ty == L->down.ty))) {
        const char* env = getenv("BIVMOE_PREFILL_MIN");
        L->prefill_min = env ? atoi(env) : L->gate_up.ty == BIVMOE_BF16 ? 9 : 96;
        L->prefill_tile = L->gate_up.ty == BIVMOE_BF16 ? kPrefillTileBf16 : kPrefillTile;
    }
    Arena probe;
    layout_workspace(L, probe);
    L->ws_bytes = probe.off;
    if ((ce = dev_alloc((void**)&L->ws_mem, L->ws_bytes)) != cudaSuccess) {
        set_err(errp, BIVMOE_ERR_OOM, "workspace of %zu bytes: %s", L->ws_bytes, cudaGetErrorString(ce));
        return fail(BIVMOE_ERR_OOM);
    }
    L->allocs.push_back(L->ws_mem);
    Arena real;
    real.base = L->ws_mem;
    layout_workspace(L, real);
    if ((ce = cudaMemset(L->ws.status, 0, 16)) != cudaSuccess) return cu_fail(ce, "status");
    if (ep_world > 1) {
        if ((ce = cudaMemset(L->ws_owner.status, 0, 16)) != cudaSuccess) return cu_fail(ce, "status");
        std::vector<float> ones((size_t)L->max_tokens * ep_world, 1.0f);
        if ((ce = cudaMemcpy(L->ep_ones, ones.data(), ones.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
            return cu_fail(ce, "weights of one");
    }
    if ((ce = cudaStreamCreateWithFlags(&L->own_stream, cudaStreamNonBlocking)) != cudaSuccess)
        return cu_fail(ce, "stream");
    if ((ce = cudaDeviceSynchronize()) != cudaSuccess) return cu_fail(ce, "upload");
    *out = L;
    return BIVMOE_OK;
}

int bivmoe_create(const bivmoe_desc* d, bivmoe_layer** out) { return create_impl(d, 0, 1, 0, out); }

int bivmoe_dense_create(int32_t device, int32_t n_embd, int32_t n_ff, int32_t max_tokens,
                        const bivmoe_experts* gate, const bivmoe_experts* up,
                        const bivmoe_experts* down, bivmoe_layer** out) {
    if (out) *out = nullptr;
    if (!gate || !up || !down || !out || n_embd <= 0)
        return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null pointer or non-positive n_embd");
    // one expert behind a router of zeros: softmax of one logit is 1, so is the
    // renormalised weight, and the combine's w * y is y
    std::vector<float> router((size_t)n_embd, 0.0f);
    bivmoe_desc d{};
    d.n_embd = n_embd; d.n_expert = 1; d.n_expert_used = 1;
    d.n_ff_exp = n_ff; d.n_ff_shexp = 0;
    d.max_tokens = max_tokens; d.device = device;
    d.router = router.data();
    d.gate = *gate; d.up = *up; d.down = *down;
    return create_impl(&d, 0, 1, 0, out);
}

int bivmoe_ep_create(const bivmoe_desc* d, int32_t ep_rank, int32_t ep_world, int32_t max_recv_rows,
                     bivmoe_layer** out) {
    if (ep_world == 1) return create_impl(d, 0, 1, 0, out);
    return create_impl(d, ep_rank, ep_world, max_recv_rows, out);
}

int bivmoe_set_post_norm(bivmoe_layer* L, const float* w, float eps) {
    if (!L || !w) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer or weights");
    std::string* errp = &L->error;
    DeviceScope on_device(L->device);
    if (!L->post_norm) {
        CU(dev_alloc((void**)&L->post_norm, (size_t)L->e * 4));
        L->allocs.push_back(L->post_norm);
        L->weight_bytes += (size_t)L->e * 4;
    }
    CU(cudaMemcpy(L->post_norm, w, (size_t)L->e * 4, cudaMemcpyHostToDevice));
    L->norm_eps = eps;
    return BIVMOE_OK;
}

// `norm`: `h` holds the residual rows and the router and dispatch kernels apply the
// layer's rms_norm themselves (bivmoe_forward_stack)
static int forward_impl(bivmoe_layer* L, const float* h, float* out, int n, int accumulate,
                        cudaStream_t stream, cudaEvent_t* ev = nullptr, const RowNorm* norm = nullptr) {
    std::string* errp = &L->error;
    if (n < 0 || n > L->max_tokens)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "n = %d outside 0..max_tokens = %d", n, L->max_tokens);
    if (n > 0 && (!h || !out)) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null activation pointer");
    if (L->ep_world > 1)
        return set_err(errp, BIVMOE_ERR_ARGUMENT,
                       "the layer holds 1/%d of the experts: use the bivmoe_ep_* steps", L->ep_world);
    L->last_n = n;
    if (n == 0) return BIVMOE_OK;
    LaunchCfg c{stream, n, L->k, L->e, L->n_expert, L->ff, L->ff_sh, L->has_shared ? 1 : 0, L->sm_count};
    c.ev = ev;
    c.prefill_min = L->prefill_min;
    c.prefill_tile = L->prefill_tile;
    mark(c, EV_START);
    CU(launch_router(c, L->router, h, L->ws, norm));
    mark(c, EV_ROUTER);
    CU(launch_route_topk(c, L->ws));
    mark(c, EV_TOPK);
    CU(launch_sort(c, L->ws));
    mark(c, EV_SORT);
    CU(launch_dispatch(c, h, L->ws, L->ws.act_t != nullptr, L->ws.act_f != nullptr, norm));
    mark(c, EV_QUANT);
    CU(launch_experts(c, L->gate_up, L->down, L->sh_gate_up, L->sh_down, L->ws));
    if (c.prefill_min > 0)
        CU(launch_experts_prefill(c, L->gate_up, L->down, L->sh_gate_up, L->sh_down, L->ws));
    mark(c, EV_DOWN);
    CU(launch_combine(c, combine_src(L->ws), out, accumulate));
    mark(c, EV_COMBINE);
    return BIVMOE_OK;
}

// forward_impl, replayed from a CUDA graph when the same call repeats: the seven
// launches then cost one graph launch and run back to back on the device.
static int forward_graphed(bivmoe_layer* L, const float* h, float* out, int n, int accumulate,
                           cudaStream_t stream) {
    std::string* errp = &L->error;
    auto& G = L->graph;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    // (the legacy default stream cannot be captured)
    if (!L->use_graph || n <= 0 || stream == nullptr || stream == cudaStreamLegacy ||
        cudaStreamIsCapturing(stream, &cap) != cudaSuccess ||
        cap != cudaStreamCaptureStatusNone)
        return forward_impl(L, h, out, n, accumulate, stream);   // also when the caller captures us
    const bool same = G.h == h && G.out == out && G.n == n && G.accumulate == accumulate &&
                      G.stream == stream;
    if (same && G.exec) {
        L->last_n = n;
        CU(cudaGraphLaunch(G.exec, stream));
        count_launch(L->launches_per_forward);
        return BIVMOE_OK;
    }
    if (!same) {
        if (G.exec) { cudaGraphExecDestroy(G.exec); G.exec = nullptr; }
        G.h = h; G.out = out; G.n = n; G.accumulate = accumulate; G.stream = stream;
        G.seen = 0;
    }
    if (++G.seen < 2)   // the first call runs plainly (it also sets the kernels' attributes)
        return forward_impl(L, h, out, n, accumulate, stream);
    cudaGraph_t graph = nullptr;
    const uint64_t before = bivmoe_launch_count();
    CU(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    int rc = forward_impl(L, h, out, n, accumulate, stream);
    cudaError_t ce = cudaStreamEndCapture(stream, &graph);
    L->launches_per_forward = (int)(bivmoe_launch_count() - before);
    if (rc || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        L->use_graph = false;   // fall back to plain launches for good
        cudaGetLastError();
        return rc ? rc : forward_impl(L, h, out, n, accumulate, stream);
    }
    ce = cudaGraphInstantiate(&G.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) {
        G.exec = nullptr;
        L->use_graph = false;
        cudaGetLastError();
        return forward_impl(L, h, out, n, accumulate, stream);
    }
    CU(cudaGraphLaunch(G.exec, stream));
    return BIVMOE_OK;
}

int bivmoe_forward(bivmoe_layer* L, const float* h_dev, float* out_dev, int32_t n,
                   int32_t accumulate, void* stream) {
    if (!L) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer");
    DeviceScope on_device(L->device);
    if (n < 0 || n > L->max_tokens)
        return set_err(&L->error, BIVMOE_ERR_ARGUMENT, "n = %d outside 0..max_tokens = %d", n,
                       L->max_tokens);
    if (n == 0) {   // no rows (their pointers may be null): nothing to do
        L->last_n = 0;
        return BIVMOE_OK;
    }
    if (!h_dev || !out_dev) return set_err(&L->error, BIVMOE_ERR_ARGUMENT, "null activation pointer");
    return forward_graphed(L, h_dev, out_dev, n, accumulate, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// expert parallelism: the device steps between the caller's two exchanges

static int ep_check(bivmoe_layer* L, const char* what) {
    if (!L) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer");
    if (L->ep_world <= 1)
        return set_err(&L->error, BIVMOE_ERR_ARGUMENT, "%s: the layer was not made by bivmoe_ep_create "
                       "with more than one rank", what);
    return BIVMOE_OK;
}

int bivmoe_ep_route(bivmoe_layer* L, const float* h_dev, int32_t n, float* send_rows_dev,
                    int32_t* send_tags_dev, int32_t* send_counts_dev, void* stream) {
    if (int rc = ep_check(L, "bivmoe_ep_route")) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    if (!h_dev || !send_rows_dev || !send_tags_dev || !send_counts_dev)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    if (n < 0 || n > L->max_tokens)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "n = %d outside 0..max_tokens = %d", n, L->max_tokens);
    cudaStream_t s = (cudaStream_t)stream;
    L->ep_n = n;
    L->last_n = n;
    if (n == 0) {
        CU(cudaMemsetAsync(send_counts_dev, 0, (size_t)L->ep_world * 4, s));
        return BIVMOE_OK;
    }
    LaunchCfg c{s, n, L->k, L->e, L->n_expert, L->ff, L->ff_sh, L->has_shared ? 1 : 0, L->sm_count};
    // the lists of the shared expert's group, which is computed here; its size decides
    // its kernel (the routed pairs are sorted by the ranks that own their experts)
    c.prefill_min = L->prefill_min;
    c.prefill_tile = L->prefill_tile;
    CU(launch_router(c, L->router, h_dev, L->ws));
    CU(launch_route_topk(c, L->ws));
    if (L->has_shared) CU(launch_shared_lists(c, L->ws));
    CU(launch_ep_gather(c, h_dev, L->ws, L->ep_world, L->n_local, L->ep_slot, L->ep_counts,
                        L->ep_rank_ids, L->ep_rank_pos, send_rows_dev, send_tags_dev, send_counts_dev));
    return BIVMOE_OK;
}

int bivmoe_ep_shared(bivmoe_layer* L, const float* h_dev, void* stream) {
    if (int rc = ep_check(L, "bivmoe_ep_shared")) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    const int n = L->ep_n;
    if (!L->has_shared || n == 0) return BIVMOE_OK;
    if (!h_dev) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    LaunchCfg c{s, n, 0, L->e, L->n_expert, L->ff, L->ff_sh, 1, L->sm_count};   // k = 0: no pair rows
    c.prefill_min = L->prefill_min;
    c.prefill_tile = L->prefill_tile;
    c.only_shared = 1;
    CU(launch_dispatch(c, h_dev, L->ws, L->ws.act_t != nullptr && !type_uses_f32_act(L->sh_gate_up.ty),
                       L->ws.act_f != nullptr && type_uses_f32_act(L->sh_gate_up.ty)));
    c.k = L->k;
    CU(launch_experts(c, L->gate_up, L->down, L->sh_gate_up, L->sh_down, L->ws));
    if (c.prefill_min > 0)
        CU(launch_experts_prefill(c, L->gate_up, L->down, L->sh_gate_up, L->sh_down, L->ws));
    return BIVMOE_OK;
}

int bivmoe_ep_experts(bivmoe_layer* L, const float* recv_rows_dev, const int32_t* recv_tags_dev,
                      int32_t m, float* out_rows_dev, void* stream) {
    if (int rc = ep_check(L, "bivmoe_ep_experts")) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    if (m < 0 || m > L->max_recv)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "m = %d outside 0..max_recv_rows = %d", m, L->max_recv);
    if (m == 0) return BIVMOE_OK;
    if (!recv_rows_dev || !recv_tags_dev || !out_rows_dev)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    // the received rows with their tags are a routing result over the local experts with
    // empty slots for the experts other ranks own; no shared expert here
    LaunchCfg c{s, m, L->k, L->e, L->n_local, L->ff, 0, 0, L->sm_count};
    c.prefill_min = L->prefill_min;
    c.prefill_tile = L->prefill_tile;
    const Workspace& w = L->ws_owner;
    const DevTiles none{};
    CU(launch_ep_localize(c, recv_tags_dev, L->ep_rank * L->n_local, w));
    CU(launch_sort(c, w));
    CU(launch_dispatch(c, recv_rows_dev, w, w.act_t != nullptr && !type_uses_f32_act(L->gate_up.ty),
                       w.act_f != nullptr && type_uses_f32_act(L->gate_up.ty)));
    CU(launch_experts(c, L->gate_up, L->down, none, none, w));
    if (c.prefill_min > 0) CU(launch_experts_prefill(c, L->gate_up, L->down, none, none, w));
    CU(launch_combine(c, combine_src(w), out_rows_dev, 0));   // the weighted sum over the local experts
    return BIVMOE_OK;
}

int bivmoe_ep_combine(bivmoe_layer* L, const float* returned_rows_dev, float* out_dev, int32_t n,
                      int32_t accumulate, void* stream) {
    if (int rc = ep_check(L, "bivmoe_ep_combine")) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    if (n != L->ep_n)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "n = %d, but bivmoe_ep_route ran on %d rows", n, L->ep_n);
    if (n == 0) return BIVMOE_OK;
    if (!returned_rows_dev || !out_dev) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    // the ranks take the experts' place: weight one, ascending rank = ascending expert id
    LaunchCfg c{(cudaStream_t)stream, n, L->ep_world, L->e, L->n_expert, L->ff, L->ff_sh,
                L->has_shared ? 1 : 0, L->sm_count};
    const CombineSrc src{L->ep_rank_ids, L->ep_ones, returned_rows_dev, L->ep_rank_pos, L->ws.pair_out,
                         L->ws.logits};
    CU(launch_combine(c, src, out_dev, accumulate));
    return BIVMOE_OK;
}

// ---- the peer-store exchange ------------------------------------------------------

static int peer_check(bivmoe_layer* L, const char* what, bool attached) {
    if (int rc = ep_check(L, what)) return rc;
    if (attached && !L->peers_attached)
        return set_err(&L->error, BIVMOE_ERR_ARGUMENT, "%s before bivmoe_ep_peer_attach", what);
    return BIVMOE_OK;
}

int bivmoe_ep_peer_info(bivmoe_layer* L, bivmoe_peer_info* info) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_info", false)) return rc;
    std::string* errp = &L->error;
    if (!info) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    DeviceScope on_device(L->device);
    if (!L->peer_block) {
        const size_t W = (size_t)L->ep_world, cap = (size_t)L->max_tokens, e = (size_t)L->e;
        if ((size_t)L->max_recv < W * cap)
            return set_err(errp, BIVMOE_ERR_ARGUMENT,
                           "max_recv_rows %d is below world * max_tokens = %zu, the rows of the regions",
                           L->max_recv, W * cap);
        PeerLayout lay{};
        lay.cap = (int)cap;
        lay.rows = 0;
        lay.returned = W * cap * e * 4;
        lay.tags = 2 * lay.returned;
        lay.counts = lay.tags + ((W * cap * 2 * (size_t)L->k * 4 + 255) & ~(size_t)255);
        lay.flags = lay.counts + 256;
        lay.bytes = lay.flags + 1024;
        void* p = nullptr;
        CU(dev_alloc(&p, lay.bytes));
        L->allocs.push_back(p);
        CU(cudaMemset(p, 0, lay.bytes));
        L->peer_block = (uint8_t*)p;
        L->peer_lay = lay;
        L->ws_bytes += lay.bytes;
    }
    memset(info, 0, sizeof(*info));
    cudaIpcMemHandle_t hnd;
    CU(cudaIpcGetMemHandle(&hnd, L->peer_block));
    static_assert(sizeof(hnd) == sizeof(info->ipc_handle), "cudaIpcMemHandle_t is 64 bytes");
    memcpy(info->ipc_handle, &hnd, sizeof(hnd));
    info->base = L->peer_block;
    info->pid = (int64_t)getpid();
    info->device = L->device;
    info->bytes = (int64_t)L->peer_lay.bytes;
    return BIVMOE_OK;
}

int bivmoe_ep_peer_attach(bivmoe_layer* L, const bivmoe_peer_info* all) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_attach", false)) return rc;
    std::string* errp = &L->error;
    if (!all) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    if (!L->peer_block) return set_err(errp, BIVMOE_ERR_ARGUMENT, "bivmoe_ep_peer_info comes first");
    if (L->peers_attached) return set_err(errp, BIVMOE_ERR_ARGUMENT, "already attached");
    DeviceScope on_device(L->device);
    for (int r = 0; r < L->ep_world; r++) {
        const bivmoe_peer_info& pi = all[r];
        if (pi.bytes != (int64_t)L->peer_lay.bytes)
            return set_err(errp, BIVMOE_ERR_ARGUMENT,
                           "rank %d's block has %lld bytes, this rank's %zu: the ranks' shapes differ", r,
                           (long long)pi.bytes, L->peer_lay.bytes);
        if (r == L->ep_rank) {
            L->peers.base[r] = L->peer_block;
        } else if (pi.pid == (int64_t)getpid()) {   // a rank of this process: its pointer as it is
            if (pi.device != L->device) {
                int can = 0;
                CU(cudaDeviceCanAccessPeer(&can, L->device, pi.device));
                if (!can)
                    return set_err(errp, BIVMOE_ERR_UNSUPPORTED, "device %d cannot map device %d's memory",
                                   L->device, pi.device);
                const cudaError_t pe = cudaDeviceEnablePeerAccess(pi.device, 0);
                if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) CU(pe);
                cudaGetLastError();
            }
            L->peers.base[r] = (uint8_t*)pi.base;
        } else {
            cudaIpcMemHandle_t hnd;
            memcpy(&hnd, pi.ipc_handle, sizeof(hnd));
            void* p = nullptr;
            CU(cudaIpcOpenMemHandle(&p, hnd, cudaIpcMemLazyEnablePeerAccess));
            L->ipc_opened.push_back(p);
            L->peers.base[r] = (uint8_t*)p;
        }
    }
    L->peers_attached = true;
    return BIVMOE_OK;
}

int bivmoe_ep_peer_dispatch(bivmoe_layer* L, const float* h_dev, int32_t n, void* stream) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_dispatch", true)) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    if (n < 0 || n > L->max_tokens)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "n = %d outside 0..max_tokens = %d", n, L->max_tokens);
    if (n > 0 && !h_dev) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    L->ep_n = n;
    LaunchCfg c{s, n, L->k, L->e, L->n_expert, L->ff, L->ff_sh, L->has_shared ? 1 : 0, L->sm_count};
    c.prefill_min = L->prefill_min;
    c.prefill_tile = L->prefill_tile;
    if (n > 0) {
        CU(launch_router(c, L->router, h_dev, L->ws));
        CU(launch_route_topk(c, L->ws));
        if (L->has_shared) CU(launch_shared_lists(c, L->ws));
    }
    CU(launch_ep_peer_scatter(c, h_dev, L->ws, L->ep_world, L->ep_rank, L->n_local, L->ep_slot, L->ep_counts,
                              L->ep_rank_ids, L->ep_rank_pos, L->peers, L->peer_lay));
    return BIVMOE_OK;
}

int bivmoe_ep_peer_experts(bivmoe_layer* L, void* stream) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_experts", true)) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    cudaStream_t s = (cudaStream_t)stream;
    const int m = L->ep_world * L->peer_lay.cap;
    LaunchCfg c{s, m, L->k, L->e, L->n_local, L->ff, 0, 0, L->sm_count};
    c.prefill_min = L->prefill_min;
    c.prefill_tile = L->prefill_tile;
    const Workspace& w = L->ws_owner;
    const DevTiles none{};
    const float* rows = (const float*)(L->peer_block + L->peer_lay.rows);
    CU(launch_ep_peer_localize(c, L->peer_block, L->peer_lay, L->ep_rank * L->n_local, w));
    CU(launch_sort(c, w));
    CU(launch_dispatch(c, rows, w, w.act_t != nullptr && !type_uses_f32_act(L->gate_up.ty),
                       w.act_f != nullptr && type_uses_f32_act(L->gate_up.ty)));
    CU(launch_experts(c, L->gate_up, L->down, none, none, w));
    if (c.prefill_min > 0) CU(launch_experts_prefill(c, L->gate_up, L->down, none, none, w));
    // the weighted sum over the local experts, stored where its home rank reads it
    CU(launch_combine_to_peers(c, combine_src(w), L->peer_block, L->ep_rank, L->peers, L->peer_lay));
    return BIVMOE_OK;
}

int bivmoe_ep_peer_combine(bivmoe_layer* L, float* out_dev, int32_t n, int32_t accumulate, void* stream) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_combine", true)) return rc;
    return bivmoe_ep_combine(L, (const float*)(L->peer_block + L->peer_lay.returned), out_dev, n, accumulate,
                             stream);
}

int bivmoe_ep_peer_signal(bivmoe_layer* L, void* stream) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_signal", true)) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    CU(launch_ep_peer_signal((cudaStream_t)stream, L->peer_block, L->ep_rank, L->ep_world, L->peers,
                             L->peer_lay));
    return BIVMOE_OK;
}

int bivmoe_ep_peer_wait(bivmoe_layer* L, void* stream) {
    if (int rc = peer_check(L, "bivmoe_ep_peer_wait", true)) return rc;
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    CU(launch_ep_peer_wait((cudaStream_t)stream, L->peer_block, L->ep_world, L->peer_lay,
                           L->barrier_limit_ns, L->ws.status));
    return BIVMOE_OK;
}

int bivmoe_ep_peer_barrier(bivmoe_layer* L, void* stream) {
    if (int rc = bivmoe_ep_peer_signal(L, stream)) return rc;
    return bivmoe_ep_peer_wait(L, stream);
}

int bivmoe_ep_peer_wait_limit(bivmoe_layer* L, uint64_t microseconds) {
    if (int rc = ep_check(L, "bivmoe_ep_peer_wait_limit")) return rc;
    if (microseconds == 0 || microseconds > 60000000ull)
        return set_err(&L->error, BIVMOE_ERR_ARGUMENT, "a wait limit of %llu us is outside 1 us .. 60 s",
                       (unsigned long long)microseconds);
    L->barrier_limit_ns = microseconds * 1000ull;
    return BIVMOE_OK;
}

int bivmoe_status(bivmoe_layer* L, void* stream) {
    if (!L) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer");
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    cudaStream_t s = (cudaStream_t)stream;
    const bool ep = L->ep_world > 1;
    int32_t st[2][4] = {};
    CU(cudaMemcpyAsync(st[0], L->ws.status, 16, cudaMemcpyDeviceToHost, s));
    if (ep) CU(cudaMemcpyAsync(st[1], L->ws_owner.status, 16, cudaMemcpyDeviceToHost, s));
    CU(cudaStreamSynchronize(s));
    if (st[0][0] || st[1][0]) {
        cudaMemsetAsync(L->ws.status, 0, 16, s);
        if (ep) cudaMemsetAsync(L->ws_owner.status, 0, 16, s);
        const int which = st[0][0] ? 0 : 1;
        return set_err(errp, st[which][0], "a device-side bounded wait gave up (status %d, wait site %d)",
                       st[which][0], st[which][2]);
    }
    return BIVMOE_OK;
}

int bivmoe_ep_status(bivmoe_layer* L, void* stream) {
    if (int rc = ep_check(L, "bivmoe_ep_status")) return rc;
    return bivmoe_status(L, stream);
}

int bivmoe_forward_profile(bivmoe_layer* L, const float* h_dev, float* out_dev, int32_t n,
                           void* stream, float* ms) {
    if (!L || !ms) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer or buffer");
    DeviceScope on_device(L->device);
    std::string* errp = &L->error;
    cudaEvent_t ev[EV_COUNT];
    for (int i = 0; i < EV_COUNT; i++) CU(cudaEventCreate(&ev[i]));
    int rc = forward_impl(L, h_dev, out_dev, n, 0, (cudaStream_t)stream, ev);
    cudaError_t ce = cudaEventSynchronize(ev[EV_COMBINE]);
    for (int i = 1; i < EV_COUNT && ce == cudaSuccess && !rc; i++)
        ce = cudaEventElapsedTime(&ms[i - 1], ev[i - 1], ev[i]);
    for (int i = 0; i < EV_COUNT; i++) cudaEventDestroy(ev[i]);
    if (rc) return rc;
    CU(ce);
    return BIVMOE_OK;
}

static bool page_locked(const void* p) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

// How many sections a host-buffer call of n rows runs in.  The layer is row-wise, so a
// section's result does not depend on the rows of the others; a section should still be
// large enough for the tensor-core kernels' 128-row tiles to fill (rows per expert =
// section * k / n_expert).  BIVMOE_HOST_SECTIONS overrides the rule (1 = no overlap).
static int host_sections(const bivmoe_layer* L, int n) {
    static const int forced = [] {
        const char* v = getenv("BIVMOE_HOST_SECTIONS");
        return v ? atoi(v) : 0;
    }();
    int c = forced > 0 ? forced : std::min(n / kHostSectionRows, kHostSectionsDefault);
    c = std::min(c, kHostSectionsMax);
    c = std::min(c, n / 8);
    return std::max(c, 1);
}

// copy in, the layer, copy out, status out - enqueued on the layer's own stream; with
// more than one section the copies run on two more streams, forked from and joined to it
// by events (so that the whole can be captured from the layer's stream)
static int forward_host_enqueue(bivmoe_layer* L, const float* h_host, float* out_host, int n) {
    std::string* errp = &L->error;
    const size_t bytes = (size_t)n * L->e * 4;
    cudaStream_t s = L->own_stream;
    const int sections = host_sections(L, n);
    if (sections > 1) {
        cudaStream_t si = L->in_stream, so = L->out_stream;
        cudaEvent_t* ev = L->host_ev;
        cudaEvent_t fork = ev[2 * (kHostSectionsMax + 1)], join = ev[2 * (kHostSectionsMax + 1) + 1];
        // Section boundaries.  With three sections or more the first and the last are half
        // as long as the others (one more section in all): what cannot overlap anything is
        // the first section's copy-in and the last one's copy-out.
        int bound[kHostSectionsMax + 2];
        int nsec = 0;
        {
            const int per = ((n + sections - 1) / sections + 7) / 8 * 8;
            const int edge = sections >= 3 ? (per / 2 + 7) / 8 * 8 : per;
            bound[0] = 0;
            for (int t0 = edge; t0 < n; t0 += (n - t0 > per + edge / 2 ? per : n - t0)) bound[++nsec] = t0;
            bound[++nsec] = n;
            if (sections >= 3 && nsec >= 3 && bound[nsec] - bound[nsec - 1] > edge) {
                // the tail came out long: cut it so that the last section is an edge
                const int cut = (bound[nsec] - edge) / 8 * 8;
                if (cut > bound[nsec - 1] && nsec < kHostSectionsMax + 1) {
                    bound[nsec + 1] = bound[nsec];
                    bound[nsec] = cut;
                    nsec++;
                }
            }
        }
        CU(cudaEventRecord(fork, s));
        CU(cudaStreamWaitEvent(si, fork, 0));
        CU(cudaStreamWaitEvent(so, fork, 0));
        for (int c = 0; c < nsec; c++) {
            const size_t off = (size_t)bound[c] * L->e, nb = (size_t)(bound[c + 1] - bound[c]) * L->e * 4;
            CU(cudaMemcpyAsync(L->host_in + off, h_host + off, nb, cudaMemcpyHostToDevice, si));
            CU(cudaEventRecord(ev[2 * c], si));
        }
        int last = 0;
        for (int c = 0; c < nsec; c++) {
            const size_t off = (size_t)bound[c] * L->e;
            last = bound[c + 1] - bound[c];
            CU(cudaStreamWaitEvent(s, ev[2 * c], 0));
            if (int rc = forward_impl(L, L->host_in + off, L->host_out + off, last, 0, s)) return rc;
            CU(cudaEventRecord(ev[2 * c + 1], s));
            CU(cudaStreamWaitEvent(so, ev[2 * c + 1], 0));
            CU(cudaMemcpyAsync(out_host + off, L->host_out + off, (size_t)last * L->e * 4,
                               cudaMemcpyDeviceToHost, so));
        }
        CU(cudaEventRecord(join, so));
        CU(cudaStreamWaitEvent(s, join, 0));
        CU(cudaMemcpyAsync(L->status_host, L->ws.status, 16, cudaMemcpyDeviceToHost, s));
        L->host_last_n = last;   // what the workspace holds afterwards: the last section
        return BIVMOE_OK;
    }
    L->host_last_n = n;
    CU(cudaMemcpyAsync(L->host_in, h_host, bytes, cudaMemcpyHostToDevice, s));
    int rc = forward_graphed(L, L->host_in, L->host_out, n, 0, s);   // plain launches under a capture
    if (rc) return rc;
    CU(cudaMemcpyAsync(out_host, L->host_out, bytes, cudaMemcpyDeviceToHost, s));
    CU(cudaMemcpyAsync(L->status_host, L->ws.status, 16, cudaMemcpyDeviceToHost, s));
    return BIVMOE_OK;
}

int bivmoe_forward_host_async(bivmoe_layer* L, const float* h_host, float* out_host, int32_t n) {
    if (!L) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer");
    std::string* errp = &L->error;
    if (n < 0 || n > L->max_tokens)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "n = %d outside 0..max_tokens = %d", n, L->max_tokens);
    if (n == 0) {
        L->last_n = 0;
        return BIVMOE_OK;
    }
    if (!h_host || !out_host) return set_err(errp, BIVMOE_ERR_ARGUMENT, "null host pointer");
    DeviceScope on_device(L->device);
    if (!L->host_in) {
        const size_t bytes = (size_t)L->max_tokens * L->e * 4;
        CU(dev_alloc((void**)&L->host_in, bytes));
        L->allocs.push_back(L->host_in);
        CU(dev_alloc((void**)&L->host_out, bytes));
        L->allocs.push_back(L->host_out);
        L->ws_bytes += 2 * bytes;
        CU(cudaHostAlloc((void**)&L->status_host, 16, cudaHostAllocDefault));
        CU(cudaStreamCreateWithFlags(&L->in_stream, cudaStreamNonBlocking));
        CU(cudaStreamCreateWithFlags(&L->out_stream, cudaStreamNonBlocking));
        for (cudaEvent_t& ev : L->host_ev) CU(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    }
    cudaStream_t s = L->own_stream;
    auto& G = L->host_graph;
    const bool same = G.h == h_host && G.out == out_host && G.n == n;
    if (!same) {
        if (G.exec) { cudaGraphExecDestroy(G.exec); G.exec = nullptr; }
        G.h = h_host; G.out = out_host; G.n = n; G.seen = 0;
    }
    bool launched = false;
    if (G.exec) {
        CU(cudaGraphLaunch(G.exec, s));
        count_launch(L->launches_per_forward);
        launched = true;
    } else if (L->use_graph && ++G.seen >= 2 && page_locked(h_host) && page_locked(out_host)) {
        // the second identical call with page-locked buffers: capture the whole sequence
        cudaGraph_t graph = nullptr;
        const uint64_t before = bivmoe_launch_count();
        CU(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        const int rc = forward_host_enqueue(L, h_host, out_host, n);
        cudaError_t ce = cudaStreamEndCapture(s, &graph);
        L->launches_per_forward = (int)(bivmoe_launch_count() - before);
        if (!rc && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&G.exec, graph, 0);
        if (graph) cudaGraphDestroy(graph);
        if (rc || ce != cudaSuccess) {
            G.exec = nullptr;
            L->use_graph = false;   // plain launches from here on
            cudaGetLastError();
            if (rc) return rc;
        } else {
            CU(cudaGraphLaunch(G.exec, s));
            launched = true;
        }
    }
    if (!launched) {
        int rc = forward_host_enqueue(L, h_host, out_host, n);
        if (rc) return rc;
    }
    L->last_n = L->host_last_n;
    return BIVMOE_OK;
}

int bivmoe_host_wait(bivmoe_layer* L) {
    if (!L) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer");
    std::string* errp = &L->error;
    if (!L->status_host) return BIVMOE_OK;   // no host-buffer call was ever made
    DeviceScope on_device(L->device);
    cudaStream_t s = L->own_stream;
    CU(cudaStreamSynchronize(s));
    if (L->status_host[0]) {
        const int code = L->status_host[0];
        cudaMemsetAsync(L->ws.status, 0, 16, s);
        return set_err(errp, code, "a device-side bounded wait gave up (status %d)", code);
    }
    return BIVMOE_OK;
}

int bivmoe_forward_host(bivmoe_layer* L, const float* h_host, float* out_host, int32_t n) {
    if (int rc = bivmoe_forward_host_async(L, h_host, out_host, n)) return rc;
    return n > 0 ? bivmoe_host_wait(L) : BIVMOE_OK;
}

// the launches of every layer of the stack, in order, on `stream`
static int stack_enqueue(bivmoe_layer* const* layers, int n_layers, float* x_dev, int n, cudaStream_t stream) {
    for (int l = 0; l < n_layers; l++) {
        bivmoe_layer* L = layers[l];
        std::string* errp = &L->error;
        DeviceScope on_device(L->device);
        LaunchCfg c{stream, n, L->k, L->e, L->n_expert, L->ff, L->ff_sh, L->has_shared ? 1 : 0, L->sm_count};
        int rc;
        if (router_fuses_norm(n, L->e)) {
            // the router kernel normalises the rows it stages and publishes the scales; the
            // dispatch kernel applies them on the fly: the normed rows never reach HBM
            const RowNorm norm{L->post_norm, L->norm_eps, L->ws.row_scale};
            rc = forward_impl(L, x_dev, x_dev, n, 1, stream, nullptr, &norm);
        } else {
            CU(launch_rms_norm(c, x_dev, L->post_norm, L->norm_eps, L->ws.h_norm));
            rc = forward_impl(L, L->ws.h_norm, x_dev, n, 1, stream);
        }
        if (rc) return rc;
    }
    return BIVMOE_OK;
}

int bivmoe_forward_stack(bivmoe_layer* const* layers, int32_t n_layers, float* x_dev, int32_t n,
                         void* stream) {
    if (!layers || n_layers <= 0 || !layers[0])
        return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "no layers");
    bool one_device = true;
    for (int l = 0; l < n_layers; l++) {
        bivmoe_layer* L = layers[l];
        std::string* errp = L ? &L->error : nullptr;
        if (!L || !L->post_norm)
            return set_err(errp, BIVMOE_ERR_ARGUMENT, "layer %d has no post_norm weights", l);
        if (n < 0 || n > L->max_tokens)
            return set_err(errp, BIVMOE_ERR_ARGUMENT, "n = %d outside 0..max_tokens", n);
        one_device = one_device && L->device == layers[0]->device;
    }
    if (n == 0) return BIVMOE_OK;
    // The same stack over the same rows again (an engine's decode loop): the launches of all
    // layers - 7 each - are replayed as one graph from the second identical call on.
    bivmoe_layer* L0 = layers[0];
    std::string* errp = &L0->error;
    cudaStream_t s = (cudaStream_t)stream;
    auto& G = L0->stack_graph;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    const bool can_graph = L0->use_graph && one_device && s != nullptr && s != cudaStreamLegacy &&
                           cudaStreamIsCapturing(s, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone;
    if (!can_graph) return stack_enqueue(layers, n_layers, x_dev, n, s);
    DeviceScope on_device(L0->device);
    const bool same = G.x == x_dev && G.n == n && G.stream == s && (int)G.layers.size() == n_layers &&
                      std::equal(G.layers.begin(), G.layers.end(), layers);
    if (same && G.exec) {
        CU(cudaGraphLaunch(G.exec, s));
        count_launch(L0->launches_per_forward * n_layers);
        for (int l = 0; l < n_layers; l++) layers[l]->last_n = n;
        return BIVMOE_OK;
    }
    if (!same) {
        if (G.exec) { cudaGraphExecDestroy(G.exec); G.exec = nullptr; }
        G.layers.assign(layers, layers + n_layers);
        G.x = x_dev; G.n = n; G.stream = s; G.seen = 0;
    }
    if (++G.seen < 2) return stack_enqueue(layers, n_layers, x_dev, n, s);   // the first call also sets kernel attributes
    cudaGraph_t graph = nullptr;
    const uint64_t before = bivmoe_launch_count();
    CU(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    const int rc = stack_enqueue(layers, n_layers, x_dev, n, s);
    cudaError_t ce = cudaStreamEndCapture(s, &graph);
    L0->launches_per_forward = (int)((bivmoe_launch_count() - before) / n_layers);
    if (!rc && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&G.exec, graph, 0);
    if (graph) cudaGraphDestroy(graph);
    if (rc || ce != cudaSuccess) {
        G.exec = nullptr;
        L0->use_graph = false;   // plain launches from here on
        cudaGetLastError();
        return rc ? rc : stack_enqueue(layers, n_layers, x_dev, n, s);
    }
    CU(cudaGraphLaunch(G.exec, s));
    return BIVMOE_OK;
}

// ---------------------------------------------------------------------------
// taps

static int copy_out(bivmoe_layer* L, void* dst, const void* src, size_t want, size_t have) {
    std::string* errp = &L->error;
    if (want != have)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "tap buffer of %zu bytes, expected %zu", want, have);
    CU(cudaMemcpy(dst, src, have, cudaMemcpyDeviceToHost));
    return BIVMOE_OK;
}

int bivmoe_tap(bivmoe_layer* L, int32_t which, void* dst, size_t bytes) {
    if (!L || !dst) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer or buffer");
    std::string* errp = &L->error;
    if (L->ep_world > 1)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "taps read a whole layer's workspace; this layer is sharded");
    CU(cudaSetDevice(L->device));
    CU(cudaDeviceSynchronize());
    const size_t n = (size_t)L->last_n, k = L->k, ne = L->n_expert, e = L->e, P = n * k;
    const size_t mid = std::max(L->ff, L->ff_sh);
    const Workspace& w = L->ws;
    switch (which) {
        case BIVMOE_TAP_LOGITS:
        case BIVMOE_TAP_SHARED_GATE: {
            std::vector<float> tmp(n * (ne + 1));
            CU(cudaMemcpy(tmp.data(), w.logits, tmp.size() * 4, cudaMemcpyDeviceToHost));
            const bool lg = which == BIVMOE_TAP_LOGITS;
            if (bytes != (lg ? n * ne : n) * 4)
                return set_err(errp, BIVMOE_ERR_ARGUMENT, "tap buffer size mismatch");
            float* o = (float*)dst;
            for (size_t t = 0; t < n; t++) {
                if (lg) memcpy(o + t * ne, tmp.data() + t * (ne + 1), ne * 4);
                else o[t] = tmp[t * (ne + 1) + ne];
            }
            return BIVMOE_OK;
        }
        case BIVMOE_TAP_IDS: return copy_out(L, dst, w.ids, bytes, P * 4);
        case BIVMOE_TAP_WEIGHTS: return copy_out(L, dst, w.weights, bytes, P * 4);
        case BIVMOE_TAP_COUNTS: return copy_out(L, dst, w.counts, bytes, ne * 4);
        case BIVMOE_TAP_ORDER: {   // the padded position space, compacted expert by expert
            if (bytes != P * 4) return set_err(errp, BIVMOE_ERR_ARGUMENT, "tap buffer size mismatch");
            std::vector<int32_t> cnt(ne), off(ne + 1), ord(w.act_rows);
            CU(cudaMemcpy(cnt.data(), w.counts, ne * 4, cudaMemcpyDeviceToHost));
            CU(cudaMemcpy(off.data(), w.offsets, (ne + 1) * 4, cudaMemcpyDeviceToHost));
            CU(cudaMemcpy(ord.data(), w.order, ord.size() * 4, cudaMemcpyDeviceToHost));
            size_t o = 0;
            for (size_t x = 0; x < ne; x++)
                for (int j = 0; j < cnt[x]; j++) ((int32_t*)dst)[o++] = ord[off[x] + j];
            return BIVMOE_OK;
        }
        case BIVMOE_TAP_ACT_Q:
        case BIVMOE_TAP_ACT_D:
        case BIVMOE_TAP_ACT_S: {
            // the tokens' rows are positions 0..n of the slice-major arrays
            if (!w.act_t) return set_err(errp, BIVMOE_ERR_ARGUMENT, "no quantised activations");
            const size_t R = w.act_rows, nsl = e / 256;
            const bool q = which == BIVMOE_TAP_ACT_Q;
            if (bytes != (q ? n * e : n * e / 32 * 4))
                return set_err(errp, BIVMOE_ERR_ARGUMENT, "tap buffer size mismatch");
            // a token's row: its position in the shared group, else its first pair's position
            std::vector<int32_t> tpos(n);
            for (size_t t = 0; t < n; t++) tpos[t] = (int32_t)t;
            if (!L->has_shared)
                CU(cudaMemcpy2D(tpos.data(), 4, w.pos_of, (size_t)k * 4, 4, n, cudaMemcpyDeviceToHost));
            std::vector<uint8_t> rec(nsl * (R / 8) * kActTileBytes);
            CU(cudaMemcpy(rec.data(), w.act_t, rec.size(), cudaMemcpyDeviceToHost));
            for (size_t t = 0; t < n; t++)
                for (size_t sl = 0; sl < nsl; sl++) {
                    const uint8_t* r0 = rec.data() + (sl * (R / 8) + tpos[t] / 8) * kActTileBytes;
                    const int tk = tpos[t] % 8;
                    if (q)
                        for (int i = 0; i < 256; i++)
                            ((int8_t*)dst)[t * e + sl * 256 + i] = (int8_t)r0[act_q_off(tk, i)];
                    else
                        for (int b = 0; b < 8; b++)
                            ((float*)dst)[t * (e / 32) + sl * 8 + b] = *(const float*)(
                                r0 + (which == BIVMOE_TAP_ACT_S ? kActOffS : kActOffDx) + (b * 8 + tk) * 4);
                }
            return BIVMOE_OK;
        }
        case BIVMOE_TAP_MID: {
            const size_t R = w.act_rows, ffw = L->ff;
            if (bytes != P * ffw * 4) return set_err(errp, BIVMOE_ERR_ARGUMENT, "tap buffer size mismatch");
            std::vector<float> tmp(R * mid);
            std::vector<int32_t> pos(P);
            CU(cudaMemcpy(tmp.data(), w.mid, tmp.size() * 4, cudaMemcpyDeviceToHost));
            CU(cudaMemcpy(pos.data(), w.pos_of, P * 4, cudaMemcpyDeviceToHost));
            // pairs of groups the BF16 tensor-core kernels took have no f32 mid row: theirs is
            // the sum of the two bf16 terms the down product reads (mid to 2^-17)
            std::vector<uint8_t> terms;
            std::vector<int32_t> ids, cnt;
            const bool has_terms = w.mid_b && L->prefill_min > 0;
            if (has_terms) {
                terms.resize((mid / 64) * (R / 8) * (size_t)kActBRec);
                ids.resize(P);
                cnt.resize(ne);
                CU(cudaMemcpy(terms.data(), w.mid_b, terms.size(), cudaMemcpyDeviceToHost));
                CU(cudaMemcpy(ids.data(), w.ids, P * 4, cudaMemcpyDeviceToHost));
                CU(cudaMemcpy(cnt.data(), w.counts, ne * 4, cudaMemcpyDeviceToHost));
            }
            auto bf = [](uint16_t v) { uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4); return f; };
            for (size_t p = 0; p < P; p++) {
                float* o = (float*)dst + p * ffw;
                if (pos[p] < 0) { memset(o, 0, ffw * 4); continue; }
                const bool big = has_terms && ids[p] >= 0 && cnt[ids[p]] >= L->prefill_min;
                for (size_t sl = 0; sl < ffw / 64; sl++) {
                    if (!big) {
                        memcpy(o + sl * 64, tmp.data() + (sl * R + pos[p]) * 64, 256);
                        continue;
                    }
                    const uint8_t* rec = terms.data() + (sl * (R / 8) + pos[p] / 8) * (size_t)kActBRec;
                    for (int i = 0; i < 64; i++) {
                        uint16_t hi, lo;
                        memcpy(&hi, rec + act_b_off(pos[p] % 8, i), 2);
                        memcpy(&lo, rec + kActBLo + act_b_off(pos[p] % 8, i), 2);
                        o[sl * 64 + i] = bf(hi) + bf(lo);
                    }
                }
            }
            return BIVMOE_OK;
        }
        case BIVMOE_TAP_PAIR_OUT: {
            if (bytes != P * e * 4) return set_err(errp, BIVMOE_ERR_ARGUMENT, "tap buffer size mismatch");
            std::vector<float> tmp((size_t)w.act_rows * e);
            std::vector<int32_t> pos(P);
            CU(cudaMemcpy(tmp.data(), w.pair_out, tmp.size() * 4, cudaMemcpyDeviceToHost));
            CU(cudaMemcpy(pos.data(), w.pos_of, P * 4, cudaMemcpyDeviceToHost));
            for (size_t p = 0; p < P; p++)
                memcpy((float*)dst + p * e, tmp.data() + (size_t)pos[p] * e, e * 4);
            return BIVMOE_OK;
        }
        case BIVMOE_TAP_SHARED_OUT:
            if (!L->has_shared) return set_err(errp, BIVMOE_ERR_ARGUMENT, "no shared expert");
            return copy_out(L, dst, w.pair_out, bytes, n * e * 4);
        default: return set_err(errp, BIVMOE_ERR_ARGUMENT, "unknown tap %d", which);
    }
}

int bivmoe_tap_block_dots(bivmoe_layer* L, int32_t matrix, int32_t expert, int32_t row,
                          int32_t act_row, int32_t* out) {
    if (!L || !out) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer or buffer");
    std::string* errp = &L->error;
    if (L->ep_world > 1)
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "taps read a whole layer's workspace; this layer is sharded");
    CU(cudaSetDevice(L->device));
    CU(cudaDeviceSynchronize());
    if (matrix < 0 || matrix > 5 || (matrix >= 3 && !L->has_shared))
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "matrix %d", matrix);
    const bool shared = matrix >= 3, is_down = matrix % 3 == 2;
    const DevTiles& m = is_down ? (shared ? L->sh_down : L->down) : (shared ? L->sh_gate_up : L->gate_up);
    const int tile_base = matrix % 3 == 1 ? 2 : 0;   // up rows are tiles 2, 3 of a gate+up chunk
    const int n = L->last_n, P = n * L->k;
    if (expert < 0 || expert >= m.n || row < 0 || row >= m.rows || act_row < 0 ||
        act_row >= (is_down && !shared ? P : n))
        return set_err(errp, BIVMOE_ERR_ARGUMENT, "index out of range");
    if (type_uses_f32_act(m.ty))
        return set_err(errp, BIVMOE_ERR_UNSUPPORTED, "type %d has no integer block dots", m.ty);
    const int nb = m.cols / 32;
    int32_t* dots = nullptr;
    CU(cudaMalloc((void**)&dots, (size_t)nb * 4));
    cudaError_t ce = cudaSuccess;
    // gate/up rows meet the token's Q8 row of h (position = token); down rows the
    // Q8 row of the pair's mid vector at the pair's position
    int32_t pos = act_row;
    if (is_down && !shared) ce = cudaMemcpy(&pos, L->ws.pos_of + act_row, 4, cudaMemcpyDeviceToHost);
    if (!is_down && !L->has_shared)
        ce = cudaMemcpy(&pos, L->ws.pos_of + (size_t)act_row * L->k, 4, cudaMemcpyDeviceToHost);
    if (ce == cudaSuccess)
        ce = launch_block_dots(m, tile_base, expert, row, is_down ? L->ws.mid_t : L->ws.act_t,
                               L->ws.act_rows, pos, dots, 0);
    if (ce == cudaSuccess) ce = cudaMemcpy(out, dots, (size_t)nb * 4, cudaMemcpyDeviceToHost);
    cudaFree(dots);
    CU(ce);
    return BIVMOE_OK;
}

int bivmoe_int8_peak(bivmoe_layer* L, double* tops) {
    if (!L || !tops) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer or result");
    std::string* errp = &L->error;
    DeviceScope on_device(L->device);
    CU(measure_int8_peak(L->sm_count, L->ws.status + 1, L->own_stream, tops));
    int32_t st = 0;
    CU(cudaMemcpy(&st, L->ws.status + 1, 4, cudaMemcpyDeviceToHost));
    if (st) {
        cudaMemset(L->ws.status + 1, 0, 4);
        return set_err(errp, st, "the probe's bounded wait gave up");
    }
    return BIVMOE_OK;
}

int bivmoe_numerics(const bivmoe_layer* L, char* buf, size_t len) {
    if (!L || !buf || !len) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer or buffer");
    // which expert kernels this layer's types get: groups of at most 8 rows (and every group
    // of types without a tcgen05 kernel) take the warp-level kernels
    const bool f32act = type_uses_f32_act(L->gate_up.ty);
    const char* small = f32act ? "f32-fma" : "mma.sync-s8-block-dots";
    char big[96] = "";
    if (L->prefill_min > 0)
        snprintf(big, sizeof big, "+tcgen05-%s-from-%d-rows", L->gate_up.ty == BIVMOE_BF16 ? "f16-two-bf16-terms" : "i8-block-dots",
                 L->prefill_min);
    snprintf(buf, len,
             "kind=cuda device=%s sms=%d repack=v%d experts=%s/bulk-copy-ring/tiled-weights%s "
             "router=f32-avx2-order combine=ordered-fma types=%d/%d/%d",
             L->device_name.c_str(), L->sm_count, kRepackVersion, small, big, L->gate_up.ty, L->gate_up.ty,
             L->down.ty);
    return BIVMOE_OK;
}

int bivmoe_memory(const bivmoe_layer* L, uint64_t* weight_bytes, uint64_t* workspace_bytes) {
    if (!L) return set_err(nullptr, BIVMOE_ERR_ARGUMENT, "null layer");
    if (weight_bytes) *weight_bytes = L->weight_bytes;
    if (workspace_bytes) *workspace_bytes = L->ws_bytes;
    return BIVMOE_OK;
}

}  // extern "C"
