// bivmoe_route_noalloc: the routing step (router product, softmax, top-k,
// renormalisation) for callers that must not allocate device memory.
//
// The routing step needs a scratch matrix of router logits between its two
// kernels.  Everywhere else in this library that scratch is part of the
// workspace `bivmoe_create` allocates; here it is a fixed array that lives in
// the library image itself, so the call performs no cudaMalloc, cudaFree or
// any other allocating routine.  The price is a hard size limit and the fact
// that every GPU that loads the library holds the array until the process exits.
#include <stdio.h>

#include "common.cuh"

using namespace bivmoe;

// n * (n_expert + 1) logits must fit: e.g. 512 tokens with 256 experts (514 KiB).
#define ROUTE_SCRATCH_FLOATS BIVMOE_ROUTE_NOALLOC_MAX_LOGITS

static __device__ __align__(256) float g_route_scratch[ROUTE_SCRATCH_FLOATS];

// The device address of the array, per device.  In host code the name
// `g_route_scratch` is only a stand-in for the symbol, not a device address, so the
// address handed to the kernels is the one cudaGetSymbolAddress returns while that
// device is current.
constexpr int kMaxDevices = 64;
static float* g_route_scratch_addr[kMaxDevices];

extern "C" int bivmoe_route_noalloc(bivmoe_layer* layer, const float* h_dev, int32_t n,
                                    int32_t* ids_dev, float* weights_dev, void* stream) {
    RouteView v;
    if (layer_route_view(layer, &v, nullptr)) return BIVMOE_ERR_ARGUMENT;
    char msg[256];
    auto fail = [&](int code, const char* text) {
        layer_route_view(layer, nullptr, text);
        return code;
    };
    if (n < 0) return fail(BIVMOE_ERR_ARGUMENT, "negative token count");
    if (n == 0) return BIVMOE_OK;   // no rows (their pointers may be null): nothing to do
    if (!h_dev || !ids_dev || !weights_dev) return fail(BIVMOE_ERR_ARGUMENT, "null device pointer");
    if ((int64_t)n * (v.n_expert + 1) > (int64_t)ROUTE_SCRATCH_FLOATS) {
        snprintf(msg, sizeof msg,
                 "bivmoe_route_noalloc: %d tokens x %d logits exceed the built-in scratch of %d "
                 "floats; use bivmoe_forward, whose workspace is sized at create",
                 n, v.n_expert + 1, (int)ROUTE_SCRATCH_FLOATS);
        return fail(BIVMOE_ERR_ARGUMENT, msg);
    }
    if (v.device < 0 || v.device >= kMaxDevices) return fail(BIVMOE_ERR_ARGUMENT, "device ordinal");
    // the layer's device is current inside the call only; the caller's comes back on return
    DeviceScope on_device(v.device);
    cudaError_t ce = cudaSuccess;
    if (!g_route_scratch_addr[v.device]) {
        // set-up, once per device, with that device current.  Two host threads that make
        // their first call on one device together both look the address up and store the
        // same value: harmless, so the cache needs no lock.
        float* p = nullptr;
        ce = cudaGetSymbolAddress((void**)&p, g_route_scratch);
        if (ce == cudaSuccess) g_route_scratch_addr[v.device] = p;
    }
    if (ce != cudaSuccess) {
        snprintf(msg, sizeof msg, "bivmoe_route_noalloc set-up: %s", cudaGetErrorString(ce));
        return fail(BIVMOE_ERR_CUDA, msg);
    }
    // the two routing kernels, with the built-in array in place of the workspace's logits
    Workspace ws{};
    ws.logits = g_route_scratch_addr[v.device];
    ws.ids = ids_dev;
    ws.weights = weights_dev;
    ws.status = v.status;
    LaunchCfg c{(cudaStream_t)stream, n, v.k, v.e, v.n_expert, 0, 0, v.has_shared, v.sm_count};
    ce = launch_router(c, v.router, h_dev, ws);
    if (ce == cudaSuccess) ce = launch_route_topk(c, ws);
    if (ce != cudaSuccess) {
        snprintf(msg, sizeof msg, "bivmoe_route_noalloc launch: %s", cudaGetErrorString(ce));
        return fail(BIVMOE_ERR_CUDA, msg);
    }
    return BIVMOE_OK;
}
