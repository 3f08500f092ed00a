// Row-wise helpers around the expert products: the Q8 activation quantiser,
// rms_norm, the weighted gather-combine, and the upload-time repack of GGUF
// rows into the device row layout.
#include "common.cuh"
#include "formats.cuh"

namespace bivmoe {

// ---------------------------------------------------------------------------
// Q8Act::quantize_into (quant.rs:368-394): one warp per 32-value block.
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const float* __restrict__ x, int64_t n_blocks, int8_t* __restrict__ q,
                     float2* __restrict__ ds) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t stride = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t b = warp0; b < n_blocks; b += stride) {
        float dd, ss;
        int qi = q8_quantize_lane(x[b * 32 + lane], dd, ss);
        q[b * 32 + lane] = (int8_t)qi;
        if (lane == 0) ds[b] = make_float2(dd, ss);
    }
}

cudaError_t launch_quantize_rows(const LaunchCfg& c, const float* x, int rows, int cols, int8_t* q,
                                 float2* ds) {
    int64_t nb = (int64_t)rows * cols / 32;
    int blocks = (int)((nb + 7) / 8);
    if (blocks > c.sm_count * 16) blocks = c.sm_count * 16;
    quantize_rows_kernel<<<blocks, 256, 0, c.stream>>>(x, nb, q, ds);
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// ops.rs:136-149: out = x * (1/sqrt(dot(x,x)/e + eps)) * w, one warp per row.
// The sum of squares uses the reference's AVX2 dot order (see router.cu).
__global__ void __launch_bounds__(128)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                float* __restrict__ out, int n, int e) {
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
    rms_norm_kernel<<<(c.n + 3) / 4, 128, 0, c.stream>>>(x, w, eps, out, c.n, c.e);
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Weighted gather-combine (model.rs:886-896; Metal moe_combine,
// kernels.metal:1885-1908): out[t] (+)= sum over the token's experts in
// ascending expert id of w * y, then sigmoid(gate) * shared, each step one
// fused multiply-add as the reference's axpy.  No atomics: run-to-run identical.
constexpr int CB_THREADS = 256, CB_MAX_K = 32;

__global__ void __launch_bounds__(CB_THREADS)
combine_kernel(Workspace ws, float* __restrict__ out, int n, int k, int e, int n_expert,
               int has_shared, int accumulate) {
    __shared__ int s_pos[CB_MAX_K];
    __shared__ float s_w[CB_MAX_K];
    __shared__ float s_gate;
    const int t = blockIdx.x;
    if (threadIdx.x < k) {
        // rank of this pair among the token's pairs by expert id (ids are distinct)
        const int my = ws.ids[(size_t)t * k + threadIdx.x];
        int rank = 0;
        for (int j = 0; j < k; j++) rank += ws.ids[(size_t)t * k + j] < my;
        s_pos[rank] = ws.pos_of[(size_t)t * k + threadIdx.x];
        s_w[rank] = ws.weights[(size_t)t * k + threadIdx.x];
    }
    if (threadIdx.x == 32 && has_shared) {
        const float g = ws.logits[(size_t)t * (n_expert + 1) + n_expert];
        s_gate = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));   // ops.rs:160-162
    }
    __syncthreads();
    const int c4 = blockIdx.y * CB_THREADS + threadIdx.x;     // float4 column
    if (c4 * 4 >= e) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; j++) {
        const float4 y = *(const float4*)(ws.pair_out + (size_t)s_pos[j] * e + c4 * 4);
        const float w = s_w[j];
        acc.x = fmaf(w, y.x, acc.x); acc.y = fmaf(w, y.y, acc.y);
        acc.z = fmaf(w, y.z, acc.z); acc.w = fmaf(w, y.w, acc.w);
    }
    if (has_shared) {
        const float4 y = *(const float4*)(ws.pair_out + ((size_t)n * k + t) * e + c4 * 4);
        const float w = s_gate;
        acc.x = fmaf(w, y.x, acc.x); acc.y = fmaf(w, y.y, acc.y);
        acc.z = fmaf(w, y.z, acc.z); acc.w = fmaf(w, y.w, acc.w);
    }
    float4* o = (float4*)(out + (size_t)t * e + c4 * 4);
    if (accumulate) {
        float4 r = *o;
        acc.x += r.x; acc.y += r.y; acc.z += r.z; acc.w += r.w;
    }
    *o = acc;
}

cudaError_t launch_combine(const LaunchCfg& c, const Workspace& ws, float* out, int accumulate) {
    if (c.k > CB_MAX_K || c.e % 4) return cudaErrorInvalidValue;
    dim3 grid(c.n, (c.e / 4 + CB_THREADS - 1) / CB_THREADS);
    combine_kernel<<<grid, CB_THREADS, 0, c.stream>>>(ws, out, c.n, c.k, c.e, c.n_expert,
                                                      c.has_shared, accumulate);
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Upload-time repack: GGUF rows -> device rows (layouts in common.cuh).  One
// thread per source block; byte-preserving except for Q6_K's padded f16 plane.
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                   int64_t n_rows, int64_t cols) {
    const int64_t nb = cols / 32, total = n_rows * nb;
    const int64_t srb = nb * 34, drb = cols + cols / 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nb, b = i % nb;
        const uint8_t* s = src + r * srb + b * 34;
        uint8_t* drow = dst + r * drb;
        drow[cols + 2 * b] = s[0];
        drow[cols + 2 * b + 1] = s[1];
        for (int j = 0; j < 32; j++) drow[32 * b + j] = s[2 + j];
    }
}
__global__ void repack_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                  int64_t n_rows, int64_t cols) {
    const int64_t nb = cols / 256, total = n_rows * nb;
    const int64_t srb = nb * 210, drb = dev_row_bytes(BIVMOE_Q6_K, cols);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nb, b = i % nb;
        const uint8_t* s = src + r * srb + b * 210;
        uint8_t* drow = dst + r * drb;
        for (int j = 0; j < 128; j++) drow[b * 128 + j] = s[j];
        for (int j = 0; j < 64; j++) drow[nb * 128 + b * 64 + j] = s[128 + j];
        for (int j = 0; j < 16; j++) drow[nb * 192 + b * 16 + j] = s[192 + j];
        drow[nb * 208 + 2 * b] = s[208];
        drow[nb * 208 + 2 * b + 1] = s[209];
        if (b == 0)
            for (int64_t j = nb * 208 + nb * 2; j < drb; j++) drow[j] = 0;
    }
}

cudaError_t launch_repack(int ty, const uint8_t* gguf_rows, uint8_t* dev_rows, int64_t n_rows,
                          int64_t cols, cudaStream_t stream) {
    if (ty == BIVMOE_Q8_0) {
        repack_q8_0_kernel<<<1024, 256, 0, stream>>>(gguf_rows, dev_rows, n_rows, cols);
    } else if (ty == BIVMOE_Q6_K) {
        repack_q6k_kernel<<<1024, 256, 0, stream>>>(gguf_rows, dev_rows, n_rows, cols);
    } else {
        return cudaMemcpyAsync(dev_rows, gguf_rows, (size_t)(n_rows * gguf_row_bytes(ty, cols)),
                               cudaMemcpyDeviceToDevice, stream);
    }
    return cudaGetLastError();
}

}  // namespace bivmoe

namespace bivmoe {

// ---------------------------------------------------------------------------
// Parity tap: the int32 dot of each 32-element block of one device-layout
// weight row with one Q8 activation row, decoded byte by byte as the
// reference's scalar kernels define the values (quant.rs:599-686).  One thread
// per block; not on the timed path.
__global__ void block_dots_kernel(int ty, const uint8_t* __restrict__ w, int cols,
                                  const int8_t* __restrict__ xq, int32_t* __restrict__ out) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;   // 32-element block
    if (b >= cols / 32) return;
    const int8_t* x = xq + 32 * b;
    const int nb = cols / 256, sbk = b / 8, sb = b % 8;
    int32_t sum = 0;
    if (ty == BIVMOE_Q8_0) {
        for (int l = 0; l < 32; l++) sum += (int)(int8_t)w[32 * b + l] * x[l];
    } else if (ty == BIVMOE_Q4_K || ty == BIVMOE_Q5_K) {
        const uint8_t* blk = w + (size_t)sbk * (ty == BIVMOE_Q4_K ? 144 : 176);
        const uint8_t* qs = blk + (ty == BIVMOE_Q4_K ? 16 : 48) + 32 * (sb / 2);
        for (int l = 0; l < 32; l++) {
            int q = (qs[l] >> (4 * (sb % 2))) & 0xF;
            if (ty == BIVMOE_Q5_K) q |= ((blk[16 + l] >> sb) & 1) << 4;
            sum += q * x[l];
        }
    } else if (ty == BIVMOE_Q6_K) {
        const int n = sb / 4, kq = sb % 4;
        const uint8_t* ql = w + (size_t)sbk * 128 + 64 * n + 32 * (kq & 1);
        const uint8_t* qh = w + (size_t)nb * 128 + (size_t)sbk * 64 + 32 * n;
        const int8_t* sc = (const int8_t*)w + (size_t)nb * 192 + (size_t)sbk * 16 + 8 * n + 2 * kq;
        for (int half = 0; half < 2; half++) {
            int32_t part = 0;
            for (int l = 16 * half; l < 16 * half + 16; l++) {
                const int nib = kq >= 2 ? ql[l] >> 4 : ql[l] & 0xF;
                const int q = (nib | (((qh[l] >> (2 * kq)) & 3) << 4)) - 32;
                part += q * x[l];
            }
            sum += sc[half] * part;
        }
    }
    out[b] = sum;
}

cudaError_t launch_block_dots(int ty, const uint8_t* dev_row, int64_t cols, const int8_t* xq,
                              int32_t* out, cudaStream_t stream) {
    const int nb = (int)(cols / 32);
    block_dots_kernel<<<(nb + 63) / 64, 64, 0, stream>>>(ty, dev_row, (int)cols, xq, out);
    return cudaGetLastError();
}

}  // namespace bivmoe
