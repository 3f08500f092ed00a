// Device-side decoding of the weight block formats (device row layouts are
// described in common.cuh) and the Q8 activation quantiser.  Shared by the
// expert kernels and by the int32 block-dot tap so both see the same integers.
// Reference: engine/src/quant.rs:144-153 (scale_min_k4), 368-394 (quantiser),
// 599-686 (scalar dots: the definition of each block's integers).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace bivmoe {

__device__ __forceinline__ int dp4a_s8(int a, int b, int c) { return __dp4a(a, b, c); }

// The 6-bit scales and mins of a Q4_K / Q5_K super-block, from its 12 packed
// bytes held as three little-endian words: byte j of sc_lo/m_lo is sub-block j
// (j < 4), byte j of sc_hi/m_hi is sub-block 4 + j.
struct K4Scales { uint32_t sc_lo, sc_hi, m_lo, m_hi; };
__device__ __forceinline__ K4Scales unpack_k4_scales(uint32_t w0, uint32_t w1, uint32_t w2) {
    K4Scales s;
    s.sc_lo = w0 & 0x3F3F3F3Fu;
    s.m_lo = w1 & 0x3F3F3F3Fu;
    s.sc_hi = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
    s.m_hi = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
    return s;
}
__device__ __forceinline__ int k4_scale(const K4Scales& s, int sb) {
    return (int)(((sb < 4 ? s.sc_lo : s.sc_hi) >> (8 * (sb & 3))) & 0xFF);
}
__device__ __forceinline__ int k4_min(const K4Scales& s, int sb) {
    return (int)(((sb < 4 ? s.m_lo : s.m_hi) >> (8 * (sb & 3))) & 0xFF);
}

// One Q8 block (32 values) held by the 32 lanes of a warp: returns the int8
// value of this lane; d and s are the block's scale and d * sum(q).
// quant.rs:380-393: d = amax/127, id = 1/d (0 when d is 0), q = round(v*id)
// with halves away from zero, s = d * (float)sum.
__device__ __forceinline__ int q8_quantize_lane(float v, float& d, float& s) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q = (int)roundf(__fmul_rn(v, id));
    int sum = q;
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    s = __fmul_rn(d, (float)sum);
    return q;
}

}  // namespace bivmoe
