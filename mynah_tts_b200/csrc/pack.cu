// Weight packing on the device, once per tensor, bit-identical to the
// reference's CPU quantizers so a packed tensor can be compared with memcmp.
//
//   int8: per output row, scale = amax/127 (1 when the row is all zero),
//         q = trunc(w/scale +- 0.5)                         (src/qmat.c:39-57)
//   int4: per group of 32 along k, scale = amax/7, clamp [-8,7], byte =
//         (q_even+8) | (q_odd+8)<<4, f32 scale per group    (src/qmat.c:59-91)
//   f16:  round-to-nearest-even cast                         (src/qmat.c:650-655)
#include "common.cuh"
#include "launch.h"

#include <cuda_fp16.h>

namespace {

__global__ void __launch_bounds__(256) k_pack_int8(const float *__restrict__ w, size_t k,
                                                    int8_t *__restrict__ q,
                                                    float *__restrict__ scales) {
    __shared__ float red[33];
    const size_t row = blockIdx.x;
    const float *src = w + row * k;
    float amax = 0.0f;
    for (size_t j = threadIdx.x; j < k; j += blockDim.x) amax = fmaxf(amax, fabsf(src[j]));
    amax = block_max(amax, red);
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    if (threadIdx.x == 0) scales[row] = scale;
    const float inv = __fdiv_rn(1.0f, scale);
    for (size_t j = threadIdx.x; j < k; j += blockDim.x)
        q[row * k + j] = (int8_t)round_half_away(__fmul_rn(src[j], inv));
}

__global__ void __launch_bounds__(256) k_pack_int4(const float *__restrict__ w, size_t total_groups,
                                                    uint8_t *__restrict__ q,
                                                    float *__restrict__ scales) {
    const size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= total_groups) return;
    const float4 *src = reinterpret_cast<const float4 *>(w + g * 32u);
    float v[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 t = src[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 7.0f) : 1.0f;
    scales[g] = scale;
    const float inv = __fdiv_rn(1.0f, scale);
    uint32_t packed[4];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            int q0 = round_half_away(__fmul_rn(v[wd * 8 + 2 * b], inv));
            int q1 = round_half_away(__fmul_rn(v[wd * 8 + 2 * b + 1], inv));
            q0 = min(7, max(-8, q0));
            q1 = min(7, max(-8, q1));
            word |= (uint32_t)(((q0 + 8) | ((q1 + 8) << 4)) & 0xff) << (8 * b);
        }
        packed[wd] = word;
    }
    reinterpret_cast<uint4 *>(q)[g] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

__global__ void k_pack_f16(const float *__restrict__ w, size_t count, __half *__restrict__ h) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) h[i] = __float2half_rn(w[i]);
}

}  // namespace

extern "C" int mb_pack_int8(const float *w, size_t n, size_t k, int8_t *q, float *scales,
                            mb_stream stream) {
    if (n == 0 || k == 0) return (int)cudaErrorInvalidValue;
    k_pack_int8<<<(unsigned)n, 256, 0, (cudaStream_t)stream>>>(w, k, q, scales);
    return mb_check_launch();
}

extern "C" int mb_pack_int4(const float *w, size_t n, size_t k, uint8_t *q, float *scales,
                            mb_stream stream) {
    if (n == 0 || k == 0 || (k % 32u) != 0) return (int)cudaErrorInvalidValue;
    const size_t groups = n * (k / 32u);
    k_pack_int4<<<(unsigned)((groups + 255) / 256), 256, 0, (cudaStream_t)stream>>>(w, groups, q,
                                                                                   scales);
    return mb_check_launch();
}

extern "C" int mb_pack_f16(const float *w, size_t count, uint16_t *h, mb_stream stream) {
    if (count == 0) return (int)cudaErrorInvalidValue;
    k_pack_f16<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        w, count, reinterpret_cast<__half *>(h));
    return mb_check_launch();
}
