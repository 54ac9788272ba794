// Device helpers shared by the sm_100a kernels.
//
// All translation units are compiled with -fmad=false: the reference rounds
// every product and sum separately (C11, no contraction), and a silently fused
// multiply-add would move activation-quantization rounding boundaries.  Where
// a fused multiply-add is wanted for speed it is written as fmaf explicitly.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "libm_parity.cuh"

#define MB_WARP 32
#define MB_FULL 0xffffffffu

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(MB_FULL, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(MB_FULL, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(MB_FULL, v, o));
    return v;
}

// Block-wide reductions; `red` is shared scratch of at least 33 floats.  Every
// thread receives the result.  The summation order is fixed (lanes by
// butterfly, then warps in index order) so results do not depend on timing.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : -3.402823466e+38f;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Round-half-away-from-zero to int with C truncation semantics:
// (int)(v >= 0 ? v + 0.5f : v - 0.5f)   (src/qmat.c:54, 107 in mynah-tts)
__device__ __forceinline__ int round_half_away(float v) {
    return __float2int_rz(v >= 0.0f ? __fadd_rn(v, 0.5f) : __fsub_rn(v, 0.5f));
}

// block_sum for a CTA that plays VT times its own size: thread t holds the partial sums of
// virtual threads t, t + blockDim.x, ...; the result has the bits block_sum gives a CTA of
// VT * blockDim.x threads (same butterflies, same order of the per-warp values).
template <int VT>
__device__ __forceinline__ float block_sum_vt(const float (&v)[VT], float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nrw = (blockDim.x + 31) >> 5;
    float t[VT];
#pragma unroll
    for (int r = 0; r < VT; ++r) t[r] = warp_sum(v[r]);
    __syncthreads();
    if (lane == 0)
#pragma unroll
        for (int r = 0; r < VT; ++r) red[warp + r * nrw] = t[r];
    __syncthreads();
    if (warp == 0) {
        float u = lane < VT * nrw ? red[lane] : 0.0f;
        u = warp_sum(u);
        if (lane == 0) red[32] = u;
    }
    __syncthreads();
    return red[32];
}

// One-barrier forms of the block reductions: every warp repeats the butterfly over the
// per-warp values (a butterfly leaves the same bits in every lane, and they are the bits
// warp 0 gets in block_sum_vt / block_max), so nothing has to be broadcast.  `buf` holds 32
// floats and must not be written again before the CTA has passed another barrier.
template <int VT>
__device__ __forceinline__ float block_sum_vt1(const float (&v)[VT], float *buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nrw = (blockDim.x + 31) >> 5;
    float t[VT];
#pragma unroll
    for (int r = 0; r < VT; ++r) t[r] = warp_sum(v[r]);
    if (lane == 0)
#pragma unroll
        for (int r = 0; r < VT; ++r) buf[warp + r * nrw] = t[r];
    __syncthreads();
    return warp_sum(lane < VT * nrw ? buf[lane] : 0.0f);
}
__device__ __forceinline__ float block_max1(float v, float *buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    return warp_max(lane < nw ? buf[lane] : -3.402823466e+38f);
}

// Non-strict layer norm of one row by one CTA, with optional int8 quantization of the
// result (src/qmat.c:93-113): `row` holds the input in shared memory and receives y.  The
// stand-alone kernel calls it with 256 threads and VT = 1, the products' fused prologue
// with 128 threads and VT = 2 (each thread plays two): a row gets the same bits from
// either.  Returns the quantization scale (0 when !quant) to every thread; q may be shared
// or global memory.  `red` is scratch of 96 floats that no thread is still reading.
template <int VT>
__device__ __forceinline__ float mb_ln_block(float *row, int width, const float *__restrict__ gain,
                                             const float *__restrict__ bias, float eps, float *red,
                                             float *y_out, bool quant, int8_t *q) {
    const int stride = VT * blockDim.x;
    float s[VT];
#pragma unroll
    for (int r = 0; r < VT; ++r) {
        s[r] = 0.0f;
        for (int i = threadIdx.x + r * blockDim.x; i < width; i += stride) s[r] += row[i];
    }
    const float mean = __fdiv_rn(block_sum_vt1<VT>(s, red), (float)width);
    float v[VT];
#pragma unroll
    for (int r = 0; r < VT; ++r) {
        v[r] = 0.0f;
        for (int i = threadIdx.x + r * blockDim.x; i < width; i += stride) {
            const float d = row[i] - mean;
            v[r] = fmaf(d, d, v[r]);
        }
    }
    const float variance = block_sum_vt1<VT>(v, red + 32);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(variance, (float)width), eps)));
    float amax = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float y = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(row[i], mean), scale), gain[i]),
                                  bias == nullptr ? 0.0f : bias[i]);
        if (y_out != nullptr) y_out[i] = y;
        row[i] = y;                  // each thread rereads only its own elements below
        amax = fmaxf(amax, fabsf(y));
    }
    if (!quant) return 0.0f;
    amax = block_max1(amax, red + 64);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        q[i] = (int8_t)min(127, max(-127, round_half_away(__fmul_rn(row[i], inv))));
    return amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
}

// ((..(v[0] + v[1]) + v[2]) ..) + v[n-1], every add rounded: the reference's `sum += v[i]`
// loop by ONE thread over shared memory.  The chain costs an add latency per element (4
// cycles); sixteen values are fetched as four 16-byte loads before their sixteen adds, which
// was measured at 4.4 cycles per element for 768 (a plain loop: 6.4; deeper software
// pipelining through register arrays: 5.6 to 6.8).  (An array that is not 16-byte aligned
// is walked with plain loads.)
__device__ __forceinline__ float mb_seq_sum(const float *v, int n) {
    float s = 0.0f;
    int i = 0;
    if ((reinterpret_cast<uintptr_t>(v) & 15u) == 0) {
        const float4 *v4 = reinterpret_cast<const float4 *>(v);
        const int n16 = n >> 4;
        for (int b = 0; b < n16; ++b) {
            const float4 a0 = v4[4 * b], a1 = v4[4 * b + 1], a2 = v4[4 * b + 2], a3 = v4[4 * b + 3];
            s = __fadd_rn(s, a0.x); s = __fadd_rn(s, a0.y); s = __fadd_rn(s, a0.z); s = __fadd_rn(s, a0.w);
            s = __fadd_rn(s, a1.x); s = __fadd_rn(s, a1.y); s = __fadd_rn(s, a1.z); s = __fadd_rn(s, a1.w);
            s = __fadd_rn(s, a2.x); s = __fadd_rn(s, a2.y); s = __fadd_rn(s, a2.z); s = __fadd_rn(s, a2.w);
            s = __fadd_rn(s, a3.x); s = __fadd_rn(s, a3.y); s = __fadd_rn(s, a3.z); s = __fadd_rn(s, a3.w);
        }
        i = n16 << 4;
    }
    for (; i < n; ++i) s = __fadd_rn(s, v[i]);
    return s;
}

// Reference-order layer norm of one row by one CTA (src/kernels.c:186-244, portable branch:
// the mean and the variance are each ONE sequential chain of rounded adds over the row, the
// squares are rounded once each), with optional int8 quantization (src/qmat.c:93-113).
// `row` (shared, 16-byte aligned) holds the input and receives y; `sq` is scratch of `width`
// floats (16-byte aligned), `stat` of
// two, `red` of 32 that no thread is still reading.  Returns the quantization scale (0 when
// !quant) to every thread.  Same bits as k_layernorm<true>.
// (MB_LN_TICK: a file of a profiling build may define it before this header to timestamp the
// steps: 0 mean, 1 squares, 2 variance, 3 normalized, 4 absmax, 5 quantized.)
#ifndef MB_LN_TICK
#define MB_LN_TICK(i)
#endif
__device__ __forceinline__ float mb_ln_block_strict(float *row, int width, const float *__restrict__ gain,
                                                    const float *__restrict__ bias, float eps, float *sq, float *stat,
                                                    float *red, float *y_out, bool quant, int8_t *q) {
    if (threadIdx.x == 0) stat[0] = __fdiv_rn(mb_seq_sum(row, width), (float)width);
    __syncthreads();
    MB_LN_TICK(0);
    const float mean = stat[0];
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float d = __fsub_rn(row[i], mean);
        sq[i] = __fmul_rn(d, d);
    }
    __syncthreads();
    MB_LN_TICK(1);
    if (threadIdx.x == 0) stat[1] = mb_seq_sum(sq, width);
    __syncthreads();
    MB_LN_TICK(2);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(stat[1], (float)width), eps)));
    float amax = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float y = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(row[i], mean), scale), gain[i]),
                                  bias == nullptr ? 0.0f : bias[i]);
        if (y_out != nullptr) y_out[i] = y;
        row[i] = y;                  // each thread rereads only its own elements below
        amax = fmaxf(amax, fabsf(y));
    }
    MB_LN_TICK(3);
    if (!quant) return 0.0f;
    amax = block_max1(amax, red);
    MB_LN_TICK(4);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        q[i] = (int8_t)min(127, max(-127, round_half_away(__fmul_rn(row[i], inv))));
    MB_LN_TICK(5);
    return amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
}

// int8 quantization of one f32 row held in shared memory by one CTA; returns the scale.
__device__ __forceinline__ float mb_quant_block(const float *row, int width, float *red, int8_t *q) {
    float amax = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
    amax = block_max(amax, red);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        q[i] = (int8_t)min(127, max(-127, round_half_away(__fmul_rn(row[i], inv))));
    return amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
}

// tanh-form GELU of the reference's decode step (src/kernels.c:382-389):
// 0.5*x*(1+tanhf(0.7978845608*(x+0.044715*x^3))), every operation rounded to
// f32 in source order.  STRICT returns the host libm's tanhf bit for bit when
// the correction table is given (libm_parity.cuh), else the correctly rounded
// value; the fast form uses CUDA's tanhf.
template <bool STRICT>
__device__ __forceinline__ float gelu_tanh(float x, const uint32_t *tanh_tab) {
    const float cubic = __fmul_rn(__fmul_rn(x, x), x);
    const float c = __fmul_rn(0.7978845608f, __fadd_rn(x, __fmul_rn(0.044715f, cubic)));
    const float t = STRICT ? mb_tanhf_host(c, tanh_tab) : tanhf(c);
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, t));
}

// The strict GELU in two steps (see mb_tanh_fetch): the argument of tanhf, and the result
// from the argument's fetched table word.
__device__ __forceinline__ float gelu_tanh_arg(float x) {
    const float cubic = __fmul_rn(__fmul_rn(x, x), x);
    return __fmul_rn(0.7978845608f, __fadd_rn(x, __fmul_rn(0.044715f, cubic)));
}
__device__ __forceinline__ float gelu_tanh_finish(float x, float c, uint32_t word, bool have_tab) {
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, mb_tanhf_host_with(c, word, have_tab)));
}

template <bool STRICT>
__device__ __forceinline__ float exp_ref(float x, const uint32_t *exp_tab = nullptr) {
    return STRICT ? mb_expf_host(x, exp_tab) : expf(x);
}

static inline int mb_check_launch() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch -----------------------------------------
// Every kernel of the step begins with mb_pdl_wait(): when it was launched with
// the programmatic-serialization attribute it may be scheduled while its
// predecessor in the stream is still running, and the wait blocks until that
// predecessor has finished and its writes are visible; without the attribute the
// instruction does nothing.  mb_pdl_trigger() then lets the next kernel in the
// stream start its own launch early.  Nothing a predecessor writes may be touched
// before the wait.
__device__ __forceinline__ void mb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The live-lane count of a step.  No kernel writes it (the host stages it before the step's
// first launch), so it may be read before mb_pdl_wait(); the load is volatile asm so that it
// stays there, off the chain of dependent round trips behind the wait.
__device__ __forceinline__ int mb_lane_count(const int *n_active) {
    if (n_active == nullptr) return 0x7fffffff;
    int v;
    asm volatile("ld.global.cg.b32 %0, [%1];" : "=r"(v) : "l"(n_active));
    return v;
}

extern "C" int mb_pdl_enabled(void);   // glue.cu: MYNAH_B200_PDL, default on

template <typename... KArgs, typename... Args>
static inline int mb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = mb_pdl_enabled() ? 1u : 0u;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
