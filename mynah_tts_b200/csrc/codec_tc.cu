// The codec's residual-layer convolutions on the 5th-generation tensor cores (tcgen05,
// kind::f16), fast mode only: strict mode keeps one sequential f32 sum per output sample
// (codec.cu), which no tensor-core accumulation order reproduces.
//
//   out[o][t] = bias[o] + sum_k sum_i W[o][i][k] * x[i][t - (K-1-k) * dilation]
//
// is one accumulation over (channel chunk, tap k) of products  X_k [128 times x 64 channels]
// . W_k^T [64 channels x N output channels]: the tile of X for tap k is the same channel-major
// slab of the activation shifted by the tap's delay.  TMA fetches the slab once per chunk with
// its halo (rows t0 - (K-1) * dilation .. t0 + 127; rows before the start of the signal arrive
// as zeros, the causal padding) and every tap's MMA reads it through a descriptor that starts
// k * dilation rows further down: rows of a 128-byte-swizzled K-major tile lie 128 bytes
// apart and the swizzle is a function of the shared-memory address, so a descriptor may
// start at any row of a 1024-byte-aligned buffer (base offset 0).  Operands are
// f16, so both sides are split in two halves that add up to the f32 value to about 22 bits,
//   hi = f16(v), lo = f16(v - hi),
// and three MMAs per K step (hi.hi + lo.hi + hi.lo) accumulate in f32 in tensor memory.  The
// weights are scaled by a power of two at pack time so that their lo halves stay normal
// numbers; the epilogue undoes it exactly.
//
// Layouts.  Activations that feed a convolution live as two f16 planes [time][Cp] (channels
// contiguous, Cp = channels rounded up to 64, pad columns zero) written by the producer's
// epilogue (k_conv1d_tc itself, or k_snake_planes at the start of a branch).  Weights:
// [plane][tap][rows = tiles * N][Cp] f16.  Everything else (residual stream, branch sum) stays
// f32 [channels][time] as in codec.cu.
//
// One CTA = 128 times x N output channels (N <= 112, a multiple of 16): two buffers of
// { X hi, X lo: (128 + halo) x 128 B each } filled once per chunk and a ring of stages of
// { W hi, W lo: N x 128 B each } filled once per (chunk, tap); one thread issues 12 tcgen05.mma (M128 N K16) per stage; sixteen warps (four per 32
// accumulator rows, each a quarter of the columns) read them with tcgen05.ld and run the same epilogue as the SIMT kernel (bias,
// residual, half-Snake copy for the next convolution, branch sum).  Every wait is bounded
// (status bits 8 and 16).
#include "common.cuh"
#include "launch.h"
#include "libm_parity.cuh"

#include "tc_common.cuh"

#include <cuda_fp16.h>
#include <string.h>

namespace {

constexpr int CT_THREADS = 512;            // 16 warps: warp w reads accumulator rows 32 (w % 4) .. +31, column groups w / 4, w / 4 + 4, ..
constexpr int CT_TM = 128;                 // times per tile
constexpr int CT_KC = 128;                 // bytes of channels per stage row: 64 halves
constexpr int CT_MAX_STAGES = 8;           // weight stages
constexpr int CT_HALO_MAX = 50;            // (kernel - 1) * dilation

struct ConvTcP {
    const float4 *chan;          // per output channel: {bias, alpha, 1 / (alpha + 1e-9), alpha2} (mb_codec_tc_channel_table)
    const float *res;
    int has_alpha, has_alpha2;
    float *out, *acc;
    __half *act_hi, *act_lo;     // planes [L][cp_out] of half-Snake(v), or NULL
    int *status;
    float inv_scale;             // 1 / the power of two the weights were scaled by
    int oc, L, K, dil, n_tile, chunks, stages, cp_out, acc_mode;
    float *rows_out;             // row-major form: out[t][o] with row stride rows_stride (the codec's form: NULL)
    int rows_stride, rows_epi;   // MB_EPI_STORE / MB_EPI_RESIDUAL / MB_EPI_GELU
    int xrows;                   // 128 + (K - 1) * dil rows per activation tile
    int x_plane_bytes;           // xrows * 128 rounded up to 1024
    int xbufs;                   // activation buffers: 2, or 1 where two do not fit beside two weight stages
};

// Descriptor of a 128-byte-swizzled K-major tile that starts at any 128-byte row of a
// 1024-byte-aligned buffer that TMA filled: both TMA and the MMA swizzle by address bits,
// so the base-offset field stays 0 (measured: setting it to the row's phase reads wrong rows).
__device__ __forceinline__ uint64_t smem_desc_sw128_row(unsigned addr) { return smem_desc_sw128(addr); }

__device__ __forceinline__ float snake_fast(float v, int c, int snake_ch, const float *alpha) {
    if (c < snake_ch) {
        const float a = alpha[c];
        const float sn = sinf(a * v);
        return v + sn * sn * (1.0f / (a + 1e-9f));
    }
    return v < 0.0f ? v * 0.01f : v;
}
// The same with the channel's constants at hand.
__device__ __forceinline__ float snake_with(float v, bool snake, float a, float inv_a) {
    if (snake) {
        const float sn = sinf(a * v);
        return fmaf(sn * sn, inv_a, v);
    }
    return v < 0.0f ? v * 0.01f : v;
}

__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float (&v)[16]) {
    int r[16];
    tmem_ld16(taddr, r);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __int_as_float(r[i]);
}

__global__ void __launch_bounds__(CT_THREADS, 2)
k_conv1d_tc(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, ConvTcP p) {
    extern __shared__ unsigned char smem_ct[];
    __shared__ __align__(8) unsigned long long full_bar[CT_MAX_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[CT_MAX_STAGES];
    __shared__ __align__(8) unsigned long long xfull_bar[2];
    __shared__ __align__(8) unsigned long long xempty_bar[2];
    __shared__ __align__(8) unsigned long long done_bar;
    __shared__ uint32_t s_tmem;
    __shared__ unsigned s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * CT_TM;
    const int ntile = blockIdx.y;
    const int N = p.n_tile;
    const int b_bytes = N * CT_KC;                           // one plane of the weight tile
    const unsigned w_stage_bytes = (unsigned)(2 * b_bytes);
    const unsigned x_buf_bytes = (unsigned)(2 * p.x_plane_bytes);
    const int S = p.stages;
    const int halo = (p.K - 1) * p.dil;
    const uint32_t tmem_cols = N <= 32 ? 32u : (N <= 64 ? 64u : 128u);
    unsigned char *base = smem_ct + ((1024u - (saddr(smem_ct) & 1023u)) & 1023u);
    unsigned char *xbuf = base;                               // [xbufs][hi plane | lo plane]
    unsigned char *wring = base + (size_t)p.xbufs * x_buf_bytes;   // [S][hi N x 128 | lo N x 128]
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            bar_init(&full_bar[s], 1u);
            bar_init(&empty_bar[s], 1u);
        }
        for (int s = 0; s < 2; ++s) {
            bar_init(&xfull_bar[s], 1u);
            bar_init(&xempty_bar[s], 1u);
        }
        bar_init(&done_bar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fail = 0u;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&s_tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    mb_pdl_wait();
    mb_pdl_trigger();
    if (warp == 0 && lane == 0) {
        int wstep = 0;
        bool ok = true;
        for (int chunk = 0; chunk < p.chunks && ok; ++chunk) {
            const int xb = chunk % p.xbufs;
            if (chunk >= p.xbufs && !bar_wait(&xempty_bar[xb], (unsigned)((chunk / p.xbufs - 1) & 1), TC_SPIN)) ok = false;
            if (!ok) break;
            bar_expect(&xfull_bar[xb], 2u * (unsigned)(p.xrows * CT_KC));
            for (int plane = 0; plane < 2; ++plane)
                asm volatile(
                    "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                    "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(saddr(xbuf + (size_t)xb * x_buf_bytes + (size_t)plane * p.x_plane_bytes)),
                    "l"(&map_x), "r"(chunk * CT_KC), "r"(t0 - halo), "r"(plane), "r"(saddr(&xfull_bar[xb]))
                    : "memory");
            for (int tap = 0; tap < p.K; ++tap, ++wstep) {
                const int s = wstep % S;
                if (wstep >= S && !bar_wait(&empty_bar[s], (unsigned)((wstep / S - 1) & 1), TC_SPIN)) {
                    ok = false;
                    break;
                }
                bar_expect(&full_bar[s], w_stage_bytes);
                asm volatile(
                    "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                    "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(saddr(wring + (size_t)s * w_stage_bytes)), "l"(&map_w),
                    "r"(chunk * CT_KC), "r"(ntile * N), "r"(tap), "r"(0), "r"(saddr(&full_bar[s]))
                    : "memory");
            }
        }
        if (!ok) {
            s_fail = 1u;
            if (p.status != nullptr) atomicOr(p.status, 8);
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = instr_desc_f16(CT_TM, N);
        int wstep = 0;
        bool ok = true;
        for (int chunk = 0; chunk < p.chunks && ok; ++chunk) {
            const int xb = chunk % p.xbufs;
            if (!bar_wait(&xfull_bar[xb], (unsigned)((chunk / p.xbufs) & 1), TC_SPIN)) {
                ok = false;
                break;
            }
            unsigned char *xh_base = xbuf + (size_t)xb * x_buf_bytes;
            for (int tap = 0; tap < p.K; ++tap, ++wstep) {
                const int s = wstep % S;
                if (!bar_wait(&full_bar[s], (unsigned)((wstep / S) & 1), TC_SPIN)) {
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // tap k reads times t - (K-1-k) * dil: rows k * dil .. k * dil + 127 of the slab
                const unsigned row_bytes = (unsigned)(tap * p.dil) * (unsigned)CT_KC;
                const uint64_t xh = smem_desc_sw128_row(saddr(xh_base) + row_bytes);
                const uint64_t xl = smem_desc_sw128_row(saddr(xh_base + p.x_plane_bytes) + row_bytes);
                unsigned char *wst = wring + (size_t)s * w_stage_bytes;
                const uint64_t wh = smem_desc_sw128(saddr(wst));
                const uint64_t wl = smem_desc_sw128(saddr(wst + b_bytes));
#pragma unroll
                for (int kk = 0; kk < CT_KC / 32; ++kk) {            // 16 halves = 32 K-bytes per instruction
                    mma_f16(tmem, xh + 2u * kk, wh + 2u * kk, idesc, (wstep | kk) != 0 ? 1u : 0u);
                    mma_f16(tmem, xl + 2u * kk, wh + 2u * kk, idesc, 1u);
                    mma_f16(tmem, xh + 2u * kk, wl + 2u * kk, idesc, 1u);
                }
                mma_commit(&empty_bar[s]);
            }
            if (ok) mma_commit(&xempty_bar[xb]);
        }
        if (!ok) {
            s_fail = 1u;
            if (p.status != nullptr) atomicOr(p.status, 8);
        }
        mma_commit(&done_bar);
    }
    const bool done = bar_wait(&done_bar, 0u, TC_SPIN);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool good = done && s_fail == 0u;
    if (!done && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, 16);
    if (!good) {
        // a wait ran out: give copies still in flight one more bounded chance to land before
        // this CTA's shared memory is released
        if (threadIdx.x == 0) {
            for (int s = 0; s < S; ++s) bar_wait(&full_bar[s], 0u, TC_SPIN >> 4);
            for (int s = 0; s < p.xbufs && s < p.chunks; ++s) bar_wait(&xfull_bar[s], 0u, TC_SPIN >> 4);
        }
    } else {
        const int quad = warp & 3;
        const int t = t0 + quad * 32 + lane;
        const bool t_ok = t < p.L;
        const int snake_ch = p.oc / 2;
        for (int g = warp >> 2; g < N / 16; g += CT_THREADS / 128) {
            float v[16];
            tmem_ld16f(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(g * 16), v);
            const int o0 = ntile * N + g * 16;
            if (p.rows_out != nullptr) {
                // products over rows (text encoder, context prefill): out[t][o0 .. o0 + 15], 64 bytes per thread
                if (t_ok && o0 < p.oc) {
                    float *dst = p.rows_out + (size_t)t * p.rows_stride + o0;
                    float y[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) y[j] = v[j] * p.inv_scale;
                    if (p.rows_epi == MB_EPI_GELU) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) y[j] = gelu_tanh<false>(y[j], nullptr);
                    }
                    if (o0 + 16 <= p.oc) {
                        float4 *d4 = reinterpret_cast<float4 *>(dst);
                        if (p.rows_epi == MB_EPI_RESIDUAL) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float4 old = d4[q];
                                y[4 * q] += old.x; y[4 * q + 1] += old.y; y[4 * q + 2] += old.z; y[4 * q + 3] += old.w;
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) d4[q] = make_float4(y[4 * q], y[4 * q + 1], y[4 * q + 2], y[4 * q + 3]);
                    } else {
                        for (int j = 0; j < 16 && o0 + j < p.oc; ++j)
                            dst[j] = p.rows_epi == MB_EPI_RESIDUAL ? dst[j] + y[j] : y[j];
                    }
                }
                continue;
            }
            // every global read of the group first (the pointers may alias, so the compiler
            // would otherwise keep each read behind the previous column's store)
            float r[16], s[16];
            const unsigned at0 = (unsigned)o0 * (unsigned)p.L + (unsigned)t;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const bool ok = t_ok && o0 + j < p.oc;
                const unsigned at = at0 + (unsigned)j * (unsigned)p.L;
                r[j] = (ok && p.res != nullptr) ? p.res[at] : 0.0f;
                s[j] = (ok && p.acc_mode >= 2) ? p.acc[at] : 0.0f;
            }
            __align__(16) __half hi[16], lo[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int o = o0 + j;
                float a = 0.0f;
                if (o < p.oc && t_ok) {
                    const unsigned at = at0 + (unsigned)j * (unsigned)p.L;
                    const float4 ch = __ldg(p.chan + o);
                    const bool snake = o < snake_ch;
                    const float y = r[j] + fmaf(v[j], p.inv_scale, ch.x);
                    if (p.out != nullptr) p.out[at] = y;
                    if (p.has_alpha) a = snake_with(y, snake, ch.y, ch.z);
                    if (p.acc_mode == 1) {
                        p.acc[at] = y;
                    } else if (p.acc_mode == 2) {
                        p.acc[at] = s[j] + y;
                    } else if (p.acc_mode == 3) {
                        float s3 = (s[j] + y) * (1.0f / 3.0f);
                        if (p.has_alpha2) s3 = snake_with(s3, snake, ch.w, 1.0f / (ch.w + 1e-9f));
                        p.acc[at] = s3;
                    }
                }
                hi[j] = __float2half_rn(a);
                lo[j] = __float2half_rn(a - __half2float(hi[j]));
            }
            if (p.act_hi != nullptr && t_ok && o0 < p.cp_out) {
                uint4 *dh = reinterpret_cast<uint4 *>(p.act_hi + (size_t)t * p.cp_out + o0);
                uint4 *dl = reinterpret_cast<uint4 *>(p.act_lo + (size_t)t * p.cp_out + o0);
                dh[0] = reinterpret_cast<const uint4 *>(hi)[0];
                dh[1] = reinterpret_cast<const uint4 *>(hi)[1];
                dl[0] = reinterpret_cast<const uint4 *>(lo)[0];
                dl[1] = reinterpret_cast<const uint4 *>(lo)[1];
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// f32 [C][L] -> half-Snake -> f16 planes [L][cp] (channels contiguous), through a 32 x 32 tile.
__global__ void __launch_bounds__(256)
k_snake_planes(const float *__restrict__ in, const float *__restrict__ alpha, __half *__restrict__ hi,
               __half *__restrict__ lo, int C, int L, int cp) {
    __shared__ float tile[32][33];
    mb_pdl_wait();
    mb_pdl_trigger();
    const int t0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 8 rows per pass
    for (int r = ty; r < 32; r += 8) {
        const int c = c0 + r, t = t0 + tx;
        tile[r][tx] = (c < C && t < L) ? snake_fast(in[(size_t)c * L + t], c, C / 2, alpha) : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int t = t0 + r, c = c0 + tx;
        if (t < L && c < cp) {
            const float v = tile[tx][r];
            const __half h = __float2half_rn(v);
            hi[(size_t)t * cp + c] = h;
            lo[(size_t)t * cp + c] = __float2half_rn(v - __half2float(h));
        }
    }
}

// f32 rows [rows][k] (row stride ld) -> f16 hi/lo planes [rows][k].
__global__ void __launch_bounds__(256)
k_split_rows(const float *__restrict__ x, __half *__restrict__ hi, __half *__restrict__ lo, int k, int ld) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const float v = x[(size_t)r * ld + i];
        const __half h = __float2half_rn(v);
        hi[(size_t)r * k + i] = h;
        lo[(size_t)r * k + i] = __float2half_rn(v - __half2float(h));
    }
}

// Per output channel {bias, alpha, 1 / (alpha + 1e-9), alpha2}: what the epilogue needs of a
// channel in one 16-byte read.
__global__ void k_channel_table(const float *__restrict__ bias, const float *__restrict__ alpha,
                                const float *__restrict__ alpha2, float4 *__restrict__ table, int oc) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= oc) return;
    const float a = alpha != nullptr ? alpha[o] : 1.0f;
    table[o] = make_float4(bias[o], a, 1.0f / (a + 1e-9f), alpha2 != nullptr ? alpha2[o] : 1.0f);
}

// [oc][ic][K] f32 -> planes [2][K][rows][cp] f16 of scale * w (zero where no channel).
__global__ void k_pack_conv_weight_tc(const float *__restrict__ w, __half *__restrict__ packed, int oc, int ic, int K,
                                      int rows, int cp, float scale) {
    const size_t plane = (size_t)K * rows * cp;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < plane; idx += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % cp);
        const int o = (int)((idx / cp) % rows);
        const int k = (int)(idx / ((size_t)cp * rows));
        const float v = (o < oc && i < ic) ? w[((size_t)o * ic + i) * K + k] * scale : 0.0f;
        const __half h = __float2half_rn(v);
        packed[idx] = h;
        packed[plane + idx] = __float2half_rn(v - __half2float(h));
    }
}

}  // namespace

extern "C" int mb_codec_tc_init(void) {
    return (int)cudaFuncSetAttribute(k_conv1d_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
}

// Output channels per tile, tiles, and padded channel count of a convolution with `oc` outputs.
extern "C" void mb_codec_tc_shape(size_t oc, size_t *n_tile, size_t *tiles, size_t *cp) {
    const size_t n = oc > 112u ? 112u : (oc + 15u) / 16u * 16u;
    *n_tile = n;
    *tiles = (oc + n - 1u) / n;
    *cp = (oc + 63u) / 64u * 64u;
}

extern "C" size_t mb_codec_tc_packed_halves(size_t oc, size_t ic, size_t kernel) {
    size_t n, tiles, cp_o, cp_i;
    mb_codec_tc_shape(oc, &n, &tiles, &cp_o);
    cp_i = (ic + 63u) / 64u * 64u;
    return 2u * kernel * tiles * n * cp_i;
}

extern "C" int mb_codec_tc_pack_weight(const float *w, void *packed, size_t oc, size_t ic, size_t kernel, float scale,
                                       mb_stream stream) {
    size_t n, tiles, cp_o;
    mb_codec_tc_shape(oc, &n, &tiles, &cp_o);
    const size_t cp_i = (ic + 63u) / 64u * 64u;
    k_pack_conv_weight_tc<<<512, 256, 0, (cudaStream_t)stream>>>(w, static_cast<__half *>(packed), (int)oc, (int)ic, (int)kernel,
                                                                 (int)(tiles * n), (int)cp_i, scale);
    return mb_check_launch();
}

extern "C" int mb_codec_tc_channel_table(const float *bias, const float *alpha, const float *alpha2, float *table, size_t oc,
                                         mb_stream stream) {
    if (bias == nullptr || table == nullptr || oc == 0 || ((uintptr_t)table & 15u) != 0) return (int)cudaErrorInvalidValue;
    k_channel_table<<<(unsigned)((oc + 127u) / 128u), 128, 0, (cudaStream_t)stream>>>(bias, alpha, alpha2,
                                                                                     reinterpret_cast<float4 *>(table), (int)oc);
    return mb_check_launch();
}

extern "C" int mb_split_rows_f16(const float *x, void *hi, void *lo, size_t rows, size_t k, size_t ld, mb_stream stream) {
    if (rows == 0 || k == 0 || ld < k) return (int)cudaErrorInvalidValue;
    mb_launch(k_split_rows, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, x, static_cast<__half *>(hi),
              static_cast<__half *>(lo), (int)k, (int)ld);
    return mb_check_launch();
}

extern "C" int mb_codec_snake_planes(const float *in, const float *alpha, void *hi, void *lo, size_t channels, size_t length,
                                     mb_stream stream) {
    if (channels == 0 || length == 0) return (int)cudaErrorInvalidValue;
    const size_t cp = (channels + 63u) / 64u * 64u;
    mb_launch(k_snake_planes, dim3((unsigned)((length + 31u) / 32u), (unsigned)(cp / 32u)), dim3(256), 0, (cudaStream_t)stream, in,
              alpha, static_cast<__half *>(hi), static_cast<__half *>(lo), (int)channels, (int)length, (int)cp);
    return mb_check_launch();
}

extern "C" int mb_codec_conv1d_tc(const mb_codec_conv_tc_args *a, mb_stream stream) {
    if (a == nullptr || a->x_planes == nullptr || a->w_packed == nullptr ||
        (a->channel_table == nullptr && a->rows_out == nullptr) || a->ic == 0 || a->oc == 0 ||
        (a->rows_out != nullptr && ((a->rows_stride % 4u) != 0 || ((uintptr_t)a->rows_out & 15u) != 0)) ||
        a->length == 0 || a->kernel == 0 || a->dilation == 0 || (a->has_alpha && a->act_planes == nullptr) ||
        a->oc * a->length > 0xffffffffull ||
        (a->acc_mode != 0 && a->acc == nullptr) || a->scale <= 0.0f ||
        (((uintptr_t)a->x_planes | (uintptr_t)a->w_packed | (uintptr_t)a->act_planes) & 15u) != 0)
        return (int)cudaErrorInvalidValue;
    size_t n, tiles, cp_o;
    mb_codec_tc_shape(a->oc, &n, &tiles, &cp_o);
    const size_t cp_i = (a->ic + 63u) / 64u * 64u, L = a->length, rows = tiles * n;
    // a short signal leaves SMs without a tile: narrower tiles of output channels then (each
    // re-reads the activation slab, which stays in L2); rows past the packed matrix read as zeros
    {
        const size_t m_tiles = (L + CT_TM - 1) / CT_TM, sms = a->sm_count > 0 ? (size_t)a->sm_count : 148u;
        static const size_t narrower[] = {64u, 48u, 32u, 16u};
        for (size_t i = 0; i < 4 && m_tiles * tiles < sms; ++i)
            if (narrower[i] < n) {
                n = narrower[i];
                tiles = (a->oc + n - 1u) / n;
            }
    }
    CUtensorMap map_x, map_w;
    // activations: (channel bytes, time, plane); box 128 B x (128 + halo) times of one plane
    const size_t xdims[3] = {cp_i * 2u, L, 2u};
    const size_t xstrides[2] = {cp_i * 2u, a->x_plane_stride * 2u};
    const size_t halo = (a->kernel - 1u) * a->dilation;
    if (halo > (size_t)CT_HALO_MAX) return (int)cudaErrorInvalidValue;
    const size_t xrows = (size_t)CT_TM + halo;
    const unsigned xbox[3] = {(unsigned)CT_KC, (unsigned)xrows, 1u};
    // weights: (channel bytes, output row, tap, plane); box 128 B x N rows x 1 tap x both planes
    const size_t wdims[4] = {cp_i * 2u, rows, a->kernel, 2u};
    const size_t wstrides[3] = {cp_i * 2u, rows * cp_i * 2u, a->kernel * rows * cp_i * 2u};
    const unsigned wbox[4] = {(unsigned)CT_KC, (unsigned)n, 1u, 2u};
    if (!mb_make_map_nd(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->x_planes, 3, xdims, xstrides, xbox, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !mb_make_map_nd(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->w_packed, 4, wdims, wstrides, wbox, CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;
    ConvTcP p;
    memset(&p, 0, sizeof(p));
    p.chan = reinterpret_cast<const float4 *>(a->channel_table);
    p.has_alpha = a->has_alpha; p.has_alpha2 = a->has_alpha2;
    p.res = a->res; p.out = a->out; p.acc = a->acc;
    p.rows_out = a->rows_out; p.rows_stride = (int)a->rows_stride; p.rows_epi = a->rows_epilogue;
    p.act_hi = static_cast<__half *>(a->act_planes);
    p.act_lo = p.act_hi != nullptr ? p.act_hi + a->act_plane_stride : nullptr;
    p.status = a->status;
    p.inv_scale = 1.0f / a->scale;
    p.oc = (int)a->oc; p.L = (int)L; p.K = (int)a->kernel; p.dil = (int)a->dilation; p.n_tile = (int)n;
    p.chunks = (int)(cp_i / 64u);
    p.cp_out = (int)cp_o;
    p.acc_mode = a->acc_mode;
    p.xrows = (int)xrows;
    p.x_plane_bytes = (int)((xrows * CT_KC + 1023u) / 1024u * 1024u);
    // two CTAs per SM (one's epilogue runs beside the other's MMAs): 111 KB each
    const size_t budget = 111u * 1024u, stage_bytes = 2u * n * CT_KC;
    const size_t steps = a->kernel * (cp_i / 64u), chunks = cp_i / 64u;
    size_t xbufs = chunks > 1 && 4u * (size_t)p.x_plane_bytes + 2u * stage_bytes <= budget ? 2u : 1u;
    const size_t x_bytes = xbufs * 2u * (size_t)p.x_plane_bytes;
    if (x_bytes + stage_bytes > budget) return (int)cudaErrorInvalidValue;
    size_t stages = (budget - x_bytes) / stage_bytes;
    if (stages > CT_MAX_STAGES) stages = CT_MAX_STAGES;
    if (stages > steps) stages = steps;
    p.stages = (int)stages;
    p.xbufs = (int)xbufs;
    const size_t smem = x_bytes + stages * stage_bytes + 1024u;
    mb_launch(k_conv1d_tc, dim3((unsigned)((L + CT_TM - 1) / CT_TM), (unsigned)tiles), dim3(CT_THREADS), smem, (cudaStream_t)stream,
              map_x, map_w, p);
    return mb_check_launch();
}
