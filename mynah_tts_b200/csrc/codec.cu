// NanoCodec decoder kernels: FSQ de-index, causal convolution with fused epilogues, grouped
// causal transposed convolution, half-Snake.  Activations are [channels][length] f32, time
// contiguous, as in the reference (decode_codec, src/graph.c:2640-2780).
//
// Summation order.  The reference forms a causal convolution as one scalar product per output
// over p = i * kernel + k (unfolded input, src/graph.c:2059-2096; scalar sgemm,
// src/backend.c:343-354), then c = 1 * sum + 1 * bias.  k_conv1d keeps exactly that order: each
// thread owns MO x MT outputs and walks the input channels and taps in order, one accumulator
// per output, no split of the reduction.  STRICT rounds the product and the sum separately
// and evaluates Snake's sinf as the host's libm does; the fast form contracts them into FMAs
// and uses CUDA's sinf.
#include "common.cuh"
#include "launch.h"
#include "libm_parity.cuh"

namespace {

constexpr int CV_MO = 7;          // output channels per thread: the codec's widths are 27 * 2^n
constexpr int CV_SLOT = 8;        // floats a thread's MO weights occupy in the packed layout
constexpr int CV_ICC = 8;         // input channels per shared-memory chunk
constexpr int CV_HALO_MAX = 52;   // (kernel - 1) * dilation <= 50, rounded to 4

template <bool STRICT>
__device__ __forceinline__ float snake_value(float v, float a, float inv_a, const uint32_t *sin_tab) {
    // snake_row, src/backend.c:643-658: v + sn * sn * (1 / (a + 1e-9))
    if (STRICT) {
        const float sn = mb_sinf_host(__fmul_rn(a, v), sin_tab);
        return __fadd_rn(v, __fmul_rn(__fmul_rn(sn, sn), inv_a));
    }
    const float sn = sinf(a * v);
    return v + sn * sn * inv_a;
}

template <bool STRICT>
__device__ __forceinline__ float half_snake_value(float v, int c, int snake_ch, const float *alpha, const uint32_t *sin_tab) {
    if (c < snake_ch) {
        const float a = alpha[c];
        const float inv_a = __fdiv_rn(1.0f, __fadd_rn(a, 1e-9f));
        return snake_value<STRICT>(v, a, inv_a, sin_tab);
    }
    return v < 0.0f ? __fmul_rn(v, 0.01f) : v;
}

struct ConvP {
    const float *in;        // [ic][L]
    const float *w;         // packed: [ic * K][groups_alloc][8], group g = output channels 7g .. 7g+6
    const float *bias;      // [oc]
    const float *res;       // optional [oc][L]: v = res + v
    float *out;             // optional [oc][L]: v
    const float *alpha;     // optional [oc]: out_act = half_snake(v)
    float *out_act;
    float *acc;             // optional [oc][L] branch sum (acc_mode)
    const float *alpha2;    // acc_mode 3: half-Snake of the finished sum (the next stage's activation), or NULL
    const uint32_t *sin_tab;
    int ic, oc, L, dil, groups_alloc;
    int acc_mode;           // 0 none; 1 acc = 0 + v; 2 acc += v; 3 acc = (acc + v) / 3 (then alpha2)
    int clip;               // clamp v to [-1, 1] before storing out
};

// CTA = WARPS warps; warp w owns output channels 7 * (blockIdx.y * WARPS + w) .. +6, lane l owns
// times t0 + l + 32 j (j < MT).
template <int K, int WARPS, int MT, bool STRICT>
__global__ void __launch_bounds__(WARPS * 32)
k_conv1d(const ConvP p) {
    constexpr int TT = 32 * MT;
    constexpr int XW = TT + CV_HALO_MAX;
    __shared__ __align__(16) float wsm[CV_ICC * K][WARPS][CV_SLOT];
    __shared__ float xsm[CV_ICC][XW];
    mb_pdl_wait();
    mb_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TT;
    const int g0 = blockIdx.y * WARPS;
    const int halo = (K - 1) * p.dil;
    float acc[CV_MO][MT];
#pragma unroll
    for (int m = 0; m < CV_MO; ++m)
#pragma unroll
        for (int j = 0; j < MT; ++j) acc[m][j] = 0.0f;

    for (int i0 = 0; i0 < p.ic; i0 += CV_ICC) {
        const int ni = min(CV_ICC, p.ic - i0);
        __syncthreads();
        // weights of the chunk: rows (i0 * K) .. of the packed matrix, WARPS groups of 8 floats
        {
            const float4 *src = reinterpret_cast<const float4 *>(p.w);
            float4 *dst = reinterpret_cast<float4 *>(&wsm[0][0][0]);
            const int per_row = WARPS * 2;
            for (int idx = threadIdx.x; idx < ni * K * per_row; idx += WARPS * 32) {
                const int row = idx / per_row, q = idx - row * per_row;
                dst[idx] = __ldg(src + ((size_t)(i0 * K + row) * p.groups_alloc + g0) * 2 + q);
            }
        }
        for (int idx = threadIdx.x; idx < ni * (TT + halo); idx += WARPS * 32) {
            const int i = idx / (TT + halo), tt = idx - i * (TT + halo);
            const int t = t0 - halo + tt;
            xsm[i][tt] = (t >= 0 && t < p.L) ? __ldg(p.in + (size_t)(i0 + i) * p.L + t) : 0.0f;
        }
        __syncthreads();
        for (int i = 0; i < ni; ++i) {
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const float4 wa = *reinterpret_cast<const float4 *>(&wsm[i * K + k][warp][0]);
                const float4 wb = *reinterpret_cast<const float4 *>(&wsm[i * K + k][warp][4]);
                const float wv[CV_MO] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z};
                const int base = k * p.dil + lane;          // halo - (K-1-k) * dil + lane
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    const float xv = xsm[i][base + 32 * j];
#pragma unroll
                    for (int m = 0; m < CV_MO; ++m)
                        acc[m][j] = STRICT ? __fadd_rn(acc[m][j], __fmul_rn(wv[m], xv)) : fmaf(wv[m], xv, acc[m][j]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < CV_MO; ++m) {
        const int o = (g0 + warp) * CV_MO + m;
        if (o >= p.oc) continue;
        const float b = p.bias[o];
#pragma unroll
        for (int j = 0; j < MT; ++j) {
            const int t = t0 + lane + 32 * j;
            if (t >= p.L) continue;
            const size_t at = (size_t)o * p.L + t;
            float v = __fadd_rn(acc[m][j], b);
            if (p.res != nullptr) v = __fadd_rn(p.res[at], v);
            if (p.clip) v = v > 1.0f ? 1.0f : (v < -1.0f ? -1.0f : v);
            if (p.out != nullptr) p.out[at] = v;
            if (p.alpha != nullptr) p.out_act[at] = half_snake_value<STRICT>(v, o, p.oc / 2, p.alpha, p.sin_tab);
            if (p.acc_mode == 1) {
                p.acc[at] = __fadd_rn(0.0f, v);
            } else if (p.acc_mode == 2) {
                p.acc[at] = __fadd_rn(p.acc[at], v);
            } else if (p.acc_mode == 3) {
                float s = __fdiv_rn(__fadd_rn(p.acc[at], v), 3.0f);
                if (p.alpha2 != nullptr) s = half_snake_value<STRICT>(s, o, p.oc / 2, p.alpha2, p.sin_tab);
                p.acc[at] = s;
            }
        }
    }
}

// [oc][ic][K] -> packed [ic * K][groups_alloc][8] (zero where no channel)
__global__ void k_pack_conv_weight(const float *__restrict__ w, float *__restrict__ packed, int oc, int ic, int K,
                                   int groups_alloc) {
    const size_t n = (size_t)ic * K * groups_alloc * CV_SLOT;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int slot = (int)(idx % CV_SLOT);
        const int g = (int)((idx / CV_SLOT) % groups_alloc);
        const size_t row = idx / ((size_t)CV_SLOT * groups_alloc);     // i * K + k
        const int o = g * CV_MO + slot;
        packed[idx] = (slot < CV_MO && o < oc) ? w[(size_t)o * ic * K + row] : 0.0f;
    }
}

// decode_codec's de-index (src/graph.c:2657-2669): codes [8][T] -> latent [32][T]
__global__ void k_fsq_latent(const unsigned *__restrict__ codes, float *__restrict__ latent, int T) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= 32 * T) return;
    const int c = idx / T, t = idx - c * T;
    const int g = c >> 2, d = c & 3;
    const unsigned levels[4] = {8u, 7u, 6u, 6u}, bases[4] = {1u, 8u, 56u, 336u};
    const unsigned digit = (codes[g * T + t] / bases[d]) % levels[d];
    const float half = (float)(levels[d] / 2u);
    latent[idx] = __fdiv_rn(__fsub_rn((float)digit, half), half);
}

// convt_channel (src/graph.c:2179-2198) with kernel = 2 * stride: output p of channel o sums,
// per input channel of its group in order, the taps of t = p / stride - 1 then t = p / stride.
template <bool STRICT>
__global__ void __launch_bounds__(256)
k_conv_transpose(const float *__restrict__ in, const float *__restrict__ w, const float *__restrict__ bias,
                 float *__restrict__ out, int ic, int oc, int L, int stride) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int out_len = L * stride, K = 2 * stride, ipg = ic / oc;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)oc * out_len) return;
    const int o = (int)(idx / out_len), pos = (int)(idx - (size_t)o * out_len);
    const int q = pos / stride, r = pos - q * stride;
    float v = bias[o];
    for (int i = o * ipg; i < (o + 1) * ipg; ++i) {
        const float *row = in + (size_t)i * L;
        const float *wk = w + (size_t)i * K;
        if (q >= 1) v = STRICT ? __fadd_rn(v, __fmul_rn(row[q - 1], wk[r + stride])) : fmaf(row[q - 1], wk[r + stride], v);
        if (q < L) v = STRICT ? __fadd_rn(v, __fmul_rn(row[q], wk[r])) : fmaf(row[q], wk[r], v);
    }
    out[idx] = v;
}

template <bool STRICT>
__global__ void __launch_bounds__(256)
k_half_snake(const float *__restrict__ in, float *__restrict__ out, const float *__restrict__ alpha, int channels,
             int L, int snake_ch, const uint32_t *__restrict__ sin_tab) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)channels * L) return;
    out[idx] = half_snake_value<STRICT>(in[idx], (int)(idx / L), snake_ch, alpha, sin_tab);
}

// unfold of the seam's im2col entry: columns[(i * K + k)][t] = in[i][t - (K-1-k) * dil]
__global__ void k_im2col_causal(const float *__restrict__ in, float *__restrict__ col, int ic, int L, int K, int dil) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)ic * K * L) return;
    const int t = (int)(idx % L);
    const int k = (int)((idx / L) % K);
    const int i = (int)(idx / ((size_t)L * K));
    const int src = t - (K - 1 - k) * dil;
    col[idx] = src >= 0 ? in[(size_t)i * L + src] : 0.0f;
}

template <int K, int WARPS, bool STRICT>
int launch_conv_mt(const ConvP &p, int sms, cudaStream_t s) {
    const int groups = (p.oc + CV_MO - 1) / CV_MO;
    const unsigned gy = (unsigned)((groups + WARPS - 1) / WARPS);
    // four times per thread unless that leaves SMs without a CTA
    const long ctas4 = (long)((p.L + 127) / 128) * gy;
    if (ctas4 >= sms || p.L <= 32)
        mb_launch(k_conv1d<K, WARPS, 4, STRICT>, dim3((unsigned)((p.L + 127) / 128), gy), dim3(WARPS * 32), 0, s, p);
    else
        mb_launch(k_conv1d<K, WARPS, 1, STRICT>, dim3((unsigned)((p.L + 31) / 32), gy), dim3(WARPS * 32), 0, s, p);
    return mb_check_launch();
}

template <int K, bool STRICT>
int launch_conv_k(const ConvP &p, int sms, cudaStream_t s) {
    const int groups = (p.oc + CV_MO - 1) / CV_MO;
    if (groups >= 8) return launch_conv_mt<K, 8, STRICT>(p, sms, s);
    return launch_conv_mt<K, 4, STRICT>(p, sms, s);
}

}  // namespace

extern "C" size_t mb_codec_conv_groups_alloc(size_t oc) {
    const size_t groups = (oc + CV_MO - 1) / CV_MO;
    return (groups + 7u) / 8u * 8u;          // whole CTAs of 8 (or 4) warps
}

extern "C" size_t mb_codec_conv_packed_floats(size_t oc, size_t ic, size_t kernel) {
    return ic * kernel * mb_codec_conv_groups_alloc(oc) * CV_SLOT;
}

extern "C" int mb_codec_pack_conv_weight(const float *w, float *packed, size_t oc, size_t ic, size_t kernel, mb_stream stream) {
    k_pack_conv_weight<<<256, 256, 0, (cudaStream_t)stream>>>(w, packed, (int)oc, (int)ic, (int)kernel,
                                                              (int)mb_codec_conv_groups_alloc(oc));
    return mb_check_launch();
}

extern "C" int mb_codec_conv1d(const mb_codec_conv_args *a, mb_stream stream) {
    if (a == nullptr || a->in == nullptr || a->w_packed == nullptr || a->bias == nullptr || a->ic == 0 || a->oc == 0 ||
        a->length == 0 || a->dilation == 0 || (a->kernel - 1u) * a->dilation > (size_t)CV_HALO_MAX - 2u ||
        (a->alpha != nullptr && a->out_act == nullptr) || (a->acc_mode != 0 && a->acc == nullptr))
        return (int)cudaErrorInvalidValue;
    ConvP p;
    p.in = a->in; p.w = a->w_packed; p.bias = a->bias; p.res = a->res; p.out = a->out; p.alpha = a->alpha;
    p.out_act = a->out_act; p.acc = a->acc; p.alpha2 = a->alpha2; p.sin_tab = a->sin_tab;
    p.ic = (int)a->ic; p.oc = (int)a->oc; p.L = (int)a->length; p.dil = (int)a->dilation;
    p.groups_alloc = (int)mb_codec_conv_groups_alloc(a->oc);
    p.acc_mode = a->acc_mode; p.clip = a->clip;
    const int sms = a->sm_count > 0 ? a->sm_count : 148;
    cudaStream_t s = (cudaStream_t)stream;
    const bool strict = a->strict != 0;
    switch (a->kernel) {
    case 3: return strict ? launch_conv_k<3, true>(p, sms, s) : launch_conv_k<3, false>(p, sms, s);
    case 7: return strict ? launch_conv_k<7, true>(p, sms, s) : launch_conv_k<7, false>(p, sms, s);
    case 11: return strict ? launch_conv_k<11, true>(p, sms, s) : launch_conv_k<11, false>(p, sms, s);
    default: return (int)cudaErrorInvalidValue;
    }
}

extern "C" int mb_codec_fsq_latent(const unsigned *codes, float *latent, size_t frames, mb_stream stream) {
    if (frames == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_fsq_latent, dim3((unsigned)((32u * frames + 255u) / 256u)), dim3(256), 0, (cudaStream_t)stream, codes, latent,
              (int)frames);
    return mb_check_launch();
}

extern "C" int mb_codec_conv_transpose(const float *in, const float *w, const float *bias, float *out, size_t ic, size_t oc,
                                       size_t length, size_t stride, int strict, mb_stream stream) {
    if (ic == 0 || oc == 0 || ic % oc != 0 || length == 0 || stride == 0) return (int)cudaErrorInvalidValue;
    const size_t n = oc * length * stride;
    const dim3 grid((unsigned)((n + 255u) / 256u)), block(256);
    if (strict) mb_launch(k_conv_transpose<true>, grid, block, 0, (cudaStream_t)stream, in, w, bias, out, (int)ic, (int)oc, (int)length, (int)stride);
    else mb_launch(k_conv_transpose<false>, grid, block, 0, (cudaStream_t)stream, in, w, bias, out, (int)ic, (int)oc, (int)length, (int)stride);
    return mb_check_launch();
}

extern "C" int mb_codec_half_snake(const float *in, float *out, const float *alpha, size_t channels, size_t length,
                                   size_t snake_channels, int strict, const uint32_t *sin_tab, mb_stream stream) {
    if (channels == 0 || length == 0) return (int)cudaErrorInvalidValue;
    const size_t n = channels * length;
    const dim3 grid((unsigned)((n + 255u) / 256u)), block(256);
    if (strict) mb_launch(k_half_snake<true>, grid, block, 0, (cudaStream_t)stream, in, out, alpha, (int)channels, (int)length, (int)snake_channels, sin_tab);
    else mb_launch(k_half_snake<false>, grid, block, 0, (cudaStream_t)stream, in, out, alpha, (int)channels, (int)length, (int)snake_channels, sin_tab);
    return mb_check_launch();
}

extern "C" int mb_codec_im2col(const float *in, float *col, size_t ic, size_t length, size_t kernel, size_t dilation,
                               mb_stream stream) {
    const size_t n = ic * kernel * length;
    if (n == 0) return (int)cudaErrorInvalidValue;
    k_im2col_causal<<<(unsigned)((n + 255u) / 256u), 256, 0, (cudaStream_t)stream>>>(in, col, (int)ic, (int)length, (int)kernel,
                                                                                   (int)dilation);
    return mb_check_launch();
}
