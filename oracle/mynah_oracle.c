/* CPU restatement of the Magpie decoder-step hot path of mynah-tts.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker for the CUDA
 * library: tests, the smoke check and the benchmark's CPU-baseline leg may call
 * it; no product code path links, loads or falls back to it.
 *
 * Every function restates, in plain scalar C11, what the reference computes
 * when its host code is built the way its own CUDA variant builds it
 * (`-std=c11 -O2`, no SIMD, no -ffast-math; Makefile:261): all reductions run
 * in source order, products and sums are rounded separately (no contraction).
 * Build this file with exactly those flags; anything else changes rounding.
 *
 * Parity pins: the reference's known answers (src/kernels.c:439-517,
 * src/qmat.c:904-1179, src/backend.c:290-310, gpu/metal/backend_metal_ops.m:
 * 1049-1079) and bit-equality with the reference's own sources compiled into
 * oracle/_ref (checked in tests/ wherever that library exists, and through
 * committed fixtures generated from it).
 *
 * f16 weights: the reference has no x86 implementation (src/qmat.c:22-28,
 * 580-583), so that mode restates the aarch64 kernel (src/qmat.c:319-377) and
 * is pinned only by the reference's own 1e-3 bound (src/qmat.c:1064-1104):
 * "parity unpinned" beyond that bound.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_F32 0
#define ORC_INT8 1
#define ORC_INT4 2
#define ORC_F16 3
#define ORC_Q4_GROUP 32u
#define ORC_K_MAX 8192u

/* ------------------------------------------------------------ half floats */
/* IEEE binary16 <-> binary32, round to nearest even: the `(__fp16)w[i]` cast
 * of src/qmat.c:655. */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | (absx > 0x7f800000u ? 0x200u | ((absx >> 13) & 0x3ffu) : 0u));
    }
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf */
    if (absx < 0x33000001u) return (uint16_t)sign;               /* rounds to zero */
    int exp = (int)(absx >> 23) - 127;
    uint32_t mant = (absx & 0x7fffffu) | 0x800000u;
    uint32_t half;
    if (exp < -14) { /* subnormal half */
        const int shift = -14 - exp + 13;
        const uint32_t rem_mask = (1u << shift) - 1u;
        const uint32_t rem = mant & rem_mask;
        const uint32_t halfway = 1u << (shift - 1);
        half = mant >> shift;
        if (rem > halfway || (rem == halfway && (half & 1u))) half += 1u;
    } else {
        half = ((uint32_t)(exp + 15) << 10) | ((mant >> 13) & 0x3ffu);
        const uint32_t rem = mant & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half += 1u;
    }
    return (uint16_t)(sign | half);
}

float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t mant = h & 0x3ffu;
    uint32_t x;
    if (exp == 0) {
        if (mant == 0) x = sign;
        else {
            int e = -1;
            do { mant <<= 1; ++e; } while ((mant & 0x400u) == 0);
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mant & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7f800000u | (mant << 13);
    } else {
        x = sign | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* -------------------------------------------------------------- quantizers */
/* src/qmat.c:39-57 */
void orc_quantize_weight_int8(const float *w, size_t n, size_t k, int8_t *q, float *scales) {
    for (size_t i = 0; i < n; ++i) {
        const float *row = w + i * k;
        float amax = 0.0f;
        for (size_t j = 0; j < k; ++j) {
            const float a = fabsf(row[j]);
            if (a > amax) amax = a;
        }
        const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        scales[i] = scale;
        const float inv = 1.0f / scale;
        for (size_t j = 0; j < k; ++j) {
            const float v = row[j] * inv;
            q[i * k + j] = (int8_t)(v >= 0.0f ? v + 0.5f : v - 0.5f);
        }
    }
}

/* src/qmat.c:59-91: groups of 32 along k, low nibble = even index, +8 offset */
void orc_quantize_weight_int4(const float *w, size_t n, size_t k, uint8_t *q, float *scales) {
    const size_t groups = k / ORC_Q4_GROUP;
    for (size_t i = 0; i < n; ++i) {
        for (size_t g = 0; g < groups; ++g) {
            const float *grp = w + i * k + g * ORC_Q4_GROUP;
            float amax = 0.0f;
            for (size_t j = 0; j < ORC_Q4_GROUP; ++j) {
                const float a = fabsf(grp[j]);
                if (a > amax) amax = a;
            }
            const float scale = amax > 0.0f ? amax / 7.0f : 1.0f;
            scales[i * groups + g] = scale;
            const float inv = 1.0f / scale;
            for (size_t j = 0; j < ORC_Q4_GROUP; j += 2) {
                const float v0 = grp[j] * inv;
                const float v1 = grp[j + 1] * inv;
                int q0 = (int)(v0 >= 0.0f ? v0 + 0.5f : v0 - 0.5f);
                int q1 = (int)(v1 >= 0.0f ? v1 + 0.5f : v1 - 0.5f);
                if (q0 < -8) q0 = -8;
                if (q0 > 7) q0 = 7;
                if (q1 < -8) q1 = -8;
                if (q1 > 7) q1 = 7;
                q[i * (k / 2u) + (g * ORC_Q4_GROUP + j) / 2u] = (uint8_t)((q0 + 8) | ((q1 + 8) << 4));
            }
        }
    }
}

/* src/qmat.c:650-655 */
void orc_quantize_weight_f16(const float *w, size_t count, uint16_t *h) {
    for (size_t i = 0; i < count; ++i) h[i] = orc_f32_to_f16(w[i]);
}

/* src/qmat.c:93-113 */
float orc_quantize_act_int8(int8_t *qx, const float *x, size_t k) {
    float amax = 0.0f;
    for (size_t i = 0; i < k; ++i) {
        const float a = fabsf(x[i]);
        if (a > amax) amax = a;
    }
    if (amax == 0.0f) {
        memset(qx, 0, k);
        return 0.0f;
    }
    const float inv = 127.0f / amax;
    for (size_t i = 0; i < k; ++i) {
        const float v = x[i] * inv;
        int q = (int)(v >= 0.0f ? v + 0.5f : v - 0.5f);
        if (q > 127) q = 127;
        if (q < -127) q = -127;
        qx[i] = (int8_t)q;
    }
    return amax / 127.0f;
}

/* ------------------------------------------------------------ dot kernels */
/* src/qmat.c:136-152 (portable branch); the int32 sum is exact. */
int32_t orc_dot_q8_i32(const int8_t *qx, const int8_t *w, size_t k) {
    int32_t s = 0;
    for (size_t j = 0; j < k; ++j) s += (int32_t)w[j] * (int32_t)qx[j];
    return s;
}

float orc_dot_q8(const int8_t *qx, float sx, const int8_t *w, float ws, size_t k) {
    return (float)orc_dot_q8_i32(qx, w, k) * ws * sx;
}

/* src/qmat.c:156-185 (portable branch): per group an exact int32 sum, then a
 * float accumulation in group order. */
float orc_dot_q4(const int8_t *qx, float sx, const uint8_t *q, const float *scales, size_t k) {
    const size_t groups = k / ORC_Q4_GROUP;
    float acc = 0.0f;
    for (size_t g = 0; g < groups; ++g) {
        int32_t gi = 0;
        for (size_t j = 0; j < ORC_Q4_GROUP; j += 2) {
            const uint8_t b = q[g * 16 + j / 2];
            const int lo = (int)(b & 0x0F) - 8;
            const int hi = (int)(b >> 4) - 8;
            gi += lo * (int32_t)qx[g * 32 + j] + hi * (int32_t)qx[g * 32 + j + 1];
        }
        acc += (float)gi * scales[g];
    }
    return acc * sx;
}

/* src/qmat.c:364-376: two 4-lane fused accumulators (j%8 in 0..3 and 4..7),
 * summed lane-wise, then a pairwise horizontal add, then the scalar tail. */
float orc_dot_f16(const float *x, const uint16_t *w, size_t k) {
    float a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
    size_t j = 0;
    for (; j + 8u <= k; j += 8u) {
        for (int l = 0; l < 4; ++l) {
            a[l] = fmaf(orc_f16_to_f32(w[j + l]), x[j + l], a[l]);
            b[l] = fmaf(orc_f16_to_f32(w[j + 4 + l]), x[j + 4 + l], b[l]);
        }
    }
    const float c0 = a[0] + b[0], c1 = a[1] + b[1], c2 = a[2] + b[2], c3 = a[3] + b[3];
    float s = (c0 + c1) + (c2 + c3);
    for (; j < k; ++j) s += orc_f16_to_f32(w[j]) * x[j];
    return s;
}

/* src/kernels.c:39-44 (portable branch) */
float orc_dot_f32(const float *a, const float *b, size_t n) {
    float sum = 0.0f;
    for (size_t i = 0; i < n; ++i) sum += a[i] * b[i];
    return sum;
}

/* -------------------------------------------------------------- layer ops */
/* src/kernels.c:186-244 (portable branch).  Magpie passes bias NULL and
 * epsilon 1e-5 (src/graph.c:147-150). */
void orc_layernorm(const float *input, const float *weight, const float *bias,
                   float *output, size_t rows, size_t width, float epsilon) {
    for (size_t row = 0; row < rows; ++row) {
        const float *x = input + row * width;
        float *y = output + row * width;
        float mean = 0.0f;
        for (size_t i = 0; i < width; ++i) mean += x[i];
        mean /= (float)width;
        float variance = 0.0f;
        for (size_t i = 0; i < width; ++i) {
            const float d = x[i] - mean;
            variance += d * d;
        }
        const float scale = 1.0f / sqrtf(variance / (float)width + epsilon);
        for (size_t i = 0; i < width; ++i) {
            y[i] = (x[i] - mean) * scale * weight[i] + (bias == NULL ? 0.0f : bias[i]);
        }
    }
}

/* src/kernels.c:382-389 */
void orc_gelu_scalar(float *data, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        const float x = data[i];
        const float cubic = x * x * x;
        const float c = 0.7978845608f * (x + 0.044715f * cubic);
        data[i] = 0.5f * x * (1.0f + tanhf(c));
    }
}

/* src/kernels.c:246-257 */
void orc_residual_add(float *output, const float *input, size_t n) {
    for (size_t i = 0; i < n; ++i) output[i] += input[i];
}

/* src/kernels.c:391-420 */
int orc_softmax(const float *logits, float *probabilities, size_t n) {
    if (n == 0) return -1;
    float maximum = logits[0];
    if (!isfinite(maximum)) return -1;
    for (size_t i = 1; i < n; ++i) {
        if (!isfinite(logits[i])) return -1;
        if (logits[i] > maximum) maximum = logits[i];
    }
    float total = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        probabilities[i] = expf(logits[i] - maximum);
        total += probabilities[i];
    }
    if (!(total > 0.0f) || !isfinite(total)) return -1;
    const float inverse_total = 1.0f / total;
    for (size_t i = 0; i < n; ++i) probabilities[i] *= inverse_total;
    return 0;
}

/* Constrained greedy pick, first index wins ties: src/backend.c:825-847 and
 * src/graph.c:1551-1566.  Candidates: ids below codebook_size, plus eos_id
 * when allow_eos. */
unsigned orc_argmax_constrained(const float *logits, size_t vocab, size_t codebook_size,
                                size_t eos_id, int allow_eos) {
    float best = -FLT_MAX;
    unsigned result = 0u;
    for (size_t i = 0; i < vocab; ++i) {
        if (!(i < codebook_size || (allow_eos && i == eos_id))) continue;
        if (logits[i] > best) {
            best = logits[i];
            result = (unsigned)i;
        }
    }
    return result;
}

/* ------------------------------------------------------- quantized linear */
typedef struct {
    int qtype;          /* effective type of this tensor (may fall back to f32) */
    size_t n, k;
    const float *w;     /* borrowed f32 weight [n,k] */
    int8_t *q8;
    uint8_t *q4;
    uint16_t *f16;
    float *scales;
} orc_qweight;

/* The get-or-create of src/qmat.c:627-679: INT4 refuses k not a multiple of 32
 * and the caller then uses the exact f32 product. */
int orc_qweight_init(orc_qweight *e, int qtype, const float *w, size_t n, size_t k) {
    memset(e, 0, sizeof(*e));
    e->n = n;
    e->k = k;
    e->w = w;
    e->qtype = qtype;
    if (k > ORC_K_MAX) e->qtype = ORC_F32;                        /* src/qmat.c:773-774 */
    if (qtype == ORC_INT4 && (k % ORC_Q4_GROUP) != 0) e->qtype = ORC_F32;
    if (e->qtype == ORC_INT8) {
        e->q8 = (int8_t *)malloc(n * k);
        e->scales = (float *)malloc(n * sizeof(float));
        if (!e->q8 || !e->scales) return -1;
        orc_quantize_weight_int8(w, n, k, e->q8, e->scales);
    } else if (e->qtype == ORC_INT4) {
        e->q4 = (uint8_t *)malloc(n * (k / 2u));
        e->scales = (float *)malloc(n * (k / ORC_Q4_GROUP) * sizeof(float));
        if (!e->q4 || !e->scales) return -1;
        orc_quantize_weight_int4(w, n, k, e->q4, e->scales);
    } else if (e->qtype == ORC_F16) {
        e->f16 = (uint16_t *)malloc(n * k * sizeof(uint16_t));
        if (!e->f16) return -1;
        orc_quantize_weight_f16(w, n * k, e->f16);
    }
    return 0;
}

void orc_qweight_free(orc_qweight *e) {
    free(e->q8);
    free(e->q4);
    free(e->f16);
    free(e->scales);
    memset(e, 0, sizeof(*e));
}

/* One activation row through a (possibly quantized) weight:
 * src/qmat.c:768-818 with the portable kernels; the f32 case is the scalar
 * backend product of src/backend.c:283-291. */
void orc_linear_row(const orc_qweight *e, const float *x, float *out, const float *bias) {
    const size_t n = e->n, k = e->k;
    if (e->qtype == ORC_F32) {
        for (size_t r = 0; r < n; ++r) out[r] = orc_dot_f32(e->w + r * k, x, k);
        if (bias != NULL) for (size_t r = 0; r < n; ++r) out[r] += bias[r];
        return;
    }
    if (e->qtype == ORC_F16) {
        for (size_t r = 0; r < n; ++r)
            out[r] = orc_dot_f16(x, e->f16 + r * k, k) + (bias == NULL ? 0.0f : bias[r]);
        return;
    }
    int8_t qx[ORC_K_MAX];
    const float sx = orc_quantize_act_int8(qx, x, k);
    for (size_t r = 0; r < n; ++r) {
        float value = e->qtype == ORC_INT8
                          ? orc_dot_q8(qx, sx, e->q8 + r * k, e->scales[r], k)
                          : orc_dot_q4(qx, sx, e->q4 + r * (k / 2u),
                                       e->scales + r * (k / ORC_Q4_GROUP), k);
        if (bias != NULL) value += bias[r];
        out[r] = value;
    }
}

/* Stand-alone form used by the single-op tests: y = LN(x) W^T + b when gain is
 * given, else y = x W^T + b.  rows are independent (src/qmat.c:790-816). */
int orc_qmat_linear(int qtype, const float *w, const float *x, float *out, size_t count,
                    size_t k, size_t n, const float *bias, const float *ln_gain) {
    orc_qweight e;
    if (orc_qweight_init(&e, qtype, w, n, k) != 0) return -1;
    float *nrm = (float *)malloc(k * sizeof(float));
    if (nrm == NULL) { orc_qweight_free(&e); return -1; }
    for (size_t t = 0; t < count; ++t) {
        const float *xr = x + t * k;
        if (ln_gain != NULL) {
            orc_layernorm(xr, ln_gain, NULL, nrm, 1u, k, 1.0e-5f);
            xr = nrm;
        }
        orc_linear_row(&e, xr, out + t * n, bias);
    }
    free(nrm);
    orc_qweight_free(&e);
    return 0;
}

/* --------------------------------------------------------------- attention */
/* Single-query attention of one head over `valid` cached rows:
 * src/graph.c:3182-3202 (self, stride = width) and 3221-3244 (cross). */
void orc_attend_head(const float *q, const float *kbase, const float *vbase, size_t valid,
                     size_t stride, size_t hw, float scale, float *scores, float *out) {
    float maxv = -FLT_MAX;
    for (size_t s = 0; s < valid; ++s) {
        const float *k = kbase + s * stride;
        float sc = 0.0f;
        for (size_t d = 0; d < hw; ++d) sc += q[d] * k[d];
        sc *= scale;
        scores[s] = sc;
        if (sc > maxv) maxv = sc;
    }
    float denom = 0.0f;
    for (size_t s = 0; s < valid; ++s) {
        scores[s] = expf(scores[s] - maxv);
        denom += scores[s];
    }
    memset(out, 0, hw * sizeof(float));
    for (size_t s = 0; s < valid; ++s) {
        const float weight = scores[s] / denom;
        const float *v = vbase + s * stride;
        for (size_t d = 0; d < hw; ++d) out[d] += weight * v[d];
    }
}

/* The resident-attention contract of src/backend.h:135-154: append K/V at
 * `position`, attend rows below `valid`, `heads` heads of `head_width`. */
void orc_self_attention(const float *qkv, float *k_cache, float *v_cache, size_t position,
                        size_t cache_stride, size_t valid, size_t heads, size_t head_width,
                        float scale, float *out, float *scores) {
    const size_t width = heads * head_width;
    memcpy(k_cache + position * cache_stride, qkv + width, width * sizeof(float));
    memcpy(v_cache + position * cache_stride, qkv + 2u * width, width * sizeof(float));
    for (size_t h = 0; h < heads; ++h)
        orc_attend_head(qkv + h * head_width, k_cache + h * head_width,
                        v_cache + h * head_width, valid, cache_stride, head_width, scale,
                        scores, out + h * head_width);
}

void orc_cross_attention(const float *q, const float *k_cache, const float *v_cache,
                         size_t valid, size_t cache_stride, size_t heads, size_t head_width,
                         float scale, float *out, float *scores) {
    for (size_t h = 0; h < heads; ++h)
        orc_attend_head(q + h * head_width, k_cache + h * head_width,
                        v_cache + h * head_width, valid, cache_stride, head_width, scale,
                        scores, out + h * head_width);
}

/* ------------------------------------------------------------------ model */
typedef struct {
    const float *norm_self, *norm_xattn_query, *norm_xattn_memory, *norm_pos_ff;
    orc_qweight qkv, o_self, q_cross, o_cross, ffn_up, ffn_down;
    const float *kv_cross_w; /* f32 [2*xw, width], used once per request */
} orc_layer;

typedef struct {
    size_t layers, width, heads, head_width, ffn_width, xattn_width;
    size_t tables, vocab, codebook_size, eos_id;
    int qtype;
    const float *position;   /* [max_positions, width] */
    const float *norm_out;   /* [width] */
    const float *const *embeddings; /* tables x [vocab, width] */
    orc_layer *layer;
    orc_qweight *head;       /* tables x [vocab, width] */
    const float *const *head_bias;
} orc_model;

/* The caller passes flat arrays of pointers, one entry per layer, in the field
 * order of decoder_layer_resolved (src/graph.c:2795-2811) plus the two
 * cross-memory tensors decoder_cache_init reads (src/graph.c:3002-3016). */
orc_model *orc_model_new(size_t layers, size_t width, size_t heads, size_t xattn_width,
                         int qtype, const float *position, const float *norm_out,
                         const float *const *norm_self, const float *const *norm_xattn_query,
                         const float *const *norm_xattn_memory, const float *const *norm_pos_ff,
                         const float *const *qkv_w, const float *const *o_self_w,
                         const float *const *q_cross_w, const float *const *kv_cross_w,
                         const float *const *o_cross_w, const float *const *ffn_up_w,
                         const float *const *ffn_down_w,
                         size_t tables, size_t vocab, size_t codebook_size, size_t eos_id,
                         const float *const *embeddings, const float *const *head_w,
                         const float *const *head_b) {
    orc_model *m = (orc_model *)calloc(1, sizeof(*m));
    if (m == NULL) return NULL;
    m->layers = layers;
    m->width = width;
    m->heads = heads;
    m->head_width = width / heads;
    m->ffn_width = width * 4u;                      /* src/graph.c:2973 */
    m->xattn_width = xattn_width;
    m->qtype = qtype;
    m->position = position;
    m->norm_out = norm_out;
    m->tables = tables;
    m->vocab = vocab;
    m->codebook_size = codebook_size;
    m->eos_id = eos_id;
    m->embeddings = embeddings;
    m->head_bias = head_b;
    m->layer = (orc_layer *)calloc(layers, sizeof(orc_layer));
    m->head = (orc_qweight *)calloc(tables ? tables : 1u, sizeof(orc_qweight));
    if (m->layer == NULL || m->head == NULL) return NULL;
    const size_t w = width, f = m->ffn_width, xw = xattn_width;
    for (size_t l = 0; l < layers; ++l) {
        orc_layer *L = &m->layer[l];
        L->norm_self = norm_self[l];
        L->norm_xattn_query = norm_xattn_query[l];
        L->norm_xattn_memory = norm_xattn_memory[l];
        L->norm_pos_ff = norm_pos_ff[l];
        L->kv_cross_w = kv_cross_w[l];
        if (orc_qweight_init(&L->qkv, qtype, qkv_w[l], 3u * w, w) != 0 ||
            orc_qweight_init(&L->o_self, qtype, o_self_w[l], w, w) != 0 ||
            orc_qweight_init(&L->q_cross, qtype, q_cross_w[l], xw, w) != 0 ||
            orc_qweight_init(&L->o_cross, qtype, o_cross_w[l], w, xw) != 0 ||
            orc_qweight_init(&L->ffn_up, qtype, ffn_up_w[l], f, w) != 0 ||
            orc_qweight_init(&L->ffn_down, qtype, ffn_down_w[l], w, f) != 0)
            return NULL;
    }
    for (size_t t = 0; t < tables; ++t)
        if (head_w != NULL && orc_qweight_init(&m->head[t], qtype, head_w[t], vocab, w) != 0)
            return NULL;
    return m;
}

void orc_model_free(orc_model *m) {
    if (m == NULL) return;
    for (size_t l = 0; l < m->layers; ++l) {
        orc_layer *L = &m->layer[l];
        orc_qweight_free(&L->qkv);
        orc_qweight_free(&L->o_self);
        orc_qweight_free(&L->q_cross);
        orc_qweight_free(&L->o_cross);
        orc_qweight_free(&L->ffn_up);
        orc_qweight_free(&L->ffn_down);
    }
    for (size_t t = 0; t < m->tables; ++t) orc_qweight_free(&m->head[t]);
    free(m->layer);
    free(m->head);
    free(m);
}

/* One request's decoder state: the KV layout of src/graph.c:2813-2826. */
typedef struct {
    const orc_model *m;
    size_t memory_length, capacity, length, layers_run;
    float *self_k, *self_v;   /* [layers][capacity][width] */
    float *cross_k, *cross_v; /* [layers][memory_length][xattn_width] */
    float *x, *nrm, *qkv, *attn, *proj, *q_x, *xctx, *hidden, *scores;
} orc_stream;

void orc_stream_free(orc_stream *s) {
    if (s == NULL) return;
    free(s->self_k); free(s->self_v); free(s->cross_k); free(s->cross_v);
    free(s->x); free(s->nrm); free(s->qkv); free(s->attn); free(s->proj);
    free(s->q_x); free(s->xctx); free(s->hidden); free(s->scores);
    free(s);
}

/* src/graph.c:2963-3030: cross K/V = LN_memory(memory) @ kv_net^T, K in the
 * first xw columns, V in the next xw; f32 product (the prefill is never
 * quantized for more than 16 rows, and this restatement keeps it f32 for any
 * row count, which equals the reference whenever memory_length > 16 or the
 * cache is f32).  Self KV starts empty. */
orc_stream *orc_stream_new(const orc_model *m, const float *memory, size_t memory_length,
                           size_t capacity) {
    orc_stream *s = (orc_stream *)calloc(1, sizeof(*s));
    if (s == NULL) return NULL;
    const size_t w = m->width, xw = m->xattn_width;
    s->m = m;
    s->memory_length = memory_length;
    s->capacity = capacity;
    s->layers_run = m->layers;
    s->self_k = (float *)calloc(m->layers * capacity * w, sizeof(float));
    s->self_v = (float *)calloc(m->layers * capacity * w, sizeof(float));
    s->cross_k = (float *)calloc(m->layers * memory_length * xw, sizeof(float));
    s->cross_v = (float *)calloc(m->layers * memory_length * xw, sizeof(float));
    s->x = (float *)calloc(w, sizeof(float));
    s->nrm = (float *)calloc(w, sizeof(float));
    s->qkv = (float *)calloc(3u * w, sizeof(float));
    s->attn = (float *)calloc(w, sizeof(float));
    s->proj = (float *)calloc(w, sizeof(float));
    s->q_x = (float *)calloc(xw, sizeof(float));
    s->xctx = (float *)calloc(xw, sizeof(float));
    s->hidden = (float *)calloc(m->ffn_width, sizeof(float));
    s->scores = (float *)calloc(capacity > memory_length ? capacity : memory_length, sizeof(float));
    float *mem_norm = (float *)calloc(memory_length * w, sizeof(float));
    float *kv = (float *)calloc(2u * xw, sizeof(float));
    if (!s->self_k || !s->self_v || !s->cross_k || !s->cross_v || !s->x || !s->nrm ||
        !s->qkv || !s->attn || !s->proj || !s->q_x || !s->xctx || !s->hidden ||
        !s->scores || !mem_norm || !kv) {
        free(mem_norm); free(kv); orc_stream_free(s);
        return NULL;
    }
    for (size_t l = 0; l < m->layers; ++l) {
        const orc_layer *L = &m->layer[l];
        orc_layernorm(memory, L->norm_xattn_memory, NULL, mem_norm, memory_length, w, 1.0e-5f);
        float *ck = s->cross_k + l * memory_length * xw;
        float *cv = s->cross_v + l * memory_length * xw;
        for (size_t t = 0; t < memory_length; ++t) {
            for (size_t r = 0; r < 2u * xw; ++r)
                kv[r] = orc_dot_f32(L->kv_cross_w + r * w, mem_norm + t * w, w);
            memcpy(ck + t * xw, kv, xw * sizeof(float));
            memcpy(cv + t * xw, kv + xw, xw * sizeof(float));
        }
    }
    free(mem_norm);
    free(kv);
    return s;
}

float *orc_stream_self_k(orc_stream *s) { return s->self_k; }
float *orc_stream_self_v(orc_stream *s) { return s->self_v; }
float *orc_stream_cross_k(orc_stream *s) { return s->cross_k; }
float *orc_stream_cross_v(orc_stream *s) { return s->cross_v; }
size_t orc_stream_length(const orc_stream *s) { return s->length; }
void orc_stream_set_length(orc_stream *s, size_t n) { s->length = n; }
/* Run only the first `n` layers (then the output norm): gives per-layer hidden
 * states for the parity ladder without touching the arithmetic. */
void orc_stream_set_layers(orc_stream *s, size_t n) { s->layers_run = n; }

/* src/graph.c:3127-3284 for one slot.  The reference's batched form runs the
 * same arithmetic per (weight row, activation) pair and asserts bit-equality
 * with the single-slot form (src/qmat.c:1107-1179), so a batch is a loop. */
int orc_decoder_step(orc_stream *s, const float *input, float *out) {
    const orc_model *m = s->m;
    const size_t w = m->width, heads = m->heads, hw = m->head_width;
    const size_t ffn = m->ffn_width, xw = m->xattn_width;
    if (s->length >= s->capacity) return -1;
    const float self_scale = 1.0f / sqrtf((float)hw);
    const float cross_scale = 1.0f / sqrtf((float)xw);
    const float *pe = m->position + s->length * w;
    for (size_t d = 0; d < w; ++d) s->x[d] = input[d] + pe[d];
    for (size_t l = 0; l < s->layers_run; ++l) {
        const orc_layer *L = &m->layer[l];
        orc_layernorm(s->x, L->norm_self, NULL, s->nrm, 1u, w, 1.0e-5f);
        orc_linear_row(&L->qkv, s->nrm, s->qkv, NULL);
        orc_self_attention(s->qkv, s->self_k + l * s->capacity * w,
                           s->self_v + l * s->capacity * w, s->length, w, s->length + 1u,
                           heads, hw, self_scale, s->attn, s->scores);
        orc_linear_row(&L->o_self, s->attn, s->proj, NULL);
        for (size_t d = 0; d < w; ++d) s->x[d] += s->proj[d];
        orc_layernorm(s->x, L->norm_xattn_query, NULL, s->nrm, 1u, w, 1.0e-5f);
        orc_linear_row(&L->q_cross, s->nrm, s->q_x, NULL);
        orc_cross_attention(s->q_x, s->cross_k + l * s->memory_length * xw,
                            s->cross_v + l * s->memory_length * xw, s->memory_length, xw,
                            1u, xw, cross_scale, s->xctx, s->scores);
        orc_linear_row(&L->o_cross, s->xctx, s->proj, NULL);
        for (size_t d = 0; d < w; ++d) s->x[d] += s->proj[d];
        orc_layernorm(s->x, L->norm_pos_ff, NULL, s->nrm, 1u, w, 1.0e-5f);
        orc_linear_row(&L->ffn_up, s->nrm, s->hidden, NULL);
        orc_gelu_scalar(s->hidden, ffn);
        orc_linear_row(&L->ffn_down, s->hidden, s->proj, NULL);
        for (size_t d = 0; d < w; ++d) s->x[d] += s->proj[d];
    }
    orc_layernorm(s->x, m->norm_out, NULL, out, 1u, w, 1.0e-5f);
    s->length += 1u;
    return 0;
}

/* decoder_run with count > 1, the multi-row prefill: src/graph.c:3286-3654 in the
 * reference's scalar build (scalar sgemm src/backend.c:343-354, scalar GELU
 * src/kernels.c:374-380).  Products of more than 16 rows use the f32 weights whatever the
 * cache's format (src/qmat.c:773-788: quantized only for count <= 16), at most 16 rows go
 * row by row through the packed weights.  Self attention per head: scores = scale * (q . k)
 * over ALL cached and new rows (src/graph.c:3532-3534), softmax_row_inplace over the first
 * start + i + 1 of them (values *= 1 / total, src/graph.c:245-257), zeros behind, then the
 * weighted sum over all rows in order (src/graph.c:3541).  Cross attention is the decode
 * step's loop (src/graph.c:3593-3611).  out_last receives the output norm of the last row. */
int orc_decoder_prefill(orc_stream *s, const float *rows, size_t count, float *out_last) {
    const orc_model *m = s->m;
    const size_t w = m->width, heads = m->heads, hw = m->head_width;
    const size_t ffn = m->ffn_width, xw = m->xattn_width, start = s->length;
    if (count == 0 || start + count > s->capacity) return -1;
    const size_t total_kv = start + count;
    const int packed = count <= 16u;
    float *x = (float *)malloc(count * w * sizeof(float));
    float *nrm = (float *)malloc(count * w * sizeof(float));
    float *qkv = (float *)malloc(count * 3u * w * sizeof(float));
    float *attn = (float *)malloc(count * w * sizeof(float));
    float *proj = (float *)malloc(count * w * sizeof(float));
    float *q_x = (float *)malloc(count * xw * sizeof(float));
    float *xctx = (float *)malloc(count * xw * sizeof(float));
    float *hidden = (float *)malloc(count * ffn * sizeof(float));
    float *score = (float *)malloc((total_kv > s->memory_length ? total_kv : s->memory_length) * sizeof(float));
    if (!x || !nrm || !qkv || !attn || !proj || !q_x || !xctx || !hidden || !score) {
        free(x); free(nrm); free(qkv); free(attn); free(proj); free(q_x); free(xctx); free(hidden); free(score);
        return -1;
    }
    const float self_scale = 1.0f / sqrtf((float)hw);
    const float cross_scale = 1.0f / sqrtf((float)xw);
    for (size_t i = 0; i < count; ++i) {
        const float *pe = m->position + (start + i) * w;
        for (size_t d = 0; d < w; ++d) x[i * w + d] = rows[i * w + d] + pe[d];
    }
/* rows through one weight: packed row by row, or the f32 product (src/backend.c:283-291) */
#define ORC_LINEAR(W_, in_, iw_, out_, ow_)                                                     \
    for (size_t i_ = 0; i_ < count; ++i_) {                                                     \
        if (packed) orc_linear_row(&(W_), (in_) + i_ * (iw_), (out_) + i_ * (ow_), NULL);       \
        else for (size_t r_ = 0; r_ < (ow_); ++r_)                                               \
            (out_)[i_ * (ow_) + r_] = orc_dot_f32((W_).w + r_ * (iw_), (in_) + i_ * (iw_), (iw_)); \
    }
    for (size_t l = 0; l < s->layers_run; ++l) {
        const orc_layer *L = &m->layer[l];
        orc_layernorm(x, L->norm_self, NULL, nrm, count, w, 1.0e-5f);
        ORC_LINEAR(L->qkv, nrm, w, qkv, 3u * w);
        float *kbase = s->self_k + l * s->capacity * w;
        float *vbase = s->self_v + l * s->capacity * w;
        for (size_t i = 0; i < count; ++i) {
            memcpy(kbase + (start + i) * w, qkv + i * 3u * w + w, w * sizeof(float));
            memcpy(vbase + (start + i) * w, qkv + i * 3u * w + 2u * w, w * sizeof(float));
        }
        for (size_t h = 0; h < heads; ++h) {
            for (size_t i = 0; i < count; ++i) {
                const float *qh = qkv + i * 3u * w + h * hw;
                const size_t valid = start + i + 1u;
                /* one row of the score matrix: alpha * sum (+ 0 * c, which changes nothing) */
                for (size_t sidx = 0; sidx < total_kv; ++sidx) {
                    const float *k = kbase + sidx * w + h * hw;
                    float sum = 0.0f;
                    for (size_t d = 0; d < hw; ++d) sum += qh[d] * k[d];
                    score[sidx] = self_scale * sum;
                }
                float maximum = -FLT_MAX;
                for (size_t sidx = 0; sidx < valid; ++sidx)
                    if (score[sidx] > maximum) maximum = score[sidx];
                float total = 0.0f;
                for (size_t sidx = 0; sidx < valid; ++sidx) {
                    score[sidx] = expf(score[sidx] - maximum);
                    total += score[sidx];
                }
                const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
                for (size_t sidx = 0; sidx < valid; ++sidx) score[sidx] *= inverse;
                for (size_t sidx = valid; sidx < total_kv; ++sidx) score[sidx] = 0.0f;
                for (size_t d = 0; d < hw; ++d) {
                    float sum = 0.0f;
                    for (size_t sidx = 0; sidx < total_kv; ++sidx) sum += score[sidx] * vbase[sidx * w + h * hw + d];
                    attn[i * w + h * hw + d] = 1.0f * sum;
                }
            }
        }
        ORC_LINEAR(L->o_self, attn, w, proj, w);
        for (size_t k = 0; k < count * w; ++k) x[k] += proj[k];
        orc_layernorm(x, L->norm_xattn_query, NULL, nrm, count, w, 1.0e-5f);
        ORC_LINEAR(L->q_cross, nrm, w, q_x, xw);
        for (size_t i = 0; i < count; ++i)
            orc_cross_attention(q_x + i * xw, s->cross_k + l * s->memory_length * xw,
                                s->cross_v + l * s->memory_length * xw, s->memory_length, xw, 1u, xw,
                                cross_scale, xctx + i * xw, score);
        ORC_LINEAR(L->o_cross, xctx, xw, proj, w);
        for (size_t k = 0; k < count * w; ++k) x[k] += proj[k];
        orc_layernorm(x, L->norm_pos_ff, NULL, nrm, count, w, 1.0e-5f);
        ORC_LINEAR(L->ffn_up, nrm, w, hidden, ffn);
        orc_gelu_scalar(hidden, count * ffn);
        ORC_LINEAR(L->ffn_down, hidden, ffn, proj, w);
        for (size_t k = 0; k < count * w; ++k) x[k] += proj[k];
    }
#undef ORC_LINEAR
    orc_layernorm(x + (count - 1u) * w, m->norm_out, NULL, out_last, 1u, w, 1.0e-5f);
    s->length += count;
    free(x); free(nrm); free(qkv); free(attn); free(proj); free(q_x); free(xctx); free(hidden); free(score);
    return 0;
}

/* ------------------------------------------------------------ text encoder */
/* encode_text (src/graph.c:709-748): token embedding rows, then transformer_stack over the
 * "encoder" tensors (src/graph.c:634-707) with 12 heads, no cross attention, the output norm
 * applied -- in the reference's scalar build: every `linear` is the f32 product of
 * src/backend.c:283-291 (never quantized: `linear` bypasses qmat, src/graph.c:259-265); the
 * self attention is causal, per head scores = (1/sqrt(hw)) * (q . k) for ALL pairs
 * (src/graph.c:442-444), softmax_row_inplace over the first t + 1 (values *= 1 / total),
 * zeros behind, weighted sum over all rows in order (src/graph.c:450); the feed-forward is
 * the causal convolution of kernel K as ONE product over the unfolded input
 * (unfold_causal, src/graph.c:267-286: col[t][i * K + k] = in[t - (K - 1) + k][i], zero
 * before the start), the scalar tanh GELU, and the same for the output convolution
 * (src/graph.c:333-350).  Per-layer weights are passed as pointer arrays of `layers`
 * entries: norm_self [W], qkv [3W][W], o [W][W], norm_ff [W], proj [F][W*K], out [W][F*K]. */
int orc_encode_text(const int *ids, size_t count, size_t layers, size_t width, size_t heads,
                    size_t kernel, size_t vocab, const float *embedding, const float *position,
                    const float *norm_out, const float *const *norm_self, const float *const *qkv_w,
                    const float *const *o_w, const float *const *norm_ff, const float *const *proj_w,
                    const float *const *out_w, float *out) {
    const size_t w = width, ffn = 4u * width, hw = width / heads;
    float *x = (float *)malloc(count * w * sizeof(float));
    float *nrm = (float *)malloc(count * w * sizeof(float));
    float *qkv = (float *)malloc(count * 3u * w * sizeof(float));
    float *ctx = (float *)malloc(count * w * sizeof(float));
    float *res = (float *)malloc(count * w * sizeof(float));
    float *hidden = (float *)malloc(count * ffn * sizeof(float));
    float *col = (float *)malloc(count * ffn * kernel * sizeof(float));
    float *score = (float *)malloc(count * sizeof(float));
    int rc = -1;
    if (!x || !nrm || !qkv || !ctx || !res || !hidden || !col || !score) goto done;
    for (size_t t = 0; t < count; ++t) {
        if (ids[t] < 0 || (size_t)ids[t] >= vocab) goto done;
        for (size_t d = 0; d < w; ++d) x[t * w + d] = embedding[(size_t)ids[t] * w + d];
    }
    for (size_t t = 0; t < count; ++t)
        for (size_t d = 0; d < w; ++d) x[t * w + d] += position[t * w + d];
    const float scale = 1.0f / sqrtf((float)hw);
    for (size_t l = 0; l < layers; ++l) {
        orc_layernorm(x, norm_self[l], NULL, nrm, count, w, 1.0e-5f);
        for (size_t t = 0; t < count; ++t)
            for (size_t r = 0; r < 3u * w; ++r) qkv[t * 3u * w + r] = orc_dot_f32(qkv_w[l] + r * w, nrm + t * w, w);
        for (size_t h = 0; h < heads; ++h) {
            for (size_t t = 0; t < count; ++t) {
                const float *q = qkv + t * 3u * w + h * hw;
                for (size_t sidx = 0; sidx < count; ++sidx) {
                    const float *k = qkv + sidx * 3u * w + w + h * hw;
                    float sum = 0.0f;
                    for (size_t d = 0; d < hw; ++d) sum += q[d] * k[d];
                    score[sidx] = scale * sum;
                }
                const size_t valid = t + 1u;
                float maximum = -FLT_MAX;
                for (size_t sidx = 0; sidx < valid; ++sidx) if (score[sidx] > maximum) maximum = score[sidx];
                float total = 0.0f;
                for (size_t sidx = 0; sidx < valid; ++sidx) { score[sidx] = expf(score[sidx] - maximum); total += score[sidx]; }
                const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
                for (size_t sidx = 0; sidx < valid; ++sidx) score[sidx] *= inverse;
                for (size_t sidx = valid; sidx < count; ++sidx) score[sidx] = 0.0f;
                for (size_t d = 0; d < hw; ++d) {
                    float sum = 0.0f;
                    for (size_t sidx = 0; sidx < count; ++sidx) sum += score[sidx] * qkv[sidx * 3u * w + 2u * w + h * hw + d];
                    ctx[t * w + h * hw + d] = 1.0f * sum;
                }
            }
        }
        for (size_t t = 0; t < count; ++t)
            for (size_t r = 0; r < w; ++r) res[t * w + r] = orc_dot_f32(o_w[l] + r * w, ctx + t * w, w);
        for (size_t i = 0; i < count * w; ++i) x[i] += res[i];
        orc_layernorm(x, norm_ff[l], NULL, nrm, count, w, 1.0e-5f);
        /* unfold, product, GELU, unfold, product */
        for (size_t t = 0; t < count; ++t)
            for (size_t i = 0; i < w; ++i)
                for (size_t k = 0; k < kernel; ++k) {
                    const long src = (long)t - (long)(kernel - 1u) + (long)k;
                    col[(t * w + i) * kernel + k] = src < 0 ? 0.0f : nrm[(size_t)src * w + i];
                }
        for (size_t t = 0; t < count; ++t)
            for (size_t r = 0; r < ffn; ++r)
                hidden[t * ffn + r] = 1.0f * orc_dot_f32(col + t * w * kernel, proj_w[l] + r * w * kernel, w * kernel);
        orc_gelu_scalar(hidden, count * ffn);
        for (size_t t = 0; t < count; ++t)
            for (size_t i = 0; i < ffn; ++i)
                for (size_t k = 0; k < kernel; ++k) {
                    const long src = (long)t - (long)(kernel - 1u) + (long)k;
                    col[(t * ffn + i) * kernel + k] = src < 0 ? 0.0f : hidden[(size_t)src * ffn + i];
                }
        for (size_t t = 0; t < count; ++t)
            for (size_t r = 0; r < w; ++r)
                res[t * w + r] = 1.0f * orc_dot_f32(col + t * ffn * kernel, out_w[l] + r * ffn * kernel, ffn * kernel);
        for (size_t i = 0; i < count * w; ++i) x[i] += res[i];
    }
    orc_layernorm(x, norm_out, NULL, out, count, w, 1.0e-5f);
    rc = 0;
done:
    free(x); free(nrm); free(qkv); free(ctx); free(res); free(hidden); free(col); free(score);
    return rc;
}

/* src/graph.c:760-804 with the table index flattened: the reference walks
 * stream = fs * codebooks + codebook over stacking * codebooks tables and
 * divides the sum by their count. */
int orc_embed_frame(const orc_model *m, const unsigned *codes, float *row) {
    const size_t w = m->width;
    memset(row, 0, w * sizeof(float));
    for (size_t t = 0; t < m->tables; ++t) {
        if (codes[t] >= m->vocab) return -1;
        const float *e = m->embeddings[t] + (size_t)codes[t] * w;
        for (size_t d = 0; d < w; ++d) row[d] += e[d];
    }
    for (size_t d = 0; d < w; ++d) row[d] /= (float)m->tables;
    return 0;
}

/* Per-table logits through the (quantized) projection with bias, then the
 * masked first-on-ties pick: src/graph.c:1538-1566.  `logits` may be NULL. */
void orc_heads_argmax(const orc_model *m, const float *hidden, int allow_eos,
                      unsigned *tokens, float *logits) {
    float *tmp = logits != NULL ? NULL : (float *)malloc(m->vocab * sizeof(float));
    for (size_t t = 0; t < m->tables; ++t) {
        float *lg = logits != NULL ? logits + t * m->vocab : tmp;
        orc_linear_row(&m->head[t], hidden, lg, m->head_bias[t]);
        tokens[t] = orc_argmax_constrained(lg, m->vocab, m->codebook_size, m->eos_id, allow_eos);
    }
    free(tmp);
}

/* One greedy frame for one request: embed the previous frame's stored codes,
 * step the decoder, pick one token per table.  The stored code collapses
 * non-code picks to 0 (src/graph.c:3900, 1626-1630); the frame reports EOS if
 * any table picked it (src/graph.c:3893-3897).  Returns 1 on EOS, 0 otherwise,
 * -1 on error. */
int orc_greedy_frame(orc_stream *s, unsigned *codes, int allow_eos, unsigned *tokens,
                     float *hidden_out) {
    const orc_model *m = s->m;
    float *row = (float *)malloc(2u * m->width * sizeof(float));
    if (row == NULL) return -1;
    float *hidden = row + m->width;
    int eos = 0;
    if (orc_embed_frame(m, codes, row) != 0 || orc_decoder_step(s, row, hidden) != 0) {
        free(row);
        return -1;
    }
    orc_heads_argmax(m, hidden, allow_eos, tokens, NULL);
    for (size_t t = 0; t < m->tables; ++t) {
        if (tokens[t] == m->eos_id) eos = 1;
        codes[t] = tokens[t] < m->codebook_size ? tokens[t] : 0u;
    }
    if (hidden_out != NULL) memcpy(hidden_out, hidden, m->width * sizeof(float));
    free(row);
    return eos;
}

/* Greedy decode of `frames` frames; tokens_out is [frames][tables].  EOS is
 * allowed from frame `min_frames` on and ends the request; returns the number
 * of frames produced (the EOS frame included). */
long orc_greedy_decode(orc_stream *s, unsigned *codes, size_t frames, size_t min_frames,
                       unsigned *tokens_out) {
    const size_t tables = s->m->tables;
    for (size_t f = 0; f < frames; ++f) {
        const int eos = orc_greedy_frame(s, codes, f >= min_frames, tokens_out + f * tables, NULL);
        if (eos < 0) return -1;
        if (eos) return (long)(f + 1u);
    }
    return (long)frames;
}

/* ---------------------------------------------------- local transformer ----
 * The autoregressive local transformer that turns one decoder output row into
 * the tables of one stacked frame (src/graph.c:806-1656).  It shares the
 * model's embedding tables (audio_embeddings.N) and per-table projections
 * (local_transformer_out_projections.N) with the greedy heads above. */
typedef struct {
    const float *norm_self, *norm_ff;
    orc_qweight qkv, o, ffn_up, ffn_down;
} orc_local_layer;

typedef struct {
    const orc_model *m;
    size_t layers, capacity, length;
    const float *position;          /* local_transformer.position_embeddings.weight */
    orc_local_layer layer[4];       /* at most 4 layers (src/graph.c:1060) */
    float *k, *v;                   /* [layers][capacity][width] */
    float *x, *nrm, *qkv, *attn, *proj, *hidden, *scores, *row_in, *row_out, *logits;
    size_t top_count;
    size_t *top_indices;
    float *top_logits;
} orc_local;

void orc_local_free(orc_local *s) {
    if (s == NULL) return;
    for (size_t l = 0; l < s->layers && l < 4u; ++l) {
        orc_qweight_free(&s->layer[l].qkv);
        orc_qweight_free(&s->layer[l].o);
        orc_qweight_free(&s->layer[l].ffn_up);
        orc_qweight_free(&s->layer[l].ffn_down);
    }
    free(s->k); free(s->v); free(s->x); free(s->nrm); free(s->qkv); free(s->attn);
    free(s->proj); free(s->hidden); free(s->scores); free(s->row_in); free(s->row_out);
    free(s->logits); free(s->top_indices); free(s->top_logits);
    free(s);
}

/* Per-layer pointer arrays in the order local_cache_init resolves them
 * (src/graph.c:1031-1056); capacity is tables + 1 (src/graph.c:1200);
 * top_count > 0 sizes the sampler scratch (src/graph.c:1217-1220). */
orc_local *orc_local_new(const orc_model *m, size_t layers, const float *position,
                         const float *const *norm_self, const float *const *qkv_w,
                         const float *const *o_w, const float *const *norm_ff,
                         const float *const *ffn_up_w, const float *const *ffn_down_w,
                         size_t top_count) {
    if (m == NULL || layers == 0u || layers > 4u) return NULL;
    orc_local *s = (orc_local *)calloc(1, sizeof(*s));
    if (s == NULL) return NULL;
    const size_t w = m->width, f = m->ffn_width;
    s->m = m;
    s->layers = layers;
    s->capacity = m->tables + 1u;
    s->position = position;
    s->top_count = top_count;
    int ok = 1;
    for (size_t l = 0; l < layers; ++l) {
        s->layer[l].norm_self = norm_self[l];
        s->layer[l].norm_ff = norm_ff[l];
        ok = ok && orc_qweight_init(&s->layer[l].qkv, m->qtype, qkv_w[l], 3u * w, w) == 0;
        ok = ok && orc_qweight_init(&s->layer[l].o, m->qtype, o_w[l], w, w) == 0;
        ok = ok && orc_qweight_init(&s->layer[l].ffn_up, m->qtype, ffn_up_w[l], f, w) == 0;
        ok = ok && orc_qweight_init(&s->layer[l].ffn_down, m->qtype, ffn_down_w[l], w, f) == 0;
    }
    s->k = (float *)calloc(layers * s->capacity * w, sizeof(float));
    s->v = (float *)calloc(layers * s->capacity * w, sizeof(float));
    s->x = (float *)calloc(w, sizeof(float));
    s->nrm = (float *)calloc(w, sizeof(float));
    s->qkv = (float *)calloc(3u * w, sizeof(float));
    s->attn = (float *)calloc(w, sizeof(float));
    s->proj = (float *)calloc(w, sizeof(float));
    s->hidden = (float *)calloc(f, sizeof(float));
    s->scores = (float *)calloc(s->capacity, sizeof(float));
    s->row_in = (float *)calloc(w, sizeof(float));
    s->row_out = (float *)calloc(w, sizeof(float));
    s->logits = (float *)calloc(m->vocab, sizeof(float));
    if (top_count > 0u) {
        s->top_indices = (size_t *)calloc(top_count, sizeof(size_t));
        s->top_logits = (float *)calloc(top_count, sizeof(float));
    }
    if (!ok || !s->k || !s->v || !s->x || !s->nrm || !s->qkv || !s->attn || !s->proj ||
        !s->hidden || !s->scores || !s->row_in || !s->row_out || !s->logits ||
        (top_count > 0u && (!s->top_indices || !s->top_logits))) {
        orc_local_free(s);
        return NULL;
    }
    return s;
}

size_t orc_local_length(const orc_local *s) { return s->length; }
void orc_local_set_length(orc_local *s, size_t n) { s->length = n; }
float *orc_local_k(orc_local *s) { return s->k; }
float *orc_local_v(orc_local *s) { return s->v; }

/* src/graph.c:1234-1343 for one slot: position row added, then per layer
 * norm -> qkv -> attention over the rows written so far -> o -> residual ->
 * norm -> up -> GELU -> down -> residual.  No cross attention, no output norm. */
int orc_local_step(orc_local *s, const float *input, float *out) {
    const orc_model *m = s->m;
    const size_t w = m->width, heads = m->heads, hw = m->head_width, ffn = m->ffn_width;
    if (s->length >= s->capacity) return -1;
    const float scale = 1.0f / sqrtf((float)hw);
    const float *pe = s->position + s->length * w;
    for (size_t d = 0; d < w; ++d) s->x[d] = input[d] + pe[d];
    for (size_t l = 0; l < s->layers; ++l) {
        const orc_local_layer *L = &s->layer[l];
        orc_layernorm(s->x, L->norm_self, NULL, s->nrm, 1u, w, 1.0e-5f);
        orc_linear_row(&L->qkv, s->nrm, s->qkv, NULL);
        orc_self_attention(s->qkv, s->k + l * s->capacity * w, s->v + l * s->capacity * w,
                           s->length, w, s->length + 1u, heads, hw, scale, s->attn, s->scores);
        orc_linear_row(&L->o, s->attn, s->proj, NULL);
        for (size_t d = 0; d < w; ++d) s->x[d] += s->proj[d];
        orc_layernorm(s->x, L->norm_ff, NULL, s->nrm, 1u, w, 1.0e-5f);
        orc_linear_row(&L->ffn_up, s->nrm, s->hidden, NULL);
        orc_gelu_scalar(s->hidden, ffn);
        orc_linear_row(&L->ffn_down, s->hidden, s->proj, NULL);
        for (size_t d = 0; d < w; ++d) s->x[d] += s->proj[d];
    }
    memcpy(out, s->x, w * sizeof(float));
    s->length += 1u;
    return 0;
}

/* xorshift64 step of the sampler (src/graph.c:1606-1610). */
uint64_t orc_xorshift64(uint64_t state) {
    state ^= state << 13;
    state ^= state >> 7;
    state ^= state << 17;
    return state == 0 ? UINT64_C(0x9e3779b97f4a7c15) : state;
}

/* One stacked frame for one request: src/graph.c:1374-1656.  decoder_last is
 * the decoder's output row; table t's token comes from position t of the
 * local transformer, whose input is the decoder row (t = 0) or the embedding
 * of the previous table's token.  Disallowed candidates are masked to -FLT_MAX
 * in place, the greedy pick is first-on-ties, and when temperature > 0 and
 * topk > 1 a token is drawn from the top-k (insertion order: higher logit
 * first, earlier index first among equals) with weights exp((l - max) / T).
 * codes[t] gets the stored code (specials collapsed to 0), values[t]
 * (optional) the token that was fed back.  EOS is seen when the greedy or the
 * drawn token is EOS; *eos_frame is the smallest t / codebooks where that
 * happened (SIZE_MAX as -1).  Returns 1 if EOS was seen, 0 if not, -1 on error. */
int orc_local_frame(orc_local *s, const float *decoder_last, float temperature, unsigned topk,
                    uint64_t *rng_state, int allow_eos, size_t codebooks, unsigned *codes,
                    unsigned *values, long *eos_frame) {
    const orc_model *m = s->m;
    const size_t w = m->width, vocab = m->vocab;
    const int sampling = temperature > 0.0f && topk > 1u && rng_state != NULL;
    const size_t top_count = topk < vocab ? topk : vocab;
    if (sampling && top_count > s->top_count) return -1;
    if (codebooks == 0u) return -1;
    int saw_eos = 0;
    long first = -1;
    s->length = 0u;
    memcpy(s->row_in, decoder_last, w * sizeof(float));
    for (size_t t = 0; t < m->tables; ++t) {
        if (orc_local_step(s, s->row_in, s->row_out) != 0) return -1;
        float *logits = s->logits;
        orc_linear_row(&m->head[t], s->row_out, logits, m->head_bias[t]);
        float best = -FLT_MAX;
        unsigned argmax = 0;
        for (size_t c = 0; c < vocab; ++c) {
            const int is_code = c < m->codebook_size;
            const int is_eos = c == m->eos_id;
            if (!is_code && !(is_eos && allow_eos)) {
                logits[c] = -FLT_MAX;
                continue;
            }
            if (logits[c] > best) {
                best = logits[c];
                argmax = (unsigned)c;
            }
        }
        unsigned value = argmax;
        int stream_eos = argmax == m->eos_id;
        if (sampling) {
            size_t used = 0;
            for (size_t c = 0; c < vocab; ++c) {
                size_t insert = used;
                while (insert > 0 && logits[c] > s->top_logits[insert - 1u]) --insert;
                if (used < top_count) {
                    for (size_t q = used; q > insert; --q) {
                        s->top_indices[q] = s->top_indices[q - 1u];
                        s->top_logits[q] = s->top_logits[q - 1u];
                    }
                    s->top_indices[insert] = c;
                    s->top_logits[insert] = logits[c];
                    ++used;
                } else if (insert < top_count) {
                    for (size_t q = top_count - 1u; q > insert; --q) {
                        s->top_indices[q] = s->top_indices[q - 1u];
                        s->top_logits[q] = s->top_logits[q - 1u];
                    }
                    s->top_indices[insert] = c;
                    s->top_logits[insert] = logits[c];
                }
            }
            const float maximum = s->top_logits[0];
            float total = 0.0f;
            for (size_t q = 0; q < used; ++q) {
                s->top_logits[q] = expf((s->top_logits[q] - maximum) / temperature);
                total += s->top_logits[q];
            }
            *rng_state = orc_xorshift64(*rng_state);
            const float draw = ((float)((*rng_state >> 40) & UINT64_C(0xffffff)) /
                                (float)UINT64_C(0x1000000)) * total;
            float cumulative = 0.0f;
            for (size_t q = 0; q < used; ++q) {
                cumulative += s->top_logits[q];
                if (draw <= cumulative || q + 1u == used) {
                    value = (unsigned)s->top_indices[q];
                    break;
                }
            }
        }
        if (value == m->eos_id) stream_eos = 1;
        if (stream_eos) {
            saw_eos = 1;
            const long frame = (long)(t / codebooks);
            if (first < 0 || frame < first) first = frame;
        }
        const unsigned emit = value < vocab ? value : 0u;
        codes[t] = value < m->codebook_size ? value : 0u;
        if (values != NULL) values[t] = value;
        memcpy(s->row_in, m->embeddings[t] + (size_t)emit * w, w * sizeof(float));
    }
    if (eos_frame != NULL) *eos_frame = first;
    return saw_eos;
}

/* ------------------------------------------------------------------ NanoCodec decoder
 * decode_codec in the reference's scalar build (src/graph.c:2640-2780): FSQ de-index of the
 * 8 codebook indices into 32 latent channels (levels 8,7,6,6 per group), a causal
 * convolution 32 -> base (kernel 7), five stages of { half-Snake, grouped causal transposed
 * convolution (kernel 2r, stride r, two input channels per output channel), residual layer },
 * half-Snake, a causal convolution to one channel (kernel 3), clip to [-1, 1].  Activations
 * are [channels][length], time contiguous.  base is 864 in the reference (hard-coded); it is
 * a parameter here so small shapes can be checked too. */
typedef struct {
    const float *in_alpha, *in_w, *in_b, *skip_alpha, *skip_w, *skip_b;
} orc_codec_block;
typedef struct {
    const float *alpha, *up_w, *up_b;
    orc_codec_block block[3][3];      /* [kernel 3,7,11][dilation 1,3,5] */
} orc_codec_stage;
typedef struct {
    size_t base;                      /* channels after the first convolution */
    const float *pre_w, *pre_b;       /* [base][32][7], [base] */
    orc_codec_stage stage[5];
    const float *post_alpha, *post_w, *post_b;   /* [base/32], [1][base/32][3], [1] */
} orc_codec;

/* conv1d_causal without BLAS (src/graph.c:2059-2096): the output is seeded with the bias,
 * the input is unfolded into columns[(i * kernel + k)][t] = in[i][t - (kernel-1-k) * dilation]
 * (zero before the start) and one scalar sgemm with beta = 1 adds the product: per output
 * c = 1.0f * sum + 1.0f * c with sum over p = i * kernel + k in order (src/backend.c:343-354). */
static void orc_conv1d_causal(const float *w, const float *b, const float *in, float *out, size_t ic,
                              size_t oc, size_t length, size_t kernel, size_t dilation) {
    for (size_t o = 0; o < oc; ++o)
        for (size_t t = 0; t < length; ++t) {
            float sum = 0.0f;
            for (size_t i = 0; i < ic; ++i)
                for (size_t k = 0; k < kernel; ++k) {
                    const size_t shift = (kernel - 1u - k) * dilation;
                    const float x = t >= shift ? in[i * length + (t - shift)] : 0.0f;
                    sum += w[(o * ic + i) * kernel + k] * x;
                }
            out[o * length + t] = 1.0f * sum + 1.0f * b[o];
        }
}

/* conv_transpose_causal / convt_channel (src/graph.c:2179-2231) with groups = out channels. */
static void orc_conv_transpose(const float *w, const float *b, const float *in, float *out, size_t ic,
                               size_t oc, size_t length, size_t kernel, size_t stride) {
    const size_t out_len = (length - 1u) * stride + kernel - (kernel - stride);
    const size_t ipg = ic / oc;
    for (size_t o = 0; o < oc; ++o) {
        float *row = out + o * out_len;
        for (size_t t = 0; t < out_len; ++t) row[t] = b[o];
        for (size_t i = o * ipg; i < (o + 1u) * ipg; ++i)
            for (size_t t = 0; t < length; ++t) {
                const float v = in[i * length + t];
                for (size_t k = 0; k < kernel; ++k) {
                    const size_t pos = t * stride + k;
                    if (pos < out_len) row[pos] += v * w[i * kernel + k];
                }
            }
    }
}

/* Snake on the first half of the channels, leaky ReLU (0.01) on the rest.  half_snake
 * (src/graph.c:2250-2323) hands the signal to mynah_backend_snake_dev whenever a backend
 * exists, and the CPU backend's form is snake_row (src/backend.c:643-658): v + sn * sn *
 * (1 / (a + 1e-9)) -- a product with the reciprocal, not the division of graph.c's own
 * snake_channel, which no CPU synthesis reaches. */
static void orc_half_snake(float *x, const float *alpha, size_t channels, size_t length) {
    const size_t snake = channels / 2u;
    for (size_t c = 0; c < channels; ++c) {
        float *row = x + c * length;
        if (c < snake) {
            const float a = alpha[c];
            const float inv_a = 1.0f / (a + 1e-9f);
            for (size_t t = 0; t < length; ++t) {
                const float v = row[t];
                const float sn = sinf(a * v);
                row[t] = v + sn * sn * inv_a;
            }
        } else {
            for (size_t t = 0; t < length; ++t)
                if (row[t] < 0.0f) row[t] *= 0.01f;
        }
    }
}

/* res_layer (src/graph.c:2325-2421). */
static int orc_res_layer(const orc_codec_stage *s, const float *in, float *out, size_t channels, size_t length) {
    static const size_t kernels[3] = {3u, 7u, 11u}, dilations[3] = {1u, 3u, 5u};
    const size_t n = channels * length;
    float *branch = (float *)malloc(n * sizeof(float)), *cur = (float *)malloc(n * sizeof(float));
    float *act = (float *)malloc(n * sizeof(float)), *res = (float *)malloc(n * sizeof(float));
    if (!branch || !cur || !act || !res) { free(branch); free(cur); free(act); free(res); return -1; }
    memset(out, 0, n * sizeof(float));
    for (size_t bi = 0; bi < 3u; ++bi) {
        memcpy(cur, in, n * sizeof(float));
        for (size_t di = 0; di < 3u; ++di) {
            const orc_codec_block *b = &s->block[bi][di];
            memcpy(act, cur, n * sizeof(float));
            orc_half_snake(act, b->in_alpha, channels, length);
            orc_conv1d_causal(b->in_w, b->in_b, act, res, channels, channels, length, kernels[bi], dilations[di]);
            orc_half_snake(res, b->skip_alpha, channels, length);
            orc_conv1d_causal(b->skip_w, b->skip_b, res, branch, channels, channels, length, kernels[bi], 1u);
            for (size_t i = 0; i < n; ++i) cur[i] += branch[i];
        }
        for (size_t i = 0; i < n; ++i) out[i] += cur[i];
    }
    for (size_t i = 0; i < n; ++i) out[i] /= 3.0f;
    free(branch); free(cur); free(act); free(res);
    return 0;
}

/* codes [8][raw_length] -> samples [raw_length * 1024].  Returns the sample count or -1.
 * stop_after: 0 = whole codec; 1 = only the first convolution (out = [base][raw_length]);
 * 2 + s = through stage s (out = [base >> (s+1)][length of that stage]) -- for stage-wise
 * comparisons. */
long orc_codec_decode(const orc_codec *c, const unsigned *codes, size_t raw_length, int stop_after, float *out) {
    static const size_t levels[4] = {8u, 7u, 6u, 6u}, bases[4] = {1u, 8u, 56u, 336u}, rates[5] = {8u, 8u, 4u, 2u, 2u};
    if (raw_length == 0u) return -1;
    float *latent = (float *)malloc(32u * raw_length * sizeof(float));
    float *cur = (float *)malloc(c->base * raw_length * sizeof(float));
    if (!latent || !cur) { free(latent); free(cur); return -1; }
    for (size_t t = 0; t < raw_length; ++t)
        for (size_t g = 0; g < 8u; ++g) {
            const unsigned index = codes[g * raw_length + t];
            for (size_t d = 0; d < 4u; ++d) {
                const size_t digit = (index / bases[d]) % levels[d];
                const float den = (float)(levels[d] / 2u);
                latent[(g * 4u + d) * raw_length + t] = ((float)digit - (float)(levels[d] / 2u)) / den;
            }
        }
    orc_conv1d_causal(c->pre_w, c->pre_b, latent, cur, 32u, c->base, raw_length, 7u, 1u);
    free(latent);
    size_t ch = c->base, len = raw_length;
    if (stop_after == 1) { memcpy(out, cur, ch * len * sizeof(float)); free(cur); return (long)(ch * len); }
    for (size_t s = 0; s < 5u; ++s) {
        orc_half_snake(cur, c->stage[s].alpha, ch, len);
        const size_t nch = ch / 2u, nlen = len * rates[s];
        float *up = (float *)malloc(nch * nlen * sizeof(float));
        float *next = (float *)malloc(nch * nlen * sizeof(float));
        if (!up || !next) { free(up); free(next); free(cur); return -1; }
        orc_conv_transpose(c->stage[s].up_w, c->stage[s].up_b, cur, up, ch, nch, len, rates[s] * 2u, rates[s]);
        free(cur);
        if (orc_res_layer(&c->stage[s], up, next, nch, nlen) != 0) { free(up); free(next); return -1; }
        free(up);
        cur = next; ch = nch; len = nlen;
        if (stop_after == 2 + (int)s) { memcpy(out, cur, ch * len * sizeof(float)); free(cur); return (long)(ch * len); }
    }
    orc_half_snake(cur, c->post_alpha, ch, len);
    orc_conv1d_causal(c->post_w, c->post_b, cur, out, ch, 1u, len, 3u, 1u);
    for (size_t i = 0; i < len; ++i) {
        if (out[i] > 1.0f) out[i] = 1.0f;
        if (out[i] < -1.0f) out[i] = -1.0f;
    }
    free(cur);
    return (long)len;
}
