/* The NanoCodec decoder on one B200 (extension of the backend seam), C11.
 *
 * Restates decode_codec of mynah-tts (src/graph.c:2640-2780; the device-resident form the
 * reference keeps for Metal is decode_codec_resident, src/graph.c:2511-2638) as one
 * device-resident pass per request: FSQ de-index -> first convolution -> five stages of
 * { half-Snake, grouped transposed convolution, residual layer } -> half-Snake -> last
 * convolution -> clip.  Every elementwise step that follows a convolution rides in that
 * convolution's epilogue: the Snake in front of the next convolution, the residual add, the
 * sum of the three branches with its division by three, the next stage's activation, the clip.
 * A residual layer is then 21 launches (3 x (Snake + 6 convolutions)) instead of the 57
 * calls of res_layer_device (src/graph.c:2423-2509).  In fast mode the 90 residual-layer
 * convolutions run on the tensor cores (codec_tc.cu) over f16 hi/lo planes that the
 * epilogues write for one another; strict mode keeps the sequential f32 sums of codec.cu.
 *
 * Convolution weights are repacked once at create ([in * kernel][groups of 7 output
 * channels][8]) so that a CTA's tile is a run of 16-byte copies; everything stays f32.
 */
#include "host_common.h"
#include "../../include/mynah_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

enum { CODEC_STAGES = 5, CODEC_BRANCHES = 3, CODEC_BLOCKS = 3, CODEC_LATENT = 32, CODEC_GROUPS = 8 };
static const size_t codec_rates[CODEC_STAGES] = {8u, 8u, 4u, 2u, 2u};
static const size_t codec_kernels[CODEC_BRANCHES] = {3u, 7u, 11u};
static const size_t codec_dilations[CODEC_BLOCKS] = {1u, 3u, 5u};

typedef struct {
    float *w, *bias;          /* packed weights, bias */
    void *w_tc;               /* tensor-core layout (fast mode), or NULL */
    float scale;              /* power of two the tensor-core weights carry */
} dev_conv;

typedef struct {
    float *in_alpha, *skip_alpha;
    dev_conv in_conv, skip_conv;
    float *in_table, *skip_table;   /* tensor-core epilogue constants per output channel */
} dev_block;

typedef struct {
    float *alpha, *up_w, *up_b;
    dev_block block[CODEC_BRANCHES][CODEC_BLOCKS];
} dev_stage;

typedef struct {
    mb_state *st;
    size_t base, max_frames;
    int strict;               /* this codec's arithmetic (the backend's unless the descriptor says otherwise) */
    dev_conv pre, post;
    dev_stage stage[CODEC_STAGES];
    float *post_alpha;
    const uint32_t *sin_tab;
    /* activations */
    unsigned *d_codes;
    float *latent, *a, *up, *cur, *act, *res, *audio;
    int use_tc;               /* fast mode: residual-layer convolutions on the tensor cores */
    void *act_planes, *res_planes;   /* f16 hi/lo planes [2][length][cp] of the widest stage */
    size_t plane_halves;
    unsigned *h_codes;   /* pinned */
    float *h_audio;      /* pinned */
    float *staging;      /* device scratch for weight uploads */
    size_t staging_floats;
} mb_codec;

static int c_malloc(void **p, size_t bytes, char *error, size_t cap) {
    *p = NULL;
    return mb_cuda((int)cudaMalloc(p, bytes ? bytes : 4u), "cudaMalloc(codec)", error, cap);
}

static int c_upload(float **dst, const float *host, size_t n, char *error, size_t cap) {
    if (host == NULL) {
        mb_set_error(error, cap, "codec tensor is missing");
        return -1;
    }
    if (c_malloc((void **)dst, n * sizeof(float), error, cap) != 0) return -1;
    return mb_cuda((int)cudaMemcpy(*dst, host, n * sizeof(float), cudaMemcpyHostToDevice), "upload", error, cap);
}

/* [oc][ic][kernel] host weights -> packed device weights. */
static int c_conv(mb_codec *c, dev_conv *dst, const float *host_w, const float *host_b, size_t oc, size_t ic,
                  size_t kernel, int tensor_core, char *error, size_t cap) {
    if (host_w == NULL || host_b == NULL) {
        mb_set_error(error, cap, "codec tensor is missing");
        return -1;
    }
    const size_t n = oc * ic * kernel;
    if (n > c->staging_floats) {
        cudaFree(c->staging);
        c->staging = NULL;
        c->staging_floats = 0;
        if (c_malloc((void **)&c->staging, n * sizeof(float), error, cap) != 0) return -1;
        c->staging_floats = n;
    }
    if (c_malloc((void **)&dst->w, mb_codec_conv_packed_floats(oc, ic, kernel) * sizeof(float), error, cap) != 0) return -1;
    MB_TRY(cudaMemcpyAsync(c->staging, host_w, n * sizeof(float), cudaMemcpyHostToDevice, c->st->stream), "upload weight");
    MB_TRY(mb_codec_pack_conv_weight(c->staging, dst->w, oc, ic, kernel, c->st->stream), "pack weight");
    c->st->launches += 1u;
    if (c->use_tc && tensor_core) {
        /* a power of two that brings the largest weight just under 2^14: the f16 lo halves
         * of all but the smallest weights are then normal numbers */
        float amax = 0.0f;
        for (size_t i = 0; i < n; ++i) {
            const float v = fabsf(host_w[i]);
            if (v > amax) amax = v;
        }
        int e = 0;
        if (amax > 0.0f) {
            (void)frexpf(amax, &e);          /* amax = f * 2^e, 0.5 <= f < 1 */
            e = 14 - e;
        }
        if (e > 30) e = 30;
        if (e < -30) e = -30;
        dst->scale = ldexpf(1.0f, e);
        if (c_malloc(&dst->w_tc, mb_codec_tc_packed_halves(oc, ic, kernel) * 2u, error, cap) != 0) return -1;
        MB_TRY(mb_codec_tc_pack_weight(c->staging, dst->w_tc, oc, ic, kernel, dst->scale, c->st->stream), "pack weight");
        c->st->launches += 1u;
    }
    MB_TRY(cudaStreamSynchronize(c->st->stream), "cudaStreamSynchronize");    /* host_w may be pageable; staging is reused */
    return c_upload(&dst->bias, host_b, oc, error, cap);
}

void mynah_b200_codec_destroy(void *codec) {
    mb_codec *c = (mb_codec *)codec;
    if (c == NULL) return;
    cudaSetDevice(c->st->device);
    cudaStreamSynchronize(c->st->stream);
    cudaFree(c->pre.w); cudaFree(c->pre.bias); cudaFree(c->post.w); cudaFree(c->post.bias); cudaFree(c->post_alpha);
    for (size_t s = 0; s < CODEC_STAGES; ++s) {
        dev_stage *S = &c->stage[s];
        cudaFree(S->alpha); cudaFree(S->up_w); cudaFree(S->up_b);
        for (size_t b = 0; b < CODEC_BRANCHES; ++b)
            for (size_t d = 0; d < CODEC_BLOCKS; ++d) {
                dev_block *B = &S->block[b][d];
                cudaFree(B->in_alpha); cudaFree(B->skip_alpha); cudaFree(B->in_table); cudaFree(B->skip_table);
                cudaFree(B->in_conv.w); cudaFree(B->in_conv.bias); cudaFree(B->in_conv.w_tc);
                cudaFree(B->skip_conv.w); cudaFree(B->skip_conv.bias); cudaFree(B->skip_conv.w_tc);
            }
    }
    void *dev[] = {c->d_codes, c->latent, c->a, c->up, c->cur, c->act, c->res, c->audio, c->staging, c->act_planes, c->res_planes};
    for (size_t i = 0; i < sizeof(dev) / sizeof(dev[0]); ++i) cudaFree(dev[i]);
    if (c->h_codes != NULL) cudaFreeHost(c->h_codes);
    if (c->h_audio != NULL) cudaFreeHost(c->h_audio);
    free(c);
}

size_t mynah_b200_codec_samples_per_frame(void) {
    size_t n = 1;
    for (size_t s = 0; s < CODEC_STAGES; ++s) n *= codec_rates[s];
    return n;
}

int mynah_b200_codec_create(void *state, const mynah_b200_codec_desc *desc, void **codec, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || desc == NULL || codec == NULL) {
        mb_set_error(error, cap, "invalid codec arguments");
        return -1;
    }
    *codec = NULL;
    if (desc->base == 0 || desc->base % 32u != 0 || desc->max_frames == 0 || desc->max_frames > 4096u) {
        mb_set_error(error, cap, "invalid codec shape");
        return -1;
    }
    MB_TRY(cudaSetDevice(st->device), "cudaSetDevice");
    mb_codec *c = (mb_codec *)calloc(1, sizeof(*c));
    if (c == NULL) {
        mb_set_error(error, cap, "out of memory creating codec");
        return -1;
    }
    c->st = st;
    c->base = desc->base;
    c->max_frames = desc->max_frames;
    if (desc->arithmetic < 0 || desc->arithmetic > 2) {
        free(c);
        mb_set_error(error, cap, "invalid codec arithmetic");
        return -1;
    }
    c->strict = desc->arithmetic == 0 ? st->strict : desc->arithmetic == 1;
    c->sin_tab = c->strict ? mb_libm_sin_table(st) : NULL;
    {
        const char *no_tc = getenv("MYNAH_B200_NO_TC");
        c->use_tc = !c->strict && !(no_tc != NULL && strcmp(no_tc, "0") != 0);
    }
    int ok = 1;
#define C_TRY(expr) do { if (ok && (expr) != 0) ok = 0; } while (0)
    C_TRY(c_conv(c, &c->pre, desc->pre_w, desc->pre_b, c->base, CODEC_LATENT, 7u, 0, error, cap));
    size_t ch = c->base;
    for (size_t s = 0; ok && s < CODEC_STAGES; ++s) {
        const mynah_b200_codec_stage *S = &desc->stage[s];
        dev_stage *D = &c->stage[s];
        const size_t nch = ch / 2u;
        C_TRY(c_upload(&D->alpha, S->alpha, ch, error, cap));
        C_TRY(c_upload(&D->up_w, S->up_w, ch * 2u * codec_rates[s], error, cap));
        C_TRY(c_upload(&D->up_b, S->up_b, nch, error, cap));
        for (size_t b = 0; ok && b < CODEC_BRANCHES; ++b)
            for (size_t d = 0; ok && d < CODEC_BLOCKS; ++d) {
                const mynah_b200_codec_block *B = &S->block[b][d];
                dev_block *DB = &D->block[b][d];
                C_TRY(c_upload(&DB->in_alpha, B->in_alpha, nch, error, cap));
                C_TRY(c_upload(&DB->skip_alpha, B->skip_alpha, nch, error, cap));
                C_TRY(c_conv(c, &DB->in_conv, B->in_w, B->in_b, nch, nch, codec_kernels[b], 1, error, cap));
                C_TRY(c_conv(c, &DB->skip_conv, B->skip_w, B->skip_b, nch, nch, codec_kernels[b], 1, error, cap));
            }
        ch = nch;
    }
    C_TRY(c_upload(&c->post_alpha, desc->post_alpha, ch, error, cap));
    /* epilogue constants of the tensor-core convolutions: the first convolution of a block is
     * followed by the block's skip activation; the second by the next block's input activation,
     * or, as the last of its branch, by the next stage's activation on the finished sum */
    for (size_t s = 0, tch = c->base / 2u; ok && c->use_tc && s < CODEC_STAGES; ++s, tch /= 2u)
        for (size_t b = 0; ok && b < CODEC_BRANCHES; ++b)
            for (size_t d = 0; ok && d < CODEC_BLOCKS; ++d) {
                dev_block *DB = &c->stage[s].block[b][d];
                const float *after = d + 1u < CODEC_BLOCKS ? c->stage[s].block[b][d + 1u].in_alpha : NULL;
                const float *next_stage = s + 1u < CODEC_STAGES ? c->stage[s + 1u].alpha : c->post_alpha;
                C_TRY(c_malloc((void **)&DB->in_table, tch * 4u * sizeof(float), error, cap));
                C_TRY(c_malloc((void **)&DB->skip_table, tch * 4u * sizeof(float), error, cap));
                if (ok) C_TRY(mb_cuda(mb_codec_tc_channel_table(DB->in_conv.bias, DB->skip_alpha, NULL, DB->in_table, tch, st->stream),
                                      "channel table", error, cap));
                if (ok) C_TRY(mb_cuda(mb_codec_tc_channel_table(DB->skip_conv.bias, after, d + 1u < CODEC_BLOCKS ? NULL : next_stage,
                                                                DB->skip_table, tch, st->stream), "channel table", error, cap));
            }
    if (ok && c->use_tc) C_TRY(mb_cuda((int)cudaStreamSynchronize(st->stream), "cudaStreamSynchronize", error, cap));
    C_TRY(c_conv(c, &c->post, desc->post_w, desc->post_b, 1u, ch, 3u, 0, error, cap));
    /* the widest activation: stages 2..4 hold base * 32 floats per frame */
    const size_t T = c->max_frames, act_floats = c->base * 32u * T, samples = mynah_b200_codec_samples_per_frame() * T;
    C_TRY(c_malloc((void **)&c->d_codes, CODEC_GROUPS * T * sizeof(unsigned), error, cap));
    C_TRY(c_malloc((void **)&c->latent, CODEC_LATENT * T * sizeof(float), error, cap));
    C_TRY(c_malloc((void **)&c->a, act_floats * sizeof(float), error, cap));
    C_TRY(c_malloc((void **)&c->up, act_floats * sizeof(float), error, cap));
    C_TRY(c_malloc((void **)&c->cur, act_floats * sizeof(float), error, cap));
    C_TRY(c_malloc((void **)&c->act, act_floats * sizeof(float), error, cap));
    C_TRY(c_malloc((void **)&c->res, act_floats * sizeof(float), error, cap));
    C_TRY(c_malloc((void **)&c->audio, samples * sizeof(float), error, cap));
    if (c->use_tc) {
        /* the widest plane: the last stage, 1024 times per frame x its channels rounded up to 64 */
        size_t widest = 0, pch = c->base, plen = T;
        for (size_t s = 0; s < CODEC_STAGES; ++s) {
            pch /= 2u;
            plen *= codec_rates[s];
            const size_t cp = (pch + 63u) / 64u * 64u;
            if (plen * cp > widest) widest = plen * cp;
        }
        c->plane_halves = widest;
        C_TRY(c_malloc(&c->act_planes, 2u * widest * 2u, error, cap));
        C_TRY(c_malloc(&c->res_planes, 2u * widest * 2u, error, cap));
        if (ok) C_TRY(mb_cuda((int)cudaMemset(c->act_planes, 0, 2u * widest * 2u), "cudaMemset", error, cap));
        if (ok) C_TRY(mb_cuda((int)cudaMemset(c->res_planes, 0, 2u * widest * 2u), "cudaMemset", error, cap));
    }
    C_TRY(mb_cuda((int)cudaMallocHost((void **)&c->h_codes, CODEC_GROUPS * T * sizeof(unsigned)), "cudaMallocHost", error, cap));
    C_TRY(mb_cuda((int)cudaMallocHost((void **)&c->h_audio, samples * sizeof(float)), "cudaMallocHost", error, cap));
#undef C_TRY
    cudaFree(c->staging);
    c->staging = NULL;
    c->staging_floats = 0;
    if (!ok) {
        mynah_b200_codec_destroy(c);
        return -1;
    }
    *codec = c;
    mb_clear_error(error, cap);
    return 0;
}

static void conv_defaults(const mb_codec *c, mb_codec_conv_args *g, const dev_conv *w, const float *in, size_t ic, size_t oc,
                          size_t length, size_t kernel, size_t dilation) {
    memset(g, 0, sizeof(*g));
    g->in = in;
    g->w_packed = w->w;
    g->bias = w->bias;
    g->ic = ic; g->oc = oc; g->length = length; g->kernel = kernel; g->dilation = dilation;
    g->strict = c->strict;
    g->sin_tab = c->sin_tab;
    g->sm_count = c->st->sm_count;
}

/* Enqueues the whole decode of `frames` frames from c->d_codes into c->audio (or, with
 * stop_after != 0, up to that point into c->a); returns the floats the result holds. */
static int codec_enqueue(mb_codec *c, size_t frames, int stop_after, size_t *result_floats, const float **result) {
    mb_state *st = c->st;
    cudaStream_t s = st->stream;
    int rc = 0;
    mb_codec_conv_args g;
#define R_TRY(expr) do { if (rc == 0) { rc = (int)(expr); st->launches += 1u; } } while (0)
    R_TRY(mb_codec_fsq_latent(c->d_codes, c->latent, frames, s));
    /* first convolution; its epilogue applies stage 0's activation */
    conv_defaults(c, &g, &c->pre, c->latent, CODEC_LATENT, c->base, frames, 7u, 1u);
    if (stop_after == 1) {
        g.out = c->a;
    } else {
        g.alpha = c->stage[0].alpha;
        g.out_act = c->a;
    }
    R_TRY(mb_codec_conv1d(&g, s));
    size_t ch = c->base, len = frames;
    *result = c->a;
    *result_floats = ch * len;
    if (stop_after == 1) return rc;
    for (size_t si = 0; si < CODEC_STAGES && rc == 0; ++si) {
        const dev_stage *D = &c->stage[si];
        const size_t nch = ch / 2u, nlen = len * codec_rates[si];
        /* c->a holds half-Snake(previous output) */
        R_TRY(mb_codec_conv_transpose(c->a, D->up_w, D->up_b, c->up, ch, nch, len, codec_rates[si], c->strict, s));
        const int raw_stage_out = stop_after == 2 + (int)si;
        const float *next_alpha = raw_stage_out ? NULL : (si + 1u < CODEC_STAGES ? c->stage[si + 1u].alpha : c->post_alpha);
        for (size_t b = 0; c->use_tc && b < CODEC_BRANCHES && rc == 0; ++b) {
            /* tensor-core form: the activations between convolutions are f16 hi/lo planes */
            const size_t cp = (nch + 63u) / 64u * 64u, pstride = nlen * cp;
            unsigned short *actp = (unsigned short *)c->act_planes, *resp = (unsigned short *)c->res_planes;
            R_TRY(mb_codec_snake_planes(c->up, D->block[b][0].in_alpha, actp, actp + pstride, nch, nlen, s));
            for (size_t d = 0; d < CODEC_BLOCKS && rc == 0; ++d) {
                const dev_block *B = &D->block[b][d];
                mb_codec_conv_tc_args t;
                memset(&t, 0, sizeof(t));
                t.x_planes = actp; t.x_plane_stride = pstride;
                t.w_packed = B->in_conv.w_tc; t.scale = B->in_conv.scale; t.channel_table = B->in_table;
                t.has_alpha = 1; t.act_planes = resp; t.act_plane_stride = pstride;
                t.ic = nch; t.oc = nch; t.length = nlen; t.kernel = codec_kernels[b]; t.dilation = codec_dilations[d];
                t.status = st->d_status; t.sm_count = st->sm_count;
                R_TRY(mb_codec_conv1d_tc(&t, s));
                memset(&t, 0, sizeof(t));
                t.x_planes = resp; t.x_plane_stride = pstride;
                t.w_packed = B->skip_conv.w_tc; t.scale = B->skip_conv.scale; t.channel_table = B->skip_table;
                t.res = d == 0 ? c->up : c->cur;
                t.ic = nch; t.oc = nch; t.length = nlen; t.kernel = codec_kernels[b]; t.dilation = 1u;
                t.status = st->d_status; t.sm_count = st->sm_count;
                if (d + 1u < CODEC_BLOCKS) {
                    t.out = c->cur;
                    t.has_alpha = 1;
                    t.act_planes = actp; t.act_plane_stride = pstride;
                } else {
                    t.acc = c->a;
                    t.acc_mode = b == 0 ? 1 : (b + 1u < CODEC_BRANCHES ? 2 : 3);
                    t.has_alpha2 = next_alpha != NULL;
                }
                R_TRY(mb_codec_conv1d_tc(&t, s));
            }
        }
        for (size_t b = 0; !c->use_tc && b < CODEC_BRANCHES && rc == 0; ++b) {
            R_TRY(mb_codec_half_snake(c->up, c->act, D->block[b][0].in_alpha, nch, nlen, nch / 2u, c->strict, c->sin_tab, s));
            for (size_t d = 0; d < CODEC_BLOCKS && rc == 0; ++d) {
                const dev_block *B = &D->block[b][d];
                /* residual = half-Snake_skip(conv_in(activated)) */
                conv_defaults(c, &g, &B->in_conv, c->act, nch, nch, nlen, codec_kernels[b], codec_dilations[d]);
                g.alpha = B->skip_alpha;
                g.out_act = c->res;
                R_TRY(mb_codec_conv1d(&g, s));
                /* current += conv_skip(residual); the next block's activation, or the branch sum */
                conv_defaults(c, &g, &B->skip_conv, c->res, nch, nch, nlen, codec_kernels[b], 1u);
                g.res = d == 0 ? c->up : c->cur;
                if (d + 1u < CODEC_BLOCKS) {
                    g.out = c->cur;
                    g.alpha = D->block[b][d + 1u].in_alpha;
                    g.out_act = c->act;
                } else {
                    g.acc = c->a;
                    g.acc_mode = b == 0 ? 1 : (b + 1u < CODEC_BRANCHES ? 2 : 3);
                    g.alpha2 = next_alpha;
                }
                R_TRY(mb_codec_conv1d(&g, s));
            }
        }
        ch = nch;
        len = nlen;
        *result_floats = ch * len;
        if (raw_stage_out) return rc;
    }
    /* c->a holds half-Snake_post(last stage) */
    conv_defaults(c, &g, &c->post, c->a, ch, 1u, len, 3u, 1u);
    g.out = c->audio;
    g.clip = 1;
    R_TRY(mb_codec_conv1d(&g, s));
#undef R_TRY
    *result = c->audio;
    *result_floats = len;
    return rc;
}

static int codec_run(mb_codec *c, const unsigned *codes, size_t frames, int stop_after, float *out, size_t out_cap,
                     size_t *count, char *error, size_t cap) {
    if (c == NULL || codes == NULL || out == NULL) {
        mb_set_error(error, cap, "invalid codec buffers");
        return -1;
    }
    if (frames == 0 || frames > c->max_frames) {
        mb_set_error(error, cap, "codec frame count is outside 1..max_frames");
        return -1;
    }
    mb_state *st = c->st;
    MB_TRY(cudaSetDevice(st->device), "cudaSetDevice");
    memcpy(c->h_codes, codes, CODEC_GROUPS * frames * sizeof(unsigned));
    MB_TRY(cudaMemcpyAsync(c->d_codes, c->h_codes, CODEC_GROUPS * frames * sizeof(unsigned), cudaMemcpyHostToDevice, st->stream),
           "stage codes");
    size_t n = 0;
    const float *result = NULL;
    const int rc = codec_enqueue(c, frames, stop_after, &n, &result);
    if (rc != 0) return mb_cuda(rc, "codec decode", error, cap);
    if (n > out_cap) {
        cudaStreamSynchronize(st->stream);
        mb_set_error(error, cap, "codec output buffer is too small");
        return -1;
    }
    if (stop_after == 0) {
        MB_TRY(cudaMemcpyAsync(c->h_audio, result, n * sizeof(float), cudaMemcpyDeviceToHost, st->stream), "read samples");
        MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
        memcpy(out, c->h_audio, n * sizeof(float));
    } else {
        MB_TRY(cudaMemcpyAsync(out, result, n * sizeof(float), cudaMemcpyDeviceToHost, st->stream), "read activations");
        MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    }
    if (c->use_tc) {
        int status = 0;
        MB_TRY(cudaMemcpy(&status, st->d_status, sizeof(int), cudaMemcpyDeviceToHost), "read status");
        if (status != 0) {
            cudaMemset(st->d_status, 0, sizeof(int));
            mb_set_error(error, cap, mb_status_message(status));
            return -1;
        }
    }
    if (count != NULL) *count = n;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_codec_decode(void *codec, const unsigned *codes, size_t frames, float *samples, size_t *sample_count,
                            char *error, size_t cap) {
    mb_codec *c = (mb_codec *)codec;
    return codec_run(c, codes, frames, 0, samples, c == NULL ? 0 : frames * mynah_b200_codec_samples_per_frame(), sample_count,
                     error, cap);
}

int mynah_b200_codec_decode_partial(void *codec, const unsigned *codes, size_t frames, int stop_after, float *out,
                                    size_t out_capacity, size_t *count, char *error, size_t cap) {
    if (stop_after < 0 || stop_after > 1 + CODEC_STAGES) {
        mb_set_error(error, cap, "invalid codec stage");
        return -1;
    }
    return codec_run((mb_codec *)codec, codes, frames, stop_after, out, out_capacity, count, error, cap);
}

/* Device time of one decode of `frames` frames (codes as last staged), averaged over `repeats`. */
int mynah_b200_codec_time(void *codec, const unsigned *codes, size_t frames, int repeats, float *ms_per_decode,
                          char *error, size_t cap) {
    mb_codec *c = (mb_codec *)codec;
    if (c == NULL || codes == NULL || ms_per_decode == NULL || repeats <= 0 || frames == 0 || frames > c->max_frames) {
        mb_set_error(error, cap, "invalid codec timing request");
        return -1;
    }
    mb_state *st = c->st;
    MB_TRY(cudaSetDevice(st->device), "cudaSetDevice");
    MB_TRY(cudaMemcpyAsync(c->d_codes, codes, CODEC_GROUPS * frames * sizeof(unsigned), cudaMemcpyHostToDevice, st->stream),
           "stage codes");
    size_t n = 0;
    const float *result = NULL;
    if (st->timer0 == NULL) {
        MB_TRY(cudaEventCreate(&st->timer0), "cudaEventCreate");
        MB_TRY(cudaEventCreate(&st->timer1), "cudaEventCreate");
    }
    int rc = codec_enqueue(c, frames, 0, &n, &result);      /* warm-up */
    if (rc == 0) rc = (int)cudaEventRecord(st->timer0, st->stream);
    for (int r = 0; r < repeats && rc == 0; ++r) rc = codec_enqueue(c, frames, 0, &n, &result);
    if (rc == 0) rc = (int)cudaEventRecord(st->timer1, st->stream);
    if (rc == 0) rc = (int)cudaEventSynchronize(st->timer1);
    float ms = 0.0f;
    if (rc == 0) rc = (int)cudaEventElapsedTime(&ms, st->timer0, st->timer1);
    if (rc != 0) return mb_cuda(rc, "codec timing", error, cap);
    *ms_per_decode = ms / (float)repeats;
    mb_clear_error(error, cap);
    return 0;
}
