/* Whole-step Magpie decoder on one B200 (extension of the backend seam), C11.
 *
 * Restates decoder_step_batch of mynah-tts (src/graph.c:3127-3284) as one
 * device-resident sequence per step -- position add, per layer LayerNorm ->
 * qkv -> KV append + self-attention -> o -> residual -> LayerNorm -> cross q ->
 * cross-attention -> o -> residual -> LayerNorm -> FFN up + GELU -> FFN down ->
 * residual, then the output norm -- for `batch` independent requests ("slots")
 * that each own a KV cache in the layout of src/graph.c:2823-2826.  The
 * sequence is captured once per batch bucket into a CUDA graph and replayed;
 * positions, slot ids and the live lane count are read from device memory so
 * one graph serves every step.  The greedy front/back ends (embedding mean,
 * logit heads, constrained argmax) follow src/graph.c:760-804 and 1538-1566.
 */
#include "host_common.h"
#include "../../include/mynah_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* STEP: host rows in/out; FRAME: embed + step + logit heads; LOCAL: embed + step + the
 * local transformer's stacked frame; LOCAL_ONLY: the stacked frame alone, from rows in d->out */
enum { MODE_STEP = 0, MODE_FRAME = 1, MODE_LOCAL = 2, MODE_LOCAL_ONLY = 3, MODE_COUNT = 4 };
#define MAX_BUCKETS 12

typedef struct {
    float *norm_self, *norm_xattn_query, *norm_pos_ff;
    mb_dev_weight qkv, o_self, q_cross, o_cross, ffn_up, ffn_down;
    /* optional f32 copies (a quantized decoder that prefills more than 16 rows at once: the
     * reference then multiplies with the f32 weights, src/qmat.c:773-788) */
    mb_dev_weight qkv32, o_self32, q_cross32, o_cross32, ffn_up32, ffn_down32;
    /* fast mode, with the f32 copies: the same weights as f16 hi/lo planes for the tensor-core
     * product of many rows (codec_tc.cu), and the power of two they carry */
    void *tc_w[6];
    float tc_scale[6];
    float *norm_xattn_memory;   /* optional: with kv_cross, lets a slot's cross K/V be made here */
    mb_dev_weight kv_cross;     /* f32 [2*xw, width]; the reference runs it unquantized */
    void *kv_tc;                /* fast mode: the same as f16 hi/lo planes for the tensor-core product */
    float kv_tc_scale;
} dec_layer;

typedef struct {
    float *norm_self, *norm_ff;
    mb_dev_weight qkv, o, ffn_up, ffn_down;
} local_layer;

/* The local transformer of src/graph.c:806-1656: at most 4 layers, no cross attention, a KV
 * of tables + 1 rows per lane that is rewritten every frame (so it belongs to lanes, not to
 * slots), and the per-lane sampler state. */
typedef struct {
    size_t layers, capacity, codebooks;
    local_layer L[4];
    float *position;               /* [position_rows][width] */
    float *k, *v;                  /* [max_batch][layers][capacity][width] */
    float *row_in;                 /* [max_batch][width]: embedding of the previous table's token */
    float *d_temp;                 /* [max_batch] */
    unsigned *d_topk;              /* [max_batch] */
    unsigned long long *d_rng;     /* [max_batch] xorshift64 states */
    int *d_eos_sub;                /* [max_batch] first stacked sub-frame with EOS in this frame */
} mb_local;

typedef struct mb_decoder {
    mb_state *st;
    size_t layers, layers_run, width, heads, hw, ffn, xw, T, capacity, slots, max_batch;
    size_t max_positions, tables, vocab, codebook_size, eos_id;
    dec_layer *L;
    float *position, *norm_out;
    float *emb;                 /* [tables][vocab][width] */
    const float **d_tables;     /* device array of table pointers */
    mb_dev_weight heads_w;      /* [tables*vocab, width] */
    float *heads_b;
    float *self_k, *self_v, *cross_k, *cross_v;
    /* activations, [max_batch][...] */
    float *x, *nrm, *qkv, *attn, *q_x, *xctx, *hidden, *out, *rows_in, *logits;
    int8_t *qx;
    float *sx;
    float *cand_v;              /* f32 heads: candidates of the fused projection + argmax */
    unsigned *cand_i, *cand_counters;
    void *row_planes;           /* prefill on the tensor cores: f16 hi/lo planes of the rows feeding a product */
    void *xsplit;               /* f16 weights: the activations' two f16 planes for the tensor-core product */
    float *partials;
    unsigned *counters;
    int use_tc, use_fuse1, use_xblock;
    int use_split_quant; /* strict: quantize the self-attention rows in a launch of their own (MYNAH_B200_NO_SPLIT_QUANT=1: off) */
    /* lane state */
    int *d_lens, *d_slots, *d_n_active, *d_allow_eos, *d_eos_flag, *d_eos_frame, *d_frame_idx, *d_status;
    int *d_min_frames;
    unsigned *d_codes, *d_tokens, *d_history;
    size_t history_frames;
    /* pinned host staging */
    float *h_rows, *h_out;
    int *h_lens, *h_slots, *h_ints, *h_table;
    unsigned *h_codes, *h_tokens;
    /* One block on each side for everything a per-frame call stages (lane state, codes) and
     * one for everything it reads back (status, tokens): a call is one copy in, one graph,
     * one copy out.  d_slots .. d_codes, d_status, d_tokens and their h_ twins point into them. */
    int *d_stage_in, *h_stage_in, *h_frame_idx;
    unsigned *d_stage_out, *h_stage_out;
    int *h_status;
    size_t stage_in_ints;
    size_t *slot_len;           /* host mirror of every slot's length */
    int *d_mem_len;             /* [slots] text states of the request in each slot (<= T) */
    size_t *slot_mem;           /* host mirror */
    float *pf_mem, *pf_nrm, *pf_kv;   /* prefill scratch: [T][W], [T][W], [T][2xw] */
    void *pf_planes;                  /* fast mode: f16 hi/lo planes of the normalized text states, [2][T][W] */
    mb_local local;             /* layers == 0: not attached */
    cudaGraphExec_t graph[MODE_COUNT][MAX_BUCKETS];
    unsigned graph_launches[MODE_COUNT][MAX_BUCKETS];
    size_t bucket_size[MAX_BUCKETS];
    size_t n_buckets;
    int use_graphs;
    cudaEvent_t ev0, ev1;
    size_t weight_bytes;
    /* per-call-site timing (profile mode: eager launches bracketed by events) */
    int profiling;
    cudaEvent_t *prof_ev;          /* PROF_POOL pairs */
    int *prof_cls;
    size_t prof_used;
    unsigned long long prof_launches[MYNAH_B200_PROFILE_CLASSES];
    double prof_ms[MYNAH_B200_PROFILE_CLASSES];
} mb_decoder;

#define PROF_POOL 4096u
enum { PC_INPUT = 0, PC_NORM, PC_QKV, PC_ATTN_SELF, PC_O_SELF, PC_Q_CROSS, PC_ATTN_CROSS,
       PC_O_CROSS, PC_FFN_UP, PC_QUANT, PC_FFN_DOWN, PC_HEADS, PC_ARGMAX, PC_ADVANCE, PC_LOCAL,
       PC_XBLOCK };
static const char *const prof_names[MYNAH_B200_PROFILE_CLASSES] = {
    "input(embed|position)", "layernorm(+quant)", "qkv product", "self attention", "o_self product",
    "q_cross product", "cross attention", "o_cross product", "ffn_up product(+gelu)",
    "row quantization (attention rows|hidden rows)", "ffn_down product", "heads product", "argmax", "advance",
    "local transformer frame (all tables)",
    "cross block (norm|q product|cross attention|o product|norm)"};

static void prof_drain(mb_decoder *d) {
    if (d->prof_used == 0) return;
    cudaStreamSynchronize(d->st->stream);
    for (size_t i = 0; i < d->prof_used; ++i) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, d->prof_ev[2 * i], d->prof_ev[2 * i + 1]) == cudaSuccess) {
            d->prof_ms[d->prof_cls[i]] += ms;
            d->prof_launches[d->prof_cls[i]] += 1u;
        }
    }
    d->prof_used = 0;
}
static void prof_begin(mb_decoder *d, int cls) {
    if (!d->profiling) return;
    if (d->prof_used == PROF_POOL) prof_drain(d);
    d->prof_cls[d->prof_used] = cls;
    cudaEventRecord(d->prof_ev[2 * d->prof_used], d->st->stream);
}
static void prof_end(mb_decoder *d) {
    if (!d->profiling) return;
    cudaEventRecord(d->prof_ev[2 * d->prof_used + 1], d->st->stream);
    d->prof_used += 1u;
}

static int quantized_mode(const mb_decoder *d) {
    return d->st->quant == MB_INT8 || d->st->quant == MB_INT4;
}

static int dmalloc(void **p, size_t bytes, char *error, size_t cap) {
    *p = NULL;
    return mb_cuda((int)cudaMalloc(p, bytes ? bytes : 4u), "cudaMalloc(decoder)", error, cap);
}

static int upload_vec(float **dst, const float *host, size_t n, char *error, size_t cap) {
    if (dmalloc((void **)dst, n * sizeof(float), error, cap) != 0) return -1;
    return mb_cuda((int)cudaMemcpy(*dst, host, n * sizeof(float), cudaMemcpyHostToDevice),
                   "upload", error, cap);
}

static void destroy_graphs(mb_decoder *d) {
    for (int m = 0; m < MODE_COUNT; ++m)
        for (size_t i = 0; i < MAX_BUCKETS; ++i)
            if (d->graph[m][i] != NULL) {
                cudaGraphExecDestroy(d->graph[m][i]);
                d->graph[m][i] = NULL;
            }
}

/* Tensor-core planes of the f32 weights are worth building: not switched off, and every
 * product's input width is a whole number of 64-column chunks. */
static int prefill_tc_wanted(size_t width, size_t xattn_width) {
    const char *no_tc = getenv("MYNAH_B200_NO_TC");
    if (no_tc != NULL && strcmp(no_tc, "0") != 0) return 0;
    return width % 64u == 0 && xattn_width % 64u == 0;
}

void mynah_b200_decoder_destroy(void *decoder) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d == NULL) return;
    cudaSetDevice(d->st->device);
    cudaStreamSynchronize(d->st->stream);
    destroy_graphs(d);
    if (d->L != NULL) {
        for (size_t l = 0; l < d->layers; ++l) {
            dec_layer *L = &d->L[l];
            cudaFree(L->norm_self); cudaFree(L->norm_xattn_query); cudaFree(L->norm_pos_ff);
            cudaFree(L->norm_xattn_memory); mb_weight_release(&L->kv_cross); cudaFree(L->kv_tc);
            mb_weight_release(&L->qkv); mb_weight_release(&L->o_self);
            mb_weight_release(&L->q_cross); mb_weight_release(&L->o_cross);
            mb_weight_release(&L->ffn_up); mb_weight_release(&L->ffn_down);
            mb_weight_release(&L->qkv32); mb_weight_release(&L->o_self32);
            mb_weight_release(&L->q_cross32); mb_weight_release(&L->o_cross32);
            mb_weight_release(&L->ffn_up32); mb_weight_release(&L->ffn_down32);
            for (int t = 0; t < 6; ++t) cudaFree(L->tc_w[t]);
        }
        free(d->L);
    }
    mb_weight_release(&d->heads_w);
    for (size_t l = 0; l < 4u; ++l) {
        mb_weight_release(&d->local.L[l].qkv); mb_weight_release(&d->local.L[l].o);
        mb_weight_release(&d->local.L[l].ffn_up); mb_weight_release(&d->local.L[l].ffn_down);
        cudaFree(d->local.L[l].norm_self); cudaFree(d->local.L[l].norm_ff);
    }
    {
        void *ldev[] = {d->local.position, d->local.k, d->local.v, d->local.row_in, d->local.d_temp,
                        d->local.d_topk, d->local.d_rng, d->local.d_eos_sub};
        for (size_t i = 0; i < sizeof(ldev) / sizeof(ldev[0]); ++i) cudaFree(ldev[i]);
    }
    void *dev[] = {d->position, d->norm_out, d->emb, (void *)d->d_tables, d->heads_b, d->self_k,
                   d->self_v, d->cross_k, d->cross_v, d->x, d->nrm, d->qkv, d->attn, d->q_x,
                   d->xctx, d->hidden, d->out, d->rows_in, d->logits, d->qx, d->sx, d->xsplit, d->row_planes, d->cand_v, d->cand_i, d->cand_counters, d->partials,
                   d->counters, d->d_stage_in, d->d_stage_out, d->d_eos_frame, d->d_min_frames,
                   d->d_history, d->d_mem_len, d->pf_mem, d->pf_nrm, d->pf_kv, d->pf_planes};
    for (size_t i = 0; i < sizeof(dev) / sizeof(dev[0]); ++i) cudaFree(dev[i]);
    void *pinned[] = {d->h_rows, d->h_out, d->h_stage_in, d->h_stage_out, d->h_ints, d->h_table};
    for (size_t i = 0; i < sizeof(pinned) / sizeof(pinned[0]); ++i)
        if (pinned[i] != NULL) cudaFreeHost(pinned[i]);
    if (d->prof_ev != NULL) {
        for (size_t i = 0; i < 2u * PROF_POOL; ++i)
            if (d->prof_ev[i] != NULL) cudaEventDestroy(d->prof_ev[i]);
        free(d->prof_ev);
    }
    free(d->prof_cls);
    if (d->ev0 != NULL) cudaEventDestroy(d->ev0);
    if (d->ev1 != NULL) cudaEventDestroy(d->ev1);
    free(d->slot_len);
    free(d->slot_mem);
    free(d);
}

static size_t pick_bucket(const mb_decoder *d, size_t batch) {
    for (size_t i = 0; i < d->n_buckets; ++i)
        if (d->bucket_size[i] >= batch) return i;
    return d->n_buckets - 1u;
}

int mynah_b200_decoder_create(void *state, const mynah_b200_decoder_desc *desc, void **decoder,
                              char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || desc == NULL || decoder == NULL) {
        mb_set_error(error, cap, "invalid decoder arguments");
        return -1;
    }
    *decoder = NULL;
    if (desc->layers == 0 || desc->width == 0 || desc->heads == 0 || desc->width % desc->heads != 0 ||
        desc->xattn_width == 0 || desc->memory_length == 0 || desc->capacity == 0 ||
        desc->slots == 0 || desc->max_batch == 0 ||
        desc->max_batch > 1024u || desc->layer == NULL || desc->position == NULL ||
        desc->norm_out == NULL || desc->max_positions < desc->capacity) {
        mb_set_error(error, cap, "invalid decoder shape");
        return -1;
    }
    if (desc->tables != 0 && (desc->embeddings == NULL || desc->head_w == NULL ||
                              desc->head_b == NULL || desc->vocab == 0 ||
                              desc->codebook_size > desc->vocab)) {
        mb_set_error(error, cap, "invalid decoder head description");
        return -1;
    }
    MB_TRY(cudaSetDevice(st->device), "cudaSetDevice");
    mb_decoder *d = (mb_decoder *)calloc(1, sizeof(*d));
    if (d == NULL) {
        mb_set_error(error, cap, "out of memory creating decoder");
        return -1;
    }
    d->st = st;
    d->layers = d->layers_run = desc->layers;
    d->width = desc->width;
    d->heads = desc->heads;
    d->hw = desc->width / desc->heads;
    d->ffn = 4u * desc->width;                     /* src/graph.c:2973 */
    d->xw = desc->xattn_width;
    d->T = desc->memory_length;
    d->capacity = desc->capacity;
    d->slots = desc->slots;
    d->max_batch = desc->max_batch;
    d->max_positions = desc->max_positions;
    d->tables = desc->tables;
    d->vocab = desc->vocab;
    d->codebook_size = desc->codebook_size;
    d->eos_id = desc->eos_id;
    const char *ng = getenv("MYNAH_B200_NO_GRAPH");
    d->use_graphs = !(ng != NULL && strcmp(ng, "0") != 0);
    const size_t W = d->width, F = d->ffn, XW = d->xw, MB = d->max_batch;
    const int q = st->quant;
    int ok = 1;
#define D_TRY(expr) do { if (ok && (expr) != 0) ok = 0; } while (0)
    d->L = (dec_layer *)calloc(d->layers, sizeof(dec_layer));
    d->slot_len = (size_t *)calloc(d->slots, sizeof(size_t));
    d->slot_mem = (size_t *)calloc(d->slots, sizeof(size_t));
    if (d->L == NULL || d->slot_len == NULL || d->slot_mem == NULL) { mb_set_error(error, cap, "out of memory"); ok = 0; }
    for (size_t l = 0; ok && l < d->layers; ++l) {
        const mynah_b200_layer_weights *s = &desc->layer[l];
        dec_layer *L = &d->L[l];
        D_TRY(upload_vec(&L->norm_self, s->norm_self, W, error, cap));
        D_TRY(upload_vec(&L->norm_xattn_query, s->norm_xattn_query, W, error, cap));
        D_TRY(upload_vec(&L->norm_pos_ff, s->norm_pos_ff, W, error, cap));
        if (s->norm_xattn_memory != NULL && s->kv_cross_w != NULL) {
            D_TRY(upload_vec(&L->norm_xattn_memory, s->norm_xattn_memory, W, error, cap));
            D_TRY(mb_weight_build(st, s->kv_cross_w, 2u * XW, W, MB_F32, &L->kv_cross, error, cap));
            if (ok && !st->strict && prefill_tc_wanted(W, 64u)) {
                /* fast mode: the text states' K/V product runs on the tensor cores */
                float amax = 0.0f;
                for (size_t i = 0; i < 2u * XW * W; ++i) {
                    const float v = fabsf(s->kv_cross_w[i]);
                    if (v > amax) amax = v;
                }
                int ex = 0;
                if (amax > 0.0f) {
                    (void)frexpf(amax, &ex);
                    ex = 14 - ex;
                }
                ex = ex > 30 ? 30 : (ex < -30 ? -30 : ex);
                L->kv_tc_scale = ldexpf(1.0f, ex);
                D_TRY(dmalloc(&L->kv_tc, mb_codec_tc_packed_halves(2u * XW, W, 1u) * 2u, error, cap));
                if (ok) D_TRY(mb_cuda(mb_codec_tc_pack_weight((const float *)L->kv_cross.w, L->kv_tc, 2u * XW, W, 1u, L->kv_tc_scale,
                                                              st->stream), "pack weight", error, cap));
            }
        }
        D_TRY(mb_weight_build(st, s->qkv_w, 3u * W, W, q, &L->qkv, error, cap));
        D_TRY(mb_weight_build(st, s->o_self_w, W, W, q, &L->o_self, error, cap));
        D_TRY(mb_weight_build(st, s->q_cross_w, XW, W, q, &L->q_cross, error, cap));
        D_TRY(mb_weight_build(st, s->o_cross_w, W, XW, q, &L->o_cross, error, cap));
        D_TRY(mb_weight_build(st, s->ffn_up_w, F, W, q, &L->ffn_up, error, cap));
        D_TRY(mb_weight_build(st, s->ffn_down_w, W, F, q, &L->ffn_down, error, cap));
        if (desc->keep_f32_weights && q != MB_F32) {
            D_TRY(mb_weight_build(st, s->qkv_w, 3u * W, W, MB_F32, &L->qkv32, error, cap));
            D_TRY(mb_weight_build(st, s->o_self_w, W, W, MB_F32, &L->o_self32, error, cap));
            D_TRY(mb_weight_build(st, s->q_cross_w, XW, W, MB_F32, &L->q_cross32, error, cap));
            D_TRY(mb_weight_build(st, s->o_cross_w, W, XW, MB_F32, &L->o_cross32, error, cap));
            D_TRY(mb_weight_build(st, s->ffn_up_w, F, W, MB_F32, &L->ffn_up32, error, cap));
            D_TRY(mb_weight_build(st, s->ffn_down_w, W, F, MB_F32, &L->ffn_down32, error, cap));
        }
        if (ok && desc->keep_f32_weights && !st->strict && prefill_tc_wanted(W, XW)) {
            /* the f32 weights once more as tensor-core planes (fast mode's many-row products) */
            const float *host[6] = {s->qkv_w, s->o_self_w, s->q_cross_w, s->o_cross_w, s->ffn_up_w, s->ffn_down_w};
            const mb_dev_weight *dev[6] = {q != MB_F32 ? &L->qkv32 : &L->qkv, q != MB_F32 ? &L->o_self32 : &L->o_self,
                                           q != MB_F32 ? &L->q_cross32 : &L->q_cross, q != MB_F32 ? &L->o_cross32 : &L->o_cross,
                                           q != MB_F32 ? &L->ffn_up32 : &L->ffn_up, q != MB_F32 ? &L->ffn_down32 : &L->ffn_down};
            for (int t = 0; ok && t < 6; ++t) {
                const size_t n = dev[t]->n, k = dev[t]->k;
                float amax = 0.0f;
                for (size_t i = 0; i < n * k; ++i) {
                    const float v = fabsf(host[t][i]);
                    if (v > amax) amax = v;
                }
                int ex = 0;
                if (amax > 0.0f) {
                    (void)frexpf(amax, &ex);
                    ex = 14 - ex;
                }
                ex = ex > 30 ? 30 : (ex < -30 ? -30 : ex);
                L->tc_scale[t] = ldexpf(1.0f, ex);
                D_TRY(dmalloc(&L->tc_w[t], mb_codec_tc_packed_halves(n, k, 1u) * 2u, error, cap));
                if (ok) D_TRY(mb_cuda(mb_codec_tc_pack_weight((const float *)dev[t]->w, L->tc_w[t], n, k, 1u, L->tc_scale[t], st->stream),
                                      "pack weight", error, cap));
            }
        }
        if (ok)
            d->weight_bytes += L->qkv.bytes + L->o_self.bytes + L->q_cross.bytes + L->o_cross.bytes +
                               L->ffn_up.bytes + L->ffn_down.bytes + 3u * W * sizeof(float);
    }
    D_TRY(upload_vec(&d->position, desc->position, d->max_positions * W, error, cap));
    D_TRY(upload_vec(&d->norm_out, desc->norm_out, W, error, cap));
    d->weight_bytes += W * sizeof(float);
    if (ok && d->tables != 0) {
        const size_t per = d->vocab * W;
        float *joined = (float *)malloc(d->tables * per * sizeof(float));
        float *joined_b = (float *)malloc(d->tables * d->vocab * sizeof(float));
        const float **ptrs = (const float **)malloc(d->tables * sizeof(*ptrs));
        if (joined == NULL || joined_b == NULL || ptrs == NULL) {
            mb_set_error(error, cap, "out of memory joining heads");
            ok = 0;
        }
        D_TRY(dmalloc((void **)&d->emb, d->tables * per * sizeof(float), error, cap));
        D_TRY(dmalloc((void **)&d->d_tables, d->tables * sizeof(float *), error, cap));
        for (size_t t = 0; ok && t < d->tables; ++t) {
            D_TRY(mb_cuda((int)cudaMemcpy(d->emb + t * per, desc->embeddings[t], per * sizeof(float),
                                          cudaMemcpyHostToDevice), "upload embeddings", error, cap));
            ptrs[t] = d->emb + t * per;
            memcpy(joined + t * per, desc->head_w[t], per * sizeof(float));
            memcpy(joined_b + t * d->vocab, desc->head_b[t], d->vocab * sizeof(float));
        }
        D_TRY(mb_cuda((int)cudaMemcpy((void *)d->d_tables, ptrs, d->tables * sizeof(float *),
                                      cudaMemcpyHostToDevice), "upload table pointers", error, cap));
        /* per-row / per-group quantization makes the joined pack identical to
         * packing each head alone */
        D_TRY(mb_weight_build(st, joined, d->tables * d->vocab, W, q, &d->heads_w, error, cap));
        D_TRY(upload_vec(&d->heads_b, joined_b, d->tables * d->vocab, error, cap));
        free(joined);
        free(joined_b);
        free(ptrs);
    }
    /* KV pools */
    const size_t self_n = d->slots * d->layers * d->capacity * W;
    const size_t cross_n = d->slots * d->layers * d->T * XW;
    D_TRY(dmalloc((void **)&d->self_k, self_n * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->self_v, self_n * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->cross_k, cross_n * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->cross_v, cross_n * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->d_mem_len, d->slots * sizeof(int), error, cap));
    if (ok) {
        /* every slot starts as a request of the full memory length over zeroed cross rows */
        int *full = (int *)malloc(d->slots * sizeof(int));
        if (full == NULL) { mb_set_error(error, cap, "out of memory"); ok = 0; }
        for (size_t i = 0; ok && i < d->slots; ++i) { full[i] = (int)d->T; d->slot_mem[i] = d->T; }
        D_TRY(mb_cuda((int)cudaMemcpy(d->d_mem_len, full, d->slots * sizeof(int), cudaMemcpyHostToDevice), "upload", error, cap));
        free(full);
        D_TRY(mb_cuda((int)cudaMemset(d->cross_k, 0, cross_n * sizeof(float)), "memset", error, cap));
        D_TRY(mb_cuda((int)cudaMemset(d->cross_v, 0, cross_n * sizeof(float)), "memset", error, cap));
    }
    {
        int have_kv = 1;
        for (size_t l = 0; l < d->layers; ++l)
            if (d->L[l].norm_xattn_memory == NULL || d->L[l].kv_cross.w == NULL) have_kv = 0;
        if (ok && have_kv) {
            /* scratch of slot_prefill, allocated once: admissions allocate and free nothing */
            D_TRY(dmalloc((void **)&d->pf_mem, d->T * W * sizeof(float), error, cap));
            D_TRY(dmalloc((void **)&d->pf_nrm, d->T * W * sizeof(float), error, cap));
            D_TRY(dmalloc((void **)&d->pf_kv, d->T * 2u * XW * sizeof(float), error, cap));
            if (d->L[0].kv_tc != NULL) D_TRY(dmalloc(&d->pf_planes, 2u * d->T * W * 2u, error, cap));
        }
    }
    /* activations */
    D_TRY(dmalloc((void **)&d->x, MB * W * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->nrm, MB * W * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->qkv, MB * 3u * W * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->attn, MB * W * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->q_x, MB * XW * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->xctx, MB * XW * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->hidden, MB * F * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->out, MB * W * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->rows_in, MB * W * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->qx, MB * F, error, cap));
    D_TRY(dmalloc((void **)&d->sx, MB * sizeof(float), error, cap));
    if (q == MB_F16)
        D_TRY(dmalloc(&d->xsplit, mb_gemm_tc_f16_split_halves(MB, F) * 2u, error, cap));
    if (d->L != NULL && d->L[0].tc_w[0] != NULL) D_TRY(dmalloc(&d->row_planes, 2u * MB * F * 2u, error, cap));
    if (d->tables != 0) {
        D_TRY(dmalloc((void **)&d->logits, MB * d->tables * d->vocab * sizeof(float), error, cap));
        if (q == MB_F32 && mb_heads_argmax_f32_supported(d->vocab, W)) {
            const size_t nc = mb_heads_argmax_candidates(MB, d->tables, d->vocab);
            D_TRY(dmalloc((void **)&d->cand_v, nc * sizeof(float), error, cap));
            D_TRY(dmalloc((void **)&d->cand_i, nc * sizeof(unsigned), error, cap));
            D_TRY(dmalloc((void **)&d->cand_counters, MB * d->tables * sizeof(unsigned), error, cap));
            if (ok) D_TRY(mb_cuda((int)cudaMemset(d->cand_counters, 0, MB * d->tables * sizeof(unsigned)), "cudaMemset", error, cap));
        }
        d->history_frames = d->capacity;
        D_TRY(dmalloc((void **)&d->d_history, d->history_frames * MB * d->tables * sizeof(unsigned), error, cap));
    }
    /* batch buckets: powers of two up to max_batch, then max_batch itself */
    for (size_t b = 1; b < MB && d->n_buckets < MAX_BUCKETS - 1u; b *= 2u) d->bucket_size[d->n_buckets++] = b;
    d->bucket_size[d->n_buckets++] = MB;
    size_t partial_floats = mb_attention_scratch_floats(MB, d->heads, d->capacity, d->hw);
    const size_t cross_floats = mb_attention_scratch_floats(MB, 1u, d->T, XW);
    if (cross_floats > partial_floats) partial_floats = cross_floats;
    const size_t n_counters = mb_attention_counters(MB, d->heads);
    {
        const char *no_tc = getenv("MYNAH_B200_NO_TC");
        d->use_tc = !(no_tc != NULL && strcmp(no_tc, "0") != 0);
        const char *no_fuse = getenv("MYNAH_B200_NO_FUSE");
        d->use_fuse1 = !(no_fuse != NULL && strcmp(no_fuse, "0") != 0);
        const char *no_xb = getenv("MYNAH_B200_NO_CROSS_BLOCK");
        d->use_xblock = !(no_xb != NULL && strcmp(no_xb, "0") != 0);
        const char *no_sq = getenv("MYNAH_B200_NO_SPLIT_QUANT");
        d->use_split_quant = !(no_sq != NULL && strcmp(no_sq, "0") != 0);
    }
    D_TRY(dmalloc((void **)&d->partials, partial_floats * sizeof(float), error, cap));
    D_TRY(dmalloc((void **)&d->counters, n_counters * sizeof(unsigned), error, cap));
    /* staged in: [slots MB | lens MB | allow_eos MB | eos_flag MB | n_active, frame_idx, 0, 0 | codes MB x tables];
     * read back: [status, 0, 0, 0 | tokens MB x tables] */
    d->stage_in_ints = 4u * MB + 4u + MB * d->tables;
    D_TRY(dmalloc((void **)&d->d_stage_in, d->stage_in_ints * sizeof(int), error, cap));
    D_TRY(dmalloc((void **)&d->d_stage_out, (4u + MB * d->tables) * sizeof(unsigned), error, cap));
    D_TRY(dmalloc((void **)&d->d_eos_frame, MB * sizeof(int), error, cap));
    if (ok) {
        D_TRY(mb_cuda((int)cudaMemset(d->d_stage_in, 0, d->stage_in_ints * sizeof(int)), "memset", error, cap));
        D_TRY(mb_cuda((int)cudaMemset(d->d_stage_out, 0, (4u + MB * d->tables) * sizeof(unsigned)), "memset", error, cap));
        d->d_slots = d->d_stage_in;
        d->d_lens = d->d_stage_in + MB;
        d->d_allow_eos = d->d_stage_in + 2u * MB;
        d->d_eos_flag = d->d_stage_in + 3u * MB;
        d->d_n_active = d->d_stage_in + 4u * MB;
        d->d_frame_idx = d->d_stage_in + 4u * MB + 1u;
        d->d_codes = (unsigned *)(d->d_stage_in + 4u * MB + 4u);
        d->d_status = (int *)d->d_stage_out;
        d->d_tokens = d->d_stage_out + 4u;
    }
    D_TRY(dmalloc((void **)&d->d_min_frames, sizeof(int), error, cap));
    if (ok) {
        D_TRY(mb_cuda((int)cudaMemset(d->counters, 0, n_counters * sizeof(unsigned)), "memset", error, cap));
        D_TRY(mb_cuda((int)cudaMemset(d->d_min_frames, 0, sizeof(int)), "memset", error, cap));
        D_TRY(mb_cuda((int)cudaMemset(d->self_k, 0, self_n * sizeof(float)), "memset", error, cap));
        D_TRY(mb_cuda((int)cudaMemset(d->self_v, 0, self_n * sizeof(float)), "memset", error, cap));
    }
    /* pinned staging */
    D_TRY(mb_cuda((int)cudaMallocHost((void **)&d->h_rows, MB * W * sizeof(float)), "cudaMallocHost", error, cap));
    D_TRY(mb_cuda((int)cudaMallocHost((void **)&d->h_out, MB * W * sizeof(float)), "cudaMallocHost", error, cap));
    D_TRY(mb_cuda((int)cudaMallocHost((void **)&d->h_stage_in, d->stage_in_ints * sizeof(int)), "cudaMallocHost", error, cap));
    D_TRY(mb_cuda((int)cudaMallocHost((void **)&d->h_stage_out, (4u + MB * d->tables) * sizeof(unsigned)), "cudaMallocHost", error, cap));
    if (ok) {
        memset(d->h_stage_in, 0, d->stage_in_ints * sizeof(int));
        memset(d->h_stage_out, 0, (4u + MB * d->tables) * sizeof(unsigned));
        d->h_slots = d->h_stage_in;
        d->h_lens = d->h_stage_in + MB;
        d->h_frame_idx = d->h_stage_in + 4u * MB + 1u;
        d->h_codes = (unsigned *)(d->h_stage_in + 4u * MB + 4u);
        d->h_status = (int *)d->h_stage_out;
        d->h_tokens = d->h_stage_out + 4u;
    }
    D_TRY(mb_cuda((int)cudaMallocHost((void **)&d->h_ints, 4u * MB * sizeof(int)), "cudaMallocHost", error, cap));
    D_TRY(mb_cuda((int)cudaMallocHost((void **)&d->h_table, (MB + 1u) * sizeof(int)), "cudaMallocHost", error, cap));
    D_TRY(mb_cuda((int)cudaEventCreate(&d->ev0), "cudaEventCreate", error, cap));
    D_TRY(mb_cuda((int)cudaEventCreate(&d->ev1), "cudaEventCreate", error, cap));
#undef D_TRY
    if (!ok) {
        mynah_b200_decoder_destroy(d);
        return -1;
    }
    for (size_t i = 0; i <= MB; ++i) d->h_table[i] = (int)i;
    *decoder = d;
    mb_clear_error(error, cap);
    return 0;
}

size_t mynah_b200_decoder_weight_bytes(const void *decoder) {
    const mb_decoder *d = (const mb_decoder *)decoder;
    return d == NULL ? 0u : d->weight_bytes;
}

/* self K+V rows [0, length] of every layer read once, one row of each written,
 * plus the constant cross K/V */
size_t mynah_b200_decoder_kv_bytes(const void *decoder, size_t length) {
    const mb_decoder *d = (const mb_decoder *)decoder;
    if (d == NULL) return 0u;
    return d->layers * (2u * (length + 1u) * d->width + 2u * d->width + 2u * d->T * d->xw) * sizeof(float);
}

/* ------------------------------------------------------------ the sequence */
/* fuse != MB_FUSE_NONE (one lane, int8, non-strict): the product makes its own quantized
 * activations from the f32 row act_f32 (layer norm with `gain`, or plain quantization). */
static int product_fused(mb_decoder *d, const mb_dev_weight *w, const float *bias, const float *act_f32,
                         float *out, size_t out_stride, size_t nb, int epilogue, int fuse,
                         const float *gain, unsigned *count) {
    mb_gemv_args g;
    memset(&g, 0, sizeof(g));
    g.fuse = fuse;
    g.fx = fuse != MB_FUSE_NONE ? act_f32 : NULL;
    g.fuse_gain = gain;
    g.fuse_eps = 1.0e-5f;
    mb_gemv_bind_weight(&g, w, bias);
    g.out = out;
    g.out_stride = out_stride;
    g.batch = nb;
    g.n_active = d->d_n_active;
    g.epilogue = epilogue;
    g.strict = d->st->strict;
    g.tanh_tab = d->st->libm.tanh_tab;
    if (w->qtype == MB_INT8 || w->qtype == MB_INT4) {
        g.qx = d->qx;
        g.sx = d->sx;
    } else {
        g.x = act_f32;
    }
    *count += 1u;
    if (d->use_tc && mb_gemm_tc_supported(w->qtype, w->n, w->k, nb))
        return mb_gemm_tc(&g, d->max_batch, d->d_status, d->st->stream);
    if (d->use_tc && w->qtype == MB_F16 && d->xsplit != NULL && w->k <= d->ffn &&
        mb_gemm_tc_f16_supported(w->n, w->k, nb)) {
        *count += 1u;   /* the activation split is a launch of its own */
        return mb_gemm_tc_f16(&g, d->xsplit, d->max_batch, d->d_status, d->st->stream);
    }
    return mb_gemv(&g, d->st->stream);
}

static int product(mb_decoder *d, const mb_dev_weight *w, const float *bias, const float *act_f32,
                   float *out, size_t out_stride, size_t nb, int epilogue, unsigned *count) {
    return product_fused(d, w, bias, act_f32, out, out_stride, nb, epilogue, MB_FUSE_NONE, NULL, count);
}

/* One lane, int8 weights: the norms and the attention row's quantization ride in the
 * products that consume them, in strict mode with the reference's summation order (the
 * hidden row's quantization stays a launch: 192 CTAs would each repeat it). */
static int fuse_one_lane(const mb_decoder *d, size_t nb) {
    return nb == 1 && d->use_fuse1 && d->st->quant == MB_INT8;
}

static int norm(mb_decoder *d, const float *in, float *out, const float *gain, size_t nb,
                unsigned *count) {
    const int q = quantized_mode(d);
    *count += 1u;
    return mb_layernorm(in, out, gain, NULL, nb, d->width, 1.0e-5f, q ? d->qx : NULL,
                        q ? d->sx : NULL, d->d_n_active, d->st->strict, d->st->stream);
}

/* Rows [row0, row0 + rows) of a packed weight as a weight of its own. */
static mb_dev_weight weight_rows(const mb_dev_weight *w, size_t row0, size_t rows) {
    mb_dev_weight v = *w;
    v.n = rows;
    unsigned char *base = (unsigned char *)w->w;
    switch (w->qtype) {
    case MB_INT8: v.w = base + row0 * w->k; v.scales = w->scales + row0; break;
    case MB_INT4: v.w = base + row0 * (w->k / 2u); v.scales = w->scales + row0 * (w->k / 32u); break;
    case MB_F16: v.w = base + row0 * w->k * 2u; break;
    default: v.w = base + row0 * w->k * 4u; break;
    }
    return v;
}

/* One stacked frame of the local transformer for nb lanes (src/graph.c:1374-1656), fully on
 * the device: table t's token is made at position t; position 0 reads `first_rows` (the
 * decoder's output rows), position t > 0 the embedding of the previous table's token, left
 * in local.row_in by the sampler. */
static int enqueue_local(mb_decoder *d, const float *first_rows, size_t nb, unsigned *count) {
    mb_state *st = d->st;
    mb_stream s = st->stream;
    mb_local *lt = &d->local;
    const size_t W = d->width, F = d->ffn;
    const int q = d->st->quant == MB_INT8 || d->st->quant == MB_INT4;
    const float scale = 1.0f / sqrtf((float)d->hw);
    int rc = 0;
#define L_TRY(expr) do { if (rc == 0) rc = (expr); } while (0)
    for (size_t t = 0; t < d->tables && rc == 0; ++t) {
        if (t == 0) {   /* later positions: the sampler of the table before wrote x = token row + position row */
            L_TRY(mb_add_row(first_rows, lt->position, d->x, nb, W, d->d_n_active, s));
            *count += 1u;
        }
        for (size_t l = 0; l < lt->layers && rc == 0; ++l) {
            const local_layer *L = &lt->L[l];
            const int f1 = fuse_one_lane(d, nb) && L->qkv.qtype == MB_INT8 && L->ffn_up.qtype == MB_INT8 &&
                           L->ffn_down.qtype == MB_INT8;
            if (f1) {
                L_TRY(product_fused(d, &L->qkv, NULL, d->x, d->qkv, 3u * W, nb, MB_EPI_STORE, MB_FUSE_LN,
                                    L->norm_self, count));
            } else {
                L_TRY(norm(d, d->x, d->nrm, L->norm_self, nb, count));
                L_TRY(product(d, &L->qkv, NULL, d->nrm, d->qkv, 3u * W, nb, MB_EPI_STORE, count));
            }
            mb_attn_args a;
            memset(&a, 0, sizeof(a));
            a.q = d->qkv;
            a.q_stride = 3u * W;
            a.k_new = d->qkv + W;
            a.v_new = d->qkv + 2u * W;
            a.k_cache = lt->k + l * lt->capacity * W;
            a.v_cache = lt->v + l * lt->capacity * W;
            a.slot_stride = lt->layers * lt->capacity * W;     /* lane b owns block b */
            a.position = t;
            a.valid = t + 1u;
            a.cache_rows = (d->max_batch - 1u) * lt->layers * lt->capacity + lt->capacity;
            a.cache_stride = W;
            a.heads = d->heads;
            a.head_width = d->hw;
            a.scale = scale;
            a.out = d->attn;
            a.out_stride = W;
            a.qx = q ? d->qx : NULL;
            a.sx = q ? d->sx : NULL;
            a.batch = nb;
            a.n_active = d->d_n_active;
            a.strict = st->strict;
            a.exp_tab = st->libm.exp_tab;
            a.partials = d->partials;
            a.counters = d->counters;
            a.status = d->d_status;
            a.sm_count = st->sm_count;
            a.early_prefetch = 1;   /* rows below t were appended at earlier positions of this frame */
            a.short_cache = lt->capacity <= 32u;
            a.launched = count;
            L_TRY(mb_attention(&a, s));
            L_TRY(product(d, &L->o, NULL, d->attn, d->x, W, nb, MB_EPI_RESIDUAL, count));
            if (f1) {
                L_TRY(product_fused(d, &L->ffn_up, NULL, d->x, d->hidden, F, nb, MB_EPI_GELU, MB_FUSE_LN,
                                    L->norm_ff, count));
                /* as in the decoder's layers: the hidden row is quantized once, by its own launch */
                L_TRY(mb_quant_rows(d->hidden, nb, F, d->qx, d->sx, d->d_n_active, s));
                *count += 1u;
                L_TRY(product(d, &L->ffn_down, NULL, d->hidden, d->x, W, nb, MB_EPI_RESIDUAL, count));
            } else {
                L_TRY(norm(d, d->x, d->nrm, L->norm_ff, nb, count));
                L_TRY(product(d, &L->ffn_up, NULL, d->nrm, d->hidden, F, nb, MB_EPI_GELU, count));
                if (q) {
                    L_TRY(mb_quant_rows(d->hidden, nb, F, d->qx, d->sx, d->d_n_active, s));
                    *count += 1u;
                }
                L_TRY(product(d, &L->ffn_down, NULL, d->hidden, d->x, W, nb, MB_EPI_RESIDUAL, count));
            }
        }
        /* this table's projection (no norm in between: src/graph.c:1339-1341, 1538-1549) */
        const mb_dev_weight head = weight_rows(&d->heads_w, t * d->vocab, d->vocab);
        if (fuse_one_lane(d, nb) && head.qtype == MB_INT8) {
            L_TRY(product_fused(d, &head, d->heads_b + t * d->vocab, d->x, d->logits, d->vocab, nb, MB_EPI_STORE,
                                MB_FUSE_QUANT, NULL, count));
        } else {
            if (q) {
                L_TRY(mb_quant_rows(d->x, nb, W, d->qx, d->sx, d->d_n_active, s));
                *count += 1u;
            }
            L_TRY(product(d, &head, d->heads_b + t * d->vocab, d->x, d->logits, d->vocab, nb, MB_EPI_STORE, count));
        }
        mb_sample_args sa;
        memset(&sa, 0, sizeof(sa));
        sa.logits = d->logits;
        sa.logits_stride = d->vocab;
        sa.vocab = d->vocab;
        sa.codebook_size = d->codebook_size;
        sa.eos_id = d->eos_id;
        sa.batch = nb;
        sa.allow_eos = d->d_allow_eos;
        sa.temperature = lt->d_temp;
        sa.topk = lt->d_topk;
        sa.rng = lt->d_rng;
        sa.table = t;
        sa.tables = d->tables;
        sa.codebooks = lt->codebooks;
        sa.tokens = d->d_tokens;
        sa.codes = d->d_codes;
        sa.eos_flag = d->d_eos_flag;
        sa.eos_sub = lt->d_eos_sub;
        sa.emb_table = d->emb + t * d->vocab * W;
        sa.row_in = lt->row_in;
        sa.next_row = t + 1u < d->tables ? lt->position + (t + 1u) * W : NULL;
        sa.x_out = d->x;
        sa.width = W;
        sa.strict = st->strict;
        sa.exp_tab = st->libm.exp_tab;
        sa.n_active = d->d_n_active;
        L_TRY(mb_local_sample(&sa, s));
        *count += 1u;
    }
#undef L_TRY
    return rc;
}

static int enqueue(mb_decoder *d, size_t bucket, int mode, unsigned *count) {
    mb_state *st = d->st;
    mb_stream s = st->stream;
    const size_t nb = d->bucket_size[bucket];
    const size_t W = d->width, F = d->ffn, XW = d->xw;
    const int q = quantized_mode(d);
    const float self_scale = 1.0f / sqrtf((float)d->hw);   /* src/graph.c:3143-3144 */
    const float cross_scale = 1.0f / sqrtf((float)XW);
    int rc = 0;
#define E_TRY(expr) do { if (rc == 0) rc = (expr); } while (0)
#define P(cls, expr) do { prof_begin(d, (cls)); E_TRY(expr); prof_end(d); } while (0)
    if (mode == MODE_LOCAL_ONLY) {
        prof_begin(d, PC_LOCAL);
        rc = enqueue_local(d, d->out, nb, count);
        prof_end(d);
        return rc;
    }
    prof_begin(d, PC_INPUT);
    if (mode == MODE_FRAME || mode == MODE_LOCAL) {
        E_TRY(mb_embed_frames(d->d_tables, d->tables, d->vocab, W, d->d_codes, d->position,
                              d->d_lens, d->x, nb, d->d_n_active, d->d_status, s));
    } else {
        E_TRY(mb_add_position(d->rows_in, d->position, d->d_lens, d->x, nb, W, d->d_n_active, s));
    }
    prof_end(d);
    *count += 1u;
    for (size_t l = 0; l < d->layers_run && rc == 0; ++l) {
        const dec_layer *L = &d->L[l];
        const int f1 = fuse_one_lane(d, nb) && L->qkv.qtype == MB_INT8 && L->q_cross.qtype == MB_INT8 &&
                       L->ffn_up.qtype == MB_INT8 && L->ffn_down.qtype == MB_INT8;
        if (f1) {
            P(PC_QKV, product_fused(d, &L->qkv, NULL, d->x, d->qkv, 3u * W, nb, MB_EPI_STORE, MB_FUSE_LN,
                                    L->norm_self, count));
        } else {
            P(PC_NORM, norm(d, d->x, d->nrm, L->norm_self, nb, count));
            P(PC_QKV, product(d, &L->qkv, NULL, d->nrm, d->qkv, 3u * W, nb, MB_EPI_STORE, count));
        }
        mb_attn_args a;
        memset(&a, 0, sizeof(a));
        a.q = d->qkv;
        a.q_stride = 3u * W;
        a.k_new = d->qkv + W;
        a.v_new = d->qkv + 2u * W;
        a.k_cache = d->self_k + l * d->capacity * W;
        a.v_cache = d->self_v + l * d->capacity * W;
        a.slot_stride = d->layers * d->capacity * W;
        a.slots = d->d_slots;
        a.lens = d->d_lens;
        a.valid = d->capacity;
        a.cache_rows = (d->slots - 1u) * d->layers * d->capacity + d->capacity;
        a.cache_stride = W;
        a.heads = d->heads;
        a.head_width = d->hw;
        a.scale = self_scale;
        a.out = d->attn;
        a.out_stride = W;
        /* one lane: the output product quantizes the row in its own prologue, which spares the
         * attention's head groups their arrival counter and the gathering tail */
        const int o_fused = f1 && L->o_self.qtype == MB_INT8;
        /* strict mode, two or more lanes: the attention leaves its rows in f32 and a launch of
         * its own quantizes them.  The attention's head groups then need no arrival counter and
         * no gathering tail, which costs more than the extra launch, hidden as it is behind its
         * neighbours (measured 1.7% to 4.9% per step between 8 and 256 streams; fast mode, whose
         * attention kernel is another, loses 0.8% and keeps the tail) */
        const int q_sep = !o_fused && q && st->strict && nb >= 2 && d->use_split_quant;
        a.qx = (q && !o_fused && !q_sep) ? d->qx : NULL;
        a.sx = (q && !o_fused && !q_sep) ? d->sx : NULL;
        a.batch = nb;
        a.n_active = d->d_n_active;
        a.strict = st->strict;
        a.exp_tab = st->libm.exp_tab;
        a.partials = d->partials;
        a.counters = d->counters;
        a.status = d->d_status;
        a.sm_count = st->sm_count;
        a.early_prefetch = 1;   /* lane state: previous step; cache rows below the position: earlier steps */
        a.launched = count;
        P(PC_ATTN_SELF, mb_attention(&a, s));
        if (q_sep) {
            P(PC_QUANT, mb_quant_rows(d->attn, nb, W, d->qx, d->sx, d->d_n_active, s));
            *count += 1u;
            P(PC_O_SELF, product(d, &L->o_self, NULL, d->attn, d->x, W, nb, MB_EPI_RESIDUAL, count));
        } else if (o_fused) {
            P(PC_O_SELF, product_fused(d, &L->o_self, NULL, d->attn, d->x, W, nb, MB_EPI_RESIDUAL, MB_FUSE_QUANT, NULL, count));
        } else {
            P(PC_O_SELF, product(d, &L->o_self, NULL, d->attn, d->x, W, nb, MB_EPI_RESIDUAL, count));
        }
        /* int8 and int4: the whole cross-attention block, with the norm before the feed-forward
         * product, is one launch with one CTA per stream */
        const int xq = L->q_cross.qtype;
        const int xb = d->use_xblock && q && (xq == MB_INT8 || (xq == MB_INT4 && W % 32u == 0 && XW % 32u == 0)) &&
                       L->o_cross.qtype == xq && (L->ffn_up.qtype == MB_INT8 || L->ffn_up.qtype == MB_INT4) &&
                       mb_cross_block_supported(W, XW, d->T);
        if (xb) {
            mb_cross_block_args cb;
            memset(&cb, 0, sizeof(cb));
            cb.x = d->x;
            cb.gain_query = L->norm_xattn_query;
            cb.gain_ff = L->norm_pos_ff;
            cb.qtype = xq;
            cb.wq = (const int8_t *)L->q_cross.w;
            cb.wq_scales = L->q_cross.scales;
            cb.wo = (const int8_t *)L->o_cross.w;
            cb.wo_scales = L->o_cross.scales;
            cb.k_cache = d->cross_k + l * d->T * XW;
            cb.v_cache = d->cross_v + l * d->T * XW;
            cb.slot_stride = d->layers * d->T * XW;
            cb.cache_rows = (d->slots - 1u) * d->layers * d->T + d->T;
            cb.slots = d->d_slots;
            cb.n_active = d->d_n_active;
            cb.batch = nb;
            cb.width = W;
            cb.xw = XW;
            cb.rows = d->T;
            cb.rows_per_slot = d->d_mem_len;
            cb.scale = cross_scale;
            cb.eps = 1.0e-5f;
            cb.qx = d->qx;
            cb.sx = d->sx;
            cb.status = d->d_status;
            cb.strict = st->strict;
            cb.exp_tab = st->libm.exp_tab;
            P(PC_XBLOCK, mb_cross_block(&cb, s));
            *count += 1u;
            P(PC_FFN_UP, product(d, &L->ffn_up, NULL, d->nrm, d->hidden, F, nb, MB_EPI_GELU, count));
            /* the hidden row is quantized by a launch of its own at every lane count: in the
             * product's prologue each of its 192 CTAs would take the absmax of all 3072 values
             * first (one lane, measured: 481 -> 443 us per frame in fast mode without that
             * prologue, strict unchanged) */
            P(PC_QUANT, mb_quant_rows(d->hidden, nb, F, d->qx, d->sx, d->d_n_active, s));
            *count += 1u;
            P(PC_FFN_DOWN, product(d, &L->ffn_down, NULL, d->hidden, d->x, W, nb, MB_EPI_RESIDUAL, count));
            continue;
        }
        if (f1) {
            P(PC_Q_CROSS, product_fused(d, &L->q_cross, NULL, d->x, d->q_x, XW, nb, MB_EPI_STORE, MB_FUSE_LN,
                                        L->norm_xattn_query, count));
        } else {
            P(PC_NORM, norm(d, d->x, d->nrm, L->norm_xattn_query, nb, count));
            P(PC_Q_CROSS, product(d, &L->q_cross, NULL, d->nrm, d->q_x, XW, nb, MB_EPI_STORE, count));
        }
        memset(&a, 0, sizeof(a));
        a.q = d->q_x;
        a.q_stride = XW;
        a.k_cache = d->cross_k + l * d->T * XW;
        a.v_cache = d->cross_v + l * d->T * XW;
        a.slot_stride = d->layers * d->T * XW;
        a.slots = d->d_slots;
        a.position = 0;
        a.valid = d->T;
        a.valid_per_slot = d->d_mem_len;
        a.cache_rows = (d->slots - 1u) * d->layers * d->T + d->T;
        a.cache_stride = XW;
        a.heads = 1;
        a.head_width = XW;
        a.scale = cross_scale;
        a.out = d->xctx;
        a.out_stride = XW;
        a.qx = q ? d->qx : NULL;
        a.sx = q ? d->sx : NULL;
        a.batch = nb;
        a.n_active = d->d_n_active;
        a.strict = st->strict;
        a.exp_tab = st->libm.exp_tab;
        a.partials = d->partials;
        a.counters = d->counters;
        a.status = d->d_status;
        a.sm_count = st->sm_count;
        a.early_prefetch = 1;   /* the cross cache is written once, when the slot is loaded */
        a.launched = count;
        P(PC_ATTN_CROSS, mb_attention(&a, s));
        P(PC_O_CROSS, product(d, &L->o_cross, NULL, d->xctx, d->x, W, nb, MB_EPI_RESIDUAL, count));
        if (f1) {
            P(PC_FFN_UP, product_fused(d, &L->ffn_up, NULL, d->x, d->hidden, F, nb, MB_EPI_GELU, MB_FUSE_LN,
                                       L->norm_pos_ff, count));
            P(PC_QUANT, mb_quant_rows(d->hidden, nb, F, d->qx, d->sx, d->d_n_active, s));
            *count += 1u;
            P(PC_FFN_DOWN, product(d, &L->ffn_down, NULL, d->hidden, d->x, W, nb, MB_EPI_RESIDUAL, count));
        } else {
            P(PC_NORM, norm(d, d->x, d->nrm, L->norm_pos_ff, nb, count));
            P(PC_FFN_UP, product(d, &L->ffn_up, NULL, d->nrm, d->hidden, F, nb, MB_EPI_GELU, count));
            if (q) {
                P(PC_QUANT, mb_quant_rows(d->hidden, nb, F, d->qx, d->sx, d->d_n_active, s));
                *count += 1u;
            }
            P(PC_FFN_DOWN, product(d, &L->ffn_down, NULL, d->hidden, d->x, W, nb, MB_EPI_RESIDUAL, count));
        }
    }
    P(PC_NORM, norm(d, d->x, d->out, d->norm_out, nb, count));
    if (mode == MODE_FRAME && d->cand_v != NULL && d->use_fuse1 && d->heads_w.qtype == MB_F32) {
        /* f32 heads: projection and constrained pick in one launch (src/qmat.c:453-536) */
        mb_heads_argmax_args ha;
        memset(&ha, 0, sizeof(ha));
        ha.w = (const float *)d->heads_w.w; ha.bias = d->heads_b; ha.x = d->out;
        ha.tables = d->tables; ha.vocab = d->vocab; ha.k = W; ha.batch = nb;
        ha.codebook_size = d->codebook_size; ha.eos_id = d->eos_id;
        ha.allow_eos = d->d_allow_eos; ha.n_active = d->d_n_active;
        ha.cand_v = d->cand_v; ha.cand_i = d->cand_i; ha.counters = d->cand_counters;
        ha.tokens = d->d_tokens; ha.codes = d->d_codes; ha.eos_flag = d->d_eos_flag;
        P(PC_HEADS, mb_heads_argmax_f32(&ha, s));
        P(PC_ADVANCE, mb_frame_advance(d->d_lens, d->d_tokens, d->d_history, d->d_frame_idx,
                                       d->d_eos_flag, d->d_eos_frame, d->d_allow_eos, nb,
                                       d->max_batch, d->tables, d->d_min_frames, d->history_frames,
                                       d->d_n_active, s));
        *count += 2u;
    } else if (mode == MODE_FRAME) {
        P(PC_HEADS, product(d, &d->heads_w, d->heads_b, d->out, d->logits, d->tables * d->vocab, nb,
                            MB_EPI_STORE, count));
        P(PC_ARGMAX, mb_argmax_rows(d->logits, nb * d->tables, d->vocab, d->codebook_size, d->eos_id,
                                    d->d_allow_eos, 0, d->d_tokens, d->d_codes, d->d_eos_flag,
                                    d->tables, d->d_n_active, s));
        P(PC_ADVANCE, mb_frame_advance(d->d_lens, d->d_tokens, d->d_history, d->d_frame_idx,
                                       d->d_eos_flag, d->d_eos_frame, d->d_allow_eos, nb,
                                       d->max_batch, d->tables, d->d_min_frames, d->history_frames,
                                       d->d_n_active, s));
        *count += 2u;
    } else if (mode == MODE_LOCAL) {
        P(PC_LOCAL, enqueue_local(d, d->out, nb, count));
        P(PC_ADVANCE, mb_frame_advance(d->d_lens, d->d_tokens, d->d_history, d->d_frame_idx,
                                       d->d_eos_flag, d->d_eos_frame, d->d_allow_eos, nb,
                                       d->max_batch, d->tables, d->d_min_frames, d->history_frames,
                                       d->d_n_active, s));
        *count += 1u;
    } else {
        P(PC_ADVANCE, mb_advance_lens(d->d_lens, nb, d->d_n_active, s));
        *count += 1u;
    }
#undef P
#undef E_TRY
    return rc;
}

/* Launch one step for the bucket that holds `batch` lanes (graph replay, or the
 * eager sequence when graphs are disabled). */
static int run(mb_decoder *d, size_t batch, int mode, char *error, size_t cap) {
    const size_t bucket = pick_bucket(d, batch);
    mb_state *st = d->st;
    if (!d->use_graphs || d->profiling) {
        unsigned count = 0;
        MB_TRY(enqueue(d, bucket, mode, &count), "decoder step");
        st->launches += count;
        return 0;
    }
    if (d->graph[mode][bucket] == NULL) {
        cudaGraph_t graph = NULL;
        unsigned count = 0;
        MB_TRY(cudaStreamBeginCapture(st->stream, cudaStreamCaptureModeThreadLocal), "begin capture");
        const int rc = enqueue(d, bucket, mode, &count);
        const int rc_end = (int)cudaStreamEndCapture(st->stream, &graph);
        if (rc != 0 || rc_end != 0) {
            if (graph != NULL) cudaGraphDestroy(graph);
            return mb_cuda(rc != 0 ? rc : rc_end, "capture decoder step", error, cap);
        }
        const int rc_inst = (int)cudaGraphInstantiate(&d->graph[mode][bucket], graph, 0);
        cudaGraphDestroy(graph);
        if (rc_inst != 0) {
            d->graph[mode][bucket] = NULL;
            return mb_cuda(rc_inst, "instantiate decoder graph", error, cap);
        }
        d->graph_launches[mode][bucket] = count;
    }
    MB_TRY(cudaGraphLaunch(d->graph[mode][bucket], st->stream), "launch decoder graph");
    st->launches += d->graph_launches[mode][bucket];
    return 0;
}

/* --------------------------------------------------------------- slot state */
static int check_slot(const mb_decoder *d, size_t slot, char *error, size_t cap) {
    if (d == NULL || slot >= d->slots) {
        mb_set_error(error, cap, "decoder slot out of range");
        return -1;
    }
    return mb_cuda((int)cudaSetDevice(d->st->device), "cudaSetDevice", error, cap);
}

/* One slot's text-state count to the device (kernels read it per lane). */
static int set_slot_memory(mb_decoder *d, size_t slot, size_t rows, char *error, size_t cap) {
    const int v = (int)rows;
    MB_TRY(cudaMemcpyAsync(d->d_mem_len + slot, &v, sizeof(int), cudaMemcpyHostToDevice, d->st->stream), "stage memory length");
    MB_TRY(cudaStreamSynchronize(d->st->stream), "cudaStreamSynchronize");   /* &v leaves scope */
    d->slot_mem[slot] = rows;
    return 0;
}

int mynah_b200_decoder_slot_load(void *decoder, size_t slot, const float *cross_k,
                                 const float *cross_v, size_t memory_length, const float *self_k,
                                 const float *self_v, size_t length, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0) return -1;
    if (cross_k == NULL || cross_v == NULL || length > d->capacity ||
        (length > 0 && (self_k == NULL || self_v == NULL))) {
        mb_set_error(error, cap, "invalid slot contents");
        return -1;
    }
    if (memory_length == 0 || memory_length > d->T) {
        mb_set_error(error, cap, "slot memory length must be 1 .. the decoder's memory_length");
        return -1;
    }
    cudaStream_t s = d->st->stream;
    const size_t cross_n = d->layers * d->T * d->xw, rows_n = memory_length * d->xw;
    /* the request's arrays are [layers][memory_length][xw]; a slot keeps [layers][T][xw] */
    for (size_t l = 0; l < d->layers; ++l) {
        MB_TRY(cudaMemcpyAsync(d->cross_k + slot * cross_n + l * d->T * d->xw, cross_k + l * rows_n,
                               rows_n * sizeof(float), cudaMemcpyHostToDevice, s), "upload cross K");
        MB_TRY(cudaMemcpyAsync(d->cross_v + slot * cross_n + l * d->T * d->xw, cross_v + l * rows_n,
                               rows_n * sizeof(float), cudaMemcpyHostToDevice, s), "upload cross V");
    }
    const size_t per_layer = d->capacity * d->width;
    for (size_t l = 0; l < d->layers && length > 0; ++l) {
        const size_t off = (slot * d->layers + l) * per_layer;
        MB_TRY(cudaMemcpyAsync(d->self_k + off, self_k + l * per_layer, length * d->width * sizeof(float),
                               cudaMemcpyHostToDevice, s), "upload self K");
        MB_TRY(cudaMemcpyAsync(d->self_v + off, self_v + l * per_layer, length * d->width * sizeof(float),
                               cudaMemcpyHostToDevice, s), "upload self V");
    }
    if (set_slot_memory(d, slot, memory_length, error, cap) != 0) return -1;
    d->slot_len[slot] = length;
    mb_clear_error(error, cap);
    return 0;
}

/* decoder_cache_init's cross K/V (src/graph.c:3002-3027) on the device: per layer
 * LayerNorm(memory, norm_xattn_memory) through kv_net in f32 (the reference calls the
 * backend's f32 matmul here whatever MYNAH_QUANT says), first xw columns K, next xw V. */
int mynah_b200_decoder_slot_prefill(void *decoder, size_t slot, const float *memory,
                                    size_t memory_length, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0) return -1;
    if (memory == NULL || memory_length == 0 || memory_length > d->T) {
        mb_set_error(error, cap, "prefill: memory must have 1 .. the decoder's memory_length rows");
        return -1;
    }
    if (d->pf_mem == NULL) {
        mb_set_error(error, cap, "prefill: the decoder was created without norm_xattn_memory / kv_net weights");
        return -1;
    }
    mb_state *st = d->st;
    cudaStream_t s = st->stream;
    const size_t W = d->width, XW = d->xw, T = d->T, M = memory_length;
    float *mem = d->pf_mem, *nrm = d->pf_nrm, *kv = d->pf_kv;
    int rc = 0;
#define F_TRY(expr, what) do { if (rc == 0 && mb_cuda((int)(expr), (what), error, cap) != 0) rc = -1; } while (0)
    F_TRY(cudaMemcpyAsync(mem, memory, M * W * sizeof(float), cudaMemcpyHostToDevice, s), "upload memory");
    const size_t cross_n = d->layers * T * XW;
    for (size_t l = 0; l < d->layers && rc == 0; ++l) {
        F_TRY(mb_layernorm(mem, nrm, d->L[l].norm_xattn_memory, NULL, M, W, 1.0e-5f, NULL, NULL, NULL,
                           st->strict, s), "layer norm of the memory");
        if (d->pf_planes != NULL && d->L[l].kv_tc != NULL && d->use_tc) {
            unsigned short *hi = (unsigned short *)d->pf_planes, *lo = hi + T * W;
            F_TRY(mb_split_rows_f16(nrm, hi, lo, M, W, W, s), "split rows");
            mb_codec_conv_tc_args t;
            memset(&t, 0, sizeof(t));
            t.x_planes = hi; t.x_plane_stride = T * W;
            t.w_packed = d->L[l].kv_tc; t.scale = d->L[l].kv_tc_scale;
            t.ic = W; t.oc = 2u * XW; t.length = M; t.kernel = 1u; t.dilation = 1u;
            t.rows_out = kv; t.rows_stride = 2u * XW; t.rows_epilogue = MB_EPI_STORE;
            t.status = d->d_status; t.sm_count = st->sm_count;
            F_TRY(mb_codec_conv1d_tc(&t, s), "kv_net product");
            st->launches += 1u;
        } else {
            mb_gemv_args g;
            memset(&g, 0, sizeof(g));
            mb_gemv_bind_weight(&g, &d->L[l].kv_cross, NULL);
            g.x = nrm;
            g.out = kv;
            g.out_stride = 2u * XW;
            g.batch = M;
            g.epilogue = MB_EPI_STORE;
            g.strict = st->strict;
            F_TRY(mb_gemv(&g, s), "kv_net product");
        }
        float *ck = d->cross_k + slot * cross_n + l * T * XW;
        float *cv = d->cross_v + slot * cross_n + l * T * XW;
        F_TRY(cudaMemcpy2DAsync(ck, XW * sizeof(float), kv, 2u * XW * sizeof(float), XW * sizeof(float), M,
                                cudaMemcpyDeviceToDevice, s), "split K");
        F_TRY(cudaMemcpy2DAsync(cv, XW * sizeof(float), kv + XW, 2u * XW * sizeof(float), XW * sizeof(float), M,
                                cudaMemcpyDeviceToDevice, s), "split V");
        st->launches += 2u;
    }
    F_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");   /* the caller's memory may go away */
#undef F_TRY
    if (rc != 0) return -1;
    if (set_slot_memory(d, slot, M, error, cap) != 0) return -1;
    d->slot_len[slot] = 0;
    mb_clear_error(error, cap);
    return 0;
}

/* Copy a slot's cross K/V back: host arrays [layers][memory_length][xattn_width]. */
int mynah_b200_decoder_slot_read_cross(void *decoder, size_t slot, float *cross_k, float *cross_v,
                                       char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0) return -1;
    if (cross_k == NULL || cross_v == NULL) {
        mb_set_error(error, cap, "invalid buffers");
        return -1;
    }
    const size_t cross_n = d->layers * d->T * d->xw;
    MB_TRY(cudaStreamSynchronize(d->st->stream), "cudaStreamSynchronize");
    MB_TRY(cudaMemcpy(cross_k, d->cross_k + slot * cross_n, cross_n * sizeof(float), cudaMemcpyDeviceToHost), "read cross K");
    MB_TRY(cudaMemcpy(cross_v, d->cross_v + slot * cross_n, cross_n * sizeof(float), cudaMemcpyDeviceToHost), "read cross V");
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_decoder_slot_length(void *decoder, size_t slot, size_t *length, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0 || length == NULL) return -1;
    *length = d->slot_len[slot];
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_decoder_slot_set_length(void *decoder, size_t slot, size_t length, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0) return -1;
    if (length > d->capacity) {
        mb_set_error(error, cap, "slot length beyond capacity");
        return -1;
    }
    d->slot_len[slot] = length;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_decoder_slot_read_kv(void *decoder, size_t slot, float *self_k, float *self_v,
                                    char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0 || self_k == NULL || self_v == NULL) return -1;
    const size_t n = d->layers * d->capacity * d->width;
    MB_TRY(cudaStreamSynchronize(d->st->stream), "cudaStreamSynchronize");
    MB_TRY(cudaMemcpy(self_k, d->self_k + slot * n, n * sizeof(float), cudaMemcpyDeviceToHost), "read K");
    MB_TRY(cudaMemcpy(self_v, d->self_v + slot * n, n * sizeof(float), cudaMemcpyDeviceToHost), "read V");
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_decoder_set_layers(void *decoder, size_t n, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d == NULL || n == 0 || n > d->layers) {
        mb_set_error(error, cap, "layer count out of range");
        return -1;
    }
    MB_TRY(cudaSetDevice(d->st->device), "cudaSetDevice");
    MB_TRY(cudaStreamSynchronize(d->st->stream), "cudaStreamSynchronize");
    if (n != d->layers_run) destroy_graphs(d);
    d->layers_run = n;
    mb_clear_error(error, cap);
    return 0;
}

/* ----------------------------------------------------------------- stepping */
/* Validate the slot list and stage slot ids and positions for the lanes. */
/* Validates the lanes of a call and writes their slots and positions to the pinned staging
 * block (the caller copies them to the device). */
static int fill_lanes(mb_decoder *d, const unsigned *slots, size_t batch, char *error, size_t cap) {
    if (d == NULL || slots == NULL || batch == 0 || batch > d->max_batch) {
        mb_set_error(error, cap, "decoder batch exceeds max_batch");   /* src/graph.c:3133-3136 */
        return -1;
    }
    MB_TRY(cudaSetDevice(d->st->device), "cudaSetDevice");
    for (size_t b = 0; b < batch; ++b) {
        if (slots[b] >= d->slots) {
            mb_set_error(error, cap, "decoder slot out of range");
            return -1;
        }
        for (size_t o = 0; o < b; ++o)
            if (slots[o] == slots[b]) {
                mb_set_error(error, cap, "a slot may appear once per step");
                return -1;
            }
        if (d->slot_len[slots[b]] >= d->capacity || d->slot_len[slots[b]] >= d->max_positions) {
            mb_set_error(error, cap, "decoder cache capacity exceeded");   /* src/graph.c:3152-3155 */
            return -1;
        }
        d->h_slots[b] = (int)slots[b];
        d->h_lens[b] = (int)d->slot_len[slots[b]];
    }
    return 0;
}

static int stage_lanes(mb_decoder *d, const unsigned *slots, size_t batch, char *error, size_t cap) {
    if (fill_lanes(d, slots, batch, error, cap) != 0) return -1;
    cudaStream_t s = d->st->stream;
    MB_TRY(cudaMemcpyAsync(d->d_slots, d->h_slots, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage slots");
    MB_TRY(cudaMemcpyAsync(d->d_lens, d->h_lens, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage positions");
    MB_TRY(cudaMemcpyAsync(d->d_n_active, &d->h_table[batch], sizeof(int), cudaMemcpyHostToDevice, s), "stage lane count");
    return 0;
}

static int check_status(mb_decoder *d, char *error, size_t cap) {
    int status = 0;
    MB_TRY(cudaMemcpy(&status, d->d_status, sizeof(int), cudaMemcpyDeviceToHost), "read status");
    if (status != 0) {
        cudaMemset(d->d_status, 0, sizeof(int));
        mb_set_error(error, cap, mb_status_message(status));
        return -1;
    }
    return 0;
}

int mynah_b200_decoder_step_batch(void *decoder, const unsigned *slots,
                                  const float *const *inputs, float *const *outs, size_t batch,
                                  char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d != NULL && batch == 0) return 0;   /* src/graph.c:3132 */
    if (inputs == NULL || outs == NULL) {
        mb_set_error(error, cap, "invalid decoder step buffers");
        return -1;
    }
    if (stage_lanes(d, slots, batch, error, cap) != 0) return -1;
    const size_t W = d->width;
    cudaStream_t s = d->st->stream;
    for (size_t b = 0; b < batch; ++b) memcpy(d->h_rows + b * W, inputs[b], W * sizeof(float));
    MB_TRY(cudaMemcpyAsync(d->rows_in, d->h_rows, batch * W * sizeof(float), cudaMemcpyHostToDevice, s), "stage inputs");
    if (run(d, batch, MODE_STEP, error, cap) != 0) return -1;
    MB_TRY(cudaMemcpyAsync(d->h_out, d->out, batch * W * sizeof(float), cudaMemcpyDeviceToHost, s), "read outputs");
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    for (size_t b = 0; b < batch; ++b) {
        memcpy(outs[b], d->h_out + b * W, W * sizeof(float));
        d->slot_len[slots[b]] += 1u;
    }
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_decoder_frame_batch(void *decoder, const unsigned *slots, const unsigned *codes,
                                   const int *allow_eos, unsigned *tokens, float *hidden,
                                   size_t batch, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d != NULL && batch == 0) return 0;
    if (d == NULL || d->tables == 0 || codes == NULL || tokens == NULL) {
        mb_set_error(error, cap, "decoder has no embedding tables or heads");
        return -1;
    }
    if (fill_lanes(d, slots, batch, error, cap) != 0) return -1;
    const size_t nt = batch * d->tables, MB = d->max_batch;
    cudaStream_t s = d->st->stream;
    /* One copy in: slots and positions (fill_lanes), the EOS rule, cleared EOS flags, the lane
     * count, frame index 0 (history row 0 is scratch for this entry point; the allow_eos
     * flags written by frame_advance are restaged on every call) and the codes.  Lanes past
     * `batch` carry what the block held before: every kernel masks them by the lane count. */
    int *in = d->h_stage_in;
    for (size_t b = 0; b < batch; ++b) {
        in[2u * MB + b] = allow_eos == NULL ? 1 : (allow_eos[b] != 0);
        in[3u * MB + b] = 0;
    }
    in[4u * MB] = (int)batch;
    in[4u * MB + 1u] = 0;
    memcpy(d->h_codes, codes, nt * sizeof(unsigned));
    MB_TRY(cudaMemcpyAsync(d->d_stage_in, d->h_stage_in, (4u * MB + 4u + nt) * sizeof(int), cudaMemcpyHostToDevice, s),
           "stage the frame");
    if (run(d, batch, MODE_FRAME, error, cap) != 0) return -1;
    /* one copy out: the status word and the tokens */
    MB_TRY(cudaMemcpyAsync(d->h_stage_out, d->d_stage_out, (4u + nt) * sizeof(unsigned), cudaMemcpyDeviceToHost, s),
           "read tokens");
    if (hidden != NULL)
        MB_TRY(cudaMemcpyAsync(d->h_out, d->out, batch * d->width * sizeof(float), cudaMemcpyDeviceToHost, s), "read hidden");
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if (*d->h_status != 0 && check_status(d, error, cap) != 0) return -1;
    memcpy(tokens, d->h_tokens, nt * sizeof(unsigned));
    if (hidden != NULL) memcpy(hidden, d->h_out, batch * d->width * sizeof(float));
    for (size_t b = 0; b < batch; ++b) d->slot_len[slots[b]] += 1u;
    mb_clear_error(error, cap);
    return 0;
}

static int stage_samplers(mb_decoder *d, const mynah_b200_sampler *samplers, const size_t *order,
                          size_t batch, char *error, size_t cap);

/* The device-resident frame loop behind _greedy (mode MODE_FRAME: logit heads) and _generate
 * (mode MODE_LOCAL: the local transformer and its sampler). */
static int decode_loop(mb_decoder *d, int mode, mynah_b200_sampler *samplers, const unsigned *slots,
                       size_t batch, unsigned *codes, const size_t *frames, size_t min_frames,
                       unsigned *tokens, long *eos_frame, float *elapsed_ms, char *error, size_t cap) {
    if (d == NULL || d->tables == 0 || codes == NULL || frames == NULL || tokens == NULL ||
        slots == NULL || batch == 0 || batch > d->max_batch ||
        (mode == MODE_LOCAL && d->local.layers == 0)) {
        mb_set_error(error, cap, "invalid decode request");
        return -1;
    }
    /* lanes ordered by frame count, longest first, so live lanes are a prefix */
    size_t *order = (size_t *)malloc(batch * sizeof(size_t));
    unsigned *lane_slots = (unsigned *)malloc(batch * sizeof(unsigned));
    if (order == NULL || lane_slots == NULL) {
        free(order); free(lane_slots);
        mb_set_error(error, cap, "out of memory");
        return -1;
    }
    for (size_t i = 0; i < batch; ++i) order[i] = i;
    for (size_t i = 1; i < batch; ++i) {           /* stable insertion sort, descending */
        const size_t v = order[i];
        size_t j = i;
        while (j > 0 && frames[order[j - 1]] < frames[v]) { order[j] = order[j - 1]; --j; }
        order[j] = v;
    }
    const size_t max_frames = frames[order[0]];
    int rc = 0;
    for (size_t i = 0; i < batch; ++i) {
        lane_slots[i] = slots[order[i]];
        if (slots[order[i]] < d->slots &&
            d->slot_len[slots[order[i]]] + frames[order[i]] > d->capacity) rc = -1;
    }
    if (rc != 0 || max_frames > d->history_frames) {
        free(order); free(lane_slots);
        mb_set_error(error, cap, "decoder cache capacity exceeded");
        return -1;
    }
    if (max_frames == 0) { free(order); free(lane_slots); return 0; }
    if (stage_lanes(d, lane_slots, batch, error, cap) != 0) { free(order); free(lane_slots); return -1; }
    if (mode == MODE_LOCAL && stage_samplers(d, samplers, order, batch, error, cap) != 0) {
        free(order); free(lane_slots);
        return -1;
    }
    const size_t T = d->tables;
    cudaStream_t s = d->st->stream;
    for (size_t i = 0; i < batch; ++i) {
        memcpy(d->h_codes + i * T, codes + order[i] * T, T * sizeof(unsigned));
        d->h_ints[i] = min_frames == 0 ? 1 : 0;                 /* allow_eos at frame 0 */
        d->h_ints[d->max_batch + i] = -1;                       /* eos_frame */
    }
    d->h_ints[2u * d->max_batch] = min_frames > 0x7fffffffu ? 0x7fffffff : (int)min_frames;
#define G_TRY(expr, what) do { if (rc == 0 && mb_cuda((int)(expr), (what), error, cap) != 0) rc = -1; } while (0)
    G_TRY(cudaMemcpyAsync(d->d_codes, d->h_codes, batch * T * sizeof(unsigned), cudaMemcpyHostToDevice, s), "stage codes");
    G_TRY(cudaMemcpyAsync(d->d_allow_eos, d->h_ints, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage eos rule");
    G_TRY(cudaMemcpyAsync(d->d_eos_frame, d->h_ints + d->max_batch, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage eos frames");
    G_TRY(cudaMemcpyAsync(d->d_min_frames, d->h_ints + 2u * d->max_batch, sizeof(int), cudaMemcpyHostToDevice, s), "stage min frames");
    G_TRY(cudaMemsetAsync(d->d_eos_flag, 0, d->max_batch * sizeof(int), s), "clear eos flags");
    G_TRY(cudaMemsetAsync(d->d_frame_idx, 0, sizeof(int), s), "clear frame index");
    G_TRY(cudaMemsetAsync(d->d_history, 0, max_frames * d->max_batch * T * sizeof(unsigned), s), "clear history");
    G_TRY(cudaEventRecord(d->ev0, s), "record event");
    size_t live = batch;
    for (size_t f = 0; f < max_frames && rc == 0; ++f) {
        size_t now = live;
        while (now > 0 && frames[order[now - 1]] <= f) --now;
        if (now != live) {
            live = now;
            G_TRY(cudaMemcpyAsync(d->d_n_active, &d->h_table[live], sizeof(int), cudaMemcpyHostToDevice, s), "stage lane count");
        }
        if (rc == 0 && run(d, live, mode, error, cap) != 0) rc = -1;
    }
    G_TRY(cudaEventRecord(d->ev1, s), "record event");
    unsigned *hist = (unsigned *)malloc(max_frames * d->max_batch * T * sizeof(unsigned));
    int *eosf = (int *)malloc(batch * sizeof(int));
    if (hist == NULL || eosf == NULL) { mb_set_error(error, cap, "out of memory"); rc = -1; }
    G_TRY(cudaMemcpyAsync(hist, d->d_history, max_frames * d->max_batch * T * sizeof(unsigned), cudaMemcpyDeviceToHost, s), "read tokens");
    G_TRY(cudaMemcpyAsync(eosf, d->d_eos_frame, batch * sizeof(int), cudaMemcpyDeviceToHost, s), "read eos frames");
    G_TRY(cudaMemcpyAsync(d->h_codes, d->d_codes, batch * T * sizeof(unsigned), cudaMemcpyDeviceToHost, s), "read codes");
    unsigned long long *rng_back = (unsigned long long *)d->h_rows;
    if (mode == MODE_LOCAL)
        G_TRY(cudaMemcpyAsync(rng_back, d->local.d_rng, batch * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s), "read rng");
    G_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if (rc == 0 && elapsed_ms != NULL) G_TRY(cudaEventElapsedTime(elapsed_ms, d->ev0, d->ev1), "event time");
    if (rc == 0 && check_status(d, error, cap) != 0) rc = -1;
#undef G_TRY
    if (rc == 0) {
        memset(tokens, 0, max_frames * batch * T * sizeof(unsigned));
        for (size_t i = 0; i < batch; ++i) {
            const size_t b = order[i];
            for (size_t f = 0; f < frames[b]; ++f)
                memcpy(tokens + (f * batch + b) * T, hist + (f * d->max_batch + i) * T, T * sizeof(unsigned));
            memcpy(codes + b * T, d->h_codes + i * T, T * sizeof(unsigned));
            if (eos_frame != NULL) eos_frame[b] = eosf[i];
            if (mode == MODE_LOCAL && samplers != NULL) samplers[b].rng_state = rng_back[i];
            d->slot_len[slots[b]] += frames[b];
        }
        mb_clear_error(error, cap);
    }
    free(hist); free(eosf); free(order); free(lane_slots);
    return rc;
}

int mynah_b200_decoder_greedy(void *decoder, const unsigned *slots, size_t batch, unsigned *codes,
                              const size_t *frames, size_t min_frames, unsigned *tokens,
                              long *eos_frame, float *elapsed_ms, char *error, size_t cap) {
    return decode_loop((mb_decoder *)decoder, MODE_FRAME, NULL, slots, batch, codes, frames, min_frames,
                       tokens, eos_frame, elapsed_ms, error, cap);
}

int mynah_b200_decoder_generate(void *decoder, const unsigned *slots, size_t batch, unsigned *codes,
                                const size_t *frames, size_t min_frames,
                                mynah_b200_sampler *samplers, unsigned *tokens, long *eos_frame,
                                float *elapsed_ms, char *error, size_t cap) {
    return decode_loop((mb_decoder *)decoder, MODE_LOCAL, samplers, slots, batch, codes, frames,
                       min_frames, tokens, eos_frame, elapsed_ms, error, cap);
}

/* ------------------------------------------------------------------ prefill */
/* One product of the prefill: through the decoder's packed weight with quantized rows
 * (d->qx/d->sx) when `packed`, else through the f32 weight with the f32 rows -- in fast mode
 * on the tensor cores when the decoder holds the weight's f16 planes (tc_w != NULL). */
static int prefill_product(mb_decoder *d, const mb_dev_weight *wq, const mb_dev_weight *w32, int packed,
                           const float *act_f32, float *out, size_t out_stride, size_t nb, int epilogue,
                           unsigned *count, const void *tc_w, float tc_scale) {
    if (packed) return product(d, wq, NULL, act_f32, out, out_stride, nb, epilogue, count);
    if (tc_w != NULL && d->row_planes != NULL && d->use_tc) {
        const size_t k = w32->k;
        unsigned short *hi = (unsigned short *)d->row_planes, *lo = hi + d->max_batch * k;
        int rc = mb_split_rows_f16(act_f32, hi, lo, nb, k, k, d->st->stream);
        if (rc != 0) return rc;
        mb_codec_conv_tc_args t;
        memset(&t, 0, sizeof(t));
        t.x_planes = hi; t.x_plane_stride = d->max_batch * k;
        t.w_packed = tc_w; t.scale = tc_scale;
        t.ic = k; t.oc = w32->n; t.length = nb; t.kernel = 1u; t.dilation = 1u;
        t.rows_out = out; t.rows_stride = out_stride; t.rows_epilogue = epilogue;
        t.status = d->d_status; t.sm_count = d->st->sm_count;
        *count += 2u;
        return mb_codec_conv1d_tc(&t, d->st->stream);
    }
    mb_gemv_args g;
    memset(&g, 0, sizeof(g));
    mb_gemv_bind_weight(&g, w32, NULL);
    g.x = act_f32;
    g.out = out;
    g.out_stride = out_stride;
    g.batch = nb;
    g.n_active = d->d_n_active;
    g.epilogue = epilogue;
    g.strict = d->st->strict;
    g.tanh_tab = d->st->libm.tanh_tab;
    *count += 1u;
    return mb_gemv(&g, d->st->stream);
}

/* decoder_run with count > 1 (src/graph.c:3506-3641): `count` new rows of ONE request go
 * through the stack together; row i attends the request's cached rows and the new rows up
 * to itself.  The rows ride as `count` lanes that share the slot at consecutive positions:
 * the new K/V rows of a layer are appended first (they lie back to back in the cache), then
 * every lane attends up to its own position.  As in the reference, more than 16 rows of a
 * quantized model are multiplied with the f32 weights (src/qmat.c:773-788: the quantized
 * product is taken for at most 16 rows), at most 16 with the packed weights row by row; the
 * self-attention weights are e * (1 / sum) (softmax_row_inplace, src/graph.c:245-257).  The
 * output-norm row of the last new row is returned (src/graph.c:3640-3642). */
int mynah_b200_decoder_prefill(void *decoder, size_t slot, const float *rows, size_t count,
                               float *out_last, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (check_slot(d, slot, error, cap) != 0) return -1;
    if (rows == NULL || out_last == NULL || count == 0) {
        mb_set_error(error, cap, "invalid prefill buffers");
        return -1;
    }
    const size_t start = d->slot_len[slot];
    if (start + count > d->capacity || start + count > d->max_positions) {
        mb_set_error(error, cap, "decoder cache capacity exceeded");          /* src/graph.c:3309-3312 */
        return -1;
    }
    if (count > d->max_batch) {
        mb_set_error(error, cap, "prefill: more rows than the decoder's max_batch");   /* src/graph.c:3313-3316 */
        return -1;
    }
    mb_state *st = d->st;
    const int q = quantized_mode(d);
    const int f32_model = st->quant == MB_F32;
    /* packed weights: an f32 or f16 model always; a quantized one for at most 16 rows */
    /* fast mode with the weights' f16 planes at hand: more than 16 rows go through the tensor cores */
    const int tc_rows = !st->strict && d->use_tc && d->row_planes != NULL && count > 16u && st->quant != MB_F16;
    const int packed = !tc_rows && (f32_model || st->quant == MB_F16 || count <= 16u);
    if (!packed && !f32_model && d->L[0].qkv32.w == NULL) {
        mb_set_error(error, cap, "prefill of more than 16 rows of a quantized model uses the f32 weights: "
                                 "create the decoder with keep_f32_weights");
        return -1;
    }
    const int quant_rows = q && packed;      /* products read int8 rows */
    cudaStream_t s = st->stream;
    const size_t W = d->width, F = d->ffn, XW = d->xw;
    const float self_scale = 1.0f / sqrtf((float)d->hw), cross_scale = 1.0f / sqrtf((float)XW);
    for (size_t b = 0; b < count; ++b) {
        d->h_slots[b] = (int)slot;
        d->h_lens[b] = (int)(start + b);
    }
    MB_TRY(cudaMemcpyAsync(d->d_slots, d->h_slots, count * sizeof(int), cudaMemcpyHostToDevice, s), "stage slots");
    MB_TRY(cudaMemcpyAsync(d->d_lens, d->h_lens, count * sizeof(int), cudaMemcpyHostToDevice, s), "stage positions");
    MB_TRY(cudaMemcpyAsync(d->d_n_active, &d->h_table[count], sizeof(int), cudaMemcpyHostToDevice, s), "stage lane count");
    memcpy(d->h_rows, rows, count * W * sizeof(float));
    MB_TRY(cudaMemcpyAsync(d->rows_in, d->h_rows, count * W * sizeof(float), cudaMemcpyHostToDevice, s), "stage rows");
    unsigned launches = 0;
    int rc = 0;
#define R_TRY(expr) do { if (rc == 0) rc = (int)(expr); } while (0)
    R_TRY(mb_add_position(d->rows_in, d->position, d->d_lens, d->x, count, W, d->d_n_active, s));
    launches += 1u;
    for (size_t l = 0; l < d->layers_run && rc == 0; ++l) {
        const dec_layer *L = &d->L[l];
        mb_attn_args a;
        R_TRY(mb_layernorm(d->x, d->nrm, L->norm_self, NULL, count, W, 1.0e-5f, quant_rows ? d->qx : NULL,
                           quant_rows ? d->sx : NULL, d->d_n_active, st->strict, s));
        launches += 1u;
        R_TRY(prefill_product(d, &L->qkv, f32_model ? &L->qkv : &L->qkv32, packed, d->nrm, d->qkv, 3u * W, count, MB_EPI_STORE, &launches, L->tc_w[0], L->tc_scale[0]));
        /* the new rows' K and V into the cache: rows start .. start + count - 1 of this layer */
        float *kc = d->self_k + ((slot * d->layers + l) * d->capacity + start) * W;
        float *vc = d->self_v + ((slot * d->layers + l) * d->capacity + start) * W;
        R_TRY(cudaMemcpy2DAsync(kc, W * sizeof(float), d->qkv + W, 3u * W * sizeof(float), W * sizeof(float), count,
                                cudaMemcpyDeviceToDevice, s));
        R_TRY(cudaMemcpy2DAsync(vc, W * sizeof(float), d->qkv + 2u * W, 3u * W * sizeof(float), W * sizeof(float), count,
                                cudaMemcpyDeviceToDevice, s));
        memset(&a, 0, sizeof(a));
        a.q = d->qkv;
        a.q_stride = 3u * W;
        a.k_cache = d->self_k + l * d->capacity * W;
        a.v_cache = d->self_v + l * d->capacity * W;
        a.slot_stride = d->layers * d->capacity * W;
        a.slots = d->d_slots;
        a.lens = d->d_lens;                 /* lane b attends rows 0 .. start + b */
        a.valid = d->capacity;
        a.cache_rows = (d->slots - 1u) * d->layers * d->capacity + d->capacity;
        a.cache_stride = W;
        a.heads = d->heads;
        a.head_width = d->hw;
        a.scale = self_scale;
        a.out = d->attn;
        a.out_stride = W;
        a.qx = quant_rows ? d->qx : NULL;
        a.sx = quant_rows ? d->sx : NULL;
        a.batch = count;
        a.n_active = d->d_n_active;
        a.strict = st->strict;
        a.exp_tab = st->libm.exp_tab;
        a.partials = d->partials;
        a.counters = d->counters;
        a.status = d->d_status;
        a.sm_count = st->sm_count;
        a.softmax_inverse = 1;
        a.launched = &launches;
        R_TRY(mb_attention(&a, s));
        R_TRY(prefill_product(d, &L->o_self, f32_model ? &L->o_self : &L->o_self32, packed, d->attn, d->x, W, count, MB_EPI_RESIDUAL, &launches, L->tc_w[1], L->tc_scale[1]));
        R_TRY(mb_layernorm(d->x, d->nrm, L->norm_xattn_query, NULL, count, W, 1.0e-5f, quant_rows ? d->qx : NULL,
                           quant_rows ? d->sx : NULL, d->d_n_active, st->strict, s));
        launches += 1u;
        R_TRY(prefill_product(d, &L->q_cross, f32_model ? &L->q_cross : &L->q_cross32, packed, d->nrm, d->q_x, XW, count, MB_EPI_STORE, &launches, L->tc_w[2], L->tc_scale[2]));
        memset(&a, 0, sizeof(a));
        a.q = d->q_x;
        a.q_stride = XW;
        a.k_cache = d->cross_k + l * d->T * XW;
        a.v_cache = d->cross_v + l * d->T * XW;
        a.slot_stride = d->layers * d->T * XW;
        a.slots = d->d_slots;
        a.valid = d->T;
        a.valid_per_slot = d->d_mem_len;
        a.cache_rows = (d->slots - 1u) * d->layers * d->T + d->T;
        a.cache_stride = XW;
        a.heads = 1;
        a.head_width = XW;
        a.scale = cross_scale;
        a.out = d->xctx;
        a.out_stride = XW;
        a.qx = quant_rows ? d->qx : NULL;
        a.sx = quant_rows ? d->sx : NULL;
        a.batch = count;
        a.n_active = d->d_n_active;
        a.strict = st->strict;
        a.exp_tab = st->libm.exp_tab;
        a.partials = d->partials;
        a.counters = d->counters;
        a.status = d->d_status;
        a.sm_count = st->sm_count;
        a.launched = &launches;
        R_TRY(mb_attention(&a, s));
        R_TRY(prefill_product(d, &L->o_cross, f32_model ? &L->o_cross : &L->o_cross32, packed, d->xctx, d->x, W, count, MB_EPI_RESIDUAL, &launches, L->tc_w[3], L->tc_scale[3]));
        R_TRY(mb_layernorm(d->x, d->nrm, L->norm_pos_ff, NULL, count, W, 1.0e-5f, quant_rows ? d->qx : NULL,
                           quant_rows ? d->sx : NULL, d->d_n_active, st->strict, s));
        launches += 1u;
        R_TRY(prefill_product(d, &L->ffn_up, f32_model ? &L->ffn_up : &L->ffn_up32, packed, d->nrm, d->hidden, F, count, MB_EPI_GELU, &launches, L->tc_w[4], L->tc_scale[4]));
        if (quant_rows) {
            R_TRY(mb_quant_rows(d->hidden, count, F, d->qx, d->sx, d->d_n_active, s));
            launches += 1u;
        }
        R_TRY(prefill_product(d, &L->ffn_down, f32_model ? &L->ffn_down : &L->ffn_down32, packed, d->hidden, d->x, W, count, MB_EPI_RESIDUAL, &launches, L->tc_w[5], L->tc_scale[5]));
    }
    /* the output norm of the last new row only */
    R_TRY(mb_layernorm(d->x + (count - 1u) * W, d->out, d->norm_out, NULL, 1u, W, 1.0e-5f, NULL, NULL, NULL, st->strict, s));
    launches += 1u;
#undef R_TRY
    if (rc != 0) return mb_cuda(rc, "decoder prefill", error, cap);
    st->launches += launches;
    MB_TRY(cudaMemcpyAsync(d->h_out, d->out, W * sizeof(float), cudaMemcpyDeviceToHost, s), "read output");
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if (check_status(d, error, cap) != 0) return -1;
    memcpy(out_last, d->h_out, W * sizeof(float));
    d->slot_len[slot] += count;
    mb_clear_error(error, cap);
    return 0;
}

/* ------------------------------------------------------- local transformer */
int mynah_b200_decoder_local_attach(void *decoder, const mynah_b200_local_desc *desc, char *error,
                                    size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d == NULL || desc == NULL || desc->layer == NULL || desc->position == NULL) {
        mb_set_error(error, cap, "invalid local transformer arguments");
        return -1;
    }
    if (d->tables == 0 || desc->layers == 0 || desc->layers > 4u || desc->codebooks == 0 ||
        desc->position_rows < d->tables || d->local.layers != 0) {
        mb_set_error(error, cap, "local transformer needs embedding tables and projections, 1..4 layers, "
                                 "one position row per table, and may be attached once");
        return -1;
    }
    MB_TRY(cudaSetDevice(d->st->device), "cudaSetDevice");
    mb_state *st = d->st;
    mb_local *lt = &d->local;
    const size_t W = d->width, F = d->ffn, MB = d->max_batch;
    const int q = st->quant;
    int ok = 1;
#define A_TRY(expr) do { if (ok && (expr) != 0) ok = 0; } while (0)
    lt->capacity = d->tables + 1u;                  /* src/graph.c:1200 */
    lt->codebooks = desc->codebooks;
    A_TRY(upload_vec(&lt->position, desc->position, desc->position_rows * W, error, cap));
    for (size_t l = 0; l < desc->layers; ++l) {
        const mynah_b200_local_layer_weights *src = &desc->layer[l];
        local_layer *L = &lt->L[l];
        A_TRY(upload_vec(&L->norm_self, src->norm_self, W, error, cap));
        A_TRY(upload_vec(&L->norm_ff, src->norm_pos_ff, W, error, cap));
        A_TRY(mb_weight_build(st, src->qkv_w, 3u * W, W, q, &L->qkv, error, cap));
        A_TRY(mb_weight_build(st, src->o_w, W, W, q, &L->o, error, cap));
        A_TRY(mb_weight_build(st, src->ffn_up_w, F, W, q, &L->ffn_up, error, cap));
        A_TRY(mb_weight_build(st, src->ffn_down_w, W, F, q, &L->ffn_down, error, cap));
        if (ok) d->weight_bytes += L->qkv.bytes + L->o.bytes + L->ffn_up.bytes + L->ffn_down.bytes;
    }
    const size_t kv = MB * desc->layers * lt->capacity * W;
    A_TRY(dmalloc((void **)&lt->k, kv * sizeof(float), error, cap));
    A_TRY(dmalloc((void **)&lt->v, kv * sizeof(float), error, cap));
    A_TRY(dmalloc((void **)&lt->row_in, MB * W * sizeof(float), error, cap));
    A_TRY(dmalloc((void **)&lt->d_temp, MB * sizeof(float), error, cap));
    A_TRY(dmalloc((void **)&lt->d_topk, MB * sizeof(unsigned), error, cap));
    A_TRY(dmalloc((void **)&lt->d_rng, MB * sizeof(unsigned long long), error, cap));
    A_TRY(dmalloc((void **)&lt->d_eos_sub, MB * sizeof(int), error, cap));
    if (ok) A_TRY(mb_cuda((int)cudaMemset(lt->d_eos_sub, 0xff, MB * sizeof(int)), "cudaMemset", error, cap));   /* -1: none yet */
    if (ok) {
        A_TRY(mb_cuda((int)cudaMemset(lt->k, 0, kv * sizeof(float)), "memset", error, cap));
        A_TRY(mb_cuda((int)cudaMemset(lt->v, 0, kv * sizeof(float)), "memset", error, cap));
        A_TRY(mb_cuda((int)cudaMemset(lt->d_temp, 0, MB * sizeof(float)), "memset", error, cap));
        A_TRY(mb_cuda((int)cudaMemset(lt->d_topk, 0, MB * sizeof(unsigned)), "memset", error, cap));
        A_TRY(mb_cuda((int)cudaMemset(lt->d_rng, 0, MB * sizeof(unsigned long long)), "memset", error, cap));
    }
#undef A_TRY
    if (!ok) return -1;     /* the decoder's destructor releases whatever was built */
    lt->layers = desc->layers;
    mb_clear_error(error, cap);
    return 0;
}

/* Sampler settings of `batch` lanes (in lane order) to the device. */
static int stage_samplers(mb_decoder *d, const mynah_b200_sampler *samplers, const size_t *order,
                          size_t batch, char *error, size_t cap) {
    mb_local *lt = &d->local;
    cudaStream_t s = d->st->stream;
    float *temp = (float *)d->h_rows;                               /* pinned, >= max_batch floats */
    unsigned *topk = (unsigned *)(d->h_rows + d->max_batch);
    unsigned long long *rng = (unsigned long long *)(d->h_rows + 2u * d->max_batch);
    for (size_t i = 0; i < batch; ++i) {
        const mynah_b200_sampler *sp = samplers == NULL ? NULL : &samplers[order == NULL ? i : order[i]];
        temp[i] = sp == NULL ? 0.0f : sp->temperature;
        topk[i] = sp == NULL ? 0u : sp->topk;
        rng[i] = sp == NULL ? 0ull : sp->rng_state;
    }
    MB_TRY(cudaMemcpyAsync(lt->d_temp, temp, batch * sizeof(float), cudaMemcpyHostToDevice, s), "stage temperatures");
    MB_TRY(cudaMemcpyAsync(lt->d_topk, topk, batch * sizeof(unsigned), cudaMemcpyHostToDevice, s), "stage top-k");
    MB_TRY(cudaMemcpyAsync(lt->d_rng, rng, batch * sizeof(unsigned long long), cudaMemcpyHostToDevice, s), "stage rng");
    /* the pinned block is reused by later calls: finish the copies first */
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    return 0;
}

int mynah_b200_decoder_local_frame(void *decoder, const float *decoder_last, size_t batch,
                                   mynah_b200_sampler *samplers, unsigned *codes, unsigned *values,
                                   int *saw_eos, long *eos_frame, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d != NULL && batch == 0) return 0;
    if (d == NULL || d->local.layers == 0 || decoder_last == NULL || codes == NULL ||
        batch > d->max_batch) {
        mb_set_error(error, cap, "local frame: no local transformer attached, or bad arguments");
        return -1;
    }
    MB_TRY(cudaSetDevice(d->st->device), "cudaSetDevice");
    cudaStream_t s = d->st->stream;
    const size_t W = d->width, T = d->tables;
    if (stage_samplers(d, samplers, NULL, batch, error, cap) != 0) return -1;
    memcpy(d->h_rows, decoder_last, batch * W * sizeof(float));
    for (size_t b = 0; b < batch; ++b) {
        d->h_ints[b] = samplers == NULL ? 1 : (samplers[b].allow_eos != 0);
        d->h_ints[d->max_batch + b] = 0x7fffffff;
    }
    MB_TRY(cudaMemcpyAsync(d->out, d->h_rows, batch * W * sizeof(float), cudaMemcpyHostToDevice, s), "stage rows");
    MB_TRY(cudaMemcpyAsync(d->d_allow_eos, d->h_ints, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage eos rule");
    MB_TRY(cudaMemcpyAsync(d->local.d_eos_sub, d->h_ints + d->max_batch, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage eos frames");
    MB_TRY(cudaMemsetAsync(d->d_eos_flag, 0, batch * sizeof(int), s), "clear eos flags");
    MB_TRY(cudaMemcpyAsync(d->d_n_active, &d->h_table[batch], sizeof(int), cudaMemcpyHostToDevice, s), "stage lane count");
    if (run(d, batch, MODE_LOCAL_ONLY, error, cap) != 0) return -1;
    unsigned long long *rng = (unsigned long long *)d->h_rows;
    MB_TRY(cudaMemcpyAsync(d->h_codes, d->d_codes, batch * T * sizeof(unsigned), cudaMemcpyDeviceToHost, s), "read codes");
    MB_TRY(cudaMemcpyAsync(d->h_tokens, d->d_tokens, batch * T * sizeof(unsigned), cudaMemcpyDeviceToHost, s), "read tokens");
    MB_TRY(cudaMemcpyAsync(d->h_ints, d->d_eos_flag, batch * sizeof(int), cudaMemcpyDeviceToHost, s), "read eos flags");
    MB_TRY(cudaMemcpyAsync(d->h_ints + d->max_batch, d->local.d_eos_sub, batch * sizeof(int), cudaMemcpyDeviceToHost, s), "read eos frames");
    MB_TRY(cudaMemcpyAsync(rng, d->local.d_rng, batch * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s), "read rng");
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if (check_status(d, error, cap) != 0) return -1;
    memcpy(codes, d->h_codes, batch * T * sizeof(unsigned));
    if (values != NULL) memcpy(values, d->h_tokens, batch * T * sizeof(unsigned));
    for (size_t b = 0; b < batch; ++b) {
        if (saw_eos != NULL) saw_eos[b] = d->h_ints[b] != 0;
        if (eos_frame != NULL) eos_frame[b] = d->h_ints[b] != 0 ? (long)d->h_ints[d->max_batch + b] : -1;
        if (samplers != NULL) samplers[b].rng_state = rng[b];
    }
    mb_clear_error(error, cap);
    return 0;
}

/* One sampled frame for `batch` slots with HOST buffers: frame_batch with the local
 * transformer and its sampler in place of the logit heads (one iteration of the loop of
 * synthesize_slots, src/graph.c:4083-4183). */
int mynah_b200_decoder_frame_batch_local(void *decoder, const unsigned *slots, const unsigned *codes,
                                         mynah_b200_sampler *samplers, unsigned *codes_out,
                                         unsigned *values, int *saw_eos, long *eos_frame,
                                         size_t batch, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d != NULL && batch == 0) return 0;
    if (d == NULL || d->local.layers == 0 || codes == NULL || codes_out == NULL) {
        mb_set_error(error, cap, "sampled frame: no local transformer attached, or bad arguments");
        return -1;
    }
    if (stage_lanes(d, slots, batch, error, cap) != 0) return -1;
    if (stage_samplers(d, samplers, NULL, batch, error, cap) != 0) return -1;
    const size_t T = d->tables, nt = batch * T;
    cudaStream_t s = d->st->stream;
    memcpy(d->h_codes, codes, nt * sizeof(unsigned));
    for (size_t b = 0; b < batch; ++b) {
        d->h_ints[b] = samplers == NULL ? 1 : (samplers[b].allow_eos != 0);
        d->h_ints[d->max_batch + b] = 0x7fffffff;
    }
    MB_TRY(cudaMemcpyAsync(d->d_codes, d->h_codes, nt * sizeof(unsigned), cudaMemcpyHostToDevice, s), "stage codes");
    MB_TRY(cudaMemcpyAsync(d->d_allow_eos, d->h_ints, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage eos rule");
    MB_TRY(cudaMemcpyAsync(d->local.d_eos_sub, d->h_ints + d->max_batch, batch * sizeof(int), cudaMemcpyHostToDevice, s), "stage eos frames");
    MB_TRY(cudaMemsetAsync(d->d_eos_flag, 0, batch * sizeof(int), s), "clear eos flags");
    MB_TRY(cudaMemsetAsync(d->d_frame_idx, 0, sizeof(int), s), "clear frame index");
    /* frame_advance rewrites the EOS rule for the next frame from min_frames; this entry
     * point restages it on every call, so park min_frames at 0 */
    MB_TRY(cudaMemsetAsync(d->d_min_frames, 0, sizeof(int), s), "clear min frames");
    if (run(d, batch, MODE_LOCAL, error, cap) != 0) return -1;
    unsigned long long *rng = (unsigned long long *)d->h_rows;
    MB_TRY(cudaMemcpyAsync(d->h_codes, d->d_codes, nt * sizeof(unsigned), cudaMemcpyDeviceToHost, s), "read codes");
    MB_TRY(cudaMemcpyAsync(d->h_tokens, d->d_tokens, nt * sizeof(unsigned), cudaMemcpyDeviceToHost, s), "read tokens");
    MB_TRY(cudaMemcpyAsync(d->h_ints, d->d_eos_flag, batch * sizeof(int), cudaMemcpyDeviceToHost, s), "read eos flags");
    MB_TRY(cudaMemcpyAsync(d->h_ints + d->max_batch, d->local.d_eos_sub, batch * sizeof(int), cudaMemcpyDeviceToHost, s), "read eos frames");
    MB_TRY(cudaMemcpyAsync(rng, d->local.d_rng, batch * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s), "read rng");
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if (check_status(d, error, cap) != 0) return -1;
    memcpy(codes_out, d->h_codes, nt * sizeof(unsigned));
    if (values != NULL) memcpy(values, d->h_tokens, nt * sizeof(unsigned));
    for (size_t b = 0; b < batch; ++b) {
        if (saw_eos != NULL) saw_eos[b] = d->h_ints[b] != 0;
        if (eos_frame != NULL) eos_frame[b] = d->h_ints[b] != 0 ? (long)d->h_ints[d->max_batch + b] : -1;
        if (samplers != NULL) samplers[b].rng_state = rng[b];
        d->slot_len[slots[b]] += 1u;
    }
    mb_clear_error(error, cap);
    return 0;
}

/* Continuous batching over the decoder's slots (the reference steps at most 16 requests
 * that all start together, src/graph.c:4046-4200, and its server never admits into a
 * running batch): requests wait in order, a free slot is filled before the next frame
 * (cross K/V made on the device), every live request advances one frame per step, and a
 * request leaves on EOS or at its frame limit, as slot_advance decides
 * (src/graph.c:3912-3913). */
int mynah_b200_decoder_serve(void *decoder, mynah_b200_request *requests, size_t count,
                             size_t *steps_out, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d == NULL || d->local.layers == 0 || (requests == NULL && count > 0)) {
        mb_set_error(error, cap, "serve: no local transformer attached, or bad arguments");
        return -1;
    }
    const size_t T = d->tables, lanes_max = d->slots < d->max_batch ? d->slots : d->max_batch;
    size_t *owner = (size_t *)malloc(lanes_max * sizeof(size_t));       /* request in slot s, or SIZE_MAX */
    unsigned *slot_ids = (unsigned *)malloc(lanes_max * sizeof(unsigned));
    unsigned *codes = (unsigned *)malloc(lanes_max * T * sizeof(unsigned));
    unsigned *next = (unsigned *)malloc(lanes_max * T * sizeof(unsigned));
    mynah_b200_sampler *sp = (mynah_b200_sampler *)malloc(lanes_max * sizeof(mynah_b200_sampler));
    int *saw = (int *)malloc(lanes_max * sizeof(int));
    int rc = 0;
    if (!owner || !slot_ids || !codes || !next || !sp || !saw) {
        mb_set_error(error, cap, "out of memory");
        rc = -1;
    }
    for (size_t i = 0; rc == 0 && i < count; ++i) {
        if (requests[i].memory == NULL || requests[i].start_codes == NULL || requests[i].codes == NULL ||
            requests[i].max_frames > d->capacity || requests[i].memory_length == 0 ||
            requests[i].memory_length > d->T) {
            mb_set_error(error, cap, "serve: a request lacks buffers, exceeds the cache capacity or has more text "
                                     "states than the decoder's memory_length");
            rc = -1;
        }
        requests[i].frames_done = 0;
        requests[i].eos_frame = -1;
        requests[i].admitted_at = 0;
    }
    for (size_t s = 0; rc == 0 && s < lanes_max; ++s) owner[s] = SIZE_MAX;
    size_t waiting = 0, live = 0, step = 0;
    while (rc == 0 && (waiting < count || live > 0)) {
        for (size_t s = 0; s < lanes_max && waiting < count && rc == 0; ++s) {
            if (owner[s] != SIZE_MAX) continue;
            mynah_b200_request *r = &requests[waiting];
            if (r->max_frames == 0) { ++waiting; --s; continue; }
            if (mynah_b200_decoder_slot_prefill(d, s, r->memory, r->memory_length, error, cap) != 0) { rc = -1; break; }
            owner[s] = waiting++;
            r->admitted_at = step;
            ++live;
        }
        if (rc != 0 || live == 0) break;
        size_t nb = 0;
        for (size_t s = 0; s < lanes_max; ++s) {
            if (owner[s] == SIZE_MAX) continue;
            mynah_b200_request *r = &requests[owner[s]];
            slot_ids[nb] = (unsigned)s;
            memcpy(codes + nb * T, r->frames_done == 0 ? r->start_codes : r->codes + (r->frames_done - 1u) * T,
                   T * sizeof(unsigned));
            sp[nb] = r->sampler;
            sp[nb].allow_eos = r->frames_done >= r->min_frames;
            ++nb;
        }
        if (mynah_b200_decoder_frame_batch_local(d, slot_ids, codes, sp, next, NULL, saw, NULL, nb, error, cap) != 0) {
            rc = -1;
            break;
        }
        for (size_t b = 0; b < nb; ++b) {
            const size_t s = slot_ids[b];
            mynah_b200_request *r = &requests[owner[s]];
            memcpy(r->codes + r->frames_done * T, next + b * T, T * sizeof(unsigned));
            r->sampler.rng_state = sp[b].rng_state;
            if (saw[b] && r->eos_frame < 0) r->eos_frame = (long)r->frames_done;
            r->frames_done += 1u;
            if (saw[b] || r->frames_done >= r->max_frames) {
                owner[s] = SIZE_MAX;
                --live;
            }
        }
        ++step;
    }
    free(owner); free(slot_ids); free(codes); free(next); free(sp); free(saw);
    if (steps_out != NULL) *steps_out = step;
    if (rc == 0) mb_clear_error(error, cap);
    return rc;
}

/* ----------------------------------------------------------------- profiling */
int mynah_b200_decoder_profile(void *decoder, int enable, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d == NULL) return -1;
    MB_TRY(cudaSetDevice(d->st->device), "cudaSetDevice");
    if (enable && d->prof_ev == NULL) {
        d->prof_ev = (cudaEvent_t *)calloc(2u * PROF_POOL, sizeof(cudaEvent_t));
        d->prof_cls = (int *)calloc(PROF_POOL, sizeof(int));
        if (d->prof_ev == NULL || d->prof_cls == NULL) {
            mb_set_error(error, cap, "out of memory");
            return -1;
        }
        for (size_t i = 0; i < 2u * PROF_POOL; ++i)
            MB_TRY(cudaEventCreate(&d->prof_ev[i]), "cudaEventCreate");
    }
    if (!enable) prof_drain(d);
    d->profiling = enable != 0;
    if (enable) {
        prof_drain(d);
        memset(d->prof_launches, 0, sizeof(d->prof_launches));
        memset(d->prof_ms, 0, sizeof(d->prof_ms));
    }
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_decoder_profile_read(void *decoder, unsigned long long *launches, double *ms,
                                    size_t n, char *error, size_t cap) {
    mb_decoder *d = (mb_decoder *)decoder;
    if (d == NULL || launches == NULL || ms == NULL) return -1;
    MB_TRY(cudaSetDevice(d->st->device), "cudaSetDevice");
    prof_drain(d);
    for (size_t i = 0; i < n && i < MYNAH_B200_PROFILE_CLASSES; ++i) {
        launches[i] = d->prof_launches[i];
        ms[i] = d->prof_ms[i];
    }
    mb_clear_error(error, cap);
    return 0;
}

const char *mynah_b200_profile_class_name(size_t cls) {
    return cls < MYNAH_B200_PROFILE_CLASSES ? prof_names[cls] : "";
}
