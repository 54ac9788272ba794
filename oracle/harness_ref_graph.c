/* Harness around the reference's own decoder step.  TEST INFRASTRUCTURE ONLY.
 *
 * This translation unit textually includes the reference's src/graph.c (from
 * the read-only reference checkout named by -I on the compile line) so that
 * its `static` decoder functions -- decoder_cache_init, decoder_step_batch,
 * decoder_run, embed_audio_frame -- can be driven on a synthetic safetensors
 * file without a model pack.  Nothing of the reference is copied here: the
 * wrappers below only marshal arguments.  The result is built into
 * oracle/_ref/ and is used to validate oracle/mynah_oracle.c and as the timed
 * CPU baseline.
 */
#include "graph.c"

#include <stdlib.h>

typedef struct {
    mynah_tts_model model;
} ref_model;

typedef struct {
    decoder_cache cache;
    size_t full_layers;
} ref_decoder;

#define REF_EXPORT __attribute__((visibility("default")))

/* Defined only in the build that binds the reference's CUDA device to libmynah_b200.so
 * (harness_ref_cuda.c); absent (NULL) in the CPU builds. */
extern int ref_backend_light_up(mynah_backend *backend) __attribute__((weak));

/* hidden_dim/layers fill mynah_tts_model_info the way model.json would
 * (src/mynah_tts.c:214-266); qtype is the enum of src/qmat.c:36
 * (0 f32, 1 int8, 2 int4, 3 f16). */
REF_EXPORT ref_model *ref_model_open(const char *safetensors_path, unsigned hidden_dim,
                                     unsigned layers, unsigned codebooks, unsigned stacking,
                                     unsigned codebook_size, unsigned vocab, unsigned eos_id,
                                     int qtype, char *error, size_t cap) {
    ref_model *r = (ref_model *)calloc(1, sizeof(*r));
    if (r == NULL) return NULL;
    r->model.info.hidden_dim = hidden_dim;
    r->model.info.decoder_layers = layers;
    r->model.info.codebook_count = codebooks;
    r->model.info.frame_stacking_factor = stacking;
    r->model.info.codebook_size = codebook_size;
    r->model.info.audio_vocab_size = vocab;
    r->model.info.audio_eos_id = eos_id;
    /* the B200 build opens the reference's CUDA device (device ordinal, weight format and
     * strictness come from the environment, as for mynah_backend_open in the application) */
    const mynah_tts_device device = ref_backend_light_up != NULL ? MYNAH_TTS_DEVICE_CUDA : MYNAH_TTS_DEVICE_CPU;
    if (mynah_weights_open(safetensors_path, &r->model.tts, error, cap) != 0 ||
        mynah_backend_open(device, &r->model.backend, error, cap) != 0) {
        free(r);
        return NULL;
    }
    if (ref_backend_light_up != NULL && ref_backend_light_up(r->model.backend) != 0) {
        snprintf(error, cap, "could not wire the resident-attention ops");
        free(r);
        return NULL;
    }
    r->model.qcache = mynah_qmat_cache_new(qtype);
    if (r->model.qcache == NULL) {
        free(r);
        return NULL;
    }
    return r;
}

REF_EXPORT void ref_model_close(ref_model *r) {
    if (r == NULL) return;
    mynah_qmat_cache_free(r->model.qcache);
    mynah_backend_close(r->model.backend);
    mynah_weights_close(r->model.tts);
    free(r);
}

REF_EXPORT int ref_num_threads(void) { return mynah_num_threads(); }

REF_EXPORT ref_decoder *ref_decoder_new(ref_model *r, const float *memory, size_t memory_length,
                                        size_t capacity, char *error, size_t cap) {
    ref_decoder *d = (ref_decoder *)calloc(1, sizeof(*d));
    if (d == NULL) return NULL;
    if (decoder_cache_init(&r->model, &d->cache, memory, memory_length, capacity, error, cap) != 0) {
        free(d);
        return NULL;
    }
    d->full_layers = d->cache.layers;
    return d;
}

REF_EXPORT void ref_decoder_free(ref_decoder *d) {
    if (d == NULL) return;
    decoder_cache_free(&d->cache);
    free(d);
}

REF_EXPORT size_t ref_decoder_length(const ref_decoder *d) { return d->cache.length; }
REF_EXPORT void ref_decoder_set_length(ref_decoder *d, size_t n) { d->cache.length = n; }
/* Run only the first n layers: per-layer hidden states without touching the
 * reference's arithmetic. */
REF_EXPORT void ref_decoder_set_layers(ref_decoder *d, size_t n) {
    d->cache.layers = n <= d->full_layers ? n : d->full_layers;
}
REF_EXPORT size_t ref_decoder_xattn_width(const ref_decoder *d) { return d->cache.xattn_width; }
REF_EXPORT float *ref_decoder_self_k(ref_decoder *d) { return d->cache.self_k; }
REF_EXPORT float *ref_decoder_self_v(ref_decoder *d) { return d->cache.self_v; }
REF_EXPORT float *ref_decoder_cross_k(ref_decoder *d) { return d->cache.cross_k; }
REF_EXPORT float *ref_decoder_cross_v(ref_decoder *d) { return d->cache.cross_v; }

/* inputs/outs are [batch][width] contiguous; the reference takes pointer
 * arrays (src/graph.c:3127-3131). */
REF_EXPORT int ref_decoder_step_batch(ref_model *r, ref_decoder **decoders, const float *inputs,
                                      float *outs, size_t batch, char *error, size_t cap) {
    if (batch == 0u || batch > MYNAH_MAX_BATCH) return -1;
    const size_t width = r->model.info.hidden_dim;
    decoder_cache *caches[MYNAH_MAX_BATCH];
    const float *in[MYNAH_MAX_BATCH];
    float *out[MYNAH_MAX_BATCH];
    for (size_t b = 0; b < batch; ++b) {
        caches[b] = &decoders[b]->cache;
        in[b] = inputs + b * width;
        out[b] = outs + b * width;
    }
    batch_scratch scratch;
    if (batch_scratch_init(&scratch, batch, caches[0]->ffn_width, error, cap) != 0) return -1;
    const int rc = decoder_step_batch(&r->model, caches, in, out, batch,
                                      batch > 1u ? &scratch : NULL, error, cap);
    batch_scratch_free(&scratch);
    return rc;
}

REF_EXPORT int ref_decoder_run(ref_model *r, ref_decoder *d, const float *rows, size_t count,
                               float *out_last, char *error, size_t cap) {
    return decoder_run(&r->model, &d->cache, rows, count, out_last, NULL, error, cap);
}

/* 1 when decoder_run's resident path (src/graph.c:3363-3368) is open for this model. */
REF_EXPORT int ref_model_resident(const ref_model *r) {
    return mynah_backend_has_dev_ops(r->model.backend) && mynah_backend_has_attention_dev(r->model.backend);
}
REF_EXPORT const char *ref_model_backend_name(const ref_model *r) { return mynah_backend_name(r->model.backend); }

/* The resident path keeps the self K/V on the device (src/graph.c:2901-2961): copy rows
 * [0, length) of every layer back into the host cache so a test can read them.  Returns -1
 * when the cache has no device copy. */
REF_EXPORT int ref_decoder_download_kv(ref_model *r, ref_decoder *d, char *error, size_t cap) {
    decoder_cache *c = &d->cache;
    if (!c->dev_attention_allocated) return -1;
    if (mynah_backend_sync(r->model.backend, error, cap) != 0) return -1;
    for (size_t layer = 0; layer < c->layers; ++layer) {
        const size_t off = layer * c->capacity * c->width;
        if (c->length > 0 &&
            (mynah_backend_d2h(r->model.backend, c->dev_self_k + off, c->self_k + off, c->length * c->width, error, cap) != 0 ||
             mynah_backend_d2h(r->model.backend, c->dev_self_v + off, c->self_v + off, c->length * c->width, error, cap) != 0))
            return -1;
    }
    return 0;
}

/* codes are [codebooks][code_stride] as in src/graph.c:760-766. */
REF_EXPORT int ref_embed_audio_frame(ref_model *r, const unsigned *codes, size_t code_stride,
                                     size_t frame, float *row, char *error, size_t cap) {
    return embed_audio_frame(&r->model, codes, code_stride, frame, row, error, cap);
}

/* Logit heads in the form of src/graph.c:1538-1566: the per-stream projection
 * `local_transformer_out_projections.N.{weight,bias}` through the quantized
 * linear, then the masked first-on-ties pick.  The mask-and-pick loop is
 * restated here because the reference has it inline in a larger function. */
REF_EXPORT int ref_heads_argmax(ref_model *r, const float *hidden, size_t streams, int allow_eos,
                                unsigned *tokens, float *logits_out, char *error, size_t cap) {
    const size_t width = r->model.info.hidden_dim;
    const size_t vocab = r->model.info.audio_vocab_size;
    const size_t codebook_size = r->model.info.codebook_size;
    const unsigned eos_id = r->model.info.audio_eos_id;
    float *logits = (float *)malloc(vocab * sizeof(float));
    if (logits == NULL) return -1;
    for (size_t stream = 0; stream < streams; ++stream) {
        char name[128];
        mynah_tensor weight, bias;
        snprintf(name, sizeof(name), "local_transformer_out_projections.%zu.bias", stream);
        if (tensor(r->model.tts, name, &bias, error, cap) != 0) { free(logits); return -1; }
        snprintf(name, sizeof(name), "local_transformer_out_projections.%zu.weight", stream);
        if (tensor(r->model.tts, name, &weight, error, cap) != 0) { free(logits); return -1; }
        if (mynah_qmat_linear_resolved(r->model.qcache, r->model.backend, name, weight.data,
                                       hidden, logits, 1u, width, vocab, bias.data,
                                       error, cap) != 0) { free(logits); return -1; }
        float best = -FLT_MAX;
        unsigned argmax = 0;
        for (size_t candidate = 0; candidate < vocab; ++candidate) {
            const int is_code = candidate < codebook_size;
            const int is_eos = candidate == eos_id;
            if (!is_code && !(is_eos && allow_eos)) continue;
            if (logits[candidate] > best) {
                best = logits[candidate];
                argmax = (unsigned)candidate;
            }
        }
        tokens[stream] = argmax;
        if (logits_out != NULL) memcpy(logits_out + stream * vocab, logits, vocab * sizeof(float));
    }
    free(logits);
    return 0;
}

/* Greedy frames for `batch` requests stepped together (<= 16, the reference's
 * cap): embed each request's stored codes, one decoder_step_batch, heads per
 * request.  codes is [batch][streams] with stream = fs * codebooks + codebook;
 * tokens_out is [frames][batch][streams].  Every request runs all frames (EOS
 * allowed from min_frames on is reported in eos_frame[b], first occurrence,
 * else -1) so the timing is a fixed amount of work. */
REF_EXPORT int ref_greedy_decode(ref_model *r, ref_decoder **decoders, size_t batch,
                                 unsigned *codes, size_t frames, size_t min_frames,
                                 unsigned *tokens_out, long *eos_frame, char *error, size_t cap) {
    const size_t width = r->model.info.hidden_dim;
    const size_t codebooks = r->model.info.codebook_count;
    const size_t stacking = r->model.info.frame_stacking_factor;
    const size_t streams = codebooks * stacking;
    const unsigned eos_id = r->model.info.audio_eos_id;
    if (batch == 0u || batch > MYNAH_MAX_BATCH) return -1;
    float *rows = (float *)malloc(2u * batch * width * sizeof(float));
    unsigned *frame_codes = (unsigned *)malloc(streams * sizeof(unsigned));
    if (rows == NULL || frame_codes == NULL) { free(rows); free(frame_codes); return -1; }
    float *hidden = rows + batch * width;
    int rc = 0;
    for (size_t b = 0; b < batch; ++b) eos_frame[b] = -1;
    for (size_t f = 0; f < frames && rc == 0; ++f) {
        for (size_t b = 0; b < batch && rc == 0; ++b) {
            /* embed_audio_frame reads codes[codebook * stride + frame * stacking + fs] */
            for (size_t fs = 0; fs < stacking; ++fs)
                for (size_t c = 0; c < codebooks; ++c)
                    frame_codes[c * stacking + fs] = codes[b * streams + fs * codebooks + c];
            rc = embed_audio_frame(&r->model, frame_codes, stacking, 0u, rows + b * width, error, cap);
        }
        if (rc == 0) rc = ref_decoder_step_batch(r, decoders, rows, hidden, batch, error, cap);
        for (size_t b = 0; b < batch && rc == 0; ++b) {
            unsigned *tok = tokens_out + (f * batch + b) * streams;
            rc = ref_heads_argmax(r, hidden + b * width, streams, f >= min_frames, tok, NULL, error, cap);
            for (size_t s = 0; s < streams && rc == 0; ++s) {
                if (tok[s] == eos_id && eos_frame[b] < 0) eos_frame[b] = (long)f;
                codes[b * streams + s] = tok[s] < r->model.info.codebook_size ? tok[s] : 0u;
            }
        }
    }
    free(rows);
    free(frame_codes);
    return rc;
}

/* encode_text (src/graph.c:709-748) on the model's "encoder" tensors; encoder_layers and
 * text_max_length stand for the manifest fields of src/mynah_tts.c:228-233.  out is
 * [count][hidden_dim]. */
REF_EXPORT int ref_encode_text(ref_model *r, unsigned encoder_layers, unsigned text_max_length,
                               const int *ids, size_t count, float *out, char *error, size_t cap) {
    r->model.info.encoder_layers = encoder_layers;
    r->model.info.text_max_length = text_max_length;
    float *encoded = NULL;
    if (cap > 0) error[0] = '\0';
    if (encode_text(&r->model, ids, count, &encoded, error, cap) != 0) return -1;
    memcpy(out, encoded, count * r->model.info.hidden_dim * sizeof(float));
    free(encoded);
    return 0;
}

/* decode_codec (src/graph.c:2640-2780) over codec tensors that live in the same synthetic
 * file as the rest (the reference keeps them in a second file, model->codec).  codes are
 * [8][raw_length]; out receives raw_length * 1024 samples.  Returns the count or -1. */
REF_EXPORT long ref_decode_codec(ref_model *r, const unsigned *codes, size_t raw_length, float *out,
                                 char *error, size_t cap) {
    if (r->model.codec == NULL) r->model.codec = r->model.tts;
    float *samples = NULL;
    size_t count = 0;
    if (cap > 0) error[0] = '\0';
    if (decode_codec(&r->model, codes, raw_length, &samples, &count, error, cap) != 0) return -1;
    memcpy(out, samples, count * sizeof(float));
    free(samples);
    return (long)count;
}

/* ------------------------------------------------------ local transformer */
typedef struct {
    local_frame_state state;
} ref_local;

/* model.json's local_transformer_layers (src/mynah_tts.c:230-231). */
REF_EXPORT void ref_model_set_local_layers(ref_model *r, unsigned layers) {
    r->model.info.local_transformer_layers = layers;
}

REF_EXPORT ref_local *ref_local_new(ref_model *r, size_t top_count, char *error, size_t cap) {
    ref_local *l = (ref_local *)calloc(1, sizeof(*l));
    if (l == NULL) return NULL;
    if (local_frame_state_init(&r->model, &l->state, top_count, error, cap) != 0) {
        free(l);
        return NULL;
    }
    return l;
}

REF_EXPORT void ref_local_free(ref_local *l) {
    if (l == NULL) return;
    local_frame_state_free(&l->state);
    free(l);
}

REF_EXPORT size_t ref_local_length(const ref_local *l) { return l->state.cache.length; }
REF_EXPORT void ref_local_set_length(ref_local *l, size_t n) { l->state.cache.length = n; }
REF_EXPORT float *ref_local_k(ref_local *l) { return l->state.cache.k; }
REF_EXPORT float *ref_local_v(ref_local *l) { return l->state.cache.v; }
REF_EXPORT size_t ref_local_capacity(const ref_local *l) { return l->state.cache.capacity; }

/* inputs/outs are [batch][width] contiguous (src/graph.c:1234-1238 takes
 * pointer arrays). */
REF_EXPORT int ref_local_step_batch(ref_model *r, ref_local **locals, const float *inputs,
                                    float *outs, size_t batch, char *error, size_t cap) {
    if (batch == 0u || batch > MYNAH_MAX_BATCH) return -1;
    const size_t width = r->model.info.hidden_dim;
    local_cache *caches[MYNAH_MAX_BATCH];
    local_workspace *workspaces[MYNAH_MAX_BATCH];
    const float *in[MYNAH_MAX_BATCH];
    float *out[MYNAH_MAX_BATCH];
    for (size_t b = 0; b < batch; ++b) {
        caches[b] = &locals[b]->state.cache;
        workspaces[b] = &locals[b]->state.workspace;
        in[b] = inputs + b * width;
        out[b] = outs + b * width;
    }
    batch_scratch scratch;
    if (batch_scratch_init(&scratch, batch, caches[0]->ffn_width, error, cap) != 0) return -1;
    const int rc = local_step_batch(&r->model, caches, workspaces, in, out, batch,
                                    batch > 1u ? &scratch : NULL, error, cap);
    batch_scratch_free(&scratch);
    return rc;
}

/* One stacked frame for `batch` requests through sample_local_frame_batch
 * (src/graph.c:1374-1656).  decoder_last is [batch][width]; rng_states are
 * updated in place; allow_eos[b] == 0 forbids EOS the way a request below its
 * minimum length does.  codes_out is [batch][streams] with stream =
 * fs * codebooks + codebook (the reference writes codes[codebook * stride +
 * offset + fs]); saw_eos/eos_frame as the reference reports them (-1: none). */
REF_EXPORT int ref_local_frame(ref_model *r, ref_local **locals, size_t batch,
                               const float *decoder_last, const float *temperature,
                               const unsigned *topk, uint64_t *rng_states, const int *allow_eos,
                               unsigned *codes_out, int *saw_eos, long *eos_frame,
                               char *error, size_t cap) {
    if (batch == 0u || batch > MYNAH_MAX_BATCH) return -1;
    const size_t width = r->model.info.hidden_dim;
    const size_t codebooks = r->model.info.codebook_count;
    const size_t stacking = r->model.info.frame_stacking_factor;
    const size_t streams = codebooks * stacking;
    local_batch_item items[MYNAH_MAX_BATCH];
    unsigned *scratch_codes = (unsigned *)calloc(batch * streams, sizeof(unsigned));
    if (scratch_codes == NULL) return -1;
    for (size_t b = 0; b < batch; ++b) {
        local_batch_item *it = &items[b];
        memset(it, 0, sizeof(*it));
        it->state = &locals[b]->state;
        it->decoder_last = decoder_last + b * width;
        it->codes = scratch_codes + b * streams;   /* [codebooks][stacking] */
        it->raw_offset = 0u;
        it->code_stride = stacking;
        it->generated_raw_length = allow_eos[b] ? 1u : 0u;
        it->min_raw_length = 1u;
        it->temperature = temperature[b];
        it->topk = topk[b];
        it->rng_state = &rng_states[b];
    }
    batch_scratch scratch;
    if (batch_scratch_init(&scratch, batch, locals[0]->state.cache.ffn_width, error, cap) != 0) {
        free(scratch_codes);
        return -1;
    }
    const int rc = sample_local_frame_batch(&r->model, items, batch, batch > 1u ? &scratch : NULL,
                                            error, cap);
    batch_scratch_free(&scratch);
    for (size_t b = 0; b < batch && rc == 0; ++b) {
        for (size_t fs = 0; fs < stacking; ++fs)
            for (size_t c = 0; c < codebooks; ++c)
                codes_out[b * streams + fs * codebooks + c] = scratch_codes[b * streams + c * stacking + fs];
        saw_eos[b] = items[b].saw_eos;
        eos_frame[b] = items[b].eos_frame == SIZE_MAX ? -1 : (long)items[b].eos_frame;
    }
    free(scratch_codes);
    return rc;
}
