/* The backend seam of mynah-tts (src/backend.h) on one B200, C11.
 *
 * Exports the symbols src/backend.c binds for its CUDA device
 * (src/backend.c:105-135) plus the resident-attention entries it wires only
 * for Metal (src/backend.c:404-428).  Device work is enqueued on one stream;
 * like the reference's CUDA file, only the host-buffer entry points
 * synchronize.  Weight quantization lives behind the seam: a weight is packed
 * on first use in the format chosen at open time and cached by its host
 * pointer, the contract of cached_weight_fp16 in the reference
 * (gpu/cuda/backend_cuda.cu:205-219).
 */
#include "host_common.h"
#include "../../include/mynah_b200.h"

#include <math.h>
#include <pthread.h>
#include <unistd.h>
#include <stdlib.h>
#include <string.h>

#define QMAT_SMALL_COUNT 16u /* src/qmat.c:32 */
#define QMAT_K_MAX 8192u     /* src/qmat.c:33 */

static int use_device(const mb_state *st, char *error, size_t cap) {
    return mb_cuda((int)cudaSetDevice(st->device), "cudaSetDevice", error, cap);
}

/* ------------------------------------------------------------ weight cache */
void mb_weight_release(mb_dev_weight *w) {
    if (w == NULL) return;
    cudaFree(w->w);
    cudaFree(w->scales);
    memset(w, 0, sizeof(*w));
}

int mb_weight_build(mb_state *st, const float *host_w, size_t n, size_t k, int qtype,
                    mb_dev_weight *out, char *error, size_t cap) {
    memset(out, 0, sizeof(*out));
    if (host_w == NULL || n == 0 || k == 0) {
        mb_set_error(error, cap, "invalid weight shape");
        return -1;
    }
    if (qtype == MB_INT4 && (k % 32u) != 0) qtype = MB_F32; /* src/qmat.c:630 */
    float *raw = NULL;
    MB_TRY(cudaMalloc((void **)&raw, n * k * sizeof(float)), "cudaMalloc(weight)");
    if (mb_cuda((int)cudaMemcpyAsync(raw, host_w, n * k * sizeof(float), cudaMemcpyHostToDevice,
                                     st->stream), "upload weight", error, cap) != 0) {
        cudaFree(raw);
        return -1;
    }
    out->host = host_w;
    out->n = n;
    out->k = k;
    out->qtype = qtype;
    int rc = 0;
    if (qtype == MB_F32) {
        out->w = raw;
        out->bytes = n * k * sizeof(float);
        raw = NULL;
    } else if (qtype == MB_INT8) {
        rc = (int)cudaMalloc(&out->w, n * k);
        if (rc == 0) rc = (int)cudaMalloc((void **)&out->scales, n * sizeof(float));
        if (rc == 0) rc = mb_pack_int8(raw, n, k, (int8_t *)out->w, out->scales, st->stream);
        out->bytes = n * k + n * sizeof(float);
    } else if (qtype == MB_INT4) {
        rc = (int)cudaMalloc(&out->w, n * (k / 2u));
        if (rc == 0) rc = (int)cudaMalloc((void **)&out->scales, n * (k / 32u) * sizeof(float));
        if (rc == 0) rc = mb_pack_int4(raw, n, k, (uint8_t *)out->w, out->scales, st->stream);
        out->bytes = n * (k / 2u) + n * (k / 32u) * sizeof(float);
    } else if (qtype == MB_F16) {
        rc = (int)cudaMalloc(&out->w, n * k * 2u);
        if (rc == 0) rc = mb_pack_f16(raw, n * k, (uint16_t *)out->w, st->stream);
        out->bytes = n * k * 2u;
    } else {
        rc = (int)cudaErrorInvalidValue;
    }
    st->launches += qtype == MB_F32 ? 0u : 1u;
    if (rc == 0) rc = (int)cudaStreamSynchronize(st->stream);
    cudaFree(raw);
    if (rc != 0) {
        mb_weight_release(out);
        return mb_cuda(rc, "pack weight", error, cap);
    }
    return 0;
}

int mb_weight_cached(mb_state *st, const float *host_w, size_t n, size_t k, int qtype,
                     const mb_dev_weight **out, char *error, size_t cap) {
    if (qtype == MB_INT4 && (k % 32u) != 0) qtype = MB_F32;
    for (size_t i = 0; i < st->weight_count; ++i) {
        const mb_dev_weight *w = &st->weights[i];
        if (w->host == host_w && w->n == n && w->k == k && w->qtype == qtype) {
            *out = w;
            return 0;
        }
    }
    if (st->weight_count == st->weight_cap) {
        const size_t next = st->weight_cap == 0 ? 64u : st->weight_cap * 2u;
        mb_dev_weight *grown = (mb_dev_weight *)realloc(st->weights, next * sizeof(*grown));
        if (grown == NULL) {
            mb_set_error(error, cap, "out of memory growing the weight cache");
            return -1;
        }
        st->weights = grown;
        st->weight_cap = next;
    }
    if (mb_weight_build(st, host_w, n, k, qtype, &st->weights[st->weight_count], error, cap) != 0)
        return -1;
    *out = &st->weights[st->weight_count++];
    return 0;
}

int mb_vector_cached(mb_state *st, const float *host_v, size_t n, const float **out, char *error,
                     size_t cap) {
    if (host_v == NULL) {
        *out = NULL;
        return 0;
    }
    for (size_t i = 0; i < st->vector_count; ++i) {
        if (st->vectors[i].host == host_v && st->vectors[i].n == n) {
            *out = st->vectors[i].dev;
            return 0;
        }
    }
    if (st->vector_count == st->vector_cap) {
        const size_t next = st->vector_cap == 0 ? 64u : st->vector_cap * 2u;
        mb_dev_vector *grown = (mb_dev_vector *)realloc(st->vectors, next * sizeof(*grown));
        if (grown == NULL) {
            mb_set_error(error, cap, "out of memory growing the vector cache");
            return -1;
        }
        st->vectors = grown;
        st->vector_cap = next;
    }
    float *dev = NULL;
    MB_TRY(cudaMalloc((void **)&dev, n * sizeof(float)), "cudaMalloc(vector)");
    if (mb_cuda((int)cudaMemcpy(dev, host_v, n * sizeof(float), cudaMemcpyHostToDevice),
                "upload vector", error, cap) != 0) {
        cudaFree(dev);
        return -1;
    }
    st->vectors[st->vector_count].host = host_v;
    st->vectors[st->vector_count].n = n;
    st->vectors[st->vector_count].dev = dev;
    st->vector_count++;
    *out = dev;
    return 0;
}

void mb_gemv_bind_weight(mb_gemv_args *g, const mb_dev_weight *w, const float *dev_bias) {
    g->qtype = w->qtype;
    g->w = w->w;
    g->scales = w->scales;
    g->bias = dev_bias;
    g->n = w->n;
    g->k = w->k;
}

/* --------------------------------------------------------------- scratch */
static int grow(void **ptr, size_t *have, size_t want, size_t elem, char *error, size_t cap) {
    if (*have >= want) return 0;
    if (*ptr != NULL) cudaFree(*ptr);
    *ptr = NULL;
    *have = 0;
    const size_t round = (want + 4095u) & ~(size_t)4095u;
    MB_TRY(cudaMalloc(ptr, round * elem), "cudaMalloc(scratch)");
    *have = round;
    return 0;
}

/* ------------------------------------------------------- libm parity tables */
/* Tables are per device and shared by every backend opened on it in this
 * process; they live until the process exits. */
#define LIBM_MAX_DEVICES 16
#define TANH_LO_BITS 0x32800000u /* must match libm_parity.cuh */
#define TANH_HI_BITS 0x41800000u
#define EXP_LO_BITS 0x38000000u
#define EXP_HI_BITS 0x43800000u
#define SIN_LO_BITS 0x39800000u
#define SIN_HI_BITS 0x42800000u
static struct { mb_libm_tables tables; int state; /* 0 none, 1 exact, -1 failed */ } g_libm[LIBM_MAX_DEVICES];
static pthread_mutex_t g_libm_lock = PTHREAD_MUTEX_INITIALIZER;

typedef struct { float *out; uint32_t first_bits; size_t begin, end; int kind; /* 0 tanhf, 1 expf(-a), 2 sinf */ } libm_job;

static void *libm_worker(void *arg) {
    const libm_job *j = (const libm_job *)arg;
    for (size_t i = j->begin; i < j->end; ++i) {
        const uint32_t bits = j->first_bits + (uint32_t)i;
        float a;
        memcpy(&a, &bits, sizeof(a));
        j->out[i] = j->kind == 1 ? expf(-a) : j->kind == 2 ? sinf(a) : tanhf(a);   /* the HOST libm, which the reference links */
    }
    return NULL;
}

static int build_libm_table(mb_state *st, int kind, uint32_t lo, uint32_t hi, uint32_t **table_out,
                            char *error, size_t cap) {
    enum { RUN = 1 << 23, MAX_THREADS = 64 };
    const size_t total = (size_t)(hi - lo);
    uint32_t *table = NULL;
    float *host = (float *)malloc((size_t)RUN * sizeof(float));
    float *dev = NULL;
    int *status = st->d_status;
    if (host == NULL) {
        mb_set_error(error, cap, "out of memory building libm tables");
        return -1;
    }
    int rc = (int)cudaMalloc((void **)&table, total / 8u * sizeof(uint32_t));
    if (rc == 0) rc = (int)cudaMalloc((void **)&dev, (size_t)RUN * sizeof(float));
    long ncpu = sysconf(_SC_NPROCESSORS_ONLN);
    size_t threads = ncpu < 1 ? 1u : (ncpu > MAX_THREADS ? MAX_THREADS : (size_t)ncpu);
    for (size_t off = 0; off < total && rc == 0; off += RUN) {
        const size_t count = total - off < RUN ? total - off : RUN;
        pthread_t tid[MAX_THREADS];
        libm_job jobs[MAX_THREADS];
        size_t started = 0;
        for (size_t t = 0; t < threads; ++t) {
            jobs[t].out = host;
            jobs[t].first_bits = lo + (uint32_t)off;
            jobs[t].begin = count * t / threads;
            jobs[t].end = count * (t + 1) / threads;
            jobs[t].kind = kind;
            if (t + 1 == threads || pthread_create(&tid[t], NULL, libm_worker, &jobs[t]) != 0) {
                jobs[t].end = count;           /* this thread takes the rest */
                libm_worker(&jobs[t]);
                break;
            }
            ++started;
        }
        for (size_t t = 0; t < started; ++t) pthread_join(tid[t], NULL);
        rc = (int)cudaMemcpyAsync(dev, host, count * sizeof(float), cudaMemcpyHostToDevice, st->stream);
        if (rc == 0) rc = mb_libm_delta(dev, lo + (uint32_t)off, count, kind, table + off / 8u, status, st->stream);
        if (rc == 0) rc = (int)cudaStreamSynchronize(st->stream);   /* host buffer is reused */
        st->launches += 1;
    }
    int flags = 0;
    if (rc == 0) rc = (int)cudaMemcpy(&flags, status, sizeof(int), cudaMemcpyDeviceToHost);
    free(host);
    cudaFree(dev);
    if (rc != 0 || (flags & 4) != 0) {
        cudaFree(table);
        if (rc == 0) cudaMemset(status, 0, sizeof(int));
        if (rc != 0) return mb_cuda(rc, "build libm tables", error, cap);
        mb_set_error(error, cap, "host libm differs from the device by more than the tables can express");
        return -1;
    }
    *table_out = table;
    return 0;
}

static void libm_tables_for(mb_state *st) {
    if (st->device < 0 || st->device >= LIBM_MAX_DEVICES) return;
    pthread_mutex_lock(&g_libm_lock);
    if (g_libm[st->device].state == 0) {
        char msg[128];
        uint32_t *tt = NULL, *et = NULL;
        if (build_libm_table(st, 0, TANH_LO_BITS, TANH_HI_BITS, &tt, msg, sizeof(msg)) == 0 &&
            build_libm_table(st, 1, EXP_LO_BITS, EXP_HI_BITS, &et, msg, sizeof(msg)) == 0) {
            g_libm[st->device].tables.tanh_tab = tt;
            g_libm[st->device].tables.exp_tab = et;
            g_libm[st->device].state = 1;
        } else {
            cudaFree(tt);
            g_libm[st->device].state = -1;
        }
    }
    if (g_libm[st->device].state == 1) {
        st->libm = g_libm[st->device].tables;
        st->libm_exact = 1;
    }
    pthread_mutex_unlock(&g_libm_lock);
}

/* The sinf table (the codec's Snake activation), built on first use by a reference-order
 * codec: backends that never decode audio that way do not pay its 76 MB.  Returns NULL when
 * the tables are switched off or the build failed (the codec then uses the correctly rounded
 * value). */
const uint32_t *mb_libm_sin_table(mb_state *st) {
    if (st->device < 0 || st->device >= LIBM_MAX_DEVICES) return NULL;
    const char *env = getenv("MYNAH_B200_LIBM_TABLES");
    if (env != NULL && strcmp(env, "0") == 0) return NULL;
    pthread_mutex_lock(&g_libm_lock);
    static int tried[LIBM_MAX_DEVICES];
    if (g_libm[st->device].tables.sin_tab == NULL && !tried[st->device]) {
        char msg[128];
        uint32_t *tab = NULL;
        tried[st->device] = 1;
        if (build_libm_table(st, 2, SIN_LO_BITS, SIN_HI_BITS, &tab, msg, sizeof(msg)) == 0)
            g_libm[st->device].tables.sin_tab = tab;
    }
    st->libm.sin_tab = g_libm[st->device].tables.sin_tab;
    pthread_mutex_unlock(&g_libm_lock);
    return st->libm.sin_tab;
}

/* 1 when strict mode reproduces the host libm's expf/tanhf bit for bit. */
int mynah_b200_libm_exact(const void *state) {
    return state == NULL ? 0 : ((const mb_state *)state)->libm_exact;
}

/* ------------------------------------------------------------ open / close */
int mynah_b200_open(void **state, int device, int quant, int strict, char *error, size_t cap) {
    if (state == NULL) {
        mb_set_error(error, cap, "invalid backend state pointer");
        return -1;
    }
    *state = NULL;
    if (quant != MB_F32 && quant != MB_INT8 && quant != MB_INT4 && quant != MB_F16) {
        mb_set_error(error, cap, "unknown weight format");
        return -1;
    }
    int count = 0;
    MB_TRY(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (device < 0 || device >= count) {
        mb_set_error(error, cap, "CUDA device ordinal out of range");
        return -1;
    }
    MB_TRY(cudaSetDevice(device), "cudaSetDevice");
    int major = 0, minor = 0, sms = 0;
    MB_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device), "device attribute");
    MB_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device), "device attribute");
    MB_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "device attribute");
    if (major != 10) {
        if (error != NULL && cap > 0)
            snprintf(error, cap, "this library holds sm_100a code only; device %d is sm_%d%d",
                     device, major, minor);
        return -1;
    }
    mb_state *st = (mb_state *)calloc(1, sizeof(*st));
    if (st == NULL) {
        mb_set_error(error, cap, "out of memory creating backend");
        return -1;
    }
    st->device = device;
    st->quant = quant;
    st->strict = strict != 0;
    st->sm_count = sms;
    if (mb_cuda((int)cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking),
                "cudaStreamCreate", error, cap) != 0 ||
        mb_cuda(mb_gemv_init(), "kernel attributes (gemv)", error, cap) != 0 ||
        mb_cuda(mb_attention_init(), "kernel attributes (attention)", error, cap) != 0 ||
        mb_cuda(mb_gemm_tc_init(), "kernel attributes (tensor-core product)", error, cap) != 0 ||
        mb_cuda(mb_gemm_tc_f16_init(), "kernel attributes (f16 tensor-core product)", error, cap) != 0 ||
        mb_cuda(mb_cross_block_init(), "kernel attributes (cross-attention block)", error, cap) != 0 ||
        mb_cuda(mb_codec_tc_init(), "kernel attributes (codec tensor-core convolution)", error, cap) != 0 ||
        mb_cuda((int)cudaMalloc((void **)&st->d_token, sizeof(unsigned)), "cudaMalloc", error, cap) != 0 ||
        mb_cuda((int)cudaMalloc((void **)&st->d_status, sizeof(int)), "cudaMalloc", error, cap) != 0 ||
        mb_cuda((int)cudaMemset(st->d_status, 0, sizeof(int)), "cudaMemset", error, cap) != 0) {
        mynah_b200_close(st);
        return -1;
    }
    st->own_stream = 1;
    if (st->strict) {
        const char *env = getenv("MYNAH_B200_LIBM_TABLES");
        if (env == NULL || strcmp(env, "0") != 0) libm_tables_for(st);
    }
    *state = st;
    mb_clear_error(error, cap);
    return 0;
}

void mynah_b200_close(void *state) {
    mb_state *st = (mb_state *)state;
    if (st == NULL) return;
    cudaSetDevice(st->device);
    if (st->stream != NULL) cudaStreamSynchronize(st->stream);
    for (size_t i = 0; i < st->weight_count; ++i) mb_weight_release(&st->weights[i]);
    for (size_t i = 0; i < st->vector_count; ++i) cudaFree(st->vectors[i].dev);
    free(st->weights);
    free(st->vectors);
    cudaFree(st->d_in);
    cudaFree(st->d_out);
    cudaFree(st->d_qx);
    cudaFree(st->d_sx);
    cudaFree(st->d_partials);
    cudaFree(st->d_counters);
    cudaFree(st->d_token);
    cudaFree(st->d_status);
    if (st->timer0 != NULL) cudaEventDestroy(st->timer0);
    if (st->timer1 != NULL) cudaEventDestroy(st->timer1);
    if (st->own_stream && st->stream != NULL) cudaStreamDestroy(st->stream);
    free(st);
}

int mynah_b200_set_stream(void *state, void *cuda_stream, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    if (st->own_stream) cudaStreamDestroy(st->stream);
    st->stream = (cudaStream_t)cuda_stream;
    st->own_stream = 0;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_quant(const void *state) { return state == NULL ? -1 : ((const mb_state *)state)->quant; }
int mynah_b200_strict(const void *state) { return state == NULL ? -1 : ((const mb_state *)state)->strict; }
unsigned long long mynah_b200_launch_count(const void *state) {
    return state == NULL ? 0ull : ((const mb_state *)state)->launches;
}

/* Device-time stopwatch on the backend's stream (two CUDA events). */
int mynah_b200_timer_start(void *state, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    if (st->timer0 == NULL) {
        MB_TRY(cudaEventCreate(&st->timer0), "cudaEventCreate");
        MB_TRY(cudaEventCreate(&st->timer1), "cudaEventCreate");
    }
    MB_TRY(cudaEventRecord(st->timer0, st->stream), "cudaEventRecord");
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_timer_stop(void *state, float *elapsed_ms, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || elapsed_ms == NULL || st->timer0 == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaEventRecord(st->timer1, st->stream), "cudaEventRecord");
    MB_TRY(cudaEventSynchronize(st->timer1), "cudaEventSynchronize");
    MB_TRY(cudaEventElapsedTime(elapsed_ms, st->timer0, st->timer1), "cudaEventElapsedTime");
    mb_clear_error(error, cap);
    return 0;
}

/* --------------------------------------------------------- product dispatch */
/* out[rows,ow] = in[rows,iw] W^T + bias with device activations.  The
 * quantized/f32 routing is mynah_qmat_linear_resolved's (src/qmat.c:773-788). */
static int product_dev(mb_state *st, const float *dev_in, float *dev_out, size_t rows, size_t iw,
                       size_t ow, const float *weight, const float *bias, char *error, size_t cap) {
    if (st == NULL || dev_in == NULL || dev_out == NULL || weight == NULL || rows == 0 ||
        iw == 0 || ow == 0) {
        mb_set_error(error, cap, "invalid backend matmul request");
        return -1;
    }
    if (use_device(st, error, cap) != 0) return -1;
    const int use_q = st->quant != MB_F32 && rows <= QMAT_SMALL_COUNT && iw <= QMAT_K_MAX;
    const mb_dev_weight *w = NULL;
    const float *dbias = NULL;
    if (mb_weight_cached(st, weight, ow, iw, use_q ? st->quant : MB_F32, &w, error, cap) != 0 ||
        mb_vector_cached(st, bias, ow, &dbias, error, cap) != 0)
        return -1;
    if (w->qtype == MB_F32 && rows > QMAT_SMALL_COUNT) {
        MB_TRY(mb_sgemm(0, 1, rows, ow, iw, 1.0f, dev_in, iw, (const float *)w->w, iw, 0.0f,
                        dev_out, ow, st->stream), "sgemm");
        st->launches += 1;
        if (dbias != NULL) {
            MB_TRY(mb_bias_add(dev_out, dbias, rows, ow, st->stream), "bias add");
            st->launches += 1;
        }
        mb_clear_error(error, cap);
        return 0;
    }
    mb_gemv_args g;
    memset(&g, 0, sizeof(g));
    mb_gemv_bind_weight(&g, w, dbias);
    g.out = dev_out;
    g.out_stride = ow;
    g.batch = rows;
    g.epilogue = MB_EPI_STORE;
    g.strict = st->strict;
    g.tanh_tab = st->libm.tanh_tab;
    if (w->qtype == MB_INT8 || w->qtype == MB_INT4) {
        if (grow((void **)&st->d_qx, &st->d_qx_cap, rows * iw, 1, error, cap) != 0 ||
            grow((void **)&st->d_sx, &st->d_sx_cap, rows, sizeof(float), error, cap) != 0)
            return -1;
        MB_TRY(mb_quant_rows(dev_in, rows, iw, st->d_qx, st->d_sx, NULL, st->stream),
               "activation quantization");
        st->launches += 1;
        g.qx = st->d_qx;
        g.sx = st->d_sx;
    } else {
        g.x = dev_in;
    }
    MB_TRY(mb_gemv(&g, st->stream), "matrix-vector product");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

static int stage_in(mb_state *st, const float *host, size_t n, char *error, size_t cap) {
    if (grow((void **)&st->d_in, &st->d_in_cap, n, sizeof(float), error, cap) != 0) return -1;
    MB_TRY(cudaMemcpyAsync(st->d_in, host, n * sizeof(float), cudaMemcpyHostToDevice, st->stream),
           "host to device copy");
    return 0;
}

static int host_matmul(void *state, const float *input, float *output, size_t rows, size_t iw,
                       size_t ow, const float *weight, const float *bias, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || input == NULL || output == NULL) {
        mb_set_error(error, cap, "invalid backend matmul request");
        return -1;
    }
    if (use_device(st, error, cap) != 0) return -1;
    if (stage_in(st, input, rows * iw, error, cap) != 0 ||
        grow((void **)&st->d_out, &st->d_out_cap, rows * ow, sizeof(float), error, cap) != 0 ||
        product_dev(st, st->d_in, st->d_out, rows, iw, ow, weight, bias, error, cap) != 0)
        return -1;
    MB_TRY(cudaMemcpyAsync(output, st->d_out, rows * ow * sizeof(float), cudaMemcpyDeviceToHost,
                           st->stream), "device to host copy");
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}

static int host_sgemm(void *state, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                      float alpha, const float *a, size_t lda, const float *b, size_t ldb,
                      float beta, float *c, size_t ldc, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || a == NULL || b == NULL || c == NULL || m == 0 || n == 0 || k == 0) {
        mb_set_error(error, cap, "invalid backend sgemm request");
        return -1;
    }
    if (use_device(st, error, cap) != 0) return -1;
    const size_t a_rows = trans_a ? k : m, b_rows = trans_b ? n : k;
    const size_t a_n = a_rows * lda, b_n = b_rows * ldb, c_n = m * ldc;
    float *da = NULL, *db = NULL, *dc = NULL;
    int rc = (int)cudaMalloc((void **)&da, a_n * sizeof(float));
    if (rc == 0) rc = (int)cudaMalloc((void **)&db, b_n * sizeof(float));
    if (rc == 0) rc = (int)cudaMalloc((void **)&dc, c_n * sizeof(float));
    if (rc == 0) rc = (int)cudaMemcpyAsync(da, a, a_n * sizeof(float), cudaMemcpyHostToDevice, st->stream);
    if (rc == 0) rc = (int)cudaMemcpyAsync(db, b, b_n * sizeof(float), cudaMemcpyHostToDevice, st->stream);
    if (rc == 0 && beta != 0.0f)
        rc = (int)cudaMemcpyAsync(dc, c, c_n * sizeof(float), cudaMemcpyHostToDevice, st->stream);
    if (rc == 0) rc = mb_sgemm(trans_a, trans_b, m, n, k, alpha, da, lda, db, ldb, beta, dc, ldc, st->stream);
    /* rows of C are ldc apart and only n wide: copy back row by row layout-safe */
    if (rc == 0)
        rc = (int)cudaMemcpy2DAsync(c, ldc * sizeof(float), dc, ldc * sizeof(float),
                                    n * sizeof(float), m, cudaMemcpyDeviceToHost, st->stream);
    if (rc == 0) rc = (int)cudaStreamSynchronize(st->stream);
    st->launches += 1;
    cudaFree(da);
    cudaFree(db);
    cudaFree(dc);
    if (rc != 0) return mb_cuda(rc, "sgemm", error, cap);
    mb_clear_error(error, cap);
    return 0;
}

static void host_close(void *state) { mynah_b200_close(state); }

/* The known answers of the reference's CUDA self-test
 * (gpu/cuda/backend_cuda.cu:514-529): a 2x3x4 product with bias and a 2x4x3
 * sgemm. */
static int host_self_test(void *state, char *error, size_t cap) {
    static const float input[6] = {1.0f, 2.0f, 3.0f, -1.0f, 0.5f, 2.0f};
    static const float weight[12] = {1.0f, 0.0f, 0.0f, 0.0f, 1.0f, 0.0f,
                                     0.0f, 0.0f, 1.0f, 1.0f, 1.0f, 1.0f};
    static const float bias[4] = {0.5f, -0.5f, 1.0f, 2.0f};
    static const float expected[8] = {1.5f, 1.5f, 4.0f, 8.0f, -0.5f, 0.0f, 3.0f, 3.5f};
    float output[8] = {0};
    mb_state *st = (mb_state *)state;
    const int saved = st->quant;
    st->quant = MB_F32; /* the known answers are exact f32 products */
    const int rc = host_matmul(state, input, output, 2u, 3u, 4u, weight, bias, error, cap);
    st->quant = saved;
    if (rc != 0) return -1;
    for (size_t i = 0; i < 8u; ++i) {
        const float d = output[i] - expected[i];
        if (d > 1.0e-5f || d < -1.0e-5f) {
            if (error != NULL && cap > 0)
                snprintf(error, cap, "B200 backend self-test mismatch at %zu", i);
            return -1;
        }
    }
    /* C[2,4] = in[2,3] * weight[4,3]^T, no bias */
    float c[8] = {0};
    if (host_sgemm(state, 0, 1, 2u, 4u, 3u, 1.0f, input, 3u, weight, 3u, 0.0f, c, 4u, error, cap) != 0)
        return -1;
    const float want[8] = {1.0f, 2.0f, 3.0f, 6.0f, -1.0f, 0.5f, 2.0f, 1.5f};
    for (size_t i = 0; i < 8u; ++i) {
        const float d = c[i] - want[i];
        if (d > 1.0e-5f || d < -1.0e-5f) {
            if (error != NULL && cap > 0)
                snprintf(error, cap, "B200 backend sgemm self-test mismatch at %zu", i);
            return -1;
        }
    }
    mb_clear_error(error, cap);
    return 0;
}

static int quant_from_env(void) {
    const char *env = getenv("MYNAH_QUANT"); /* src/qmat.c:571-576 */
    if (env != NULL && strcmp(env, "int8") == 0) return MB_INT8;
    if (env != NULL && strcmp(env, "int4") == 0) return MB_INT4;
    if (env != NULL && strcmp(env, "f16") == 0) return MB_F16;
    return MB_F32;
}

int mynah_backend_cuda_open(void **state, mynah_backend_matmul_fn *matmul,
                            mynah_backend_sgemm_fn *sgemm, mynah_backend_close_fn *close,
                            mynah_backend_self_test_fn *self_test, char *error, size_t cap) {
    const char *dev_env = getenv("MYNAH_B200_DEVICE");
    const char *strict_env = getenv("MYNAH_B200_STRICT");
    const int device = dev_env != NULL ? atoi(dev_env) : 0;
    const int strict = strict_env != NULL && strcmp(strict_env, "0") != 0;
    if (mynah_b200_open(state, device, quant_from_env(), strict, error, cap) != 0) return -1;
    if (matmul != NULL) *matmul = host_matmul;
    if (sgemm != NULL) *sgemm = host_sgemm;
    if (close != NULL) *close = host_close;
    if (self_test != NULL) *self_test = host_self_test;
    return 0;
}

/* --------------------------------------------------------- memory and copies */
int mynah_cuda_dev_alloc(void *state, size_t n, float **dev_ptr, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || dev_ptr == NULL || n == 0) {
        mb_set_error(error, cap, "invalid device allocation request");
        return -1;
    }
    *dev_ptr = NULL;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaMalloc((void **)dev_ptr, n * sizeof(float)), "cudaMalloc");
    mb_clear_error(error, cap);
    return 0;
}

void mynah_cuda_dev_free(void *state, float *dev_ptr) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || dev_ptr == NULL) return;
    cudaSetDevice(st->device);
    cudaStreamSynchronize(st->stream);
    cudaFree(dev_ptr);
}

int mynah_cuda_h2d(void *state, const float *host, float *dev_ptr, size_t n, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || host == NULL || dev_ptr == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaMemcpyAsync(dev_ptr, host, n * sizeof(float), cudaMemcpyHostToDevice, st->stream),
           "host to device copy");
    /* the host buffer may be reused by the caller as soon as this returns */
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}

int mynah_cuda_d2h(void *state, const float *dev_ptr, float *host, size_t n, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || host == NULL || dev_ptr == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaMemcpyAsync(host, dev_ptr, n * sizeof(float), cudaMemcpyDeviceToHost, st->stream),
           "device to host copy");
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}

/* Upload into the backend's own scratch and hand back its address
 * (src/backend.h:78-82). */
int mynah_cuda_upload(void *state, const float *host, size_t n, float **dev_ptr, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || host == NULL || dev_ptr == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    if (stage_in(st, host, n, error, cap) != 0) return -1;
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    *dev_ptr = st->d_in;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_cuda_download(void *state, const float *dev_ptr, float *host, size_t n, char *error, size_t cap) {
    return mynah_cuda_d2h(state, dev_ptr, host, n, error, cap);
}

int mynah_cuda_sync(void *state, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    /* the seam ops enqueue and return: a bounded device wait that ran out since the last
     * sync is reported here, where the caller collects the step's result */
    int status = 0;
    MB_TRY(cudaMemcpy(&status, st->d_status, sizeof(int), cudaMemcpyDeviceToHost), "read status");
    if (status != 0) {
        cudaMemset(st->d_status, 0, sizeof(int));
        mb_set_error(error, cap, mb_status_message(status));
        return -1;
    }
    mb_clear_error(error, cap);
    return 0;
}

/* Work is stream-ordered already; nothing to open (src/backend.h:90-93). */
int mynah_cuda_batch_begin(void *state, char *error, size_t cap) {
    if (state == NULL) return -1;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_cuda_copy_dev(void *state, float *dev_dst, const float *dev_src, size_t n, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || dev_dst == NULL || dev_src == NULL) return -1;
    if (use_device(st, error, cap) != 0) return -1;
    MB_TRY(cudaMemcpyAsync(dev_dst, dev_src, n * sizeof(float), cudaMemcpyDeviceToDevice, st->stream),
           "device copy");
    mb_clear_error(error, cap);
    return 0;
}

/* --------------------------------------------------------- element-wise ops */
#define SEAM_PROLOGUE()                                              \
    mb_state *st = (mb_state *)state;                                \
    if (st == NULL) return -1;                                       \
    if (use_device(st, error, cap) != 0) return -1

int mynah_cuda_gelu_inplace(void *state, float *dev_data, size_t n, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_data == NULL) return -1;
    MB_TRY(mb_gelu(dev_data, n, st->strict, st->libm.tanh_tab, st->stream), "gelu");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}
int mynah_cuda_gelu_dev(void *state, float *dev_data, size_t n, char *error, size_t cap) {
    return mynah_cuda_gelu_inplace(state, dev_data, n, error, cap);
}

/* 1 when `p` is memory a kernel may read (device or managed / registered host memory), 0 for a
 * plain host pointer.  The reference's resident paths were written for a unified-memory
 * device and hand some operands as host pointers. */
static int device_readable(const void *p) {
    struct cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged || attr.type == cudaMemoryTypeHost;
}

int mynah_cuda_residual_inplace(void *state, float *dev_out, const float *dev_in, size_t n,
                                char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_out == NULL || dev_in == NULL) return -1;
    if (!device_readable(dev_in)) {
        /* local_step_device adds a row of the position table straight from the weight file
         * (src/graph.c:1119-1121: a host pointer, fine on the reference's unified-memory
         * device): stage it */
        if (grow((void **)&st->d_in, &st->d_in_cap, n, sizeof(float), error, cap) != 0) return -1;
        MB_TRY(cudaMemcpyAsync(st->d_in, dev_in, n * sizeof(float), cudaMemcpyHostToDevice, st->stream), "host to device copy");
        dev_in = st->d_in;
    }
    MB_TRY(mb_residual_add(dev_out, dev_in, n, st->stream), "residual add");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}
int mynah_cuda_residual_add_dev(void *state, float *dev_out, const float *dev_in, size_t n,
                                char *error, size_t cap) {
    return mynah_cuda_residual_inplace(state, dev_out, dev_in, n, error, cap);
}

int mynah_cuda_layer_norm_dev(void *state, const float *dev_in, float *dev_out, const float *gain,
                              const float *bias, size_t rows, size_t width, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_in == NULL || dev_out == NULL || gain == NULL) return -1;
    const float *dgain = NULL, *dbias = NULL;
    if (mb_vector_cached(st, gain, width, &dgain, error, cap) != 0 ||
        mb_vector_cached(st, bias, width, &dbias, error, cap) != 0)
        return -1;
    /* epsilon 1e-5 as everywhere in Magpie (src/graph.c:147-150, src/backend.c:599) */
    MB_TRY(mb_layernorm(dev_in, dev_out, dgain, dbias, rows, width, 1.0e-5f, NULL, NULL, NULL,
                        st->strict, st->stream), "layer norm");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}
int mynah_cuda_layer_norm_inplace(void *state, const float *dev_in, float *dev_out,
                                  const float *gain, size_t rows, size_t width, char *error,
                                  size_t cap) {
    return mynah_cuda_layer_norm_dev(state, dev_in, dev_out, gain, NULL, rows, width, error, cap);
}

int mynah_cuda_scale_dev(void *state, float *dev_data, size_t n, float scale, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_data == NULL) return -1;
    MB_TRY(mb_scale(dev_data, n, scale, st->stream), "scale");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_cuda_clip_dev(void *state, float *dev_data, size_t n, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_data == NULL) return -1;
    MB_TRY(mb_clip(dev_data, n, st->stream), "clip");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_cuda_argmax_dev(void *state, const float *dev_logits, size_t vocab, size_t codebook_size,
                          size_t eos_id, int allow_eos, unsigned *argmax, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_logits == NULL || argmax == NULL || vocab == 0u || codebook_size > vocab) return -1;
    MB_TRY(mb_argmax_rows(dev_logits, 1u, vocab, codebook_size, eos_id, NULL, allow_eos,
                          st->d_token, NULL, NULL, 1u, NULL, st->stream), "argmax");
    st->launches += 1;
    MB_TRY(cudaMemcpyAsync(argmax, st->d_token, sizeof(unsigned), cudaMemcpyDeviceToHost, st->stream),
           "device to host copy");
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}

static int gelu_host_common(void *state, float *host_data, size_t n, int strict, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (host_data == NULL) return -1;
    if (stage_in(st, host_data, n, error, cap) != 0) return -1;
    MB_TRY(mb_gelu(st->d_in, n, strict, st->libm.tanh_tab, st->stream), "gelu");
    st->launches += 1;
    MB_TRY(cudaMemcpyAsync(host_data, st->d_in, n * sizeof(float), cudaMemcpyDeviceToHost, st->stream),
           "device to host copy");
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}
int mynah_cuda_gelu_host(void *state, float *host_data, size_t n, char *error, size_t cap) {
    return gelu_host_common(state, host_data, n, ((mb_state *)state)->strict, error, cap);
}
/* The double-precision tanh form (gpu/cuda/backend_cuda.cu:828-837 there). */
int mynah_cuda_gelu_host_f64(void *state, float *host_data, size_t n, char *error, size_t cap) {
    if (state == NULL) return -1;
    return gelu_host_common(state, host_data, n, 1, error, cap);
}

/* ------------------------------------------------------------------ products */
int mynah_cuda_matmul_d2d(void *state, const float *dev_in, float *dev_out, size_t rows, size_t iw,
                          size_t ow, const float *weight, const float *bias, char *error, size_t cap) {
    return product_dev((mb_state *)state, dev_in, dev_out, rows, iw, ow, weight, bias, error, cap);
}
int mynah_cuda_matmul_dev(void *state, const float *dev_in, float *dev_out, size_t rows, size_t iw,
                          size_t ow, const float *weight, const float *bias, char *error, size_t cap) {
    return product_dev((mb_state *)state, dev_in, dev_out, rows, iw, ow, weight, bias, error, cap);
}
int mynah_cuda_matvec_dev(void *state, const float *dev_in, float *dev_out, size_t K, size_t N,
                          const float *weight, const float *bias, char *error, size_t cap) {
    return product_dev((mb_state *)state, dev_in, dev_out, 1u, K, N, weight, bias, error, cap);
}
int mynah_cuda_matmul_to_dev(void *state, const float *host_in, float *dev_out, size_t rows,
                             size_t iw, size_t ow, const float *weight, const float *bias,
                             char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (host_in == NULL) return -1;
    if (stage_in(st, host_in, rows * iw, error, cap) != 0) return -1;
    return product_dev(st, st->d_in, dev_out, rows, iw, ow, weight, bias, error, cap);
}
int mynah_cuda_matmul_graph(void *state, const float *host_in, float *host_out, size_t rows,
                            size_t iw, size_t ow, const float *weight, const float *bias,
                            char *error, size_t cap) {
    return host_matmul(state, host_in, host_out, rows, iw, ow, weight, bias, error, cap);
}
int mynah_cuda_sgemm_dev(void *state, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                         float alpha, const float *dev_a, size_t lda, const float *dev_b,
                         size_t ldb, float beta, float *dev_c, size_t ldc, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_a == NULL || dev_b == NULL || dev_c == NULL) return -1;
    MB_TRY(mb_sgemm(trans_a, trans_b, m, n, k, alpha, dev_a, lda, dev_b, ldb, beta, dev_c, ldc,
                    st->stream), "sgemm");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

/* ----------------------------------------------------------------- attention */
static int attention_common(mb_state *st, const float *q, size_t q_stride, const float *k_new,
                            const float *v_new, float *kc, float *vc, size_t position,
                            size_t cache_stride, size_t valid, size_t heads, size_t hw, float scale,
                            float *out, char *error, size_t cap) {
    if (q == NULL || kc == NULL || vc == NULL || out == NULL || heads == 0 || hw == 0 ||
        valid == 0 || cache_stride < heads * hw) {
        mb_set_error(error, cap, "invalid attention request");
        return -1;
    }
    mb_attn_args a;
    memset(&a, 0, sizeof(a));
    a.q = q;
    a.q_stride = q_stride;
    a.k_new = k_new;
    a.v_new = v_new;
    a.k_cache = kc;
    a.v_cache = vc;
    a.position = position;
    a.valid = valid;
    a.cache_stride = cache_stride;
    a.heads = heads;
    a.head_width = hw;
    a.scale = scale;
    a.out = out;
    a.out_stride = heads * hw;
    a.batch = 1;
    a.strict = st->strict;
    a.exp_tab = st->libm.exp_tab;
    a.status = st->d_status;
    a.sm_count = st->sm_count;
    if (!st->strict) {
        const size_t need = mb_attention_scratch_floats(1u, heads, valid, hw);
        const size_t ctrs = mb_attention_counters(1u, heads);
        const size_t had = st->d_counters_cap;
        if (grow((void **)&st->d_partials, &st->d_partials_cap, need, sizeof(float), error, cap) != 0 ||
            grow((void **)&st->d_counters, &st->d_counters_cap, ctrs, sizeof(unsigned), error, cap) != 0)
            return -1;
        if (st->d_counters_cap != had)
            MB_TRY(cudaMemsetAsync(st->d_counters, 0, st->d_counters_cap * sizeof(unsigned), st->stream),
                   "cudaMemset");
        a.partials = st->d_partials;
        a.counters = st->d_counters;
    }
    MB_TRY(mb_attention(&a, st->stream), "attention");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

int mynah_cuda_self_attention_dev(void *state, const float *dev_qkv, float *dev_k_cache,
                                  float *dev_v_cache, size_t position, size_t cache_stride,
                                  size_t valid, size_t heads, size_t head_width, float scale,
                                  float *dev_out, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_qkv == NULL) return -1;
    const size_t width = heads * head_width;
    return attention_common(st, dev_qkv, 3u * width, dev_qkv + width, dev_qkv + 2u * width,
                            dev_k_cache, dev_v_cache, position, cache_stride, valid, heads,
                            head_width, scale, dev_out, error, cap);
}

int mynah_cuda_cross_attention_dev(void *state, const float *dev_q, const float *dev_k_cache,
                                   const float *dev_v_cache, size_t valid, size_t cache_stride,
                                   size_t heads, size_t head_width, float scale, float *dev_out,
                                   char *error, size_t cap) {
    SEAM_PROLOGUE();
    return attention_common(st, dev_q, heads * head_width, NULL, NULL, (float *)dev_k_cache,
                            (float *)dev_v_cache, 0u, cache_stride, valid, heads, head_width,
                            scale, dev_out, error, cap);
}

/* ------------------------------------------------------------- codec ops */
/* snake_dev (src/backend.h:128-133): device signal [channels][length] in place, HOST alpha
 * (cached by pointer like the weights). */
int mynah_cuda_snake_dev(void *state, float *dev_data, const float *alpha, size_t channels,
                         size_t length, size_t snake_channels, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (dev_data == NULL || alpha == NULL || channels == 0u || length == 0u || snake_channels > channels) return -1;
    const float *d_alpha = NULL;
    if (snake_channels > 0u && mb_vector_cached(st, alpha, snake_channels, &d_alpha, error, cap) != 0) return -1;
    MB_TRY(mb_codec_half_snake(dev_data, dev_data, d_alpha, channels, length, snake_channels, st->strict,
                               mb_libm_sin_table(st), st->stream), "snake");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

/* im2col (src/backend.h:59): device input [in_ch][length] -> device columns
 * [in_ch * kernel][length]. */
int mynah_cuda_im2col(void *state, const float *in, float *cols, int in_ch, int length, int kernel,
                      int dilation, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (in == NULL || cols == NULL || in_ch <= 0 || length <= 0 || kernel <= 0 || dilation <= 0) return -1;
    MB_TRY(mb_codec_im2col(in, cols, (size_t)in_ch, (size_t)length, (size_t)kernel, (size_t)dilation, st->stream), "im2col");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

/* conv1d (src/backend.h:60).  The reference calls it two ways: conv1d_causal hands HOST
 * input/output (what its CUDA backend serves, gpu/cuda/backend_cuda.cu:746-810: synchronous),
 * decode_codec_resident hands DEVICE buffers from dev_alloc (what its Metal backend serves,
 * src/graph.c:2552-2556: enqueued, no sync).  The kind of `in` decides; weight and bias are
 * host pointers used as cache keys either way.  Shapes the convolution kernel does not take
 * (a kernel other than 3, 7, 11) return -1 and the caller keeps its CPU path. */
int mynah_cuda_conv1d(void *state, const float *in, float *out, int in_ch, int out_ch, int length,
                      int kernel, int dilation, const float *weight, const float *bias,
                      char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (in == NULL || out == NULL || weight == NULL || bias == NULL || in_ch <= 0 || out_ch <= 0 || length <= 0 ||
        dilation <= 0 || (kernel != 3 && kernel != 7 && kernel != 11) || (kernel - 1) * dilation > 50) {
        mb_set_error(error, cap, "conv1d shape is not served by the B200 backend; use the CPU path");
        return -1;
    }
    const size_t ic = (size_t)in_ch, oc = (size_t)out_ch, L = (size_t)length, K = (size_t)kernel;
    struct cudaPointerAttributes attr;
    const int on_device = cudaPointerGetAttributes(&attr, in) == cudaSuccess && attr.type == cudaMemoryTypeDevice;
    if (!on_device) (void)cudaGetLastError();      /* an unregistered host pointer is not an error here */
    const float *d_w = NULL, *d_b = NULL;
    if (mb_vector_cached(st, weight, oc * ic * K, &d_w, error, cap) != 0 ||
        mb_vector_cached(st, bias, oc, &d_b, error, cap) != 0) return -1;
    const size_t packed = mb_codec_conv_packed_floats(oc, ic, K);
    const size_t staged_in = on_device ? 0u : ic * L;
    if (grow((void **)&st->d_in, &st->d_in_cap, staged_in + packed, sizeof(float), error, cap) != 0) return -1;
    if (!on_device && grow((void **)&st->d_out, &st->d_out_cap, oc * L, sizeof(float), error, cap) != 0) return -1;
    float *d_packed = st->d_in + staged_in;
    if (!on_device)
        MB_TRY(cudaMemcpyAsync(st->d_in, in, ic * L * sizeof(float), cudaMemcpyHostToDevice, st->stream), "host to device copy");
    MB_TRY(mb_codec_pack_conv_weight(d_w, d_packed, oc, ic, K, st->stream), "pack weight");
    mb_codec_conv_args g;
    memset(&g, 0, sizeof(g));
    g.in = on_device ? in : st->d_in; g.w_packed = d_packed; g.bias = d_b; g.out = on_device ? out : st->d_out;
    g.ic = ic; g.oc = oc; g.length = L; g.kernel = K; g.dilation = (size_t)dilation;
    g.strict = st->strict; g.sm_count = st->sm_count;
    MB_TRY(mb_codec_conv1d(&g, st->stream), "conv1d");
    st->launches += 2;
    if (!on_device) {
        MB_TRY(cudaMemcpyAsync(out, st->d_out, oc * L * sizeof(float), cudaMemcpyDeviceToHost, st->stream), "device to host copy");
        MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    }
    mb_clear_error(error, cap);
    return 0;
}

/* conv_transpose_dev (src/backend.h:61; the reference wires it for Metal only): device input
 * [in_ch][length] -> device output [out_ch][output_length], host weight [in_ch][out_ch / groups]
 * [kernel] and bias as cache keys.  Served: the codec's shape -- one output channel per group,
 * kernel = 2 * stride, output_length = length * stride (src/graph.c:2596-2601); anything else
 * returns -1. */
int mynah_cuda_conv_transpose_dev(void *state, const float *in, float *out, int in_ch, int out_ch, int length,
                                  int output_length, int kernel, int stride, int groups, const float *weight,
                                  const float *bias, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (in == NULL || out == NULL || weight == NULL || bias == NULL || in_ch <= 0 || out_ch <= 0 || length <= 0 ||
        stride <= 0 || groups != out_ch || in_ch % out_ch != 0 || kernel != 2 * stride ||
        (long)output_length != (long)length * stride) {
        mb_set_error(error, cap, "conv_transpose shape is not served by the B200 backend");
        return -1;
    }
    const float *d_w = NULL, *d_b = NULL;
    if (mb_vector_cached(st, weight, (size_t)in_ch * (size_t)kernel, &d_w, error, cap) != 0 ||
        mb_vector_cached(st, bias, (size_t)out_ch, &d_b, error, cap) != 0) return -1;
    MB_TRY(mb_codec_conv_transpose(in, d_w, d_b, out, (size_t)in_ch, (size_t)out_ch, (size_t)length, (size_t)stride,
                                   st->strict, st->stream), "conv_transpose");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

/* ------------------------------------------------ packing / single-op extension */
int mynah_b200_pack_weight(void *state, int quant, const float *host_w, size_t n, size_t k,
                           void *host_q, float *host_scales, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (host_w == NULL || host_q == NULL) return -1;
    if (quant == MB_INT4 && (k % 32u) != 0) {
        mb_set_error(error, cap, "int4 needs k to be a multiple of 32");
        return -1;
    }
    mb_dev_weight w;
    if (mb_weight_build(st, host_w, n, k, quant, &w, error, cap) != 0) return -1;
    size_t wbytes = n * k * sizeof(float), sbytes = 0;
    if (quant == MB_INT8) { wbytes = n * k; sbytes = n * sizeof(float); }
    else if (quant == MB_INT4) { wbytes = n * (k / 2u); sbytes = n * (k / 32u) * sizeof(float); }
    else if (quant == MB_F16) wbytes = n * k * 2u;
    int rc = (int)cudaMemcpy(host_q, w.w, wbytes, cudaMemcpyDeviceToHost);
    if (rc == 0 && sbytes != 0 && host_scales != NULL)
        rc = (int)cudaMemcpy(host_scales, w.scales, sbytes, cudaMemcpyDeviceToHost);
    mb_weight_release(&w);
    if (rc != 0) return mb_cuda(rc, "copy packed weight", error, cap);
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_quantize_act(void *state, const float *host_x, size_t rows, size_t k,
                            int8_t *host_q, float *host_sx, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (host_x == NULL || host_q == NULL || host_sx == NULL || rows == 0 || k == 0) return -1;
    if (stage_in(st, host_x, rows * k, error, cap) != 0 ||
        grow((void **)&st->d_qx, &st->d_qx_cap, rows * k, 1, error, cap) != 0 ||
        grow((void **)&st->d_sx, &st->d_sx_cap, rows, sizeof(float), error, cap) != 0)
        return -1;
    MB_TRY(mb_quant_rows(st->d_in, rows, k, st->d_qx, st->d_sx, NULL, st->stream), "quantize");
    st->launches += 1;
    MB_TRY(cudaMemcpyAsync(host_q, st->d_qx, rows * k, cudaMemcpyDeviceToHost, st->stream), "copy");
    MB_TRY(cudaMemcpyAsync(host_sx, st->d_sx, rows * sizeof(float), cudaMemcpyDeviceToHost, st->stream), "copy");
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}

int mynah_b200_qmat_linear(void *state, const float *weight, const float *x, float *out,
                           size_t count, size_t k, size_t n, const float *bias,
                           const float *ln_gain, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (weight == NULL || x == NULL || out == NULL || count == 0 || k == 0 || n == 0) {
        mb_set_error(error, cap, "invalid linear request");
        return -1;
    }
    const int use_q = st->quant != MB_F32 && count <= QMAT_SMALL_COUNT && k <= QMAT_K_MAX;
    const mb_dev_weight *w = NULL;
    const float *dbias = NULL, *dgain = NULL;
    if (mb_weight_cached(st, weight, n, k, use_q ? st->quant : MB_F32, &w, error, cap) != 0 ||
        mb_vector_cached(st, bias, n, &dbias, error, cap) != 0 ||
        mb_vector_cached(st, ln_gain, k, &dgain, error, cap) != 0)
        return -1;
    if (stage_in(st, x, count * k, error, cap) != 0 ||
        grow((void **)&st->d_out, &st->d_out_cap, count * (n + k), sizeof(float), error, cap) != 0 ||
        grow((void **)&st->d_qx, &st->d_qx_cap, count * k, 1, error, cap) != 0 ||
        grow((void **)&st->d_sx, &st->d_sx_cap, count, sizeof(float), error, cap) != 0)
        return -1;
    const int quantized = w->qtype == MB_INT8 || w->qtype == MB_INT4;
    float *d_y = st->d_out;                 /* [count][n] */
    float *d_nrm = st->d_out + count * n;   /* [count][k] */
    const float *act = st->d_in;
    if (dgain != NULL) {
        MB_TRY(mb_layernorm(st->d_in, quantized ? NULL : d_nrm, dgain, NULL, count, k, 1.0e-5f,
                            quantized ? st->d_qx : NULL, quantized ? st->d_sx : NULL, NULL,
                            st->strict, st->stream), "layer norm");
        st->launches += 1;
        act = d_nrm;
    } else if (quantized) {
        MB_TRY(mb_quant_rows(st->d_in, count, k, st->d_qx, st->d_sx, NULL, st->stream), "quantize");
        st->launches += 1;
    }
    if (w->qtype == MB_F32 && count > QMAT_SMALL_COUNT) {
        MB_TRY(mb_sgemm(0, 1, count, n, k, 1.0f, act, k, (const float *)w->w, k, 0.0f, d_y, n,
                        st->stream), "sgemm");
        st->launches += 1;
        if (dbias != NULL) {
            MB_TRY(mb_bias_add(d_y, dbias, count, n, st->stream), "bias add");
            st->launches += 1;
        }
    } else {
        mb_gemv_args g;
        memset(&g, 0, sizeof(g));
        mb_gemv_bind_weight(&g, w, dbias);
        g.out = d_y;
        g.out_stride = n;
        g.batch = count;
        g.strict = st->strict;
    g.tanh_tab = st->libm.tanh_tab;
        if (quantized) { g.qx = st->d_qx; g.sx = st->d_sx; }
        else g.x = act;
        MB_TRY(mb_gemv(&g, st->stream), "matrix-vector product");
        st->launches += 1;
    }
    MB_TRY(cudaMemcpyAsync(out, d_y, count * n * sizeof(float), cudaMemcpyDeviceToHost, st->stream),
           "device to host copy");
    MB_TRY(cudaStreamSynchronize(st->stream), "cudaStreamSynchronize");
    mb_clear_error(error, cap);
    return 0;
}

/* ------------------------------------------------------------- matrix pool */
typedef struct {
    mb_state *st;
    size_t n, k, groups;
    int qtype;
    void *w;
    float *scales, *bias, *gain;
    int8_t *qx;
    float *sx, *nrm;
    size_t w_stride, scale_stride;
} mb_pool;

/* `groups` distinct matrices derived from one host matrix: group g is the host
 * matrix rotated by g rows, so every group has different bytes but known
 * contents (out_g[r] == out_0[(r + g) % n]). */
int mynah_b200_pool_create(void *state, const float *host_w, size_t n, size_t k, size_t groups,
                           const float *host_bias, const float *host_gain, void **pool,
                           char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (pool == NULL || host_w == NULL || n == 0 || k == 0 || groups == 0) return -1;
    *pool = NULL;
    int qtype = st->quant;
    if (qtype == MB_INT4 && (k % 32u) != 0) qtype = MB_F32;
    mb_pool *p = (mb_pool *)calloc(1, sizeof(*p));
    if (p == NULL) return -1;
    p->st = st; p->n = n; p->k = k; p->groups = groups; p->qtype = qtype;
    mb_dev_weight w;
    if (mb_weight_build(st, host_w, n, k, qtype, &w, error, cap) != 0) { free(p); return -1; }
    const size_t row_bytes = qtype == MB_INT8 ? k : qtype == MB_INT4 ? k / 2u : qtype == MB_F16 ? k * 2u : k * 4u;
    const size_t srow = qtype == MB_INT8 ? 1u : qtype == MB_INT4 ? k / 32u : 0u;
    p->w_stride = n * row_bytes;
    p->scale_stride = n * srow;
    int rc = (int)cudaMalloc(&p->w, groups * p->w_stride);
    if (rc == 0 && srow != 0) rc = (int)cudaMalloc((void **)&p->scales, groups * p->scale_stride * sizeof(float));
    if (rc == 0) rc = (int)cudaMalloc((void **)&p->qx, groups * k);
    if (rc == 0) rc = (int)cudaMalloc((void **)&p->sx, groups * sizeof(float));
    if (rc == 0) rc = (int)cudaMalloc((void **)&p->nrm, groups * k * sizeof(float));
    for (size_t g = 0; g < groups && rc == 0; ++g) {
        const size_t rot = g % n;
        /* rows [rot, n) then [0, rot) */
        unsigned char *dst = (unsigned char *)p->w + g * p->w_stride;
        rc = (int)cudaMemcpyAsync(dst, (const unsigned char *)w.w + rot * row_bytes,
                                  (n - rot) * row_bytes, cudaMemcpyDeviceToDevice, st->stream);
        if (rc == 0 && rot != 0)
            rc = (int)cudaMemcpyAsync(dst + (n - rot) * row_bytes, w.w, rot * row_bytes,
                                      cudaMemcpyDeviceToDevice, st->stream);
        if (rc == 0 && srow != 0) {
            float *sd = p->scales + g * p->scale_stride;
            rc = (int)cudaMemcpyAsync(sd, w.scales + rot * srow, (n - rot) * srow * sizeof(float),
                                      cudaMemcpyDeviceToDevice, st->stream);
            if (rc == 0 && rot != 0)
                rc = (int)cudaMemcpyAsync(sd + (n - rot) * srow, w.scales, rot * srow * sizeof(float),
                                          cudaMemcpyDeviceToDevice, st->stream);
        }
    }
    if (rc == 0) rc = (int)cudaStreamSynchronize(st->stream);
    mb_weight_release(&w);
    if (rc == 0 && host_bias != NULL) {
        rc = (int)cudaMalloc((void **)&p->bias, n * sizeof(float));
        if (rc == 0) rc = (int)cudaMemcpy(p->bias, host_bias, n * sizeof(float), cudaMemcpyHostToDevice);
    }
    if (rc == 0 && host_gain != NULL) {
        rc = (int)cudaMalloc((void **)&p->gain, k * sizeof(float));
        if (rc == 0) rc = (int)cudaMemcpy(p->gain, host_gain, k * sizeof(float), cudaMemcpyHostToDevice);
    }
    if (rc != 0) {
        mynah_b200_pool_destroy(p);
        return mb_cuda(rc, "matrix pool", error, cap);
    }
    *pool = p;
    mb_clear_error(error, cap);
    return 0;
}

void mynah_b200_pool_destroy(void *pool) {
    mb_pool *p = (mb_pool *)pool;
    if (p == NULL) return;
    cudaSetDevice(p->st->device);
    cudaStreamSynchronize(p->st->stream);
    cudaFree(p->w); cudaFree(p->scales); cudaFree(p->bias); cudaFree(p->gain);
    cudaFree(p->qx); cudaFree(p->sx); cudaFree(p->nrm);
    free(p);
}

size_t mynah_b200_pool_bytes_per_pass(const void *pool) {
    const mb_pool *p = (const mb_pool *)pool;
    if (p == NULL) return 0;
    /* per matrix: packed weights + scales + bias + x + gain + y */
    const size_t per = p->w_stride + p->scale_stride * sizeof(float) +
                       (p->bias != NULL ? p->n * sizeof(float) : 0u) + p->k * sizeof(float) +
                       (p->gain != NULL ? p->k * sizeof(float) : 0u) + p->n * sizeof(float);
    return per * p->groups;
}

int mynah_b200_pool_linear(void *pool, const float *dev_x, float *dev_out, char *error, size_t cap) {
    mb_pool *p = (mb_pool *)pool;
    if (p == NULL || dev_x == NULL || dev_out == NULL) return -1;
    mb_state *st = p->st;
    if (use_device(st, error, cap) != 0) return -1;
    const int quantized = p->qtype == MB_INT8 || p->qtype == MB_INT4;
    const float *act = dev_x;
    if (p->gain != NULL) {
        MB_TRY(mb_layernorm(dev_x, quantized ? NULL : p->nrm, p->gain, NULL, p->groups, p->k, 1.0e-5f,
                            quantized ? p->qx : NULL, quantized ? p->sx : NULL, NULL, st->strict,
                            st->stream), "layer norm");
        act = p->nrm;
        st->launches += 1;
    } else if (quantized) {
        MB_TRY(mb_quant_rows(dev_x, p->groups, p->k, p->qx, p->sx, NULL, st->stream), "quantize");
        st->launches += 1;
    }
    mb_gemv_args g;
    memset(&g, 0, sizeof(g));
    g.qtype = p->qtype;
    g.w = p->w;
    g.scales = p->scales;
    g.bias = p->bias;
    g.n = p->n;
    g.k = p->k;
    g.out = dev_out;
    g.out_stride = p->n;
    g.batch = 1;
    g.strict = st->strict;
    g.tanh_tab = st->libm.tanh_tab;
    g.groups = p->groups;
    g.w_group_stride = p->w_stride;
    g.scale_group_stride = p->scale_stride;
    g.act_group_stride = p->k;
    g.out_group_stride = p->n;
    if (quantized) { g.qx = p->qx; g.sx = p->sx; }
    else g.x = act;
    MB_TRY(mb_gemv(&g, st->stream), "matrix-vector product");
    st->launches += 1;
    mb_clear_error(error, cap);
    return 0;
}

/* ---------------------------------------------------------------- diagnostics */
/* Time one int8 product shape in isolation: `iters` back-to-back launches on the
 * backend's stream between two events, weights and activations resident.  path:
 * 0 = SIMT kernel, 1 = tensor-core kernel.  Returns the mean device time per
 * launch in microseconds. */
int mynah_b200_time_product(void *state, size_t n, size_t k, size_t batch, int path, int epilogue,
                            size_t iters, float *us_per_launch, char *error, size_t cap) {
    SEAM_PROLOGUE();
    if (n == 0 || k == 0 || batch == 0 || iters == 0 || us_per_launch == NULL) return -1;
    int8_t *w = NULL, *qx = NULL;
    float *scales = NULL, *sx = NULL, *out = NULL;
    cudaEvent_t e0 = NULL, e1 = NULL;
    int rc = (int)cudaMalloc((void **)&w, n * k);
    if (rc == 0) rc = (int)cudaMalloc((void **)&qx, batch * k);
    if (rc == 0) rc = (int)cudaMalloc((void **)&scales, n * sizeof(float));
    if (rc == 0) rc = (int)cudaMalloc((void **)&sx, batch * sizeof(float));
    if (rc == 0) rc = (int)cudaMalloc((void **)&out, batch * n * sizeof(float));
    if (rc == 0) rc = (int)cudaMemset(w, 1, n * k);
    if (rc == 0) rc = (int)cudaMemset(qx, 1, batch * k);
    if (rc == 0) rc = (int)cudaMemset(scales, 0, n * sizeof(float));
    if (rc == 0) rc = (int)cudaMemset(sx, 0, batch * sizeof(float));
    if (rc == 0) rc = (int)cudaMemset(out, 0, batch * n * sizeof(float));
    if (rc == 0) rc = (int)cudaEventCreate(&e0);
    if (rc == 0) rc = (int)cudaEventCreate(&e1);
    mb_gemv_args g;
    memset(&g, 0, sizeof(g));
    g.qtype = MB_INT8; g.w = w; g.scales = scales; g.n = n; g.k = k; g.qx = qx; g.sx = sx;
    g.out = out; g.out_stride = n; g.batch = batch; g.epilogue = epilogue;
    for (size_t i = 0; i < iters + 3 && rc == 0; ++i) {
        if (i == 3) rc = (int)cudaEventRecord(e0, st->stream);
        if (rc == 0)
            rc = path == 1 ? mb_gemm_tc(&g, batch, st->d_status, st->stream)
                           : mb_gemv(&g, st->stream);
    }
    if (rc == 0) rc = (int)cudaEventRecord(e1, st->stream);
    if (rc == 0) rc = (int)cudaEventSynchronize(e1);
    float ms = 0.0f;
    if (rc == 0) rc = (int)cudaEventElapsedTime(&ms, e0, e1);
    st->launches += iters + 3;
    cudaFree(w); cudaFree(qx); cudaFree(scales); cudaFree(sx); cudaFree(out);
    if (e0 != NULL) cudaEventDestroy(e0);
    if (e1 != NULL) cudaEventDestroy(e1);
    if (rc != 0) return mb_cuda(rc, "time product", error, cap);
    *us_per_launch = ms * 1000.0f / (float)iters;
    mb_clear_error(error, cap);
    return 0;
}
