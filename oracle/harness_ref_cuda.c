/* The reference's backend layer bound to libmynah_b200.so.  TEST INFRASTRUCTURE ONLY.
 *
 * This translation unit textually includes the reference's src/backend.c (found through
 * -I on the compile line) compiled with -DMYNAH_ENABLE_CUDA, so that the CUDA branch of
 * mynah_backend_open (src/backend.c:434-465) binds the `mynah_cuda_*` symbols -- which the
 * link line resolves against libmynah_b200.so instead of the reference's own
 * gpu/cuda/backend_cuda.cu.  ref_backend_light_up then performs, on the opened backend,
 * the assignments a maintainer adds to that branch to wire the resident ops the reference
 * assigns only for its Metal device (src/backend.c:404-428): seven for the decoder step,
 * one (conv_transpose_dev) for the codec.  With them
 * mynah_backend_has_attention_dev is true (src/backend.c:681-684) and the reference's own
 * decoder_run takes its resident path (src/graph.c:3363-3491) through this library.
 * Nothing of the reference is copied: the wrapper only assigns function pointers.
 */
#include "backend.c"

extern int mynah_cuda_batch_begin(void *, char *, size_t);
extern int mynah_cuda_copy_dev(void *, float *, const float *, size_t, char *, size_t);
extern int mynah_cuda_scale_dev(void *, float *, size_t, float, char *, size_t);
extern int mynah_cuda_clip_dev(void *, float *, size_t, char *, size_t);
extern int mynah_cuda_argmax_dev(void *, const float *, size_t, size_t, size_t, int, unsigned *,
                                 char *, size_t);
extern int mynah_cuda_self_attention_dev(void *, const float *, float *, float *, size_t, size_t,
                                         size_t, size_t, size_t, float, float *, char *, size_t);
extern int mynah_cuda_cross_attention_dev(void *, const float *, const float *, const float *,
                                          size_t, size_t, size_t, size_t, float, float *, char *,
                                          size_t);

extern int mynah_cuda_conv_transpose_dev(void *, const float *, float *, int, int, int, int, int, int, int,
                                         const float *, const float *, char *, size_t);

__attribute__((visibility("default")))
int ref_backend_light_up(mynah_backend *backend) {
    if (backend == NULL || backend->device != MYNAH_TTS_DEVICE_CUDA) return -1;
    backend->batch_begin = mynah_cuda_batch_begin;
    backend->copy_dev = mynah_cuda_copy_dev;
    backend->scale_dev = mynah_cuda_scale_dev;
    backend->clip_dev = mynah_cuda_clip_dev;
    backend->argmax_dev = mynah_cuda_argmax_dev;
    backend->self_attention_dev = mynah_cuda_self_attention_dev;
    backend->cross_attention_dev = mynah_cuda_cross_attention_dev;
    /* with the attention ops wired, decode_codec takes its resident path too
     * (src/graph.c:2511-2638), which needs the transposed convolution the reference assigns
     * only for Metal; conv1d, im2col and snake_dev are already bound by the CUDA branch */
    backend->conv_transpose_dev = mynah_cuda_conv_transpose_dev;
    return 0;
}
