// Builds the libm correction tables described in libm_parity.cuh: the host
// hands over its own expf/tanhf/sinf results for a run of consecutive float bit
// patterns, the device compares them with its base values and packs the
// differences, 4 bits each.
#include "common.cuh"
#include "launch.h"
#include "libm_parity.cuh"

namespace {

// Thread t packs values [8t, 8t+8) of this run into one table word.
__global__ void k_libm_delta(const float *__restrict__ host_vals, uint32_t first_bits, size_t count,
                             int kind, uint32_t *__restrict__ table_words, int *__restrict__ status) {
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t * 8 >= count) return;
    uint32_t word = 0;
    for (int j = 0; j < 8; ++j) {
        const size_t i = t * 8 + j;
        if (i >= count) break;
        const float a = __int_as_float((int)(first_bits + (uint32_t)i));
        const uint32_t bits = first_bits + (uint32_t)i;
        const float base = kind == MB_LIBM_EXP ? mb_exp_base(a, bits, true)
                           : kind == MB_LIBM_SIN ? mb_sin_base(a) : mb_tanh_base(a, bits, true);
        const int delta = __float_as_int(host_vals[i]) - __float_as_int(base);
        if (delta < -8 || delta > 7) {
            atomicOr(status, 4);   // the table format cannot express this libm
        } else {
            word |= (uint32_t)(delta & 15) << (4 * j);
        }
    }
    table_words[t] = word;
}

}  // namespace

extern "C" int mb_libm_delta(const float *host_vals_dev, uint32_t first_bits, size_t count, int kind,
                             uint32_t *table_words, int *status, mb_stream stream) {
    if (count == 0 || (count % 8u) != 0) return (int)cudaErrorInvalidValue;
    const size_t threads = count / 8;
    k_libm_delta<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        host_vals_dev, first_bits, count, kind, table_words, status);
    return mb_check_launch();
}
