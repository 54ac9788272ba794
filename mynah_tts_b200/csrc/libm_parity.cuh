// Bit-for-bit reproduction of the HOST libm's expf and tanhf on the device.
//
// The reference's decode step calls libm's expf (softmax, src/graph.c:3195) and
// tanhf (GELU, src/kernels.c:382-389).  Neither is correctly rounded, so no
// device formula returns the same bits for every argument, and with int8
// activation quantization behind them a single last-bit difference can move a
// rounding boundary and change every later frame.  Strict mode therefore
// carries two correction tables, built at open time from the host's own libm:
// for every float argument in the range where host and device can differ, a
// signed 4-bit field says by how many units in the last place the host's result
// differs from the device's base value, which is the double-precision function
// rounded once to float (glibc 2.39: tanhf is off by up to 2 ulp on 15-50% of
// the arguments between 2^-25 and 8; expf by 1 ulp on about 0.06% between 2^-14
// and 128; outside those ranges the two agree everywhere).  Both functions are evaluated on |x| (tanhf
// is odd; the softmax argument is never positive), so the tables cover positive
// magnitudes only.
#pragma once

#include <stdint.h>

#include "launch.h"

// First and one-past-last float bit patterns covered by each table.
#define MB_TANH_LO_BITS 0x32800000u   // 2^-26
#define MB_TANH_HI_BITS 0x41800000u   // 16
#define MB_EXP_LO_BITS 0x38000000u    // 2^-15
#define MB_EXP_HI_BITS 0x43800000u    // 256


#ifdef __CUDACC__
__device__ __forceinline__ float mb_apply_delta(float base, const uint32_t *tab, uint32_t idx) {
    const uint32_t d = (__ldg(tab + (idx >> 3)) >> ((idx & 7u) * 4u)) & 15u;
    const int delta = (int)(d ^ 8u) - 8;   // sign-extend the nibble
    return __int_as_float(__float_as_int(base) + delta);   // base >= 0 here
}

// tanhf as the host computes it (tables present) or correctly rounded (absent).
__device__ __forceinline__ float mb_tanhf_host(float x, const uint32_t *tab) {
    const float a = fabsf(x);
    float r = (float)tanh((double)a);
    const uint32_t bits = (uint32_t)__float_as_int(a);
    if (tab != nullptr && bits >= MB_TANH_LO_BITS && bits < MB_TANH_HI_BITS)
        r = mb_apply_delta(r, tab, bits - MB_TANH_LO_BITS);
    return copysignf(r, x);
}

// expf(x) for x <= 0 as the host computes it.
__device__ __forceinline__ float mb_expf_host(float x, const uint32_t *tab) {
    float r = (float)exp((double)x);
    const uint32_t bits = (uint32_t)__float_as_int(-x);
    if (tab != nullptr && x <= 0.0f && bits >= MB_EXP_LO_BITS && bits < MB_EXP_HI_BITS)
        r = mb_apply_delta(r, tab, bits - MB_EXP_LO_BITS);
    return r;
}
#endif
