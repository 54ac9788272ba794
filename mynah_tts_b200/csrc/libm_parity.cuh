// Bit-for-bit reproduction of the HOST libm's expf, tanhf and sinf on the device.
//
// The reference's decode step calls libm's expf (softmax, src/graph.c:3195) and
// tanhf (GELU, src/kernels.c:382-389).  Neither is correctly rounded, so no
// device formula returns the same bits for every argument, and with int8
// activation quantization behind them a single last-bit difference can move a
// rounding boundary and change every later frame.  Strict mode therefore
// carries two correction tables, built at open time from the host's own libm:
// for every float argument in the range where host and device can differ, a
// signed 4-bit field says by how many units in the last place the host's result
// differs from the device's base value (glibc 2.39: tanhf is off the correctly
// rounded value by up to 2 ulp on 15-50% of the arguments between 2^-25 and 8;
// expf by 1 ulp on about 0.06% between 2^-14 and 128).  The base value is the
// device's own single-precision function where the table covers the argument
// (any deterministic base within 7 ulp of the host will do, and the
// single-precision one costs a tenth of a double-precision evaluation), and the
// double-precision function rounded once to float elsewhere, where host and
// device agree everywhere.  Both functions are evaluated on |x| (tanhf
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
// expf arguments from here on (results below 2^-92) keep the double-precision base: the
// single-precision function is not held to a few ulp among denormal results
#define MB_EXP_FLOAT_HI_BITS 0x42800000u   // 64
// sinf (the codec's Snake activation, src/backend.c:643-658): below 2^-12 the host returns its
// argument, which is also the correctly rounded value; the table covers 2^-12 .. 64
#define MB_SIN_LO_BITS 0x39800000u    // 2^-12
#define MB_SIN_HI_BITS 0x42800000u    // 64
#define MB_LIBM_TANH 0
#define MB_LIBM_EXP 1
#define MB_LIBM_SIN 2


#ifdef __CUDACC__
// The base values the tables correct (used by the table builder and by every lookup).
__device__ __forceinline__ float mb_tanh_base(float a, uint32_t bits, bool have_tab) {
    return (have_tab && bits >= MB_TANH_LO_BITS && bits < MB_TANH_HI_BITS) ? tanhf(a) : (float)tanh((double)a);
}
__device__ __forceinline__ float mb_exp_base(float a, uint32_t bits, bool have_tab) {   // exp(-a), a >= 0
    return (have_tab && bits >= MB_EXP_LO_BITS && bits < MB_EXP_FLOAT_HI_BITS) ? expf(-a) : (float)exp(-(double)a);
}
__device__ __forceinline__ float mb_sin_base(float a) { return (float)sin((double)a); }   // a >= 0
__device__ __forceinline__ float mb_apply_nibble(float base, uint32_t word, uint32_t idx) {
    const uint32_t d = (word >> ((idx & 7u) * 4u)) & 15u;
    const int delta = (int)(d ^ 8u) - 8;   // sign-extend the nibble
    return __int_as_float(__float_as_int(base) + delta);   // raw bit patterns, as the builder subtracts them
}

// tanhf as the host computes it (tables present) or correctly rounded (absent).
__device__ __forceinline__ float mb_tanhf_host(float x, const uint32_t *tab) {
    const float a = fabsf(x);
    const uint32_t bits = (uint32_t)__float_as_int(a);
    float r = mb_tanh_base(a, bits, tab != nullptr);
    if (tab != nullptr && bits >= MB_TANH_LO_BITS && bits < MB_TANH_HI_BITS)
        r = mb_apply_nibble(r, __ldg(tab + ((bits - MB_TANH_LO_BITS) >> 3)), bits - MB_TANH_LO_BITS);
    return copysignf(r, x);
}

// The same in two steps, for code that evaluates many arguments in a row: mb_tanh_fetch
// only loads the table word of an argument (the index depends on the argument alone), so a
// batch of fetches can be in flight together before the first evaluation starts;
// mb_tanhf_host_with then gives mb_tanhf_host's bits from the fetched word (tables present).
__device__ __forceinline__ uint32_t mb_tanh_fetch(float x, const uint32_t *tab) {
    const uint32_t bits = (uint32_t)__float_as_int(fabsf(x));
    if (tab == nullptr || bits < MB_TANH_LO_BITS || bits >= MB_TANH_HI_BITS) return 0x88888888u;   // delta 0
    return __ldg(tab + ((bits - MB_TANH_LO_BITS) >> 3));
}
__device__ __forceinline__ float mb_tanhf_host_with(float x, uint32_t word, bool have_tab) {
    const float a = fabsf(x);
    const uint32_t bits = (uint32_t)__float_as_int(a);
    float r = mb_tanh_base(a, bits, have_tab);
    if (have_tab && bits >= MB_TANH_LO_BITS && bits < MB_TANH_HI_BITS) r = mb_apply_nibble(r, word, bits - MB_TANH_LO_BITS);
    return copysignf(r, x);
}

// sinf as the host computes it (table present) or correctly rounded (absent).  The table
// holds host - base as a difference of raw bit patterns, whatever the base's sign.
__device__ __forceinline__ float mb_sinf_host(float x, const uint32_t *tab) {
    const float a = fabsf(x);
    const uint32_t bits = (uint32_t)__float_as_int(a);
    float r = mb_sin_base(a);
    if (tab != nullptr && bits >= MB_SIN_LO_BITS && bits < MB_SIN_HI_BITS)
        r = mb_apply_nibble(r, __ldg(tab + ((bits - MB_SIN_LO_BITS) >> 3)), bits - MB_SIN_LO_BITS);
    return x < 0.0f ? -r : r;
}

// expf(x) for x <= 0 as the host computes it.
__device__ __forceinline__ float mb_expf_host(float x, const uint32_t *tab) {
    if (!(x <= 0.0f)) return (float)exp((double)x);
    const float a = -x;
    const uint32_t bits = (uint32_t)__float_as_int(a);
    float r = mb_exp_base(a, bits, tab != nullptr);
    if (tab != nullptr && bits >= MB_EXP_LO_BITS && bits < MB_EXP_HI_BITS)
        r = mb_apply_nibble(r, __ldg(tab + ((bits - MB_EXP_LO_BITS) >> 3)), bits - MB_EXP_LO_BITS);
    return r;
}
// Two-step form of mb_expf_host (x <= 0), as for tanhf: fetch the table word first.
__device__ __forceinline__ uint32_t mb_exp_fetch(float x, const uint32_t *tab) {
    const uint32_t bits = (uint32_t)__float_as_int(-x);
    if (tab == nullptr || !(x <= 0.0f) || bits < MB_EXP_LO_BITS || bits >= MB_EXP_HI_BITS) return 0x88888888u;   // delta 0
    return __ldg(tab + ((bits - MB_EXP_LO_BITS) >> 3));
}
__device__ __forceinline__ float mb_expf_host_with(float x, uint32_t word, bool have_tab) {
    if (!(x <= 0.0f)) return (float)exp((double)x);
    const float a = -x;
    const uint32_t bits = (uint32_t)__float_as_int(a);
    float r = mb_exp_base(a, bits, have_tab);
    if (have_tab && bits >= MB_EXP_LO_BITS && bits < MB_EXP_HI_BITS) r = mb_apply_nibble(r, word, bits - MB_EXP_LO_BITS);
    return r;
}
#endif
