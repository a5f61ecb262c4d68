// The rotary position encoding's arithmetic, shared by the kernels that apply it
// (rope_kv.cu on its own; attention_decode.cu when it rotates its own q and the new
// key), so that a key is the same bits whichever of them stored it.
//
// The angle pos * f_j is formed in fp64 from the fp64 table, reduced to (-pi, pi] in
// fp64 and only then rounded to fp32 for sincosf. A pair (lo, hi) = (x[j], x[j +
// rotary/2]) turns into (lo c - hi s, hi c + lo s), each as one multiply and one fused
// multiply-add, spelled out so that every caller rounds alike. The reference's form:
// pulsarlm-core/src/kernels/rope.cu:33-84.
#pragma once

#include "common.cuh"

__device__ __forceinline__ void rope_sincos(int pos, double radians_per_position, float& c, float& s) {
    const double kInvTwoPi = 0.15915494309189533576888376337251436;
    const double kTwoPi = 6.28318530717958647692528676655900577;
    const double turns = static_cast<double>(pos) * radians_per_position * kInvTwoPi;
    const double frac = turns - rint(turns);
    sincosf(static_cast<float>(frac * kTwoPi), &s, &c);
}

__device__ __forceinline__ float rope_lo(float lo, float hi, float c, float s) {
    return __fmaf_rn(lo, c, -__fmul_rn(hi, s));
}
__device__ __forceinline__ float rope_hi(float lo, float hi, float c, float s) {
    return __fmaf_rn(hi, c, __fmul_rn(lo, s));
}
