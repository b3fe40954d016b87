// Rotary-embedding arithmetic shared by the stand-alone kernel and the decode-attention prologue.
#pragma once

#include "common.cuh"

namespace mkv {

// (x0, x1) -> (x0*c - x1*s, x0*s + x1*c) on two fp16 lanes, each product and each sum rounded to
// fp16 separately (no fma contraction), as the reference's fp16 arithmetic does.
__device__ __forceinline__ void rope_rotate2(uint32_t &x0, uint32_t &x1, uint32_t c, uint32_t s) {
    const __half2 a = *reinterpret_cast<const __half2 *>(&x0), b = *reinterpret_cast<const __half2 *>(&x1);
    const __half2 hc = *reinterpret_cast<const __half2 *>(&c), hs = *reinterpret_cast<const __half2 *>(&s);
    const __half2 r0 = __hsub2_rn(__hmul2_rn(a, hc), __hmul2_rn(b, hs));
    const __half2 r1 = __hadd2_rn(__hmul2_rn(a, hs), __hmul2_rn(b, hc));
    x0 = *reinterpret_cast<const uint32_t *>(&r0);
    x1 = *reinterpret_cast<const uint32_t *>(&r1);
}

__device__ __forceinline__ void rope_rotate8(uint4 &x0, uint4 &x1, const uint4 &c, const uint4 &s) {
    rope_rotate2(x0.x, x1.x, c.x, s.x);
    rope_rotate2(x0.y, x1.y, c.y, s.y);
    rope_rotate2(x0.z, x1.z, c.z, s.z);
    rope_rotate2(x0.w, x1.w, c.w, s.w);
}

}  // namespace mkv
