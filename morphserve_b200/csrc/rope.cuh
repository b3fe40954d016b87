// Rotary-embedding arithmetic shared by the stand-alone kernel and the decode-attention prologue.
#pragma once

#include "common.cuh"

namespace mkv {

// (x0, x1) -> (x0*c - x1*s, x0*s + x1*c) on two fp16 lanes.  The reference writes this in fp16
// (worker/kernels/rotary_emb.py:36-41) and there are two ways to round it:
//   as written: each product and each sum rounded to fp16 separately, which is what the kernel's source gives when it
//     is run operation by operation (the Triton interpreter);
//   as compiled (`fused`): Triton's compiler contracts the FIRST product of each output into the add, so that
//     x0*c - rn(x1*s) and x0*s + rn(x1*c) round once.  This is what the reference computes on a GPU (verified
//     against the kernel compiled by Triton 3.6 for sm_100: all outputs equal).
__device__ __forceinline__ void rope_rotate2(uint32_t &x0, uint32_t &x1, uint32_t c, uint32_t s, bool fused) {
    const __half2 a = *reinterpret_cast<const __half2 *>(&x0), b = *reinterpret_cast<const __half2 *>(&x1);
    const __half2 hc = *reinterpret_cast<const __half2 *>(&c), hs = *reinterpret_cast<const __half2 *>(&s);
    __half2 r0, r1;
    if (fused) {
        r0 = __hfma2(a, hc, __hneg2(__hmul2_rn(b, hs)));
        r1 = __hfma2(a, hs, __hmul2_rn(b, hc));
    } else {
        r0 = __hsub2_rn(__hmul2_rn(a, hc), __hmul2_rn(b, hs));
        r1 = __hadd2_rn(__hmul2_rn(a, hs), __hmul2_rn(b, hc));
    }
    x0 = *reinterpret_cast<const uint32_t *>(&r0);
    x1 = *reinterpret_cast<const uint32_t *>(&r1);
}

__device__ __forceinline__ void rope_rotate8(uint4 &x0, uint4 &x1, const uint4 &c, const uint4 &s, bool fused) {
    rope_rotate2(x0.x, x1.x, c.x, s.x, fused);
    rope_rotate2(x0.y, x1.y, c.y, s.y, fused);
    rope_rotate2(x0.z, x1.z, c.z, s.z, fused);
    rope_rotate2(x0.w, x1.w, c.w, s.w, fused);
}

bool rope_fused_rounding();  // process-wide choice (mkv_rope_set_rounding), read per call

}  // namespace mkv
