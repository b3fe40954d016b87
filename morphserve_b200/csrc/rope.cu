// Rotary position embedding of q and k in place, the step in front of the KV
// append.  Element-wise, HBM/latency bound.  Follows the reference kernel's
// arithmetic (worker/kernels/rotary_emb.py:7-41): the halves [0, D/2) and
// [D/2, D) of every head rotate as (x0*cos - x1*sin, x0*sin + x1*cos), rounded
// either as the compiled reference kernel rounds (default) or operation by
// operation, as its source reads; see rope.cuh.
#include <atomic>
#include <stdlib.h>

#include "rope.cuh"

namespace mkv {

static std::atomic<int> g_rope_fused{-1};
bool rope_fused_rounding() {
    int v = g_rope_fused.load(std::memory_order_relaxed);
    if (v < 0) {
        const char *e = getenv("MKV_ROPE_ROUNDING");  // "written" = every operation rounds; default: as compiled
        v = (e && e[0] == 'w') ? 0 : 1;
        g_rope_fused.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

// fp16 rows: one thread per 8-element piece of the low half of one head (16-byte loads), kRopeUnroll pieces per
// loop pass with all of their loads issued before the first store (4 x 16 B of rows in flight per thread: with two,
// a full SM held 64 KiB in flight, which is about what 1/148 of the HBM bandwidth needs and leaves no slack).
constexpr int kRopeUnroll = 2;
__global__ void rope_f16_kernel(__half *__restrict__ q, __half *__restrict__ k, const __half *__restrict__ cos_t,
                                const __half *__restrict__ sin_t, int64_t num_tokens, int num_q_heads,
                                int num_kv_heads, int head_dim, bool fused) {
    const int half_dim = head_dim >> 1;
    const int pieces = half_dim >> 3;
    const int heads = num_q_heads + num_kv_heads;
    const int64_t total = num_tokens * heads * pieces;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += stride * kRopeUnroll) {
        __half *row[kRopeUnroll];
        uint4 x0[kRopeUnroll], x1[kRopeUnroll], c[kRopeUnroll], s[kRopeUnroll];
        int piece[kRopeUnroll];
#pragma unroll
        for (int u = 0; u < kRopeUnroll; ++u) {
            const int64_t idx = base + u * stride;
            if (idx >= total) {
                row[u] = nullptr;
                continue;
            }
            piece[u] = (int)(idx % pieces);
            const int64_t r = idx / pieces;
            const int head = (int)(r % heads);
            const int64_t tok = r / heads;
            row[u] = head < num_q_heads ? q + (tok * num_q_heads + head) * head_dim
                                        : k + (tok * num_kv_heads + (head - num_q_heads)) * head_dim;
            x0[u] = *reinterpret_cast<const uint4 *>(row[u] + piece[u] * 8);
            x1[u] = *reinterpret_cast<const uint4 *>(row[u] + half_dim + piece[u] * 8);
            c[u] = __ldg(reinterpret_cast<const uint4 *>(cos_t + tok * half_dim + piece[u] * 8));
            s[u] = __ldg(reinterpret_cast<const uint4 *>(sin_t + tok * half_dim + piece[u] * 8));
        }
#pragma unroll
        for (int u = 0; u < kRopeUnroll; ++u) {
            if (row[u] == nullptr) continue;
            rope_rotate8(x0[u], x1[u], c[u], s[u], fused);
            *reinterpret_cast<uint4 *>(row[u] + piece[u] * 8) = x0[u];
            *reinterpret_cast<uint4 *>(row[u] + half_dim + piece[u] * 8) = x1[u];
        }
    }
}

// Any head_dim / fp32 rows: one thread per element pair.  fp16 tables, as the reference builds them
// (worker/model.py:240-241); with fp32 rows the products and sums round to fp32.
template <typename T>
__global__ void rope_scalar_kernel(T *__restrict__ q, T *__restrict__ k, const __half *__restrict__ cos_t,
                                   const __half *__restrict__ sin_t, int64_t num_tokens, int num_q_heads,
                                   int num_kv_heads, int head_dim, bool fused) {
    const int half_dim = head_dim >> 1;
    const int heads = num_q_heads + num_kv_heads;
    const int64_t total = num_tokens * heads * half_dim;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(idx % half_dim);
        const int64_t r = idx / half_dim;
        const int head = (int)(r % heads);
        const int64_t tok = r / heads;
        T *row = head < num_q_heads ? q + (tok * num_q_heads + head) * head_dim
                                    : k + (tok * num_kv_heads + (head - num_q_heads)) * head_dim;
        const __half c = cos_t[tok * half_dim + d], s = sin_t[tok * half_dim + d];
        const T x0 = row[d], x1 = row[half_dim + d];
        if constexpr (sizeof(T) == 2) {
            if (fused) {
                row[d] = __hfma(x0, c, __hneg(__hmul_rn(x1, s)));
                row[half_dim + d] = __hfma(x0, s, __hmul_rn(x1, c));
            } else {
                row[d] = __hsub_rn(__hmul_rn(x0, c), __hmul_rn(x1, s));
                row[half_dim + d] = __hadd_rn(__hmul_rn(x0, s), __hmul_rn(x1, c));
            }
        } else {
            const float cf = __half2float(c), sf = __half2float(s);
            if (fused) {
                row[d] = __fmaf_rn(x0, cf, -__fmul_rn(x1, sf));
                row[half_dim + d] = __fmaf_rn(x0, sf, __fmul_rn(x1, cf));
            } else {
                row[d] = __fsub_rn(__fmul_rn(x0, cf), __fmul_rn(x1, sf));
                row[half_dim + d] = __fadd_rn(__fmul_rn(x0, sf), __fmul_rn(x1, cf));
            }
        }
    }
}

}  // namespace mkv

using namespace mkv;

extern "C" int mkv_rotary_embedding(int device, void *stream, void *q, void *k, const void *cos_table,
                                    const void *sin_table, int64_t num_tokens, int num_q_heads, int num_kv_heads,
                                    int head_dim, int elem_bytes) {
    if (num_tokens < 0 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 2 || (head_dim & 1)) return MKV_ERR_SHAPE;
    if (elem_bytes != 2 && elem_bytes != 4) return MKV_ERR_DTYPE;
    if (num_tokens == 0) return MKV_OK;
    if (!q || !k || !cos_table || !sin_table) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    int sms = 0;
    int st = mkv_sm_count(device, &sms);
    if (st) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const int half_dim = head_dim / 2;
    const int64_t heads = (int64_t)num_q_heads + num_kv_heads;
    const bool vec = elem_bytes == 2 && half_dim % 8 == 0 &&
                     (((uintptr_t)q | (uintptr_t)k | (uintptr_t)cos_table | (uintptr_t)sin_table) % 16) == 0;
    const int64_t items = num_tokens * heads * (vec ? half_dim / 8 : half_dim);
    int64_t blocks = ceil_div64(items, threads);
    const int64_t cap = (int64_t)sms * 16;
    if (blocks > cap) blocks = cap;
    const bool fused = rope_fused_rounding();
    if (vec)
        rope_f16_kernel<<<(unsigned)blocks, threads, 0, s>>>((__half *)q, (__half *)k, (const __half *)cos_table,
                                                            (const __half *)sin_table, num_tokens, num_q_heads,
                                                            num_kv_heads, head_dim, fused);
    else if (elem_bytes == 2)
        rope_scalar_kernel<__half><<<(unsigned)blocks, threads, 0, s>>>(
            (__half *)q, (__half *)k, (const __half *)cos_table, (const __half *)sin_table, num_tokens, num_q_heads,
            num_kv_heads, head_dim, fused);
    else
        rope_scalar_kernel<float><<<(unsigned)blocks, threads, 0, s>>>(
            (float *)q, (float *)k, (const __half *)cos_table, (const __half *)sin_table, num_tokens, num_q_heads,
            num_kv_heads, head_dim, fused);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

extern "C" int mkv_rope_set_rounding(int as_compiled) {
    mkv::g_rope_fused.store(as_compiled ? 1 : 0, std::memory_order_relaxed);
    return MKV_OK;
}
