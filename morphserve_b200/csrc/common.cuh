// Shared host/device helpers of the morphkv library (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "morphkv.h"

namespace mkv {

// Device-side view of mkv_pool, passed by value as a kernel parameter so that
// the segment bases are read from the constant bank.
struct PoolView {
    int32_t num_segments;
    int32_t elem_bytes;
    int32_t num_layers;
    int32_t num_kv_heads;
    int32_t block_size;
    int32_t head_dim;
    int64_t num_blocks_org;
    int64_t chunk_blocks;
    int64_t total_blocks;
    int64_t block_bytes;  // bytes of one block in K (or V): L*Hkv*bs*D*elem
    char *k_base[MKV_MAX_SEGMENTS];
    char *v_base[MKV_MAX_SEGMENTS];
};

// Byte offset of block `blk` inside its segment and the segment index.
// Follows worker/kernels/paged_attn.py:354-360 of the reference.
__device__ __forceinline__ void locate_block(const PoolView &p, int64_t blk, int &seg, int64_t &row) {
    if (blk < p.num_blocks_org) {
        seg = 0;
        row = blk;
    } else {
        int64_t rel = blk - p.num_blocks_org;
        int64_t j = rel / p.chunk_blocks;
        seg = 1 + (int)j;
        row = rel - j * p.chunk_blocks;
    }
}

__device__ __forceinline__ bool block_in_pool(const PoolView &p, int64_t blk) {
    return blk >= 0 && blk < p.total_blocks;
}

// ---- host side -----------------------------------------------------------
int set_cuda_error(cudaError_t e);            // records text, returns MKV_ERR_CUDA
int validate_pool(const mkv_pool *pool, PoolView *out);

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
            switched = (err == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

#define MKV_CUDA_TRY(expr)                                   \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return mkv::set_cuda_error(_e); \
    } while (0)

#define MKV_LAUNCH_CHECK() MKV_CUDA_TRY(cudaGetLastError())

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace mkv
