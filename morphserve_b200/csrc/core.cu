// Library plumbing: status text, pool validation, device info, and the two
// host-only entry points (chunk sizing, block swap).
#include <string.h>

#include <vector>

#include <mutex>

#include "common.cuh"

namespace mkv {

static thread_local char g_cuda_error[256] = "";

int set_cuda_error(cudaError_t e) {
    const char *s = cudaGetErrorString(e);
    strncpy(g_cuda_error, s ? s : "unknown", sizeof(g_cuda_error) - 1);
    g_cuda_error[sizeof(g_cuda_error) - 1] = 0;
    return MKV_ERR_CUDA;
}

int validate_pool(const mkv_pool *pool, PoolView *out) {
    if (!pool) return MKV_ERR_NULL;
    if (pool->num_segments < 1 || pool->num_segments > MKV_MAX_SEGMENTS) return MKV_ERR_SHAPE;
    if (pool->elem_bytes != 2 && pool->elem_bytes != 4) return MKV_ERR_DTYPE;
    if (pool->num_layers < 1 || pool->num_kv_heads < 1 || pool->block_size < 1 || pool->head_dim < 1)
        return MKV_ERR_SHAPE;
    if (pool->num_blocks_org < 0) return MKV_ERR_SHAPE;
    if (pool->num_segments > 1 && pool->chunk_blocks < 1) return MKV_ERR_SHAPE;
    PoolView v;
    memset(&v, 0, sizeof(v));
    v.num_segments = pool->num_segments;
    v.elem_bytes = pool->elem_bytes;
    v.num_layers = pool->num_layers;
    v.num_kv_heads = pool->num_kv_heads;
    v.block_size = pool->block_size;
    v.head_dim = pool->head_dim;
    v.num_blocks_org = pool->num_blocks_org;
    v.chunk_blocks = pool->num_segments > 1 ? pool->chunk_blocks : 1;
    v.total_blocks = pool->num_blocks_org + (int64_t)(pool->num_segments - 1) * v.chunk_blocks;
    v.block_bytes = (int64_t)pool->num_layers * pool->num_kv_heads * pool->block_size * pool->head_dim *
                    pool->elem_bytes;
    for (int i = 0; i < pool->num_segments; ++i) {
        bool empty_org = (i == 0 && pool->num_blocks_org == 0);
        if (!empty_org && (!pool->k_base[i] || !pool->v_base[i])) return MKV_ERR_NULL;
        v.k_base[i] = (char *)pool->k_base[i];
        v.v_base[i] = (char *)pool->v_base[i];
    }
    *out = v;
    return MKV_OK;
}

}  // namespace mkv

using namespace mkv;

extern "C" {

int mkv_version(void) { return 100; }

const char *mkv_status_string(int status) {
    switch (status) {
        case MKV_OK: return "ok";
        case MKV_ERR_NULL: return "a required pointer is NULL";
        case MKV_ERR_SHAPE: return "size, stride or count out of range or unsupported";
        case MKV_ERR_DTYPE: return "element size must be 2 (fp16) or 4 (fp32)";
        case MKV_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case MKV_ERR_RANGE: return "id out of range";
        case MKV_ERR_CUDA: return "CUDA runtime error";
        case MKV_ERR_NOSPACE: return "not enough space";
        case MKV_ERR_ALIGN: return "pointer or row size not aligned as required";
        case MKV_ERR_TOO_LARGE: return "request exceeds the built-in scratch of the no-allocation entry point";
        default: return "unknown status";
    }
}

const char *mkv_last_cuda_error(void) { return g_cuda_error; }

int mkv_sm_count(int device, int *sm_count) {
    static int cache[64];
    if (!sm_count) return MKV_ERR_NULL;
    if (device < 0 || device >= 64) return MKV_ERR_RANGE;
    int v = cache[device];
    if (v == 0) {
        MKV_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
        cache[device] = v;
    }
    *sm_count = v;
    return MKV_OK;
}

int mkv_chunk_layout(uint64_t org_start, uint64_t org_size, uint64_t quant_size, int num_layers,
                     int num_kv_heads, int block_size, int head_dim, int elem_bytes, uint64_t *k_addr,
                     uint64_t *v_addr, int64_t *num_blocks) {
    if (!k_addr || !v_addr || !num_blocks) return MKV_ERR_NULL;
    if (num_layers < 1 || num_kv_heads < 1 || block_size < 1 || head_dim < 1) return MKV_ERR_SHAPE;
    if (elem_bytes != 2 && elem_bytes != 4) return MKV_ERR_DTYPE;
    uint64_t layer_end = org_start + quant_size;
    uint64_t kv_start = (layer_end + 255u) & ~(uint64_t)255u;
    uint64_t used = kv_start - org_start;
    if (used >= org_size) return MKV_ERR_NOSPACE;
    uint64_t available = org_size - used;
    uint64_t kv_block = 2ull * num_layers * num_kv_heads * head_dim * elem_bytes * block_size;
    uint64_t n = available / kv_block;
    if (n == 0) return MKV_ERR_NOSPACE;
    *k_addr = kv_start;
    *v_addr = kv_start + n * (kv_block / 2);
    *num_blocks = (int64_t)n;
    return MKV_OK;
}

int mkv_swap_blocks(int device, void *stream, const mkv_pool *pool, void *k_swap, void *v_swap,
                    int64_t num_swap_blocks, const int64_t *src_ids, const int64_t *dst_ids, int64_t n,
                    int is_swap_in, int64_t *num_copies) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (n < 0) return MKV_ERR_SHAPE;
    if (num_copies) *num_copies = 0;
    if (n == 0) return MKV_OK;
    if (!k_swap || !v_swap || !src_ids || !dst_ids) return MKV_ERR_NULL;

    // validate every id before the first copy is issued
    auto seg_of = [&](int64_t b) -> int {
        return b < pv.num_blocks_org ? 0 : 1 + (int)((b - pv.num_blocks_org) / pv.chunk_blocks);
    };
    for (int64_t i = 0; i < n; ++i) {
        int64_t dev_id = is_swap_in ? dst_ids[i] : src_ids[i];
        int64_t host_id = is_swap_in ? src_ids[i] : dst_ids[i];
        if (dev_id < 0 || dev_id >= pv.total_blocks) return MKV_ERR_RANGE;
        if (host_id < 0 || host_id >= num_swap_blocks) return MKV_ERR_RANGE;
    }
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    cudaStream_t s = (cudaStream_t)stream;
    int64_t copies = 0;
    int64_t i = 0;
    while (i < n) {
        const int64_t *dev_ids = is_swap_in ? dst_ids : src_ids;
        int64_t j = i + 1;
        int seg = seg_of(dev_ids[i]);
        while (j < n && src_ids[j] == src_ids[j - 1] + 1 && dst_ids[j] == dst_ids[j - 1] + 1 &&
               seg_of(dev_ids[j]) == seg)
            ++j;
        int64_t row = seg == 0 ? dev_ids[i] : (dev_ids[i] - pv.num_blocks_org) - (int64_t)(seg - 1) * pv.chunk_blocks;
        size_t bytes = (size_t)(j - i) * (size_t)pv.block_bytes;
        char *dk = pv.k_base[seg] + row * pv.block_bytes;
        char *dv = pv.v_base[seg] + row * pv.block_bytes;
        int64_t host_id = is_swap_in ? src_ids[i] : dst_ids[i];
        char *hk = (char *)k_swap + host_id * pv.block_bytes;
        char *hv = (char *)v_swap + host_id * pv.block_bytes;
        if (is_swap_in) {
            MKV_CUDA_TRY(cudaMemcpyAsync(dk, hk, bytes, cudaMemcpyHostToDevice, s));
            MKV_CUDA_TRY(cudaMemcpyAsync(dv, hv, bytes, cudaMemcpyHostToDevice, s));
        } else {
            MKV_CUDA_TRY(cudaMemcpyAsync(hk, dk, bytes, cudaMemcpyDeviceToHost, s));
            MKV_CUDA_TRY(cudaMemcpyAsync(hv, dv, bytes, cudaMemcpyDeviceToHost, s));
        }
        copies += 2;
        i = j;
    }
    if (num_copies) *num_copies = copies;
    return MKV_OK;
}

// Layer slab upload: the quantised (or the original fp16) image of a transformer layer from host memory
// into the layer's slab on the GPU, complete on return (csrc/src/memory_manager.cpp:179-231, :274-320).
// The reference creates and destroys a stream per call; here one non-blocking copy stream per device is
// kept, so the copy overlaps whatever runs on the compute streams and the call costs no stream set-up.
int mkv_slab_upload(int device, void *dst_device, size_t dst_capacity, const void *src_host, size_t bytes) {
    static cudaStream_t copy_streams[64];
    static std::mutex copy_streams_lock;  // callers may come from different host threads
    if (device < 0 || device >= 64) return MKV_ERR_RANGE;
    if (bytes > dst_capacity) return MKV_ERR_NOSPACE;
    if (bytes == 0) return MKV_OK;
    if (!dst_device || !src_host) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    std::lock_guard<std::mutex> hold(copy_streams_lock);  // one upload per process at a time: they share PCIe anyway
    if (!copy_streams[device]) MKV_CUDA_TRY(cudaStreamCreateWithFlags(&copy_streams[device], cudaStreamNonBlocking));
    MKV_CUDA_TRY(cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, copy_streams[device]));
    MKV_CUDA_TRY(cudaStreamSynchronize(copy_streams[device]));
    return MKV_OK;
}

}  // extern "C"
