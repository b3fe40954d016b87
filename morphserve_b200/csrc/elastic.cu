// Elastic pool resize, device side: whole-block copies for compaction and the
// block-table remap that follows.  HBM-bound streaming copy; no arithmetic.
#include "common.cuh"

namespace mkv {

constexpr int kCopyThreads = 256;
// 16-byte vectors in flight per thread, i.e. the slice one thread block copies at a time: 8 KiB inside the pool,
// 32 KiB to or from the host swap space.  Measured on the compaction of a 32 GiB pool (3683 blocks of 2 x 1 MiB moved,
// plan and table remap included): slices of 8 / 16 / 32 / 64 KiB with plain loads and stores 6.36 / 6.27 / 6.22 /
// 5.88 TB/s read+write; streaming hints (ld.cs / st.cs) cost 3-4 % inside the pool; the grid is a multiple of 16
// blocks per SM (24 per SM: 5.95 TB/s).
constexpr int kVecPool = 2, kVecHost = 8;
template <int MODE>
__host__ __device__ constexpr int vec_per_thread() { return MODE == 0 ? kVecPool : kVecHost; }
template <int MODE>
__host__ __device__ constexpr int slice_bytes() { return kCopyThreads * vec_per_thread<MODE>() * 16; }

// Work item = (pair, K|V, slice).  grid-stride over items; each thread issues
// all its loads before its stores.
// MODE 0: pool -> pool (compaction).  MODE 1: host swap space -> pool (swap in).
// MODE 2: pool -> host swap space (swap out).  The host side must be pinned memory
// that the device can address (zero-copy over PCIe / NVLink-C2C).
template <int MODE>
__global__ void __launch_bounds__(kCopyThreads) copy_blocks_kernel(const __grid_constant__ PoolView pool,
                                                                  const int64_t *__restrict__ src_ids,
                                                                  const int64_t *__restrict__ dst_ids, int64_t n,
                                                                  int slices_per_block, char *host_k, char *host_v,
                                                                  int64_t host_blocks,
                                                                  const int64_t *__restrict__ n_dev) {
    if (n_dev) n = min(n, *n_dev);  // pair count decided on the device (compaction plan); n is then the capacity
    const int64_t items = n * 2 * slices_per_block;
    const int64_t vec_per_block = pool.block_bytes / 16;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t pair = item / (2 * slices_per_block);
        const int rem = (int)(item - pair * 2 * slices_per_block);
        const int which = rem / slices_per_block;
        const int slice = rem - which * slices_per_block;
        const int64_t s = src_ids[pair], d = dst_ids[pair];
        const uint4 *sp;
        uint4 *dp;
        if (MODE == 1) {
            if (s < 0 || s >= host_blocks) continue;
            sp = reinterpret_cast<const uint4 *>((which ? host_v : host_k) + s * pool.block_bytes);
        } else {
            if (!block_in_pool(pool, s)) continue;
            int seg;
            int64_t row;
            locate_block(pool, s, seg, row);
            sp = reinterpret_cast<const uint4 *>((which ? pool.v_base[seg] : pool.k_base[seg]) + row * pool.block_bytes);
        }
        if (MODE == 2) {
            if (d < 0 || d >= host_blocks) continue;
            dp = reinterpret_cast<uint4 *>((which ? host_v : host_k) + d * pool.block_bytes);
        } else {
            if (!block_in_pool(pool, d)) continue;
            int seg;
            int64_t row;
            locate_block(pool, d, seg, row);
            dp = reinterpret_cast<uint4 *>((which ? pool.v_base[seg] : pool.k_base[seg]) + row * pool.block_bytes);
        }
        constexpr int VEC = vec_per_thread<MODE>();
        const int64_t v0 = (int64_t)slice * (slice_bytes<MODE>() / 16) + threadIdx.x;
        uint4 r[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            int64_t vi = v0 + (int64_t)j * kCopyThreads;
            if (vi < vec_per_block) r[j] = MODE == 0 ? sp[vi] : __ldcs(sp + vi);
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            int64_t vi = v0 + (int64_t)j * kCopyThreads;
            if (vi < vec_per_block) {
                if (MODE == 0) dp[vi] = r[j];
                else __stcs(dp + vi, r[j]);
            }
        }
    }
}

// One warp per table row; lanes stride over the live columns.  An entry is
// looked up in the ascending src list by binary search.
__global__ void remap_block_table_kernel(int32_t *__restrict__ block_table, int64_t table_stride, int64_t num_rows,
                                         const int32_t *__restrict__ num_allocated,
                                         const int64_t *__restrict__ src_ids, const int64_t *__restrict__ dst_ids,
                                         int64_t n, const int64_t *__restrict__ n_dev) {
    if (n_dev) n = min(n, *n_dev);
    if (n <= 0) return;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t lowest = src_ids[0];
    for (int64_t r = warp; r < num_rows; r += nwarps) {
        int64_t c = num_allocated[r];
        if (c > table_stride) c = table_stride;
        for (int64_t j = lane; j < c; j += 32) {
            const int64_t e = block_table[r * table_stride + j];
            if (e < lowest) continue;
            int64_t lo = 0, hi = n;
            while (lo < hi) {
                int64_t mid = (lo + hi) >> 1;
                if (src_ids[mid] < e) lo = mid + 1;
                else hi = mid;
            }
            if (lo < n && src_ids[lo] == e) block_table[r * table_stride + j] = (int32_t)dst_ids[lo];
        }
    }
}

}  // namespace mkv

using namespace mkv;

extern "C" {

static int copy_blocks_launch(int device, void *stream, const mkv_pool *pool, const int64_t *src_ids,
                              const int64_t *dst_ids, int64_t n, const int64_t *n_dev) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (n < 0) return MKV_ERR_SHAPE;
    if (n == 0) return MKV_OK;
    if (!src_ids || !dst_ids) return MKV_ERR_NULL;
    if (pv.block_bytes % 16 != 0) return MKV_ERR_ALIGN;
    for (int i = 0; i < pv.num_segments; ++i)
        if ((((uintptr_t)pv.k_base[i]) | ((uintptr_t)pv.v_base[i])) % 16 != 0) return MKV_ERR_ALIGN;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    int sms = 148;
    mkv_sm_count(device, &sms);
    const int slices = (int)ceil_div64(pv.block_bytes, slice_bytes<0>());
    const int64_t items = n * 2 * slices;
    int64_t grid = (int64_t)sms * 64;  // 8 x 256 threads resident per SM, eight rounds of them
    if (grid > items) grid = items;
    copy_blocks_kernel<0><<<(unsigned)grid, kCopyThreads, 0, (cudaStream_t)stream>>>(pv, src_ids, dst_ids, n, slices,
                                                                                     nullptr, nullptr, 0, n_dev);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_copy_blocks(int device, void *stream, const mkv_pool *pool, const int64_t *src_ids,
                    const int64_t *dst_ids, int64_t n) {
    return copy_blocks_launch(device, stream, pool, src_ids, dst_ids, n, nullptr);
}

int mkv_copy_blocks_counted(int device, void *stream, const mkv_pool *pool, const int64_t *src_ids,
                            const int64_t *dst_ids, int64_t capacity, const int64_t *n_dev) {
    if (!n_dev) return MKV_ERR_NULL;
    return copy_blocks_launch(device, stream, pool, src_ids, dst_ids, capacity, n_dev);
}

int mkv_swap_blocks_pinned(int device, void *stream, const mkv_pool *pool, void *k_swap, void *v_swap,
                           int64_t num_swap_blocks, const int64_t *src_ids, const int64_t *dst_ids, int64_t n,
                           int is_swap_in) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (n < 0 || num_swap_blocks < 0) return MKV_ERR_SHAPE;
    if (n == 0) return MKV_OK;
    if (!k_swap || !v_swap || !src_ids || !dst_ids) return MKV_ERR_NULL;
    if (pv.block_bytes % 16 != 0 || (((uintptr_t)k_swap | (uintptr_t)v_swap) % 16) != 0) return MKV_ERR_ALIGN;
    for (int i = 0; i < pv.num_segments; ++i)
        if ((((uintptr_t)pv.k_base[i]) | ((uintptr_t)pv.v_base[i])) % 16 != 0) return MKV_ERR_ALIGN;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    // the swap space must be host memory the device can address
    for (void *hp : {k_swap, v_swap}) {
        cudaPointerAttributes attr;
        MKV_CUDA_TRY(cudaPointerGetAttributes(&attr, hp));
        if (attr.type != cudaMemoryTypeHost && attr.type != cudaMemoryTypeManaged) return MKV_ERR_ALIGN;
    }
    int sms = 148;
    mkv_sm_count(device, &sms);
    const int slices = (int)ceil_div64(pv.block_bytes, slice_bytes<1>());
    const int64_t items = n * 2 * slices;
    int64_t grid = (int64_t)sms * 4;
    if (grid > items) grid = items;
    if (is_swap_in)
        copy_blocks_kernel<1><<<(unsigned)grid, kCopyThreads, 0, (cudaStream_t)stream>>>(
            pv, src_ids, dst_ids, n, slices, (char *)k_swap, (char *)v_swap, num_swap_blocks, nullptr);
    else
        copy_blocks_kernel<2><<<(unsigned)grid, kCopyThreads, 0, (cudaStream_t)stream>>>(
            pv, src_ids, dst_ids, n, slices, (char *)k_swap, (char *)v_swap, num_swap_blocks, nullptr);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

static int remap_launch(int device, void *stream, int32_t *block_table, int64_t table_stride, int64_t num_rows,
                        const int32_t *num_allocated, const int64_t *src_ids, const int64_t *dst_ids, int64_t n,
                        const int64_t *n_dev) {
    if (n < 0 || num_rows < 0 || table_stride < 1) return MKV_ERR_SHAPE;
    if (n == 0 || num_rows == 0) return MKV_OK;
    if (!block_table || !num_allocated || !src_ids || !dst_ids) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    const int threads = 256;
    int64_t grid = ceil_div64(num_rows, threads / 32);
    if (grid > 148 * 8) grid = 148 * 8;
    remap_block_table_kernel<<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>(
        block_table, table_stride, num_rows, num_allocated, src_ids, dst_ids, n, n_dev);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_remap_block_table(int device, void *stream, int32_t *block_table, int64_t table_stride,
                          int64_t num_rows, const int32_t *num_allocated, const int64_t *src_ids,
                          const int64_t *dst_ids, int64_t n) {
    return remap_launch(device, stream, block_table, table_stride, num_rows, num_allocated, src_ids, dst_ids, n,
                        nullptr);
}

int mkv_remap_block_table_counted(int device, void *stream, int32_t *block_table, int64_t table_stride,
                                  int64_t num_rows, const int32_t *num_allocated, const int64_t *src_ids,
                                  const int64_t *dst_ids, int64_t capacity, const int64_t *n_dev) {
    if (!n_dev) return MKV_ERR_NULL;
    return remap_launch(device, stream, block_table, table_stride, num_rows, num_allocated, src_ids, dst_ids,
                        capacity, n_dev);
}

}  // extern "C"
