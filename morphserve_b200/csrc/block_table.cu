// Block-table maintenance: integer kernels, exact.  Each runs as ONE thread
// block (the tables are small: batch <= a few thousand rows, bitmap <= a few
// million bytes) so that prefix sums need no scratch memory and no second
// launch.  None of them synchronises with the host.
#include "common.cuh"

namespace mkv {

constexpr int kThreads = 1024;

// Exclusive prefix sum of one int per thread across the block; returns the
// exclusive offset of this thread and the block total in `total`.
__device__ __forceinline__ int block_exclusive_scan(int v, int &total, int *warp_sums /* [32] shared */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    __syncthreads();  // protect warp_sums from the previous use
    if (lane == 31) warp_sums[wid] = incl;
    __syncthreads();
    if (wid == 0) {
        int w = (lane < (int)(blockDim.x >> 5)) ? warp_sums[lane] : 0;
        int wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += n;
        }
        warp_sums[lane] = wi - w;  // exclusive offsets of the warps
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    total = warp_sums[32];
    return warp_sums[wid] + incl - v;
}

__global__ void __launch_bounds__(kThreads) block_need_kernel(const int32_t *__restrict__ num_allocated,
                                                            const int32_t *__restrict__ seq_ids,
                                                            const int32_t *__restrict__ target_lens, int batch,
                                                            int block_size, int num_rows, int32_t *__restrict__ need,
                                                            int64_t *__restrict__ totals) {
    __shared__ long long s_sum;
    __shared__ int s_neg;
    if (threadIdx.x == 0) {
        s_sum = 0;
        s_neg = 0;
    }
    __syncthreads();
    long long sum = 0;
    int neg = 0;
    for (int i = threadIdx.x; i < batch; i += blockDim.x) {
        int target = (target_lens[i] + (block_size - 1)) / block_size;
        const int s = seq_ids[i];
        if ((unsigned)s >= (unsigned)num_rows) {  // no such row: nothing is needed for it, reported like a shrink
            need[i] = 0;
            ++neg;
            continue;
        }
        int n = target - num_allocated[s];
        need[i] = n;
        sum += n;
        neg += (n < 0);
    }
    for (int d = 16; d > 0; d >>= 1) {
        sum += __shfl_down_sync(0xffffffffu, sum, d);
        neg += __shfl_down_sync(0xffffffffu, neg, d);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd((unsigned long long *)&s_sum, (unsigned long long)sum);
        atomicAdd(&s_neg, neg);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        totals[0] = s_sum;
        totals[1] = s_neg;
    }
}

constexpr int kPerThread = 16;

__global__ void __launch_bounds__(kThreads) bitmap_select_kernel(uint8_t *__restrict__ bitmap, int64_t lo, int64_t hi,
                                                               int want, int64_t max_out, int flip,
                                                               int64_t *__restrict__ out_ids,
                                                               int64_t *__restrict__ out_count,
                                                               int64_t *__restrict__ out_total) {
    __shared__ int warp_sums[33];
    int64_t carry = 0;
    const bool need_total = out_total != nullptr;
    for (int64_t base = lo; base < hi; base += (int64_t)kThreads * kPerThread) {
        if (!need_total && carry >= max_out) break;  // uniform across the block
        const int64_t i0 = base + (int64_t)threadIdx.x * kPerThread;
        unsigned mask = 0;
#pragma unroll
        for (int j = 0; j < kPerThread; ++j) {
            int64_t i = i0 + j;
            if (i < hi) {
                bool set = bitmap[i] != 0;
                if (set == (want != 0)) mask |= 1u << j;
            }
        }
        int total;
        int off = block_exclusive_scan(__popc(mask), total, warp_sums);
        int64_t pos = carry + off;
        while (mask) {
            int j = __ffs(mask) - 1;
            mask &= mask - 1;
            if (pos < max_out) {
                out_ids[pos] = i0 + j;
                if (flip) bitmap[i0 + j] = want ? 0 : 1;
            }
            ++pos;
        }
        carry += total;
    }
    if (threadIdx.x == 0) {
        if (out_count) *out_count = carry < max_out ? carry : max_out;
        if (out_total) *out_total = carry;
    }
}

// Compaction plan as ONE launch with no host round trip.  Rule (the reference has no compaction: its release needs a
// tail that is already empty, server/memory_utils.py:529-544): every live block with id >= target, ascending, moves to
// the first free ids below target, ascending.  src_ids/dst_ids receive the pairs; the bitmap is updated (destinations
// used, sources free) only when every source has a destination.  result[0] = pairs to move (0 when refused),
// result[1] = 1 when refused (too few free ids below target, or more sources than `capacity`), result[2] = live ids
// found at or above target, result[3] = free ids found below target (the search stops once it has enough).
__global__ void __launch_bounds__(kThreads) compact_plan_kernel(uint8_t *__restrict__ bitmap, int64_t total,
                                                              int64_t target, int64_t *__restrict__ src_ids,
                                                              int64_t *__restrict__ dst_ids, int64_t capacity,
                                                              int64_t *__restrict__ result) {
    __shared__ int warp_sums[33];
    int64_t found[2] = {0, 0};
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
        const int64_t lo = pass == 0 ? target : 0, hi = pass == 0 ? total : target;
        const uint8_t want = pass == 0 ? 0 : 1;  // live above the target, free below it
        int64_t *out = pass == 0 ? src_ids : dst_ids;
        const int64_t max_out = pass == 0 ? capacity : min(found[0], capacity);
        int64_t carry = 0;
        for (int64_t base = lo; base < hi; base += (int64_t)kThreads * kPerThread) {
            if (pass == 1 && carry >= found[0]) break;  // uniform across the block
            const int64_t i0 = base + (int64_t)threadIdx.x * kPerThread;
            unsigned mask = 0;
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) {
                const int64_t i = i0 + j;
                if (i < hi && (bitmap[i] != 0) == (want != 0)) mask |= 1u << j;
            }
            int sum;
            const int off = block_exclusive_scan(__popc(mask), sum, warp_sums);
            int64_t pos = carry + off;
            while (mask) {
                const int j = __ffs(mask) - 1;
                mask &= mask - 1;
                if (pos < max_out) out[pos] = i0 + j;
                ++pos;
            }
            carry += sum;
        }
        found[pass] = carry;
    }
    __syncthreads();  // the pairs written above are read by other threads of this block below
    const bool ok = found[0] <= capacity && found[1] >= found[0];
    if (ok)
        for (int64_t i = threadIdx.x; i < found[0]; i += kThreads) {
            bitmap[dst_ids[i]] = 0;
            bitmap[src_ids[i]] = 1;
        }
    if (threadIdx.x == 0) {
        result[0] = ok ? found[0] : 0;
        result[1] = ok ? 0 : 1;
        result[2] = found[0];
        result[3] = found[1];
    }
}

// allocate_blocks_for_seqs (worker/block_manager.py:87-112) as ONE launch with no host round trip:
// need per sequence -> first-fit ascending selection of sum(need) free ids (the order of
// torch.nonzero(is_block_free)[:n], :75) -> rows and counts updated in batch order.  Nothing is changed
// unless the whole request can be served.  status[0] += blocks allocated; status[1..3] are sticky error
// counts (sequences that own more blocks than they need; blocks missing; sequences whose row is full).
__global__ void __launch_bounds__(kThreads) block_allocate_kernel(
    int32_t *__restrict__ num_allocated, int32_t *__restrict__ block_table, int64_t table_stride,
    const int32_t *__restrict__ seq_ids, const int32_t *__restrict__ target_lens, int batch, int block_size,
    uint8_t *__restrict__ bitmap, int64_t num_blocks, int32_t *__restrict__ need, int64_t *__restrict__ ids,
    int64_t ids_capacity, int64_t *__restrict__ status, int num_rows) {
    __shared__ int warp_sums[33];
    __shared__ long long s_sum;
    __shared__ int s_neg, s_full;
    if (threadIdx.x == 0) {
        s_sum = 0;
        s_neg = 0;
        s_full = 0;
    }
    __syncthreads();
    long long sum = 0;
    int neg = 0, full = 0;
    for (int i = threadIdx.x; i < batch; i += blockDim.x) {
        const int s = seq_ids[i];
        if ((unsigned)s >= (unsigned)num_rows) {  // a sequence id without a row: the whole request is refused
            need[i] = 0;
            ++full;
            continue;
        }
        const int have = num_allocated[s];
        const int n = (target_lens[i] + (block_size - 1)) / block_size - have;
        need[i] = n;
        sum += n;
        neg += (n < 0);
        full += ((int64_t)have + n > table_stride);
    }
    for (int d = 16; d > 0; d >>= 1) {
        sum += __shfl_down_sync(0xffffffffu, sum, d);
        neg += __shfl_down_sync(0xffffffffu, neg, d);
        full += __shfl_down_sync(0xffffffffu, full, d);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd((unsigned long long *)&s_sum, (unsigned long long)sum);
        atomicAdd(&s_neg, neg);
        atomicAdd(&s_full, full);
    }
    __syncthreads();
    const int64_t total = s_sum;
    if (s_neg > 0 || s_full > 0 || total > ids_capacity) {
        if (threadIdx.x == 0) {
            status[1] += s_neg;
            status[3] += s_full + (total > ids_capacity);
        }
        return;
    }
    if (total <= 0) return;

    // first `total` free ids, ascending; the bitmap is not touched yet
    int64_t carry = 0;
    for (int64_t base = 0; base < num_blocks && carry < total; base += (int64_t)kThreads * kPerThread) {
        const int64_t i0 = base + (int64_t)threadIdx.x * kPerThread;
        unsigned mask = 0;
#pragma unroll
        for (int j = 0; j < kPerThread; ++j)
            if (i0 + j < num_blocks && bitmap[i0 + j] != 0) mask |= 1u << j;
        int found;
        const int off = block_exclusive_scan(__popc(mask), found, warp_sums);
        int64_t pos = carry + off;
        while (mask) {
            const int j = __ffs(mask) - 1;
            mask &= mask - 1;
            if (pos < total) ids[pos] = i0 + j;
            ++pos;
        }
        carry += found;
    }
    if (carry < total) {
        if (threadIdx.x == 0) status[2] += total - carry;
        return;
    }
    __syncthreads();  // ids[] written by the whole block are visible to it
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) bitmap[ids[i]] = 0;
    int64_t taken = 0;
    for (int base = 0; base < batch; base += kThreads) {
        const int i = base + threadIdx.x;
        const int n = (i < batch) ? need[i] : 0;
        int chunk_total;
        const int off = block_exclusive_scan(n, chunk_total, warp_sums);
        if (i < batch && n > 0) {
            const int64_t s = seq_ids[i];
            const int have = num_allocated[s];
            for (int j = 0; j < n; ++j) block_table[s * table_stride + have + j] = (int32_t)ids[taken + off + j];
            num_allocated[s] = have + n;
        }
        taken += chunk_total;
    }
    if (threadIdx.x == 0) status[0] += total;
}

__global__ void bitmap_scatter_kernel(uint8_t *__restrict__ bitmap, int64_t bitmap_len,
                                      const int64_t *__restrict__ ids, int64_t n, int value) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t id = ids[i];
        if (id >= 0 && id < bitmap_len) bitmap[id] = (uint8_t)(value != 0);
    }
}

__global__ void __launch_bounds__(kThreads) block_table_set_kernel(int32_t *__restrict__ num_allocated,
                                                                 int32_t *__restrict__ block_table,
                                                                 int64_t table_stride,
                                                                 const int64_t *__restrict__ candidates,
                                                                 const int32_t *__restrict__ seq_ids,
                                                                 const int32_t *__restrict__ need, int batch,
                                                                 int num_rows) {
    __shared__ int warp_sums[33];
    int64_t carry = 0;
    for (int base = 0; base < batch; base += kThreads) {
        const int i = base + threadIdx.x;
        int n = (i < batch) ? max(need[i], 0) : 0;
        int total;
        int off = block_exclusive_scan(n, total, warp_sums);
        if (i < batch && n > 0 && (unsigned)seq_ids[i] < (unsigned)num_rows) {
            const int64_t s = seq_ids[i];
            const int have = num_allocated[s];
            int room = (int)max((int64_t)0, min((int64_t)n, table_stride - have));  // never write past the row
            for (int j = 0; j < room; ++j)
                block_table[s * table_stride + have + j] = (int32_t)candidates[carry + off + j];
            num_allocated[s] = have + room;  // the count never names columns the row does not have
        }
        carry += total;
    }
}

__global__ void __launch_bounds__(kThreads) block_table_unset_kernel(int32_t *__restrict__ num_allocated,
                                                                   const int32_t *__restrict__ block_table,
                                                                   int64_t table_stride,
                                                                   const int32_t *__restrict__ seq_ids, int batch,
                                                                   uint8_t *__restrict__ is_block_free,
                                                                   int64_t num_blocks, int32_t *__restrict__ gathered,
                                                                   int64_t gathered_capacity,
                                                                   int64_t *__restrict__ total_out, int accumulate,
                                                                   int num_rows) {
    __shared__ int warp_sums[33];
    int64_t carry = 0;
    for (int base = 0; base < batch; base += kThreads) {
        const int i = base + threadIdx.x;
        int64_t s = 0;
        int n = 0;
        if (i < batch && (unsigned)seq_ids[i] < (unsigned)num_rows) {
            s = seq_ids[i];
            n = (int)min((int64_t)max(num_allocated[s], 0), table_stride);  // a row holds table_stride columns
        }
        int total;
        int off = block_exclusive_scan(n, total, warp_sums);
        if (i < batch) {
            for (int j = 0; j < n; ++j) {
                int32_t id = block_table[s * table_stride + j];
                if (gathered && carry + off + j < gathered_capacity) gathered[carry + off + j] = id;
                if (id >= 0 && id < num_blocks) is_block_free[id] = 1;
            }
        }
        carry += total;
    }
    __syncthreads();  // every count was read before any is cleared (duplicate ids in a batch)
    for (int i = threadIdx.x; i < batch; i += blockDim.x)
        if ((unsigned)seq_ids[i] < (unsigned)num_rows) num_allocated[seq_ids[i]] = 0;
    if (threadIdx.x == 0 && total_out) *total_out = accumulate ? *total_out + carry : carry;
}

__global__ void __launch_bounds__(kThreads) block_table_count_kernel(const int32_t *__restrict__ num_allocated,
                                                                   const int32_t *__restrict__ seq_ids, int batch,
                                                                   int64_t *__restrict__ total_out, int num_rows) {
    __shared__ long long s_sum;
    if (threadIdx.x == 0) s_sum = 0;
    __syncthreads();
    long long sum = 0;
    for (int i = threadIdx.x; i < batch; i += blockDim.x)
        if ((unsigned)seq_ids[i] < (unsigned)num_rows) sum += num_allocated[seq_ids[i]];
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, d);
    if ((threadIdx.x & 31) == 0) atomicAdd((unsigned long long *)&s_sum, (unsigned long long)sum);
    __syncthreads();
    if (threadIdx.x == 0) *total_out = s_sum;
}

}  // namespace mkv

using namespace mkv;

extern "C" {

int mkv_block_need(int device, void *stream, const int32_t *num_allocated, int num_rows, const int32_t *seq_ids,
                   const int32_t *target_lens, int batch, int block_size, int32_t *need, int64_t *totals) {
    if (batch < 0 || block_size < 1 || num_rows < 0) return MKV_ERR_SHAPE;
    if (!totals) return MKV_ERR_NULL;
    if (batch > 0 && (!num_allocated || !seq_ids || !target_lens || !need)) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    block_need_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(num_allocated, seq_ids, target_lens, batch,
                                                               block_size, num_rows, need, totals);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_block_allocate(int device, void *stream, int32_t *num_allocated, int num_rows, int32_t *block_table,
                       int64_t table_stride, const int32_t *seq_ids, const int32_t *target_lens, int batch, int block_size,
                       uint8_t *bitmap, int64_t num_blocks, int32_t *need, int64_t *ids, int64_t ids_capacity,
                       int64_t *status) {
    if (batch < 0 || block_size < 1 || table_stride < 1 || num_blocks < 0 || ids_capacity < 0 || num_rows < 0)
        return MKV_ERR_SHAPE;
    if (!status) return MKV_ERR_NULL;
    if (batch == 0) return MKV_OK;
    if (!num_allocated || !block_table || !seq_ids || !target_lens || !need) return MKV_ERR_NULL;
    if ((num_blocks > 0 && !bitmap) || (ids_capacity > 0 && !ids)) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    block_allocate_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(num_allocated, block_table, table_stride, seq_ids,
                                                                   target_lens, batch, block_size, bitmap, num_blocks,
                                                                   need, ids, ids_capacity, status, num_rows);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_bitmap_select(int device, void *stream, uint8_t *bitmap, int64_t lo, int64_t hi, int want,
                      int64_t max_out, int flip, int64_t *out_ids, int64_t *out_count, int64_t *out_total) {
    if (lo < 0 || hi < lo || max_out < 0) return MKV_ERR_SHAPE;
    if (!bitmap && hi > lo) return MKV_ERR_NULL;
    if (max_out > 0 && !out_ids) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    bitmap_select_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(bitmap, lo, hi, want, max_out, flip, out_ids,
                                                                  out_count, out_total);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_compact_plan(int device, void *stream, uint8_t *bitmap, int64_t num_blocks, int64_t target,
                     int64_t *src_ids, int64_t *dst_ids, int64_t capacity, int64_t *result) {
    if (num_blocks < 0 || target < 0 || target > num_blocks || capacity < 0) return MKV_ERR_SHAPE;
    if (!result || (num_blocks > 0 && !bitmap)) return MKV_ERR_NULL;
    if (capacity > 0 && (!src_ids || !dst_ids)) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    compact_plan_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(bitmap, num_blocks, target, src_ids, dst_ids,
                                                                 capacity, result);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_bitmap_scatter(int device, void *stream, uint8_t *bitmap, int64_t bitmap_len, const int64_t *ids,
                       int64_t n, int value) {
    if (n < 0 || bitmap_len < 0) return MKV_ERR_SHAPE;
    if (n == 0) return MKV_OK;
    if (!bitmap || !ids) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    int blocks = (int)(ceil_div64(n, 256) > 1024 ? 1024 : ceil_div64(n, 256));
    bitmap_scatter_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(bitmap, bitmap_len, ids, n, value);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_block_table_set(int device, void *stream, int32_t *num_allocated, int num_rows, int32_t *block_table,
                        int64_t table_stride, const int64_t *candidates, const int32_t *seq_ids,
                        const int32_t *need, int batch) {
    if (batch < 0 || table_stride < 1 || num_rows < 0) return MKV_ERR_SHAPE;
    if (batch == 0) return MKV_OK;
    if (!num_allocated || !block_table || !candidates || !seq_ids || !need) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    block_table_set_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(num_allocated, block_table, table_stride,
                                                                    candidates, seq_ids, need, batch, num_rows);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_block_table_unset(int device, void *stream, int32_t *num_allocated, int num_rows, const int32_t *block_table,
                          int64_t table_stride, const int32_t *seq_ids, int batch, uint8_t *is_block_free,
                          int64_t num_blocks, int32_t *gathered, int64_t gathered_capacity, int64_t *total_out,
                          int accumulate) {
    if (batch < 0 || table_stride < 1 || num_blocks < 0 || gathered_capacity < 0 || num_rows < 0) return MKV_ERR_SHAPE;
    if (batch == 0) return MKV_OK;
    if (!num_allocated || !block_table || !seq_ids || !is_block_free) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    block_table_unset_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(num_allocated, block_table, table_stride,
                                                                      seq_ids, batch, is_block_free, num_blocks,
                                                                      gathered, gathered_capacity, total_out,
                                                                      accumulate, num_rows);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_block_table_count(int device, void *stream, const int32_t *num_allocated, int num_rows,
                          const int32_t *seq_ids, int batch, int64_t *total_out) {
    if (batch < 0 || num_rows < 0) return MKV_ERR_SHAPE;
    if (!total_out) return MKV_ERR_NULL;
    if (batch > 0 && (!num_allocated || !seq_ids)) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    block_table_count_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(num_allocated, seq_ids, batch, total_out,
                                                                      num_rows);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

}  // extern "C"
