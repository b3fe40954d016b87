// KV append (decode) and prefill scatter into the paged pool: vectorised byte
// copies through the block table.  HBM/latency bound; no arithmetic.
#include "common.cuh"

namespace mkv {

// One thread per VEC-byte piece of one (sequence, kv head) row, K and V.
// Row = head_dim*elem bytes, contiguous in both source and pool.
template <int VEC>
__global__ void store_kv_decode_kernel(const char *__restrict__ k, const char *__restrict__ v,
                                       const __grid_constant__ PoolView pool,
                                       const int32_t *__restrict__ block_table, int64_t table_stride,
                                       const int32_t *__restrict__ seq_ids,
                                       const int32_t *__restrict__ seq_lens, int batch, int cur_layer,
                                       int row_bytes) {
    const int pieces_per_row = row_bytes / VEC;
    const int64_t per_seq = (int64_t)pool.num_kv_heads * pieces_per_row;
    const int64_t total = (int64_t)batch * per_seq * 2;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int which = (int)(idx / ((int64_t)batch * per_seq));  // 0 = K, 1 = V
        int64_t r = idx - (int64_t)which * batch * per_seq;
        int b = (int)(r / per_seq);
        int rem = (int)(r - (int64_t)b * per_seq);
        int h = rem / pieces_per_row;
        int piece = rem - h * pieces_per_row;
        int len = seq_lens[b];
        if (len <= 0) continue;
        int pos = len - 1;
        int64_t blk = block_table[(int64_t)seq_ids[b] * table_stride + pos / pool.block_size];
        if (!block_in_pool(pool, blk)) continue;
        int slot = pos % pool.block_size;
        int seg;
        int64_t row;
        locate_block(pool, blk, seg, row);
        int64_t dst_off = row * pool.block_bytes +
                          ((((int64_t)cur_layer * pool.num_kv_heads + h) * pool.block_size + slot) * (int64_t)row_bytes) +
                          (int64_t)piece * VEC;
        int64_t src_off = ((int64_t)b * pool.num_kv_heads + h) * row_bytes + (int64_t)piece * VEC;
        const char *src = (which ? v : k) + src_off;
        char *dst = (which ? pool.v_base[seg] : pool.k_base[seg]) + dst_off;
        if (VEC == 16)
            *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
        else if (VEC == 4)
            *reinterpret_cast<uint32_t *>(dst) = *reinterpret_cast<const uint32_t *>(src);
        else
            *reinterpret_cast<uint16_t *>(dst) = *reinterpret_cast<const uint16_t *>(src);
    }
}

// grid = (logical block of the prompt, prompt).  A thread block moves the <= bs
// tokens of one logical block for all heads, K and V, transposing
// [token, head, :] -> [head, token, :].
template <int VEC>
__global__ void store_kv_prefill_kernel(const char *__restrict__ k, const char *__restrict__ v,
                                       const __grid_constant__ PoolView pool,
                                        const int32_t *__restrict__ block_table, int64_t table_stride,
                                        const int32_t *__restrict__ seq_ids,
                                        const int32_t *__restrict__ start_locs,
                                        const int32_t *__restrict__ seq_lens, int cur_layer, int row_bytes) {
    const int i = blockIdx.y;
    const int lb = blockIdx.x;
    const int len = seq_lens[i];
    const int t0 = lb * pool.block_size;
    if (t0 >= len) return;
    const int ntok = min(pool.block_size, len - t0);
    const int64_t blk = block_table[(int64_t)seq_ids[i] * table_stride + lb];
    if (!block_in_pool(pool, blk)) return;
    int seg;
    int64_t row;
    locate_block(pool, blk, seg, row);
    const int64_t start = start_locs[i];
    const int pieces_per_row = row_bytes / VEC;
    const int per_tok = pool.num_kv_heads * pieces_per_row;
    const int total = ntok * per_tok * 2;
    const int64_t blk_base = row * pool.block_bytes +
                             (int64_t)cur_layer * pool.num_kv_heads * pool.block_size * (int64_t)row_bytes;
    // U pieces per thread and pass: all loads are issued before the first store, so that a thread has U requests
    // in flight instead of one (the kernel is latency bound otherwise: 59 % of DRAM peak with one).
    constexpr int U = 4;
    const int half = ntok * per_tok;
    for (int base = threadIdx.x; base < total; base += U * blockDim.x) {
        const char *src[U];
        char *dst[U];
        bool on[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + u * blockDim.x;
            on[u] = idx < total;
            const int which = idx >= half;
            const int r = idx - which * half;
            const int t = r / per_tok;
            const int rem = r - t * per_tok;
            const int h = rem / pieces_per_row;
            const int piece = rem - h * pieces_per_row;
            const int64_t src_off = ((start + t0 + t) * pool.num_kv_heads + h) * (int64_t)row_bytes + (int64_t)piece * VEC;
            const int64_t dst_off = blk_base + ((int64_t)h * pool.block_size + t) * row_bytes + (int64_t)piece * VEC;
            src[u] = (which ? v : k) + src_off;
            dst[u] = (which ? pool.v_base[seg] : pool.k_base[seg]) + dst_off;
        }
        if (VEC == 16) {
            uint4 x[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (on[u]) x[u] = __ldcs(reinterpret_cast<const uint4 *>(src[u]));   // read once: streaming
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (on[u]) *reinterpret_cast<uint4 *>(dst[u]) = x[u];
        } else if (VEC == 4) {
            uint32_t x[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (on[u]) x[u] = *reinterpret_cast<const uint32_t *>(src[u]);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (on[u]) *reinterpret_cast<uint32_t *>(dst[u]) = x[u];
        } else {
            uint16_t x[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (on[u]) x[u] = *reinterpret_cast<const uint16_t *>(src[u]);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (on[u]) *reinterpret_cast<uint16_t *>(dst[u]) = x[u];
        }
    }
}

static int pick_vec(const PoolView &pv, const void *k, const void *v, int row_bytes) {
    bool a16 = (row_bytes % 16 == 0) && (((uintptr_t)k | (uintptr_t)v) % 16 == 0);
    for (int i = 0; i < pv.num_segments && a16; ++i)
        a16 = (((uintptr_t)pv.k_base[i] | (uintptr_t)pv.v_base[i]) % 16 == 0);
    if (a16) return 16;
    bool a4 = (row_bytes % 4 == 0) && (((uintptr_t)k | (uintptr_t)v) % 4 == 0);
    for (int i = 0; i < pv.num_segments && a4; ++i)
        a4 = (((uintptr_t)pv.k_base[i] | (uintptr_t)pv.v_base[i]) % 4 == 0);
    return a4 ? 4 : 2;
}

}  // namespace mkv

using namespace mkv;

extern "C" {

int mkv_store_kv_decode(int device, void *stream, const void *k, const void *v, const mkv_pool *pool,
                        const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids,
                        const int32_t *seq_lens, int batch, int cur_layer) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (batch < 0 || table_stride < 1) return MKV_ERR_SHAPE;
    if (cur_layer < 0 || cur_layer >= pv.num_layers) return MKV_ERR_RANGE;
    if (batch == 0) return MKV_OK;
    if (!k || !v || !block_table || !seq_ids || !seq_lens) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    const int row_bytes = pv.head_dim * pv.elem_bytes;
    const int vec = pick_vec(pv, k, v, row_bytes);
    const int64_t total = (int64_t)batch * pv.num_kv_heads * (row_bytes / vec) * 2;
    const int threads = 256;
    int64_t blocks = ceil_div64(total, threads);
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(V)                                                                                          \
    store_kv_decode_kernel<V><<<(unsigned)blocks, threads, 0, s>>>((const char *)k, (const char *)v, pv,   \
                                                                  block_table, table_stride, seq_ids,      \
                                                                  seq_lens, batch, cur_layer, row_bytes)
    if (vec == 16) LAUNCH(16);
    else if (vec == 4) LAUNCH(4);
    else LAUNCH(2);
#undef LAUNCH
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_store_kv_prefill(int device, void *stream, const void *k, const void *v, const mkv_pool *pool,
                         const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids,
                         const int32_t *start_locs, const int32_t *seq_lens, int num_seqs, int max_seq_len,
                         int cur_layer) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (num_seqs < 0 || max_seq_len < 0 || table_stride < 1) return MKV_ERR_SHAPE;
    if (cur_layer < 0 || cur_layer >= pv.num_layers) return MKV_ERR_RANGE;
    if (num_seqs == 0 || max_seq_len == 0) return MKV_OK;
    if (!k || !v || !block_table || !seq_ids || !seq_lens || !start_locs) return MKV_ERR_NULL;
    if (num_seqs > 65535) return MKV_ERR_SHAPE;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    const int row_bytes = pv.head_dim * pv.elem_bytes;
    const int vec = pick_vec(pv, k, v, row_bytes);
    dim3 grid((unsigned)ceil_div64(max_seq_len, pv.block_size), (unsigned)num_seqs);
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(V)                                                                                         \
    store_kv_prefill_kernel<V><<<grid, threads, 0, s>>>((const char *)k, (const char *)v, pv, block_table, \
                                                       table_stride, seq_ids, start_locs, seq_lens,       \
                                                       cur_layer, row_bytes)
    if (vec == 16) LAUNCH(16);
    else if (vec == 4) LAUNCH(4);
    else LAUNCH(2);
#undef LAUNCH
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

}  // extern "C"
