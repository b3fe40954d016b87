/*
 * morphkv.h - C ABI of the B200 (sm_100a) KV-cache hot path for MorphServe / SwiftLLM.
 *
 * The library replaces, behind the reference's Python worker API, the Triton
 * kernels of worker/kernels/{paged_attn,kvcache_mgmt,block_mgmt}.py and the
 * block-copy / pool-carving routines of csrc/src/{block_swapping,memory_manager}.cpp
 * (paths relative to the reference project root).  Every entry point cites the
 * reference interface it stands in for.
 *
 * Conventions
 *  - plain C linkage, plain pointers and sizes; no torch / pybind types.
 *  - every function returns an int status: MKV_OK (0) or a negative mkv_status.
 *    Nothing throws, exits, traps or prints.  Arguments are validated on the
 *    host before any launch.
 *  - the caller owns every buffer and the stream.  Unless stated otherwise a call
 *    allocates nothing, never synchronises and never reads device memory from
 *    the host; it enqueues work on `stream` and returns.
 *  - `device` is the CUDA ordinal the pointers live on; the calling thread's
 *    current device is saved and restored around the call, so calls may come
 *    from any host thread.
 *  - pointers marked "device" must be device-accessible; "host" pointers are
 *    ordinary host memory.
 */
#ifndef MORPHKV_H
#define MORPHKV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MKV_MAX_SEGMENTS 65 /* original pool + up to 64 elastic chunks */

typedef enum mkv_status {
    MKV_OK = 0,
    MKV_ERR_NULL = -1,      /* a required pointer is NULL */
    MKV_ERR_SHAPE = -2,     /* a size / stride / count is out of range or unsupported */
    MKV_ERR_DTYPE = -3,     /* element size not 2 (fp16) or 4 (fp32) */
    MKV_ERR_WORKSPACE = -4, /* workspace missing, misaligned or too small */
    MKV_ERR_RANGE = -5,     /* an id (layer, block, segment) is out of range */
    MKV_ERR_CUDA = -6,      /* a CUDA runtime call failed; see mkv_last_cuda_error */
    MKV_ERR_NOSPACE = -7,   /* no room: chunk does not fit / too few free blocks */
    MKV_ERR_ALIGN = -8,     /* a pointer or row size is not aligned as required */
    MKV_ERR_TOO_LARGE = -9  /* the request needs more scratch than the no-allocation entry point has */
} mkv_status;

/*
 * The paged pool, K and V separately, each segment laid out as
 *   [blocks, num_layers, num_kv_heads, block_size, head_dim]   (contiguous)
 * (reference: worker/model.py:180-190).  Segment 0 is the original pool with
 * `num_blocks_org` blocks; segment 1+j is elastic chunk j with `chunk_blocks`
 * blocks, holding block ids num_blocks_org + j*chunk_blocks + i.  This is the
 * id -> address rule of worker/kernels/paged_attn.py:354-360 with the chunk
 * bases stated explicitly instead of derived by negative offsets from chunk 0.
 */
typedef struct mkv_pool {
    int32_t num_segments; /* 1 + number of elastic chunks, <= MKV_MAX_SEGMENTS */
    int32_t elem_bytes;   /* 2 = fp16, 4 = fp32 */
    int32_t num_layers;
    int32_t num_kv_heads;
    int32_t block_size;   /* tokens per block */
    int32_t head_dim;
    int64_t num_blocks_org;
    int64_t chunk_blocks; /* ignored when num_segments == 1 */
    void *k_base[MKV_MAX_SEGMENTS]; /* device */
    void *v_base[MKV_MAX_SEGMENTS]; /* device */
} mkv_pool;

/* ---- library --------------------------------------------------------- */
int mkv_version(void);
const char *mkv_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library. */
const char *mkv_last_cuda_error(void);
/* Number of SMs of `device` (cached after the first call). */
int mkv_sm_count(int device, int *sm_count);

/* ---- decode attention ------------------------------------------------ */
/*
 * Replaces paged_attention() and its Triton phases
 * (worker/kernels/paged_attn.py:59-240 phase 1, :243-437 elastic phase 1,
 * :658-696 phase 2, :700-1015 wrapper).
 *
 * The work is split in two calls.  mkv_attn_plan runs once per decode step (the
 * schedule depends only on the sequence lengths, which all layers of a step
 * share); mkv_paged_attention_decode runs once per layer and uses the plan.
 * Both need the same `workspace` (device memory, 256-byte aligned, at least
 * mkv_attn_workspace_bytes(...) bytes, contents private to the library between
 * the plan and the last attention call that uses it).  Calls that share a
 * workspace must be ordered on the GPU (same stream or event-ordered).
 *
 * fast path: fp16, head_dim 128, block_size 16, num_q_heads/num_kv_heads <= 16.
 * Everything else (fp32 pools, other head_dim <= 256 / block sizes) takes a
 * plain kernel that ignores the plan.
 */
size_t mkv_attn_workspace_bytes(int device, int batch, int num_q_heads, int num_kv_heads,
                                int head_dim, int max_blocks_per_seq_in_batch);

int mkv_attn_plan(int device, void *stream, void *workspace, size_t workspace_bytes,
                  const int32_t *seq_lens /* device [batch] */, const int32_t *seq_ids /* device [batch] */,
                  int batch, int num_q_heads,
                  int num_kv_heads, int head_dim, int block_size,
                  int max_blocks_per_seq_in_batch /* host upper bound of ceil(len/block_size) */);

int mkv_paged_attention_decode(
    int device, void *stream,
    const void *q,               /* device [batch, num_q_heads, head_dim], pool dtype, contiguous */
    void *o,                     /* device [batch, num_q_heads, head_dim], pool dtype, contiguous */
    const mkv_pool *pool,        /* host */
    const int32_t *block_table,  /* device [*, table_stride] */
    int64_t table_stride,        /* = max_blocks_per_seq */
    const int32_t *seq_ids,      /* device [batch]: row of the block table */
    const int32_t *seq_lens,     /* device [batch]: tokens to attend to (includes the newest) */
    int batch, int num_q_heads, int cur_layer, float softmax_scale,
    int max_blocks_per_seq_in_batch, /* the value given to mkv_attn_plan */
    void *workspace, size_t workspace_bytes);

/*
 * mkv_store_kv_decode + mkv_paged_attention_decode of one layer in ONE launch:
 * the warp that attends over the block holding token len-1 of a (sequence, kv
 * head) also writes that token's new K/V row (k_new, v_new: device
 * [batch, num_kv_heads, head_dim]) into the pool and into its staged tile.
 * Same results as the two separate calls (the append is bit-exact); saves one
 * launch per layer.  Shapes outside the fast path fall back to the two kernels.
 * Replaces the pair of call sites worker/layers/transformer_layer.py:117-126 and
 * :181-187 when the caller opts in.
 */
int mkv_paged_attention_decode_append(
    int device, void *stream, const void *q, void *o, const void *k_new, const void *v_new,
    const mkv_pool *pool, const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids,
    const int32_t *seq_lens, int batch, int num_q_heads, int cur_layer, float softmax_scale,
    int max_blocks_per_seq_in_batch, void *workspace, size_t workspace_bytes);

/*
 * Decode attention whose result is PUSHED into several output matrices at once:
 * row b, columns [out_col_offset + hq*head_dim, +head_dim) of every
 * out_ptrs[i] (row stride out_row_stride elements, fp16).  Made for KV-head
 * sharding across GPUs (no counterpart in the single-GPU reference): each rank
 * attends over its own KV heads and stores its column slice straight into every
 * rank's full-width [batch, Hq_total*head_dim] matrix through peer-mapped
 * pointers - plain stores over NVLink from the kernel's epilogue, so the
 * "all-gather" rides inside the attention launch.  Nothing is loaded from a
 * peer.  Before a rank reads its matrix the peers' stores must have landed: either
 * the caller runs a barrier across the ranks after the launch, or it passes
 * `ready_ptrs` (HOST array of n_ready <= 8 device-accessible int32 words, one per
 * destination, each in THAT destination's memory; NULL / 0: no signal): when the last store
 * of the launch is done the kernel writes `epoch` into every one of them behind a
 * system-wide fence, and the destination waits with mkv_wait_ready.  Epochs must grow
 * from launch to launch.  out_ptrs is a HOST array of n_out <= 8 device-accessible
 * pointers; k_new / v_new as in mkv_paged_attention_decode_append, or NULL.
 * fp16 / head_dim 128 / block 16.
 */
int mkv_paged_attention_decode_push(
    int device, void *stream, const void *q, void *const *out_ptrs, int n_out, int64_t out_row_stride,
    int64_t out_col_offset, int32_t *const *ready_ptrs, int n_ready, int32_t epoch,
    const void *k_new, const void *v_new, const mkv_pool *pool,
    const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids, const int32_t *seq_lens,
    int batch, int num_q_heads, int cur_layer, float softmax_scale, int max_blocks_per_seq_in_batch,
    void *workspace, size_t workspace_bytes);

/*
 * Waits, on `stream`, until flags[0..n) (device memory of THIS GPU, written by the peers' push launches) have all
 * reached `epoch`, for at most timeout_ns (capped at two seconds): one warp polls with system-scope acquire loads.
 * A flag that does not arrive in time sets its bit in *status (device int32, accumulated; the caller clears and
 * reads it) and the kernel returns - a rank that died or skipped its launch costs the others the timeout, never a
 * hang.  Kernels queued behind it on the stream may read the pushed data.  No counterpart in the reference.
 */
int mkv_wait_ready(int device, void *stream, const int32_t *flags, int n, int32_t epoch, int64_t timeout_ns,
                   int32_t *status);

/*
 * Rotary position embedding of q [num_tokens, Hq, D] and k [num_tokens, Hkv, D] in place
 * (replaces rotary_embedding_inplace, worker/kernels/rotary_emb.py:43-58, the step in front
 * of store_kvcache: worker/layers/transformer_layer.py:93-98).  cos_table / sin_table:
 * fp16 [num_tokens, D/2], the rows of the reference's tables gathered for the tokens'
 * positions (worker/model.py:240-241, 432-433).  Halves [0, D/2) and [D/2, D) of every head
 * become (x0*cos - x1*sin, x0*sin + x1*cos), rounded as mkv_rope_set_rounding selects.
 * elem_bytes 2 (fp16) or 4 (fp32).
 */
int mkv_rotary_embedding(int device, void *stream, void *q, void *k, const void *cos_table, const void *sin_table,
                         int64_t num_tokens, int num_q_heads, int num_kv_heads, int head_dim, int elem_bytes);

/*
 * How the rotation is rounded (process-wide; applies to mkv_rotary_embedding and to the rotation fused into the
 * decode kernel).  The reference writes it in the data's precision (worker/kernels/rotary_emb.py:36-41):
 *   as_compiled != 0 (default): x0*cos - rn(x1*sin) and x0*sin + rn(x1*cos), the first product fused into the add
 *     with one rounding - what the reference's kernel computes once Triton has compiled it for a GPU (bit-equal to
 *     the kernel compiled by Triton 3.6 for sm_100);
 *   as_compiled == 0: every product and every sum rounded on its own - what the same source gives when run
 *     operation by operation (the Triton interpreter); also selected by MKV_ROPE_ROUNDING=written.
 */
int mkv_rope_set_rounding(int as_compiled);

/*
 * mkv_rotary_embedding (decode rows) + mkv_store_kv_decode + mkv_paged_attention_decode of one
 * layer in ONE launch: q is rotated as it is loaded, the k_new row is rotated before it is
 * patched into the staged tile and written to the pool.  rope_cos / rope_sin: fp16
 * [batch, D/2], 16-byte aligned.  On the fused path (fp16, head_dim 128, block 16) q and k_new
 * are left untouched in memory; for other shapes they are rotated in place by the stand-alone
 * kernel first - either way `o` and the pool hold the same values as the three separate calls.
 */
int mkv_paged_attention_decode_rope_append(
    int device, void *stream, void *q, void *o, void *k_new, const void *v_new, const void *rope_cos,
    const void *rope_sin, const mkv_pool *pool, const int32_t *block_table, int64_t table_stride,
    const int32_t *seq_ids, const int32_t *seq_lens, int batch, int num_q_heads, int cur_layer, float softmax_scale,
    int max_blocks_per_seq_in_batch, void *workspace, size_t workspace_bytes);

/*
 * Tuning knobs of the decode kernel (process-wide; not needed for normal use):
 * warps per SM and ring stages (values <= 0 keep the current ones) and the
 * number of work units planned per worker warp (<= 0 keeps).  Changing the item
 * factor changes mkv_attn_workspace_bytes: re-query it and plan again; changing
 * warps / stages needs a new plan too (a plan is made for a number of worker
 * warps; a launch with another number refuses to run, error bit 1).
 * `split_balance` (< 0 keeps; default 1.5): a sequence is only cut into chunks
 * when it is longer than split_balance x the mean number of KV blocks per worker
 * warp, since every cut costs fp32 partial rows and a merge; 0 cuts as finely as
 * the item factor allows.  `loader` (other values keep): 0 = K/V tiles arrive by 16-byte
 * cp.async (default), 1 = by TMA (cp.async.bulk.tensor, pools of up to 8 segments), 2 = the
 * tensor-core kernel is not used at all: every shape goes through the plain kernel (one warp per
 * query head, fp32 FMA) - an independent implementation for cross-checks at full size.
 */
int mkv_attn_configure(int warps, int stages, double item_factor, double split_balance, int loader);

/*
 * How the plan deals the launch's K/V tiles to the worker warps (process-wide tuning knobs).
 *   mode 0: always in chunks drawn from a shared counter, longest first (sequences longer than the chunk are cut);
 *   mode 1 (default): as 0 while no sequence has to be cut (none longer than `ratio` chunks, default 1); otherwise
 *      every worker gets an equal contiguous range of the tile stream, sequences are cut only where a range ends (all
 *      workers finish together), pieces that meet in one thread block are merged through shared memory and the rest
 *      in two levels;
 *   mode 2: equal ranges whenever the workspace allows it.
 * `unit_cost` (default 3): with equal ranges, what starting a unit is worth in tiles - every (sequence, kv head)
 * counts as that many tiles more than it has, so a worker that is dealt many short sequences is dealt fewer tiles.
 * mode / unit_cost < 0 and ratio < 0 keep the current setting.
 * Part of the scheduling the reference leaves to its launch grid (worker/kernels/paged_attn.py:832-853).
 */
int mkv_attn_set_static_deal(int mode, int unit_cost, int ratio);

/*
 * Testing / debugging aid: byte offsets of the regions inside an attention workspace of the given shape and the
 * capacities the plan works with.  out[10] = {unit records, arrival counters, per-worker unit ranges, group
 * counters, lse rows, partial rows, item capacity, unit-record capacity, most worker warps a launch can have,
 * worker warps of a launch under the current tuning}.  No counterpart in the reference.
 */
int mkv_attn_workspace_layout(int device, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                              int max_blocks_per_seq_in_batch, int64_t *out);

/*
 * Copies the device-side error word of a workspace to `*flags` (synchronises the
 * stream).  Bit 0: a block-table entry was outside the pool and was skipped; bit 1: a
 * launch found no plan for its batch (or one made for more worker warps) and did
 * nothing; bit 2: the plan ran out of item records; bits 3, 4: the TMA loader gave up.
 * `workspace` NULL reads the word of the library's own scratch array on `device`, the
 * one mkv_paged_attention_decode_noalloc works in.
 */
int mkv_attn_read_error_flags(int device, void *stream, const void *workspace, int *flags /* host */);

/*
 * Decode attention for callers that cannot allocate device memory.
 * (No counterpart in the reference: its wrapper allocates two tensors per call.)
 *
 * Who needs it: a caller that is in the middle of capturing work on the stream,
 * a server that gave all device memory to the KV pool at start-up so that a late
 * cudaMalloc may fail, or a plug-in that only receives a stream and pointers and
 * has no allocator of its own.  Such a caller cannot provide the workspace that
 * mkv_attn_plan / mkv_paged_attention_decode ask for.
 *
 * This one call plans and runs the attention of one layer using a scratch array
 * built into the library: mkv_noalloc_scratch_bytes() = 16 MiB of device memory,
 * held on every GPU the library is used on from the first use until process exit.
 * It calls no cudaMalloc / cudaFree / allocating routine and never synchronises.
 * Results equal mkv_paged_attention_decode's.
 *
 *  - Limit: if the batch needs more scratch than the array holds (roughly
 *    batch * num_q_heads * head_dim beyond 256 x 32 x 128 on a 148-SM part; the
 *    exact need is mkv_attn_workspace_bytes(...)), the call returns
 *    MKV_ERR_TOO_LARGE and launches nothing.
 *  - The first call on each device resolves the array's device address
 *    (cudaGetSymbolAddress, with that device current).  Make that first call
 *    outside any stream capture.
 *  - All calls on a device share the one array, and it keeps the previous
 *    call's contents; each call re-initialises what it needs at its start.  Two
 *    calls that overlap on the GPU (different streams without an event between
 *    them) race on it: order them.
 *  - Error bits (a block-table entry outside the pool, ...) land in the array's
 *    header; read them with mkv_attn_read_error_flags(device, stream, NULL, &flags).
 *    Every call starts with the word cleared.
 */
int mkv_paged_attention_decode_noalloc(
    int device, void *stream, const void *q, void *o, const mkv_pool *pool, const int32_t *block_table,
    int64_t table_stride, const int32_t *seq_ids, const int32_t *seq_lens, int batch, int num_q_heads,
    int cur_layer, float softmax_scale, int max_blocks_per_seq_in_batch);
size_t mkv_noalloc_scratch_bytes(void);

/* ---- KV append / scatter --------------------------------------------- */
/*
 * Decode append: token len-1 of every sequence goes to
 * pool[block_table[seq, (len-1)/bs], layer, :, (len-1)%bs, :], K and V.
 * Replaces _fwd_kvcache_mgmt_decoding_kernel{,_new_kv_combined}
 * (worker/kernels/kvcache_mgmt.py:52-81, :189-251).  Pure byte copy.
 */
int mkv_store_kv_decode(int device, void *stream, const void *k, const void *v, /* device [batch, Hkv, D] */
                        const mkv_pool *pool, const int32_t *block_table, int64_t table_stride,
                        const int32_t *seq_ids, const int32_t *seq_lens, int batch, int cur_layer);

/*
 * Prefill scatter: token t of prompt i (rows start_locs[i]+t of k/v) goes to
 * pool[block_table[seq_ids[i], t/bs], layer, :, t%bs, :].  Replaces
 * _fwd_kvcache_mgmt_prefill_kernel{,_new_kv_combined}
 * (worker/kernels/kvcache_mgmt.py:12-50, :84-187).
 */
int mkv_store_kv_prefill(int device, void *stream, const void *k, const void *v, /* device [tokens, Hkv, D] */
                         const mkv_pool *pool, const int32_t *block_table, int64_t table_stride,
                         const int32_t *seq_ids, const int32_t *start_locs, const int32_t *seq_lens,
                         int num_seqs, int max_seq_len, int cur_layer);

/* ---- block table ------------------------------------------------------ */
/*
 * `num_rows` (everywhere below) = entries of num_allocated = rows of block_table (the reference's
 * max_seqs_in_block_table).  A sequence id outside [0, num_rows) touches nothing: the reference's torch indexing
 * would raise for it; here it is skipped, and reported by the calls that have a status to report into
 * (mkv_block_need counts it with the shrinking sequences, mkv_block_allocate refuses the whole request).
 */
/*
 * need[i] = ceil(target_lens[i]/block_size) - num_allocated[seq_ids[i]];
 * totals[0] = sum(need), totals[1] = number of negative entries (the reference
 * asserts there are none, worker/block_manager.py:94-99).
 */
int mkv_block_need(int device, void *stream, const int32_t *num_allocated, int num_rows, const int32_t *seq_ids,
                   const int32_t *target_lens, int batch, int block_size,
                   int32_t *need /* device [batch] */, int64_t *totals /* device [2] */);

/*
 * BlockManager.allocate_blocks_for_seqs (worker/block_manager.py:87-112) in one launch and without
 * the reference's host round trips (:95, :100): need as in mkv_block_need, the first sum(need) free
 * ids in ascending order as in mkv_bitmap_select (= torch.nonzero(is_block_free)[:n], :75), rows and
 * counts as in mkv_block_table_set.  All or nothing: when the request cannot be served the tables
 * stay as they are.  `status` (device, int64[4], zeroed by the caller once, then accumulated):
 *   [0] blocks allocated so far, [1] sequences that owned more blocks than their target (the
 *   reference's assertion, :95-98), [2] blocks that were missing (its RuntimeError, :69-70),
 *   [3] sequences whose table row would overflow (or a request larger than ids_capacity).
 * `need` [batch] and `ids` [ids_capacity] are caller-provided scratch; after the call they hold the
 * per-sequence need and the new ids in batch order.  Contains no synchronisation and no
 * allocation, so a whole decode step can be enqueued (or captured in a CUDA graph) ahead of time;
 * the host reads `status` whenever it next needs the free-block count.
 */
int mkv_block_allocate(int device, void *stream, int32_t *num_allocated, int num_rows, int32_t *block_table,
                       int64_t table_stride, const int32_t *seq_ids, const int32_t *target_lens, int batch, int block_size,
                       uint8_t *bitmap /* is_block_free */, int64_t num_blocks, int32_t *need, int64_t *ids,
                       int64_t ids_capacity, int64_t *status);

/*
 * Ascending ids i in [lo, hi) with bitmap[i] == want, at most max_out of them,
 * written to out_ids; *out_count = min(matches, max_out) and *out_total = all
 * matches in the range.  If flip != 0 the selected entries are set to !want.
 * With lo=0, hi=num_blocks, want=1, flip=1 this is the first-fit allocation of
 * worker/block_manager.py:75-77 (torch.nonzero(...)[:n]) without a host sync.
 * One thread block; needs no scratch.
 */
int mkv_bitmap_select(int device, void *stream, uint8_t *bitmap, int64_t lo, int64_t hi, int want,
                      int64_t max_out, int flip, int64_t *out_ids /* device [max_out] */,
                      int64_t *out_count /* device */, int64_t *out_total /* device */);

/* bitmap[ids[i]] = value for i < n. */
int mkv_bitmap_scatter(int device, void *stream, uint8_t *bitmap, int64_t bitmap_len,
                       const int64_t *ids, int64_t n, int value);

/*
 * Appends candidate ids to the rows of the batch and bumps the counts:
 * replaces set_block_table_and_num_seq_alloc_blocks
 * (worker/kernels/block_mgmt.py:5-46).  Sequence i takes
 * candidates[cumsum(need)[i]-need[i] : cumsum(need)[i]] (batch order).
 */
int mkv_block_table_set(int device, void *stream, int32_t *num_allocated, int num_rows, int32_t *block_table,
                        int64_t table_stride, const int64_t *candidates, const int32_t *seq_ids,
                        const int32_t *need, int batch);

/*
 * Marks the blocks of the given sequences free and zeroes their counts; rows
 * keep their entries.  Replaces unset_block_table_and_num_seq_alloc_blocks
 * (worker/kernels/block_mgmt.py:49-80).  If gathered != NULL the ids are also
 * written there in batch order (int32), which replaces
 * gather_allocated_blocks_and_unset (:83-125); gathered_capacity guards it.
 * total_out (device, may be NULL) receives the number of blocks freed, or, with
 * accumulate != 0, is increased by it (a running count the host reads later).
 */
int mkv_block_table_unset(int device, void *stream, int32_t *num_allocated, int num_rows, const int32_t *block_table,
                          int64_t table_stride, const int32_t *seq_ids, int batch, uint8_t *is_block_free,
                          int64_t num_blocks, int32_t *gathered, int64_t gathered_capacity,
                          int64_t *total_out, int accumulate);

/* sum over the batch of num_allocated[seq_ids[i]] -> *total_out (device). */
int mkv_block_table_count(int device, void *stream, const int32_t *num_allocated, int num_rows,
                          const int32_t *seq_ids, int batch, int64_t *total_out);

/* ---- elastic resize --------------------------------------------------- */
/*
 * Where an elastic chunk sits in a freed weight slab and how many blocks it
 * holds: the sizing rule of MemoryManager::acquire_new_kvcache
 * (csrc/src/memory_manager.cpp:84-97,129-147; fp16 is fixed there, elem_bytes
 * generalises it).  Host arithmetic only.  MKV_ERR_NOSPACE when no block fits.
 */
int mkv_chunk_layout(uint64_t org_start, uint64_t org_size, uint64_t quant_size, int num_layers,
                     int num_kv_heads, int block_size, int head_dim, int elem_bytes,
                     uint64_t *k_addr, uint64_t *v_addr, int64_t *num_blocks);

/*
 * Whole-block copies inside the pool: block src_ids[i] -> dst_ids[i], K and V,
 * all layers (one block is contiguous).  Used by compaction; the reference has
 * no counterpart (its release needs an already-empty tail,
 * server/memory_utils.py:529-544).  src and dst sets must be disjoint.
 */
int mkv_copy_blocks(int device, void *stream, const mkv_pool *pool, const int64_t *src_ids /* device */,
                    const int64_t *dst_ids /* device */, int64_t n);

/*
 * Rewrites live block-table entries: for every row r < num_rows and column
 * j < num_allocated[r], an entry equal to src_ids[i] becomes dst_ids[i].
 * src_ids must be ascending.  Columns >= num_allocated[r] are left alone.
 */
int mkv_remap_block_table(int device, void *stream, int32_t *block_table, int64_t table_stride,
                          int64_t num_rows, const int32_t *num_allocated, const int64_t *src_ids,
                          const int64_t *dst_ids, int64_t n);

/*
 * Compaction without a host round trip (three launches: plan, copy, remap).
 * mkv_compact_plan: every live block with id >= target, ascending, is paired with the first free ids below target,
 * ascending (src_ids / dst_ids, device arrays of `capacity` entries; capacity >= num_blocks - target always
 * suffices).  The bitmap is updated - destinations used, sources free - only when every source found a destination.
 * result (device, 4 x int64): [0] pairs to move, 0 when refused; [1] 1 when refused (too few free ids below target or
 * more sources than capacity), nothing changed; [2] live ids found at or above target; [3] free ids found below it
 * (the search stops once it has enough).  The reference has no counterpart: its release rule needs a tail that is
 * already empty (server/memory_utils.py:529-544).
 * mkv_copy_blocks_counted / mkv_remap_block_table_counted: as the calls above, with the pair count read on the
 * device from *n_dev (result[0] of the plan), at most `capacity`; the launch is sized for `capacity`.
 */
int mkv_compact_plan(int device, void *stream, uint8_t *bitmap, int64_t num_blocks, int64_t target,
                     int64_t *src_ids /* device */, int64_t *dst_ids /* device */, int64_t capacity,
                     int64_t *result /* device [4] */);
int mkv_copy_blocks_counted(int device, void *stream, const mkv_pool *pool, const int64_t *src_ids /* device */,
                            const int64_t *dst_ids /* device */, int64_t capacity, const int64_t *n_dev /* device */);
int mkv_remap_block_table_counted(int device, void *stream, int32_t *block_table, int64_t table_stride,
                                  int64_t num_rows, const int32_t *num_allocated, const int64_t *src_ids,
                                  const int64_t *dst_ids, int64_t capacity, const int64_t *n_dev /* device */);

/* ---- swap -------------------------------------------------------------- */
/*
 * Block copies between the device pool and the host swap space
 * [num_cpu_blocks, L, Hkv, bs, D].  Replaces swap_blocks and
 * swap_blocks_new_kv_combined (csrc/src/block_swapping.cpp:22-85, :88-202):
 * runs in which both id lists advance by one, and stay inside one pool
 * segment, become one cudaMemcpyAsync for K and one for V on `stream`.
 * Swap-in: host block src -> device block dst.  Swap-out: device src -> host dst.
 * (The reference's elastic variant derives the device address of a swap-in
 * from the source id, :156-161; here it always comes from the device-side id.)
 * ids are HOST arrays.  *num_copies (may be NULL) receives the copies issued.
 */
int mkv_swap_blocks(int device, void *stream, const mkv_pool *pool, void *k_swap /* host */,
                    void *v_swap /* host */, int64_t num_swap_blocks, const int64_t *src_ids /* host */,
                    const int64_t *dst_ids /* host */, int64_t n, int is_swap_in, int64_t *num_copies);

/*
 * The same block copies as mkv_swap_blocks done by ONE kernel that reads / writes
 * the swap space directly, for a swap space in pinned (device-addressable) host
 * memory.  Ids are DEVICE arrays, so the ids that BlockManager produces on the
 * GPU (worker/model.py:476-477) need no .tolist() round trip, and fragmented id
 * lists cost one launch instead of two copies per run.  Ids out of range are
 * skipped.  MKV_ERR_ALIGN if the swap space is not host memory the device can
 * address (use mkv_swap_blocks for pageable memory, as worker/model.py:196-204
 * allocates it).
 */
int mkv_swap_blocks_pinned(int device, void *stream, const mkv_pool *pool, void *k_swap /* pinned host */,
                           void *v_swap /* pinned host */, int64_t num_swap_blocks,
                           const int64_t *src_ids /* device */, const int64_t *dst_ids /* device */, int64_t n,
                           int is_swap_in);

/*
 * Copies `bytes` of a layer image from host memory (pinned for full PCIe speed) to the start of
 * the layer's slab on the GPU and returns when the copy is complete: the data movement of
 * MemoryManager::replace_layer_org2quant / replace_layer_quant2org
 * (csrc/src/memory_manager.cpp:179-231, :274-320).  MKV_ERR_NOSPACE if the image is larger than
 * the slab (the reference's "Layer requires ... bytes" error, :195-200), nothing copied then.
 * Runs on a copy stream of its own, like the reference; it is not ordered against the caller's
 * compute streams.
 */
int mkv_slab_upload(int device, void *dst_device, size_t dst_capacity, const void *src_host, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* MORPHKV_H */
