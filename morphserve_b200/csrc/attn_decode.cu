// Paged-attention decode for sm_100a.
//
// HBM-bound: per layer every K and V tile ([16 tokens x 128] fp16 = 4 KiB,
// contiguous in the pool) is read exactly once per KV head; the G = Hq/Hkv query
// heads that share it are packed as the M rows of a 16 x 16 x 16 tensor-core tile.
//
// Structure
//   plan kernel (once per decode step): cuts every sequence into chunks of
//     `chunk` blocks so that there are a few work items per resident warp, and
//     sorts the (sequence, chunk) items longest first.
//     When no sequence is longer than the mean load of a worker warp allows,
//     nothing is cut and the warps draw whole (sequence, kv head) units from a
//     global counter (dynamic, longest first).  Otherwise the launch's tiles
//     are dealt out STATICALLY: every worker warp gets an equal contiguous
//     range of the tile stream, sequences are cut only where a range ends.
//   decode kernel (once per layer): one persistent thread block per SM; every
//     WARP is an independent worker that streams its units' K/V tiles through a
//     private ring in shared memory - filled by 16-byte cp.async with an XOR
//     swizzle (default) or by TMA (cp.async.bulk.tensor, 128-byte swizzle, one
//     mbarrier per stage; four 2 KiB boxes per tile issued by one lane; pools
//     of up to 8 segments) - reads it with ldmatrix, and keeps an fp32 online
//     softmax in base 2.  The next unit is claimed in three
//     non-blocking steps a few tiles before the current one ends and its first
//     tiles are fetched into the stages the current unit frees, so the ring
//     stays full across unit boundaries.  A sequence cut into several chunks
//     goes through fp32 partials in the workspace; the warp that finishes a
//     (sequence, kv head) last merges them (no second launch, no waiting); with
//     many pieces the merge has two levels (groups of pieces first).
//     Optionally the unit that owns the newest token's block also appends that
//     token's K/V row (fused store_kvcache).
//   plain kernel: any dtype / head_dim / block size, one warp per (seq, q head).
//
// No kernel here waits on another thread block; the only wait is a warp's wait for its
// own bulk copy (mbarrier), which gives up after about a second and reports it.
#include <algorithm>
#include <atomic>
#include <type_traits>
#include <mutex>

#include <cuda.h>  // CUtensorMap and its enums (types only: the encoder is fetched from the driver at run time)
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "rope.cuh"

namespace mkv {

constexpr int kD = 128;                 // head_dim of the fast path
constexpr int kBS = 16;                 // block_size of the fast path
constexpr int kTileBytes = kBS * kD * 2;  // 4 KiB
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kNumCand = 40;
constexpr int kMinChunk = 4;            // blocks
constexpr int kSortBins = 1024;
constexpr unsigned kMagic = 0x4d4b5631u;  // "MKV1"
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegBig = -1e20f;       // the reference's mask / initial max
constexpr int kClaimAhead = 6;          // tiles before the end of a unit at which the next one is claimed

struct alignas(256) WsHeader {
    unsigned magic;
    int batch;
    int n_items;        // (sequence, chunk) items; work units = n_items * Hkv
    int chunk_blocks;
    unsigned work_counter;
    unsigned done_counter;
    int error_flags;
    int n_partial_rows;
    int cap_items;
    int mode;           // 0: units = items x kv heads, drawn from work_counter; 1: static ranges per worker (wstart)
    int n_workers;      // static deal: worker warps that own a range (the launch must bring at least as many);
                        // dynamic deal: worker warps of the launch the plan was made for (must match exactly)
    int n_units;        // unit records (static deal) or items x kv heads (dynamic deal)
    unsigned counter_init;  // dynamic deal: worker w starts on unit w, the counter hands out the units after those
};

struct WsLayout {
    size_t items, items_tmp, arrive, wstart, wrec, garrive, lse, part_o, total;
    int cap_items;
    int cap_units;   // records the items region holds (static mode needs batch * Hkv + workers)
    int max_workers;
};
constexpr int kMaxWarpsPerSm = 8;   // largest WARPS any variant of the decode kernel runs with

static inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Tuning knobs.  Process-wide, read with relaxed atomics on every call and initialised once from the environment:
// mkv_attn_configure may run on one host thread while another launches; a launch then sees either the old or the
// new value of each knob, never a torn one.  What a PLAN decided travels in the workspace header, so a launch
// always follows the plan it was given.
struct Tuning {
    std::atomic<int> warps{8}, stages{3};
    std::atomic<int> loader{0};        // 0 cp.async, 1 TMA, 2 no fast path at all (testing)
    std::atomic<int> static_mode{1};   // 0 never deal statically, 1 when a sequence must be cut, 2 whenever possible
    std::atomic<int> unit_cost{3};     // static deal: tiles that starting a unit is worth
    std::atomic<int> static_ratio{1};  // mode 1: static when the longest sequence exceeds this many chunks
    std::atomic<int> hints{1};         // L2 eviction hints of the decode kernel (AttnParams::hints)
    std::atomic<double> item_factor{4.0};    // work units per worker warp that bound the dynamic item list
    std::atomic<double> split_balance{1.5};  // see plan_balance()
    std::once_flag once;
};
static Tuning g_tuning;
constexpr int kDefaultLoader = 0;  // 0 = cp.async (measured 1-2 % faster), 1 = TMA

static Tuning &tuning() {
    std::call_once(g_tuning.once, [] {
        Tuning &t = g_tuning;
        if (const char *e = getenv("MKV_ATTN_ITEM_FACTOR")) {
            const double v = atof(e);
            if (v > 0.0) t.item_factor = v;
        }
        if (const char *e = getenv("MKV_ATTN_SPLIT_BALANCE")) {  // 0 = cut as fine as the item cap allows
            const double v = atof(e);
            t.split_balance = v < 0.0 ? 0.0 : v;
        }
        if (const char *e = getenv("MKV_ATTN_VARIANT")) {  // "<warps>x<stages>"
            int w = 0, st = 0;
            if (sscanf(e, "%dx%d", &w, &st) == 2 && w > 0 && st > 1) {
                t.warps = w;
                t.stages = st;
            }
        }
        t.loader = kDefaultLoader;
        if (const char *e = getenv("MKV_ATTN_LOADER")) t.loader = strcmp(e, "cpasync") == 0 ? 0 : 1;
        if (const char *e = getenv("MKV_ATTN_STATIC")) t.static_mode = atoi(e);
        if (const char *e = getenv("MKV_ATTN_HINTS")) t.hints = atoi(e) & 3;
        if (const char *e = getenv("MKV_ATTN_UNIT_COST")) t.unit_cost = std::max(0, std::min(64, atoi(e)));
        if (const char *e = getenv("MKV_ATTN_STATIC_RATIO")) t.static_ratio = std::max(1, std::min(1 << 20, atoi(e)));
    });
    return g_tuning;
}
static double item_factor() { return tuning().item_factor.load(std::memory_order_relaxed); }

// A sequence is only cut when it is longer than split_balance x the mean number of blocks per worker warp:
// a cut costs fp32 partial rows and a merge, and pays only when one unit would otherwise outlast the rest.
static float plan_balance(int sm_count, int num_kv_heads) {
    return (float)(tuning().split_balance.load(std::memory_order_relaxed) * (double)num_kv_heads /
                   ((double)sm_count * 8.0));
}

// Warps per thread block of the decode kernel the current tuning selects (one of the compiled variants).
static int decode_warps() {
    const int w = tuning().warps.load(std::memory_order_relaxed), st = tuning().stages.load(std::memory_order_relaxed);
    if (w == 6 && st == 4) return 6;
    return 8;
}

static WsLayout make_layout(int sm_count, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                            int max_blocks) {
    WsLayout L;
    const int64_t workers = (int64_t)sm_count * 8;
    int64_t target = (int64_t)ceil(item_factor() * (double)workers / (double)num_kv_heads);
    int64_t cap = (int64_t)batch + target;
    int64_t most = (int64_t)batch * ceil_div64(max_blocks > 0 ? max_blocks : 1, kMinChunk);
    if (cap > most) cap = most;
    if (cap < batch) cap = batch;
    if (cap < 1) cap = 1;
    L.cap_items = (int)cap;
    L.max_workers = sm_count * kMaxWarpsPerSm;
    int64_t units = (int64_t)batch * num_kv_heads + L.max_workers;
    if (units < cap) units = cap;
    L.cap_units = (int)units;
    size_t off = sizeof(WsHeader);
    L.items = off;       off = align256(off + (size_t)units * 2 * sizeof(int4));  // 2 x int4 per item / unit
    L.items_tmp = off;   off = align256(off + (size_t)cap * 2 * sizeof(int4));
    L.arrive = off;      off = align256(off + (size_t)batch * num_kv_heads * sizeof(int));
    L.wstart = off;      off = align256(off + (size_t)(L.max_workers + 1) * sizeof(int));
    L.wrec = off;        off = align256(off + (size_t)L.max_workers * 2 * sizeof(int4));  // first record of each worker
    L.garrive = off;     off = align256(off + (size_t)2 * L.max_workers * sizeof(int));
    L.lse = off;         off = align256(off + (size_t)cap * num_q_heads * sizeof(float));
    L.part_o = off;      off = align256(off + (size_t)cap * num_q_heads * head_dim * sizeof(float));
    L.total = off;
    return L;
}

__host__ __device__ __forceinline__ int chunk_candidate(int k) {
    return (k & 1) ? (6 << (k >> 1)) : (4 << (k >> 1));  // 4,6,8,12,16,24,...
}

// ------------------------------------------------------------------ plan
__device__ __forceinline__ int plan_scan(int v, int &total, int *warp_sums) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    __syncthreads();
    if (lane == 31) warp_sums[wid] = incl;
    __syncthreads();
    if (wid == 0) {
        int w = warp_sums[lane];
        int wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += n;
        }
        warp_sums[lane] = wi - w;
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    total = warp_sums[32];
    return warp_sums[wid] + incl - v;
}

struct PlanArgs {
    WsHeader *hdr;
    int4 *items;       // [cap_units] x 2
    int4 *items_tmp;   // [cap_items] x 2; static mode: int prefix[batch + 1]
    int *arrive;       // [batch * Hkv]
    int *wstart;       // [max_workers + 1]
    int4 *wrec;        // [max_workers] x 2: copy of every worker's first record (static deal)
    int *garrive;      // [2 * max_workers]
    const int32_t *seq_lens;
    const int32_t *seq_ids;
    int batch, num_kv_heads, group, block_size;
    int cap_items, cap_units, cap_rows;  // cap_rows: (row, query head) slots of the partial buffers
    int workers;       // worker warps of the decode launch this plan is for
    int max_workers;
    int static_mode;   // 0 never, 1 when the longest sequence dwarfs the chunk, 2 whenever the buffers allow it
    int static_ratio;  // mode 1: "dwarfs" = longer than static_ratio chunks
    int unit_cost;     // static deal: what starting a unit costs a worker, in tiles
    float balance;
};

// Worker that owns tile t when W workers own the ranges [floor(w T / W), floor((w + 1) T / W)).
__device__ __forceinline__ int static_owner(long long t, long long T, int W) {
    return (int)(((t + 1) * (long long)W - 1) / T);
}

// Static deal (mode 1).  The launch's tiles are ordered sequence by sequence, inside a sequence kv head by kv
// head, inside a head block by block; in front of every (sequence, head) stand `unit_cost` PHANTOM tiles, which
// stand for what starting a unit costs a worker (descriptor, block ids, query fragments, the first tile's
// latency).  Worker w takes tiles [w T / W, (w + 1) T / W) of that order, phantoms included, so a worker that
// gets many short sequences gets fewer tiles.  Its range is cut into units where the (sequence, head) changes, so a
// (sequence, head) is split only where a range ends.  `prefix[b]` = tiles, phantoms included, of ONE head of all
// sequences before b.  Walks worker w's range; with `out` it writes the unit records, and always returns how many
// there are.
__device__ int static_walk(const PlanArgs &a, const int *prefix, long long T, int W, int w, int4 *out) {
    const int Hkv = a.num_kv_heads, oc = a.unit_cost;
    long long t = (long long)w * T / W;
    const long long hi = (long long)(w + 1) * T / W;
    if (t >= hi) return 0;
    // sequence holding tile t: the largest b with Hkv * prefix[b] <= t (empty sequences share their successor's start)
    int lo_b = 0, hi_b = a.batch - 1;
    while (lo_b < hi_b) {
        const int mid = (lo_b + hi_b + 1) >> 1;
        if ((long long)Hkv * prefix[mid] <= t) lo_b = mid; else hi_b = mid - 1;
    }
    int b = lo_b;
    int nb = prefix[b + 1] - prefix[b];  // phantoms included
    long long rem = t - (long long)Hkv * prefix[b];
    int h = (int)(rem / nb);
    int blk = (int)(rem - (long long)h * nb);
    int n_units = 0;
    while (t < hi) {
        const int n = (int)min((long long)(nb - blk), hi - t);
        if (blk + n > oc) {  // the piece holds real tiles: blocks [max(blk, oc) - oc, blk + n - oc)
            if (out) {
                const long long p0 = (long long)Hkv * prefix[b] + (long long)h * nb;  // first tile of this (sequence, head)
                const int f = static_owner(p0 + oc, T, W), l = static_owner(p0 + nb - 1, T, W);
                const int first = max(blk, oc) - oc;
                // (batch index, first block, blocks, piece | head << 16) (len, pieces, first owner, table row)
                out[2 * n_units] = make_int4(b, first, blk + n - oc - first, (w - f) | (h << 16));
                out[2 * n_units + 1] = make_int4(a.seq_lens[b], l - f + 1, f, a.seq_ids[b]);
            }
            ++n_units;
        }
        t += n;
        blk += n;
        if (blk == nb) {
            blk = 0;
            if (++h == Hkv) {
                h = 0;
                do { ++b; } while (b < a.batch && prefix[b + 1] == prefix[b]);
                if (b >= a.batch) break;
                nb = prefix[b + 1] - prefix[b];
            }
        }
    }
    return n_units;
}

__global__ void __launch_bounds__(1024) attn_plan_kernel(const PlanArgs a) {
    __shared__ int cnt[kNumCand];
    __shared__ int s_total_blocks, s_max_blocks;
    __shared__ int hist[kSortBins + 1];
    __shared__ int start[kSortBins + 1];
    __shared__ int warp_sums[33];
    __shared__ int s_chunk;
    const int tid = threadIdx.x;
    WsHeader *hdr = a.hdr;
    int4 *items = a.items, *items_tmp = a.items_tmp;
    const int batch = a.batch, block_size = a.block_size, cap_items = a.cap_items;

    for (int k = tid; k < kNumCand; k += blockDim.x) cnt[k] = 0;
    if (tid == 0) s_total_blocks = s_max_blocks = 0;
    for (int k = tid; k <= kSortBins; k += blockDim.x) hist[k] = 0;
    __syncthreads();
    for (int b = tid; b < batch; b += blockDim.x) {
        int len = a.seq_lens[b];
        int nblk = len > 0 ? (len + block_size - 1) / block_size : 0;
        if (nblk > 0) {
            atomicAdd(&s_total_blocks, nblk);
            atomicMax(&s_max_blocks, nblk);
            for (int k = 0; k < kNumCand; ++k) {
                int c = chunk_candidate(k);
                atomicAdd(&cnt[k], (nblk + c - 1) / c);
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int k = 0;
        while (k < kNumCand - 1 && cnt[k] > cap_items) ++k;
        // balance x total blocks = the longest chunk worth keeping whole (see plan_balance())
        const float keep_whole = a.balance * (float)s_total_blocks;
        while (k < kNumCand - 1 && (float)chunk_candidate(k + 1) <= keep_whole) ++k;
        s_chunk = chunk_candidate(k);
    }
    __syncthreads();
    const int chunk = s_chunk;
    for (int i = tid; i < batch * a.num_kv_heads; i += blockDim.x) a.arrive[i] = 0;
    for (int i = tid; i < 2 * a.max_workers; i += blockDim.x) a.garrive[i] = 0;

    // ---- static deal: taken when some sequence would have to be cut (longer than static_ratio chunks; default 1).
    // A cut costs partial rows and a merge either way; chunks of a fixed size leave the workers unevenly loaded and,
    // for one very long sequence, one warp with a long merge at the very end, while equal ranges make every worker
    // finish together, most pieces of a cut sequence meet inside one thread block (merged through shared memory) and
    // the rest is merged in two levels.
    __shared__ int s_nonempty;
    if (tid == 0) s_nonempty = 0;
    __syncthreads();
    {
        int mine = 0;
        for (int b = tid; b < batch; b += blockDim.x) mine += a.seq_lens[b] > 0;
        if (mine) atomicAdd(&s_nonempty, mine);
    }
    __syncthreads();
    // tiles of the launch, the phantom tiles in front of every non-empty (sequence, head) included
    const long long T = ((long long)s_total_blocks + (long long)s_nonempty * a.unit_cost) * a.num_kv_heads;
    int W = a.workers;
    if ((long long)W > T) W = (int)T;
    if (W > a.cap_rows / (2 * a.group)) W = a.cap_rows / (2 * a.group);
    const bool cuts = (long long)s_max_blocks > (long long)chunk * a.static_ratio;
    if (((a.static_mode == 1 && cuts) || a.static_mode == 2) && W >= 1 &&
        (long long)batch * a.num_kv_heads + W <= a.cap_units && a.num_kv_heads < 32768) {
        int *prefix = reinterpret_cast<int *>(items_tmp);  // tiles of one head before sequence b; [batch] = all
        int carry = 0;
        for (int base = 0; base < batch; base += blockDim.x) {
            const int b = base + tid;
            int nblk = 0;
            if (b < batch) {
                const int len = a.seq_lens[b];
                nblk = len > 0 ? (len + block_size - 1) / block_size + a.unit_cost : 0;
            }
            int tot;
            const int off = plan_scan(nblk, tot, warp_sums);
            if (b < batch) prefix[b] = carry + off;
            carry += tot;
        }
        if (tid == 0) prefix[batch] = carry;
        __syncthreads();
        int carry_u = 0;
        for (int base = 0; base < a.max_workers + 1; base += blockDim.x) {
            const int w = base + tid;
            const int n = (w < W) ? static_walk(a, prefix, T, W, w, nullptr) : 0;
            int tot;
            const int off = plan_scan(n, tot, warp_sums);
            if (w <= a.max_workers) a.wstart[w] = carry_u + off;  // workers >= W own an empty range
            if (w < W) {
                int4 *mine = items + 2 * (size_t)(carry_u + off);
                static_walk(a, prefix, T, W, w, mine);
                if (n > 0) {  // a copy at a place the worker can address before it has read anything else
                    a.wrec[2 * w] = mine[0];
                    a.wrec[2 * w + 1] = mine[1];
                }
            }
            carry_u += tot;
        }
        if (tid == 0) {
            hdr->magic = kMagic;
            hdr->batch = batch;
            hdr->n_items = 0;
            hdr->chunk_blocks = 0;
            hdr->work_counter = 0;
            hdr->done_counter = 0;
            hdr->error_flags = 0;
            hdr->n_partial_rows = 2 * W;
            hdr->cap_items = cap_items;
            hdr->mode = 1;
            hdr->n_workers = W;
            hdr->n_units = carry_u;
            hdr->counter_init = 0;
        }
        return;
    }

    int carry_items = 0, carry_rows = 0;
    for (int base = 0; base < batch; base += blockDim.x) {
        const int b = base + tid;
        int nblk = 0, len = 0, row = 0;
        if (b < batch) {
            len = a.seq_lens[b];
            row = a.seq_ids[b];
            nblk = len > 0 ? (len + block_size - 1) / block_size : 0;
        }
        // chunk-sized pieces; a remainder of up to a quarter chunk stays with the piece before it (a 97-block
        // context cut at 96 is one unit, not 96 + 1).  Equal pieces measured faster than an even division.
        int ns = (nblk + chunk - 1) / chunk;
        if (ns > 1 && nblk - (ns - 1) * chunk <= chunk / 4) --ns;
        const int pr = ns > 1 ? ns : 0;
        int tot_i, tot_r;
        const int off_i = plan_scan(ns, tot_i, warp_sums);
        const int off_r = plan_scan(pr, tot_r, warp_sums);
        if (b < batch) {
            for (int s = 0; s < ns; ++s) {
                int pos = carry_items + off_i + s;
                int n = (s == ns - 1) ? nblk - s * chunk : chunk;
                if (pos < cap_items) {
                    // item = (batch index, first block, blocks, chunk index | len, chunks, partial row, table row)
                    items_tmp[2 * pos] = make_int4(b, s * chunk, n, s);
                    items_tmp[2 * pos + 1] = make_int4(len, ns, carry_rows + off_r + s, row);
                    atomicAdd(&hist[min(n, kSortBins)], 1);
                }
            }
        }
        carry_items += tot_i;
        carry_rows += tot_r;
    }
    const int n_items = min(carry_items, cap_items);
    __syncthreads();
    // longest first: thread t owns bin kSortBins - t
    {
        int total;
        int bin = kSortBins - tid;
        int v = (bin >= 0) ? hist[bin] : 0;
        int off = plan_scan(v, total, warp_sums);
        if (bin >= 0) start[bin] = off;
        if (tid == 0) start[0] = 0;  // bin 0 is never used (n >= 1); 1025 bins, 1024 threads
    }
    __syncthreads();
    for (int i = tid; i < n_items; i += blockDim.x) {
        int4 it = items_tmp[2 * i];
        int pos = atomicAdd(&start[min(it.z, kSortBins)], 1);
        items[2 * pos] = it;
        items[2 * pos + 1] = items_tmp[2 * i + 1];
    }
    if (tid == 0) {
        hdr->magic = kMagic;
        hdr->batch = batch;
        hdr->n_items = n_items;
        hdr->chunk_blocks = chunk;
        // worker w of the launch starts on unit w without asking (the units are sorted longest first, so these are the
        // longest ones either way); the counter hands out what is left
        const long long units = (long long)n_items * a.num_kv_heads;
        hdr->counter_init = (unsigned)(units < a.workers ? units : a.workers);
        hdr->work_counter = hdr->counter_init;
        hdr->done_counter = 0;
        hdr->error_flags = (carry_items > cap_items) ? 4 : 0;
        hdr->n_partial_rows = carry_rows;
        hdr->cap_items = cap_items;
        hdr->mode = 0;
        hdr->n_workers = a.workers;
        hdr->n_units = (int)units;
    }
}

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
// The same copy with an L2 eviction policy (createpolicy).  K/V tiles are read once per launch; marked evict-first
// they leave the partial rows, counters, block table and q of the launch resident in L2.  Measured: 2-3 % faster on
// batches whose sequences are cut (the statically dealt ones, where merges end the launch), 1 % slower on the large
// batches - so the policy follows the deal.
__device__ __forceinline__ void cp_async16_hint(uint32_t dst, const void *src, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ uint64_t l2_policy(bool evict_first) {
    uint64_t pol;
    if (evict_first)
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
    else
        asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
// ---- TMA (cp.async.bulk.tensor) + mbarrier: the alternative tile loader (kDefaultLoader selects cp.async)
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after about a second of GPU clock and reports it, so a copy that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000000ll)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// One box of the 2-D tensor map (64 halfs x 16 rows = 2 KiB, 128-byte swizzle) into shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// Byte offset of the 16-byte piece c (0..15) of token row r inside a staged 4 KiB tile.
//   cp.async path: rows of 256 B, piece index XOR (r & 7).
//   TMA path: the tile arrives as two boxes (dims 0-63 and 64-127) of 16 rows x 128 B, each in the hardware's
//   128-byte swizzle: piece (c & 7) XOR (r & 7) inside the row.  ldmatrix is bank-conflict free in both.
template <bool TMA>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return TMA ? (uint32_t)((c >> 3) * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4))
               : (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                                  uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// ------------------------------------------------------------------ decode kernel
struct AttnParams {
    PoolView pool;
    const __half *q;
    // Result: row b, columns [out_col_off + hq*128, +128) of every matrix in out[0..n_out).  Normally one
    // local [batch, Hq*128] matrix; with head sharding the same slice is stored into every rank's full-width
    // matrix (out[] then holds peer-mapped pointers: plain stores over NVLink, nothing is loaded from a peer).
    __half *out[8];
    int n_out;
    int64_t out_row_stride;
    int64_t out_col_off;
    // "My slice has landed" signals for pushed outputs: when the launch's last store is done, `epoch` is written to
    // ready[0..n_ready) - one word per destination, in the destination GPU's memory - after a system-wide fence.
    int32_t *ready[8];
    int n_ready;
    int32_t epoch;
    const __half *k_new;  // fused append: [batch, Hkv, D] rows of the newest token, or nullptr
    const __half *v_new;
    // fused rotary embedding: cos/sin rows [batch, 64] of the newest token's position, or nullptr.  q and the
    // k_new row are then rotated on their way in (q in the A fragments, k_new before it is patched and stored).
    const __half *rope_cos;
    const __half *rope_sin;
    int rope_fused;  // rounding of the rotation: as the compiled reference kernel (1) or operation by operation (0)
    const int32_t *block_table;
    int64_t table_stride;
    const int32_t *seq_ids;
    const int32_t *seq_lens;
    int batch;
    int num_q_heads;
    int group;          // Hq / Hkv, <= 16
    int cur_layer;
    float scale_log2;   // softmax_scale * log2(e)
    WsHeader *hdr;
    const int4 *items;
    int *arrive;
    const int *wstart;  // static deal: worker w owns the unit records [wstart[w], wstart[w + 1])
    const int4 *wrec;   // static deal: copy of worker w's first record at [2w, 2w + 1]
    int *garrive;       // static deal: arrival counters of the piece groups of a two-level merge
    float *lse;
    float *part_o;
    int hints;  // K/V tiles evict-first in L2: bit 0 under the static deal, bit 1 under the dynamic deal
};

// Tensor maps of the pool segments for the TMA loader: segment s of K (and of V) as a 2-D fp16 tensor
// [rows = blocks * L * Hkv * 16, 128], box 64 x 16, 128-byte swizzle.
constexpr int kTmaMaxSegments = 8;
struct TmaMaps {
    CUtensorMap k[kTmaMaxSegments];
    CUtensorMap v[kTmaMaxSegments];
};

// Where the partial rows of one (sequence, kv head) live.  Piece s of it has the row
// `base + s * stride + (s == 0 ? first_off : 0)`; query head r of the group sits at element row
// `row * row_mul + head_off + r` of the lse / part_o buffers.
//   dynamic deal: rows are per (sequence, chunk) item and hold all query heads: stride 1, row_mul = Hq, head_off = first
//     query head of the group.
//   static deal: worker w owns rows 2w and 2w + 1 (a worker holds at most two pieces of cut sequences: one that
//     continues from the worker before it, one that continues into the next), piece s of a (sequence, head) whose
//     first piece is at worker f lies at worker f + s: base = 2f, stride 2, first_off 1; rows hold one group.
struct RowMap {
    int64_t base;
    int stride, first_off, row_mul, head_off;
    __device__ __forceinline__ int64_t elem_row(int s, int r) const {
        return (base + (int64_t)s * stride + (s == 0 ? first_off : 0)) * row_mul + head_off + r;
    }
};

// Merge of `n` partial rows (pieces s0, s0 + step, ...) of one (sequence, kv head): for each of the G query
// heads, o = sum_s 2^(lse_s - m) o_s / sum_s 2^(lse_s - m).  FINAL: the result is the attention output (fp16,
// every destination matrix).  Otherwise it replaces the partial row of piece s0 (normalised, with its own lse),
// one level of a two-level merge.  Loads are issued in batches (4 heads x 4 rows) before any of them is used: the
// usual merge - two to four rows of a group of four query heads - is one L2 round trip.
template <bool FINAL, int SB /* rows per batch of loads */>
__device__ __forceinline__ void merge_rows_batched(const AttnParams &p, int b, int hq0, int G, const RowMap &map,
                                                   int s0, int step, int n, int lane) {
    constexpr int HP = 4;  // query heads per pass
    for (int r = 0; r < G; r += HP) {
        int rr[HP];
#pragma unroll
        for (int h = 0; h < HP; ++h) rr[h] = min(r + h, G - 1);  // a short last pass repeats its last head
        float m[HP], w[HP];
        float4 acc[HP];
#pragma unroll
        for (int h = 0; h < HP; ++h) {
            m[h] = -INFINITY;
            w[h] = 0.f;
            acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int i0 = 0; i0 < n; i0 += SB) {
            float l[HP][SB];
            float4 v[HP][SB];
#pragma unroll
            for (int i = 0; i < SB; ++i) {
                const bool ok = (i0 + i) < n;
                const int sp = s0 + (ok ? i0 + i : i0) * step;
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    const int64_t e = map.elem_row(sp, rr[h]);
                    l[h][i] = __ldcg(p.lse + e);
                    v[h][i] = __ldcg(reinterpret_cast<const float4 *>(p.part_o + e * kD + lane * 4));
                    if (!ok) l[h][i] = -INFINITY;
                }
            }
#pragma unroll
            for (int h = 0; h < HP; ++h) {
                float nm = m[h];
#pragma unroll
                for (int i = 0; i < SB; ++i) nm = fmaxf(nm, l[h][i]);
                const float sc = exp2f(m[h] - nm);  // 0 on the first batch (m = -inf)
                acc[h].x *= sc; acc[h].y *= sc; acc[h].z *= sc; acc[h].w *= sc;
                w[h] *= sc;
#pragma unroll
                for (int i = 0; i < SB; ++i) {
                    const float e = exp2f(l[h][i] - nm);  // 0 for the padding entries
                    acc[h].x += e * v[h][i].x; acc[h].y += e * v[h][i].y;
                    acc[h].z += e * v[h][i].z; acc[h].w += e * v[h][i].w;
                    w[h] += e;
                }
                m[h] = nm;
            }
        }
#pragma unroll
        for (int h = 0; h < HP; ++h) {
            if (r + h >= G) break;
            const float inv = 1.f / w[h];
            if (FINAL) {
                __half2 h01 = __floats2half2_rn(acc[h].x * inv, acc[h].y * inv);
                __half2 h23 = __floats2half2_rn(acc[h].z * inv, acc[h].w * inv);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t *>(&h01);
                pk.y = *reinterpret_cast<uint32_t *>(&h23);
                const int64_t at =
                    (int64_t)b * p.out_row_stride + p.out_col_off + (int64_t)(hq0 + rr[h]) * kD + lane * 4;
                for (int o = 0; o < p.n_out; ++o) *reinterpret_cast<uint2 *>(p.out[o] + at) = pk;
            } else {
                const int64_t e = map.elem_row(s0, rr[h]);
                __stcg(reinterpret_cast<float4 *>(p.part_o + e * kD + lane * 4),
                       make_float4(acc[h].x * inv, acc[h].y * inv, acc[h].z * inv, acc[h].w * inv));
                if (lane == 0) __stcg(p.lse + e, log2f(w[h]) + m[h]);
            }
        }
    }
}

// The merge runs on ONE warp at the end of a launch, where every instruction is on the critical path: the usual case
// (a (sequence, head) that spans two thread blocks: two rows) gets a body without padding.
template <bool FINAL>
__device__ __forceinline__ void merge_rows(const AttnParams &p, int b, int hq0, int G, const RowMap &map, int s0,
                                           int step, int n, int lane) {
    if (n <= 2)
        merge_rows_batched<FINAL, 2>(p, b, hq0, G, map, s0, step, n, lane);
    else
        merge_rows_batched<FINAL, 4>(p, b, hq0, G, map, s0, step, n, lane);
}

// Pieces per group of a two-level merge: one level up to 16 pieces (four batches of row loads cost less than a second
// level's counter, fence and extra pass: measured on a sequence whose heads span 9-10 thread blocks), otherwise about
// the square root of the count.
__device__ __forceinline__ int merge_fan_in(int nsplit) {
    if (nsplit <= 16) return nsplit;
    int f = 8;
    while (f * f < nsplit) ++f;
    return f;
}

// ---- CTA-local merge (static deal, groups of up to 8 query heads) -------------------------------------------
// With the static deal consecutive workers are the warps of one thread block, so most pieces of a cut (sequence,
// head) belong to warps of the SAME block.  Those are merged through shared memory: a piece is parked as fp32 rows
// [8][128] plus 8 lse values, either in its warp's ring (the piece that starts a (sequence, head): it is the warp's
// last unit, the ring is idle by then) or in the warp's "head slot" behind the rings (the piece that continues one:
// the warp's first unit), and the last of the block's pieces to finish folds them - no global partial rows, no
// device-wide fence, no global atomic.  Only a (sequence, head) that spans several blocks goes on to the global merge,
// one row per block.
constexpr int kSlotBytes = 8 * kD * 4 + 8 * 4;  // 4128

template <int WARPS, int STAGES, bool TMA>
__device__ __forceinline__ float *parked_piece(uint8_t *smem, int x, bool starts_pair) {
    uint8_t *at = starts_pair ? smem + (size_t)x * (STAGES * kStageBytes)
                              : smem + (size_t)WARPS * STAGES * kStageBytes + (TMA ? WARPS * STAGES * 8 : 0) +
                                    (size_t)x * kSlotBytes;
    return reinterpret_cast<float *>(at);
}

struct WorkMeta {
    bool valid;
    int b, h, start, nblk, split, nsplit, prow, len;
    const int32_t *table;  // first entry of the item in the block table
    int ids;               // lane l: block id of tile l of the item
};

// HI: the GQA group has more than 8 query heads, so rows 8-15 of the tensor-core tile carry data.
// For G <= 8 (every Llama shape) their softmax, rescale and write-out work is compiled out.
template <int WARPS, int STAGES, bool HI, bool TMA>
__global__ void __launch_bounds__(WARPS * 32, 1) attn_decode_f16_kernel(const __grid_constant__ AttnParams p,
                                                                        const __grid_constant__ TmaMaps tm) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ring = smem_u32(smem) + warp * (STAGES * kStageBytes);
    // TMA path: one mbarrier per ring stage of this warp, behind the rings
    const uint32_t bars = smem_u32(smem) + WARPS * STAGES * kStageBytes + warp * (STAGES * 8);

    WsHeader *hdr = p.hdr;
    // Everything the plan left for this launch, requested in ONE round trip before any of it is looked at: the
    // header's first and third 16 bytes (magic, batch, n_items, chunk | cap_items, mode, n_workers, n_units) and,
    // for the static deal, this worker's range of unit records.
    const int wid = (int)blockIdx.x * WARPS + warp;  // consecutive workers are the warps of one block (CTA-local merge)
    // arrival counters of the CTA-local merge, one per warp (keyed by the first warp of a group of pieces)
    int *grp_cnt = reinterpret_cast<int *>(smem + (size_t)WARPS * STAGES * kStageBytes + (TMA ? WARPS * STAGES * 8 : 0) +
                                           (size_t)WARPS * kSlotBytes);
    const int4 hdr_a = __ldcg(reinterpret_cast<const int4 *>(hdr));
    const int4 hdr_c = __ldcg(reinterpret_cast<const int4 *>(&hdr->cap_items));
    const unsigned range_lo = (unsigned)__ldcg(p.wstart + wid), range_hi = (unsigned)__ldcg(p.wstart + wid + 1);
    // ... and the worker's FIRST unit record, from where it would be under either deal (both addresses lie inside the
    // workspace whatever the plan did): the static deal's copy, or unit number `wid` of the dynamic deal
    const int4 rec_s0 = __ldcg(p.wrec + 2 * wid), rec_s1 = __ldcg(p.wrec + 2 * wid + 1);
    const int first_item = wid / p.pool.num_kv_heads;
    const int4 rec_d0 = __ldcg(p.items + 2 * first_item), rec_d1 = __ldcg(p.items + 2 * first_item + 1);
    if (!HI) {
        if (threadIdx.x < WARPS) grp_cnt[threadIdx.x] = 0;
        __syncthreads();  // the only block-wide barrier of the kernel, before any work (the loads above are in flight)
    }
    if ((unsigned)hdr_a.x != kMagic || hdr_a.y != p.batch) {  // no plan for this batch: refuse, touch nothing
        if (threadIdx.x == 0) atomicOr(&hdr->error_flags, 2);
        return;
    }
    if (TMA) {
        if (smem_u32(smem) & 1023u) {  // the swizzle pattern repeats every 1 KiB: the rings must start on one
            if (threadIdx.x == 0) atomicOr(&hdr->error_flags, 16);
            return;
        }
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncwarp();
    }
    const int Hkv = p.pool.num_kv_heads;
    const int G = p.group;
    const bool static_deal = hdr_c.y == 1;
    // planned for more workers than this launch has (static), or for another number (dynamic: the first units are
    // dealt by worker number)
    if (static_deal ? (int)(gridDim.x * WARPS) < hdr_c.z : (int)(gridDim.x * WARPS) != hdr_c.z) {
        if (threadIdx.x == 0) atomicOr(&hdr->error_flags, 2);
        return;
    }
    // static deal: this worker's unit records are [my_next, my_end).  Lane l keeps record win_base + l in registers
    // (a window of 32 records, refilled when it runs out), so that claiming a unit is a shuffle, not a load.
    unsigned my_next = static_deal ? range_lo + 1u : 0u, my_end = static_deal ? range_hi : 0u;
    unsigned win_base = static_deal ? range_lo : 0u;
    int4 win_a = make_int4(0, 0, 0, 0), win_b = make_int4(0, 0, 0, 0);
    auto load_window = [&]() {
        const unsigned i = win_base + (unsigned)lane;
        if (i < my_end) {
            win_a = __ldg(p.items + 2 * (size_t)i);
            win_b = __ldg(p.items + 2 * (size_t)i + 1);
        }
    };
    if (static_deal) load_window();
    const unsigned total_units = static_deal ? my_end : (unsigned)hdr_c.w;
    const bool row0 = g < G, row1 = HI && (g + 8) < G;

    // Claiming the next unit is a chain of three dependent global accesses (counter ->
    // unit descriptor -> block ids).  It is cut into three steps that run one per tile
    // iteration, so that each step finds the previous one's result already landed.
    // The first unit needs no claim: its record came with the header (stage 2 = fetch its block ids).
    const bool first_valid = static_deal ? range_lo < range_hi : (unsigned)wid < total_units;
    int fstage = first_valid ? 2 : 3;  // 0 claim, 1 read descriptor, 2 read block ids, 3 done
    unsigned f_idx = 0;
    int4 f_it = static_deal ? rec_s0 : rec_d0, f_it1 = static_deal ? rec_s1 : rec_d1;
    auto fetch_step = [&](WorkMeta &m) {
        if (fstage == 0 && static_deal) {
            // the record comes out of the window by shuffle; only the block ids are fetched (asynchronously: they
            // are first used when this unit's tiles are requested)
            const unsigned idx = my_next++;
            m.valid = idx < my_end;
            if (m.valid) {
                if (idx >= win_base + 32u) {
                    win_base = idx;
                    load_window();
                }
                const int src = (int)(idx - win_base);
                f_it.x = __shfl_sync(0xffffffffu, win_a.x, src);
                f_it.y = __shfl_sync(0xffffffffu, win_a.y, src);
                f_it.z = __shfl_sync(0xffffffffu, win_a.z, src);
                f_it.w = __shfl_sync(0xffffffffu, win_a.w, src);
                f_it1.x = __shfl_sync(0xffffffffu, win_b.x, src);
                f_it1.y = __shfl_sync(0xffffffffu, win_b.y, src);
                f_it1.z = __shfl_sync(0xffffffffu, win_b.z, src);
                f_it1.w = __shfl_sync(0xffffffffu, win_b.w, src);
                fstage = 2;
            } else {
                fstage = 3;
            }
        }
        if (fstage == 0) {
            if (lane == 0) f_idx = atomicAdd(&hdr->work_counter, 1u);
            fstage = 1;
        } else if (fstage == 1) {
            const unsigned idx = __shfl_sync(0xffffffffu, f_idx, 0);
            m.valid = idx < total_units;
            if (!m.valid) {
                fstage = 3;
            } else {
                const unsigned bc = idx / (unsigned)Hkv;
                m.h = (int)(idx - bc * (unsigned)Hkv);
                f_it = __ldg(p.items + 2 * bc);       // (batch index, first block, blocks, chunk index)
                f_it1 = __ldg(p.items + 2 * bc + 1);  // (len, chunks, partial row, table row)
                fstage = 2;
            }
        } else if (fstage == 2) {
            m.b = f_it.x;
            m.start = f_it.y;
            m.nblk = f_it.z;
            m.split = f_it.w;
            if (static_deal) {  // (piece | head << 16); the third word of the second half is the first owner
                m.split = f_it.w & 0xffff;
                m.h = f_it.w >> 16;
            }
            m.len = f_it1.x;
            m.nsplit = f_it1.y;
            m.prow = f_it1.z;
            m.table = p.block_table + (int64_t)f_it1.w * p.table_stride + f_it.y;
            m.ids = (lane < m.nblk) ? __ldg(m.table + lane) : 0;
            fstage = 3;
        }
    };

    // lane-constant pieces of the shared-memory addressing (bytes inside a 4 KiB tile)
    // K (S = Q K^T): matrix mi = lane>>3 : token half = mi>>1, k half = mi&1
    const int k_tok = ((lane >> 4) << 3) + (lane & 7);
    const int k_half = (lane >> 3) & 1;
    // V (O += P V): matrix mi: token half = mi&1, dim chunk half = mi>>1
    const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7);
    const int v_half = lane >> 4;

    const uint64_t kv_policy = l2_policy(static_deal ? (p.hints & 1) != 0 : (p.hints & 2) != 0);
    // One tile (K and V of one block for kv head `head_off`) into a ring stage.
    auto issue_raw = [&](int64_t blk, int64_t head_off, unsigned slot) {
        const uint32_t st = ring + slot * kStageBytes;
        if (!block_in_pool(p.pool, blk)) {
            if (lane == 0) atomicOr(&hdr->error_flags, 1);
            blk = 0;
        }
        int seg;
        int64_t brow;
        locate_block(p.pool, blk, seg, brow);
        if (TMA) {
            if (lane == 0) {
                // first row of the tile in the segment's [rows, 128] view: head_off counts bytes, a row is 256
                const int row0 = (int)((brow * p.pool.block_bytes + head_off) >> 8);
                const uint32_t bar = bars + slot * 8;
                mbar_expect_tx(bar, kStageBytes);
                tma_load_2d(st, &tm.k[seg], 0, row0, bar);
                tma_load_2d(st + 2048, &tm.k[seg], 64, row0, bar);
                tma_load_2d(st + kTileBytes, &tm.v[seg], 0, row0, bar);
                tma_load_2d(st + kTileBytes + 2048, &tm.v[seg], 64, row0, bar);
            }
            return;
        }
        const char *kt = p.pool.k_base[seg] + brow * p.pool.block_bytes + head_off;
        const char *vt = p.pool.v_base[seg] + brow * p.pool.block_bytes + head_off;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int id = i * 32 + lane;           // 16-byte piece of the tile
            const int r = id >> 4, c = id & 15;     // token row, piece in the row
            const uint32_t off = r * 256 + ((c ^ (r & 7)) << 4);
            cp_async16_hint(st + off, kt + id * 16, kv_policy);
            cp_async16_hint(st + kTileBytes + off, vt + id * 16, kv_policy);
        }
    };

    // The ring is continuous across units: tile j of a unit sits in stage (ring_pos + j) % STAGES,
    // and while a unit consumes its last STAGES-1 tiles the freed stages already receive the
    // first tiles of the next unit (`pre` of them), so the ring never runs empty at a boundary.
    unsigned ring_pos = 0;
    int pre = 0;
    bool failed = false;

    WorkMeta nxt;
    nxt.valid = first_valid;
    nxt.h = wid - first_item * Hkv;  // dynamic deal: unit `wid` = (item wid / Hkv, head wid % Hkv); static: from the record
    while (fstage < 3) fetch_step(nxt);
    while (nxt.valid) {
        const WorkMeta cur = nxt;
        nxt.valid = false;  // until the next claim lands, `nxt` is this unit: nothing may be prefetched from it
        const int pre_cur = pre;
        pre = 0;
        __syncwarp();  // the previous unit's ldmatrix reads are done before its stages are refilled

        // ---- tile loader ------------------------------------------------------
        int ids_cur = cur.ids;
        int ids_nxt = (32 + lane < cur.nblk) ? __ldg(cur.table + 32 + lane) : 0;
        int win = 0;  // window of 32 tiles that ids_cur covers
        const int64_t head_off = ((int64_t)p.cur_layer * Hkv + cur.h) * kTileBytes;
        auto issue_tile = [&](int j) {
            if ((j >> 5) != win) {
                ids_cur = ids_nxt;
                ++win;
                const int nj = (win + 1) * 32 + lane;
                ids_nxt = (nj < cur.nblk) ? __ldg(cur.table + nj) : 0;
            }
            const int64_t blk = __shfl_sync(0xffffffffu, ids_cur, j & 31);
            issue_raw(blk, head_off, (ring_pos + (unsigned)j) % STAGES);
        };

#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s >= pre_cur) {  // tiles below pre_cur were issued during the previous unit's tail
                if (s < cur.nblk) issue_tile(s);
                if (!TMA) cp_async_commit();
            }
        }

        // ---- Q fragments (A operand, rows = query heads of the group) -----------
        uint32_t qf[8][4];
        {
            const __half *qb = p.q + ((int64_t)cur.b * p.num_q_heads + (int64_t)cur.h * G) * kD;
            const uint32_t *q0 = reinterpret_cast<const uint32_t *>(qb + (int64_t)g * kD) + t;
            const uint32_t *q1 = reinterpret_cast<const uint32_t *>(qb + (int64_t)(g + 8) * kD) + t;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                qf[kk][0] = row0 ? __ldg(q0 + kk * 8) : 0u;
                qf[kk][1] = row1 ? __ldg(q1 + kk * 8) : 0u;
                qf[kk][2] = row0 ? __ldg(q0 + kk * 8 + 4) : 0u;
                qf[kk][3] = row1 ? __ldg(q1 + kk * 8 + 4) : 0u;
            }
            if (p.rope_cos != nullptr) {
                // k-step kk < 4 holds dims [16kk, 16kk+16) of the low half, kk+4 their partners in the high half;
                // this thread's columns are 16kk + 2t (+1) and 16kk + 8 + 2t (+1)
                const uint32_t *cb = reinterpret_cast<const uint32_t *>(p.rope_cos + (int64_t)cur.b * (kD / 2)) + t;
                const uint32_t *sb = reinterpret_cast<const uint32_t *>(p.rope_sin + (int64_t)cur.b * (kD / 2)) + t;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint32_t c0 = __ldg(cb + kk * 8), c1 = __ldg(cb + kk * 8 + 4);
                    const uint32_t s0 = __ldg(sb + kk * 8), s1 = __ldg(sb + kk * 8 + 4);
                    const bool rf = p.rope_fused != 0;
                    rope_rotate2(qf[kk][0], qf[kk + 4][0], c0, s0, rf);
                    rope_rotate2(qf[kk][2], qf[kk + 4][2], c1, s1, rf);
                    if (HI) {
                        rope_rotate2(qf[kk][1], qf[kk + 4][1], c0, s0, rf);
                        rope_rotate2(qf[kk][3], qf[kk + 4][3], c1, s1, rf);
                    }
                }
            }
        }

        // Fused append: the unit that holds the block of token len-1 also stores that token's new
        // K/V row.  No other unit reads that (sequence, kv head) tile in this launch, so the row is
        // patched into the staged tile and written to the pool by this warp alone.
        // lanes 0-15 carry the 16 pieces of the K row, lanes 16-31 those of the V row.
        const int new_blk = (cur.len - 1) >> 4;  // logical block of the newest token
        const bool has_new = p.k_new != nullptr && new_blk >= cur.start && new_blk < cur.start + cur.nblk;
        uint4 new_row = make_uint4(0u, 0u, 0u, 0u);
        if (has_new) {
            const __half *src = (lane < 16 ? p.k_new : p.v_new) + ((int64_t)cur.b * Hkv + cur.h) * kD + (lane & 15) * 8;
            new_row = __ldg(reinterpret_cast<const uint4 *>(src));
        }
        if (p.rope_cos != nullptr) {  // warp-uniform; has_new is uniform too
            if (has_new) {
                // K row: piece c (lanes 0-7) pairs with piece c+8 (lanes 8-15); V lanes only take part in the shuffles
                uint4 other;
                other.x = __shfl_xor_sync(0xffffffffu, new_row.x, 8);
                other.y = __shfl_xor_sync(0xffffffffu, new_row.y, 8);
                other.z = __shfl_xor_sync(0xffffffffu, new_row.z, 8);
                other.w = __shfl_xor_sync(0xffffffffu, new_row.w, 8);
                if (lane < 16) {
                    const int64_t off = (int64_t)cur.b * (kD / 2) + (lane & 7) * 8;
                    const uint4 c = __ldg(reinterpret_cast<const uint4 *>(p.rope_cos + off));
                    const uint4 sn = __ldg(reinterpret_cast<const uint4 *>(p.rope_sin + off));
                    uint4 lo = lane < 8 ? new_row : other, hi = lane < 8 ? other : new_row;
                    rope_rotate8(lo, hi, c, sn, p.rope_fused != 0);
                    new_row = lane < 8 ? lo : hi;
                }
            }
        }

        // The next unit is claimed late (kClaimAhead tiles before this one ends, or now if it is
        // that short): a warp that holds an unstarted unit for long hurts the longest-first balance.
        // (With the static deal the order of units is fixed, so the next one is claimed at once: its block ids and
        // first tiles are then on their way even when this unit is a single tile.)
        const int claim_at = static_deal ? 0 : max(cur.nblk - kClaimAhead, 0);

        float oacc[16][4];
#pragma unroll
        for (int n = 0; n < 16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
        float m0 = kNegBig, m1 = kNegBig, l0 = 0.f, l1 = 0.f;

        for (int j = 0; j < cur.nblk; ++j) {
            const bool patch_tile = has_new && cur.start + j == new_blk;
            if (TMA) {
                // tile number ring_pos + j of this warp lands in stage (ring_pos + j) % STAGES on that stage's
                // ((ring_pos + j) / STAGES)-th use; ring_pos counts every tile since the kernel started
                const unsigned n = ring_pos + (unsigned)j;
                const bool landed = mbar_wait(bars + (n % STAGES) * 8, (n / STAGES) & 1u);
                if (!__all_sync(0xffffffffu, landed)) {  // warp-uniform: the lanes leave together
                    if (lane == 0) atomicOr(&hdr->error_flags, 8);
                    failed = true;
                    break;
                }
            } else {
                cp_async_wait<STAGES - 2>();
            }
            __syncwarp();
            if (j + STAGES - 1 < cur.nblk) {
                issue_tile(j + STAGES - 1);
            } else if (fstage == 3 && nxt.valid && pre < nxt.nblk) {
                // nothing left to fetch for this unit: start on the next one (pre <= j+STAGES-1-nblk < STAGES-1)
                const int64_t blk = __shfl_sync(0xffffffffu, nxt.ids, pre);
                issue_raw(blk, ((int64_t)p.cur_layer * Hkv + nxt.h) * kTileBytes,
                          (ring_pos + (unsigned)(cur.nblk + pre)) % STAGES);
                ++pre;
            }
            if (!TMA) cp_async_commit();
            if (j == claim_at) fstage = 0;
            if (j >= claim_at && fstage < 3) fetch_step(nxt);
            const uint32_t st = ring + ((ring_pos + (unsigned)j) % STAGES) * kStageBytes;
            if (patch_tile) {
                const int slot = (cur.len - 1) & 15, c = lane & 15;
                const uint32_t off = (lane < 16 ? 0 : kTileBytes) + tile_off<TMA>(slot, c);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(st + off),
                             "r"(new_row.x), "r"(new_row.y), "r"(new_row.z), "r"(new_row.w)
                             : "memory");
                // this stage is written again later by a bulk copy (async proxy): order the plain store before it
                if (TMA) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                // the same row into the pool, for the steps to come
                const int64_t blk = __ldg(cur.table + j);
                if (block_in_pool(p.pool, blk)) {
                    int seg;
                    int64_t brow;
                    locate_block(p.pool, blk, seg, brow);
                    char *dst = (lane < 16 ? p.pool.k_base[seg] : p.pool.v_base[seg]) + brow * p.pool.block_bytes +
                                head_off + slot * 256 + c * 16;
                    *reinterpret_cast<uint4 *>(dst) = new_row;
                }
                __syncwarp();
            }
            // S = Q K^T   (16 heads x 16 tokens)
            float sc[2][4];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) sc[jj][0] = sc[jj][1] = sc[jj][2] = sc[jj][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                uint32_t b0, b1, b2, b3;
                const int c = 2 * kk + k_half;
                ldmatrix_x4(b0, b1, b2, b3, st + tile_off<TMA>(k_tok, c));
                mma_16816(sc[0], qf[kk], b0, b1);
                mma_16816(sc[1], qf[kk], b2, b3);
            }
            // scale, mask the tail of the sequence
            const int valid = cur.len - (cur.start + j) * kBS;  // tokens of this tile inside the sequence
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int tok = jj * 8 + 2 * t + (e & 1);
                    const float v = sc[jj][e] * p.scale_log2;
                    sc[jj][e] = (tok < valid) ? v : kNegBig;
                }
            }
            if (valid < kBS) {  // warp-uniform: the last tile of the sequence
                // Slots behind the sequence's end may hold anything (a pool that was never zeroed, a recycled
                // block).  Their P is exactly 0, but 0 x NaN would still poison the accumulators - the reference
                // zero-fills its pools for that reason (worker/model.py:187-188) - so the staged V rows are cleared.
                for (int i = lane; i < (kBS - valid) * 16; i += 32) {
                    const uint32_t at = st + kTileBytes + tile_off<TMA>(valid + (i >> 4), i & 15);
                    asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(at), "r"(0u) : "memory");
                }
                if (TMA) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
            }
            float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
            float mx1 = HI ? fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3])) : kNegBig;
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            if (HI) {
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            }
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            // The running maxima settle after the first tiles of a sequence; when none moved in the whole
            // warp the 64 accumulator rescales are skipped (they would multiply by exactly 1).
            const bool moved = (mn0 != m0) || (HI && mn1 != m1);
            const float a0 = fast_exp2(m0 - mn0), a1 = HI ? fast_exp2(m1 - mn1) : 1.f;
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                sc[jj][0] = fast_exp2(sc[jj][0] - mn0);
                sc[jj][1] = fast_exp2(sc[jj][1] - mn0);
                ps0 += sc[jj][0] + sc[jj][1];
                if (HI) {
                    sc[jj][2] = fast_exp2(sc[jj][2] - mn1);
                    sc[jj][3] = fast_exp2(sc[jj][3] - mn1);
                    ps1 += sc[jj][2] + sc[jj][3];
                } else {
                    sc[jj][2] = sc[jj][3] = 0.f;  // rows 8-15 are padding: P = 0 keeps their accumulators at 0
                }
            }
            l0 = l0 * a0 + ps0;  // per-thread share of the row sum; reduced over the quad at the end
            if (HI) l1 = l1 * a1 + ps1;
            if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    oacc[n][0] *= a0;
                    oacc[n][1] *= a0;
                    if (HI) {
                        oacc[n][2] *= a1;
                        oacc[n][3] *= a1;
                    }
                }
            }
            // P (16 heads x 16 tokens) as the A operand of O += P V
            uint32_t pa[4];
            pa[0] = pack_half2(sc[0][0], sc[0][1]);
            pa[1] = pack_half2(sc[0][2], sc[0][3]);
            pa[2] = pack_half2(sc[1][0], sc[1][1]);
            pa[3] = pack_half2(sc[1][2], sc[1][3]);
#pragma unroll
            for (int np = 0; np < 8; ++np) {
                uint32_t b0, b1, b2, b3;
                const int c = 2 * np + v_half;
                ldmatrix_x4_trans(b0, b1, b2, b3, st + kTileBytes + tile_off<TMA>(v_tok, c));
                mma_16816(oacc[2 * np], pa, b0, b1);
                mma_16816(oacc[2 * np + 1], pa, b2, b3);
            }
        }
        if (failed) break;  // a copy did not land in time: reported in the error word, nothing more is done
        ring_pos += (unsigned)cur.nblk;
        if (!TMA) ring_pos %= STAGES;  // TMA: kept absolute, the stage's barrier phase is derived from it
        while (fstage < 3) fetch_step(nxt);  // short unit: finish the claim now

        // ---- epilogue ---------------------------------------------------------
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float inv0 = 1.f / l0, inv1 = 1.f / l1;
        const int hq0 = cur.h * G;  // first query head of the group
        if (cur.nsplit == 1) {
            const int64_t at = (int64_t)cur.b * p.out_row_stride + p.out_col_off + (int64_t)hq0 * kD;
            for (int r = 0; r < p.n_out; ++r) {
                __half *ob = p.out[r] + at;
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    if (row0)
                        *reinterpret_cast<__half2 *>(ob + (int64_t)g * kD + n * 8 + 2 * t) =
                            __floats2half2_rn(oacc[n][0] * inv0, oacc[n][1] * inv0);
                    if (row1)
                        *reinterpret_cast<__half2 *>(ob + (int64_t)(g + 8) * kD + n * 8 + 2 * t) =
                            __floats2half2_rn(oacc[n][2] * inv1, oacc[n][3] * inv1);
                }
            }
        } else {
            // Announce a piece (or a block's group of pieces) of a cut (sequence, head) whose partial row is in the
            // workspace; whoever announces last merges.  With many rows the rows form groups of F: the last row of a
            // group folds the group into its first row, and the last GROUP to finish folds those rows into the
            // output, so no warp ever reads more than F + rows/F rows in a row.
            auto announce = [&](const RowMap &map, int split, int nsplit, bool two_level) {
                const int F = two_level ? merge_fan_in(nsplit) : nsplit;
                int *cnt = p.arrive + (int64_t)cur.b * Hkv + cur.h;
                bool last = true;
                int top_n = nsplit, top_step = 1;
                if (F < nsplit) {
                    const int grp = split / F;
                    const int gsize = min(F, nsplit - grp * F);
                    // counter of the group: one per partial row, indexed by the row of the group's first piece
                    int *gc = p.garrive + (map.base + (int64_t)(grp * F) * map.stride + (grp == 0 ? map.first_off : 0));
                    int old = 0;
                    if (lane == 0) old = atomicAdd(gc, 1);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    last = old == gsize - 1;
                    if (last) {
                        __threadfence();
                        if (lane == 0) *gc = 0;
                        if (gsize > 1) {
                            merge_rows<false>(p, cur.b, hq0, G, map, grp * F, 1, gsize, lane);
                            __threadfence();
                            __syncwarp();
                        }
                    }
                    top_n = (nsplit + F - 1) / F;
                    top_step = F;
                }
                if (last) {
                    int old = 0;
                    if (lane == 0) old = atomicAdd(cnt, 1);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old == top_n - 1) {  // every row of this (sequence, kv head) is in the workspace
                        __threadfence();
                        if (lane == 0) *cnt = 0;
                        merge_rows<true>(p, cur.b, hq0, G, map, 0, top_step, top_n, lane);
                    }
                }
            };

            if (static_deal && !HI) {
                // ---- CTA-local merge through shared memory (see parked_piece) ----
                const int f = cur.prow, l = f + cur.nsplit - 1;      // owners (worker numbers) of the first / last piece
                const int cta0 = (int)blockIdx.x * WARPS;
                const int wlo = max(f, cta0) - cta0, whi = min(l, cta0 + WARPS - 1) - cta0;  // this block's pieces
                const int gsz = whi - wlo + 1;
                __syncwarp();  // every lane is done reading the last tile: the ring may be written
                float *mine = parked_piece<WARPS, STAGES, TMA>(smem, warp, cur.split == 0);
#pragma unroll
                for (int n = 0; n < 16; ++n)
                    if (row0)
                        *reinterpret_cast<float2 *>(mine + g * kD + n * 8 + 2 * t) =
                            make_float2(oacc[n][0] * inv0, oacc[n][1] * inv0);
                if (t == 0 && row0) mine[8 * kD + g] = log2f(l0) + m0;
                __syncwarp();
                bool group_last = true;
                if (gsz > 1) {
                    int old = 0;
                    if (lane == 0) {
                        __threadfence_block();
                        old = atomicAdd(&grp_cnt[wlo], 1);
                    }
                    old = __shfl_sync(0xffffffffu, old, 0);
                    group_last = old == gsz - 1;
                }
                if (group_last) {
                    __threadfence_block();
                    const int cta_f = f / WARPS, ng = l / WARPS - cta_f + 1;  // blocks this (sequence, head) spans
                    const int gi = (int)blockIdx.x - cta_f;
                    // rows of the global merge: block c owns rows 2c (a (sequence, head) entering it) and 2c + 1 (one
                    // leaving it), so group gi of a (sequence, head) starting in block cta_f has row 2 (cta_f + gi) + (gi == 0)
                    const RowMap map{2 * (int64_t)cta_f, 2, 1, G, 0};
                    // Every piece's row is requested before any is used.  NP bounds the pieces (2, 4 or all the block's
                    // warps): this runs on one warp at the end of the launch, so padding is time on the critical path.
                    auto fold = [&](auto np_tag) {
                        constexpr int NP = decltype(np_tag)::value;
                        const float *pp[NP];
#pragma unroll
                        for (int k = 0; k < NP; ++k) {
                            const int xc = min(wlo + k, whi);  // entries behind whi re-read a real piece, weight 0
                            pp[k] = parked_piece<WARPS, STAGES, TMA>(smem, xc, cta0 + xc == f);
                        }
                        for (int r = 0; r < G; ++r) {
                            float ls[NP];
                            float4 vs[NP];
#pragma unroll
                            for (int k = 0; k < NP; ++k) {
                                ls[k] = pp[k][8 * kD + r];
                                vs[k] = *reinterpret_cast<const float4 *>(pp[k] + r * kD + lane * 4);
                            }
                            float m = -INFINITY;
#pragma unroll
                            for (int k = 0; k < NP; ++k) {
                                if (wlo + k > whi) ls[k] = -INFINITY;  // not a piece of this (sequence, head)
                                m = fmaxf(m, ls[k]);
                            }
                            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                            float wsum = 0.f;
#pragma unroll
                            for (int k = 0; k < NP; ++k) {
                                const float e = exp2f(ls[k] - m);  // 0 for the entries that are not pieces
                                acc.x += e * vs[k].x; acc.y += e * vs[k].y; acc.z += e * vs[k].z; acc.w += e * vs[k].w;
                                wsum += e;
                            }
                            const float inv = 1.f / wsum;
                            if (ng == 1) {  // the whole (sequence, head) lies in this block: this is the output
                                __half2 h01 = __floats2half2_rn(acc.x * inv, acc.y * inv);
                                __half2 h23 = __floats2half2_rn(acc.z * inv, acc.w * inv);
                                uint2 pk;
                                pk.x = *reinterpret_cast<uint32_t *>(&h01);
                                pk.y = *reinterpret_cast<uint32_t *>(&h23);
                                const int64_t at = (int64_t)cur.b * p.out_row_stride + p.out_col_off +
                                                   (int64_t)(hq0 + r) * kD + lane * 4;
                                for (int o = 0; o < p.n_out; ++o) *reinterpret_cast<uint2 *>(p.out[o] + at) = pk;
                            } else {
                                const int64_t e = map.elem_row(gi, r);
                                __stcg(reinterpret_cast<float4 *>(p.part_o + e * kD + lane * 4),
                                       make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
                                if (lane == 0) __stcg(p.lse + e, log2f(wsum) + m);
                            }
                        }
                    };
                    if (gsz <= 2)
                        fold(std::integral_constant<int, 2>{});
                    else if (gsz <= 4)
                        fold(std::integral_constant<int, 4>{});
                    else
                        fold(std::integral_constant<int, WARPS>{});
                    if (ng > 1) {
                        __threadfence();
                        __syncwarp();
                        announce(map, gi, ng, true);
                    }
                }
            } else {
                RowMap map;
                if (static_deal) {
                    map = RowMap{2 * (int64_t)cur.prow, 2, 1, G, 0};  // cur.prow = first owner of this (sequence, head)
                } else {
                    map = RowMap{(int64_t)cur.prow - cur.split, 1, 0, p.num_q_heads, hq0};
                }
                const int64_t e0 = map.elem_row(cur.split, 0);
                float *po = p.part_o + e0 * kD;
                float *pl = p.lse + e0;
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    if (row0)
                        __stcg(reinterpret_cast<float2 *>(po + (int64_t)g * kD + n * 8 + 2 * t),
                               make_float2(oacc[n][0] * inv0, oacc[n][1] * inv0));
                    if (row1)
                        __stcg(reinterpret_cast<float2 *>(po + (int64_t)(g + 8) * kD + n * 8 + 2 * t),
                               make_float2(oacc[n][2] * inv1, oacc[n][3] * inv1));
                }
                if (t == 0) {
                    if (row0) __stcg(pl + g, log2f(l0) + m0);
                    if (row1) __stcg(pl + g + 8, log2f(l1) + m1);
                }
                __threadfence();
                __syncwarp();
                announce(map, cur.split, cur.nsplit, static_deal);
            }
        }
    }
    if (!TMA) cp_async_wait<0>();
    if (p.n_ready) {  // this warp's output stores (possibly into other GPUs) are visible everywhere before it counts as done
        __threadfence_system();
        __syncwarp();
    }
    // the last worker to run dry re-arms the counters for the next launch
    if (lane == 0) {
        const unsigned workers = gridDim.x * WARPS;
        const unsigned d = atomicAdd(&hdr->done_counter, 1u);
        if (d == workers - 1) {
            hdr->work_counter = hdr->counter_init;
            hdr->done_counter = 0;
            if (p.n_ready) {  // every worker's stores are behind its fence and its count: tell the destinations
                __threadfence_system();
                for (int i = 0; i < p.n_ready; ++i) *reinterpret_cast<volatile int32_t *>(p.ready[i]) = p.epoch;
            }
        }
    }
}

// ------------------------------------------------------------------ waiting for pushed outputs
// One warp; lane r polls flags[r] until it has reached `epoch` (flags only grow; the comparison survives wrap-around)
// or `timeout_ns` have passed, in which case bit r of *status is set.  Never waits longer than the timeout: a rank
// that does not signal costs its peers that much time and an error bit, not a hang.
__global__ void wait_ready_kernel(const int32_t *flags, int n, int32_t epoch, long long timeout_ns, int32_t *status) {
    const int lane = threadIdx.x;
    if (lane >= n) return;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        int32_t v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
        if ((int32_t)(v - epoch) >= 0) return;
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if ((long long)(t - t0) > timeout_ns) {
            atomicOr(status, 1 << lane);
            return;
        }
        __nanosleep(200);
    }
}

// ------------------------------------------------------------------ plain kernel
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T from_f32_via_half(float x);  // the reference stores fp16-rounded values
template <>
__device__ __forceinline__ float from_f32_via_half<float>(float x) { return __half2float(__float2half_rn(x)); }
template <>
__device__ __forceinline__ __half from_f32_via_half<__half>(float x) { return __float2half_rn(x); }

constexpr int kMaxDimsPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void attn_decode_plain_kernel(const __grid_constant__ PoolView pool, const T *__restrict__ q, T *__restrict__ o,
                                         const int32_t *__restrict__ block_table, int64_t table_stride,
                                         const int32_t *__restrict__ seq_ids, const int32_t *__restrict__ seq_lens,
                                         int batch, int num_q_heads, int cur_layer, float scale_log2, int *error_flags) {
    const int lane = threadIdx.x & 31;
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= (int64_t)batch * num_q_heads) return;
    const int b = (int)(wid / num_q_heads);
    const int hq = (int)(wid - (int64_t)b * num_q_heads);
    const int G = num_q_heads / pool.num_kv_heads;
    const int h = hq / G;
    const int D = pool.head_dim, bs = pool.block_size;
    const int len = seq_lens[b];
    if (len <= 0) return;
    const int64_t row = seq_ids[b];
    float qr[kMaxDimsPerLane], acc[kMaxDimsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < D ? to_f32<T>(q[((int64_t)b * num_q_heads + hq) * D + d]) : 0.f;
        acc[i] = 0.f;
    }
    float m = kNegBig, l = 0.f;
    const int nblk = (len + bs - 1) / bs;
    const int64_t tile_elems = (int64_t)bs * D;
    for (int jb = 0; jb < nblk; ++jb) {
        const int64_t blk = block_table[row * table_stride + jb];
        if (!block_in_pool(pool, blk)) {
            if (lane == 0 && error_flags) atomicOr(error_flags, 1);
            continue;
        }
        int seg;
        int64_t brow;
        locate_block(pool, blk, seg, brow);
        const int64_t off = brow * pool.block_bytes +
                            ((int64_t)cur_layer * pool.num_kv_heads + h) * tile_elems * (int64_t)sizeof(T);
        const T *kt = reinterpret_cast<const T *>(pool.k_base[seg] + off);
        const T *vt = reinterpret_cast<const T *>(pool.v_base[seg] + off);
        const int ntok = min(bs, len - jb * bs);
        for (int tk = 0; tk < ntok; ++tk) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < kMaxDimsPerLane; ++i) {
                const int d = lane + 32 * i;
                if (d < D) dot += qr[i] * to_f32<T>(kt[(int64_t)tk * D + d]);
            }
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
            const float sc = dot * scale_log2;
            const float mn = fmaxf(m, sc);
            const float a = exp2f(m - mn), pr = exp2f(sc - mn);
            l = l * a + pr;
#pragma unroll
            for (int i = 0; i < kMaxDimsPerLane; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = acc[i] * a + pr * to_f32<T>(vt[(int64_t)tk * D + d]);
            }
            m = mn;
        }
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) o[((int64_t)b * num_q_heads + hq) * D + d] = from_f32_via_half<T>(acc[i] * inv);
    }
}

// ------------------------------------------------------------------ host side
template <int WARPS, int STAGES, bool HI, bool TMA>
static cudaError_t launch_decode_one(const AttnParams &p, const TmaMaps &tm, int sm_count, cudaStream_t s) {
    // rings (+ TMA barriers) + for groups of up to 8 query heads the head slots and counters of the CTA-local merge
    const int smem = WARPS * STAGES * kStageBytes + (TMA ? WARPS * STAGES * 8 : 0) +
                     (HI ? 0 : WARPS * kSlotBytes + WARPS * (int)sizeof(int));
    static std::atomic<bool> configured[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_f16_kernel<WARPS, STAGES, HI, TMA>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    attn_decode_f16_kernel<WARPS, STAGES, HI, TMA><<<sm_count, WARPS * 32, smem, s>>>(p, tm);
    return cudaGetLastError();
}

template <int WARPS, int STAGES>
static cudaError_t launch_decode(const AttnParams &p, const TmaMaps *tm, int sm_count, cudaStream_t s) {
    static const TmaMaps no_maps = {};
    if (tm)
        return p.group > 8 ? launch_decode_one<WARPS, STAGES, true, true>(p, *tm, sm_count, s)
                           : launch_decode_one<WARPS, STAGES, false, true>(p, *tm, sm_count, s);
    return p.group > 8 ? launch_decode_one<WARPS, STAGES, true, false>(p, no_maps, sm_count, s)
                       : launch_decode_one<WARPS, STAGES, false, false>(p, no_maps, sm_count, s);
}

static cudaError_t launch_decode_configured(const AttnParams &p, const TmaMaps *tm, int sms, cudaStream_t s) {
    const int w = decode_warps();
    if (w == 6) return launch_decode<6, 4>(p, tm, sms, s);
    return launch_decode<8, 3>(p, tm, sms, s);
}

// ---- tensor maps for the TMA loader ------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver function; it is looked up at run time so that the library has no link
// dependency on the driver (it loads, and every host-side check works, on a machine without a GPU).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    });
    return fn;
}

static int loader_choice() { return tuning().loader.load(std::memory_order_relaxed); }

// Fills `tm` for the pool; false if the TMA loader cannot serve it (then the cp.async loader runs).
static bool make_tma_maps(const PoolView &pv, TmaMaps *tm) {
    if (loader_choice() != 1 || pv.num_segments > kTmaMaxSegments) return false;
    EncodeTiledFn encode = tensor_map_encoder();
    if (!encode) return false;
    const cuuint64_t rows_per_block = (cuuint64_t)pv.num_layers * pv.num_kv_heads * kBS;
    for (int i = 0; i < pv.num_segments; ++i) {
        const cuuint64_t blocks = i == 0 ? (cuuint64_t)pv.num_blocks_org : (cuuint64_t)pv.chunk_blocks;
        const cuuint64_t dims[2] = {(cuuint64_t)kD, blocks * rows_per_block};
        const cuuint64_t strides[1] = {(cuuint64_t)kD * 2};      // bytes between rows
        const cuuint32_t box[2] = {64, (cuuint32_t)kBS};         // 128 B x 16 rows
        const cuuint32_t elem_strides[2] = {1, 1};
        if (dims[1] == 0 || dims[1] > 0x7fffffffull) return false;
        for (int kv = 0; kv < 2; ++kv) {
            void *base = kv ? pv.v_base[i] : pv.k_base[i];
            CUresult r = encode(kv ? &tm->v[i] : &tm->k[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides,
                                box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return false;
        }
    }
    return true;
}

static bool fast_path_ok(const PoolView &pv, int num_q_heads, const void *q, const void *o) {
    if (loader_choice() == 2) return false;  // testing knob: everything through the plain kernel
    if (pv.elem_bytes != 2 || pv.head_dim != kD || pv.block_size != kBS) return false;
    if (num_q_heads % pv.num_kv_heads != 0 || num_q_heads / pv.num_kv_heads > 16) return false;
    if ((((uintptr_t)q) | ((uintptr_t)o)) % 16 != 0) return false;
    for (int i = 0; i < pv.num_segments; ++i)
        if ((((uintptr_t)pv.k_base[i]) | ((uintptr_t)pv.v_base[i])) % 16 != 0) return false;
    return true;
}

// One plan launch for `ws` (laid out by L).  `workers` = worker warps of the decode launch that will follow.
static void launch_plan(char *ws, const WsLayout &L, const int32_t *seq_lens, const int32_t *seq_ids, int batch,
                        int num_q_heads, int num_kv_heads, int block_size, int sm_count, int workers, cudaStream_t s) {
    PlanArgs a;
    a.hdr = (WsHeader *)ws;
    a.items = (int4 *)(ws + L.items);
    a.items_tmp = (int4 *)(ws + L.items_tmp);
    a.arrive = (int *)(ws + L.arrive);
    a.wstart = (int *)(ws + L.wstart);
    a.wrec = (int4 *)(ws + L.wrec);
    a.garrive = (int *)(ws + L.garrive);
    a.seq_lens = seq_lens;
    a.seq_ids = seq_ids;
    a.batch = batch;
    a.num_kv_heads = num_kv_heads;
    a.group = num_q_heads / num_kv_heads;
    a.block_size = block_size;
    a.cap_items = L.cap_items;
    a.cap_units = L.cap_units;
    a.cap_rows = (int)std::min<int64_t>((int64_t)L.cap_items * num_q_heads, 0x7fffffff);
    a.workers = workers;
    a.max_workers = L.max_workers;
    // the static deal exists in the tensor-core kernel only (fp16, head_dim 128, block 16, groups of up to 16)
    const bool fast_shape = block_size == kBS && num_q_heads % num_kv_heads == 0 && a.group <= 16;
    a.static_mode = fast_shape ? tuning().static_mode.load(std::memory_order_relaxed) : 0;
    a.unit_cost = tuning().unit_cost.load(std::memory_order_relaxed);
    a.static_ratio = tuning().static_ratio.load(std::memory_order_relaxed);
    a.balance = plan_balance(sm_count, num_kv_heads);
    attn_plan_kernel<<<1, 1024, 0, s>>>(a);
}

static cudaError_t builtin_scratch_address(int device, void **out);  // defined with the array, at the end of the file

static void fill_workspace_params(AttnParams &p, char *ws, const WsLayout &L) {
    p.hdr = (WsHeader *)ws;
    p.items = (const int4 *)(ws + L.items);
    p.arrive = (int *)(ws + L.arrive);
    p.wstart = (const int *)(ws + L.wstart);
    p.wrec = (const int4 *)(ws + L.wrec);
    p.garrive = (int *)(ws + L.garrive);
    p.lse = (float *)(ws + L.lse);
    p.part_o = (float *)(ws + L.part_o);
}

}  // namespace mkv

using namespace mkv;

extern "C" {

size_t mkv_attn_workspace_bytes(int device, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                int max_blocks_per_seq_in_batch) {
    int sms = 0;
    if (mkv_sm_count(device, &sms) != MKV_OK) return 0;
    if (batch < 0 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 1) return 0;
    return make_layout(sms, batch, num_q_heads, num_kv_heads, head_dim, max_blocks_per_seq_in_batch).total;
}

int mkv_attn_plan(int device, void *stream, void *workspace, size_t workspace_bytes, const int32_t *seq_lens,
                  const int32_t *seq_ids, int batch, int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                  int max_blocks_per_seq_in_batch) {
    if (batch < 0 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 1 || block_size < 1) return MKV_ERR_SHAPE;
    if (num_q_heads % num_kv_heads != 0) return MKV_ERR_SHAPE;
    if (!workspace || ((uintptr_t)workspace % 256) != 0) return MKV_ERR_WORKSPACE;
    if (batch > 0 && (!seq_lens || !seq_ids)) return MKV_ERR_NULL;
    int sms = 0;
    int st = mkv_sm_count(device, &sms);
    if (st) return st;
    WsLayout L = make_layout(sms, batch, num_q_heads, num_kv_heads, head_dim, max_blocks_per_seq_in_batch);
    if (workspace_bytes < L.total) return MKV_ERR_WORKSPACE;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    launch_plan((char *)workspace, L, seq_lens, seq_ids, batch, num_q_heads, num_kv_heads, block_size, sms,
                sms * decode_warps(), (cudaStream_t)stream);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

struct OutputSpec {  // where the attention result goes (see AttnParams::out)
    void *const *ptrs;
    int n;
    int64_t row_stride, col_off;
    int32_t *const *ready;  // may be null: no signal
    int n_ready;
    int32_t epoch;
};

static int attention_decode_impl(int device, void *stream, const void *q, void *o, const OutputSpec *push,
                                 const void *k_new, const void *v_new, const mkv_pool *pool,
                                 const int32_t *block_table,
                                 int64_t table_stride, const int32_t *seq_ids, const int32_t *seq_lens, int batch,
                                 int num_q_heads, int cur_layer, float softmax_scale,
                                 int max_blocks_per_seq_in_batch, void *workspace, size_t workspace_bytes,
                                 const void *rope_cos = nullptr, const void *rope_sin = nullptr) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (batch < 0 || num_q_heads < 1 || table_stride < 1) return MKV_ERR_SHAPE;
    if (num_q_heads % pv.num_kv_heads != 0) return MKV_ERR_SHAPE;
    if (pv.head_dim > 32 * kMaxDimsPerLane) return MKV_ERR_SHAPE;
    if (cur_layer < 0 || cur_layer >= pv.num_layers) return MKV_ERR_RANGE;
    if (batch == 0) return MKV_OK;
    if (!q || !o || !block_table || !seq_ids || !seq_lens) return MKV_ERR_NULL;
    if (pv.total_blocks < 1) return MKV_ERR_SHAPE;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    cudaStream_t s = (cudaStream_t)stream;
    const float scale_log2 = softmax_scale * kLog2e;

    if ((k_new == nullptr) != (v_new == nullptr)) return MKV_ERR_NULL;
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return MKV_ERR_NULL;
    if (rope_cos && (!k_new || (((uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)rope_cos | (uintptr_t)rope_sin) % 16) != 0 ||
                     !fast_path_ok(pv, num_q_heads, q, o))) {
        // no fused rotation for this shape / alignment: rotate q and k_new in place with the stand-alone kernel
        int rc = mkv_rotary_embedding(device, stream, const_cast<void *>(q), const_cast<void *>(k_new), rope_cos,
                                      rope_sin, batch, num_q_heads, pv.num_kv_heads, pv.head_dim, pv.elem_bytes);
        if (rc) return rc;
        rope_cos = rope_sin = nullptr;
    }
    if (k_new && (((uintptr_t)k_new | (uintptr_t)v_new) % 16 != 0 || !fast_path_ok(pv, num_q_heads, q, o))) {
        // no fused path for this shape / alignment: append with the copy kernel, then attend
        int rc = mkv_store_kv_decode(device, stream, k_new, v_new, pool, block_table, table_stride, seq_ids, seq_lens,
                                     batch, cur_layer);
        if (rc) return rc;
        k_new = v_new = nullptr;
    }
    if (!fast_path_ok(pv, num_q_heads, q, o)) {
        int *flags = nullptr;
        if (workspace && workspace_bytes >= sizeof(WsHeader) && ((uintptr_t)workspace % 256) == 0)
            flags = &((WsHeader *)workspace)->error_flags;
        const int threads = 128;
        const int64_t warps = (int64_t)batch * num_q_heads;
        const unsigned grid = (unsigned)ceil_div64(warps, threads / 32);
        if (pv.elem_bytes == 2)
            attn_decode_plain_kernel<__half><<<grid, threads, 0, s>>>(pv, (const __half *)q, (__half *)o, block_table,
                                                                     table_stride, seq_ids, seq_lens, batch,
                                                                     num_q_heads, cur_layer, scale_log2, flags);
        else
            attn_decode_plain_kernel<float><<<grid, threads, 0, s>>>(pv, (const float *)q, (float *)o, block_table,
                                                                    table_stride, seq_ids, seq_lens, batch,
                                                                    num_q_heads, cur_layer, scale_log2, flags);
        MKV_LAUNCH_CHECK();
        return MKV_OK;
    }

    if (!workspace || ((uintptr_t)workspace % 256) != 0) return MKV_ERR_WORKSPACE;
    int sms = 0;
    st = mkv_sm_count(device, &sms);
    if (st) return st;
    WsLayout L = make_layout(sms, batch, num_q_heads, pv.num_kv_heads, pv.head_dim, max_blocks_per_seq_in_batch);
    if (workspace_bytes < L.total) return MKV_ERR_WORKSPACE;
    char *ws = (char *)workspace;
    AttnParams p;
    p.pool = pv;
    p.q = (const __half *)q;
    p.n_ready = 0;
    p.epoch = 0;
    if (push) {
        p.n_out = push->n;
        for (int i = 0; i < push->n; ++i) p.out[i] = (__half *)push->ptrs[i];
        p.out_row_stride = push->row_stride;
        p.out_col_off = push->col_off;
        if (push->ready) {
            p.n_ready = push->n_ready;
            for (int i = 0; i < push->n_ready; ++i) p.ready[i] = push->ready[i];
            p.epoch = push->epoch;
        }
    } else {
        p.n_out = 1;
        p.out[0] = (__half *)o;
        p.out_row_stride = (int64_t)num_q_heads * kD;
        p.out_col_off = 0;
    }
    p.k_new = (const __half *)k_new;
    p.v_new = (const __half *)v_new;
    p.rope_cos = (const __half *)rope_cos;
    p.rope_sin = (const __half *)rope_sin;
    p.rope_fused = rope_fused_rounding() ? 1 : 0;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.seq_ids = seq_ids;
    p.seq_lens = seq_lens;
    p.batch = batch;
    p.num_q_heads = num_q_heads;
    p.group = num_q_heads / pv.num_kv_heads;
    p.cur_layer = cur_layer;
    p.scale_log2 = scale_log2;
    fill_workspace_params(p, ws, L);
    p.hints = tuning().hints.load(std::memory_order_relaxed);

    TmaMaps tm;
    const bool use_tma = make_tma_maps(pv, &tm);
    cudaError_t e = launch_decode_configured(p, use_tma ? &tm : nullptr, sms, s);
    if (e != cudaSuccess) return set_cuda_error(e);
    return MKV_OK;
}

int mkv_paged_attention_decode(int device, void *stream, const void *q, void *o, const mkv_pool *pool,
                               const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids,
                               const int32_t *seq_lens, int batch, int num_q_heads, int cur_layer,
                               float softmax_scale, int max_blocks_per_seq_in_batch, void *workspace,
                               size_t workspace_bytes) {
    return attention_decode_impl(device, stream, q, o, nullptr, nullptr, nullptr, pool, block_table, table_stride, seq_ids,
                                 seq_lens, batch, num_q_heads, cur_layer, softmax_scale,
                                 max_blocks_per_seq_in_batch, workspace, workspace_bytes);
}

int mkv_paged_attention_decode_append(int device, void *stream, const void *q, void *o, const void *k_new,
                                      const void *v_new, const mkv_pool *pool, const int32_t *block_table,
                                      int64_t table_stride, const int32_t *seq_ids, const int32_t *seq_lens,
                                      int batch, int num_q_heads, int cur_layer, float softmax_scale,
                                      int max_blocks_per_seq_in_batch, void *workspace, size_t workspace_bytes) {
    if (batch > 0 && (!k_new || !v_new)) return MKV_ERR_NULL;
    return attention_decode_impl(device, stream, q, o, nullptr, k_new, v_new, pool, block_table, table_stride, seq_ids,
                                 seq_lens, batch, num_q_heads, cur_layer, softmax_scale,
                                 max_blocks_per_seq_in_batch, workspace, workspace_bytes);
}

int mkv_paged_attention_decode_rope_append(int device, void *stream, void *q, void *o, void *k_new, const void *v_new,
                                           const void *rope_cos, const void *rope_sin, const mkv_pool *pool,
                                           const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids,
                                           const int32_t *seq_lens, int batch, int num_q_heads, int cur_layer,
                                           float softmax_scale, int max_blocks_per_seq_in_batch, void *workspace,
                                           size_t workspace_bytes) {
    if (batch > 0 && (!k_new || !v_new || !rope_cos || !rope_sin)) return MKV_ERR_NULL;
    return attention_decode_impl(device, stream, q, o, nullptr, k_new, v_new, pool, block_table, table_stride, seq_ids,
                                 seq_lens, batch, num_q_heads, cur_layer, softmax_scale,
                                 max_blocks_per_seq_in_batch, workspace, workspace_bytes, rope_cos, rope_sin);
}

int mkv_paged_attention_decode_push(int device, void *stream, const void *q, void *const *out_ptrs, int n_out,
                                    int64_t out_row_stride, int64_t out_col_offset, int32_t *const *ready_ptrs,
                                    int n_ready, int32_t epoch, const void *k_new,
                                    const void *v_new, const mkv_pool *pool, const int32_t *block_table,
                                    int64_t table_stride, const int32_t *seq_ids, const int32_t *seq_lens, int batch,
                                    int num_q_heads, int cur_layer, float softmax_scale,
                                    int max_blocks_per_seq_in_batch, void *workspace, size_t workspace_bytes) {
    if (n_out < 1 || n_out > 8 || n_ready < 0 || n_ready > 8) return MKV_ERR_SHAPE;
    if (!out_ptrs || (n_ready > 0 && !ready_ptrs)) return MKV_ERR_NULL;
    for (int i = 0; i < n_ready; ++i) {
        if (!ready_ptrs[i]) return MKV_ERR_NULL;
        if (((uintptr_t)ready_ptrs[i]) % 4 != 0) return MKV_ERR_ALIGN;
    }
    if (out_row_stride < (int64_t)num_q_heads * 128 + out_col_offset || out_col_offset < 0) return MKV_ERR_SHAPE;
    if ((out_row_stride % 8) != 0 || (out_col_offset % 8) != 0) return MKV_ERR_ALIGN;
    for (int i = 0; i < n_out; ++i) {
        if (!out_ptrs[i]) return MKV_ERR_NULL;
        if (((uintptr_t)out_ptrs[i]) % 16 != 0) return MKV_ERR_ALIGN;
    }
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (!fast_path_ok(pv, num_q_heads, q, out_ptrs[0])) return MKV_ERR_SHAPE;  // fp16, head_dim 128, block 16 only
    OutputSpec spec{out_ptrs, n_out, out_row_stride, out_col_offset, n_ready > 0 ? ready_ptrs : nullptr, n_ready, epoch};
    return attention_decode_impl(device, stream, q, out_ptrs[0], &spec, k_new, v_new, pool, block_table,
                                 table_stride, seq_ids, seq_lens, batch, num_q_heads, cur_layer, softmax_scale,
                                 max_blocks_per_seq_in_batch, workspace, workspace_bytes);
}

int mkv_wait_ready(int device, void *stream, const int32_t *flags, int n, int32_t epoch, int64_t timeout_ns,
                   int32_t *status) {
    if (n < 0 || n > 32 || timeout_ns < 0) return MKV_ERR_SHAPE;
    if (n == 0) return MKV_OK;
    if (!flags || !status) return MKV_ERR_NULL;
    if (timeout_ns > 2000000000ll) timeout_ns = 2000000000ll;  // two seconds at most, whatever the caller asks for
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    wait_ready_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, epoch, (long long)timeout_ns, status);
    MKV_LAUNCH_CHECK();
    return MKV_OK;
}

int mkv_attn_configure(int warps, int stages, double item_factor_value, double split_balance_value, int loader) {
    Tuning &t = tuning();
    if (warps > 0 && stages > 1) {
        t.warps.store(warps, std::memory_order_relaxed);
        t.stages.store(stages, std::memory_order_relaxed);
    }
    if (item_factor_value > 0.0) t.item_factor.store(item_factor_value, std::memory_order_relaxed);
    if (split_balance_value >= 0.0) t.split_balance.store(split_balance_value, std::memory_order_relaxed);
    if (loader >= 0 && loader <= 2) t.loader.store(loader, std::memory_order_relaxed);
    return MKV_OK;
}

int mkv_attn_workspace_layout(int device, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                              int max_blocks_per_seq_in_batch, int64_t *out) {
    if (!out) return MKV_ERR_NULL;
    if (batch < 0 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 1) return MKV_ERR_SHAPE;
    int sms = 0;
    int st = mkv_sm_count(device, &sms);
    if (st) return st;
    const WsLayout L = make_layout(sms, batch, num_q_heads, num_kv_heads, head_dim, max_blocks_per_seq_in_batch);
    const int64_t v[10] = {(int64_t)L.items, (int64_t)L.arrive, (int64_t)L.wstart, (int64_t)L.garrive, (int64_t)L.lse,
                           (int64_t)L.part_o, L.cap_items, L.cap_units, L.max_workers, (int64_t)sms * decode_warps()};
    for (int i = 0; i < 10; ++i) out[i] = v[i];
    return MKV_OK;
}

int mkv_attn_set_static_deal(int mode, int unit_cost, int ratio) {
    if (mode > 2 || unit_cost > 64 || ratio == 0 || ratio > (1 << 20)) return MKV_ERR_RANGE;
    if (mode >= 0) tuning().static_mode.store(mode, std::memory_order_relaxed);
    if (unit_cost >= 0) tuning().unit_cost.store(unit_cost, std::memory_order_relaxed);
    if (ratio > 0) tuning().static_ratio.store(ratio, std::memory_order_relaxed);
    return MKV_OK;
}

int mkv_attn_read_error_flags(int device, void *stream, const void *workspace, int *flags) {
    if (!flags) return MKV_ERR_NULL;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    if (!workspace) {  // the library's own scratch array on `device` (mkv_paged_attention_decode_noalloc)
        void *builtin = nullptr;
        MKV_CUDA_TRY(builtin_scratch_address(device, &builtin));
        workspace = builtin;
    }
    const WsHeader *hdr = (const WsHeader *)workspace;
    MKV_CUDA_TRY(cudaMemcpyAsync(flags, &hdr->error_flags, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    MKV_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return MKV_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ entry point that allocates nothing
//
// Some hosts of this library may not allocate device memory at the moment they
// need attention: code running while a CUDA graph is being captured on the
// stream, a serving loop whose memory budget was handed out in full at start-up
// (the KV pool is sized to fill the GPU, so a late cudaMalloc can fail), or a
// plug-in that is only given a stream and raw pointers and owns no allocator.
// For them the scratch of the decode kernel (plan, split-KV partials, counters)
// lives in the fixed array below.  Every GPU on which the library is used holds
// these 16 MiB from the first use until the process exits.
namespace mkv {

constexpr size_t kBuiltinScratchBytes = (size_t)16 << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

// Device address of the array on `device`.  In host code the array's NAME is only
// a handle for the runtime, not a device address, so it is resolved once per
// device, with that device current, and the resolved pointer is what kernels get.
static cudaError_t builtin_scratch_address(int device, void **out) {
    static std::atomic<void *> ptrs[64];  // published with release / read with acquire: host threads may race here
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    void *ptr = ptrs[device].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_builtin_scratch);  // current device == `device`
        if (e != cudaSuccess) return e;
        if (ptr == nullptr) return cudaErrorInvalidSymbol;
        ptrs[device].store(ptr, std::memory_order_release);  // two threads resolving at once store the same value
    }
    *out = ptr;
    return cudaSuccess;
}

}  // namespace mkv

extern "C" {

int mkv_paged_attention_decode_noalloc(int device, void *stream, const void *q, void *o, const mkv_pool *pool,
                                       const int32_t *block_table, int64_t table_stride, const int32_t *seq_ids,
                                       const int32_t *seq_lens, int batch, int num_q_heads, int cur_layer,
                                       float softmax_scale, int max_blocks_per_seq_in_batch) {
    PoolView pv;
    int st = validate_pool(pool, &pv);
    if (st) return st;
    if (batch < 0 || num_q_heads < 1 || table_stride < 1) return MKV_ERR_SHAPE;
    if (num_q_heads % pv.num_kv_heads != 0) return MKV_ERR_SHAPE;
    if (pv.head_dim > 32 * kMaxDimsPerLane) return MKV_ERR_SHAPE;
    if (cur_layer < 0 || cur_layer >= pv.num_layers) return MKV_ERR_RANGE;
    if (batch == 0) return MKV_OK;
    if (!q || !o || !block_table || !seq_ids || !seq_lens) return MKV_ERR_NULL;
    if (pv.total_blocks < 1) return MKV_ERR_SHAPE;
    int sms = 0;
    st = mkv_sm_count(device, &sms);
    if (st) return st;
    const bool fast = fast_path_ok(pv, num_q_heads, q, o);
    WsLayout L;
    if (fast) {
        L = make_layout(sms, batch, num_q_heads, pv.num_kv_heads, pv.head_dim, max_blocks_per_seq_in_batch);
        if (L.total > kBuiltinScratchBytes) return MKV_ERR_TOO_LARGE;  // before anything is launched
    }
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return set_cuda_error(guard.err);
    void *scratch = nullptr;
    MKV_CUDA_TRY(builtin_scratch_address(device, &scratch));
    cudaStream_t s = (cudaStream_t)stream;
    const float scale_log2 = softmax_scale * kLog2e;
    char *ws = (char *)scratch;

    if (scratch == nullptr) return MKV_ERR_WORKSPACE;  // never hand a null scratch pointer to a kernel

    if (!fast) {  // the plain kernel needs no scratch beyond the error word, which starts clean for every call
        const int threads = 128;
        const unsigned grid = (unsigned)ceil_div64((int64_t)batch * num_q_heads, threads / 32);
        int *flags = &((WsHeader *)ws)->error_flags;
        MKV_CUDA_TRY(cudaMemsetAsync(flags, 0, sizeof(int), s));
        if (pv.elem_bytes == 2)
            attn_decode_plain_kernel<__half><<<grid, threads, 0, s>>>(pv, (const __half *)q, (__half *)o, block_table,
                                                                     table_stride, seq_ids, seq_lens, batch,
                                                                     num_q_heads, cur_layer, scale_log2, flags);
        else
            attn_decode_plain_kernel<float><<<grid, threads, 0, s>>>(pv, (const float *)q, (float *)o, block_table,
                                                                    table_stride, seq_ids, seq_lens, batch,
                                                                    num_q_heads, cur_layer, scale_log2, flags);
        MKV_LAUNCH_CHECK();
        return MKV_OK;
    }

    // The plan kernel rewrites everything that must start clean: header (error word included), work and done
    // counters, the arrival counters of every (sequence, kv head) and of the piece groups, the unit list.
    launch_plan(ws, L, seq_lens, seq_ids, batch, num_q_heads, pv.num_kv_heads, pv.block_size, sms, sms * 8, s);
    MKV_LAUNCH_CHECK();
    AttnParams p;
    p.pool = pv;
    p.q = (const __half *)q;
    p.n_out = 1;
    p.out[0] = (__half *)o;
    p.out_row_stride = (int64_t)num_q_heads * kD;
    p.out_col_off = 0;
    p.n_ready = 0;
    p.epoch = 0;
    p.k_new = nullptr;
    p.v_new = nullptr;
    p.rope_cos = nullptr;
    p.rope_sin = nullptr;
    p.rope_fused = 0;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.seq_ids = seq_ids;
    p.seq_lens = seq_lens;
    p.batch = batch;
    p.num_q_heads = num_q_heads;
    p.group = num_q_heads / pv.num_kv_heads;
    p.cur_layer = cur_layer;
    p.scale_log2 = scale_log2;
    fill_workspace_params(p, ws, L);
    p.hints = tuning().hints.load(std::memory_order_relaxed);
    TmaMaps tm;
    const bool use_tma = make_tma_maps(pv, &tm);
    cudaError_t e = launch_decode<8, 3>(p, use_tma ? &tm : nullptr, sms, s);
    if (e != cudaSuccess) return set_cuda_error(e);
    return MKV_OK;
}

size_t mkv_noalloc_scratch_bytes(void) { return kBuiltinScratchBytes; }

}  // extern "C"
