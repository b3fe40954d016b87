"""CPU restatement of the reference KV-cache kernels.  TEST INFRASTRUCTURE ONLY.

Each function names the reference lines it follows (paths are relative to the
reference project root).  numpy is used for the byte/integer work and for the
split-KV arithmetic; torch (CPU) only for the live restatement of the
reference's commented PyTorch loop, which is also the timed CPU baseline.

Pool layout, K and V separately (worker/model.py:180-190):
    [num_blocks, num_layers, num_kv_heads, block_size, head_dim], contiguous.
Elastic chunks (server/memory_utils.py:389-407) are further arrays of the same
trailing shape; block id ``b >= num_blocks_org`` lives in chunk
``(b - num_blocks_org) // chunk_blocks`` at row ``(b - num_blocks_org) %
chunk_blocks`` (worker/kernels/paged_attn.py:354-360).
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import numpy as np

LOG2E = 1.442695040888963  # worker/kernels/paged_attn.py:837


# --------------------------------------------------------------------------
# per-step metadata (worker/model.py:318-436)
# --------------------------------------------------------------------------
def infer_state_fields(prompt_lens: Sequence[int], decoding_seq_lens: Sequence[int], num_kv_heads: int,
                       head_dim: int) -> dict:
    """The integer fields the reference's forward() derives from its Python lists before it builds the
    LlamaInferState: prefill sequences first, decoding sequences after them (worker/model.py:318-352), token
    positions 0..len-1 for prompts and len-1 for decoding sequences (:354-372), the split size (:397-402, :426)."""
    prompt_lens = [int(x) for x in prompt_lens]
    dec = [int(x) for x in decoding_seq_lens]
    num_tokens = sum(prompt_lens) + len(dec)
    starts = np.cumsum(prompt_lens) - np.asarray(prompt_lens) if prompt_lens else np.zeros(0)
    positions = np.concatenate([np.arange(n) for n in prompt_lens] + [np.asarray(dec, dtype=np.int64) - 1]) \
        if (prompt_lens or dec) else np.zeros(0, dtype=np.int64)
    sbs, nsb = seq_block_size_heuristic(num_kv_heads, dec)
    return dict(batch_size=len(prompt_lens) + len(dec), num_tokens=num_tokens, num_prefill_seqs=len(prompt_lens),
                num_prefill_tokens=sum(prompt_lens), prefill_seq_start_locs=starts.astype(np.int32),
                prefill_seq_start_locs_with_end=np.concatenate([starts, [num_tokens]]).astype(np.int32),
                prefill_seq_lens=np.asarray(prompt_lens, dtype=np.int32), max_prefill_len=max(prompt_lens, default=0),
                num_decoding_seqs=len(dec), decoding_seq_lens=np.asarray(dec, dtype=np.int32),
                max_decoding_len=max(dec, default=0), seq_block_size=sbs, num_seq_blocks=nsb,
                seq_lengths=np.asarray(prompt_lens + dec, dtype=np.int32), position_indices=positions.astype(np.int64),
                softmax_scale=float(head_dim) ** -0.5)


# --------------------------------------------------------------------------
# rotary embedding (the step before the append: worker/layers/transformer_layer.py:93-98)
# --------------------------------------------------------------------------
def rotary_embedding(q: np.ndarray, k: np.ndarray, cos: np.ndarray, sin: np.ndarray, rounding: str = "written"):
    """worker/kernels/rotary_emb.py:7-41: halves [0, D/2) and [D/2, D) of every head rotate as
    (x0*cos - x1*sin, x0*sin + x1*cos) with the token's cos/sin row.  All operands are fp16 in the
    reference (tables: worker/model.py:240-241).
    rounding="written": every product and every sum rounds to the data type on its own (numpy's fp16
    arithmetic does exactly that) - the kernel's source run operation by operation, which is how the
    Triton interpreter runs it and where the committed fixtures come from.
    rounding="compiled": x0*cos - rn(x1*sin) and x0*sin + rn(x1*cos) with ONE rounding of the outer
    expression - what the kernel computes once Triton has compiled it for a GPU (the first product is
    contracted into the add).  float64 holds the exact product and sum of the narrower operands.
    Returns new arrays (the reference writes in place)."""
    h = q.shape[-1] // 2
    c = cos[:, None, :].astype(q.dtype)
    s = sin[:, None, :].astype(q.dtype)

    def rot(x):
        x0, x1 = x[..., :h], x[..., h:]
        if rounding == "compiled":
            w0, w1, wc, ws = (a.astype(np.float64) for a in (x0, x1, c, s))
            lo = w0 * wc - (x1 * s).astype(np.float64)
            hi = w0 * ws + (x1 * c).astype(np.float64)
            return np.concatenate([lo, hi], axis=-1).astype(x.dtype)
        assert rounding == "written"
        return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1).astype(x.dtype)

    return rot(q), rot(k)


# --------------------------------------------------------------------------
# addressing
# --------------------------------------------------------------------------
def locate_block(block_id: int, num_blocks_org: int, chunk_blocks: int) -> Tuple[int, int]:
    """(segment, row) of a block id.  Segment 0 is the original pool, segment
    j+1 is elastic chunk j.  worker/kernels/paged_attn.py:354-360."""
    block_id = int(block_id)
    if block_id < num_blocks_org:
        return 0, block_id
    j = (block_id - num_blocks_org) // chunk_blocks
    i = block_id - num_blocks_org - j * chunk_blocks
    return 1 + j, i


def seq_block_size_heuristic(num_kv_heads: int, decoding_seq_lens: Sequence[int]) -> Tuple[int, int]:
    """(seq_block_size, num_seq_blocks) as worker/model.py:397-402,426."""
    seq_block_size = 512
    total = sum(int(x) for x in decoding_seq_lens)
    max_len = max((int(x) for x in decoding_seq_lens), default=0)
    while (num_kv_heads * (total / seq_block_size) < 1024
           and seq_block_size // 2 >= 64
           and max_len / (seq_block_size // 2) <= 128):
        seq_block_size //= 2
    return seq_block_size, (max_len + seq_block_size - 1) // seq_block_size


# --------------------------------------------------------------------------
# KV append / scatter (bit copies)
# --------------------------------------------------------------------------
def store_kvcache_decode(k, v, k_pools: List[np.ndarray], v_pools: List[np.ndarray],
                         block_table: np.ndarray, seq_ids, seq_lens, cur_layer: int,
                         num_blocks_org: int, chunk_blocks: int) -> None:
    """Append token ``len-1`` of every decoding sequence, in place.
    worker/kernels/kvcache_mgmt.py:52-81 and :189-251."""
    block_size = k_pools[0].shape[3]
    for b in range(len(seq_ids)):
        pos = int(seq_lens[b]) - 1
        blk = int(block_table[int(seq_ids[b]), pos // block_size])
        slot = pos % block_size
        seg, row = locate_block(blk, num_blocks_org, chunk_blocks)
        k_pools[seg][row, cur_layer, :, slot, :] = k[b]
        v_pools[seg][row, cur_layer, :, slot, :] = v[b]


def store_kvcache_prefill(k, v, k_pools, v_pools, block_table, seq_ids, start_locs, seq_lens,
                          cur_layer: int, num_blocks_org: int, chunk_blocks: int) -> None:
    """Scatter prompt tokens into their blocks, transposing token<->head.
    worker/kernels/kvcache_mgmt.py:12-50 and :84-187."""
    block_size = k_pools[0].shape[3]
    for i in range(len(seq_ids)):
        n = int(seq_lens[i])
        s0 = int(start_locs[i])
        for t in range(n):
            blk = int(block_table[int(seq_ids[i]), t // block_size])
            seg, row = locate_block(blk, num_blocks_org, chunk_blocks)
            k_pools[seg][row, cur_layer, :, t % block_size, :] = k[s0 + t]
            v_pools[seg][row, cur_layer, :, t % block_size, :] = v[s0 + t]


def gather_sequence_kv(k_pools, v_pools, block_table, seq_id: int, seq_len: int, cur_layer: int,
                       num_blocks_org: int, chunk_blocks: int):
    """[Hkv, len, D] K and V of one sequence, in token order."""
    block_size = k_pools[0].shape[3]
    nblk = (seq_len + block_size - 1) // block_size
    ks, vs = [], []
    for j in range(nblk):
        seg, row = locate_block(block_table[seq_id, j], num_blocks_org, chunk_blocks)
        ks.append(k_pools[seg][row, cur_layer])
        vs.append(v_pools[seg][row, cur_layer])
    kk = np.concatenate(ks, axis=1)[:, :seq_len]
    vv = np.concatenate(vs, axis=1)[:, :seq_len]
    return kk, vv


# --------------------------------------------------------------------------
# decode attention
# --------------------------------------------------------------------------
def round_to_output(x: np.ndarray, out_dtype) -> np.ndarray:
    """The reference casts the merged result to fp16 before storing it, whatever
    the dtype of ``o`` (worker/kernels/paged_attn.py:695-696)."""
    return x.astype(np.float16).astype(out_dtype)


def paged_attention_splitkv(q, k_pools, v_pools, block_table, seq_ids, seq_lens, cur_layer: int,
                            softmax_scale: float, seq_block_size: int,
                            num_blocks_org: int, chunk_blocks: int, out_dtype=np.float16) -> np.ndarray:
    """fp32 restatement of the two Triton phases.

    Phase 1 (worker/kernels/paged_attn.py:59-240): per (seq, q head, chunk of
    ``seq_block_size`` tokens) an online softmax in base 2 over 16-token blocks
    with max initialised to -1e20 and masked tokens set to -1e20; stores
    acc/sum and log2(sum)+max.  Phase 2 (:658-696): merge of the chunks.
    All arithmetic here is fp32 (the reference forms q*k in the input dtype).
    """
    B, Hq, D = q.shape
    Hkv = k_pools[0].shape[2]
    bs = k_pools[0].shape[3]
    G = Hq // Hkv
    scale = np.float32(softmax_scale * LOG2E)
    neg = np.float32(-1e20)
    out = np.zeros((B, Hq, D), dtype=out_dtype)
    for b in range(B):
        n = int(seq_lens[b])
        kk, vv = gather_sequence_kv(k_pools, v_pools, block_table, int(seq_ids[b]), n, cur_layer,
                                    num_blocks_org, chunk_blocks)
        kk = kk.astype(np.float32)
        vv = vv.astype(np.float32)
        nchunks = (n + seq_block_size - 1) // seq_block_size
        for hq in range(Hq):
            h = hq // G
            qv = q[b, hq].astype(np.float32)
            mids, lses = [], []
            for c in range(nchunks):
                lo = c * seq_block_size
                hi = min(n, lo + seq_block_size)
                m = neg
                s = np.float32(0.0)
                acc = np.zeros(D, dtype=np.float32)
                for t0 in range(lo, hi, bs):
                    t1 = min(t0 + bs, hi)
                    sc = np.full(bs, neg, dtype=np.float32)
                    sc[: t1 - t0] = (kk[h, t0:t1] @ qv) * scale
                    vb = np.zeros((bs, D), dtype=np.float32)
                    vb[: t1 - t0] = vv[h, t0:t1]
                    new_m = np.maximum(m, sc.max())
                    p = np.exp2(sc - new_m).astype(np.float32)
                    a = np.exp2(m - new_m).astype(np.float32)
                    acc = acc * a + p @ vb
                    s = s * a + p.sum(dtype=np.float32)
                    m = new_m
                mids.append(acc / s)
                lses.append(np.float32(np.log2(s) + m))
            m = neg
            s = np.float32(0.0)
            acc = np.zeros(D, dtype=np.float32)
            for mid, lse in zip(mids, lses):
                new_m = np.maximum(m, lse)
                a = np.exp2(m - new_m).astype(np.float32)
                e = np.exp2(lse - new_m).astype(np.float32)
                acc = acc * a + e * mid
                s = s * a + e
                m = new_m
            out[b, hq] = round_to_output(acc / s, out_dtype)
    return out


def paged_attention_exact(q, k_pools, v_pools, block_table, seq_ids, seq_lens, cur_layer: int,
                          softmax_scale: float, num_blocks_org: int, chunk_blocks: int) -> np.ndarray:
    """float64 softmax(q k^T * scale) v per sequence, unrounded.  The yardstick
    both the reference and the CUDA path are measured against."""
    B, Hq, D = q.shape
    Hkv = k_pools[0].shape[2]
    G = Hq // Hkv
    out = np.zeros((B, Hq, D), dtype=np.float64)
    for b in range(B):
        n = int(seq_lens[b])
        kk, vv = gather_sequence_kv(k_pools, v_pools, block_table, int(seq_ids[b]), n, cur_layer,
                                    num_blocks_org, chunk_blocks)
        kk = np.repeat(kk.astype(np.float64), G, axis=0)      # [Hq, n, D]
        vv = np.repeat(vv.astype(np.float64), G, axis=0)
        sc = np.einsum("hd,hnd->hn", q[b].astype(np.float64), kk) * softmax_scale
        sc -= sc.max(axis=1, keepdims=True)
        p = np.exp(sc)
        p /= p.sum(axis=1, keepdims=True)
        out[b] = np.einsum("hn,hnd->hd", p, vv)
    return out


def paged_attention_torch_loop(q, k_pools, v_pools, block_table, seq_ids, seq_lens, cur_layer: int,
                               softmax_scale: float, num_blocks_org: int, chunk_blocks: int, o=None):
    """Live restatement of the reference's commented PyTorch path
    (worker/kernels/paged_attn.py:1397-1432): per sequence gather the blocks
    through the block table, concatenate along tokens, repeat_interleave the KV
    heads, fp32 bmm -> scale -> mask with -1e20 -> softmax -> bmm -> fp16.

    Arguments are torch CPU tensors (pools: lists of tensors).  This function is
    the "reference's PyTorch paged-attention path" that the benchmark times on
    the host cores.
    """
    import torch

    B, Hq, D = q.shape
    Hkv = k_pools[0].shape[2]
    bs = k_pools[0].shape[3]
    G = Hq // Hkv
    if o is None:
        o = torch.empty((B, Hq * D), dtype=torch.float16)
    lens = [int(x) for x in seq_lens]
    ids = [int(x) for x in seq_ids]
    for b in range(B):
        my_q = q[b]
        my_block_table = block_table[ids[b]]
        my_num_blocks = (lens[b] + bs - 1) // bs
        my_k_blocks, my_v_blocks = [], []
        for j in range(my_num_blocks):
            seg, row = locate_block(int(my_block_table[j]), num_blocks_org, chunk_blocks)
            my_k_blocks.append(k_pools[seg][row][cur_layer])
            my_v_blocks.append(v_pools[seg][row][cur_layer])
        my_k = torch.cat(my_k_blocks, dim=1).repeat_interleave(G, dim=0).to(torch.float32)
        my_v = torch.cat(my_v_blocks, dim=1).repeat_interleave(G, dim=0).to(torch.float32)
        my_q = my_q.reshape(Hq, 1, D).to(torch.float32)
        score = torch.bmm(my_q, my_k.transpose(1, 2)).squeeze(1) * softmax_scale
        score = torch.where(torch.arange(score.shape[1]) < lens[b], score,
                            torch.full_like(score, float("-1e20")))
        score = torch.softmax(score, dim=1).unsqueeze(1)
        res = torch.bmm(score, my_v).squeeze(1)
        o[b] = res.reshape(-1).to(torch.float16).to(o.dtype)
    return o


# --------------------------------------------------------------------------
# block table (integers, exact)
# --------------------------------------------------------------------------
class BlockManagerOracle:
    """CPU restatement of worker/block_manager.py:5-137 and the three kernels
    of worker/kernels/block_mgmt.py.  State is numpy; ``num_free_blocks`` is a
    plain int (the reference's becomes a 0-d tensor after the first free,
    block_manager.py:118 - a type quirk, not a value difference)."""

    def __init__(self, num_blocks: int, max_seqs: int, max_blocks_per_seq: int, block_size: int):
        self.num_blocks = num_blocks
        self.num_free_blocks = num_blocks
        self.num_blocks_org = num_blocks
        self.num_free_blocks_org = num_blocks
        self.block_size = block_size
        self.num_seq_allocated_blocks = np.zeros(max_seqs, dtype=np.int32)
        self.block_table = np.full((max_seqs, max_blocks_per_seq), -1, dtype=np.int32)
        self.is_block_free = np.ones(num_blocks, dtype=bool)

    def get_num_used_blocks(self) -> int:
        return self.num_blocks - self.num_free_blocks

    def _allocate_blocks(self, n: int) -> np.ndarray:
        # block_manager.py:64-79: first-fit, ascending ids.
        if n > self.num_free_blocks:
            raise RuntimeError("No enough free blocks available")
        sel = np.nonzero(self.is_block_free)[0][:n].astype(np.int64)
        self.num_free_blocks -= n
        self.is_block_free[sel] = False
        return sel

    def allocate_blocks_for_seqs(self, seq_ids, target_lens) -> np.ndarray:
        # block_manager.py:87-112 + block_mgmt.py:5-46.
        seq_ids = np.asarray(seq_ids, dtype=np.int64)
        target = (np.asarray(target_lens, dtype=np.int64) + (self.block_size - 1)) // self.block_size
        have = self.num_seq_allocated_blocks[seq_ids].astype(np.int64)
        assert (have <= target).all(), "Logic error: Some sequences have more blocks already allocated than needed."
        need = target - have
        n = int(need.sum())
        if n == 0:
            return np.empty(0, dtype=np.int64)
        new_blocks = self._allocate_blocks(n)
        cum = np.cumsum(need)
        for i, s in enumerate(seq_ids):
            lo = cum[i] - need[i]
            a = int(self.num_seq_allocated_blocks[s])
            self.block_table[s, a:a + need[i]] = new_blocks[lo:cum[i]]
            self.num_seq_allocated_blocks[s] = a + need[i]
        return new_blocks

    def free_blocks_for_seqs(self, seq_ids) -> None:
        # block_manager.py:114-119 + block_mgmt.py:49-80.  Rows keep their ids.
        seq_ids = np.asarray(seq_ids, dtype=np.int64)
        self.num_free_blocks += int(self.num_seq_allocated_blocks[seq_ids].sum())
        for s in seq_ids:
            c = int(self.num_seq_allocated_blocks[s])
            self.is_block_free[self.block_table[s, :c]] = True
            self.num_seq_allocated_blocks[s] = 0

    def gather_allocated_blocks_and_free(self, seq_ids) -> np.ndarray:
        # block_manager.py:121-129 + block_mgmt.py:83-125.  int32 ids, batch order.
        seq_ids = np.asarray(seq_ids, dtype=np.int64)
        out = []
        for s in seq_ids:
            c = int(self.num_seq_allocated_blocks[s])
            ids = self.block_table[s, :c].copy()
            out.append(ids)
            self.is_block_free[ids] = True
            self.num_seq_allocated_blocks[s] = 0
        g = np.concatenate(out).astype(np.int32) if out else np.empty(0, dtype=np.int32)
        self.num_free_blocks += len(g)
        return g

    def get_num_allocated_blocks(self, seq_ids) -> np.ndarray:
        return self.num_seq_allocated_blocks[np.asarray(seq_ids, dtype=np.int64)]


# --------------------------------------------------------------------------
# elastic resize
# --------------------------------------------------------------------------
def chunk_layout(org_start: int, org_size: int, quant_size: int,
                 num_layers: int, num_kv_heads: int, block_size: int, head_dim: int):
    """Where an elastic chunk sits inside a freed weight slab, and how many
    blocks it holds.  csrc/src/memory_manager.cpp:84-97,129-147 (fp16 is
    hard-coded there).  Returns (k_addr, v_addr, n_blocks); raises RuntimeError
    when no block fits (:99-101)."""
    layer_end = org_start + quant_size
    new_kv_start = (layer_end + 255) & ~255
    available = org_size - (new_kv_start - org_start)
    kv_slot = 2 * num_layers * num_kv_heads * head_dim * 2
    kv_block = kv_slot * block_size
    n = available // kv_block if available > 0 else 0
    if n == 0:
        raise RuntimeError("No space available for new KV cache blocks")
    return new_kv_start, new_kv_start + n * (kv_block // 2), n


def expand(bm: BlockManagerOracle, n_new: int) -> None:
    """Bookkeeping after a chunk of ``n_new`` blocks was attached.
    server/memory_utils.py:405-417."""
    bm.num_blocks += n_new
    bm.num_free_blocks += n_new
    bm.is_block_free = np.concatenate([bm.is_block_free, np.ones(n_new, dtype=bool)])


def can_release_last_chunk(bm: BlockManagerOracle, n_chunks: int, chunk_blocks: int) -> bool:
    """server/memory_utils.py:529-544: only the last chunk, only if all free."""
    start = bm.num_blocks_org + chunk_blocks * (n_chunks - 1)
    return bool(bm.is_block_free[start:start + chunk_blocks].all())


def release_last_chunk(bm: BlockManagerOracle, chunk_blocks: int) -> None:
    """server/memory_utils.py:648-651."""
    bm.num_blocks -= chunk_blocks
    bm.num_free_blocks -= chunk_blocks
    bm.is_block_free = bm.is_block_free[:-chunk_blocks]


def compaction_plan(is_block_free: np.ndarray, target_blocks: int):
    """Move plan that empties every block id >= ``target_blocks``.

    The reference has no compaction (release needs an already-empty tail,
    server/memory_utils.py:529-544,622-624); this is the rule the product
    defines: ``src`` = ascending used ids >= T, ``dst`` = the first len(src)
    ascending free ids < T (the same first-fit order as
    worker/block_manager.py:75).  Returns None when too few free ids exist.
    """
    used_hi = np.nonzero(~is_block_free[target_blocks:])[0] + target_blocks
    free_lo = np.nonzero(is_block_free[:target_blocks])[0]
    if len(free_lo) < len(used_hi):
        return None
    return used_hi.astype(np.int64), free_lo[:len(used_hi)].astype(np.int64)


def compact(bm: BlockManagerOracle, k_pools, v_pools, target_blocks: int, chunk_blocks: int) -> int:
    """Apply compaction_plan: copy K/V blocks (all layers), rewrite live table
    entries, flip the free bitmap.  Source blocks keep their bytes; stale table
    columns and rows of freed sequences are left as they are.  Returns the
    number of moved blocks, or -1 (nothing changed) when it does not fit."""
    plan = compaction_plan(bm.is_block_free, target_blocks)
    if plan is None:
        return -1
    src, dst = plan
    for s, d in zip(src, dst):
        ss, sr = locate_block(s, bm.num_blocks_org, chunk_blocks)
        ds, dr = locate_block(d, bm.num_blocks_org, chunk_blocks)
        k_pools[ds][dr] = k_pools[ss][sr]
        v_pools[ds][dr] = v_pools[ss][sr]
    remap = {int(s): int(d) for s, d in zip(src, dst)}
    for row in range(bm.block_table.shape[0]):
        c = int(bm.num_seq_allocated_blocks[row])
        for j in range(c):
            e = int(bm.block_table[row, j])
            if e in remap:
                bm.block_table[row, j] = remap[e]
    bm.is_block_free[dst] = False
    bm.is_block_free[src] = True
    return len(src)


# --------------------------------------------------------------------------
# swap
# --------------------------------------------------------------------------
def coalesce_runs(src_ids: Sequence[int], dst_ids: Sequence[int],
                  num_blocks_org: int = None, chunk_blocks: int = None):
    """Runs (start index, length) in which source and target ids both advance
    by one (csrc/src/block_swapping.cpp:36-43); with elastic chunks a run also
    ends where either side crosses a chunk boundary (:109-118,138-147)."""
    def flag(x):
        if num_blocks_org is None or x < num_blocks_org:
            return -1
        return (x - num_blocks_org) // chunk_blocks
    runs = []
    i, n = 0, len(src_ids)
    while i < n:
        j = i + 1
        while (j < n and src_ids[j] == src_ids[j - 1] + 1 and dst_ids[j] == dst_ids[j - 1] + 1
               and flag(src_ids[j]) == flag(src_ids[j - 1]) and flag(dst_ids[j]) == flag(dst_ids[j - 1])):
            j += 1
        runs.append((i, j - i))
        i = j
    return runs


def swap_blocks(src_ids, dst_ids, is_swap_in: bool, k_pools, v_pools, k_swap, v_swap,
                num_blocks_org: int, chunk_blocks: int) -> None:
    """Block copy between the device pool and the host swap space.
    csrc/src/block_swapping.cpp:22-85.  On swap-in the device address comes
    from the TARGET id, the host address from the source id (:49-64); the
    elastic variant of the reference takes the device address from the source
    id on swap-in (:156-161), which is a defect and is not restated."""
    for s, d in zip(src_ids, dst_ids):
        if is_swap_in:
            seg, row = locate_block(d, num_blocks_org, chunk_blocks)
            k_pools[seg][row] = k_swap[s]
            v_pools[seg][row] = v_swap[s]
        else:
            seg, row = locate_block(s, num_blocks_org, chunk_blocks)
            k_swap[d] = k_pools[seg][row]
            v_swap[d] = v_pools[seg][row]
