"""Seeded input builders shared by the golden-vector generator and the tests.

Inputs are drawn with numpy's legacy ``RandomState`` (a frozen bit stream), so
the same seed reproduces the same bytes on any machine; every fixture also
records a SHA-256 of the inputs it was generated from.

A case is a dict of numpy arrays plus scalars:
  q [B,Hq,D], k_new/v_new [B,Hkv,D], pools (lists of [n,L,Hkv,bs,D]),
  block_table [max_seqs, max_blocks_per_seq] int32, seq_ids [B] int32,
  seq_lens [B] int32 (length INCLUDING the token appended this step),
  layer, num_blocks_org, chunk_blocks, scale.
"""
from __future__ import annotations

import hashlib

import numpy as np


def sha256_of(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(a)
        h.update(str(a.dtype).encode())
        h.update(str(a.shape).encode())
        h.update(a.tobytes())
    return h.hexdigest()


def build_decode_case(seed: int, B: int, Hq: int, Hkv: int, D: int, bs: int, L: int, layer: int,
                      num_blocks_org: int, dtype, lens=None, max_len: int = 512,
                      chunk_blocks: int = 0, n_chunks: int = 0, max_seqs: int = None,
                      max_blocks_per_seq: int = None, force_high_ids: bool = False):
    """Draw order: lengths -> permutation -> K -> V -> q -> k_new -> v_new."""
    rs = np.random.RandomState(seed)
    if lens is None:
        lens = rs.randint(1, max_len + 1, size=B)
    lens = np.asarray(lens, dtype=np.int32)
    total_blocks = num_blocks_org + chunk_blocks * n_chunks
    perm = rs.permutation(total_blocks)
    if force_high_ids:
        # put elastic ids first so that short cases still touch every chunk
        perm = np.concatenate([perm[perm >= num_blocks_org], perm[perm < num_blocks_org]])
    need = (lens + bs - 1) // bs
    assert need.sum() <= total_blocks, "pool too small for the case"
    max_seqs = max_seqs or (B + 3)
    max_blocks_per_seq = max_blocks_per_seq or int(need.max()) + 2
    seq_ids = rs.permutation(max_seqs)[:B].astype(np.int32)
    block_table = np.full((max_seqs, max_blocks_per_seq), -1, dtype=np.int32)
    pos = 0
    for b in range(B):
        block_table[seq_ids[b], :need[b]] = perm[pos:pos + need[b]]
        pos += need[b]

    def pool_list():
        pools = [rs.standard_normal((num_blocks_org, L, Hkv, bs, D)).astype(dtype)]
        for _ in range(n_chunks):
            pools.append(rs.standard_normal((chunk_blocks, L, Hkv, bs, D)).astype(dtype))
        return pools

    k_pools = pool_list()
    v_pools = pool_list()
    q = rs.standard_normal((B, Hq, D)).astype(dtype)
    k_new = rs.standard_normal((B, Hkv, D)).astype(dtype)
    v_new = rs.standard_normal((B, Hkv, D)).astype(dtype)
    return dict(q=q, k_new=k_new, v_new=v_new, k_pools=k_pools, v_pools=v_pools,
                block_table=block_table, seq_ids=seq_ids, seq_lens=lens, layer=layer,
                num_blocks_org=num_blocks_org, chunk_blocks=chunk_blocks, n_chunks=n_chunks,
                scale=float(D) ** -0.5, B=B, Hq=Hq, Hkv=Hkv, D=D, bs=bs, L=L)


def case_inputs_hash(c) -> str:
    return sha256_of(c["q"], c["k_new"], c["v_new"], *c["k_pools"], *c["v_pools"],
                     c["block_table"], c["seq_ids"], c["seq_lens"])


# name -> kwargs of build_decode_case.  cfg1* is the CPU-plumbing configuration: 4 sequences, 32 MHA heads,
# head_dim 128, block 16, fp32, contexts uniform in [1,512], 256-block pool.
DECODE_CASES = {
    "cfg1_mha_fp32": dict(seed=1000, B=4, Hq=32, Hkv=32, D=128, bs=16, L=1, layer=0,
                          num_blocks_org=256, dtype=np.float32, max_len=512),
    "cfg1_mha_fp32_layer1": dict(seed=1001, B=4, Hq=32, Hkv=32, D=128, bs=16, L=2, layer=1,
                                 num_blocks_org=160, dtype=np.float32, max_len=512),
    "gqa4_fp16": dict(seed=2000, B=7, Hq=8, Hkv=2, D=128, bs=16, L=2, layer=1,
                      num_blocks_org=96, dtype=np.float16,
                      lens=[1, 15, 16, 17, 100, 512, 333]),
    "gqa8_fp16": dict(seed=2001, B=3, Hq=8, Hkv=1, D=128, bs=16, L=3, layer=2,
                      num_blocks_org=64, dtype=np.float16, lens=[64, 129, 600]),
    "mha_fp16": dict(seed=2002, B=5, Hq=4, Hkv=4, D=128, bs=16, L=2, layer=0,
                     num_blocks_org=64, dtype=np.float16, lens=[2, 31, 32, 33, 257]),
    "gqa4_fp16_elastic": dict(seed=3000, B=6, Hq=8, Hkv=2, D=128, bs=16, L=2, layer=1,
                              num_blocks_org=24, dtype=np.float16, chunk_blocks=8, n_chunks=2,
                              lens=[5, 40, 130, 16, 77, 200], force_high_ids=True),
}


def build_prefill_case(seed: int, lens, Hkv: int, D: int, bs: int, L: int, layer: int,
                       num_blocks_org: int, dtype, chunk_blocks: int = 0, n_chunks: int = 0,
                       n_decode: int = 0, decode_lens=None):
    """Mixed batch for store_kvcache: prefill sequences first, decode after."""
    rs = np.random.RandomState(seed)
    lens = np.asarray(lens, dtype=np.int32)
    decode_lens = np.asarray(decode_lens if decode_lens is not None else [], dtype=np.int32)
    all_lens = np.concatenate([lens, decode_lens])
    nseq = len(all_lens)
    total_blocks = num_blocks_org + chunk_blocks * n_chunks
    perm = rs.permutation(total_blocks)
    need = (all_lens + bs - 1) // bs
    assert need.sum() <= total_blocks
    max_seqs = nseq + 2
    mbps = int(need.max()) + 1
    seq_ids = rs.permutation(max_seqs)[:nseq].astype(np.int32)
    block_table = np.full((max_seqs, mbps), -1, dtype=np.int32)
    pos = 0
    for i in range(nseq):
        block_table[seq_ids[i], :need[i]] = perm[pos:pos + need[i]]
        pos += need[i]
    ntok = int(lens.sum()) + len(decode_lens)
    k = rs.standard_normal((ntok, Hkv, D)).astype(dtype)
    v = rs.standard_normal((ntok, Hkv, D)).astype(dtype)
    k_pools = [np.zeros((num_blocks_org, L, Hkv, bs, D), dtype=dtype)]
    v_pools = [np.zeros((num_blocks_org, L, Hkv, bs, D), dtype=dtype)]
    for _ in range(n_chunks):
        k_pools.append(np.zeros((chunk_blocks, L, Hkv, bs, D), dtype=dtype))
        v_pools.append(np.zeros((chunk_blocks, L, Hkv, bs, D), dtype=dtype))
    start_locs = (np.cumsum(lens) - lens).astype(np.int32)
    return dict(k=k, v=v, k_pools=k_pools, v_pools=v_pools, block_table=block_table,
                seq_ids=seq_ids, prefill_lens=lens, prefill_start_locs=start_locs,
                decode_lens=decode_lens, layer=layer, num_blocks_org=num_blocks_org,
                chunk_blocks=chunk_blocks, n_chunks=n_chunks, Hkv=Hkv, D=D, bs=bs, L=L,
                num_prefill_tokens=int(lens.sum()))


PREFILL_CASES = {
    "mixed_fp16": dict(seed=4000, lens=[1, 16, 17, 50], Hkv=2, D=128, bs=16, L=2, layer=1,
                       num_blocks_org=32, dtype=np.float16, decode_lens=[3, 33]),
    "mixed_fp16_elastic": dict(seed=4001, lens=[20, 7, 48], Hkv=2, D=128, bs=16, L=2, layer=0,
                               num_blocks_org=6, dtype=np.float16, chunk_blocks=4, n_chunks=2,
                               decode_lens=[18]),
}


def rope_tables(positions, D: int, theta: float = 10000.0, scaling: float = 1.0):
    """cos/sin rows for the given token positions, built like the reference's table
    (worker/model.py:229-241): fp32 angles, rounded to fp16."""
    inv_freq = (1.0 / (np.float32(theta) ** (np.arange(0, D, 2, dtype=np.float32) / np.float32(D)))).astype(np.float32)
    t = (np.asarray(positions, dtype=np.float32) / np.float32(scaling)).astype(np.float32)
    freqs = np.outer(t, inv_freq).astype(np.float32)
    return np.cos(freqs).astype(np.float16), np.sin(freqs).astype(np.float16)


def build_rope_case(seed: int, T: int, Hq: int, Hkv: int, D: int, max_pos: int = 4096, dtype=np.float16):
    """Draw order: positions -> q -> k."""
    rs = np.random.RandomState(seed)
    pos = rs.randint(0, max_pos, size=T)
    q = rs.standard_normal((T, Hq, D)).astype(dtype)
    k = rs.standard_normal((T, Hkv, D)).astype(dtype)
    cos, sin = rope_tables(pos, D)
    return dict(q=q, k=k, cos=cos, sin=sin, positions=pos.astype(np.int32), T=T, Hq=Hq, Hkv=Hkv, D=D)


ROPE_CASES = {
    "gqa4_fp16": dict(seed=6000, T=9, Hq=8, Hkv=2, D=128),
    "mha_fp16": dict(seed=6001, T=5, Hq=4, Hkv=4, D=128),
    "gqa8_d64_fp16": dict(seed=6002, T=3, Hq=8, Hkv=1, D=64),
    "mha_fp32": dict(seed=6003, T=4, Hq=4, Hkv=4, D=128, dtype=np.float32),
}


def block_manager_trace(seed: int = 5000, num_blocks: int = 64, max_seqs: int = 12,
                        max_blocks_per_seq: int = 16, block_size: int = 16, steps: int = 40):
    """A seeded sequence of BlockManager operations: list of (op, seq_ids, lens)."""
    rs = np.random.RandomState(seed)
    lens = np.zeros(max_seqs, dtype=np.int64)
    ops = []
    free = num_blocks
    for _ in range(steps):
        r = rs.rand()
        if r < 0.6:
            n = rs.randint(1, 5)
            ids = rs.permutation(max_seqs)[:n]
            new = lens[ids] + rs.randint(0, 40, size=n)
            new = np.minimum(new, max_blocks_per_seq * block_size)
            need = ((new + block_size - 1) // block_size - (lens[ids] + block_size - 1) // block_size).sum()
            if need > free:
                continue
            free -= need
            lens[ids] = new
            ops.append(("alloc", ids.astype(np.int32), new.astype(np.int32)))
        elif r < 0.8:
            n = rs.randint(1, 4)
            ids = rs.permutation(max_seqs)[:n]
            free += ((lens[ids] + block_size - 1) // block_size).sum()
            lens[ids] = 0
            ops.append(("free", ids.astype(np.int32), None))
        else:
            n = rs.randint(1, 4)
            ids = rs.permutation(max_seqs)[:n]
            if ((lens[ids] + block_size - 1) // block_size).sum() == 0:
                continue
            free += ((lens[ids] + block_size - 1) // block_size).sum()
            lens[ids] = 0
            ops.append(("gather", ids.astype(np.int32), None))
    return dict(num_blocks=num_blocks, max_seqs=max_seqs, max_blocks_per_seq=max_blocks_per_seq,
                block_size=block_size, ops=ops)
