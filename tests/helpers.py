"""Helpers shared by the GPU parity tests: move a seeded case to the device and
call the package exactly as the reference's worker would."""
from __future__ import annotations

import types

import numpy as np
import torch


def cfgs(c, max_blocks_per_seq):
    model_config = types.SimpleNamespace(num_layers=c["L"], num_q_heads=c.get("Hq", c["Hkv"]),
                                         num_kv_heads=c["Hkv"], head_dim=c["D"])
    engine_config = types.SimpleNamespace(block_size=c["bs"], max_blocks_per_seq=max_blocks_per_seq)
    return model_config, engine_config


def to_dev(a, dev="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def decode_state(c, seq_ids, seq_lens, sbs=512):
    from morphserve_b200.worker.infer_state import LlamaInferState
    lens_list = [int(x) for x in seq_lens.tolist()]
    z = torch.zeros(0, dtype=torch.int32, device="cuda")
    max_len = max(lens_list) if lens_list else 0
    return LlamaInferState(
        batch_size=len(lens_list), num_tokens=len(lens_list), seq_ids=seq_ids, softmax_scale=c["scale"],
        num_prefill_seqs=0, num_prefill_tokens=0, prefill_seq_start_locs=z, prefill_seq_start_locs_with_end=z,
        prefill_seq_lens=z, max_prefill_len=0, num_decoding_seqs=len(lens_list), decoding_seq_lens=seq_lens,
        max_decoding_len=max_len, seq_block_size=sbs, num_seq_blocks=(max_len + sbs - 1) // sbs,
        num_blocks_org=c["num_blocks_org"], kv_cache_new_block_size=c["chunk_blocks"],
        org_layer_param_size=0, position_cos=z, position_sin=z, ignore_kvcache=False)


def device_case(c):
    """numpy case -> dict of CUDA tensors (pools as [main] + chunks)."""
    d = dict(c)
    d["k_pools_t"] = [to_dev(p) for p in c["k_pools"]]
    d["v_pools_t"] = [to_dev(p) for p in c["v_pools"]]
    d["q_t"] = to_dev(c["q"])
    d["k_new_t"] = to_dev(c["k_new"])
    d["v_new_t"] = to_dev(c["v_new"])
    d["block_table_t"] = to_dev(c["block_table"])
    d["seq_ids_t"] = to_dev(c["seq_ids"])
    d["seq_lens_t"] = to_dev(c["seq_lens"])
    return d


def run_decode_step(d):
    """store_kvcache + paged_attention through the public API; returns o [B,Hq,D] (numpy)
    and the pools after the append (numpy lists)."""
    from morphserve_b200 import paged_attention, store_kvcache
    mc, ec = cfgs(d, d["block_table_t"].shape[1])
    st = decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    kc, vc = d["k_pools_t"][0], d["v_pools_t"][0]
    kn, vn = d["k_pools_t"][1:], d["v_pools_t"][1:]
    store_kvcache(d["k_new_t"], d["v_new_t"], kc, vc, kn, vn, d["block_table_t"], mc, ec, st, d["layer"])
    o = torch.zeros((d["B"], d["Hq"] * d["D"]), dtype=d["q_t"].dtype, device="cuda")
    paged_attention(d["q_t"], kc, vc, kn, vn, d["block_table_t"], mc, ec, st, d["layer"], o)
    torch.cuda.synchronize()
    return (o.cpu().numpy().reshape(d["B"], d["Hq"], d["D"]),
            [p.cpu().numpy() for p in d["k_pools_t"]], [p.cpu().numpy() for p in d["v_pools_t"]])


def plan_rule(lens, num_kv_heads, batch_cap_items, sm_count, split_balance=1.5, block_size=16):
    """What the decode plan kernel must decide for a batch (restated on the host for the tests): chunk size in
    blocks, number of (sequence, chunk) items, number of partial rows.  Candidates 4,6,8,12,...; the smallest one
    whose item count fits the cap, raised to the largest one not above split_balance x the mean number of blocks per
    worker warp; a remainder of up to a quarter chunk stays with the piece before it."""
    nblk = [(int(n) + block_size - 1) // block_size for n in lens if n > 0]
    cand = [(6 << (k >> 1)) if k & 1 else (4 << (k >> 1)) for k in range(40)]
    k = 0
    while k < 39 and sum(-(-n // cand[k]) for n in nblk) > batch_cap_items:
        k += 1
    keep_whole = np.float32(np.float32(split_balance * num_kv_heads / (sm_count * 8.0)) * np.float32(sum(nblk)))
    while k < 39 and np.float32(cand[k + 1]) <= keep_whole:
        k += 1
    chunk = cand[k]
    items = rows = 0
    for n in nblk:
        ns = -(-n // chunk)
        if ns > 1 and n - (ns - 1) * chunk <= chunk // 4:
            ns -= 1
        items += ns
        rows += ns if ns > 1 else 0
    return chunk, items, rows


def static_deal(lens, num_kv_heads, workers, cap_rows, group, unit_cost=1, block_size=16):
    """The plan's static deal restated on the host.  Tiles are ordered sequence by sequence, kv head by kv head,
    block by block, with `unit_cost` phantom tiles in front of every non-empty (sequence, head); worker w of W owns
    tiles [w*T//W, (w+1)*T//W) of that order, phantoms included, where W = min(workers, T, cap_rows // (2 * group)).
    A range is cut into units where the (sequence, head) changes; pieces made of phantoms only are no units.
    Returns (W, wstart, units) with units[i] = (batch index, first block, blocks, piece, head, len, pieces, first
    owner)."""
    oc = unit_cost
    nblk = [(int(n) + block_size - 1) // block_size + oc if n > 0 else 0 for n in lens]
    T = sum(nblk) * num_kv_heads
    W = min(workers, T, cap_rows // (2 * group))
    pairs = []                                   # (first tile, b, h, tiles incl. phantoms)
    t = 0
    for b, n in enumerate(nblk):
        for h in range(num_kv_heads if n else 0):
            pairs.append((t, b, h, n))
            t += n

    def owner(tile):
        return ((tile + 1) * W - 1) // T

    units, wstart = [], [0]
    pi = 0
    for w in range(W):
        lo, hi = w * T // W, (w + 1) * T // W
        while pi < len(pairs) and pairs[pi][0] + pairs[pi][3] <= lo:
            pi += 1
        pj = pi
        while pj < len(pairs) and pairs[pj][0] < hi:
            p0, b, h, n = pairs[pj]
            a, z = max(lo, p0), min(hi, p0 + n)
            if z - p0 > oc:                      # real tiles in the piece
                f, last = owner(p0 + oc), owner(p0 + n - 1)
                first = max(a - p0, oc) - oc
                units.append((b, first, z - p0 - oc - first, w - f, h, int(lens[b]), last - f + 1, f))
            pj += 1
        wstart.append(len(units))
    return W, wstart, units
