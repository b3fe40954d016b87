"""GPU parity for the elastic pool: expand, release rule, compaction with
block-table remap, and swap.  After every mutation the device state is compared
with the CPU oracle: tables, counts and bitmap exactly, K/V bytes exactly."""
import types

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from tests import helpers as H
from tests.golden import cases

pytestmark = pytest.mark.gpu


class Twin:
    """The product objects on the GPU next to the oracle on the CPU, driven in lockstep."""

    def __init__(self, L, Hkv, D, bs, nb_org, max_seqs, mbps, seed):
        from morphserve_b200 import BlockManager
        self.L, self.Hkv, self.D, self.bs = L, Hkv, D, bs
        self.rs = np.random.RandomState(seed)
        shape = (nb_org, L, Hkv, bs, D)
        self.model = types.SimpleNamespace(
            k_cache=torch.zeros(shape, dtype=torch.float16, device="cuda"),
            v_cache=torch.zeros(shape, dtype=torch.float16, device="cuda"),
            k_cache_new=[], v_cache_new=[], kv_cache_new_block_size=0,
            gpu_block_manager=BlockManager("GPU", nb_org, max_seqs, mbps, bs))
        self.engine = types.SimpleNamespace(model=self.model, scheduler=types.SimpleNamespace(num_gpu_blocks=nb_org))
        self.obm = O.BlockManagerOracle(nb_org, max_seqs, mbps, bs)
        self.ok = [np.zeros(shape, dtype=np.float16)]
        self.ov = [np.zeros(shape, dtype=np.float16)]
        self.chunk = 0
        self.lens = {}

    # ---- mutations -----------------------------------------------------------
    def admit(self, seq_id, length):
        ids = np.array([seq_id], dtype=np.int32)
        ln = np.array([length], dtype=np.int32)
        new = self.model.gpu_block_manager.allocate_blocks_for_seqs(H.to_dev(ids), H.to_dev(ln))
        onew = self.obm.allocate_blocks_for_seqs(ids, ln)
        np.testing.assert_array_equal(new.cpu().numpy(), onew)
        self.lens[seq_id] = length
        # fill the new blocks with data (stands for prefill)
        for b in onew:
            kb = self.rs.standard_normal((self.L, self.Hkv, self.bs, self.D)).astype(np.float16)
            vb = self.rs.standard_normal((self.L, self.Hkv, self.bs, self.D)).astype(np.float16)
            seg, row = O.locate_block(b, self.obm.num_blocks_org, max(self.chunk, 1))
            self.ok[seg][row] = kb
            self.ov[seg][row] = vb
            kt = self.model.k_cache if seg == 0 else self.model.k_cache_new[seg - 1]
            vt = self.model.v_cache if seg == 0 else self.model.v_cache_new[seg - 1]
            kt[row].copy_(H.to_dev(kb))
            vt[row].copy_(H.to_dev(vb))

    def free(self, seq_ids):
        ids = np.array(seq_ids, dtype=np.int32)
        self.model.gpu_block_manager.free_blocks_for_seqs(H.to_dev(ids))
        self.obm.free_blocks_for_seqs(ids)
        for s in seq_ids:
            self.lens.pop(s, None)

    def expand(self, n):
        from morphserve_b200.server import memory_utils as MU
        shape = (n, self.L, self.Hkv, self.bs, self.D)
        MU.attach_kvcache_chunk(self.engine, torch.zeros(shape, dtype=torch.float16, device="cuda"),
                                torch.zeros(shape, dtype=torch.float16, device="cuda"))
        O.expand(self.obm, n)
        self.ok.append(np.zeros(shape, dtype=np.float16))
        self.ov.append(np.zeros(shape, dtype=np.float16))
        self.chunk = n

    def decode_step(self, seq_ids, layers):
        """allocate -> per layer (append, attention); compares attention with the oracle."""
        from morphserve_b200 import paged_attention, store_kvcache
        for s in seq_ids:
            self.lens[s] += 1
        ids = np.array(seq_ids, dtype=np.int32)
        lens = np.array([self.lens[s] for s in seq_ids], dtype=np.int32)
        bm = self.model.gpu_block_manager
        new = bm.allocate_blocks_for_seqs(H.to_dev(ids), H.to_dev(lens))
        onew = self.obm.allocate_blocks_for_seqs(ids, lens)
        np.testing.assert_array_equal(new.cpu().numpy(), onew)
        c = dict(L=self.L, Hq=self.Hkv * 4, Hkv=self.Hkv, D=self.D, bs=self.bs, scale=self.D ** -0.5,
                 num_blocks_org=self.obm.num_blocks_org, chunk_blocks=self.chunk)
        mc, ec = H.cfgs(c, bm.block_table.shape[1])
        st = H.decode_state(c, H.to_dev(ids), H.to_dev(lens))
        for layer in layers:
            q = self.rs.standard_normal((len(ids), c["Hq"], self.D)).astype(np.float16)
            k = self.rs.standard_normal((len(ids), self.Hkv, self.D)).astype(np.float16)
            v = self.rs.standard_normal((len(ids), self.Hkv, self.D)).astype(np.float16)
            store_kvcache(H.to_dev(k), H.to_dev(v), self.model.k_cache, self.model.v_cache, self.model.k_cache_new,
                          self.model.v_cache_new, bm.block_table, mc, ec, st, layer)
            O.store_kvcache_decode(k, v, self.ok, self.ov, self.obm.block_table, ids, lens, layer,
                                   self.obm.num_blocks_org, max(self.chunk, 1))
            o = torch.zeros((len(ids), c["Hq"] * self.D), dtype=torch.float16, device="cuda")
            paged_attention(H.to_dev(q), self.model.k_cache, self.model.v_cache, self.model.k_cache_new,
                            self.model.v_cache_new, bm.block_table, mc, ec, st, layer, o)
            ex = O.paged_attention_exact(q, self.ok, self.ov, self.obm.block_table, ids, lens, layer, c["scale"],
                                         self.obm.num_blocks_org, max(self.chunk, 1))
            np.testing.assert_allclose(o.cpu().numpy().reshape(ex.shape).astype(np.float64), ex, rtol=2e-3, atol=1e-2)

    # ---- comparison ------------------------------------------------------------
    def check(self, raw_pools=True):
        bm = self.model.gpu_block_manager
        np.testing.assert_array_equal(bm.block_table.cpu().numpy(), self.obm.block_table)
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), self.obm.num_seq_allocated_blocks)
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), self.obm.is_block_free)
        assert bm.num_blocks == self.obm.num_blocks
        assert int(bm.num_free_blocks) == self.obm.num_free_blocks
        assert self.engine.scheduler.num_gpu_blocks == self.obm.num_blocks
        assert len(self.model.k_cache_new) == len(self.ok) - 1
        if raw_pools:
            dk = [self.model.k_cache] + self.model.k_cache_new
            dv = [self.model.v_cache] + self.model.v_cache_new
            for a, b in zip(dk + dv, self.ok + self.ov):
                assert a.cpu().numpy().tobytes() == b.tobytes()


def _trace(nb_org, chunk, n_chunks, release, L, Hkv, batch, steps, seed, max_len):
    from morphserve_b200.server import memory_utils as MU
    bs, D = 16, 128
    mbps = (max_len + steps * 3) // bs + 2
    tw = Twin(L, Hkv, D, bs, nb_org, max_seqs=4096, mbps=mbps, seed=seed)
    rs = np.random.RandomState(seed + 1)
    next_id = [0]

    def admit_until(frac):
        while tw.obm.get_num_used_blocks() < frac * tw.obm.num_blocks:
            ln = int(rs.randint(1, max_len + 1))
            if (ln + bs - 1) // bs > tw.obm.num_free_blocks:
                break
            tw.admit(next_id[0], ln)
            next_id[0] += 1

    layers = list(range(L))
    admit_until(0.85)
    tw.check()
    running = list(rs.permutation(list(tw.lens))[:batch])
    for _ in range(steps):
        tw.decode_step(running, layers)
    tw.check()
    for _ in range(n_chunks):
        tw.expand(chunk)
    tw.check()
    admit_until(0.85)
    running = list(rs.permutation(list(tw.lens))[:batch])
    for _ in range(steps):
        tw.decode_step(running, layers)
    tw.check()
    # free a seeded random subset until 40 % of the pool is free
    order = list(rs.permutation(list(tw.lens)))
    while tw.obm.num_free_blocks < 0.4 * tw.obm.num_blocks + 1 and order:
        tw.free([order.pop()])
    tw.check()
    assert not MU.if_kv_cache_unused(tw.engine) or True    # may or may not be empty; release decides below
    target = tw.obm.num_blocks_org + (n_chunks - release) * chunk
    moved = MU.compact_kvcache(tw.engine, target)
    omoved = O.compact(tw.obm, tw.ok, tw.ov, target, chunk)
    assert moved == omoved and moved >= 0
    tw.check()                                   # raw pools: source blocks keep their bytes
    for _ in range(release):
        assert MU.release_last_kvcache_chunk(tw.engine)
        assert O.can_release_last_chunk(tw.obm, len(tw.ok) - 1, chunk)
        O.release_last_chunk(tw.obm, chunk)
        tw.ok.pop()
        tw.ov.pop()
    tw.check()
    running = [s for s in running if s in tw.lens][:batch]
    for _ in range(steps):
        tw.decode_step(running, layers)
    tw.check()
    return moved


def test_elastic_trace_small():
    moved = _trace(nb_org=96, chunk=16, n_chunks=4, release=3, L=2, Hkv=2, batch=6, steps=5, seed=41, max_len=200)
    assert moved > 0


def test_elastic_trace_medium():
    _trace(nb_org=512, chunk=64, n_chunks=8, release=6, L=2, Hkv=2, batch=24, steps=6, seed=42, max_len=600)


def test_release_refused_while_last_chunk_is_live():
    from morphserve_b200.server import memory_utils as MU
    tw = Twin(1, 1, 128, 16, 8, max_seqs=16, mbps=8, seed=3)
    tw.expand(4)
    for s in range(5):
        tw.admit(s, 32)          # 10 blocks -> ids 0..9, two of them in the chunk
    assert not MU.release_last_kvcache_chunk(tw.engine)
    assert MU.compact_kvcache(tw.engine, 8) == -1      # low region is full: nothing may change
    tw.check()
    tw.free([0])
    assert MU.compact_kvcache(tw.engine, 8) == 2
    assert O.compact(tw.obm, tw.ok, tw.ov, 8, 4) == 2
    tw.check()
    assert MU.release_last_kvcache_chunk(tw.engine)
    O.release_last_chunk(tw.obm, 4)
    tw.ok.pop()
    tw.ov.pop()
    tw.check()


def test_compaction_without_a_host_round_trip_replayed_from_a_cuda_graph():
    """compact_kvcache_nosync keeps the pair count on the device, so the whole compaction (plan, block copy, table
    remap) can be captured once and replayed: first replay moves the two live blocks of the chunk, the second finds
    nothing to move, and a replay on a full low region is refused with nothing changed."""
    import torch
    from morphserve_b200.server import memory_utils as MU
    tw = Twin(2, 2, 128, 16, 8, max_seqs=16, mbps=8, seed=5)
    tw.expand(4)
    for s in range(5):
        tw.admit(s, 32)          # ids 0..9: the low region (8 blocks) is full, two blocks live in the chunk
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rec = MU.compact_kvcache_nosync(tw.engine, 8)          # warm-up outside the capture: refused
        side.synchronize()
        assert rec.tolist() == [0, 1, 2, 0]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            rec = MU.compact_kvcache_nosync(tw.engine, 8)
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    assert rec.tolist() == [0, 1, 2, 0]
    tw.check()                                                   # refused: bitmap, table and pools untouched
    tw.free([0])                                                 # frees ids 0 and 1
    g.replay()
    torch.cuda.synchronize()
    assert rec.tolist() == [2, 0, 2, 2]
    assert O.compact(tw.obm, tw.ok, tw.ov, 8, 4) == 2
    tw.check()
    g.replay()
    torch.cuda.synchronize()
    assert rec.tolist() == [0, 0, 0, 0]                          # nothing above the target any more
    tw.check()
    assert MU.release_last_kvcache_chunk(tw.engine)


@pytest.mark.parametrize("pinned", [False, True])
def test_swap_roundtrip_and_chunk_addressing(pinned):
    from morphserve_b200 import swiftllm_c
    L, Hkv, bs, D = 2, 2, 16, 128
    rs = np.random.RandomState(8)
    nb_org, chunk, n_chunks, ncpu = 12, 4, 2, 20
    elems = chunk * L * Hkv * bs * D
    P = 2 * elems + 1024                   # "layer parameter size" in elements
    slab = torch.zeros(n_chunks * P, dtype=torch.float16, device="cuda")
    k_new, v_new = [], []
    for j in range(n_chunks):              # chunk j sits j*P elements below chunk 0
        base = (n_chunks - 1 - j) * P
        k_new.append(slab[base:base + elems].view(chunk, L, Hkv, bs, D))
        v_new.append(slab[base + elems:base + 2 * elems].view(chunk, L, Hkv, bs, D))
    kp = [rs.standard_normal((nb_org, L, Hkv, bs, D)).astype(np.float16)] + \
         [rs.standard_normal((chunk, L, Hkv, bs, D)).astype(np.float16) for _ in range(n_chunks)]
    vp = [rs.standard_normal(p.shape).astype(np.float16) for p in kp]
    k_cache, v_cache = H.to_dev(kp[0]), H.to_dev(vp[0])
    for j in range(n_chunks):
        k_new[j].copy_(H.to_dev(kp[1 + j]))
        v_new[j].copy_(H.to_dev(vp[1 + j]))
    k_swap = torch.zeros((ncpu, L, Hkv, bs, D), dtype=torch.float16)
    v_swap = torch.zeros((ncpu, L, Hkv, bs, D), dtype=torch.float16)
    if pinned:      # pinned swap space: one zero-copy kernel instead of run-coalesced copies
        k_swap, v_swap = k_swap.pin_memory(), v_swap.pin_memory()
    oks, ovs = k_swap.numpy().copy(), v_swap.numpy().copy()

    # swap out: device ids (runs, a chunk boundary at 15|16, original/elastic boundary at 11|12)
    src = [3, 4, 5, 10, 11, 12, 13, 14, 15, 16, 19]
    dst = [0, 1, 2, 7, 8, 9, 10, 11, 12, 13, 5]
    swiftllm_c.swap_blocks_new_kv_combined(src, dst, False, nb_org, P, chunk, 2, k_cache, v_cache, k_swap, v_swap,
                                           k_new[0], v_new[0])
    torch.cuda.synchronize()
    O.swap_blocks(src, dst, False, kp, vp, oks, ovs, nb_org, chunk)
    assert k_swap.numpy().tobytes() == oks.tobytes() and v_swap.numpy().tobytes() == ovs.tobytes()

    # swap in to other device blocks, original pool only -> plain variant
    src2, dst2 = [0, 1, 2, 5], [6, 7, 8, 0]
    swiftllm_c.swap_blocks(src2, dst2, True, k_cache, v_cache, k_swap, v_swap)
    O.swap_blocks(src2, dst2, True, kp, vp, oks, ovs, nb_org, chunk)
    # swap in into elastic blocks: the device address comes from the TARGET id
    src3, dst3 = [7, 8, 9, 10], [18, 19, 12, 13]
    if pinned:      # ids may stay on the GPU
        src3, dst3 = torch.tensor(src3, device="cuda"), torch.tensor(dst3, device="cuda", dtype=torch.int32)
    swiftllm_c.swap_blocks_new_kv_combined(src3, dst3, True, nb_org, P, chunk, 2, k_cache, v_cache, k_swap, v_swap,
                                           k_new[0], v_new[0])
    O.swap_blocks([7, 8, 9, 10], [18, 19, 12, 13], True, kp, vp, oks, ovs, nb_org, chunk)
    torch.cuda.synchronize()
    got = [k_cache] + k_new + [v_cache] + v_new
    for a, b in zip(got, kp + vp):
        assert a.cpu().numpy().tobytes() == b.tobytes()
    with pytest.raises(RuntimeError):
        swiftllm_c.swap_blocks([0], [ncpu], False, k_cache, v_cache, k_swap, v_swap)   # host id out of range


def test_acquire_new_kvcache_carves_the_slab_like_the_reference():
    from morphserve_b200 import swiftllm_c
    L, Hkv, bs, D = 2, 2, 16, 128
    org_size, quant_size = 1 << 20, 300_001
    slab = torch.full((org_size,), 7, dtype=torch.uint8, device="cuda")
    swiftllm_c.register_kv_cache_info(L, Hkv, bs, D)
    with pytest.raises(RuntimeError):
        swiftllm_c.acquire_new_kvcache(5)
    swiftllm_c.register_layer_memory_org_gpu(5, slab.data_ptr(), org_size)
    swiftllm_c.register_layer_memory_quant(5, 0, quant_size)
    k, v = swiftllm_c.acquire_new_kvcache(5)
    ka, va, n = O.chunk_layout(slab.data_ptr(), org_size, quant_size, L, Hkv, bs, D)
    assert (k.data_ptr(), v.data_ptr(), k.shape[0]) == (ka, va, n)
    assert tuple(k.shape) == (n, L, Hkv, bs, D) and k.dtype == torch.float16
    host = slab.cpu().numpy()
    off = ka - slab.data_ptr()
    assert (host[:off] == 7).all()                                   # the quantised layer's bytes are untouched
    assert (host[off:off + 2 * k.numel() * 2] == 0).all()            # chunk is zero-filled
    swiftllm_c.register_layer_memory_quant(6, 0, org_size - 100)
    swiftllm_c.register_layer_memory_org_gpu(6, slab.data_ptr(), org_size)
    with pytest.raises(RuntimeError):
        swiftllm_c.acquire_new_kvcache(6)


def test_layer_slab_replace_and_restore_round_trip():
    """org -> quant -> (elastic chunk in the freed tail) -> org, as server/memory_utils.py:93-367 and :617-662
    drive it: the slab holds the host images byte for byte, returned tensors are views into the slab with the
    registered shapes and dtypes, bytes behind the quantised image stay as they were until the chunk is zeroed."""
    from morphserve_b200 import swiftllm_c as c
    layer = 700
    rs = np.random.RandomState(12)
    # "fp16 layer": three tensors back to back; "quantised layer": int32 / fp16 / int32 / bf16 tensors, smaller
    org_np = {"a.weight": rs.standard_normal((256, 512)).astype(np.float16),
              "b.weight": rs.standard_normal((512, 300)).astype(np.float16),
              "norm.weight": rs.standard_normal((512,)).astype(np.float16)}
    q_np = {"a.qweight": rs.randint(-2 ** 31, 2 ** 31 - 1, size=(256, 64)).astype(np.int32),
            "a.scales": rs.standard_normal((4, 512)).astype(np.float16),
            "a.qzeros": rs.randint(0, 2 ** 31 - 1, size=(4, 64)).astype(np.int32),
            "norm.weight": rs.standard_normal((512,)).astype(np.float32),
            "b.lowrank": rs.randint(-2 ** 15, 2 ** 15 - 1, size=(8, 300)).astype(np.int16)}    # stands for bf16 bits

    def pack(d, torch_dtypes):
        blob, maps, off = [], [], 0
        for (name, a), dt in zip(d.items(), torch_dtypes):
            maps.append({name: {"offset": off, "shape": list(a.shape), "dtype": dt, "size": a.nbytes, "is_param": False}})
            blob.append(a.tobytes())
            off += a.nbytes
        return np.frombuffer(b"".join(blob), dtype=np.uint8).copy(), maps

    org_blob, org_map = pack(org_np, [torch.float16] * 3)
    q_blob, q_map = pack(q_np, [torch.int32, torch.float16, torch.int32, torch.float32, torch.bfloat16])
    slab = torch.from_numpy(org_blob).cuda()                       # the layer as it sits on the GPU
    org_host = torch.from_numpy(org_blob).pin_memory()
    q_host = torch.from_numpy(q_blob).pin_memory()
    c.register_layer_memory_org_gpu(layer, slab.data_ptr(), slab.numel())
    c.register_layer_memory_org_cpu(layer, org_host.data_ptr(), org_host.numel())
    c.register_layer_memory_tensor_map_org(layer, org_map)
    c.register_layer_memory_quant(layer, q_host.data_ptr(), q_host.numel())
    c.register_layer_memory_tensor_map_quant(layer, q_map)

    got = c.replace_layer_org2quant(layer)
    torch.cuda.synchronize()
    after = slab.cpu().numpy()
    assert after[: q_blob.size].tobytes() == q_blob.tobytes()
    assert after[q_blob.size:].tobytes() == org_blob[q_blob.size:].tobytes()      # tail untouched
    assert len(got) == 5 and got[4].dtype == torch.bfloat16 and got[0].dtype == torch.int32
    for t, (name, a) in zip(got, q_np.items()):
        assert tuple(t.shape) == a.shape and t.is_cuda
        bits = t.view(torch.int16) if t.dtype == torch.bfloat16 else t
        assert bits.cpu().numpy().tobytes() == a.tobytes(), name
        assert slab.data_ptr() <= t.data_ptr() < slab.data_ptr() + slab.numel()      # a view, not a copy
    assert c.verify_tensor_continuity(got)
    assert c.get_freed_memory_size(layer, q_blob.size) == org_blob.size - q_blob.size

    # the freed tail becomes an elastic KV chunk (csrc/src/memory_manager.cpp:69-176)
    c.register_kv_cache_info(2, 2, 16, 128)
    k, v = c.acquire_new_kvcache(layer)
    assert k.shape[0] >= 1 and k.data_ptr() >= slab.data_ptr() + q_blob.size
    torch.cuda.synchronize()
    assert slab.cpu().numpy()[: q_blob.size].tobytes() == q_blob.tobytes()          # zeroing the chunk spared the layer

    back = c.replace_layer_quant2org(layer)
    torch.cuda.synchronize()
    assert slab.cpu().numpy().tobytes() == org_blob.tobytes()
    for t, (name, a) in zip(back, org_np.items()):
        assert t.dtype == torch.float16 and t.cpu().numpy().tobytes() == a.tobytes(), name


@pytest.mark.parametrize("sync_free", [False, True])
@pytest.mark.parametrize("with_chunks", [False, True])
def test_model_level_swap_out_and_in_against_oracle(with_chunks, sync_free):
    """KVCacheModelState (the KV half of the reference's LlamaModel: worker/model.py:176-227, :468-550): sequences
    are swapped out, others admitted, the first swapped back in - block managers, pools and swap space in lockstep
    with the oracle's managers and its swap rule.  ``sync_free``: the same moves through ``swap_seqs_nosync`` (ids
    and counts stay on the GPU)."""
    from types import SimpleNamespace
    from morphserve_b200 import KVCacheModelState
    rs = np.random.RandomState(5 + with_chunks)
    L, Hkv, bs, D = 2, 2, 16, 128
    nb, n_cpu, max_seqs, cols = 48, 40, 12, 12
    chunk = 8 if with_chunks else 0
    mc = SimpleNamespace(num_layers=L, num_q_heads=4, num_kv_heads=Hkv, head_dim=D)
    ec = SimpleNamespace(block_size=bs, num_cpu_blocks=n_cpu, max_seqs_in_block_table=max_seqs, max_blocks_per_seq=cols)
    m = KVCacheModelState(mc, ec)
    m.init_kvcache_and_swap(nb)
    assert m.k_swap.is_pinned() and float(m.k_cache.abs().sum()) == 0.0
    g_or, c_or = O.BlockManagerOracle(nb, max_seqs, cols, bs), O.BlockManagerOracle(n_cpu, max_seqs, cols, bs)
    shapes = [(nb, L, Hkv, bs, D)]
    if with_chunks:         # two elastic chunks, attached the way server/memory_utils.py:389-420 does it
        for _ in range(2):
            m.k_cache_new.append(torch.zeros((chunk, L, Hkv, bs, D), dtype=torch.float16, device="cuda"))
            m.v_cache_new.append(torch.zeros((chunk, L, Hkv, bs, D), dtype=torch.float16, device="cuda"))
            m.gpu_block_manager.num_blocks += chunk
            m.gpu_block_manager.num_free_blocks += chunk
            m.gpu_block_manager.is_block_free = torch.cat(
                [m.gpu_block_manager.is_block_free, torch.ones(chunk, dtype=torch.bool, device="cuda")])
            O.expand(g_or, chunk)
            shapes.append((chunk, L, Hkv, bs, D))
        m.kv_cache_new_block_size = chunk
    k_or = [rs.standard_normal(sh).astype(np.float16) for sh in shapes]
    v_or = [rs.standard_normal(sh).astype(np.float16) for sh in shapes]
    with torch.inference_mode():    # the pools are inference tensors, like the reference's (worker/model.py:176)
        for t, a in zip([m.k_cache] + m.k_cache_new + [m.v_cache] + m.v_cache_new, k_or + v_or):
            t.copy_(H.to_dev(a))
    ks_or = np.zeros((n_cpu, L, Hkv, bs, D), dtype=np.float16)
    vs_or = np.zeros_like(ks_or)

    def both_allocate(ids, lens):
        ids, lens = np.asarray(ids, dtype=np.int32), np.asarray(lens, dtype=np.int32)
        m.gpu_block_manager.allocate_blocks_for_seqs(H.to_dev(ids), H.to_dev(lens))
        g_or.allocate_blocks_for_seqs(ids, lens)

    def oracle_swap(ids, is_in):
        src, dst = (c_or, g_or) if is_in else (g_or, c_or)
        ids = np.asarray(ids, dtype=np.int32)
        lens = src.get_num_allocated_blocks(ids) * bs
        s_ids = src.gather_allocated_blocks_and_free(ids)
        d_ids = dst.allocate_blocks_for_seqs(ids, lens)
        O.swap_blocks(s_ids, d_ids, is_in, k_or, v_or, ks_or, vs_or, nb, chunk)

    def check_all():
        torch.cuda.synchronize()
        for bm, ob in ((m.gpu_block_manager, g_or), (m.cpu_block_manager, c_or)):
            live = ob.num_seq_allocated_blocks > 0
            np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), ob.num_seq_allocated_blocks)
            np.testing.assert_array_equal(bm.block_table.cpu().numpy()[live], ob.block_table[live])
            np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), ob.is_block_free)
            assert int(bm.num_free_blocks) == int(ob.num_free_blocks)
        for t, a in zip([m.k_cache] + m.k_cache_new + [m.v_cache] + m.v_cache_new, k_or + v_or):
            assert t.cpu().numpy().tobytes() == a.tobytes()
        assert m.k_swap.numpy().tobytes() == ks_or.tobytes() and m.v_swap.numpy().tobytes() == vs_or.tobytes()

    def swap_out(ids):
        if sync_free:
            m.swap_seqs_nosync(H.to_dev(np.asarray(ids, dtype=np.int32)), False)
        else:
            m.swap_out_seqs(ids)

    def swap_in(ids):
        if sync_free:
            m.swap_seqs_nosync(H.to_dev(np.asarray(ids, dtype=np.int32)), True)
        else:
            m.swap_in_seqs(ids)

    if with_chunks:     # three resident sequences fill most of the original pool: the rest spills into the chunks
        both_allocate([9, 10, 11], [192, 192, 192])
    both_allocate([0, 1, 2, 3, 4, 5], [100, 30, 64, 60, 17, 90] if with_chunks else [100, 30, 64, 120, 17, 90])
    if with_chunks:
        assert int(m.gpu_block_manager.block_table[:6].max()) >= nb, "the case must reach the elastic chunks"
    check_all()
    swap_out([1, 3, 4])
    oracle_swap([1, 3, 4], False)
    check_all()
    both_allocate([6, 7], [70, 33])                       # takes some of the freed blocks
    swap_out([0])
    oracle_swap([0], False)
    swap_in([3, 1])
    oracle_swap([3, 1], True)
    check_all()
    m.free_seqs_resources([2, 4])
    g_or.free_blocks_for_seqs(np.array([2, 4], dtype=np.int32))
    c_or.free_blocks_for_seqs(np.array([2, 4], dtype=np.int32))
    swap_in([0])
    oracle_swap([0], True)
    check_all()
    assert (int(m.block_swap_device) if sync_free else m.block_swap) == (28 if with_chunks else 36)
    if sync_free:
        # a swap-in the GPU pool cannot hold: nothing is copied, the sequence's swap blocks are released like the
        # reference releases them before its allocation fails, and the failure is raised at the next look
        gbm = m.gpu_block_manager

        def fill_gpu_pool(rows):
            for sid in rows:                          # a row holds 12 blocks: spread what is free over spare rows
                take = min(cols - int(gbm.num_seq_allocated_blocks[sid]), int(gbm.num_free_blocks))
                if take > 0:
                    have = int(gbm.num_seq_allocated_blocks[sid])
                    gbm.allocate_blocks_for_seqs(H.to_dev(np.array([sid], dtype=np.int32)),
                                                 H.to_dev(np.array([16 * (have + take)], dtype=np.int32)))
            assert int(gbm.num_free_blocks) == 0

        fill_gpu_pool([8, 2, 4])
        swap_out([1])
        before = [t.clone() for t in [m.k_cache] + m.k_cache_new + [m.v_cache] + m.v_cache_new]
        fill_gpu_pool([8, 2, 4, 7])                   # takes the two blocks the swap-out freed
        swap_in([1])
        torch.cuda.synchronize()
        for t, b in zip([m.k_cache] + m.k_cache_new + [m.v_cache] + m.v_cache_new, before):
            assert t.view(torch.int16).equal(b.view(torch.int16))
        with pytest.raises(RuntimeError, match="No enough free blocks"):
            int(m.gpu_block_manager.num_free_blocks)


@pytest.mark.parametrize("sync_free", [False, True])
def test_prepare_step_builds_the_reference_metadata(sync_free):
    """KVCacheModelState.prepare_step against the restated list-to-tensor logic of the reference's forward()
    (worker/model.py:318-436): every field of the infer state, the cos/sin rows, and the block allocation, over a
    prefill-only step, a mixed step and decode-only steps."""
    from types import SimpleNamespace
    from morphserve_b200 import KVCacheModelState
    rs = np.random.RandomState(9)
    mc = SimpleNamespace(num_layers=2, num_q_heads=8, num_kv_heads=2, head_dim=128, rope_theta=10000.0,
                         rope_scaling=1, max_position_embeddings=2048)
    ec = SimpleNamespace(block_size=16, num_cpu_blocks=8, max_seqs_in_block_table=16, max_blocks_per_seq=40)
    m = KVCacheModelState(mc, ec)
    m.init_kvcache_and_swap(400)
    ob = O.BlockManagerOracle(400, 16, 40, 16)
    cos_tab, sin_tab = cases.rope_tables(np.arange(2048 + 128), 128)
    lens = {}

    def step(prompts, dec_ids):
        """prompts: {seq id: prompt length}; dec_ids: running sequences that generate one more token."""
        for s, n in prompts.items():
            lens[s] = n
        for s in dec_ids:
            lens[s] += 1
        input_ids = [list(rs.randint(0, 1000, size=n)) for n in prompts.values()] + [[7] for _ in dec_ids]
        seq_ids = list(prompts) + list(dec_ids)
        dec_lens = [lens[s] for s in dec_ids]
        st = m.prepare_step(input_ids, seq_ids, dec_lens, sync_free=sync_free)
        f = O.infer_state_fields(list(prompts.values()), dec_lens, mc.num_kv_heads, mc.head_dim)
        ob.allocate_blocks_for_seqs(np.asarray(seq_ids, dtype=np.int32), f["seq_lengths"])
        torch.cuda.synchronize()
        for name in ("batch_size", "num_tokens", "num_prefill_seqs", "num_prefill_tokens", "max_prefill_len",
                     "num_decoding_seqs", "max_decoding_len", "seq_block_size", "num_seq_blocks", "softmax_scale"):
            assert getattr(st, name) == f[name], name
        for name in ("prefill_seq_start_locs", "prefill_seq_start_locs_with_end", "prefill_seq_lens", "decoding_seq_lens"):
            got = getattr(st, name)
            assert got.dtype == torch.int32 and got.is_cuda
            np.testing.assert_array_equal(got.cpu().numpy(), f[name], err_msg=name)
        np.testing.assert_array_equal(st.seq_ids.cpu().numpy(), np.asarray(seq_ids, dtype=np.int32))
        # the rows are those of the model's tables at the tokens' positions; the tables are the reference's formula
        # (fp32 angles -> fp16), equal to a numpy evaluation up to the last bit of the angle
        for got, table, want in ((st.position_cos, m._cos_cached, cos_tab), (st.position_sin, m._sin_cached, sin_tab)):
            assert got.cpu().numpy().tobytes() == table.cpu().numpy()[f["position_indices"]].tobytes()
            np.testing.assert_allclose(table.cpu().numpy().astype(np.float64), want.astype(np.float64), atol=2e-3)
        assert st.num_blocks_org == 400 and st.ignore_kvcache is False
        bm = m.gpu_block_manager
        assert int(bm.num_free_blocks) == int(ob.num_free_blocks)
        np.testing.assert_array_equal(bm.block_table.cpu().numpy(), ob.block_table)
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), ob.num_seq_allocated_blocks)
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), ob.is_block_free)
        return st

    step({3: 70, 5: 16, 0: 1}, [])                       # prefill only
    step({9: 33}, [3, 5, 0])                             # mixed
    for _ in range(3):
        step({}, [3, 5, 0, 9])                           # decode only
    st = step({11: 200, 2: 15}, [9, 3])
    # the state drives the kernels: rotary -> store -> attention of the mixed step run without error
    import morphserve_b200 as mk
    T = st.num_tokens
    q = torch.randn((T, 8, 128), dtype=torch.float16, device="cuda")
    k = torch.randn((T, 2, 128), dtype=torch.float16, device="cuda")
    v = torch.randn((T, 2, 128), dtype=torch.float16, device="cuda")
    mk.rotary_embedding_inplace(q, k, st)
    mk.store_kvcache(k, v, m.k_cache, m.v_cache, [], [], m.gpu_block_manager.block_table, mc, ec, st, 1)
    o = torch.zeros((st.num_decoding_seqs, 8 * 128), dtype=torch.float16, device="cuda")
    mk.paged_attention(q[st.num_prefill_tokens:], m.k_cache, m.v_cache, [], [], m.gpu_block_manager.block_table, mc, ec,
                       st, 1, o)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(o).all())
