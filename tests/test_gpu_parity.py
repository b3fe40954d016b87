"""GPU parity: the CUDA path (through the public API -> C ABI) against the
reference's outputs (golden fixtures) and against the CPU oracle on seeded
inputs.  Bit-exact for byte/integer work; rtol 2e-3 / atol 1e-2 for attention
(fp16 data, fp32 accumulation)."""
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from tests import helpers as H
from tests.golden import cases

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
RTOL, ATOL = 2e-3, 1e-2
DEFAULT_LOADER = 1 if os.environ.get("MKV_ATTN_LOADER") == "tma" else 0      # the library's default is cp.async


@pytest.fixture(params=["separate", "fused_append"], autouse=True)
def append_mode(request):
    """Every test in this file runs twice: with the decode append as its own kernel, and with
    the append fused into the attention kernel."""
    import morphserve_b200
    morphserve_b200.set_fused_decode_append(request.param == "fused_append")
    yield request.param
    morphserve_b200.set_fused_decode_append(False)


@pytest.fixture(params=["tma", "cpasync"], autouse=True)
def tile_loader(request):
    """... and with both tile loaders of the decode kernel (TMA boxes / 16-byte cp.async)."""
    from morphserve_b200._lib import lib, check
    check(lib.mkv_attn_configure(-1, -1, -1.0, -1.0, 1 if request.param == "tma" else 0), "mkv_attn_configure")
    yield request.param
    check(lib.mkv_attn_configure(-1, -1, -1.0, -1.0, DEFAULT_LOADER), "mkv_attn_configure")


def _close(a, b):
    np.testing.assert_allclose(np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_decode_step_matches_reference_fixture(name):
    c = cases.build_decode_case(**cases.DECODE_CASES[name])
    gold = np.load(os.path.join(G, f"decode_{name}.npz"))
    o, kp, vp = H.run_decode_step(H.device_case(c))
    assert cases.sha256_of(*kp, *vp) == str(gold["pools_after_sha256"]), "KV append is not bit-exact"
    _close(o, gold["o"])
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], c["layer"],
                                 c["scale"], c["num_blocks_org"], c["chunk_blocks"])
    _close(o, ex)


@pytest.mark.parametrize("name", list(cases.PREFILL_CASES))
def test_prefill_scatter_matches_reference_fixture(name, append_mode):
    from morphserve_b200 import store_kvcache
    from morphserve_b200.worker.infer_state import LlamaInferState
    c = cases.build_prefill_case(**cases.PREFILL_CASES[name])
    gold = np.load(os.path.join(G, f"prefill_{name}.npz"))
    kp = [H.to_dev(p) for p in c["k_pools"]]
    vp = [H.to_dev(p) for p in c["v_pools"]]
    bt = H.to_dev(c["block_table"])
    npre = len(c["prefill_lens"])
    z = torch.zeros(0, dtype=torch.int32, device="cuda")
    st = LlamaInferState(
        batch_size=len(c["seq_ids"]), num_tokens=c["k"].shape[0], seq_ids=H.to_dev(c["seq_ids"]), softmax_scale=1.0,
        num_prefill_seqs=npre, num_prefill_tokens=c["num_prefill_tokens"],
        prefill_seq_start_locs=H.to_dev(c["prefill_start_locs"]), prefill_seq_start_locs_with_end=z,
        prefill_seq_lens=H.to_dev(c["prefill_lens"]), max_prefill_len=int(c["prefill_lens"].max()),
        num_decoding_seqs=len(c["decode_lens"]), decoding_seq_lens=H.to_dev(c["decode_lens"]),
        max_decoding_len=int(c["decode_lens"].max()), seq_block_size=512, num_seq_blocks=1,
        num_blocks_org=c["num_blocks_org"], kv_cache_new_block_size=c["chunk_blocks"], org_layer_param_size=0,
        position_cos=z, position_sin=z, ignore_kvcache=False)
    mc, ec = H.cfgs(c, bt.shape[1])
    k_dev, v_dev = H.to_dev(c["k"]), H.to_dev(c["v"])
    store_kvcache(k_dev, v_dev, kp[0], vp[0], kp[1:], vp[1:], bt, mc, ec, st, c["layer"])
    if append_mode == "fused_append":
        # the decode rows of the mixed batch are appended by the attention call of the same layer
        from morphserve_b200 import paged_attention
        nd = len(c["decode_lens"])
        mc.num_q_heads = c["Hkv"] * 2
        q = torch.randn((nd, mc.num_q_heads, c["D"]), dtype=torch.float16, device="cuda")
        o = torch.empty((nd, mc.num_q_heads * c["D"]), dtype=torch.float16, device="cuda")
        paged_attention(q, kp[0], vp[0], kp[1:], vp[1:], bt, mc, ec, st, c["layer"], o)
    torch.cuda.synchronize()
    after = [p.cpu().numpy() for p in kp] + [p.cpu().numpy() for p in vp]
    assert cases.sha256_of(*after) == str(gold["pools_after_sha256"])


def test_block_manager_trace_matches_reference_fixture():
    from morphserve_b200 import BlockManager
    tr = cases.block_manager_trace()
    gold = np.load(os.path.join(G, "block_manager_trace.npz"))
    bm = BlockManager("GPU", tr["num_blocks"], tr["max_seqs"], tr["max_blocks_per_seq"], tr["block_size"])
    for i, (op, ids, lens) in enumerate(tr["ops"]):
        if op == "alloc":
            r = bm.allocate_blocks_for_seqs(H.to_dev(ids), H.to_dev(lens))
            assert r.dtype == torch.int64
        elif op == "free":
            bm.free_blocks_for_seqs(H.to_dev(ids))
            r = torch.empty(0)
        else:
            r = bm.gather_allocated_blocks_and_free(H.to_dev(ids))
            assert r.dtype == torch.int32
        np.testing.assert_array_equal(r.cpu().numpy().astype(np.int64), gold[f"ret_{i}"])
        np.testing.assert_array_equal(bm.block_table.cpu().numpy(), gold[f"table_{i}"])
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), gold[f"count_{i}"])
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), gold[f"free_{i}"])
        assert int(bm.num_free_blocks) == int(gold[f"nfree_{i}"])
        assert bm.num_free_blocks.item() == int(gold[f"nfree_{i}"])
    with pytest.raises(RuntimeError):
        bm._allocate_blocks(int(bm.num_free_blocks) + 1)
    # _allocate_blocks / _free_blocks (worker/block_manager.py:64-85): first-fit ascending, then back
    before = bm.is_block_free.clone()
    nfree = int(bm.num_free_blocks)
    got = bm._allocate_blocks(5)
    expect = torch.nonzero(before)[:5].view(-1)
    assert torch.equal(got, expect) and not bm.is_block_free[got].any() and int(bm.num_free_blocks) == nfree - 5
    bm._free_blocks(got)
    assert torch.equal(bm.is_block_free, before) and int(bm.num_free_blocks) == nfree
    ids = H.to_dev(np.array([0], dtype=np.int32))
    bm.allocate_blocks_for_seqs(ids, H.to_dev(np.array([40], dtype=np.int32)))
    with pytest.raises(AssertionError):
        bm.allocate_blocks_for_seqs(ids, H.to_dev(np.array([1], dtype=np.int32)))


# (B, Hq, Hkv, max_len, L, layer): every group size of the fast path, odd batch sizes,
# sequences long enough to be cut into several chunks (merge path) and lengths at block edges
SWEEP = [
    (1, 8, 8, 1, 1, 0), (1, 4, 1, 4096, 1, 0), (3, 16, 1, 700, 2, 1), (5, 12, 4, 300, 2, 0),
    (17, 32, 8, 1536, 2, 1), (64, 32, 32, 768, 1, 0), (9, 2, 1, 2500, 1, 0), (33, 64, 8, 1536, 1, 0),
    (2, 32, 8, 20000, 1, 0),        # long context, tiny batch: every sequence is cut into dozens of chunks
]


@pytest.mark.parametrize("B,Hq,Hkv,max_len,L,layer", SWEEP)
def test_decode_attention_sweep_against_oracle(B, Hq, Hkv, max_len, L, layer):
    rs = np.random.RandomState(B * 1000 + Hq)
    lens = rs.randint(1, max_len + 1, size=B)
    lens[0] = max_len
    if B > 2:
        lens[1] = max(1, (max_len // 16) * 16)      # exactly full last block
        lens[2] = 1
    nb = int(((lens + 15) // 16).sum()) + 5
    c = cases.build_decode_case(seed=B * 77 + Hq, B=B, Hq=Hq, Hkv=Hkv, D=128, bs=16, L=L, layer=layer,
                                num_blocks_org=nb, dtype=np.float16, lens=lens)
    o, kp, vp = H.run_decode_step(H.device_case(c))
    # append: bit-exact against the oracle
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_decode(c["k_new"], c["v_new"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"],
                           c["layer"], c["num_blocks_org"], c["chunk_blocks"])
    for a, b in zip(kp + vp, kpo + vpo):
        assert a.tobytes() == b.tobytes()
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], c["layer"],
                                 c["scale"], c["num_blocks_org"], c["chunk_blocks"])
    _close(o, ex)
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0


@pytest.mark.parametrize("deal", [(0, 1), (1, 0), (1, 1), (2, 3)])
@pytest.mark.parametrize("balance", [0.0, 1.5, 1000.0])
@pytest.mark.parametrize("shape", ["spread", "one_long"])
def test_split_rule_extremes(balance, shape, deal):
    """The plan cuts a sequence only when it is long against the mean load of a worker warp.  Finest cut (0),
    the default, and "never cut" (1000) must all give the oracle's result, on a batch with a spread of lengths
    and on one long sequence among short ones - with chunks drawn from the shared counter (deal 0), with equal
    ranges per worker when something has to be cut (1) or always (2), and with several unit costs."""
    from morphserve_b200._lib import lib, check
    rs = np.random.RandomState(314)
    if shape == "spread":
        B, Hq, Hkv = 48, 32, 8
        lens = rs.randint(1, 1553, size=B)
        lens[0] = 1552            # 97 blocks: one more than a power-of-two-times-three chunk
    else:
        B, Hq, Hkv = 24, 16, 4
        lens = rs.randint(1, 200, size=B)
        lens[5] = 9000
    nb = int(((lens + 15) // 16).sum()) + 5
    c = cases.build_decode_case(seed=2718, B=B, Hq=Hq, Hkv=Hkv, D=128, bs=16, L=1, layer=0, num_blocks_org=nb,
                                dtype=np.float16, lens=lens)
    check(lib.mkv_attn_configure(-1, -1, -1.0, balance, -1), "mkv_attn_configure")
    check(lib.mkv_attn_set_static_deal(deal[0], deal[1], 1), "mkv_attn_set_static_deal")
    try:
        o, kp, vp = H.run_decode_step(H.device_case(c))
    finally:
        check(lib.mkv_attn_configure(-1, -1, -1.0, 1.5, -1), "mkv_attn_configure")
        check(lib.mkv_attn_set_static_deal(1, 3, 1), "mkv_attn_set_static_deal")
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], 0, c["scale"],
                                 c["num_blocks_org"], 0)
    _close(o, ex)
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0


@pytest.mark.parametrize("deal", [1, 2])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (16, 16)])
def test_many_short_sequences_per_worker(Hq, Hkv, deal):
    """More (sequence, kv head) units than worker warps, nearly all of one or two blocks, a few long ones in
    between: every warp runs several short units back to back, so the hand-over between units (claim of the next
    unit, prefetch of its first tiles into freed stages) is exercised where it has the least slack - with units
    drawn from the shared counter (`deal` 1: nothing needs cutting here) and with equal ranges per worker (2), where
    the records come out of the register window and the next unit is claimed at once."""
    from morphserve_b200._lib import lib, check
    rs = np.random.RandomState(Hq)
    B = 1400
    lens = rs.randint(1, 41, size=B)
    lens[rs.permutation(B)[:40]] = rs.randint(41, 400, size=40)
    nb = int(((lens + 15) // 16).sum()) + 7
    c = cases.build_decode_case(seed=4242 + Hkv, B=B, Hq=Hq, Hkv=Hkv, D=128, bs=16, L=1, layer=0, num_blocks_org=nb,
                                dtype=np.float16, lens=lens)
    check(lib.mkv_attn_set_static_deal(deal, -1, 1), "mkv_attn_set_static_deal")
    try:
        o, kp, vp = H.run_decode_step(H.device_case(c))
    finally:
        check(lib.mkv_attn_set_static_deal(1, -1, 1), "mkv_attn_set_static_deal")
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], 0, c["scale"],
                                 c["num_blocks_org"], 0)
    _close(o, ex)
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0


def _random_batch(rs):
    """A batch shape drawn to stress the scheduler: batch size from a handful to thousands, group size 1-16,
    lengths from one of several mixtures (all short, uniform, a few giants among short ones, all equal)."""
    Hkv = int(rs.choice([1, 2, 4, 8, 16]))
    G = int(rs.choice([1, 2, 4, 8, 16]))
    kind = int(rs.randint(0, 4))
    B = int(rs.choice([3, 40, 300, 1300, 2600])) if kind != 2 else int(rs.choice([40, 300, 1300]))
    if kind == 0:
        lens = rs.randint(1, 49, size=B)
    elif kind == 1:
        lens = rs.randint(1, 700, size=B) if B <= 300 else rs.randint(1, 120, size=B)
    elif kind == 2:
        lens = rs.randint(1, 60, size=B)
        lens[rs.permutation(B)[: max(1, B // 100)]] = rs.randint(1500, 6000, size=max(1, B // 100))
    else:
        lens = np.full(B, int(rs.choice([16, 17, 64, 130])))
    return B, Hkv * G, Hkv, lens


@pytest.mark.parametrize("deal", [0, 1, 2])
@pytest.mark.parametrize("seed", range(8))
def test_random_batches_fast_path_against_plain_kernel(seed, deal):
    """Seeded random batches, all sequences compared on the GPU: the tensor-core kernel (plan, either deal of the
    tiles - `deal` 2 forces equal ranges per worker on every batch -, split-KV merge in one and two levels, fused
    append when the fixture says so) against the library's plain kernel, which shares none of that machinery and is
    held to the oracle by the tests above."""
    from morphserve_b200._lib import lib, check
    check(lib.mkv_attn_set_static_deal(deal, seed % 4, 1 + seed % 2 * 7), "mkv_attn_set_static_deal")
    rs = np.random.RandomState(1000 + seed)
    B, Hq, Hkv, lens = _random_batch(rs)
    nb = int(((lens + 15) // 16).sum()) + 3
    L = 2
    g = torch.Generator(device="cuda").manual_seed(seed)
    # odd seeds: the pool is an original part plus two elastic chunks (three segments)
    nb_org, chunk = (nb, 0) if seed % 2 == 0 else (nb // 3, (nb - nb // 3 + 1) // 2)
    sizes = [nb_org] + ([chunk, chunk] if chunk else [])
    nb = sum(sizes)
    kseg = [torch.randn((n, L, Hkv, 16, 128), generator=g, dtype=torch.float16, device="cuda") for n in sizes]
    vseg = [torch.randn((n, L, Hkv, 16, 128), generator=g, dtype=torch.float16, device="cuda") for n in sizes]
    q = torch.randn((B, Hq, 128), generator=g, dtype=torch.float16, device="cuda")
    kn = torch.randn((B, Hkv, 128), generator=g, dtype=torch.float16, device="cuda")
    vn = torch.randn((B, Hkv, 128), generator=g, dtype=torch.float16, device="cuda")
    need = (lens + 15) // 16
    perm = rs.permutation(nb)
    table = np.full((B, int(need.max()) + 1), -1, dtype=np.int32)
    pos = 0
    for b in range(B):
        table[b, : need[b]] = perm[pos:pos + need[b]]
        pos += need[b]
    c = dict(L=L, Hq=Hq, Hkv=Hkv, D=128, bs=16, scale=128 ** -0.5, num_blocks_org=nb_org, chunk_blocks=chunk)
    bt, ids, lens_t = H.to_dev(table), torch.arange(B, dtype=torch.int32, device="cuda"), H.to_dev(lens.astype(np.int32))
    mc, ec = H.cfgs(c, bt.shape[1])
    from morphserve_b200 import paged_attention, store_kvcache
    outs = []
    for force_plain in (False, True):
        k2, v2 = [t.clone() for t in kseg], [t.clone() for t in vseg]
        if force_plain:
            check(lib.mkv_attn_configure(-1, -1, -1.0, -1.0, 2), "mkv_attn_configure")
        try:
            st = H.decode_state(c, ids, lens_t)
            o = torch.zeros((B, Hq * 128), dtype=torch.float16, device="cuda")
            store_kvcache(kn, vn, k2[0], v2[0], k2[1:], v2[1:], bt, mc, ec, st, 1)
            paged_attention(q, k2[0], v2[0], k2[1:], v2[1:], bt, mc, ec, st, 1, o)
            torch.cuda.synchronize()
        finally:
            if force_plain:
                check(lib.mkv_attn_configure(-1, -1, -1.0, -1.0, DEFAULT_LOADER), "mkv_attn_configure")
        outs.append((o, k2, v2))
    check(lib.mkv_attn_set_static_deal(1, 3, 1), "mkv_attn_set_static_deal")
    (o_fast, k_fast, v_fast), (o_plain, k_plain, v_plain) = outs
    for a, b in zip(k_fast + v_fast, k_plain + v_plain):
        assert torch.equal(a, b), "appended pools differ"
    diff = (o_fast.float() - o_plain.float()).abs()
    bad = diff > ATOL + RTOL * o_plain.float().abs()
    assert not bool(bad.any()), f"B={B} Hq={Hq} Hkv={Hkv}: {int(bad.any(dim=1).sum())} sequences differ, max {float(diff.max())}"
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0


def test_slots_behind_the_sequence_end_may_hold_nan():
    """A pool that was never zeroed (or recycled blocks): every slot that no sequence owns holds NaN.  The reference
    zero-fills its pools to survive this (worker/model.py:187-188); here the result must not depend on those slots."""
    rs = np.random.RandomState(12)
    lens = np.array([1, 5, 16, 17, 31, 100, 333, 1000, 47])
    nb = int(((lens + 15) // 16).sum()) + 9
    c = cases.build_decode_case(seed=31, B=len(lens), Hq=8, Hkv=2, D=128, bs=16, L=2, layer=1, num_blocks_org=nb,
                                dtype=np.float16, lens=lens)
    owned = np.zeros((nb, 16), dtype=bool)
    for b, n in enumerate(lens):
        row = c["block_table"][c["seq_ids"][b]]
        for t in range(n):
            owned[row[t // 16], t % 16] = True
    for pool in (c["k_pools"][0], c["v_pools"][0]):
        pool[~owned[:, None, None, :].repeat(2, 1).repeat(2, 2)] = np.nan      # [nb, L, Hkv, 16, D]
    o, kp, vp = H.run_decode_step(H.device_case(c))
    assert np.isfinite(o).all()
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], 1, c["scale"],
                                 c["num_blocks_org"], 0)
    _close(o, ex)


def test_every_length_across_block_and_chunk_edges():
    """lens 1..160 in one batch: every len % 16, single- and multi-block sequences."""
    lens = np.arange(1, 161)
    B = len(lens)
    nb = int(((lens + 15) // 16).sum()) + 3
    c = cases.build_decode_case(seed=99, B=B, Hq=8, Hkv=2, D=128, bs=16, L=1, layer=0, num_blocks_org=nb,
                                dtype=np.float16, lens=lens)
    o, kp, vp = H.run_decode_step(H.device_case(c))
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], 0, c["scale"],
                                 c["num_blocks_org"], 0)
    _close(o, ex)


def test_repeated_layers_reuse_one_plan():
    """All layers of a step share the plan; counters must re-arm between launches."""
    from morphserve_b200 import paged_attention
    L = 4
    c = cases.build_decode_case(seed=5, B=12, Hq=8, Hkv=2, D=128, bs=16, L=L, layer=0, num_blocks_org=1200,
                                dtype=np.float16, max_len=1500)
    d = H.device_case(c)
    mc, ec = H.cfgs(d, d["block_table_t"].shape[1])
    st = H.decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    for rep in range(2):
        for layer in range(L):
            o = torch.zeros((d["B"], d["Hq"] * d["D"]), dtype=torch.float16, device="cuda")
            paged_attention(d["q_t"], d["k_pools_t"][0], d["v_pools_t"][0], [], [], d["block_table_t"], mc, ec, st,
                            layer, o)
            ex = O.paged_attention_exact(c["q"], c["k_pools"], c["v_pools"], c["block_table"], c["seq_ids"],
                                         c["seq_lens"], layer, c["scale"], c["num_blocks_org"], 0)
            _close(o.cpu().numpy().reshape(ex.shape), ex)


def test_plain_kernel_other_shapes():
    """head_dim 64 / block_size 8 (fp16) and fp32 pools take the plain kernel."""
    for dtype, D, bs in ((np.float16, 64, 8), (np.float32, 128, 16), (np.float32, 96, 32)):
        c = cases.build_decode_case(seed=11, B=5, Hq=6, Hkv=3, D=D, bs=bs, L=2, layer=1, num_blocks_org=240,
                                    dtype=dtype, max_len=300)
        o, kp, vp = H.run_decode_step(H.device_case(c))
        ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], 1, c["scale"],
                                     c["num_blocks_org"], 0)
        _close(o, ex)
        # the reference stores fp16-rounded values even into an fp32 `o`
        assert np.array_equal(o, o.astype(np.float16).astype(o.dtype))


def test_push_variant_writes_the_column_slice_of_every_destination():
    """mkv_paged_attention_decode_push with two destination matrices on one GPU (they stand for two ranks'
    buffers): both get this "rank's" heads at the column offset, nothing else is touched, and the fused
    append still lands in the pool."""
    from morphserve_b200 import paged_attention, paged_attention_push
    c = cases.build_decode_case(seed=31, B=21, Hq=8, Hkv=2, D=128, bs=16, L=2, layer=1, num_blocks_org=900,
                                dtype=np.float16, max_len=1200)
    d = H.device_case(c)
    mc, ec = H.cfgs(d, d["block_table_t"].shape[1])
    st = H.decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    kc, vc = d["k_pools_t"][0], d["v_pools_t"][0]
    total_heads, first_head = 24, 8                      # this shard holds heads 8..15 of 24
    outs = [torch.full((d["B"], total_heads * 128), 7.0, dtype=torch.float16, device="cuda") for _ in range(2)]
    paged_attention_push(d["q_t"], kc, vc, [], [], d["block_table_t"], mc, ec, st, d["layer"],
                         [o.data_ptr() for o in outs], total_heads * 128, first_head * 128,
                         k_new=d["k_new_t"], v_new=d["v_new_t"])
    ref = torch.zeros((d["B"], d["Hq"] * 128), dtype=torch.float16, device="cuda")
    st2 = H.decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    paged_attention(d["q_t"], kc, vc, [], [], d["block_table_t"], mc, ec, st2, d["layer"], ref)   # pool already appended
    torch.cuda.synchronize()
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_decode(c["k_new"], c["v_new"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"],
                           c["layer"], c["num_blocks_org"], 0)
    assert kc.cpu().numpy().tobytes() == kpo[0].tobytes() and vc.cpu().numpy().tobytes() == vpo[0].tobytes()
    for o in outs:
        assert torch.equal(o[:, first_head * 128:(first_head + 8) * 128], ref)
        assert (o[:, : first_head * 128] == 7.0).all() and (o[:, (first_head + 8) * 128:] == 7.0).all()


@pytest.mark.parametrize("seed", range(10))
def test_plan_kernel_follows_the_stated_rule(seed):
    """What the plan leaves in the workspace against the rules restated on the host (tests/helpers.py), for batches
    from 1 to 3000 sequences and several split_balance settings.  No sequence longer than `ratio` chunks: chunk size, item
    count and partial-row count of the dynamic deal (`plan_rule`).  A longest sequence of more than `ratio` chunks:
    the static deal, every worker's range of unit records, record by record (`static_deal`)."""
    import ctypes as C
    from morphserve_b200._lib import lib, check
    from morphserve_b200.worker.kernels._common import attn_workspace
    rs = np.random.RandomState(77 + seed)
    B = int(rs.choice([1, 7, 64, 256, 900, 3000]))
    Hkv = int(rs.choice([1, 2, 8, 32]))
    G = int(rs.choice([1, 4, 8]))
    Hq = Hkv * G
    max_len = int(rs.choice([40, 700, 1536, 30000])) if B <= 256 else int(rs.choice([40, 700]))
    lens = rs.randint(1, max_len + 1, size=B).astype(np.int32)
    if seed % 3 == 0:
        lens[rs.randint(0, B, size=max(1, B // 10))] = 0            # sequences without any token
    balance = float(rs.choice([0.0, 1.0, 1.5, 4.0]))
    unit_cost = int(rs.choice([0, 1, 3]))
    ratio = int(rs.choice([1, 8]))
    max_blocks = (int(lens.max()) + 15) // 16
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    check(lib.mkv_attn_configure(-1, -1, -1.0, balance, -1), "mkv_attn_configure")
    check(lib.mkv_attn_set_static_deal(1, unit_cost, ratio), "mkv_attn_set_static_deal")
    try:
        ws = attn_workspace(0, B, Hq, Hkv, 128, max_blocks)
        lay = (C.c_int64 * 10)()
        check(lib.mkv_attn_workspace_layout(0, B, Hq, Hkv, 128, max_blocks, lay), "mkv_attn_workspace_layout")
        lens_t, ids_t = H.to_dev(lens), torch.arange(B, dtype=torch.int32, device="cuda") + 3
        stream = torch.cuda.current_stream().cuda_stream
        check(lib.mkv_attn_plan(0, stream, ws.tensor.data_ptr(), ws.nbytes, lens_t.data_ptr(), ids_t.data_ptr(), B,
                                Hq, Hkv, 128, 16, max_blocks), "mkv_attn_plan")
        ws.generation += 1
        torch.cuda.synchronize()
        raw = ws.tensor.cpu().numpy()
    finally:
        check(lib.mkv_attn_configure(-1, -1, -1.0, 1.5, -1), "mkv_attn_configure")
        check(lib.mkv_attn_set_static_deal(1, 3, 1), "mkv_attn_set_static_deal")
    hdr = raw[:64].view(np.int32)
    magic, batch, n_items, chunk, counter, _, flags, n_rows, cap, mode, n_workers, n_units, counter_init = \
        [int(x) for x in hdr[:13]]
    off_items, _, off_wstart, _, _, _, cap_items, cap_units, max_workers, workers = [int(x) for x in lay]
    assert magic == 0x4d4b5631 and batch == B and flags == 0 and cap == cap_items
    exp_chunk, exp_items, exp_rows = H.plan_rule(lens, Hkv, cap, sms, balance)
    longest = (int(lens.max()) + 15) // 16
    if longest <= ratio * exp_chunk:        # not skewed: chunks from the shared counter (cut or not)
        assert mode == 0 and (chunk, n_items, n_rows) == (exp_chunk, exp_items, exp_rows)
        assert n_units == n_items * Hkv and n_workers == workers
        assert counter == counter_init == min(n_units, workers)     # worker w starts on unit w without a claim
        return
    W, wstart, units = H.static_deal(lens, Hkv, workers, cap_items * Hq, G, unit_cost=unit_cost)
    assert B * Hkv + W <= cap_units
    assert (mode, n_workers, n_units, n_rows) == (1, W, len(units), 2 * W)
    got_start = raw[off_wstart:off_wstart + 4 * (max_workers + 1)].view(np.int32)
    np.testing.assert_array_equal(got_start[:W + 1], wstart)
    assert (got_start[W:] == len(units)).all()
    rec = raw[off_items:off_items + 32 * len(units)].view(np.int32).reshape(-1, 8)
    exp = np.array([(b, first, n, piece | (h << 16), ln, pieces, owner, b + 3)
                    for (b, first, n, piece, h, ln, pieces, owner) in units], dtype=np.int32)
    np.testing.assert_array_equal(rec, exp)


def test_launch_without_a_matching_plan_touches_nothing():
    """The decode kernel checks the workspace header before anything else: a plan made for another batch size
    (or none at all) makes it set bit 1 of the error word and return; `o` and the pool stay as they were.  A later
    call with a fresh plan works."""
    from morphserve_b200._lib import lib, check
    from morphserve_b200.worker.kernels._common import attn_workspace, make_pool, read_attn_error_flags
    lens = np.array([40, 17, 300, 5])
    c = cases.build_decode_case(seed=8, B=4, Hq=8, Hkv=2, D=128, bs=16, L=1, layer=0, num_blocks_org=40,
                                dtype=np.float16, lens=lens)
    d = H.device_case(c)
    bt = d["block_table_t"]
    pool = make_pool(d["k_pools_t"][0], d["v_pools_t"][0], [], [], 40, 0)
    ws = attn_workspace(0, 4, 8, 2, 128, bt.shape[1])
    stream = torch.cuda.current_stream().cuda_stream
    # a plan for the first three sequences only
    check(lib.mkv_attn_plan(0, stream, ws.tensor.data_ptr(), ws.nbytes, d["seq_lens_t"].data_ptr(),
                            d["seq_ids_t"].data_ptr(), 3, 8, 2, 128, 16, bt.shape[1]), "mkv_attn_plan")
    ws.generation += 1
    o = torch.full((4, 8 * 128), 7.0, dtype=torch.float16, device="cuda")
    k_before = d["k_pools_t"][0].clone()

    def attend():
        check(lib.mkv_paged_attention_decode_append(
            0, stream, d["q_t"].data_ptr(), o.data_ptr(), d["k_new_t"].data_ptr(), d["v_new_t"].data_ptr(), pool,
            bt.data_ptr(), bt.stride(0), d["seq_ids_t"].data_ptr(), d["seq_lens_t"].data_ptr(), 4, 8, 0,
            float(c["scale"]), bt.shape[1], ws.tensor.data_ptr(), ws.nbytes), "mkv_paged_attention_decode_append")
        torch.cuda.synchronize()

    attend()
    assert read_attn_error_flags(0) & 2
    assert bool((o == 7.0).all()) and torch.equal(d["k_pools_t"][0], k_before)
    check(lib.mkv_attn_plan(0, stream, ws.tensor.data_ptr(), ws.nbytes, d["seq_lens_t"].data_ptr(),
                            d["seq_ids_t"].data_ptr(), 4, 8, 2, 128, 16, bt.shape[1]), "mkv_attn_plan")
    ws.generation += 1
    attend()
    assert read_attn_error_flags(0) == 0
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_decode(c["k_new"], c["v_new"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], 0, 40, 0)
    ex = O.paged_attention_exact(c["q"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], 0, c["scale"], 40, 0)
    _close(o.cpu().numpy().reshape(ex.shape), ex)


def test_reused_infer_state_with_lengths_updated_in_place_is_planned_again():
    """A caller may keep ONE LlamaInferState object and update ``decoding_seq_lens`` in place from step to step.  The
    kernel takes the lengths from the plan, so a plan kept from the previous step would silently attend over the old
    lengths: a call whose layer number is not above the previous call's starts a new step and must plan afresh.
    Step two changes the lengths drastically (a 30-token sequence becomes 900 tokens long and the other way round)."""
    from morphserve_b200 import paged_attention
    lens1 = np.array([30, 900, 64, 17, 333, 5], dtype=np.int32)
    lens2 = np.array([900, 30, 65, 300, 2, 512], dtype=np.int32)
    B, Hq, Hkv, L = len(lens1), 8, 2, 2
    nb = int(((np.maximum(lens1, lens2) + 15) // 16).sum()) + 4
    c = cases.build_decode_case(seed=99, B=B, Hq=Hq, Hkv=Hkv, D=128, bs=16, L=L, layer=0, num_blocks_org=nb,
                                dtype=np.float16, lens=np.maximum(lens1, lens2))
    d = H.device_case(c)
    mc, ec = H.cfgs(d, d["block_table_t"].shape[1])
    lens_t = H.to_dev(lens1.copy())
    st = H.decode_state(d, d["seq_ids_t"], lens_t)
    st.max_decoding_len = int(max(lens1.max(), lens2.max()))
    kp, vp = [p for p in c["k_pools"]], [p for p in c["v_pools"]]
    for lens in (lens1, lens2):
        lens_t.copy_(H.to_dev(lens))                       # in place: same tensor, same infer state object
        for layer in range(L):
            o = torch.zeros((B, Hq * 128), dtype=torch.float16, device="cuda")
            paged_attention(d["q_t"], d["k_pools_t"][0], d["v_pools_t"][0], [], [], d["block_table_t"], mc, ec, st, layer, o)
            torch.cuda.synchronize()
            ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], lens, layer, c["scale"],
                                         c["num_blocks_org"], 0)
            _close(o.cpu().numpy().reshape(ex.shape), ex)
