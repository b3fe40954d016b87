"""Pins the CPU oracle against outputs of the reference's own kernels (golden
fixtures made by tests/golden/make_golden.py in the Triton interpreter)."""
import os

import numpy as np
import pytest

from oracle import kv_oracle as O
from tests.golden import cases

G = os.path.join(os.path.dirname(__file__), "golden")
RTOL, ATOL = 2e-3, 1e-2          # attention tolerance of the path (fp16 data, fp32 accumulation)


def _copy_pools(c):
    return [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]


@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_decode_append_and_attention_match_reference(name):
    c = cases.build_decode_case(**cases.DECODE_CASES[name])
    gold = np.load(os.path.join(G, f"decode_{name}.npz"))
    assert str(gold["inputs_sha256"]) == cases.case_inputs_hash(c), "seeded inputs differ from the fixture's"
    kp, vp = _copy_pools(c)
    O.store_kvcache_decode(c["k_new"], c["v_new"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"],
                           c["layer"], c["num_blocks_org"], c["chunk_blocks"])
    # append is a bit copy: the whole pool must hash identically to the reference's
    assert cases.sha256_of(*kp, *vp) == str(gold["pools_after_sha256"])
    sbs = int(gold["seq_block_size"])
    o = O.paged_attention_splitkv(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], c["layer"],
                                  c["scale"], sbs, c["num_blocks_org"], c["chunk_blocks"], out_dtype=c["q"].dtype)
    ref = gold["o"].astype(np.float64)
    np.testing.assert_allclose(o.astype(np.float64), ref, rtol=RTOL, atol=ATOL)
    # and both sit on the exact softmax
    ex = O.paged_attention_exact(c["q"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"], c["layer"],
                                 c["scale"], c["num_blocks_org"], c["chunk_blocks"])
    np.testing.assert_allclose(ref, ex, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(o.astype(np.float64), ex, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("name", ["gqa4_fp16", "gqa4_fp16_elastic", "cfg1_mha_fp32"])
def test_torch_loop_matches_reference(name):
    import torch
    c = cases.build_decode_case(**cases.DECODE_CASES[name])
    gold = np.load(os.path.join(G, f"decode_{name}.npz"))
    kp, vp = _copy_pools(c)
    O.store_kvcache_decode(c["k_new"], c["v_new"], kp, vp, c["block_table"], c["seq_ids"], c["seq_lens"],
                           c["layer"], c["num_blocks_org"], c["chunk_blocks"])
    t = torch.from_numpy
    o = O.paged_attention_torch_loop(t(c["q"]), [t(p) for p in kp], [t(p) for p in vp], t(c["block_table"]),
                                     c["seq_ids"], c["seq_lens"], c["layer"], c["scale"],
                                     c["num_blocks_org"], c["chunk_blocks"])
    np.testing.assert_allclose(o.numpy().reshape(gold["o"].shape).astype(np.float64),
                               gold["o"].astype(np.float64), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("name", list(cases.PREFILL_CASES))
def test_prefill_scatter_matches_reference(name):
    c = cases.build_prefill_case(**cases.PREFILL_CASES[name])
    gold = np.load(os.path.join(G, f"prefill_{name}.npz"))
    assert str(gold["inputs_sha256"]) == cases.sha256_of(c["k"], c["v"], c["block_table"], c["seq_ids"])
    kp, vp = _copy_pools(c)
    npre = len(c["prefill_lens"])
    O.store_kvcache_prefill(c["k"], c["v"], kp, vp, c["block_table"], c["seq_ids"][:npre],
                            c["prefill_start_locs"], c["prefill_lens"], c["layer"],
                            c["num_blocks_org"], c["chunk_blocks"])
    nt = c["num_prefill_tokens"]
    O.store_kvcache_decode(c["k"][nt:], c["v"][nt:], kp, vp, c["block_table"], c["seq_ids"][npre:],
                           c["decode_lens"], c["layer"], c["num_blocks_org"], c["chunk_blocks"])
    assert cases.sha256_of(*kp, *vp) == str(gold["pools_after_sha256"])


def test_block_manager_trace_matches_reference():
    tr = cases.block_manager_trace()
    gold = np.load(os.path.join(G, "block_manager_trace.npz"))
    assert int(gold["n_ops"]) == len(tr["ops"])
    bm = O.BlockManagerOracle(tr["num_blocks"], tr["max_seqs"], tr["max_blocks_per_seq"], tr["block_size"])
    for i, (op, ids, lens) in enumerate(tr["ops"]):
        if op == "alloc":
            r = bm.allocate_blocks_for_seqs(ids, lens)
        elif op == "free":
            bm.free_blocks_for_seqs(ids)
            r = np.empty(0, dtype=np.int64)
        else:
            r = bm.gather_allocated_blocks_and_free(ids)
        np.testing.assert_array_equal(r.astype(np.int64), gold[f"ret_{i}"])
        np.testing.assert_array_equal(bm.block_table, gold[f"table_{i}"])
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks, gold[f"count_{i}"])
        np.testing.assert_array_equal(bm.is_block_free, gold[f"free_{i}"])
        assert bm.num_free_blocks == int(gold[f"nfree_{i}"])


def test_seq_block_size_heuristic_examples():
    # worker/model.py:397-402 evaluated by hand
    assert O.seq_block_size_heuristic(32, [100, 200])[0] == 64
    assert O.seq_block_size_heuristic(8, [1536] * 256) == (512, 3)
    assert O.seq_block_size_heuristic(8, [1536] * 16) == (128, 12)


@pytest.mark.parametrize("name", list(cases.ROPE_CASES))
def test_rotary_embedding_matches_reference(name):
    """worker/kernels/rotary_emb.py run in the interpreter vs the oracle: bit-exact (fp16 and fp32 rows)."""
    c = cases.build_rope_case(**cases.ROPE_CASES[name])
    gold = np.load(os.path.join(G, f"rope_{name}.npz"))
    assert str(gold["inputs_sha256"]) == cases.sha256_of(c["q"], c["k"], c["cos"], c["sin"])
    q, k = O.rotary_embedding(c["q"], c["k"], c["cos"], c["sin"])
    assert q.dtype == c["q"].dtype and q.tobytes() == gold["q"].tobytes()
    assert k.tobytes() == gold["k"].tobytes()


def test_rotary_embedding_properties():
    """Position 0 is the identity (cos 1, sin 0); a rotation keeps the norm of every (x0, x1) pair up to fp16
    rounding; rotating by p and then by -p returns the input up to rounding."""
    rs = np.random.RandomState(7)
    q = rs.standard_normal((6, 4, 128)).astype(np.float16)
    k = rs.standard_normal((6, 2, 128)).astype(np.float16)
    cos0, sin0 = cases.rope_tables(np.zeros(6), 128)
    q0, k0 = O.rotary_embedding(q, k, cos0, sin0)
    assert q0.tobytes() == q.tobytes() and k0.tobytes() == k.tobytes()
    pos = rs.randint(1, 5000, size=6)
    cos, sin = cases.rope_tables(pos, 128)
    q1, k1 = O.rotary_embedding(q, k, cos, sin)
    n_in = np.hypot(q[..., :64].astype(np.float64), q[..., 64:].astype(np.float64))
    n_out = np.hypot(q1[..., :64].astype(np.float64), q1[..., 64:].astype(np.float64))
    np.testing.assert_allclose(n_out, n_in, rtol=0, atol=6e-3)
    q2, k2 = O.rotary_embedding(q1, k1, cos, (-sin).astype(np.float16))
    np.testing.assert_allclose(q2.astype(np.float64), q.astype(np.float64), rtol=0, atol=1e-2)
    np.testing.assert_allclose(k2.astype(np.float64), k.astype(np.float64), rtol=0, atol=1e-2)
