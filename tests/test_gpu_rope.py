"""GPU parity of the rotary embedding (the step in front of the KV append): the stand-alone
kernel bit-exact against the reference's output (fixtures) and the oracle, and the form fused
into the decode-attention launch against the three separate calls.

Every test runs under both roundings the library offers: "written" (each operation rounds, the
reference kernel in the Triton interpreter - the committed fixtures) and "compiled" (one multiply
of each output fused into the add, the reference kernel compiled for a GPU; held to the compiled
kernel itself in tests/test_gpu_reference.py)."""
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
ROUNDING = "written"


@pytest.fixture(params=["written", "compiled"], autouse=True)
def rounding(request):
    import morphserve_b200 as mk
    global ROUNDING
    ROUNDING = request.param
    mk.set_rope_rounding(ROUNDING)
    yield ROUNDING
    ROUNDING = "written"
    mk.set_rope_rounding("compiled")      # the library's default


def _state(c, cos, sin, n_dec=0):
    st = H.decode_state(dict(scale=1.0, num_blocks_org=0, chunk_blocks=0), torch.zeros(0, dtype=torch.int32, device="cuda"),
                        torch.zeros(0, dtype=torch.int32, device="cuda"))
    st.position_cos, st.position_sin = cos, sin
    st.num_decoding_seqs = n_dec
    return st


@pytest.mark.parametrize("name", list(cases.ROPE_CASES))
def test_rotary_embedding_matches_reference_fixture(name):
    from morphserve_b200 import rotary_embedding_inplace
    if ROUNDING != "written":
        pytest.skip("the fixtures hold the reference kernel's output in the Triton interpreter: rounding as written")
    c = cases.build_rope_case(**cases.ROPE_CASES[name])
    gold = np.load(os.path.join(G, f"rope_{name}.npz"))
    q, k = H.to_dev(c["q"]), H.to_dev(c["k"])
    rotary_embedding_inplace(q, k, _state(c, H.to_dev(c["cos"]), H.to_dev(c["sin"])))
    torch.cuda.synchronize()
    assert q.cpu().numpy().tobytes() == gold["q"].tobytes()
    assert k.cpu().numpy().tobytes() == gold["k"].tobytes()


# (T, Hq, Hkv, D, dtype): vector path (D/2 a multiple of 8), scalar path (odd sizes, fp32), a prefill-sized batch
ROPE_SWEEP = [(1, 1, 1, 128, np.float16), (300, 32, 8, 128, np.float16), (17, 6, 3, 96, np.float16),
              (5, 4, 2, 20, np.float16), (33, 8, 8, 128, np.float32), (4097, 32, 8, 128, np.float16),
              (0, 4, 4, 128, np.float16)]


@pytest.mark.parametrize("T,Hq,Hkv,D,dtype", ROPE_SWEEP)
def test_rotary_embedding_sweep_against_oracle(T, Hq, Hkv, D, dtype):
    from morphserve_b200 import rotary_embedding_inplace
    c = cases.build_rope_case(seed=T * 31 + D, T=T, Hq=Hq, Hkv=Hkv, D=D, dtype=dtype, max_pos=8192)
    q, k = H.to_dev(c["q"]), H.to_dev(c["k"])
    rotary_embedding_inplace(q, k, _state(c, H.to_dev(c["cos"]), H.to_dev(c["sin"])))
    torch.cuda.synchronize()
    qo, ko = O.rotary_embedding(c["q"], c["k"], c["cos"], c["sin"], rounding=ROUNDING)
    assert q.cpu().numpy().tobytes() == qo.tobytes()
    assert k.cpu().numpy().tobytes() == ko.tobytes()


def _decode_layer(d, cos, sin, fused):
    """rotary -> store_kvcache -> paged_attention through the public API, as the reference's layer code
    calls them (worker/layers/transformer_layer.py:93-126,181-187)."""
    import morphserve_b200 as mk
    mc, ec = H.cfgs(d, d["block_table_t"].shape[1])
    st = H.decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    st.position_cos, st.position_sin = cos, sin
    kc, vc = d["k_pools_t"][0], d["v_pools_t"][0]
    kn, vn = d["k_pools_t"][1:], d["v_pools_t"][1:]
    mk.set_fused_decode_append(fused)
    mk.set_fused_decode_rope(fused)
    try:
        mk.rotary_embedding_inplace(d["q_t"], d["k_new_t"], st)
        mk.store_kvcache(d["k_new_t"], d["v_new_t"], kc, vc, kn, vn, d["block_table_t"], mc, ec, st, d["layer"])
        o = torch.zeros((d["B"], d["Hq"] * d["D"]), dtype=d["q_t"].dtype, device="cuda")
        mk.paged_attention(d["q_t"], kc, vc, kn, vn, d["block_table_t"], mc, ec, st, d["layer"], o)
        torch.cuda.synchronize()
    finally:
        mk.set_fused_decode_append(False)
        mk.set_fused_decode_rope(False)
    assert "_mkv_pending_rope" not in st.__dict__ and "_mkv_pending_append" not in st.__dict__
    return (o.cpu().numpy().reshape(d["B"], d["Hq"], d["D"]),
            [p.cpu().numpy() for p in d["k_pools_t"]], [p.cpu().numpy() for p in d["v_pools_t"]])


# (B, Hq, Hkv, max_len, chunks): group sizes 1, 4, 8, 16 (16 uses the padded-row code), split sequences, elastic pool
FUSED_SWEEP = [(5, 8, 2, 300, 0), (24, 32, 32, 768, 0), (33, 64, 8, 1536, 0), (3, 16, 1, 5000, 0), (6, 8, 2, 200, 2)]


@pytest.mark.parametrize("B,Hq,Hkv,max_len,n_chunks", FUSED_SWEEP)
def test_fused_rope_append_attention_equals_separate_calls(B, Hq, Hkv, max_len, n_chunks):
    rs = np.random.RandomState(B * 13 + Hq)
    lens = rs.randint(1, max_len + 1, size=B)
    lens[0] = max_len
    need = int(((lens + 15) // 16).sum())
    kw = dict(num_blocks_org=need + 5)
    if n_chunks:
        kw = dict(num_blocks_org=need // 2, chunk_blocks=(need - need // 2 + n_chunks) // n_chunks + 1, n_chunks=n_chunks)
    c = cases.build_decode_case(seed=B * 7 + Hkv, B=B, Hq=Hq, Hkv=Hkv, D=128, bs=16, L=2, layer=1, dtype=np.float16,
                                lens=lens, **kw)
    cos_np, sin_np = cases.rope_tables(lens - 1, 128)
    cos, sin = H.to_dev(cos_np), H.to_dev(sin_np)

    o_sep, kp_sep, vp_sep = _decode_layer(H.device_case(c), cos, sin, fused=False)
    d = H.device_case(c)
    o_fus, kp_fus, vp_fus = _decode_layer(d, cos, sin, fused=True)
    # fused form: q and k_new stay as they were in memory; pool and output equal the separate calls bit for bit
    assert d["q_t"].cpu().numpy().tobytes() == c["q"].tobytes()
    assert d["k_new_t"].cpu().numpy().tobytes() == c["k_new"].tobytes()
    for a, b in zip(kp_fus + vp_fus, kp_sep + vp_sep):
        assert a.tobytes() == b.tobytes()
    assert o_fus.tobytes() == o_sep.tobytes()
    # and both agree with the oracle: rotated rows bit-exact in the pool, attention within tolerance
    q_rot, k_rot = O.rotary_embedding(c["q"], c["k_new"], cos_np, sin_np, rounding=ROUNDING)
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_decode(k_rot, c["v_new"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], c["layer"],
                           c["num_blocks_org"], c["chunk_blocks"])
    for a, b in zip(kp_fus + vp_fus, kpo + vpo):
        assert a.tobytes() == b.tobytes()
    ex = O.paged_attention_exact(q_rot, kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], c["layer"],
                                 c["scale"], c["num_blocks_org"], c["chunk_blocks"])
    np.testing.assert_allclose(o_fus.astype(np.float64), ex, rtol=RTOL, atol=ATOL)


def test_fused_rope_with_prefill_rows_in_the_batch():
    """Mixed batch: the prefill rows are rotated in place by rotary_embedding_inplace itself, only the decode
    rows wait for the attention launch."""
    import morphserve_b200 as mk
    c = cases.build_prefill_case(**cases.PREFILL_CASES["mixed_fp16"])
    npre_tok, nd = c["num_prefill_tokens"], len(c["decode_lens"])
    T, Hkv, D = c["k"].shape[0], c["Hkv"], c["D"]
    Hq = 2 * Hkv
    rs = np.random.RandomState(1)
    q_np = rs.standard_normal((T, Hq, D)).astype(np.float16)
    pos = np.concatenate([np.concatenate([np.arange(n) for n in c["prefill_lens"]]), c["decode_lens"] - 1])
    cos_np, sin_np = cases.rope_tables(pos, D)
    q_rot, k_rot = O.rotary_embedding(q_np, c["k"], cos_np, sin_np, rounding=ROUNDING)

    kp = [H.to_dev(p) for p in c["k_pools"]]
    vp = [H.to_dev(p) for p in c["v_pools"]]
    bt = H.to_dev(c["block_table"])
    q, k, v = H.to_dev(q_np), H.to_dev(c["k"]), H.to_dev(c["v"])
    z = torch.zeros(0, dtype=torch.int32, device="cuda")
    from morphserve_b200.worker.infer_state import LlamaInferState
    st = LlamaInferState(
        batch_size=len(c["seq_ids"]), num_tokens=T, seq_ids=H.to_dev(c["seq_ids"]), softmax_scale=D ** -0.5,
        num_prefill_seqs=len(c["prefill_lens"]), num_prefill_tokens=npre_tok,
        prefill_seq_start_locs=H.to_dev(c["prefill_start_locs"]), prefill_seq_start_locs_with_end=z,
        prefill_seq_lens=H.to_dev(c["prefill_lens"]), max_prefill_len=int(c["prefill_lens"].max()),
        num_decoding_seqs=nd, decoding_seq_lens=H.to_dev(c["decode_lens"]),
        max_decoding_len=int(c["decode_lens"].max()), seq_block_size=512, num_seq_blocks=1,
        num_blocks_org=c["num_blocks_org"], kv_cache_new_block_size=c["chunk_blocks"], org_layer_param_size=0,
        position_cos=H.to_dev(cos_np), position_sin=H.to_dev(sin_np), ignore_kvcache=False)
    mc, ec = H.cfgs(c, bt.shape[1])
    mc.num_q_heads = Hq
    mk.set_fused_decode_append(True)
    mk.set_fused_decode_rope(True)
    try:
        mk.rotary_embedding_inplace(q, k, st)
        mk.store_kvcache(k, v, kp[0], vp[0], kp[1:], vp[1:], bt, mc, ec, st, c["layer"])
        o = torch.zeros((nd, Hq * D), dtype=torch.float16, device="cuda")
        mk.paged_attention(q[npre_tok:], kp[0], vp[0], kp[1:], vp[1:], bt, mc, ec, st, c["layer"], o)
        torch.cuda.synchronize()
    finally:
        mk.set_fused_decode_append(False)
        mk.set_fused_decode_rope(False)
    assert q[:npre_tok].cpu().numpy().tobytes() == q_rot[:npre_tok].tobytes()
    assert k[:npre_tok].cpu().numpy().tobytes() == k_rot[:npre_tok].tobytes()
    assert q[npre_tok:].cpu().numpy().tobytes() == q_np[npre_tok:].tobytes()       # decode rows untouched
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_prefill(k_rot, c["v"], kpo, vpo, c["block_table"], c["seq_ids"][:len(c["prefill_lens"])],
                            c["prefill_start_locs"],
                            c["prefill_lens"], c["layer"], c["num_blocks_org"], c["chunk_blocks"])
    O.store_kvcache_decode(k_rot[npre_tok:], c["v"][npre_tok:], kpo, vpo, c["block_table"],
                           c["seq_ids"][len(c["prefill_lens"]):], c["decode_lens"], c["layer"], c["num_blocks_org"],
                           c["chunk_blocks"])
    for a, b in zip(kp + vp, kpo + vpo):
        assert a.cpu().numpy().tobytes() == b.tobytes()
    ex = O.paged_attention_exact(q_rot[npre_tok:], kpo, vpo, c["block_table"], c["seq_ids"][len(c["prefill_lens"]):],
                                 c["decode_lens"], c["layer"], D ** -0.5, c["num_blocks_org"], c["chunk_blocks"])
    np.testing.assert_allclose(o.cpu().numpy().reshape(ex.shape).astype(np.float64), ex, rtol=RTOL, atol=ATOL)


def test_pending_rope_is_flushed_when_no_fused_attention_follows():
    """rotary_embedding_inplace in fused mode followed by a store_kvcache that cannot fuse (append mode switched
    off in between): the decode rows are rotated in place before they are appended."""
    import morphserve_b200 as mk
    lens = np.array([5, 40, 17])
    c = cases.build_decode_case(seed=77, B=3, Hq=8, Hkv=2, D=128, bs=16, L=1, layer=0, num_blocks_org=16,
                                dtype=np.float16, lens=lens)
    cos_np, sin_np = cases.rope_tables(lens - 1, 128)
    d = H.device_case(c)
    mc, ec = H.cfgs(d, d["block_table_t"].shape[1])
    st = H.decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    st.position_cos, st.position_sin = H.to_dev(cos_np), H.to_dev(sin_np)
    mk.set_fused_decode_append(True)
    mk.set_fused_decode_rope(True)
    try:
        mk.rotary_embedding_inplace(d["q_t"], d["k_new_t"], st)
        assert "_mkv_pending_rope" in st.__dict__
        mk.set_fused_decode_append(False)
        mk.store_kvcache(d["k_new_t"], d["v_new_t"], d["k_pools_t"][0], d["v_pools_t"][0], [], [], d["block_table_t"],
                         mc, ec, st, 0)
        torch.cuda.synchronize()
    finally:
        mk.set_fused_decode_append(False)
        mk.set_fused_decode_rope(False)
    q_rot, k_rot = O.rotary_embedding(c["q"], c["k_new"], cos_np, sin_np, rounding=ROUNDING)
    assert d["q_t"].cpu().numpy().tobytes() == q_rot.tobytes()
    assert d["k_new_t"].cpu().numpy().tobytes() == k_rot.tobytes()
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_decode(k_rot, c["v_new"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], 0, 16, 0)
    assert d["k_pools_t"][0].cpu().numpy().tobytes() == kpo[0].tobytes()


def test_rope_append_entry_on_a_shape_without_fused_path():
    """head_dim 64: mkv_paged_attention_decode_rope_append rotates q and k_new in place with the stand-alone
    kernel, appends, then attends - same result as the separate calls."""
    from morphserve_b200._lib import lib, check
    from morphserve_b200.worker.kernels._common import attn_workspace, make_pool
    lens = np.array([9, 33, 64, 100])
    c = cases.build_decode_case(seed=5, B=4, Hq=6, Hkv=3, D=64, bs=8, L=2, layer=1, num_blocks_org=40,
                                dtype=np.float16, lens=lens)
    cos_np, sin_np = cases.rope_tables(lens - 1, 64)
    d = H.device_case(c)
    cos, sin = H.to_dev(cos_np), H.to_dev(sin_np)
    pool = make_pool(d["k_pools_t"][0], d["v_pools_t"][0], [], [], c["num_blocks_org"], 0)
    bt = d["block_table_t"]
    ws = attn_workspace(0, 4, 6, 3, 64, bt.shape[1])
    o = torch.zeros((4, 6 * 64), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    check(lib.mkv_attn_plan(0, stream, ws.tensor.data_ptr(), ws.nbytes, d["seq_lens_t"].data_ptr(),
                            d["seq_ids_t"].data_ptr(), 4, 6, 3, 64, 8, bt.shape[1]), "plan")
    ws.generation += 1
    check(lib.mkv_paged_attention_decode_rope_append(
        0, stream, d["q_t"].data_ptr(), o.data_ptr(), d["k_new_t"].data_ptr(), d["v_new_t"].data_ptr(),
        cos.data_ptr(), sin.data_ptr(), pool, bt.data_ptr(), bt.stride(0), d["seq_ids_t"].data_ptr(),
        d["seq_lens_t"].data_ptr(), 4, 6, 1, float(c["scale"]), bt.shape[1], ws.tensor.data_ptr(), ws.nbytes), "rope_append")
    torch.cuda.synchronize()
    q_rot, k_rot = O.rotary_embedding(c["q"], c["k_new"], cos_np, sin_np, rounding=ROUNDING)
    assert d["q_t"].cpu().numpy().tobytes() == q_rot.tobytes()
    kpo, vpo = [p.copy() for p in c["k_pools"]], [p.copy() for p in c["v_pools"]]
    O.store_kvcache_decode(k_rot, c["v_new"], kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], 1, 40, 0)
    assert d["k_pools_t"][0].cpu().numpy().tobytes() == kpo[0].tobytes()
    ex = O.paged_attention_exact(q_rot, kpo, vpo, c["block_table"], c["seq_ids"], c["seq_lens"], 1, c["scale"], 40, 0)
    np.testing.assert_allclose(o.cpu().numpy().reshape(ex.shape).astype(np.float64), ex, rtol=RTOL, atol=ATOL)
