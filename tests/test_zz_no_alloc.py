"""The no-allocation attention entry point, called straight through the C ABI.

Why it exists: some callers of the library cannot hand it a workspace because
they cannot allocate device memory when they need attention - code that runs
while work is being captured on the stream, a server that gave the whole GPU to
the KV pool at start-up (a late cudaMalloc may fail), a plug-in that only gets a
stream and raw pointers.  ``mkv_paged_attention_decode_noalloc`` keeps its scratch
in a 16 MiB array inside the library instead.

Checked here: its output equals the regular entry point's (same tolerance as the
other attention tests) on two calls in a row with different batches - the
second call starts from whatever the first left in the shared array - and a
request that does not fit the array is refused with MKV_ERR_TOO_LARGE.

This file sorts last on purpose, so that a run that stops at the first failure
has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.golden import cases

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-2


def _regular(d):
    """Existing entry point (plan + decode with a caller-provided workspace), via the public API."""
    from morphserve_b200 import paged_attention
    mc, ec = H.cfgs(d, d["block_table_t"].shape[1])
    st = H.decode_state(d, d["seq_ids_t"], d["seq_lens_t"])
    o = torch.zeros((d["B"], d["Hq"] * d["D"]), dtype=torch.float16, device="cuda")
    paged_attention(d["q_t"], d["k_pools_t"][0], d["v_pools_t"][0], d["k_pools_t"][1:], d["v_pools_t"][1:],
                    d["block_table_t"], mc, ec, st, d["layer"], o)
    torch.cuda.synchronize()
    return o.cpu().numpy()


def _noalloc(d):
    from morphserve_b200._lib import lib
    from morphserve_b200.worker.kernels._common import make_pool
    pool = make_pool(d["k_pools_t"][0], d["v_pools_t"][0], d["k_pools_t"][1:], d["v_pools_t"][1:],
                     d["num_blocks_org"], d["chunk_blocks"])
    o = torch.zeros((d["B"], d["Hq"] * d["D"]), dtype=d["q_t"].dtype, device="cuda")
    max_blocks = int((int(d["seq_lens"].max()) + 15) // 16)
    before = torch.cuda.memory_allocated()
    st = lib.mkv_paged_attention_decode_noalloc(
        0, torch.cuda.current_stream().cuda_stream, d["q_t"].data_ptr(), o.data_ptr(), C.byref(pool),
        d["block_table_t"].data_ptr(), d["block_table_t"].stride(0), d["seq_ids_t"].data_ptr(),
        d["seq_lens_t"].data_ptr(), d["B"], d["Hq"], d["layer"], C.c_float(d["scale"]), max_blocks)
    assert st == 0, lib.mkv_status_string(st)
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    return o.cpu().numpy()


def test_noalloc_entry_point_matches_regular_one_on_two_calls_in_a_row():
    from morphserve_b200._lib import lib
    assert lib.mkv_noalloc_scratch_bytes() == 16 << 20
    a = cases.build_decode_case(seed=71, B=40, Hq=32, Hkv=8, D=128, bs=16, L=2, layer=1, num_blocks_org=2600,
                                dtype=np.float16, max_len=1536)
    b = cases.build_decode_case(seed=72, B=7, Hq=8, Hkv=2, D=128, bs=16, L=1, layer=0, num_blocks_org=40,
                                dtype=np.float16, chunk_blocks=16, n_chunks=3, lens=[1, 17, 300, 16, 255, 64, 5],
                                force_high_ids=True)
    da, db = H.device_case(a), H.device_case(b)
    ref_a, ref_b = _regular(da), _regular(db)
    got_a = _noalloc(da)          # first call on this device also resolves the array's address
    got_b = _noalloc(db)          # second call reuses the array with call one's leftovers in it
    np.testing.assert_allclose(got_a.astype(np.float64), ref_a.astype(np.float64), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(got_b.astype(np.float64), ref_b.astype(np.float64), rtol=RTOL, atol=ATOL)
    got_a2 = _noalloc(da)
    np.testing.assert_allclose(got_a2.astype(np.float64), ref_a.astype(np.float64), rtol=RTOL, atol=ATOL)


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from morphserve_b200._lib import MkvPool, lib
    pool = MkvPool()
    pool.num_segments, pool.elem_bytes, pool.num_layers, pool.num_kv_heads = 1, 2, 1, 8
    pool.block_size, pool.head_dim, pool.num_blocks_org = 16, 128, 1000
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")        # valid addresses; never dereferenced
    pool.k_base[0] = buf.data_ptr()
    pool.v_base[0] = buf.data_ptr()
    p = buf.data_ptr()
    st = lib.mkv_paged_attention_decode_noalloc(0, None, p, p, C.byref(pool), p, 128, p, p, 2048, 64, 0,
                                                C.c_float(0.1), 96)
    assert st == -9
    assert b"built-in scratch" in lib.mkv_status_string(st)
    torch.cuda.synchronize()


def _builtin_flags():
    from morphserve_b200._lib import lib
    flags = C.c_int(-1)
    st = lib.mkv_attn_read_error_flags(0, torch.cuda.current_stream().cuda_stream, None, C.byref(flags))
    assert st == 0
    return flags.value


@pytest.mark.parametrize("fp32", [False, True])
def test_noalloc_entry_point_reports_a_block_id_outside_the_pool(fp32):
    """Error bits of this entry point live in the library's own array; a NULL workspace makes
    mkv_attn_read_error_flags read them.  A block-table entry that names no block of the pool is never turned into
    an address (the kernels compare it with the pool's size first and read block 0 instead): the call completes,
    bit 0 is set, and the next clean call starts with the word cleared - on the tensor-core path and on the plain
    kernel (fp32 pool) alike."""
    kw = dict(seed=73, B=5, Hq=8, Hkv=2, D=128, bs=16, L=1, layer=0, num_blocks_org=64,
              dtype=np.float32 if fp32 else np.float16, lens=[40, 3, 100, 16, 33])
    good = H.device_case(cases.build_decode_case(**kw))
    _noalloc(good)
    assert _builtin_flags() == 0
    bad = cases.build_decode_case(**kw)
    table = bad["block_table"].copy()
    table[int(bad["seq_ids"][2]), 1] = 10 ** 6            # second block of the third sequence: far outside the pool
    bad["block_table"] = table
    _noalloc(H.device_case(bad))
    assert _builtin_flags() & 1
    _noalloc(good)
    assert _builtin_flags() == 0
