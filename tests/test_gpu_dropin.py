"""The drop-in contract, exercised on the reference's own call sites.

``tests/dropin_runner.py`` runs the reference's unmodified ``LlamaModel`` (worker/model.py:302-436 ``forward``,
:468-534 ``_swap`` / ``free_seqs_resources``, :176-227 ``init_kvcache_and_swap``) and its unmodified layer code
(worker/layers/transformer_layer.py:111-191: append on the default stream, an event, attention on the
piggyback stream behind it, a second event back) through a serving scenario - prompts, decode steps, a swap-out,
a free, a swap-in, a mixed prefill+decode step, decode steps across block boundaries - once with the reference's
own kernels, BlockManager and ``swiftllm_c``, and once after ``morphserve_b200.install_as_swiftllm()`` in each of the
three modes (separate launches, append fused into attention, rotary embedding fused too).  Compared after
every step: block tables, counts, bitmaps and free counts of both managers (exact), the K/V pools and the host swap
space (layer 0 bit-equal: its rows depend on nothing this package computes differently - the rotary embedding
rounds like the reference's compiled kernel; deeper layers inherit the attention tolerance), the final hidden
states, the sampled tokens.

The last test replays the scenario through ``KVCacheModelState`` (this package's stand-alone form of the same model
methods) and holds ``prepare_step`` to the LlamaInferState objects the reference's ``forward`` built.
"""
import dataclasses
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import ref_loader

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (ref_loader.available() and ref_loader.ext_available()),
                                 reason=ref_loader.why_unavailable())]


def _run(tmp_path_factory, impl, fused=0):
    out = str(tmp_path_factory.mktemp("dropin") / f"{impl}{fused}.npz")
    cmd = [sys.executable, os.path.join(ROOT, "tests", "dropin_runner.py"), "--impl", impl, "--fused", str(fused),
           "--out", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, f"{' '.join(cmd)} failed:\n{r.stdout[-3000:]}\n{r.stderr[-6000:]}"
    return np.load(out, allow_pickle=False)


@pytest.fixture(scope="module")
def reference_run(tmp_path_factory):
    return _run(tmp_path_factory, "reference")


def _scenario():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dropin_runner
    return dropin_runner


@pytest.mark.parametrize("fused", [0, 1, 2])
def test_reference_model_runs_unchanged_on_this_package(reference_run, tmp_path_factory, fused):
    ref = reference_run
    got = _run(tmp_path_factory, "morphkv", fused)
    n = int(ref["n_steps"])
    assert int(got["n_steps"]) == n and int(got["attn_error_flags"]) == 0
    calls = __import__("json").loads(str(got["calls"]))
    assert calls.get("mkv_block_allocate", 0) > 0 and calls.get("mkv_store_kv_prefill", 0) > 0
    if fused == 0:
        assert calls.get("mkv_paged_attention_decode", 0) > 0 and calls.get("mkv_store_kv_decode", 0) > 0
        assert calls.get("mkv_rotary_embedding", 0) > 0
    elif fused == 1:
        assert calls.get("mkv_paged_attention_decode_append", 0) > 0
    else:
        assert calls.get("mkv_paged_attention_decode_rope_append", 0) > 0
    agree = total = 0
    worst = 0.0
    for i in range(n):
        for bm in ("gpu", "cpu"):
            for what in ("table", "count", "free", "nfree"):
                key = f"{bm}_{what}_{i}"
                assert np.array_equal(ref[key], got[key]), f"step {i}: {key} differs"
        for pool in ("k_cache", "v_cache", "k_swap", "v_swap"):
            a, b = got[f"{pool}_{i}"], ref[f"{pool}_{i}"]
            assert a[:, 0].tobytes() == b[:, 0].tobytes(), f"step {i}: layer 0 of {pool} is not bit-equal"
            np.testing.assert_allclose(a.astype(np.float32), b.astype(np.float32), rtol=2e-2, atol=2e-2,
                                       err_msg=f"step {i}: {pool}")
        if f"hidden_{i}" in ref.files:
            a, b = got[f"hidden_{i}"], ref[f"hidden_{i}"]
            scale = float(np.abs(b).max())
            worst = max(worst, float(np.abs(a - b).max()) / scale)
            np.testing.assert_allclose(a, b, rtol=2e-2, atol=2e-2 * scale, err_msg=f"step {i}: hidden states")
            agree += int((got[f"tokens_{i}"] == ref[f"tokens_{i}"]).sum())
            total += ref[f"tokens_{i}"].size
            for f in ref.files:
                if f.startswith(f"state_{i}_"):
                    assert np.array_equal(ref[f], got[f]), f"step {i}: {f}"
    assert agree >= 0.95 * total, f"only {agree} of {total} sampled tokens agree"
    print(f"fused={fused}: hidden states within {worst:.2e} of their range, {agree}/{total} tokens equal")


@pytest.mark.parametrize("pin_swap", [False, True])
def test_prepare_step_and_model_methods_against_the_reference_run(reference_run, pin_swap):
    """KVCacheModelState.prepare_step / swap_in_seqs / swap_out_seqs / free_seqs_resources against what the
    reference's LlamaModel did in the same scenario: every LlamaInferState field forward() built
    (worker/model.py:318-436), both managers' integer state after every step, and the bytes the swaps moved."""
    import types
    import morphserve_b200 as mk
    R = _scenario()
    ref = reference_run
    M = R.MODEL
    mc = types.SimpleNamespace(num_layers=M["num_hidden_layers"], num_q_heads=M["num_attention_heads"],
                               num_kv_heads=M["num_key_value_heads"], head_dim=M["hidden_size"] // M["num_attention_heads"],
                               rope_theta=M["rope_theta"], rope_scaling=1.0,
                               max_position_embeddings=M["max_position_embeddings"])
    ec = types.SimpleNamespace(block_size=R.BLOCK, num_cpu_blocks=R.NUM_CPU_BLOCKS, max_seqs_in_block_table=R.MAX_SEQS,
                               max_blocks_per_seq=R.MAX_BLOCKS_PER_SEQ)
    state = mk.KVCacheModelState(mc, ec, pin_swap=pin_swap)
    state.init_kvcache_and_swap(R.NUM_BLOCKS)
    with torch.inference_mode():        # the model's tensors are inference tensors (worker/model.py:175)
        _replay(R, ref, state)


def _replay(R, ref, state):
    for i, step in enumerate(R.scenario()):
        if step[0] == "forward":
            st = state.prepare_step(step[1], step[2], step[3])
            for f in dataclasses.fields(st):
                key = f"state_{i}_{f.name}"
                val = getattr(st, f.name)
                if key not in ref.files:
                    assert val is None, f"step {i}: {f.name}"
                    continue
                if isinstance(val, torch.Tensor):
                    assert val.dtype == torch.from_numpy(ref[key]).dtype, f"step {i}: dtype of {f.name}"
                    assert np.array_equal(val.cpu().numpy(), ref[key]), f"step {i}: {f.name}"
                else:
                    assert type(val) is type(ref[key].item()) and val == ref[key].item(), f"step {i}: {f.name}"
            # the layers' writes are not replayed here: take the pools the reference run held after this step
            state.k_cache.copy_(torch.from_numpy(ref[f"k_cache_{i}"]))
            state.v_cache.copy_(torch.from_numpy(ref[f"v_cache_{i}"]))
        elif step[0] == "swap_out":
            state.swap_out_seqs(step[1])
        elif step[0] == "swap_in":
            state.swap_in_seqs(step[1])
        else:
            state.free_seqs_resources(step[1])
        torch.cuda.synchronize()
        for nm, bm in (("gpu", state.gpu_block_manager), ("cpu", state.cpu_block_manager)):
            assert np.array_equal(bm.block_table.cpu().numpy(), ref[f"{nm}_table_{i}"]), f"step {i}: {nm} table"
            assert np.array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), ref[f"{nm}_count_{i}"])
            assert np.array_equal(bm.is_block_free.cpu().numpy(), ref[f"{nm}_free_{i}"])
            assert int(bm.num_free_blocks) == int(ref[f"{nm}_nfree_{i}"])
        if step[0] in ("swap_out", "swap_in"):
            assert state.k_swap.numpy().tobytes() == ref[f"k_swap_{i}"].tobytes(), f"step {i}: k_swap"
            assert state.v_swap.numpy().tobytes() == ref[f"v_swap_{i}"].tobytes(), f"step {i}: v_swap"
            assert state.k_cache.cpu().numpy().tobytes() == ref[f"k_cache_{i}"].tobytes(), f"step {i}: k_cache"
            assert state.v_cache.cpu().numpy().tobytes() == ref[f"v_cache_{i}"].tobytes(), f"step {i}: v_cache"
