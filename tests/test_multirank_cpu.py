"""Host-side logic of the N > 1 path on two gloo ranks (CPU): how a workload is
cut across ranks, that sequence shards are independent and head shards tile the
head dimension, that the slowest rank's time is what gets reported, and that
attention over a head shard equals the matching slice of the unsharded result
(checked with the oracle, gathered the way the benchmark gathers `o`)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import bench
        from oracle import kv_oracle as O
        from tests.golden import cases

        # --- reported time is the slowest rank's
        assert bench.max_over_ranks(10.0 + rank, dist, torch.device("cpu")) == 10.0 + world - 1

        # --- sequence sharding: own seed, own batch, all heads
        w = bench.shard_workload(bench.WORKLOADS["llama3-8b-gqa-decode"], rank, world)
        assert (w["B"], w["Hq"], w["Hkv"], w["tokens_per_step"]) == (256, 32, 8, 256 * world)
        lens = bench.draw_lengths_and_tables(w, rank, 8)[0]
        gathered = [torch.zeros_like(lens) for _ in range(world)]
        dist.all_gather(gathered, lens)
        assert not torch.equal(gathered[0], gathered[1]), "ranks must draw different sequences"

        # --- head sharding: same sequences everywhere, heads tile [0, Hq)
        h = bench.shard_workload(bench.WORKLOADS["codellama-34b-gqa-decode-headshard"], rank, world)
        assert (h["B"], h["Hq"], h["Hkv"], h["tokens_per_step"]) == (512 * world, 64 // world, 8 // world, 512 * world)
        assert h["head_offset"] == rank * (64 // world)
        hl = bench.draw_lengths_and_tables(h, rank, 8)[0]
        gathered = [torch.zeros_like(hl) for _ in range(world)]
        dist.all_gather(gathered, hl)
        assert torch.equal(gathered[0], gathered[1]), "head shards must share sequences and block tables"

        # --- attention on a head shard == slice of the full result, after the benchmark's gather layout
        c = cases.build_decode_case(seed=7, B=5, Hq=8, Hkv=4, D=128, bs=16, L=1, layer=0, num_blocks_org=64,
                                    dtype=np.float16, max_len=150)
        full = O.paged_attention_exact(c["q"], c["k_pools"], c["v_pools"], c["block_table"], c["seq_ids"],
                                       c["seq_lens"], 0, c["scale"], 64, 0)
        hk, hq = 4 // world, 8 // world
        ks = [p[:, :, rank * hk:(rank + 1) * hk] for p in c["k_pools"]]
        vs = [p[:, :, rank * hk:(rank + 1) * hk] for p in c["v_pools"]]
        part = O.paged_attention_exact(c["q"][:, rank * hq:(rank + 1) * hq], ks, vs, c["block_table"], c["seq_ids"],
                                       c["seq_lens"], 0, c["scale"], 64, 0)
        shard = torch.from_numpy(part.reshape(5, hq * 128))
        o_full = torch.zeros((world, 5, hq * 128), dtype=shard.dtype)
        dist.all_gather_into_tensor(o_full.view(world * 5, hq * 128), shard)
        view = o_full.permute(1, 0, 2).reshape(5, 8, 128).numpy()      # what the consumer reads
        np.testing.assert_allclose(view, full, rtol=1e-12, atol=1e-12)
        out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        out.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_logic():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results


def test_head_sharding_needs_divisible_heads():
    import pytest

    import bench
    with pytest.raises(ValueError):
        bench.shard_workload(bench.WORKLOADS["codellama-34b-gqa-decode-headshard"], 0, 3)


def test_head_shard_column_fails_soft_without_gpus():
    """The head-sharded side column of `bench.py --gpus N` runs as jobs of its own under a time limit.  Here, without a
    GPU, each job ends with an error: the column must come back as a record of "unavailable" entries, never raise, and
    refuse a rank count that does not divide the 8 KV heads without starting anything."""
    import bench
    assert "unavailable" in bench.headshard_column(3, K=1, W=1)
    if torch.cuda.is_available():
        return                                    # with GPUs present the jobs would really run: covered on the GPU box
    out = bench.headshard_column(2, K=1, W=1, layers=1, timeout_s=240)
    assert out["layers_run"] == 1 and out["layers_of_model"] == 48
    for name in ("codellama-34b-gqa-decode-headshard", "codellama-34b-gqa-decode-headshard-push"):
        assert "unavailable" in out[name] and "value" not in out[name], out[name]
