"""Run under torchrun with >= 2 GPUs (see test_gpu_multi.py): the head-sharded decode step with the
output pushed to every rank from the attention epilogue - each rank then waits for the other ranks'
"slice landed" words, a bounded wait - must equal, bit for bit, the same step followed by an NCCL
all-gather.  Then one launch in which the last rank does NOT signal: every rank's wait must run out
after its timeout, report exactly that rank in its status word and return; the next launch, signalled
by everyone again, must go through."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    base = dict(bench.WORKLOADS["codellama-34b-gqa-decode-headshard-push"])
    base.update(B=24, L=2)
    res = {}
    for push in (True, False):
        b = dict(base)
        b["push"] = push
        w = bench.shard_workload(b, rank, world)
        job = bench.DecodeJob(w, rank, growth_tokens=32, device=dev)
        job.step_resident()
        torch.cuda.synchronize()
        dist.barrier()
        res[push] = (job.o_full.clone() if push
                     else job.o_full.permute(0, 2, 1, 3).reshape(w["L"], w["B"], -1).clone())
    ok = torch.equal(res[True], res[False]) and bool(res[True].abs().sum() > 0)

    # ---- a rank that does not signal: the wait gives up, says who was missing, and the context stays usable
    import time
    import morphserve_b200 as mk
    w = bench.shard_workload(dict(base, push=True), rank, world)
    job = bench.DecodeJob(w, rank, growth_tokens=32, device=dev)
    job.step_resident()                                   # a regular step first: flags and epochs in use
    torch.cuda.synchronize()
    dist.barrier()
    ok = ok and int(job.ready_status.item()) == 0
    st = job.infer_state(job.seq_ids, job.lens_dev)
    outs = [p for p in job.peer_ptrs]

    def launch(signal):
        job.push_epoch += 1
        mk.paged_attention_push(job.q[0], job.k_cache, job.v_cache, [], [], job.bm.block_table, job.model_config,
                                job.engine_config, st, 0, outs, w["Hq_global"] * bench.D, w["head_offset"] * bench.D,
                                ready_ptrs=job.ready_ptrs if signal else None, epoch=job.push_epoch)

    status = torch.zeros((1,), dtype=torch.int32, device=dev)
    launch(signal=rank != world - 1)
    t0 = time.perf_counter()
    mk.wait_ready(job.ready, job.push_epoch, status, timeout_s=0.05)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    ok = ok and int(status.item()) == 1 << (world - 1) and 0.04 < waited < 1.0
    dist.barrier()                                        # host-side: everyone has seen its timeout
    status.zero_()
    launch(signal=True)
    mk.wait_ready(job.ready, job.push_epoch, status, timeout_s=1.0)
    torch.cuda.synchronize()
    ok = ok and int(status.item()) == 0
    dist.barrier()
    if rank == 0:
        print(f"wait without the last rank's signal: {waited * 1e3:.1f} ms, status {1 << (world - 1):#x}")
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if rank == 0:
        print("PUSH_EQUALS_ALLGATHER" if int(flag.item()) == 1 else "PUSH_DIFFERS")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
