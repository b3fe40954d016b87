"""Run under torchrun with >= 2 GPUs (see test_gpu_multi.py): the head-sharded decode step with the
output pushed to every rank from the attention epilogue must equal, bit for bit, the same step
followed by an NCCL all-gather."""
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
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if rank == 0:
        print("PUSH_EQUALS_ALLGATHER" if int(flag.item()) == 1 else "PUSH_DIFFERS")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
