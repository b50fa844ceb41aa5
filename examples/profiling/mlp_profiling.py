"""torch.profiler chrome traces per rank plus the schedule's own per-action timing and bubble
(reference examples/profiling/mlp_profiling.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/profiling/mlp_profiling.py --out traces
"""
import argparse
import os
import tempfile

import torch
import torch.distributed as dist
from torch.profiler import ProfilerActivity, profile

import pippy_b200 as pp
from pippy_b200.models.mlp import ReadmeMLP

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.environ.get("TRACE_DIR"),
                    help="directory for the trace files (default: a fresh directory under the system temp dir)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    torch.manual_seed(0)
    x, target = torch.randn(64, 512), torch.randn(64, 10)
    pipe = pp.pipeline(ReadmeMLP(), 8, (x,), split_policy=pp.split_into_equal_size(world))
    stage = pp.PipelineStage(pipe, rank, torch.device("cpu"))
    schedule = pp.Schedule1F1B(stage, 8, loss_fn=torch.nn.MSELoss(reduction="sum"), record_timing=True)
    with profile(activities=[ProfilerActivity.CPU]) as prof:
        for _ in range(5):
            if rank == 0:
                schedule.step(x)
            elif rank == world - 1:
                schedule.step(target=target, losses=[])
            else:
                schedule.step()
    out = args.out
    if out is None:
        # every rank must write into the same directory: rank 0 makes it and tells the others
        box = [tempfile.mkdtemp(prefix="pippy_b200_traces_") if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        out = box[0]
    os.makedirs(out, exist_ok=True)
    prof.export_chrome_trace(os.path.join(out, f"pipeline_rank{rank}.json"))
    stats = schedule.last_step_stats
    print(f"rank {rank}: bubble {stats['bubble']:.3f}, per-op seconds {stats['per_op_s']}")
    # every rank's measured actions of the last step on one time axis (open in chrome://tracing or Perfetto)
    from pippy_b200.schedules import gather_measured_trace

    gather_measured_trace(schedule, os.path.join(out, "pipeline_schedule.json"))
    if rank == 0:
        print(f"traces written to {out}")
    dist.barrier()
    dist.destroy_process_group()
