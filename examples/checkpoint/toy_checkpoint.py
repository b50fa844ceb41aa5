"""Periodic sharded checkpoints in the HuggingFace index layout and resume (reference examples/checkpoint/toy_model.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/checkpoint/toy_checkpoint.py
"""
import os
import tempfile

import torch
import torch.distributed as dist

import pippy_b200 as pp
from pippy_b200.checkpoint import CKPT_INDEX_JSON_FILENAME
from pippy_b200.models.mlp import ReadmeMLP

if __name__ == "__main__":
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    torch.manual_seed(0)
    model = ReadmeMLP()
    x, target = torch.randn(32, 512), torch.randn(32, 10)
    pipe = pp.pipeline(model, 4, (x,), split_policy=pp.split_into_equal_size(world))
    stage = pp.PipelineStage(pipe, rank, torch.device("cpu"))
    schedule = pp.Schedule1F1B(stage, 4, loss_fn=torch.nn.MSELoss(reduction="sum"))
    optimizer = torch.optim.SGD(stage.submod.parameters(), lr=0.01, momentum=0.9)
    root = os.environ.get("CKPT_DIR") or os.path.join(tempfile.gettempdir(), "pippy_b200_ckpt")
    for epoch in range(4):
        optimizer.zero_grad()
        if rank == 0:
            schedule.step(x)
        elif rank == world - 1:
            schedule.step(target=target, losses=[])
        else:
            schedule.step()
        optimizer.step()
        if (epoch + 1) % 2 == 0:
            pp.save_checkpoint(stage, os.path.join(root, str(epoch + 1)), optimizer)
    # resume: load the last checkpoint into a freshly split model
    fresh = pp.pipeline(ReadmeMLP(), 4, (x,), split_policy=pp.split_into_equal_size(world))
    sub = fresh.get_stage_module(rank)
    pp.load_checkpoint(sub, os.path.join(root, "4", CKPT_INDEX_JSON_FILENAME))
    for k, v in sub.state_dict().items():
        torch.testing.assert_close(v, stage.submod.state_dict()[k])
    if rank == 0:
        print("checkpoint round trip ok:", sorted(os.listdir(os.path.join(root, "4"))))
    dist.barrier()
    dist.destroy_process_group()
