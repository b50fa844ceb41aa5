"""GPT-2 small with pipeline x data parallelism: tied embedding / LM head across the first and last pipeline rank,
stage gradients all-reduced by the fused NVLink kernel as each stage finishes its backward.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/gpt2/train_gpt2_pp_dp.py --pp 4 --dp 2
"""
import argparse
import os

import torch
import torch.distributed as dist

from pippy_b200.models.gpt2 import GPT2Config
from pippy_b200.ops.gemm import set_sm_reserve
from pippy_b200.parallel.mesh import init_mesh
from pippy_b200.train import build_gpt2_pipeline

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp", type=int, default=4)
    ap.add_argument("--dp", type=int, default=2)
    ap.add_argument("--batch", type=int, default=64, help="global batch over all replicas")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--microbatches", type=int, default=16)
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    set_sm_reserve(8)
    mesh = init_mesh(pp_size=args.pp, dp_size=args.dp)
    cfg = GPT2Config.small()
    per_replica = args.batch // args.dp
    pipe = build_gpt2_pipeline(cfg, per_replica, args.seq, args.microbatches, device, schedule="1f1b",
                               group=mesh.pp_group, dp_group=mesh.dp_group)
    g = torch.Generator().manual_seed(mesh.dp_rank)
    ids = torch.randint(0, cfg.vocab_size, (per_replica, args.seq), generator=g).to(device)
    labels = torch.roll(ids, -1, 1)
    for step in range(args.steps):
        loss = pipe.train_step(ids if pipe.holds_first else None, labels if pipe.holds_last else None)
        if loss is not None and mesh.dp_rank == 0:
            print(f"step {step}: loss {loss.item():.4f}")
    dist.destroy_process_group()
