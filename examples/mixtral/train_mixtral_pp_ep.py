"""Mixtral-shaped sparse MoE with pipeline x expert parallelism (fused dispatch / combine over NVLink).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/mixtral/train_mixtral_pp_ep.py --pp 2 --ep 4
"""
import argparse
import os

import torch
import torch.distributed as dist

from pippy_b200.models.mixtral import MixtralConfig
from pippy_b200.ops.gemm import set_sm_reserve
from pippy_b200.parallel.mesh import init_mesh
from pippy_b200.train import build_mixtral_pipeline

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--ep", type=int, default=4)
    ap.add_argument("--batch", type=int, default=32, help="global batch over all expert-parallel ranks")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    set_sm_reserve(8)
    mesh = init_mesh(pp_size=args.pp, dp_size=1, tp_size=args.ep)  # the "tp" axis of the mesh carries the experts
    cfg = MixtralConfig.mixtral_16l()
    cfg.n_layers = args.layers
    per_rank = args.batch // args.ep
    pipe = build_mixtral_pipeline(cfg, per_rank, args.seq, args.microbatches, device, schedule="1f1b",
                                  pp_group=mesh.pp_group, ep_group=mesh.tp_group)
    g = torch.Generator().manual_seed(mesh.tp_rank)
    ids = torch.randint(0, cfg.vocab_size, (per_rank, args.seq), generator=g).to(device)
    labels = torch.roll(ids, -1, 1)
    for step in range(args.steps):
        loss = pipe.train_step(ids if pipe.holds_first else None, labels if pipe.holds_last else None)
        if loss is not None and mesh.tp_rank == 0:
            print(f"step {step}: loss {loss.item():.4f}")
    dist.destroy_process_group()
