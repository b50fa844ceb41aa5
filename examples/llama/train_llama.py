"""Llama training under pipeline parallelism with the package's kernels (the benchmark's model at a chosen size).

    python examples/llama/train_llama.py --layers 8 --dim 2048                      # one GPU, two virtual stages
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 4 examples/llama/train_llama.py --schedule zero_bubble
"""
import argparse
import os

import torch
import torch.distributed as dist

from pippy_b200.models.llama import LlamaConfig
from pippy_b200.ops import _lib
from pippy_b200.ops.gemm import set_sm_reserve
from pippy_b200.train import build_llama_pipeline

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ffn", type=int, default=5504)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--schedule", default="interleaved_1f1b")
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        set_sm_reserve(8)
    cfg = LlamaConfig(vocab_size=32000, dim=args.dim, n_layers=args.layers, n_heads=args.heads, ffn_dim=args.ffn)
    pipe = build_llama_pipeline(cfg, args.batch, args.seq, args.microbatches, device, schedule=args.schedule,
                                virtual_stages=2, record_timing=True)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), device=device)
    labels = torch.roll(ids, -1, 1)
    for step in range(args.steps):
        loss = pipe.train_step(ids if pipe.holds_first else None, labels if pipe.holds_last else None)
        if loss is not None:
            print(f"step {step}: loss {loss.item():.4f}  bubble {pipe.schedule.last_step_stats['bubble']:.3f}")
    _lib.check_device_errors()
    if world > 1:
        dist.destroy_process_group()
