"""Llama with tensor (+ sequence) x pipeline parallelism: fused all-gather->GEMM and GEMM->reduce-scatter inside each
stage, token shards shipped between stages (the capability the reference sketches in examples/tp+pp/pippy_tp.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/tp_pp/llama_tp_pp.py --tp 4 --pp 2
"""
import argparse
import os

import torch
import torch.distributed as dist

import pippy_b200 as pp
from pippy_b200.models.llama import LlamaConfig, causal_lm_loss
from pippy_b200.models.llama_tp import build_tp_llama_stage
from pippy_b200.ops.gemm import set_sm_reserve
from pippy_b200.optim import FlatParams, FusedAdamW
from pippy_b200.parallel.mesh import init_mesh
from pippy_b200.parallel.tp import TPContext

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=4)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--microbatches", type=int, default=16)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    set_sm_reserve(8)
    mesh = init_mesh(pp_size=args.pp, tp_size=args.tp)
    cfg = LlamaConfig.llama2_13b()
    cfg.n_layers = args.layers
    mb = args.batch // args.microbatches
    rows = mb * args.seq // args.tp
    tp = TPContext(mesh.tp_group, max_rows=rows, max_cols=max(cfg.dim, 2 * cfg.ffn_dim // args.tp), device=device)
    torch.manual_seed(mesh.pp_rank * 100 + mesh.tp_rank)
    module = build_tp_llama_stage(cfg, mesh.pp_rank, args.pp, tp, args.tp, mesh.tp_rank, mb, args.seq, device=device)
    first, last = mesh.pp_rank == 0, mesh.pp_rank == args.pp - 1
    inp = (torch.empty(mb, args.seq, dtype=torch.int64, device="meta") if first
           else torch.empty(rows, cfg.dim, dtype=torch.bfloat16, device="meta"))
    out = (torch.empty(mb, args.seq, cfg.vocab_size, dtype=torch.bfloat16, device="meta") if last
           else torch.empty(rows, cfg.dim, dtype=torch.bfloat16, device="meta"))
    stage = pp.ManualPipelineStage(module, mesh.pp_rank, args.pp, device, args.microbatches, input_args=inp,
                                   output_args=out, group=mesh.pp_group)
    schedule = pp.Schedule1F1B(stage, args.microbatches, loss_fn=causal_lm_loss)
    flat = FlatParams(module.parameters())
    opt = FusedAdamW(flat, lr=3e-4)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), generator=torch.Generator().manual_seed(0)).to(device)
    labels = torch.roll(ids, -1, 1)
    for step in range(args.steps):
        losses = []
        if first and last:
            schedule.step(ids, target=labels, losses=losses)
        elif first:
            schedule.step(ids)
        elif last:
            schedule.step(target=labels, losses=losses)
        else:
            schedule.step()
        opt.step(grad_scale=1.0 / args.microbatches, zero_grad=True)
        if losses and mesh.tp_rank == 0:
            print(f"step {step}: loss {torch.stack(losses).mean().item():.4f}")
    dist.destroy_process_group()
