"""Pipeline any of the registered Hugging Face families: trace, cut into world-size stages, GPipe forward.

One driver for every family instead of one script each (reference examples/huggingface/pippy_bert.py ...
pippy_xlnet.py, all of which differ only in model class, layer path and inputs; those live in hf_utils.FAMILIES).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/huggingface/pippy_hf.py --model gpt2
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 4 examples/huggingface/pippy_hf.py --model bert --size base

The last rank checks the pipeline's output against the unsplit model on the same inputs.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist
import torch.utils._pytree as pytree

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import hf_utils  # noqa: E402

import pippy_b200 as pp  # noqa: E402


def first_tensor(tree):
    if hasattr(tree, "to_tuple"):
        tree = tree.to_tuple()
    return next(x for x in pytree.tree_leaves(tree) if isinstance(x, torch.Tensor))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2", choices=sorted(hf_utils.FAMILIES))
    ap.add_argument("--size", default="tiny", choices=["tiny", "base"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=16)
    ap.add_argument("--batches", type=int, default=1)
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")

    torch.manual_seed(0)
    model, config, _ = hf_utils.build_model(args.model, args.size)
    n_params = hf_utils.get_number_of_params(model)
    ex_args, ex_kwargs = hf_utils.generate_inputs(args.model, config, args.batch, args.seq_len)
    split = hf_utils.equal_layer_split(args.model, config, world)
    pipe = pp.pipeline(model, args.chunks, example_args=ex_args, example_kwargs=ex_kwargs, split_spec=split)
    assert pipe.num_stages == world, (pipe.num_stages, world)
    if rank == 0:
        print(f"{args.model}: {n_params / 1e6:.2f} M parameters in {pipe.num_stages} stages, "
              f"{hf_utils.calc_flop(config, args.batch, args.seq_len, n_params) / 1e9:.2f} GFLOP per batch")

    stage = pp.PipelineStage(pipe, rank, device)
    schedule = pp.ScheduleGPipe(stage, args.chunks)
    dev_args = tuple(a.to(device) for a in ex_args)
    dev_kwargs = {k: v.to(device) for k, v in ex_kwargs.items()}
    for _ in range(args.batches):
        out = schedule.step(*dev_args, **dev_kwargs) if rank == 0 else schedule.step()

    if rank == world - 1:
        # The traced graph carries the microbatch shapes, so the unsplit model is run microbatch by microbatch too.
        mb = args.batch // args.chunks
        with torch.no_grad():
            ref = torch.cat([
                first_tensor(model(*(a[i * mb:(i + 1) * mb] for a in ex_args),
                                   **{k: v[i * mb:(i + 1) * mb] for k, v in ex_kwargs.items()}))
                for i in range(args.chunks)])
        torch.testing.assert_close(first_tensor(out).float().cpu(), ref, rtol=1e-3, atol=1e-3)
        print(f"{args.model}: pipeline output equals the unsplit model")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
