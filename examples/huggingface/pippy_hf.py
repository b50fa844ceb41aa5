"""Pipeline any of the registered Hugging Face families: trace, cut into world-size stages, GPipe forward.

One driver for every family instead of one script each (reference examples/huggingface/pippy_bert.py ...
pippy_xlnet.py, all of which differ only in model class, layer path and inputs; those live in hf_utils.FAMILIES).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/huggingface/pippy_hf.py --model gpt2
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 4 examples/huggingface/pippy_hf.py --model bert --size base

The last rank checks the pipeline's output against the unsplit model on the same inputs.  With ``--train`` the
stages run forward and backward under 1F1B with a next-token / masked-token loss on the logits, and every parameter
gradient is compared with the unsplit model's; a weight tied across stages (GPT-2's ``wte`` / ``lm_head``, BERT's
word embeddings / decoder) is replicated per stage and the copies' gradients sum to the tied gradient (reference
test/hf_test.py:1047-1062 syncs them the same way).
"""
import argparse
import copy
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


def train_and_compare(args, pipe, stage, unsplit, config, ex_args, ex_kwargs, rank, world, device):
    vocab = config.vocab_size

    def loss_fn(out, target):
        return torch.nn.functional.cross_entropy(first_tensor(out).reshape(-1, vocab).float(), target.reshape(-1),
                                                 reduction="sum")

    labels = ex_args[0].clone()
    schedule = pp.Schedule1F1B(stage, args.chunks, loss_fn=loss_fn)
    losses = []
    dev_args = tuple(a.to(device) for a in ex_args)
    dev_kwargs = {k: v.to(device) for k, v in ex_kwargs.items()}
    if rank == 0:
        schedule.step(*dev_args, **dev_kwargs)
    elif rank == world - 1:
        schedule.step(target=labels.to(device), losses=losses)
    else:
        schedule.step()

    # the unsplit model, microbatch by microbatch (the traced program carries the microbatch shapes)
    mb = args.batch // args.chunks
    want_loss = 0.0
    for i in range(args.chunks):
        sl = slice(i * mb, (i + 1) * mb)
        out = unsplit(*(a[sl] for a in ex_args), **{k: v[sl] for k, v in ex_kwargs.items()})
        loss = loss_fn(out, labels[sl])
        loss.backward()
        want_loss += loss.item()
    if rank == world - 1:
        got_loss = sum(x.item() for x in losses)
        assert abs(got_loss - want_loss) <= 1e-3 * abs(want_loss), (got_loss, want_loss)
    want = {n: p.grad for n, p in unsplit.named_parameters(remove_duplicate=False)}
    mine = {n: (p.grad.detach().cpu() if p.grad is not None else None) for n, p in stage.submod.named_parameters()}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        copies = {}
        for group in pipe.replicated_params:
            key = tuple(sorted(group.items()))
            for sub, qualname in group.items():
                copies[(int(sub.split("_")[1]), qualname)] = key
        tied_sum, tied_name, checked = {}, {}, 0
        for st, part in enumerate(gathered):
            for name, grad in part.items():
                if grad is None:
                    continue
                key = copies.get((st, name))
                if key is not None:
                    tied_sum[key] = tied_sum.get(key, 0) + grad
                    tied_name[key] = name
                    continue
                torch.testing.assert_close(grad, want[name], rtol=1e-3, atol=1e-5, msg=f"stage {st} {name}")
                checked += 1
        for key, grad in tied_sum.items():
            torch.testing.assert_close(grad, want[tied_name[key]], rtol=1e-3, atol=1e-5, msg=f"tied {tied_name[key]}")
            checked += 1
        print(f"{args.model}: loss and {checked} parameter gradients ({len(tied_sum)} tied across stages) equal the "
              "unsplit model's")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2", choices=sorted(hf_utils.FAMILIES))
    ap.add_argument("--size", default="tiny", choices=["tiny", "base"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=16)
    ap.add_argument("--batches", type=int, default=1)
    ap.add_argument("--train", action="store_true", help="forward + backward with a loss; compare every gradient")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")

    torch.manual_seed(0)
    model, config, _ = hf_utils.build_model(args.model, args.size)
    unsplit = copy.deepcopy(model) if args.train else model  # the stages take over `model`'s parameters
    n_params = hf_utils.get_number_of_params(model)
    ex_args, ex_kwargs = hf_utils.generate_inputs(args.model, config, args.batch, args.seq_len)
    split = hf_utils.equal_layer_split(args.model, config, world)
    pipe = pp.pipeline(model, args.chunks, example_args=ex_args, example_kwargs=ex_kwargs, split_spec=split)
    assert pipe.num_stages == world, (pipe.num_stages, world)
    if rank == 0:
        print(f"{args.model}: {n_params / 1e6:.2f} M parameters in {pipe.num_stages} stages, "
              f"{hf_utils.calc_flop(config, args.batch, args.seq_len, n_params) / 1e9:.2f} GFLOP per batch")

    stage = pp.PipelineStage(pipe, rank, device)
    if args.train:
        train_and_compare(args, pipe, stage, unsplit, config, ex_args, ex_kwargs, rank, world, device)
        dist.barrier()
        dist.destroy_process_group()
        return
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
