"""Hugging Face Llama inference through the traced pipeline: greedy decoding on 2, 4 or 8 ranks.

Counterpart of the reference's examples/llama/pippy_llama.py (which prints the next token of eight prompts and
expects the same words on 2, 4 and 8 ranks, examples/llama/README.md:1-17).  With ``--weights DIR`` the model and
tokenizer are loaded from a local Hugging Face checkpoint directory (there is no network here, so the reference's
hub download of Llama-2-7b-chat is replaced by a path); without it a small random-init ``LlamaForCausalLM`` and
synthetic prompts are used.  Either way every rank checks nothing and the last rank prints the decoded tokens; with
``--check`` the last rank also runs the unsplit model and asserts that the pipeline chose the same tokens.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 4 examples/llama/pippy_llama.py --check --new-tokens 4

The model is cut at equal numbers of decoder layers per rank (``model.layers.{i * k}``: BEGINNING); the full batch of
eight prompts runs as four microbatches under GPipe, forward only.  Each new token is appended and the (left-padded)
batch goes through the pipeline again: the traced program has a fixed sequence length, so the prompts sit at the
right end of a window of ``--window`` positions and the window slides (no KV cache, as in the reference).
"""
import argparse
import os

import torch
import torch.distributed as dist

import pippy_b200 as pp

PROMPTS = ("How do you", "I like to", "Can I help", "You need to", "The weather is", "I found a", "What is your",
           "You are so")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default=None, help="local Hugging Face checkpoint directory (model + tokenizer)")
    ap.add_argument("--new-tokens", type=int, default=1)
    ap.add_argument("--window", type=int, default=16, help="sequence length the pipeline is traced for")
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--layers", type=int, default=8, help="decoder layers of the random-init model")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--cuda", type=int, default=int(torch.cuda.is_available()))
    args = ap.parse_args()

    from transformers import LlamaConfig, LlamaForCausalLM

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", rank % torch.cuda.device_count()) if args.cuda else torch.device("cpu")
    dist.init_process_group("nccl" if args.cuda else "gloo")

    tokenizer = None
    if args.weights:
        from transformers import AutoModelForCausalLM, AutoTokenizer

        llama = AutoModelForCausalLM.from_pretrained(args.weights, low_cpu_mem_usage=True)
        tokenizer = AutoTokenizer.from_pretrained(args.weights)
        tokenizer.pad_token = tokenizer.eos_token
        tokenizer.padding_side = "left"
        ids = tokenizer(list(PROMPTS), return_tensors="pt", padding="max_length", max_length=args.window)["input_ids"]
    else:
        torch.manual_seed(0)  # the same weights on every rank
        llama = LlamaForCausalLM(LlamaConfig(vocab_size=1000, hidden_size=128, intermediate_size=256,
                                             num_hidden_layers=args.layers, num_attention_heads=4,
                                             num_key_value_heads=4, max_position_embeddings=256))
        ids = torch.randint(3, 1000, (len(PROMPTS), args.window), generator=torch.Generator().manual_seed(1))
    llama.eval()
    llama.config.use_cache = False  # no KV cache object in the traced outputs: the window is re-run every step
    n_layers = llama.config.num_hidden_layers
    if n_layers % world != 0:
        raise SystemExit(f"{n_layers} decoder layers do not divide into {world} ranks")
    per_rank = n_layers // world
    split_spec = {f"model.layers.{i * per_rank}": pp.SplitPoint.BEGINNING for i in range(1, world)}

    mb = len(PROMPTS) // args.chunks
    with torch.no_grad():
        pipe = pp.pipeline(llama, args.chunks, example_args=(ids,), split_spec=split_spec)
    assert pipe.num_stages == world, (pipe.num_stages, world)
    stage = pp.PipelineStage(pipe, rank, device)
    schedule = pp.ScheduleGPipe(stage, args.chunks)

    batch = ids.to(device)
    chosen = []
    for _ in range(args.new_tokens):
        with torch.no_grad():
            out = schedule.step(batch) if rank == 0 else schedule.step()
        # the last rank picks the next token; everybody needs it to extend the batch
        nxt = torch.empty(len(PROMPTS), dtype=torch.long, device=device)
        if rank == world - 1:
            logits = out[0] if isinstance(out, (tuple, list)) else getattr(out, "logits", out)
            nxt = logits[:, -1, :].argmax(dim=-1)
        dist.broadcast(nxt, src=world - 1)
        chosen.append(nxt.cpu())
        batch = torch.cat([batch[:, 1:], nxt[:, None]], dim=1)  # slide the window
    chosen = torch.stack(chosen, dim=1)

    if rank == world - 1:
        if tokenizer is not None:
            print([tokenizer.decode(row) for row in chosen])
        else:
            print("next tokens:", chosen.tolist())
        if args.check:
            ref_batch, ref = ids.clone(), []
            with torch.no_grad():
                for _ in range(args.new_tokens):
                    n = llama(ref_batch).logits[:, -1, :].argmax(dim=-1)
                    ref.append(n)
                    ref_batch = torch.cat([ref_batch[:, 1:], n[:, None]], dim=1)
            ref = torch.stack(ref, dim=1)
            assert torch.equal(ref, chosen), (ref.tolist(), chosen.tolist())
            print(f"pipeline on {world} ranks chose the same {args.new_tokens} token(s) per prompt as the unsplit model")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
