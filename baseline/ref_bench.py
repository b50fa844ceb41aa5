"""Reference arm of bench.py: the UNMODIFIED reference (installed under baseline/_ref) driving a stock PyTorch
model through its own public API (ManualPipelineStage + Schedule1F1B / ScheduleInterleaved1F1B) with
torch.optim.AdamW, on the same config, metric and timing rules as the main arm."""
import json
import os
import sys
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)


class _Watchdog:
    """Ends the process if the reference makes no progress: its schedules block inside NCCL when ranks fall out of
    step, and a blocked rank would otherwise keep the whole job (and its GPUs) until an outer timeout."""

    def __init__(self, limit_s: float):
        import threading

        self.limit_s = limit_s
        self.last = None
        self.what = "start-up"
        self._stop = False
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self):
        import time

        self.last = time.time()
        self._thread.start()

    def kick(self, what: str):
        import time

        self.last = time.time()
        self.what = what

    def stop(self):
        self._stop = True

    def _run(self):
        import time

        while not self._stop:
            time.sleep(1.0)
            if time.time() - self.last > self.limit_s:
                _unavailable(f"the reference made no progress for {self.limit_s:.0f}s during {self.what} "
                             "(its schedule blocked inside NCCL); run abandoned")
                sys.stdout.flush()
                os._exit(0)


def main(args) -> None:
    ref_path = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_path, "pippy")):
        _unavailable("baseline/_ref/pippy is missing: the offline install of the reference was not done on this box")
        return
    if int(os.environ.get("WORLD_SIZE", "1")) >= 8:
        # Two attempts on 8 B200s completed no step: ScheduleInterleaved1F1B (killed by a 200 s timeout) and
        # Schedule1F1B (no progress for 150 s, ended by the watchdog below).
        # All of a rank's transfers share one NCCL stream there, so a send that waits for its peer blocks the
        # receive the peer is waiting for.  The reference's GPU code is not run again at this size.
        _unavailable("the reference's schedules (interleaved 1F1B and 1F1B) blocked inside NCCL on 8 GPUs on this "
                     "box and completed no step (two attempts); not run again")
        return
    try:
        _run(args, ref_path)
    except Exception as e:  # report instead of failing the driver
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"{type(e).__name__}: {e}")


def _run(args, ref_path) -> None:
    import warnings

    warnings.filterwarnings("ignore")
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    sys.path.insert(0, ref_path)
    sys.path.insert(0, HERE)
    from pippy.ManualPipelineStage import ManualPipelineStage
    from pippy.PipelineSchedule import Schedule1F1B, ScheduleInterleaved1F1B

    import ref_model
    from bench import ClockSampler  # nvidia-smi sampling only; no model/engine code

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl", device_id=device)

    if args.model == "llama2-7b":
        vocab, dim, n_layers, n_heads, ffn = 32000, 4096, 32, 32, 11008
        desc = "Llama-2-7B shape (32L, d4096, 32h, ffn 11008, vocab 32000)"
    else:
        vocab, dim, n_layers, n_heads, ffn = 32000, 2048, 8, 16, 5504
        desc = "llama-small (8L, d2048)"
    dtype = torch.bfloat16
    n_mb = args.microbatches
    mb = args.batch // n_mb
    # one rank cannot send to itself over NCCL, so a single GPU runs one stage under 1F1B; two or more GPUs
    # run the named interleaved schedule with `virtual` stages per rank
    virtual = args.virtual if world > 1 else 1
    num_stages = world * virtual
    per = n_layers // num_stages
    stages, params = [], []
    for k in range(virtual):
        s = rank + k * world
        torch.manual_seed(s)
        mod = ref_model.Stage(range(s * per, (s + 1) * per), s == 0, s == num_stages - 1, vocab, dim, n_heads, ffn,
                              1e-5, 10000.0, args.seq, dtype, device)
        inp = (torch.empty(mb, args.seq, dtype=torch.int64, device=device) if s == 0
               else torch.empty(mb, args.seq, dim, dtype=dtype, device=device))
        out = (torch.empty(mb, args.seq, vocab, dtype=dtype, device="meta") if s == num_stages - 1
               else torch.empty(mb, args.seq, dim, dtype=dtype, device="meta"))
        stages.append(ManualPipelineStage(mod, s, num_stages, device, n_mb, input_args=inp, output_args=out))
        params.extend(mod.parameters())
        del inp

    def loss_fn(logits, target):
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), ignore_index=-100) / n_mb

    if virtual == 1:
        sched = Schedule1F1B(stages[0], n_mb, loss_fn=loss_fn)
        sched_name = "1f1b (single stage)"
    else:
        sched = ScheduleInterleaved1F1B(stages, n_mb, loss_fn=loss_fn)
        sched_name = "interleaved_1f1b"
    opt = torch.optim.AdamW(params, lr=3e-4, weight_decay=0.1, fused=True)
    holds_first = rank == 0
    holds_last = (num_stages - 1) % world == rank

    g = torch.Generator().manual_seed(1234)
    host_ids = [torch.randint(0, vocab, (args.batch, args.seq), generator=g).pin_memory() for _ in range(2)]
    host_lbl = []
    for ids in host_ids:
        lbl = torch.roll(ids, -1, dims=1)
        lbl[:, -1] = -100
        host_lbl.append(lbl.pin_memory())
    dev_ids = [t.to(device) for t in host_ids]
    dev_lbl = [t.to(device) for t in host_lbl]

    def step(ids, lbl):
        losses = []
        if holds_first and holds_last:
            sched.step(ids, target=lbl, losses=losses)
        elif holds_first:
            sched.step(ids)
        elif holds_last:
            sched.step(target=lbl, losses=losses)
        else:
            sched.step()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return torch.stack(losses).sum() if losses else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(x, op):
        t = torch.tensor([x], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=op)
        return float(t.item())

    dog = _Watchdog(150.0)
    dog.start()
    loss = None
    for i in range(args.warmup):
        loss = step(dev_ids[i % 2], dev_lbl[i % 2])
        torch.cuda.synchronize()
        dog.kick(f"warm-up step {i + 1}")
    barrier()
    dog.kick("timed region")
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        loss = step(dev_ids[i % 2], dev_lbl[i % 2])
    ev1.record()
    barrier()
    ms_total = reduce(ev0.elapsed_time(ev1), dist.ReduceOp.MAX)
    dog.kick("end-to-end region")
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss.item()) if loss is not None else None

    e2e = None
    if not args.no_e2e:
        h2d = d2h = 0
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            ids = lbl = None
            if holds_first:
                ids = host_ids[i % 2].to(device, non_blocking=True)
                h2d += ids.numel() * ids.element_size()
            if holds_last:
                lbl = host_lbl[i % 2].to(device, non_blocking=True)
                h2d += lbl.numel() * lbl.element_size()
            l = step(ids, lbl)
            if l is not None:
                hl = l.float().cpu()
                d2h += hl.numel() * hl.element_size()
        e1.record()
        barrier()
        e2e_ms = reduce(e0.elapsed_time(e1), dist.ReduceOp.MAX)
        e2e = {
            "value": args.batch * args.seq * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": int(reduce(float(h2d), dist.ReduceOp.SUM) / args.steps),
            "d2h_bytes_per_step": int(reduce(float(d2h), dist.ReduceOp.SUM) / args.steps),
            "ms_per_step": e2e_ms / args.steps,
        }
    dog.stop()
    if rank == 0:
        value = args.batch * args.seq * args.steps / (ms_total * 1e-3)
        print(json.dumps({
            "metric": "tokens/sec (whole job, device-timed, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform token ids, labels shifted by one; random-init weights)", "impl": "reference",
            "config": {"model": desc, "global_batch": args.batch, "seq_len": args.seq, "microbatches": n_mb,
                       "parallelism": f"pp{world}" + (f"x{virtual}v" if virtual > 1 else ""), "schedule": sched_name,
                       "optimizer": "torch.optim.AdamW(fused=True) lr 3e-4",
                       "l2": "inputs larger than L2 (13.5 GB of weights stream every step)"},
            "final_loss": final_loss, "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
        }), flush=True)
    dist.destroy_process_group()
