"""Reference arm of bench.py: the reference's own runtime driving a stock PyTorch model with torch.optim.AdamW,
on the same config, metric and timing rules as the main arm.

Two systems answer to "the reference", and the printed line names which one ran (``reference_system``):

* ``pippy``: the UNMODIFIED reference installed under baseline/_ref, through its public API
  (ManualPipelineStage + Schedule1F1B on one GPU, ScheduleInterleaved1F1B on two).
* ``torch.distributed.pipelining``: the form the reference migrated into (its README says so), as shipped with the
  installed torch: PipelineStage + ScheduleInterleaved1F1B, stock code path.  It runs where the reference's own
  interleaved schedule completes no step (four or more ranks; see ``_pippy_blocks``).

Both drive the same ``ref_model.Stage`` slices, the same optimizer and the same watchdog.  The composed configs
(pipeline x data / tensor / expert parallelism) have their arms in ``ref_composed.py``."""
import json
import os
import sys
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)


class _Watchdog:
    """Ends the process when the device stops completing steps, so that a blocked rank cannot keep the whole job
    (and its GPUs) until an outer timeout.

    Progress is what the DEVICE finished, not what the host queued: after every step the caller records a CUDA event
    (``mark``) and this thread polls ``event.query()``.  The limit starts generous (first step: context, NCCL
    communicators, allocator warm-up) and is then derived from the measured step time (``set_step_time``)."""

    def __init__(self, startup_limit_s: float, device=None):
        import threading

        self.limit_s = startup_limit_s
        self.device = device
        self.last = None
        self.what = "start-up"
        self._events = []  # (event, label) recorded but not yet seen complete
        self._lock = threading.Lock()
        self._stop = False
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self):
        import time

        self.last = time.time()
        self._thread.start()

    def mark(self, what: str):
        """Records an event on the current stream; the watchdog counts it as progress once the device reaches it."""
        import torch

        ev = torch.cuda.Event()
        ev.record()
        with self._lock:
            self._events.append((ev, what))

    def set_step_time(self, step_s: float, factor: float = 5.0, floor_s: float = 60.0):
        self.limit_s = max(floor_s, factor * step_s)

    def stop(self):
        self._stop = True

    def _run(self):
        import time

        import torch

        if self.device is not None:
            torch.cuda.set_device(self.device)
        while not self._stop:
            time.sleep(0.5)
            with self._lock:
                while self._events and self._events[0][0].query():
                    _, self.what = self._events.pop(0)
                    self.last = time.time()
            if time.time() - self.last > self.limit_s:
                _unavailable(f"no step completed on the device for {self.limit_s:.0f}s after {self.what}; "
                             "run abandoned by the arm's watchdog")
                sys.stdout.flush()
                os._exit(0)


def _pippy_blocks(world: int) -> bool:
    """The reference's ScheduleInterleaved1F1B completed no step at 4 ranks (no progress in the first step for
    150 s, all four GPUs spinning) nor at 8 (ended by a 200 s timeout; its Schedule1F1B made no progress at 8
    either).  Each rank issues its transfers as coalesced NCCL groups on one communicator, in program order, and in
    its 1F1B phase one group mixes a step's receives with the previous step's sends to up to four peers
    (pippy/PipelineSchedule.py:706-742); its own comment says the groups "need to be aligned to prevent a hang" and
    its 4-GPU test is disabled as "not working" (test/test_pipeline_schedule.py:333-336).  A replay of the groups
    per rank shows that the order completes only if a send may finish before its receiver's matching group reaches
    the head of that rank's queue, i.e. it relies on how much NCCL buffers per connection; with 64 MiB activations
    that held at 2 ranks and not at 4 or 8.  That code is not run again at those sizes."""
    return world >= 4


def main(args) -> None:
    ref_path = os.path.join(HERE, "_ref")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if getattr(args, "config", "llama7b-pp") != "llama7b-pp":
        # the composed configs: the pipeline runtime the reference migrated into plus the stock PyTorch library for
        # the second dimension (DDP, DTensor tensor parallelism, all_to_all_single experts)
        try:
            import ref_composed

            ref_composed.run(args, _Watchdog, _unavailable)
        except Exception as e:
            traceback.print_exc(file=sys.stderr)
            _unavailable(f"{type(e).__name__}: {e}")
        return
    system = os.environ.get("PIPPY_REF_SYSTEM") or ("torch.distributed.pipelining" if _pippy_blocks(world) else "pippy")
    if system == "pippy":
        if not os.path.isdir(os.path.join(ref_path, "pippy")):
            _unavailable("baseline/_ref/pippy is missing: the offline install of the reference was not done on this box")
            return
        if _pippy_blocks(world):
            _unavailable("the reference's own schedules blocked inside NCCL at 4 and 8 ranks on this pool and are not "
                         "run again at those sizes")
            return
    try:
        _run(args, ref_path, system)
    except Exception as e:  # report instead of failing the driver
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"{type(e).__name__}: {e}")


def _run(args, ref_path, system: str) -> None:
    import time
    import warnings

    warnings.filterwarnings("ignore")
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    sys.path.insert(0, HERE)
    if system == "pippy":
        sys.path.insert(0, ref_path)
        from pippy.ManualPipelineStage import ManualPipelineStage
        from pippy.PipelineSchedule import Schedule1F1B, ScheduleInterleaved1F1B
    else:
        from torch.distributed.pipelining import PipelineStage, Schedule1F1B, ScheduleInterleaved1F1B

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
        if system == "pippy":
            inp = (torch.empty(mb, args.seq, dtype=torch.int64, device=device) if s == 0
                   else torch.empty(mb, args.seq, dim, dtype=dtype, device=device))
            out = (torch.empty(mb, args.seq, vocab, dtype=dtype, device="meta") if s == num_stages - 1
                   else torch.empty(mb, args.seq, dim, dtype=dtype, device="meta"))
            stages.append(ManualPipelineStage(mod, s, num_stages, device, n_mb, input_args=inp, output_args=out))
            del inp
        else:
            inp = (torch.empty(mb, args.seq, dtype=torch.int64, device="meta") if s == 0
                   else torch.empty(mb, args.seq, dim, dtype=dtype, device="meta"))
            out = (torch.empty(mb, args.seq, vocab, dtype=dtype, device="meta") if s == num_stages - 1
                   else torch.empty(mb, args.seq, dim, dtype=dtype, device="meta"))
            stages.append(PipelineStage(mod, s, num_stages, device, input_args=(inp,), output_args=(out,)))
        params.extend(mod.parameters())

    def loss_fn(logits, target):
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), ignore_index=-100) / n_mb

    # the loss already carries 1/n_mb, so upstream's own gradient scaling stays off
    extra = {} if system == "pippy" else {"scale_grads": False}
    if virtual == 1:
        sched = Schedule1F1B(stages[0], n_mb, loss_fn=loss_fn, **extra)
        sched_name = "1f1b (single stage)"
    else:
        sched = ScheduleInterleaved1F1B(stages, n_mb, loss_fn=loss_fn, **extra)
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

    dog = _Watchdog(300.0, device)
    dog.start()
    loss = None
    for i in range(args.warmup):
        t0 = time.time()
        loss = step(dev_ids[i % 2], dev_lbl[i % 2])
        dog.mark(f"warm-up step {i + 1}")
        torch.cuda.synchronize()
        if i > 0 or args.warmup == 1:
            dog.set_step_time(time.time() - t0)
    barrier()
    dog.mark("warm-up")
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        loss = step(dev_ids[i % 2], dev_lbl[i % 2])
        dog.mark(f"timed step {i + 1}")
    ev1.record()
    barrier()
    ms_total = reduce(ev0.elapsed_time(ev1), dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    # the loss lives on the rank that holds the last stage; every rank learns it so that rank 0 can print it
    final_loss = reduce(float(loss.item()) if loss is not None else float("-inf"), dist.ReduceOp.MAX)

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
            dog.mark(f"end-to-end step {i + 1}")
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
            "reference_system": system,
            "config": {"model": desc, "global_batch": args.batch, "seq_len": args.seq, "microbatches": n_mb,
                       "parallelism": f"pp{world}" + (f"x{virtual}v" if virtual > 1 else ""), "schedule": sched_name,
                       "optimizer": "torch.optim.AdamW(fused=True) lr 3e-4",
                       "l2": "inputs larger than L2 (13.5 GB of weights stream every step)"},
            "final_loss": final_loss, "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
        }), flush=True)
    dist.destroy_process_group()
