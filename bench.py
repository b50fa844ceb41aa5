#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s) of a Llama-2-7B-shaped decoder under pipeline parallelism.

Config (the one the baseline names): 32 layers, d_model 4096, 32 heads, SwiGLU 11008, vocab 32000, bf16,
global batch 64 x seq 4096, 32 microbatches, 2 virtual stages per rank, AdamW lr 3e-4, PP = number of GPUs.
Strong scaling: the global batch is fixed, so per-GPU work shrinks as GPUs are added.

  python bench.py --gpus 1 --steps 2 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
      bench.py --gpus 8 --steps 2 --warmup 3
  python bench.py --impl reference ...     # the unmodified reference (baseline/_ref) on the same config

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with inputs resident on the
device; ``e2e`` repeats the measurement through the public API with a pinned-host -> device copy of every step's
inputs and a device -> host read of the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_PUBLISHED = None  # the reference publishes no throughput number


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--schedule", default=None, help="interleaved_1f1b | zero_bubble | zbv | 1f1b | gpipe | looped_bfs")
    ap.add_argument("--config", default="llama7b-pp",
                    help="llama7b-pp (the headline config, PP = number of GPUs) | gpt2-pp4dp2 | llama13b-tp4pp2 | "
                         "mixtral-pp2ep4 (the other composed configs; on fewer than 8 GPUs the pipeline dimension "
                         "shrinks first)")
    ap.add_argument("--model", default="llama2-7b", help="llama2-7b | llama-small (for quick checks only)")
    ap.add_argument("--batch", type=int, default=None, help="global batch (default: the config's)")
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--microbatches", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (quick checks only)")
    ap.add_argument("--weigh-head", action="store_true",
                    help="gpt2 config: give the stage with the LM head fewer blocks (measured slower: launch-bound)")
    ap.add_argument("--inner", type=int, default=None,
                    help="size of the composed configs' second dimension (dp / tp / ep); the rest of the GPUs form the "
                         "pipeline (quick checks on fewer than 8 GPUs)")
    ap.add_argument("--virtual", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-retune", action="store_true",
                    help="keep the zero-bubble order of the fixed 2:3:2 cost guess instead of rebuilding it from the "
                         "per-stage times measured in the second warm-up step")
    ap.add_argument("--extra-in-flight", type=int, default=None,
                    help="upper limit of microbatches beyond the 1F1B depth that the cost-aware order may keep in "
                         "flight per rank (default: derived from the memory left after the first steps)")
    ap.add_argument("--p2p-gbs", type=float, default=20.0,
                    help="rate at which the cost-aware order assumes activations reach the next rank (the NCCL "
                         "point-to-point kernels are capped at two thread blocks per link, far below link speed; "
                         "measured arrival delays at 8 GPUs: median 1.3-2.5 ms, a tenth above 9 ms, so the assumption "
                         "is kept pessimistic: an order with slack costs under 1 % when transfers are fast and "
                         "avoids a stall per transfer when they are not)")
    ap.add_argument("--sm-reserve", type=int, default=None,
                    help="SMs kept out of the GEMM grid for communication kernels (default: 0 on 1 GPU, 8 otherwise)")
    args = ap.parse_args()
    defaults = {  # global batch, sequence length, microbatches per pipeline replica
        "llama7b-pp": (64, 4096, 32), "gpt2-pp4dp2": (64, 1024, 16), "llama13b-tp4pp2": (32, 4096, 16),
        "mixtral-pp2ep4": (32, 4096, 8),
    }
    if args.config not in defaults:
        raise SystemExit(f"unknown config {args.config}")
    b, sq, mbs = defaults[args.config]
    args.batch = b if args.batch is None else args.batch
    args.seq = sq if args.seq is None else args.seq
    args.microbatches = mbs if args.microbatches is None else args.microbatches
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)],
                stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # "under load": drop idle samples taken before the first kernel or after the last
        busy = [c for c, p in zip(sm, power) if p > 300] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


def model_config(name: str):
    from pippy_b200.models.llama import LlamaConfig

    if name == "llama2-7b":
        return LlamaConfig.llama2_7b(), "Llama-2-7B shape (32L, d4096, 32h, ffn 11008, vocab 32000)"
    if name == "llama-small":
        return LlamaConfig(vocab_size=32000, dim=2048, n_layers=8, n_heads=16, ffn_dim=5504), "llama-small (8L, d2048)"
    raise SystemExit(f"unknown model {name}")


def build_job(args, world: int, device):
    """Builds this rank's pipeline for ``args.config``.  Returns ``(pipe, info)``; ``info`` says which slice of the
    global batch this rank feeds, the model's training FLOPs per token and how the job is laid out."""
    import torch.distributed as dist

    from pippy_b200 import train
    from pippy_b200.parallel.mesh import init_mesh

    if args.config == "llama7b-pp":
        cfg, model_desc = model_config(args.model)
        if args.layers:
            cfg.n_layers = args.layers
        schedule = args.schedule or ("interleaved_1f1b" if world == 1 else "zero_bubble")
        virtual = 1 if schedule in ("gpipe", "1f1b") else args.virtual
        pipe = train.build_llama_pipeline(cfg, args.batch, args.seq, args.microbatches, device, schedule=schedule,
                                          virtual_stages=virtual, lr=3e-4, weight_decay=0.1)
        return pipe, dict(cfg=cfg, model=model_desc, schedule=schedule, virtual=virtual, replica=0, replicas=1,
                          parallelism=f"pp{world}" + (f"x{virtual}v" if virtual > 1 else ""),
                          flops_per_token=cfg.flops_per_token(args.seq), vocab=cfg.vocab_size)
    if world == 1:
        raise SystemExit(f"--config {args.config} composes parallel dimensions: run it on 2 or more GPUs")
    if args.config == "gpt2-pp4dp2":
        from pippy_b200.models.gpt2 import GPT2Config

        dp = args.inner or (2 if world % 2 == 0 else 1)
        pp = world // dp
        mesh = init_mesh(pp_size=pp, dp_size=dp)
        cfg = GPT2Config.small()
        if args.layers:
            cfg.n_layers = args.layers
        schedule = args.schedule or "1f1b"
        virtual = 1 if schedule in ("gpipe", "1f1b") else args.virtual
        pipe = train.build_gpt2_pipeline(cfg, args.batch // dp, args.seq, args.microbatches, device, schedule=schedule,
                                         virtual_stages=virtual, group=mesh.pp_group, dp_group=mesh.dp_group,
                                         balance=args.weigh_head)
        d, L, V = cfg.dim, cfg.n_layers, cfg.vocab_size
        flops = 6.0 * (L * 12 * d * d + V * d) + 3.0 * L * 2 * args.seq * d
        return pipe, dict(cfg=cfg, model=f"GPT-2 small ({L}L, d{d}, vocab {V}, tied embedding / LM head)",
                          schedule=schedule, virtual=virtual, replica=mesh.dp_rank, replicas=dp,
                          parallelism=f"pp{pp}xdp{dp}", flops_per_token=flops, vocab=V)
    if args.config == "llama13b-tp4pp2":
        from pippy_b200.models.llama import LlamaConfig

        tp = args.inner or (4 if world % 4 == 0 else 2)
        pp = world // tp
        mesh = init_mesh(pp_size=pp, tp_size=tp)
        cfg = LlamaConfig.llama2_13b()
        if args.layers:
            cfg.n_layers = args.layers
        schedule = args.schedule or "1f1b"
        pipe = train.build_llama_tp_pipeline(cfg, args.batch, args.seq, args.microbatches, device, schedule=schedule,
                                             pp_group=mesh.pp_group, tp_group=mesh.tp_group)
        return pipe, dict(cfg=cfg, model=f"Llama-2-13B shape ({cfg.n_layers}L, d5120, 40h, ffn 13824, vocab 32000)",
                          schedule=schedule, virtual=1, replica=0, replicas=1,
                          parallelism=f"tp{tp}xpp{pp} (sequence-parallel activations)",
                          flops_per_token=cfg.flops_per_token(args.seq), vocab=cfg.vocab_size)
    if args.config == "mixtral-pp2ep4":
        from pippy_b200.models.mixtral import MixtralConfig

        ep = args.inner or (4 if world % 4 == 0 else 2)
        pp = world // ep
        mesh = init_mesh(pp_size=pp, tp_size=ep)  # the mesh's fastest axis carries the experts
        cfg = MixtralConfig.mixtral_16l()
        if args.layers:
            cfg.n_layers = args.layers
        schedule = args.schedule or ("1f1b" if pp > 1 else "gpipe")
        pipe = train.build_mixtral_pipeline(cfg, args.batch // ep, args.seq, args.microbatches, device,
                                            schedule=schedule, pp_group=mesh.pp_group, ep_group=mesh.tp_group)
        d, hd = cfg.dim, cfg.head_dim
        attn_mm = d * (cfg.n_heads + 2 * cfg.kv_heads) * hd + d * d
        moe_mm = cfg.top_k * 3 * d * cfg.ffn_dim + d * cfg.n_experts
        flops = 6.0 * (cfg.n_layers * (attn_mm + moe_mm) + cfg.vocab_size * d) + 3.0 * cfg.n_layers * 2 * args.seq * d
        return pipe, dict(cfg=cfg, model=f"Mixtral shape ({cfg.n_layers}L, d4096, 32q/8kv heads, 8 experts of ffn 14336, "
                                         "top-2)",
                          schedule=schedule, virtual=1, replica=mesh.tp_rank, replicas=ep,
                          parallelism=f"pp{pp}xep{ep} (expert-parallel ranks are data-parallel for the dense layers)",
                          flops_per_token=flops, vocab=cfg.vocab_size)
    raise SystemExit(f"unknown config {args.config}")


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import ref_bench  # noqa: E402

        ref_bench.main(args)
        return

    import torch
    import torch.distributed as dist

    from pippy_b200.ops import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from pippy_b200.ops.gemm import set_sm_reserve

    sm_reserve = args.sm_reserve if args.sm_reserve is not None else (0 if world == 1 else 8)
    set_sm_reserve(sm_reserve)
    pipe, info = build_job(args, world, device)
    schedule, virtual, model_desc = info["schedule"], info["virtual"], info["model"]

    # synthetic data of the named shape: uniform token ids, labels = ids shifted by one; a data- (or expert-)
    # parallel replica feeds its own slice of the global batch
    g = torch.Generator().manual_seed(1234)
    n_sets = 2
    per_replica = args.batch // info["replicas"]
    rows = slice(info["replica"] * per_replica, (info["replica"] + 1) * per_replica)
    host_ids, host_lbl = [], []
    for _ in range(n_sets):
        ids = torch.randint(0, info["vocab"], (args.batch, args.seq), generator=g)
        lbl = torch.roll(ids, -1, dims=1)
        lbl[:, -1] = -100
        host_ids.append(ids[rows].contiguous().pin_memory())
        host_lbl.append(lbl[rows].contiguous().pin_memory())
    dev_ids = [t.to(device) for t in host_ids] if pipe.holds_first else [None] * n_sets
    dev_lbl = [t.to(device) for t in host_lbl] if pipe.holds_last else [None] * n_sets

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---------------------------------------------------------------- warm-up
    # The second warm-up step of a zero-bubble run is timed per action, and the order of the remaining steps is
    # rebuilt from those measured per-stage costs (the generator's default is a 2:3:2 guess with equal stages).
    loss = None
    retuned = None
    for i in range(args.warmup):
        measure = (i == 1 and world > 1 and hasattr(pipe.schedule, "retune_from_last_step")
                   and not args.no_retune and args.warmup >= 3)
        if measure:
            pipe.schedule.record_timing = True
        loss = pipe.train_step(dev_ids[i % n_sets], dev_lbl[i % n_sets])
        if measure:
            pipe.schedule.record_timing = False
            # Memory decides how many extra microbatches a rank may keep in flight: what the step needed beyond its
            # resident state, per microbatch-stage of the current depth, against what is left below 80 % of the GPU (at most 8 more).
            torch.cuda.synchronize()
            peak, resident = torch.cuda.max_memory_allocated(), torch.cuda.memory_allocated()
            depth = (virtual - 1) * world + (world - 1 - rank) + 1
            per_unit = max(peak - resident, 1) / depth
            room = 0.80 * torch.cuda.mem_get_info()[1] - torch.cuda.max_memory_reserved()  # reserved: with fragmentation
            allowed = int(min(8, max(0, room // per_unit)))
            extra = int(-max_over_ranks(-float(allowed)))  # the minimum over ranks: every rank builds the same order
            retuned = pipe.schedule.retune_from_last_step(p2p_bytes_per_s=args.p2p_gbs * 1e9,
                                                          max_extra_in_flight=max(extra, 2) if args.extra_in_flight
                                                          is None else args.extra_in_flight)
    barrier()
    _lib.check_device_errors()

    # ---------------------------------------------------------------- device-timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        loss = pipe.train_step(dev_ids[i % n_sets], dev_lbl[i % n_sets])
    ev1.record()
    barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    launches = sum_over_ranks(float(_lib.launch_count() - launches0))
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_device_errors()
    # the loss lives on the rank that holds the last stage; every rank learns it so that rank 0 can print it
    final_loss = max_over_ranks(float(loss.item()) if loss is not None else float("-inf"))

    # ---------------------------------------------------------------- end-to-end region (H2D inputs + D2H loss each step)
    e2e = None
    if not args.no_e2e:
        h2d = d2h = 0
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            ids = lbl = None
            if pipe.holds_first:
                ids = host_ids[i % n_sets].to(device, non_blocking=True)
                h2d += ids.numel() * ids.element_size()
            if pipe.holds_last:
                lbl = host_lbl[i % n_sets].to(device, non_blocking=True)
                h2d += lbl.numel() * lbl.element_size()
            l = pipe.train_step(ids, lbl)
            if l is not None:
                host_loss = l.float().cpu()  # device -> host read of the step's result
                d2h += host_loss.numel() * host_loss.element_size()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1))
        tokens = args.batch * args.seq * args.steps
        e2e = {
            "value": tokens / (e2e_ms * 1e-3),
            "unit": "tokens/s",
            "h2d_bytes_per_step": int(sum_over_ranks(float(h2d)) / args.steps),
            "d2h_bytes_per_step": int(sum_over_ranks(float(d2h)) / args.steps),
            "ms_per_step": e2e_ms / args.steps,
        }
        _lib.check_device_errors()

    # ---------------------------------------------------------------- one more step with per-action CUDA events
    # (outside both timed regions: the events cost a few hundred host calls per step)
    pipe.schedule.record_timing = True
    barrier()
    pipe.train_step(dev_ids[0], dev_lbl[0])
    barrier()
    pipe.schedule.record_timing = False
    stats = pipe.schedule.last_step_stats
    bubble = max_over_ranks(stats["bubble"])
    per_op = {k: max_over_ranks(stats["per_op_s"].get(k, 0.0)) for k in ("F", "B", "I", "W")}
    busy_min = -max_over_ranks(-stats["busy_s"])
    busy_max = max_over_ranks(stats["busy_s"])
    # every stage's mean F / B / I / W milliseconds per microbatch and every rank's busy time, for the record
    stage_ms, busy_per_rank = dict(stats["per_stage_op_mean_s"]), [stats["busy_s"]]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (stage_ms, stats["busy_s"]))
        stage_ms, busy_per_rank = {}, []
        for tbl, b in gathered:
            stage_ms.update(tbl)
            busy_per_rank.append(b)
    stage_ms = {k: round(v * 1e3, 3) for k, v in sorted(stage_ms.items(), key=lambda kv: (int(kv[0].split(":")[0]), kv[0]))}
    dump_dir = os.environ.get("PIPPY_TIMELINE_DIR")
    if dump_dir:
        os.makedirs(dump_dir, exist_ok=True)
        with open(os.path.join(dump_dir, f"timeline_rank{rank}.json"), "w") as f:
            json.dump(stats, f)

    # ---------------------------------------------------------------- same stages under interleaved 1F1B (the
    # schedule the reference arm runs), so that the runtime's and the schedule's share of a gain can be told apart
    like_for_like = None
    if args.config == "llama7b-pp" and world > 1 and schedule != "interleaved_1f1b" \
            and args.microbatches % world == 0 and virtual > 1 and schedule != "zbv":
        from pippy_b200.models.llama import causal_lm_loss
        from pippy_b200.schedules import ScheduleInterleaved1F1B

        main_schedule = pipe.schedule
        pipe.schedule = ScheduleInterleaved1F1B(pipe.stages, args.microbatches, loss_fn=causal_lm_loss)
        n_il = max(1, min(args.steps, 3))
        pipe.train_step(dev_ids[0], dev_lbl[0])  # builds the action list, untimed
        barrier()
        i0, i1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        i0.record()
        for i in range(n_il):
            pipe.train_step(dev_ids[i % n_sets], dev_lbl[i % n_sets])
        i1.record()
        barrier()
        il_ms = max_over_ranks(i0.elapsed_time(i1))
        like_for_like = {"value": args.batch * args.seq * n_il / (il_ms * 1e-3), "unit": "tokens/s",
                         "ms_per_step": il_ms / n_il, "steps": n_il}
        pipe.schedule = main_schedule
        _lib.check_device_errors()

    peak_mem = max_over_ranks(torch.cuda.max_memory_allocated() / 2**30)
    if rank == 0:
        tokens = args.batch * args.seq * args.steps
        value = tokens / (ms_total * 1e-3)
        ms_per_step = ms_total / args.steps
        tflops = info["flops_per_token"] * value / 1e12
        out = {
            "metric": "tokens/sec (whole job, device-timed, max over ranks)",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None if BASELINE_PUBLISHED is None else value / BASELINE_PUBLISHED,
            "dtype": "bf16",
            "data": "synthetic (uniform token ids, labels shifted by one; random-init weights)",
            "impl": "ours",
            "config": {
                "model": model_desc,
                "global_batch": args.batch,
                "seq_len": args.seq,
                "microbatches": args.microbatches,
                "name": args.config,
                "parallelism": info["parallelism"],
                "schedule": schedule,
                "sm_reserve": sm_reserve,
                "order": ("measured per-stage costs, up to %d extra microbatches in flight"
                          % pipe.schedule.max_extra_in_flight if retuned is not None else "generator defaults"),
                "optimizer": "AdamW lr 3e-4 (fused, fp32 moments, fp32 gradient accumulation)",
                "l2": "inputs larger than L2 (13.5 GB of weights and GBs of activations stream every step)",
            },
            "model_tflops_per_gpu": tflops / world,
            "final_loss": final_loss,
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "peak_mem_gb_max_rank": peak_mem,
        }
        out["bubble_measured"] = bubble
        out["per_op_s_max_rank"] = per_op
        out["busy_s_min_max_rank"] = [busy_min, busy_max]
        out["busy_s_per_rank"] = [round(b, 4) for b in busy_per_rank]
        out["stage_op_ms"] = stage_ms
        if like_for_like is not None:
            out["interleaved_1f1b"] = like_for_like
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
