"""Spawns N ranks on this host (gloo on CPU, nccl on GPUs) and re-raises the first failure in the parent."""
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world_size, fn, init_file, backend, args, err_queue, timeout_s):
    try:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime

        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(
            backend, init_method=f"file://{init_file}", rank=rank, world_size=world_size,
            timeout=datetime.timedelta(seconds=timeout_s),
        )
        try:
            fn(rank, world_size, *args)
        finally:
            dist.destroy_process_group()
    except Exception:
        err_queue.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world_size, *args, backend="gloo", timeout_s=120):
    ctx = mp.get_context("spawn")
    err_queue = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rdzv")
        procs = []
        for rank in range(world_size):
            p = ctx.Process(target=_worker, args=(rank, world_size, fn, init_file, backend, args, err_queue, timeout_s))
            p.start()
            procs.append(p)
        for p in procs:
            p.join(timeout_s + 30)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:
            p.kill()
        errors = []
        while not err_queue.empty():
            errors.append(err_queue.get())
        if errors:
            rank, tb = errors[0]
            raise AssertionError(f"rank {rank} failed:\n{tb}")
        if hung:
            raise AssertionError(f"{len(hung)} rank(s) did not finish within {timeout_s}s")
        bad = [p.exitcode for p in procs if p.exitcode != 0]
        if bad:
            raise AssertionError(f"rank exit codes: {[p.exitcode for p in procs]}")
