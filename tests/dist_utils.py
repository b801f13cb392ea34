"""Run a function on N CPU ranks (gloo) as child processes and collect their results."""
import os
import tempfile
import traceback

import torch
import torch.multiprocessing as mp


def _entry(rank, world, store_path, fn, args, queue, backend="gloo"):
    try:
        os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), BAMBOO_QUIET="1",
                          MASTER_ADDR="127.0.0.1")
        torch.set_num_threads(1)
        import torch.distributed as dist
        store = dist.FileStore(store_path, world)
        if backend == "nccl":
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # a rank may leave the job in these tests
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, store=dist.PrefixStore("pg", store), rank=rank, world_size=world)
        out = fn(rank, world, dist.PrefixStore("engine", store), *args)
        queue.put((rank, "ok", out))
    except SystemExit as e:
        queue.put((rank, "exit", e.code))
    except BaseException:
        queue.put((rank, "error", traceback.format_exc()))


def run_ranks(fn, world, *args, timeout=240, backend="gloo"):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_entry, args=(r, world, path, fn, args, queue, backend)) for r in range(world)]
        for p in procs:
            p.start()
        results = {}
        try:
            import queue as _q
            import time as _t
            deadline = _t.monotonic() + timeout
            while len(results) < world and _t.monotonic() < deadline:
                try:
                    rank, status, payload = queue.get(timeout=0.5)
                    results[rank] = (status, payload)
                except _q.Empty:
                    # a rank that vanished without reporting (killed, os._exit) is recorded as such
                    for r, p in enumerate(procs):
                        if r not in results and not p.is_alive() and queue.empty():
                            results[r] = ("dead", p.exitcode)
            if len(results) < world:
                raise AssertionError(f"ranks {sorted(set(range(world)) - set(results))} did not finish in {timeout} s")
        finally:
            for p in procs:
                p.join(timeout=20)
                if p.is_alive():
                    p.kill()
    errors = [f"rank {rank} failed:\n{payload}" for rank, (status, payload) in sorted(results.items())
              if status == "error"]
    if errors:
        raise AssertionError("\n".join(errors))
    return results
