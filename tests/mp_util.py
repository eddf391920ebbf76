"""Run one function as `world` spawned processes and collect one result per rank.

A worker that raises sends its traceback back instead of a result; whatever happens, every process that is still
alive when the collection ends is terminated (then killed), so a rank blocked in a collective whose peer is gone
does not outlive the test holding a GPU.
"""
import os
import queue
import traceback


def _entry(fn, rank, world, port, args, out_q):
    try:
        out_q.put((rank, "ok", fn(rank, world, port, *args)))
    except BaseException:  # noqa: BLE001 - the parent re-raises with this text
        out_q.put((rank, "error", traceback.format_exc()))


def run_ranks(fn, world, args=(), timeout=300, port_base=29500):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = port_base + (os.getpid() * 7 + world) % 2000
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, tuple(args), q)) for r in range(world)]
    results = {}
    try:
        for p in procs:
            p.start()
        for _ in procs:
            try:
                rank, status, payload = q.get(timeout=timeout)
            except queue.Empty:
                raise AssertionError(f"no answer from {world - len(results)} of {world} ranks within {timeout} s")
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0, f"a rank exited with code {p.exitcode}"
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    return [results[r] for r in range(world)]
