"""Spawn `world_size` CPU ranks over gloo on 127.0.0.1 and run a function in each."""
import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist

    torch.set_num_threads(2)   # ranks share the host's cores; oversubscription makes tiny ops crawl
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_distributed(fn, world_size: int = 2, args: tuple = (), timeout: float = 300.0):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn, args, errq)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    for p in procs:
        if p.is_alive():
            p.terminate()
            failed.append("timeout")
        elif p.exitcode != 0:
            failed.append(f"exit {p.exitcode}")
    msgs = []
    while not errq.empty():
        msgs.append("rank %d:\n%s" % errq.get())
    assert not failed, "distributed run failed: " + ", ".join(failed) + "\n" + "\n".join(msgs)
