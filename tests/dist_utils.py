"""Spawn helper for multi-process CPU (gloo) tests."""
import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _to_plain(x):
    """Tensors -> numpy so that results survive the child's exit (no shared-memory handles)."""
    import torch
    if torch.is_tensor(x):
        return ("__tensor__", x.detach().cpu().double().numpy() if x.is_floating_point() else x.detach().cpu().numpy())
    if isinstance(x, dict):
        return {k: _to_plain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_plain(v) for v in x)
    return x


def _from_plain(x):
    import torch
    if isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) and x[0] == "__tensor__":
        return torch.from_numpy(x[1])
    if isinstance(x, dict):
        return {k: _from_plain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_from_plain(v) for v in x)
    return x


def _entry(rank, world, port, fn, args, queue):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        import torch
        torch.set_num_threads(2)
        out = fn(rank, world, *args)
        queue.put((rank, "ok", _to_plain(out)))
    except Exception:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world: int, *args, timeout: float = 300.0):
    """Run fn(rank, world, *args) in `world` processes; returns the list of results by rank."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = queue.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = _from_plain(payload)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
    return [results[r] for r in range(world)]
