"""Spawn N ranks on localhost (Gloo on CPU, or NCCL with one GPU per rank), run `fn(rank, world, *args)`
in each, collect results."""
import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fn, args, outdir, backend="gloo"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        if backend == "nccl":
            # The watchdog below may end a rank that hangs. A rank that dies while its memory is bound
            # to an NVLink multicast object can raise faults on its peers' GPUs, so the test ranks keep
            # NCCL off the in-switch (NVLS) path; nothing here measures NCCL's speed.
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        result = fn(rank, world, *args)
        torch.save({"ok": True, "result": result}, os.path.join(outdir, f"rank{rank}.pt"))
    except Exception:
        torch.save({"ok": False, "error": traceback.format_exc()}, os.path.join(outdir, f"rank{rank}.pt"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(world, fn, *args, timeout=240, backend="gloo"):
    port = _free_port()
    with tempfile.TemporaryDirectory() as outdir:
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, outdir, backend)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        hung = [r for r, p in enumerate(procs) if p.is_alive()]
        for r in hung:
            procs[r].terminate()
        if hung:
            # a rank that failed or died leaves its peers waiting in their next collective: say what
            # happened to the ranks that did finish, not only that the others never did
            notes = []
            for r in range(world):
                path = os.path.join(outdir, f"rank{r}.pt")
                if r in hung:
                    notes.append(f"rank {r}: still running")
                elif not os.path.exists(path):
                    notes.append(f"rank {r}: exited with code {procs[r].exitcode} and no result")
                else:
                    rec = torch.load(path, weights_only=False)
                    notes.append(f"rank {r}: finished" if rec["ok"] else f"rank {r} failed:\n{rec['error']}")
            raise RuntimeError(f"{len(hung)} rank(s) did not finish within {timeout}s (deadlock watchdog)\n" +
                               "\n".join(notes))
        out = []
        for r in range(world):
            path = os.path.join(outdir, f"rank{r}.pt")
            if not os.path.exists(path):
                raise RuntimeError(f"rank {r} produced no result (exit code {procs[r].exitcode})")
            rec = torch.load(path, weights_only=False)
            if not rec["ok"]:
                raise RuntimeError(f"rank {r} failed:\n{rec['error']}")
            out.append(rec["result"])
        return out
