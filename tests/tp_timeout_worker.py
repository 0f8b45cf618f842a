"""Two ranks of the bounded-wait test; run under torchrun by test_tp_gpu.py:

    python -m torch.distributed.run --nproc-per-node 2 tests/tp_timeout_worker.py <out.json>

Both ranks run two rounds together over the peer-memory transport with the wait limit set to 50 ms.  Rank 1
then stops taking part — between rounds, with nothing of its own in flight — and only idles on the host.
Rank 0 (a) learns of it on the host through the roll call (StepRendezvous) before launching, and (b) launches
the round anyway to show the device-side path: its kernels' waits on rank 1 run out, raise the status bit and
return, the status read makes the error sticky and the next lcu_step fails with LCU_ERR_TIMEOUT.  The failure is
made on the host; no kernel faults, traps or spins without a limit."""
import ctypes as C
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]
import llama_cu_b200 as L  # noqa: E402
from llama_cu_b200.model import reduced  # noqa: E402
from tp_worker import make_comm  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device(dev))
    lib = L.load_library()
    comm = make_comm(lib, rank, world, dev)
    cfg = reduced(L.CONFIGS["tiny"], 2, 2048)
    w = L.synth_weights_numpy(cfg, 0)
    ctx = L.load_model(cfg, w, device=local, tp_rank=rank, tp_size=world, comm=comm, max_seqs=2)

    def gather(b):
        got = [None] * world
        dist.all_gather_object(got, b)
        return got
    ctx.p2p_connect(gather)
    ctx.set_wait_limit_us(50_000)
    store = dist.TCPStore("127.0.0.1", 29534, world, is_master=(rank == 0))
    roll = L.StepRendezvous(store, rank, world, timeout_s=1.0)
    stream = torch.cuda.Stream(device=dev)
    out = torch.zeros(2, 2, dtype=torch.int32, device=dev)
    seq = ctx.seq_create()
    prompt = np.arange(3, 12, dtype=np.uint32)
    res = {}
    with torch.cuda.stream(stream):
        roll.wait(0)
        ctx.step([(seq, 0, len(prompt))], prompt, out, stream=stream)     # round 0: prefill, both ranks
        roll.wait(1)
        ctx.step([(seq, len(prompt), 1)], np.array([5], np.uint32), out, stream=stream)  # round 1: decode, both ranks
        stream.synchronize()
        res["status_before"] = ctx.device_status(stream)
        dist.barrier()
        if rank == 0:
            # round 2: rank 1 has stopped.  (a) the host roll call reports it before anything is launched
            try:
                roll.wait(2)
                res["roll_call_error"] = (0, "")
            except L.LcuError as e:
                res["roll_call_error"] = (e.code, str(e))
            # (b) launched all the same, the kernels' bounded waits run out and the round returns
            t0 = time.perf_counter()
            ctx.step([(seq, len(prompt) + 1, 1)], np.array([7], np.uint32), out, stream=stream)
            stream.synchronize()
            res["seconds_for_the_abandoned_round"] = time.perf_counter() - t0
            res["status_after"] = ctx.device_status(stream)
            try:
                ctx.step([(seq, len(prompt) + 2, 1)], np.array([7], np.uint32), out, stream=stream)
                res["next_step_error"] = 0
            except L.LcuError as e:
                res["next_step_error"] = e.code
            ctx.reset_status()
            res["after_reset_status"] = ctx.device_status(stream)
            json.dump(res, open(out_path, "w"))
        # rank 1 idles on the host until rank 0 is done; neither has anything in flight when the contexts close
        torch.cuda.synchronize()
        dist.barrier()
    ctx.close()
    L.check(lib.lcu_comm_destroy(comm))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
