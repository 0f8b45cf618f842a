"""One rank of the tensor-parallel parity check; run under torchrun by test_tp_gpu.py:

    python -m torch.distributed.run --nproc-per-node N tests/tp_worker.py <config> <layers> <vocab> <steps> <out.json> [p2p]

Every rank loads its slice of the same seeded weights, all ranks run the same rounds, rank 0
writes the greedy ids and the last round's logits.  With `p2p` the all-reduces and the token
broadcast go over NVLink peer memory instead of NCCL."""
import ctypes as C
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]
import llama_cu_b200 as L  # noqa: E402
from llama_cu_b200.model import reduced  # noqa: E402


def main():
    name, layers, vocab, steps, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    use_p2p = len(sys.argv) > 6 and sys.argv[6] == "p2p"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device(dev))
    lib = L.load_library()
    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        L.check(lib.lcu_comm_unique_id(uid.numpy().ctypes.data))
    uid = uid.to(dev)
    dist.broadcast(uid, 0)
    uid = uid.cpu().contiguous()
    comm = C.c_void_p()
    L.check(lib.lcu_comm_init_rank(uid.numpy().ctypes.data, rank, world, C.byref(comm)))

    cfg = reduced(L.CONFIGS[name], layers, vocab)
    w = L.synth_weights_numpy(cfg, 0)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in (5, 9, 40)]
    ctx = L.load_model(cfg, w, device=local, tp_rank=rank, tp_size=world, comm=comm)
    if use_p2p and world > 1:
        def gather(b):
            got = [None] * world
            dist.all_gather_object(got, b)
            return got
        ctx.p2p_connect(gather)
        assert ctx.p2p_enabled
    stream = torch.cuda.Stream(device=dev)
    n = len(prompts)
    out = torch.zeros(n, 2, dtype=torch.int32, device=dev)
    seqs = [ctx.seq_create() for _ in prompts]
    ids = [[] for _ in prompts]
    with torch.cuda.stream(stream):
        for i, p in enumerate(prompts):
            ctx.step([(seqs[i], 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            t = out[0, :1].clone().to(torch.int64)
            dist.broadcast(t, 0)
            ids[i].append(int(t.item()))
        pos = [len(p) for p in prompts]
        fm = np.array([[i, i] for i in range(n)], np.uint32)
        keep = []
        for s in range(steps - 1):
            reqs = [(seqs[i], pos[i], 1) for i in range(n)]
            toks = np.array([ids[i][0] for i in range(n)], np.uint32) if s == 0 else np.zeros(n, np.uint32)
            ctx.step(reqs, toks, out, fast_map=None if s == 0 else fm, stream=stream)
            keep.append(out.clone())
            for i in range(n):
                pos[i] += 1
        stream.synchronize()
    torch.cuda.synchronize()
    if rank == 0:
        for o in keep:
            h = o.cpu().numpy().view(np.uint32)
            for i in range(n):
                ids[i].append(int(h[i, 0]))
        lg = ctx.logits(n).float().cpu().numpy()
        json.dump({"ids": ids, "logits_last": lg.tolist(), "launches": ctx.last_launch_count,
                   "status": ctx.device_status(), "p2p": ctx.p2p_enabled}, open(out_path, "w"))
    assert ctx.device_status() == 0, f"rank {rank}: device status {ctx.device_status()}"
    dist.barrier()
    ctx.close()
    L.check(lib.lcu_comm_destroy(comm))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
