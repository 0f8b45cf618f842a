"""One rank of the tensor-parallel parity check; run under torchrun by test_tp_gpu.py:

    python -m torch.distributed.run --nproc-per-node N tests/tp_worker.py <spec.json> <out.npz> [nccl|p2p]

spec.json: {"name", "layers", "vocab", "steps", "lengths": [...], "ids": [[...]]} where `ids` are the
ORACLE's greedy ids.  Every rank loads its slice of the same seeded weights and all ranks run the same
rounds.  Phase 1 is teacher-forced (the oracle's ids go in on every rank) and rank 0 keeps the logits of
EVERY step; phase 2 repeats the run free-running with the sampled ids fed back on the device, which under
tensor parallelism also exercises the token broadcast from the lead rank.  With `p2p` the all-reduces and
the broadcast go over NVLink peer memory instead of NCCL.  Rank 0 writes logits, ids and the device status
word of every rank.
"""
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


def make_comm(lib, rank, world, dev):
    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        L.check(lib.lcu_comm_unique_id(uid.numpy().ctypes.data))
    uid = uid.to(dev)
    dist.broadcast(uid, 0)
    uid = uid.cpu().contiguous()
    comm = C.c_void_p()
    L.check(lib.lcu_comm_init_rank(uid.numpy().ctypes.data, rank, world, C.byref(comm)))
    return comm


def main():
    spec = json.load(open(sys.argv[1]))
    out_path = sys.argv[2]
    use_p2p = len(sys.argv) > 3 and sys.argv[3] == "p2p"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device(dev))
    lib = L.load_library()
    comm = make_comm(lib, rank, world, dev)

    for key, value in spec.get("tuning", {}).items():  # e.g. force the scatter form of the peer all-reduce
        L.set_tuning(key, value)
    cfg = reduced(L.CONFIGS[spec["name"]], spec["layers"], spec["vocab"])
    steps = spec["steps"]
    w = L.synth_weights_numpy(cfg, 0)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in spec["lengths"]]
    o_ids = spec["ids"]
    n = len(prompts)
    ctx = L.load_model(cfg, w, device=local, tp_rank=rank, tp_size=world, comm=comm, max_seqs=max(n, 1))
    # head_shard 0: the head runs on the lead rank alone and its logits cover the vocabulary; 1: arg-max rounds shard
    # the head, the lead rank's logits then cover only its own vocab / tp columns
    head_shard = int(spec.get("head_shard", 0))
    ctx.set_head_sharding(head_shard)
    v_cols = cfg.vocab // world if (head_shard and use_p2p and world > 1) else cfg.vocab
    if use_p2p and world > 1:
        def gather(b):
            got = [None] * world
            dist.all_gather_object(got, b)
            return got
        ctx.p2p_connect(gather)
        assert ctx.p2p_enabled
    stream = torch.cuda.Stream(device=dev)
    out = torch.zeros(n, 2, dtype=torch.int32, device=dev)
    logits = np.zeros((n, steps, cfg.vocab), np.float32)
    tf_ids = np.zeros((n, steps), np.int64)
    free_ids = np.zeros((n, steps), np.int64)

    with torch.cuda.stream(stream):
        # ---- phase 1: teacher-forced, logits of every step
        seqs = [ctx.seq_create() for _ in prompts]
        for i, p in enumerate(prompts):
            ctx.step([(seqs[i], 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            if rank == 0:
                logits[i, 0, :v_cols] = ctx.logits(1).reshape(-1)[:v_cols].float().cpu().numpy()
                tf_ids[i, 0] = int(out[0, 0].item())
        pos = [len(p) for p in prompts]
        for s in range(steps - 1):
            reqs = [(seqs[i], pos[i], 1) for i in range(n)]
            ctx.step(reqs, np.array([o_ids[i][s] for i in range(n)], np.uint32), out, stream=stream)
            stream.synchronize()
            if rank == 0:
                logits[:, s + 1, :v_cols] = ctx.logits(n).reshape(-1)[:n * v_cols].view(n, v_cols).float().cpu().numpy()
                tf_ids[:, s + 1] = out[:n, 0].cpu().numpy().view(np.uint32)
            for i in range(n):
                pos[i] += 1
        for sq in seqs:
            ctx.seq_free(sq)

        # ---- phase 2: free-running with device-side feedback (fast_map) and the token broadcast
        seqs = [ctx.seq_create() for _ in prompts]
        first = []
        for i, p in enumerate(prompts):
            ctx.step([(seqs[i], 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            t = out[0, :1].clone().to(torch.int64)
            dist.broadcast(t, 0)
            first.append(int(t.item()))
        free_ids[:, 0] = first
        pos = [len(p) for p in prompts]
        fm = np.array([[i, i] for i in range(n)], np.uint32)
        keep = []
        for s in range(steps - 1):
            reqs = [(seqs[i], pos[i], 1) for i in range(n)]
            toks = np.array(first, np.uint32) if s == 0 else np.zeros(n, np.uint32)
            ctx.step(reqs, toks, out, fast_map=None if s == 0 else fm, stream=stream)
            keep.append(out.clone())
            for i in range(n):
                pos[i] += 1
        stream.synchronize()
    torch.cuda.synchronize()
    launches = ctx.last_launch_count
    status = torch.tensor([ctx.device_status()], dtype=torch.int64, device=dev)
    all_status = [torch.zeros_like(status) for _ in range(world)]
    dist.all_gather(all_status, status)
    if rank == 0:
        for s, o in enumerate(keep):
            free_ids[:, s + 1] = o[:n, 0].cpu().numpy().view(np.uint32)
        np.savez(out_path, logits=logits, tf_ids=tf_ids, free_ids=free_ids, launches=launches,
                 status=np.array([int(t.item()) for t in all_status]), p2p=int(ctx.p2p_enabled), v_cols=v_cols)
    dist.barrier()
    ctx.close()
    L.check(lib.lcu_comm_destroy(comm))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
