"""World-size-2 `gloo` test (CPU) of the host-side tensor-parallel logic: each rank takes its
slice of every weight with `tp_slice_numpy` (the cut `TPAction::move_data` makes,
llama.cu/src/load/mod.rs:86-99), computes its part of one transformer block with the oracle's
operators, the partial sums are all-reduced, and the result must equal the unsharded block."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import llama_cu_b200 as L
    from llama_cu_b200.model import ModelConfig
    from oracle import oracle as O
    cfg = ModelConfig("tp", 1, 128, 4, 2, 64, 256, 64, 1e4, nctx=32)
    w = L.synth_weights_numpy(cfg, 3)
    f = {k: O.to_f32(v, 0).reshape(v.shape) for k, v in w.items()}
    dt = 2  # f32: sharding must be exact up to summation order
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, cfg.d)).astype(np.float32)
    pos = np.array([0, 1, 2], np.uint32)
    sin, cos = O.build_sin_cos(cfg.nctx, cfg.dh, cfg.theta)

    def block(nh, nkvh, di, qkv, o, gu, down, add_residual):
        h = O.rms_norm(x, f[(0, L.W_ATTN_NORM)], cfg.eps, dt)
        y = O.linear(h, qkv, None, dt)
        qd, kvd = nh * cfg.dh, nkvh * cfg.dh
        q = O.rope(y[:, :qd], nh, cfg.dh, pos, sin, cos, dt)
        k = O.rope(y[:, qd:qd + kvd], nkvh, cfg.dh, pos, sin, cos, dt)
        v = y[:, qd + kvd:]
        att = O.attention(q, k, v, nh, nkvh, cfg.dh, 0, dt)
        return O.linear(att, o, x if add_residual else None, dt)

    full = block(cfg.nh, cfg.nkvh, cfg.di, f[(0, L.W_QKV)], f[(0, L.W_O)], None, None, True)
    sl = {k: L.tp_slice_numpy(cfg, k, f[(0, k)], rank, world) for k in (L.W_QKV, L.W_O, L.W_GATE_UP, L.W_DOWN)}
    part = block(cfg.nh // world, cfg.nkvh // world, cfg.di // world, sl[L.W_QKV], sl[L.W_O], None, None, rank == 0)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    err_attn = float(np.abs(t.numpy() - full).max())

    # FFN: gate|up rows and down columns
    h2 = O.rms_norm(full, f[(0, L.W_FFN_NORM)], cfg.eps, dt)
    gu = O.linear(h2, f[(0, L.W_GATE_UP)], None, dt)
    want = O.linear(O.swiglu(gu[:, :cfg.di], gu[:, cfg.di:], dt), f[(0, L.W_DOWN)], full, dt)
    di_l = cfg.di // world
    gul = O.linear(h2, sl[L.W_GATE_UP], None, dt)
    part = O.linear(O.swiglu(gul[:, :di_l], gul[:, di_l:], dt), sl[L.W_DOWN], full if rank == 0 else None, dt)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    err_ffn = float(np.abs(t.numpy() - want).max())
    shapes_ok = (sl[L.W_QKV].shape == ((cfg.nh + 2 * cfg.nkvh) // world * cfg.dh, cfg.d)
                 and sl[L.W_O].shape == (cfg.d, cfg.nh // world * cfg.dh)
                 and sl[L.W_GATE_UP].shape == (2 * di_l, cfg.d) and sl[L.W_DOWN].shape == (cfg.d, di_l))
    ret[rank] = (err_attn, err_ffn, shapes_ok)
    dist.destroy_process_group()


def test_tp_sharding_plan_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, 29611, ret), nprocs=world, join=True)
    for r in range(world):
        err_attn, err_ffn, shapes_ok = ret[r]
        assert shapes_ok
        assert err_attn < 1e-4 and err_ffn < 1e-4, (err_attn, err_ffn)


# ------------------------------------------------------------------ sharded LM head: candidate pick
def _head_worker(rank, world, port, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    rng = np.random.default_rng(9)
    vocab, rows = 4096, 5
    # f16-representable logits with many exact ties (values on a coarse grid), the same on every rank
    logits = (rng.integers(-40, 41, (rows, vocab)) / 16.0).astype(np.float32)
    v_l = vocab // world
    cand = torch.zeros(rows, 2, dtype=torch.float64)
    for i in range(rows):  # this rank's arg-max over its vocabulary rows, index made global
        idx, val = O.argmax(logits[i, rank * v_l:(rank + 1) * v_l])
        cand[i, 0], cand[i, 1] = idx + rank * v_l, val
    got = [torch.zeros_like(cand) for _ in range(world)]
    dist.all_gather(got, cand)
    picked = []
    for i in range(rows):  # the lead rank's rule: largest value, lowest index among equals
        best = None
        for r in range(world):
            idx, val = int(got[r][i, 0]), float(got[r][i, 1])
            if best is None or val > best[1] or (val == best[1] and idx < best[0]):
                best = (idx, val)
        picked.append(best[0])
    want = [O.argmax(logits[i])[0] for i in range(rows)]
    ret[rank] = (picked, want)
    dist.destroy_process_group()


def test_sharded_head_pick_equals_full_argmax_world2():
    """The rule the lead rank applies to the ranks' candidates gives the arg-max of the whole row, ties included."""
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_head_worker, args=(world, 29613, ret), nprocs=world, join=True)
    for r in range(world):
        picked, want = ret[r]
        assert picked == want


# ------------------------------------------------------------------ host roll call: a rank that never arrives
def _roll_call_worker(rank, world, port, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]
    import datetime
    import llama_cu_b200 as L
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    rv = L.StepRendezvous(store, rank, world, timeout_s=0.5)
    rv.wait(0)                      # round 0: everybody arrives
    out = {"round0": True}
    if rank == 1:
        out["round1"] = "skipped"   # this rank fails between two rounds: it never arrives at round 1
    else:
        try:
            rv.wait(1)
            out["round1"] = "passed"
        except L.LcuError as e:
            out["round1"] = (e.code, str(e))
    ret[rank] = out
    store.set(f"done/{rank}", b"1")
    store.wait([f"done/{r}" for r in range(world)])  # keep the store's host alive until everyone has reported


def test_roll_call_names_the_missing_rank():
    """Host-made failure, no GPU involved: rank 1 never joins round 1, rank 0 learns of it within the limit and
    gets LCU_ERR_TIMEOUT naming rank 1 before it would launch anything."""
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_roll_call_worker, args=(world, 29617, ret), nprocs=world, join=True)
    assert ret[0]["round0"] and ret[1]["round0"]
    code, msg = ret[0]["round1"]
    assert code == -7 and "[1]" in msg
