"""Tensor-parallel parity (needs >= 2 GPUs of one box).

The reference's residual placement under TP lives in crate `nn` and cannot be pinned, so TP parity is
defined as: TP=N logits equal the oracle's AND the TP=1 logits of this build within the logits tolerance,
at EVERY teacher-forced step, for each transport — ncclAllReduce, the peer-memory push form and (forced
with 2 ranks) the scatter form of the peer all-reduce; device status word zero on every rank.
Set LCU_TP_LOG to a file name to append one summary line per run (kept as evidence of a multi-GPU run).
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = (5, 9, 40)


def spec_with(spec_path, tmp_path, **kw):
    spec = json.load(open(spec_path))
    spec.update(kw)
    path = tmp_path / ("spec_" + "_".join(sorted(kw)) + f"_{abs(hash(json.dumps(kw, sort_keys=True))) % 10**6}.json")
    json.dump(spec, open(path, "w"))
    return path


def run_world(world, spec_path, tmp_path, mode, extra_env=None, tag=""):
    out = tmp_path / f"tp{world}_{mode}{tag}.npz"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), os.path.join(ROOT, "tests", "tp_worker.py"),
           str(spec_path), str(out), mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return dict(np.load(out))


def compare(tag, got, o_ids, o_lgs, one, tol, log):
    """Unconditional checks of one run against the oracle and against TP=1."""
    v = int(got["v_cols"])  # columns of the vocabulary the lead rank's logits cover (all of them unless the head is sharded)
    lg = got["logits"][:, :, :v]
    err_oracle = float(np.abs(lg - o_lgs[:, :, :v]).max())
    err_tp1 = float(np.abs(lg - one["logits"][:, :, :v]).max()) if one is not None else 0.0
    exact = int((got["tf_ids"] == o_ids).sum())
    line = {"run": tag, "max_err_vs_oracle": err_oracle, "max_err_vs_tp1": err_tp1, "argmax_equal": exact,
            "steps": int(o_ids.size), "status": [int(s) for s in got["status"]], "launches": int(got["launches"])}
    print("[tp-parity]", json.dumps(line))
    if log:
        with open(log, "a") as f:
            f.write(json.dumps(line) + "\n")
    assert all(int(s) == 0 for s in got["status"]), f"{tag}: device status {got['status']}"
    assert err_oracle <= tol, f"{tag}: logits differ from the oracle by {err_oracle}"
    assert err_tp1 <= tol, f"{tag}: logits differ from TP=1 by {err_tp1}"
    for i, s in zip(*np.nonzero(got["tf_ids"] != o_ids)):
        top = np.sort(o_lgs[i, s])
        assert top[-1] - top[-2] <= 2 * err_oracle + 1e-6, (tag, "teacher-forced", int(i), int(s))
    for i in range(o_ids.shape[0]):  # free-running: first divergence must sit on a near-tie
        for s in range(o_ids.shape[1]):
            if got["free_ids"][i, s] != o_ids[i, s]:
                top = np.sort(o_lgs[i, s])
                assert top[-1] - top[-2] <= 2 * err_oracle + 1e-6, (tag, "free-running", i, s)
                break


@pytest.mark.parametrize("name,layers,vocab", [("llama8b", 2, 4096), ("llama1b", 2, 4096)])
def test_tp_matches_tp1_and_oracle(L, O, name, layers, vocab, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from llama_cu_b200.model import reduced
    steps = 8
    worlds = [int(w) for w in os.environ.get("LCU_TP_WORLDS", "2,4,8").split(",")]
    log = os.environ.get("LCU_TP_LOG")
    cfg = reduced(L.CONFIGS[name], layers, vocab)
    w = L.synth_weights_numpy(cfg, 0)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in LENGTHS]
    ids, lgs = O.Model(cfg, w).generate(prompts, steps)
    o_ids, o_lgs = np.array(ids, np.int64), np.array(lgs, np.float32)
    spec = tmp_path / "spec.json"
    json.dump({"name": name, "layers": layers, "vocab": vocab, "steps": steps, "lengths": list(LENGTHS), "ids": ids},
              open(spec, "w"))
    tol = 8e-2 if cfg.act_dtype == 1 else 2e-2
    one = run_world(1, spec, tmp_path, "nccl")
    compare(f"{name} tp1", one, o_ids, o_lgs, None, tol, log)
    for world in (2, 4, 8):
        if world not in worlds or torch.cuda.device_count() < world or cfg.nkvh % world or cfg.nh % world:
            continue
        if world == 2:
            got = run_world(2, spec, tmp_path, "nccl")
            assert not got["p2p"] and got["launches"] > one["launches"]  # the all-reduces are part of the step
            compare(f"{name} tp2 nccl", got, o_ids, o_lgs, one, tol, log)
        got = run_world(world, spec, tmp_path, "p2p")
        assert got["p2p"]
        compare(f"{name} tp{world} p2p push", got, o_ids, o_lgs, one, tol, log)
        # the scatter (reduce-scatter + all-gather) form, forced for every round size
        got = run_world(world, spec_with(spec, tmp_path, tuning={"p2p_scatter_ranks": 2, "p2p_scatter_min": 0}), tmp_path, "p2p",
                        tag="_sc")
        assert got["p2p"]
        compare(f"{name} tp{world} p2p scatter", got, o_ids, o_lgs, one, tol, log)
        # LM head sharded by vocabulary rows: the lead rank picks among the ranks' candidates (ids cover the whole
        # vocabulary, the logits compared are the lead rank's columns)
        got = run_world(world, spec_with(spec, tmp_path, head_shard=1), tmp_path, "p2p", tag="_hs")
        assert got["p2p"] and int(got["v_cols"]) == cfg.vocab // world
        compare(f"{name} tp{world} p2p push, sharded head", got, o_ids, o_lgs, one, tol, log)


def test_bounded_wait_runs_out_and_step_reports_timeout(L, tmp_path):
    """A rank that stops between two rounds: the other rank's kernels give up after the configured limit, raise bit
    16 of the status word and RETURN (the context stays usable), and its next lcu_step answers LCU_ERR_TIMEOUT.
    Two ranks on two GPUs, NVLS off, plain peer stores; nothing faults, traps or hangs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = tmp_path / "timeout.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "tp_timeout_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.load(open(out))
    print("[tp-timeout]", json.dumps(res))
    assert res["status_before"] == 0
    assert res["roll_call_error"][0] == -7 and "[1]" in res["roll_call_error"][1]   # host side: learnt before launching
    assert res["status_after"] & 16                                                 # device side: the wait ran out ...
    assert res["seconds_for_the_abandoned_round"] < 5.0                             # ... within the limit, and returned
    assert res["next_step_error"] == -7                                             # LCU_ERR_TIMEOUT
    assert res["after_reset_status"] == 0
