"""Decode-loop benchmark: tokens/s of the B200 token loop on the Llama-3-8B-shape model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one decode round (one new token per sequence).  With N > 1 the launcher is
torchrun (one process per GPU) and the model is tensor-parallel over the N GPUs with an
all-reduce after the attention-output and FFN-down projections, as in the reference.
Prints ONE JSON line on rank 0.  Weights are seeded synthetic values of the named shape.

With N > 1 the line also carries
  "tp_parity": a reduced-shape tensor-parallel run through the same communicator and the same
               peer-memory transport, checked against committed golden vectors BEFORE timing;
  "c5":        a bounded record of the 70B-shape batch-64 tensor-parallel workload (the
               configuration the reference's tensor parallelism is quoted on), measured after
               the headline in the same process.
The process exits non-zero when any rank's device status word is non-zero after timing.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name -> (model config, batch, prompt length range)
WORKLOADS = {
    "llama8b-f16-b1": ("llama8b", 1, (128, 128)),
    "llama8b-f16-b32": ("llama8b", 32, (128, 1024)),
    "llama1b-bf16-b1": ("llama1b", 1, (128, 128)),
    "llama8b-q8_0-b1": ("llama8b_q8", 1, (128, 128)),
    "llama8b-q8_0-b16": ("llama8b_q8", 16, (128, 128)),
    "llama70b-f16-b64": ("llama70b", 64, (1024, 1024)),
    "llama70b-tp8shard-f16-b64": ("llama70b_tp8shard", 64, (1024, 1024)),  # one rank's share, for profiling
    "tiny-f16-b1": ("tiny", 1, (16, 16)),
}
DEFAULT_WORKLOAD = "llama8b-f16-b1"
C5_WORKLOAD = "llama70b-f16-b64"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def profiled_traffic(rows, cols, wdt):
    """DRAM bytes per launch of the roofline kernel from the committed profiler capture of this shape
    (profiles/traffic.json, written by hand from an ncu report), or None when the shape was not captured."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            rec = json.load(f).get(f"gemv_kernel[{rows}x{cols},wdt{wdt},1tok]")
        return rec
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.05)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_reference(cfg, steps, warmup, budget_s=120.0):
    """Times the CPU restatement of the same decode step (oracle/, f32, all host cores).

    The reference is CUDA-only; its CPU stand-in is the oracle port.  A bounded, SCALED sample is
    timed: `layers` of the model's layers plus the full LM head, batch 1 after a 16-token
    prompt; the per-token time is layers-time scaled to the full depth plus the head time."""
    import numpy as np
    from llama_cu_b200.model import reduced
    from oracle import oracle as O
    try:
        host_cores = len(os.sched_getaffinity(0))
    except AttributeError:
        host_cores = os.cpu_count() or 1
    cores = O.set_threads(host_cores)  # torchrun exports OMP_NUM_THREADS=1
    layers = min(cfg.n_layers, 4)
    small = reduced(cfg, layers)
    m = O.Model(small, None, act_dtype=2)
    s = m.seq_new()
    _, ids = m.forward([(s, 0, 16)], np.arange(3, 19, dtype=np.uint32))
    pos = 16
    times = []
    t_start = time.time()
    for i in range(warmup + steps):
        _, ids = m.forward([(s, pos, 1)], ids)
        pos += 1
        tl, th = m.last_times()
        if i >= warmup:
            times.append(tl * cfg.n_layers / layers + th)
        if time.time() - t_start > budget_s and len(times) >= 3:
            break
    per_tok = sum(times) / len(times)
    return {"value": 1.0 / per_tok, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"scaled sample: {layers} of {cfg.n_layers} layers + full LM head in f32, batch 1, 16-token prompt, "
                      f"{len(times)} decode steps; layer time scaled to {cfg.n_layers} layers",
            "ms_per_token": per_tok * 1e3}


def probe_linear(n_tok, reps=5, q8=False, shape="gate_up"):
    """Small stand-alone case of the linear-layer kernels for profiler captures: `lcu_op_linear` on a projection
    shape of the 8B model over 4 distinct weight matrices in turn (larger than L2 together).  n_tok = 1 runs the
    GEMV, 3..8 the mma.sync kernel, more the tcgen05 kernel (f16 weights) or the mma.sync kernel (Q8_0)."""
    import ctypes as C
    import torch
    import llama_cu_b200 as L
    lib = L.load_library()
    out, k = {"gate_up": (28672, 4096), "down": (4096, 14336), "qkv": (6144, 4096), "o": (4096, 4096)}[shape]
    nmat = 4 if out * k >= 100e6 else 12
    if q8:
        ws = []
        for _ in range(nmat):
            buf = torch.empty(out * k + out * k // 32 * 2, dtype=torch.uint8, device="cuda")
            buf[:out * k] = torch.randint(-127, 128, (out * k,), dtype=torch.int8, device="cuda").view(torch.uint8)
            sc = torch.empty(out * k // 32, dtype=torch.float32, device="cuda").uniform_(1e-4, 4e-4)
            buf[out * k:] = sc.to(torch.float16).view(torch.uint8)
            ws.append(buf)
        wdt, wbytes = L.Q8_0, out * k * 34 / 32
    else:
        ws = [torch.randn(out, k, device="cuda", dtype=torch.float16) * 0.02 for _ in range(nmat)]
        wdt, wbytes = L.F16, out * k * 2
    x = torch.randn(n_tok, k, device="cuda", dtype=torch.float16)
    y = torch.empty(n_tok, out, device="cuda", dtype=torch.float16)
    sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run():
        for w in ws:
            L.check(lib.lcu_op_linear(y.data_ptr(), out, x.data_ptr(), k, w.data_ptr(), wdt, None, 0, n_tok, k, out, 0, sp))
    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / (reps * len(ws)) * 1e3
    print(json.dumps({"probe": "linear", "tokens": n_tok, "shape": [out, k], "q8_0": bool(q8), "us_per_launch": us,
                      "GBps": wbytes / us / 1e3}), flush=True)


class Env:
    """Process-group facts of this rank."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = f"cuda:{self.local_rank}"
        self.comm = None
        self.use_p2p = True       # --tp-transport
        self.head_sharding = True  # --no-head-sharding

    def barrier(self):
        import torch
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, v):
        if self.world == 1:
            return v
        import torch
        import torch.distributed as dist
        t = torch.tensor([v], dtype=torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def connect(self, ctx):
        """Switches a tensor-parallel context to the peer-memory transport (all ranks together)."""
        if not self.head_sharding:  # A/B switch: head on the lead rank alone
            ctx.set_head_sharding(0)
        if self.world > 1 and self.use_p2p:
            import torch.distributed as dist

            def gather(b):
                got = [None] * self.world
                dist.all_gather_object(got, b)
                return got
            ctx.p2p_connect(gather)

    def status_all_ranks(self, ctx):
        """Every rank's device status word (bit 4/16/32: a bounded device-side wait ran out)."""
        import torch
        st = ctx.device_status()
        if self.world == 1:
            return [st]
        import torch.distributed as dist
        t = torch.tensor([st], dtype=torch.int64, device=self.dev)
        got = [torch.zeros_like(t) for _ in range(self.world)]
        dist.all_gather(got, t)
        return [int(g.item()) for g in got]


def tp_parity(L, env):
    """Reduced-shape tensor-parallel check before timing: the golden case `llama8b_L2_tp` (8B widths, 2 layers,
    vocabulary 2048, prompts of 5 / 9 / 40 tokens, 8 steps; vectors made by the independent PyTorch restatement
    and committed under tests/golden/) run teacher-forced through this process group's communicator and
    transport.  Compares rank 0's arg-max ids and logit probes with the golden vectors."""
    import numpy as np
    import torch
    from llama_cu_b200.model import reduced
    case = json.load(open(os.path.join(ROOT, "tests", "golden", "decode_golden.json")))["llama8b_L2_tp"]
    cfg = reduced(L.CONFIGS[case["config"]], case["reduced"][0], case["reduced"][1])
    w = L.synth_weights_numpy(cfg, case["weight_seed"])
    rng = np.random.default_rng(case["prompt_seed"])
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in case["lengths"]]
    steps, n = case["steps"], len(prompts)
    ctx = L.load_model(cfg, w, device=env.local_rank, tp_rank=env.rank, tp_size=env.world, comm=env.comm, max_seqs=n)
    env.connect(ctx)
    stream = torch.cuda.Stream(device=env.dev)
    out = torch.zeros(n, 2, dtype=torch.int32, device=env.dev)
    ids_equal, total, worst = 0, 0, 0.0

    # columns of the vocabulary the lead rank's logits cover: all of them, or its own slice when the head is sharded
    sharded = (ctx.p2p_enabled and env.head_sharding and cfg.vocab % env.world == 0
               and (cfg.vocab // env.world) % 2 == 0)
    v_cols = cfg.vocab // env.world if sharded else cfg.vocab

    def probe(i, s, lg, picked):
        nonlocal ids_equal, total, worst
        want_id = case["ids"][i][s]
        total += 1
        ids_equal += int(picked == want_id)  # the arg-max over the WHOLE vocabulary either way
        cols = [0, 1, cfg.vocab // 2, cfg.vocab - 1, want_id]
        for c, want in zip(cols, case["logit_probes"][i][s]):
            if c < v_cols:
                worst = max(worst, abs(float(lg[c]) - want))

    with torch.cuda.stream(stream):
        seqs = [ctx.seq_create() for _ in prompts]
        for i, p in enumerate(prompts):
            ctx.step([(seqs[i], 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            if env.rank == 0:
                probe(i, 0, ctx.logits(1).reshape(-1)[:v_cols].float().cpu().numpy(), int(out[0, 0].item()))
        pos = [len(p) for p in prompts]
        for s in range(steps - 1):
            ctx.step([(seqs[i], pos[i], 1) for i in range(n)], np.array([case["ids"][i][s] for i in range(n)], np.uint32),
                     out, stream=stream)
            stream.synchronize()
            if env.rank == 0:
                lg = ctx.logits(n).reshape(-1)[:n * v_cols].view(n, v_cols).float().cpu().numpy()
                got = out[:n, 0].cpu().numpy().view(np.uint32)
                for i in range(n):
                    probe(i, s + 1, lg[i], int(got[i]))
            for i in range(n):
                pos[i] += 1
    torch.cuda.synchronize(env.dev)
    status = env.status_all_ranks(ctx)
    transport = "peer memory" if ctx.p2p_enabled else "nccl"
    ctx.close()
    return {"case": "llama8b_L2_tp (golden vectors, teacher-forced)", "transport": transport,
            "lm_head": "sharded by vocabulary rows" if v_cols < cfg.vocab else "lead rank", "ids_equal": ids_equal,
            "steps": total, "max_logit_err": worst, "tolerance": 2e-2, "device_status_all_ranks": status,
            "ok": bool(ids_equal == total and worst <= 2e-2 and not any(status))}


def run_decode(L, env, cfg, batch, prompt_range, steps, warmup, want_e2e=True, want_roofline=True, max_prefill=1024,
               timeline=None):
    """Loads the model (this rank's slice), prefills, then times `steps` decode rounds with CUDA events.
    Returns a dict of results; the caller prints."""
    import numpy as np
    import torch
    import torch.distributed as dist
    rank, world, dev = env.rank, env.world, env.dev
    pmin, pmax = prompt_range
    rng = np.random.default_rng(1234)
    lengths = [int(x) for x in rng.integers(pmin, pmax + 1, batch)]
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in lengths]
    steps_total = warmup + steps
    nctx = max(lengths) + 2 * steps_total + 8
    nctx = (nctx + 63) // 64 * 64
    weights = L.iter_synth_weights_torch(cfg, seed=0, device=dev)  # one tensor at a time, sliced per rank
    kv_tokens = sum(n + 2 * steps_total + 64 for n in lengths)
    kv_bytes = kv_tokens * cfg.kv_bytes_per_token(world) + (64 << 20)
    ctx = L.load_model(cfg, weights, device=env.local_rank, kv_bytes=kv_bytes, tp_rank=rank, tp_size=world, comm=env.comm,
                       max_tokens=max_prefill, max_seqs=max(batch, 1), nctx=nctx)
    del weights
    torch.cuda.empty_cache()
    # tensor parallelism: all-reduce fused into the projections over NVLink peer memory (--tp-transport nccl: ncclAllReduce)
    env.connect(ctx)
    res = {"tp_collectives": "peer memory, fused into the projections" if (world > 1 and ctx.p2p_enabled) else
           ("nccl" if world > 1 else "none"), "nctx": nctx}

    stream = torch.cuda.Stream(device=dev)
    out = torch.zeros(batch, 2, dtype=torch.int32, device=dev)
    seqs = [ctx.seq_create() for _ in prompts]

    with torch.cuda.stream(stream):
        # ---- prefill (untimed), one sequence per round as the reference's 1024-token round limit requires
        first = []
        t_pre = time.perf_counter()
        for s, p in zip(seqs, prompts):
            ctx.step([(s, 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            first.append(int(out[0, 0].item()) if rank == 0 else 0)
        res["prefill_tokens_s"] = sum(lengths) / (time.perf_counter() - t_pre)
        if world > 1:
            t = torch.tensor(first, dtype=torch.int64, device=dev)
            dist.broadcast(t, 0)
            first = [int(v) for v in t.tolist()]
        pos = list(lengths)
        fast_map = np.array([[i, i] for i in range(batch)], dtype=np.uint32)
        zeros = np.zeros(batch, np.uint32)

        def decode_round(tokens, fm):
            reqs = [(seqs[i], pos[i], 1) for i in range(batch)]
            ctx.step(reqs, tokens, out, fast_map=fm, stream=stream)
            for i in range(batch):
                pos[i] += 1

        # ---- device-resident loop: sampled ids feed the next round on the device (no host read)
        decode_round(np.array(first, np.uint32), None)
        for _ in range(warmup - 1):
            decode_round(zeros, fast_map)
        env.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        step_bytes = 0.0
        with ClockSampler(env.local_rank) as clocks:
            ev0.record(stream)
            for _ in range(steps):
                decode_round(zeros, fast_map)
                step_bytes += ctx.last_step_bytes
            ev1.record(stream)
            env.barrier()
        ms = env.max_over_ranks(ev0.elapsed_time(ev1))
        res.update(ms_per_step=ms / steps, value=batch * steps / (ms / 1e3), clocks=clocks.summary(),
                   launches_per_step=ctx.last_launch_count, step_bytes=step_bytes / steps)

        # ---- device timeline of one decode step (outside the timed region): start and end of every kernel as CUPTI
        # reports them through torch.profiler, overlaps of programmatically launched kernels included
        if timeline and rank == 0:
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(4):
                    decode_round(zeros, fast_map)
                stream.synchronize()
            ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                        key=lambda e: e.time_range.start)
            marks = [i for i, e in enumerate(ev) if "fast_embedding" in e.name]
            if len(marks) >= 2:
                t0 = ev[marks[-2]].time_range.start
                with open(timeline, "w") as f:
                    f.write("# kernel | start us | end us | duration us   (one decode step, batch %d, %d layers)\n" % (batch, cfg.n_layers))
                    for e in ev[marks[-2]:marks[-1]]:
                        f.write("%-72s %9.2f %9.2f %8.2f\n" % (e.name[:72], e.time_range.start - t0, e.time_range.end - t0,
                                                              e.time_range.end - e.time_range.start))
                    f.write("# step: %.2f us\n" % (ev[marks[-1]].time_range.start - t0))
        elif timeline:
            for _ in range(4):
                decode_round(zeros, fast_map)

        # ---- end to end: host tokens in (pinned staging inside lcu_step), sampled pair read back every step
        if want_e2e:
            host_out = torch.zeros(batch, 2, dtype=torch.int32).pin_memory()
            host_out.copy_(out, non_blocking=True)
            stream.synchronize()
            toks = host_out[:, 0].numpy().astype(np.uint32).copy() if rank == 0 else zeros.copy()
            n_e2e = max(8, steps // 2)
            env.barrier()
            t0 = time.perf_counter()
            for _ in range(n_e2e):
                if world > 1:
                    tt = torch.from_numpy(toks.astype(np.int64)).to(dev)
                    dist.broadcast(tt, 0)
                    toks = tt.cpu().numpy().astype(np.uint32)
                decode_round(toks, None)
                host_out.copy_(out, non_blocking=True)
                stream.synchronize()
                if rank == 0:
                    toks = host_out[:, 0].numpy().astype(np.uint32).copy()
            env.barrier()
            dt_s = env.max_over_ranks(time.perf_counter() - t0)
            desc_bytes = 4 * batch * 3 + 4 * batch + 8 * batch + 16 * batch + 4 * batch + 4 * batch * ((nctx + ctx.page_tokens - 1) // ctx.page_tokens)
            res["e2e"] = {"value": batch * n_e2e / dt_s, "unit": "tokens/s", "h2d_bytes_per_step": desc_bytes,
                          "d2h_bytes_per_step": 8 * batch, "steps": n_e2e}

        # ---- roofline of the dominant kernel: the weight-streaming GEMV on the gate|up projection shape,
        # timed alone with CUDA events over every layer's weights in turn (so the inputs exceed L2)
        if want_roofline and rank == 0:
            peak, peak_kind = load_peaks()
            lib = L.load_library()
            sh = cfg.shapes(world)
            rows, cols = sh[L.W_GATE_UP]
            wbytes = rows * cols * (34.0 / 32.0 if cfg.wdt == L.Q8_0 else 2.0)
            x = torch.randn(1, cols, device=dev).to(L.torch_dtype(cfg.act_dtype))
            y = torch.empty(1, rows, device=dev, dtype=x.dtype)
            gate_ups = [t for t in ctx._keep if t.numel() * t.element_size() == int(wbytes)]
            sp = L.stream_ptr(stream)

            def run_all():
                for w in gate_ups:
                    L.check(lib.lcu_op_linear(y.data_ptr(), rows, x.data_ptr(), cols, w.data_ptr(), cfg.wdt, None, 0, 1,
                                              cols, rows, cfg.act_dtype, sp))
            for _ in range(3):
                run_all()
            stream.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 5
            a.record(stream)
            for _ in range(reps):
                run_all()
            b.record(stream)
            stream.synchronize()
            per_launch_ms = a.elapsed_time(b) / (reps * len(gate_ups))
            achieved = wbytes / (per_launch_ms * 1e-3) / 1e9
            prof = profiled_traffic(rows, cols, cfg.wdt)
            res["roofline"] = {"bound": "hbm", "kernel": "gemv_kernel, gate|up projection shape [%d x %d], 1 token" % (rows, cols),
                               "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                               "traffic": prof["dram_bytes_per_launch"] if prof else None,
                               "traffic_source": prof["source"] if prof else None,
                               "us_per_launch": per_launch_ms * 1e3, "algorithmic_bytes_per_launch": wbytes}
    torch.cuda.synchronize(dev)
    res["device_status_all_ranks"] = env.status_all_ranks(ctx)
    ctx.close()
    del ctx
    torch.cuda.empty_cache()
    return res


def step_roofline(res):
    peak, _ = load_peaks()
    gbs = res["step_bytes"] / (res["ms_per_step"] * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "frac_of_8TBs": gbs / 8000.0,
            "algorithmic_bytes_per_step": res["step_bytes"],
            "note": "weights of every linear layer + LM head (lead rank) + cached K/V of this rank, per decode step"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-c5", action="store_true", help="N > 1: skip the 70B-shape tensor-parallel record")
    ap.add_argument("--no-tp-parity", action="store_true", help="N > 1: skip the reduced-shape parity check")
    ap.add_argument("--no-ref-kernels", action="store_true", help="skip the reference-kernel baseline record")
    ap.add_argument("--tp-transport", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: all-reduce over NVLink peer memory fused into the projections (default) or ncclAllReduce")
    ap.add_argument("--no-head-sharding", action="store_true", help="N > 1: LM head on the lead rank alone, as in the reference")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="library tuning value (lcu_set_tuning), e.g. pdl_edges=29; for A/B measurements")
    ap.add_argument("--timeline", default=None, metavar="PATH",
                    help="after the timed region: write start / end of every kernel of one decode step (CUPTI via torch.profiler)")
    ap.add_argument("--layers", type=int, default=0, metavar="N",
                    help="cut the model to its first N layers: a small case for profiler captures, not a bench line")
    ap.add_argument("--probe-linear", type=int, default=0, metavar="TOKENS",
                    help="run only the small linear-layer case used for profiler captures")
    ap.add_argument("--probe-q8", action="store_true", help="with --probe-linear: Q8_0 weights")
    ap.add_argument("--probe-shape", default="gate_up", choices=["gate_up", "down", "qkv", "o"])
    args = ap.parse_args()
    if args.probe_linear > 0:
        probe_linear(args.probe_linear, q8=args.probe_q8, shape=args.probe_shape)
        return 0
    args.warmup = max(args.warmup, 3)
    env = Env()
    env.use_p2p = args.tp_transport == "p2p"
    env.head_sharding = not args.no_head_sharding
    rank, world = env.rank, env.world

    import llama_cu_b200 as L
    for kv in args.tune:
        key, value = kv.split("=", 1)
        L.set_tuning(key, int(value))
    cname, batch, prange = WORKLOADS[args.workload]
    cfg = L.CONFIGS[cname]
    if args.layers > 0:
        from llama_cu_b200.model import reduced
        cfg = reduced(cfg, min(args.layers, cfg.n_layers))
    dtype_name = {(0, 0): "f16", (1, 1): "bf16", (0, 3): "f16 activations, q8_0 weights"}[(cfg.act_dtype, cfg.wdt)]
    config = {"workload": args.workload, "shape": cname, "batch": batch, "prompt_tokens": list(prange),
              "parallelism": f"tp{args.gpus}", "l2": "inputs larger than L2 (weights streamed once per step)"}
    if args.layers > 0:
        config["layers"] = cfg.n_layers  # profiling case only
    if args.tune:
        config["tuning"] = args.tune

    if args.impl == "reference":
        # the reference's own CPU implementation does not exist (it is CUDA-only and its Rust
        # host cannot be built here); this arm times the oracle port on the host cores
        if rank != 0:
            return 0
        r = cpu_reference(cfg, args.steps, args.warmup)
        line = {"impl": "reference", "metric": "decode tokens/s", "value": r["value"] * 1.0, "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_token"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": dict(config, batch=1), "cpu_baseline": r,
                "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return 0

    import torch
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(env.local_rank)
    t_begin = time.time()
    if world > 1:
        import ctypes as C
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(env.dev))
        lib = L.load_library()
        uid = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            L.check(lib.lcu_comm_unique_id(uid.numpy().ctypes.data))
        uid = uid.to(env.dev)
        dist.broadcast(uid, 0)
        uid = uid.cpu().contiguous()
        h = C.c_void_p()
        L.check(lib.lcu_comm_init_rank(uid.numpy().ctypes.data, rank, world, C.byref(h)))
        env.comm = h

    # ---- tensor-parallel parity of the transports, before and outside the timed region
    parity = None
    if world > 1 and not args.no_tp_parity:
        parity = tp_parity(L, env)

    # ---- the headline workload
    res = run_decode(L, env, cfg, batch, prange, args.steps, args.warmup, want_e2e=not args.no_e2e, timeline=args.timeline)
    config["tp_collectives"] = res["tp_collectives"]
    bad_status = any(res["device_status_all_ranks"])

    # ---- the reference's own kernels + cuBLAS on the same shapes (single GPU; oracle/_ref, built from the reference tree)
    ref_kernels = None
    if rank == 0 and world == 1 and not args.no_ref_kernels and args.layers == 0:
        try:
            from oracle import ref_baseline
            ref_kernels = ref_baseline.bench_record(cfg, batch, prange, res["nctx"])
        except Exception as e:  # the stand-in is optional evidence, never the product
            ref_kernels = {"unavailable": f"{type(e).__name__}: {e}"[:200]}

    # ---- the 70B-shape tensor-parallel record (config 5), bounded, after the headline
    c5 = None
    if world > 1 and not args.no_c5 and args.workload == DEFAULT_WORKLOAD and args.layers == 0:
        c5cfg = L.CONFIGS[WORKLOADS[C5_WORKLOAD][0]]
        need = c5cfg.weight_bytes_per_step(world) / 1.0 + 64 * 1100 * c5cfg.kv_bytes_per_token(world) + (6 << 30)
        free_b, total_b = torch.cuda.mem_get_info(env.local_rank)
        if need > free_b:
            c5 = {"workload": C5_WORKLOAD, "unavailable": f"does not fit: {need / 1e9:.0f} GB needed per GPU at TP{world}, "
                  f"{free_b / 1e9:.0f} GB free"}
        elif time.time() - t_begin > 240:
            c5 = {"workload": C5_WORKLOAD, "unavailable": "skipped: the headline run used the time budget"}
        else:
            r5 = run_decode(L, env, c5cfg, WORKLOADS[C5_WORKLOAD][1], WORKLOADS[C5_WORKLOAD][2], 16, 3, want_e2e=False,
                            want_roofline=False)
            sr = step_roofline(r5)
            c5 = {"workload": C5_WORKLOAD, "parallelism": f"tp{world}", "steps": 16, "warmup": 3, "ms_per_step": r5["ms_per_step"],
                  "tokens_s": r5["value"], "frac_of_measured_peak_per_rank": sr["frac"], "frac_of_8TBs_per_rank": sr["frac_of_8TBs"],
                  "algorithmic_bytes_per_step_lead_rank": sr["algorithmic_bytes_per_step"], "launches_per_step": r5["launches_per_step"],
                  "clocks": r5["clocks"], "device_status_all_ranks": r5["device_status_all_ranks"],
                  "prefill_tokens_s": r5["prefill_tokens_s"]}
            bad_status = bad_status or any(r5["device_status_all_ranks"])

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference(cfg, 6, 2, budget_s=30.0)

    if rank == 0:
        line = {"metric": "decode tokens/s", "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config,
                "clocks": res["clocks"], "e2e": res.get("e2e"), "gpu_launches": res["launches_per_step"] * args.steps,
                "roofline": res.get("roofline"), "step_roofline": step_roofline(res),
                "cpu_baseline": cpu, "launches_per_step": res["launches_per_step"],
                "prefill_tokens_s": res["prefill_tokens_s"],
                "device_status_all_ranks": res["device_status_all_ranks"]}
        if parity is not None:
            line["tp_parity"] = parity
        if c5 is not None:
            line["c5"] = c5
        if ref_kernels is not None:
            line["ref_kernel_baseline"] = ref_kernels
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if bad_status or (parity is not None and not parity["ok"]):
        print("bench: a bounded device-side wait ran out or the tensor-parallel parity check failed "
              f"(status {res['device_status_all_ranks']}, parity {parity})", file=sys.stderr)
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
