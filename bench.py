"""Decode-loop benchmark: tokens/s of the B200 token loop on the Llama-3-8B-shape model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one decode round (one new token per sequence).  With N > 1 the launcher is
torchrun (one process per GPU) and the model is tensor-parallel over the N GPUs with an
all-reduce after the attention-output and FFN-down projections, as in the reference.
Prints ONE JSON line on rank 0.  Weights are seeded synthetic values of the named shape.
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

# name -> (model config, batch, prompt length range, note)
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


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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

    The reference is CUDA-only; its CPU stand-in is the oracle port.  A bounded sample is
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
            "sample": f"{layers} of {cfg.n_layers} layers + full LM head in f32, batch 1, 16-token prompt, "
                      f"{len(times)} decode steps; layer time scaled to {cfg.n_layers} layers",
            "ms_per_token": per_tok * 1e3}


def probe_linear(n_tok, reps=5):
    """Small stand-alone case of the linear-layer kernels for profiler captures: `lcu_op_linear` on the
    gate|up shape of the 8B model [28672 x 4096] over 4 distinct weight matrices in turn (940 MB, larger
    than L2).  n_tok = 1 runs the GEMV, 5..8 the mma.sync kernel, more the tcgen05 kernel."""
    import ctypes as C
    import torch
    import llama_cu_b200 as L
    lib = L.load_library()
    k, out = 4096, 28672
    ws = [torch.randn(out, k, device="cuda", dtype=torch.float16) * 0.02 for _ in range(4)]
    x = torch.randn(n_tok, k, device="cuda", dtype=torch.float16)
    y = torch.empty(n_tok, out, device="cuda", dtype=torch.float16)
    sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run():
        for w in ws:
            L.check(lib.lcu_op_linear(y.data_ptr(), out, x.data_ptr(), k, w.data_ptr(), 0, None, 0, n_tok, k, out, 0, sp))
    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / (reps * len(ws)) * 1e3
    print(json.dumps({"probe": "linear", "tokens": n_tok, "shape": [out, k], "us_per_launch": us,
                      "GBps": out * k * 2 / us / 1e3}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", type=int, default=0, metavar="N",
                    help="cut the model to its first N layers: a small case for profiler captures, not a bench line")
    ap.add_argument("--probe-linear", type=int, default=0, metavar="TOKENS",
                    help="run only the small linear-layer case used for profiler captures")
    args = ap.parse_args()
    if args.probe_linear > 0:
        probe_linear(args.probe_linear)
        return
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    import llama_cu_b200 as L
    cname, batch, (pmin, pmax) = WORKLOADS[args.workload]
    cfg = L.CONFIGS[cname]
    if args.layers > 0:
        from llama_cu_b200.model import reduced
        cfg = reduced(cfg, min(args.layers, cfg.n_layers))
    dtype_name = {(0, 0): "f16", (1, 1): "bf16", (0, 3): "f16 activations, q8_0 weights"}[(cfg.act_dtype, cfg.wdt)]
    config = {"workload": args.workload, "shape": cname, "batch": batch, "prompt_tokens": [pmin, pmax],
              "parallelism": f"tp{args.gpus}", "l2": "inputs larger than L2 (weights streamed once per step)"}
    if args.layers > 0:
        config["layers"] = cfg.n_layers  # profiling case only

    if args.impl == "reference":
        # the reference's own CPU implementation does not exist (it is CUDA-only and its Rust
        # host cannot be built here); this arm times the oracle port on the host cores
        if rank != 0:
            return
        r = cpu_reference(cfg, args.steps, args.warmup)
        line = {"impl": "reference", "metric": "decode tokens/s", "value": r["value"] * 1.0, "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_token"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": dict(config, batch=1), "cpu_baseline": r,
                "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(dev))
        lib = L.load_library()
        uid = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            L.check(lib.lcu_comm_unique_id(uid.numpy().ctypes.data))
        uid = uid.to(dev)
        dist.broadcast(uid, 0)
        uid = uid.cpu().contiguous()
        import ctypes as C
        h = C.c_void_p()
        L.check(lib.lcu_comm_init_rank(uid.numpy().ctypes.data, rank, world, C.byref(h)))
        comm = h

    # ---- model: seeded synthetic weights generated on the device, sliced per rank
    rng = np.random.default_rng(1234)
    lengths = [int(x) for x in rng.integers(pmin, pmax + 1, batch)]
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in lengths]
    steps_total = args.warmup + args.steps
    nctx = max(lengths) + 2 * steps_total + 8
    nctx = (nctx + 63) // 64 * 64
    weights = L.iter_synth_weights_torch(cfg, seed=0, device=dev)  # one tensor at a time, sliced per rank
    kv_tokens = sum(n + 2 * steps_total + 64 for n in lengths)
    kv_bytes = kv_tokens * cfg.kv_bytes_per_token(world) + (64 << 20)
    ctx = L.load_model(cfg, weights, device=local_rank, kv_bytes=kv_bytes, tp_rank=rank, tp_size=world, comm=comm,
                       max_tokens=1024, max_seqs=max(batch, 1), nctx=nctx)
    del weights
    torch.cuda.empty_cache()
    # tensor parallelism: all-reduce fused into the projections over NVLink peer memory (LCU_BENCH_NCCL=1: ncclAllReduce)
    if world > 1 and os.environ.get("LCU_BENCH_NCCL", "0") != "1":
        def gather(b):
            got = [None] * world
            dist.all_gather_object(got, b)
            return got
        ctx.p2p_connect(gather)
    config["tp_collectives"] = "peer-memory push + local reduce" if (world > 1 and ctx.p2p_enabled) else ("nccl" if world > 1 else "none")

    stream = torch.cuda.Stream(device=dev)
    out = torch.zeros(batch, 2, dtype=torch.int32, device=dev)
    seqs = [ctx.seq_create() for _ in prompts]

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    with torch.cuda.stream(stream):
        # ---- prefill (untimed), one sequence per round as the reference's 1024-token round limit requires
        first = []
        for s, p in zip(seqs, prompts):
            ctx.step([(s, 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            first.append(int(out[0, 0].item()) if rank == 0 else 0)
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
        for _ in range(args.warmup - 1):
            decode_round(zeros, fast_map)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        step_bytes = 0.0
        with ClockSampler(local_rank) as clocks:
            ev0.record(stream)
            for _ in range(args.steps):
                decode_round(zeros, fast_map)
                step_bytes += ctx.last_step_bytes
            ev1.record(stream)
            barrier()
        ms = ev0.elapsed_time(ev1)
        launches = ctx.last_launch_count * args.steps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ms_per_step = ms / args.steps
        value = batch * args.steps / (ms / 1e3)

        # ---- end to end: host tokens in (pinned staging inside lcu_step), sampled pair read back every step
        e2e = None
        if not args.no_e2e:
            host_out = torch.zeros(batch, 2, dtype=torch.int32).pin_memory()
            host_out.copy_(out, non_blocking=True)
            stream.synchronize()
            toks = host_out[:, 0].numpy().astype(np.uint32).copy() if rank == 0 else zeros.copy()
            n_e2e = max(8, args.steps // 2)
            barrier()
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
            barrier()
            dt_s = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([dt_s], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dt_s = float(t.item())
            desc_bytes = 4 * batch * 3 + 4 * batch + 8 * batch + 16 * batch + 4 * batch + 4 * batch * ((nctx + ctx.page_tokens - 1) // ctx.page_tokens)
            e2e = {"value": batch * n_e2e / dt_s, "unit": "tokens/s", "h2d_bytes_per_step": desc_bytes,
                   "d2h_bytes_per_step": 8 * batch, "steps": n_e2e}

        # ---- roofline of the dominant kernel: the weight-streaming GEMV on the gate|up projection shape,
        # timed alone with CUDA events over every layer's weights in turn (so the inputs exceed L2)
        peak, peak_kind = load_peaks()
        roof = None
        if rank == 0:
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
            roof = {"bound": "hbm", "kernel": "gemv_kernel, gate|up projection shape [%d x %d], 1 token" % (rows, cols),
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                    # dram__bytes_read + dram__bytes_write of one launch from the committed ncu capture of this
                    # shape (profiles/gemv_kernel_gate_up_shape_ncu_full.md); other shapes were not captured
                    "traffic": 238.9e6 if (rows, cols, cfg.wdt) == (28672, 4096, 0) else None, "us_per_launch": per_launch_ms * 1e3,
                    "algorithmic_bytes_per_launch": wbytes}
        step_gbs = step_bytes / args.steps / (ms_per_step * 1e-3) / 1e9

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference(cfg, 6, 2, budget_s=30.0)

    if rank == 0:
        line = {"metric": "decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config,
                "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": launches,
                "roofline": roof,
                "step_roofline": {"bound": "hbm", "achieved": step_gbs, "peak": peak, "unit": "GB/s",
                                  "frac": step_gbs / peak, "frac_of_8TBs": step_gbs / 8000.0,
                                  "algorithmic_bytes_per_step": step_bytes / args.steps,
                                  "note": "weights of every linear layer + LM head + cached K/V, per decode step"},
                "cpu_baseline": cpu, "launches_per_step": ctx.last_launch_count}
        print(json.dumps(line), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
