"""ctypes binding of the reference-kernel baseline (oracle/ref_step.cu inside oracle/_ref/libref_ops.so) —
TEST / MEASUREMENT INFRASTRUCTURE.

The baseline replays the reference's launch sequence of a decode round with the reference's own kernels,
cuBLAS and a restated attention operator (see ref_step.cu).  It is the stand-in for "the reference's own
CUDA build" (the Rust binary cannot be built here) and the second witness of whole-step parity.  f16
models on one GPU only — the reference has no bf16 and no quantised path.  Only tests and the benchmark's
`ref_kernel_baseline` record may import this module; the product package never does.
"""
import ctypes as C
import os

import numpy as np

from . import oracle as O

F16 = 0


class Desc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d", "nh", "nkvh", "dh", "di", "vocab", "nctx")] + [
        ("eps", C.c_float), ("theta", C.c_float)]


class Req(C.Structure):
    _fields_ = [("seq", C.c_int32), ("pos", C.c_uint32), ("len", C.c_uint32)]


_lib = None


def lib():
    """The library with the round replay, or None when oracle/_ref was never built (no reference tree)."""
    global _lib
    if _lib is None:
        if not os.path.exists(O.REF_LIB):
            return None
        R = C.CDLL(O.REF_LIB)
        if not hasattr(R, "refstep_create"):
            return None
        vp = C.c_void_p
        R.refstep_last_error.restype = C.c_char_p
        R.refstep_create.argtypes = [C.POINTER(Desc), C.POINTER(vp)]
        R.refstep_destroy.argtypes = [vp]
        R.refstep_set_weight.argtypes = [vp, C.c_int, C.c_int, vp]
        R.refstep_seq_new.argtypes = [vp]
        R.refstep_round.argtypes = [vp, vp, C.c_int, C.POINTER(Req), vp, vp, C.c_int, vp, C.POINTER(C.c_long)]
        R.refstep_logits.restype = vp
        R.refstep_logits.argtypes = [vp]
        _lib = R
    return _lib


class RefModel:
    """One f16 model on the current device; weights are caller-owned device tensors {(layer, kind): tensor}."""

    def __init__(self, cfg, dev_weights):
        R = lib()
        if R is None:
            raise RuntimeError("oracle/_ref/libref_ops.so is not built (needs the reference tree at build time)")
        if cfg.act_dtype != F16 or cfg.wdt != F16:
            raise ValueError("the reference has an f16 path only")
        self.R, self.cfg = R, cfg
        d = Desc(cfg.n_layers, cfg.d, cfg.nh, cfg.nkvh, cfg.dh, cfg.di, cfg.vocab, cfg.nctx, cfg.eps, cfg.theta)
        h = C.c_void_p()
        self._check(R.refstep_create(C.byref(d), C.byref(h)))
        self.h = h
        self._keep = []
        for (layer, kind), t in dev_weights.items():
            self._check(R.refstep_set_weight(h, max(layer, 0), kind, t.data_ptr()))
            self._keep.append(t)
        self.launches = 0

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(f"ref baseline error {rc}: {self.R.refstep_last_error().decode()}")

    def close(self):
        if self.h:
            self.R.refstep_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def seq_new(self):
        s = self.R.refstep_seq_new(self.h)
        if s < 0:
            raise RuntimeError("ref baseline: KV cache allocation failed")
        return s

    def round(self, reqs, tokens, out, fast_map=None, stream=None):
        """reqs [(seq, pos, len)], flat host tokens, out: device tensor of n_req KVPairs.  Does not synchronise."""
        import torch
        n = len(reqs)
        creqs = (Req * n)(*[Req(*r) for r in reqs])
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        fm = None if fast_map is None else np.ascontiguousarray(fast_map, dtype=np.uint32).reshape(-1, 2)
        s = stream if stream is not None else torch.cuda.current_stream()
        cnt = C.c_long()
        self._check(self.R.refstep_round(self.h, C.c_void_p(s.cuda_stream), n, creqs, tokens.ctypes.data,
                                         None if fm is None else fm.ctypes.data, 0 if fm is None else len(fm),
                                         out.data_ptr(), C.byref(cnt)))
        self.launches = cnt.value

    def logits(self, n_req):
        import torch
        torch.cuda.synchronize()

        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (n_req * self.cfg.vocab,), "typestr": "<i2",
                                        "data": (self.R.refstep_logits(self.h), False), "version": 2}
        return torch.as_tensor(raw, device="cuda").view(torch.float16).view(n_req, self.cfg.vocab).clone()


def bench_record(cfg, batch, prompt_range, nctx, steps=64, warmup=8, device="cuda:0"):
    """Times the reference-kernel baseline on the benchmark workload (same seeded weights, prompts and timing
    method as the product arm: staged prefill, then `steps` decode rounds between CUDA events with the sampled
    ids fed back on the device).  Returns the `ref_kernel_baseline` record of bench.py."""
    import torch
    import llama_cu_b200 as L
    if lib() is None:
        return {"unavailable": "unavailable on this box: oracle/_ref/libref_ops.so was not built (no reference tree)"}
    if cfg.act_dtype != F16 or cfg.wdt != F16:
        return {"unavailable": "unsupported by reference: it has an f16 path only"}
    from dataclasses import replace
    cfg = replace(cfg, nctx=nctx)
    rng = np.random.default_rng(1234)
    pmin, pmax = prompt_range
    lengths = [int(x) for x in rng.integers(pmin, pmax + 1, batch)]
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in lengths]
    weights = L.synth_weights_torch(cfg, seed=0, device=device)
    m = RefModel(cfg, weights)
    stream = torch.cuda.Stream(device=device)
    out = torch.zeros(max(batch, 1), 2, dtype=torch.int32, device=device)
    seqs = [m.seq_new() for _ in prompts]
    with torch.cuda.stream(stream):
        first = []
        for s, p in zip(seqs, prompts):  # staged prefill: each prompt alone, as the 1024-token round limit requires
            m.round([(s, 0, len(p))], p, out, stream=stream)
            stream.synchronize()
            first.append(int(out[0, 0].item()))
        pos = list(lengths)
        fm = np.array([[i, i] for i in range(batch)], np.uint32)
        zeros = np.zeros(batch, np.uint32)

        def decode(tokens, fast_map):
            m.round([(seqs[i], pos[i], 1) for i in range(batch)], tokens, out, fast_map=fast_map, stream=stream)
            for i in range(batch):
                pos[i] += 1
        decode(np.array(first, np.uint32), None)
        for _ in range(warmup - 1):
            decode(zeros, fm)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            decode(zeros, fm)
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / steps
    rec = {"ms_per_step": ms, "tokens_s": batch / (ms * 1e-3), "steps": steps, "warmup": warmup, "batch": batch,
           "launches_per_step": m.launches,
           "what": "the reference's own kernels + cublasGemmEx + restated per-request attention, L+1 graph segments, "
                   "32-token bucket padding, per-row arg-max loop (single GPU)"}
    m.close()
    del weights
    torch.cuda.empty_cache()
    return rec
