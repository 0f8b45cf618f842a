"""ctypes binding of the CPU oracle (oracle/lcu_oracle.c) and of the reference-kernel
witness library (oracle/_ref/libref_ops.so) — TEST INFRASTRUCTURE.

Only tests, the smoke check and the CPU-baseline / reference legs of the benchmark may
import this module; the product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liblcu_oracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libref_ops.so")
REF_DIR = os.environ.get("LCU_REF_DIR", "/root/reference")

F16, BF16, F32, Q8_0 = 0, 1, 2, 3


class Desc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d", "nh", "nkvh", "dh", "di", "vocab", "nctx")] + [
        ("eps", C.c_float), ("theta", C.c_float), ("act_dtype", C.c_int32)]


def build(force=False):
    """Compiles the C oracle and, when the reference tree is present, the witness library
    from the reference's own sources (nothing is copied; see oracle/Makefile)."""
    need = force or not os.path.exists(LIB) or os.path.getmtime(LIB) < max(
        os.path.getmtime(os.path.join(HERE, f)) for f in ("lcu_oracle.c", "lcu_oracle.h"))
    if need:
        subprocess.run(["make", "-C", HERE, "liblcu_oracle.so"], check=True, capture_output=True)
    shim = os.path.join(HERE, "ref_shim.cu")
    if os.path.isdir(os.path.join(REF_DIR, "llama.cu", "src", "op")):
        step = os.path.join(HERE, "ref_step.cu")
        if force or not os.path.exists(REF_LIB) or os.path.getmtime(REF_LIB) < max(os.path.getmtime(shim), os.path.getmtime(step)):
            subprocess.run(["make", "-C", HERE, "ref", f"REF_DIR={REF_DIR}"], check=True, capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB)
        L.orc_round.restype = C.c_float
        L.orc_round.argtypes = [C.c_float, C.c_int]
        L.orc_model_new.restype = C.c_void_p
        L.orc_model_new.argtypes = [C.POINTER(Desc)]
        L.orc_model_free.argtypes = [C.c_void_p]
        L.orc_model_set_weight.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_size_t]
        L.orc_seq_new.argtypes = [C.c_void_p]
        L.orc_model_fill_synthetic.argtypes = [C.c_void_p, C.c_uint64]
        L.orc_seq_free.argtypes = [C.c_void_p, C.c_int]
        L.orc_forward.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6
        L.orc_last_hidden.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_set_threads.restype = C.c_int
        L.orc_last_times.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.orc_to_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]
        L.orc_from_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]
        L.orc_build_sin_cos.argtypes = [C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        L.orc_embedding.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.orc_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int]
        L.orc_linear.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
        L.orc_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_swiglu.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_attention.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 6
        L.orc_argmax.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_uint32), C.POINTER(C.c_float)]
        L.orc_sample.restype = C.c_uint32
        L.orc_sample.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_float, C.c_size_t, C.POINTER(C.c_float)]
        _lib = L
    return _lib


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def to_f32(bits, dt):
    """uint16 bit patterns (f16 / bf16) or ggml Q8_0 bytes -> float32 array."""
    bits = np.ascontiguousarray(bits)
    n = bits.size if dt != Q8_0 else bits.size // 34 * 32
    out = np.empty(n, np.float32)
    lib().orc_to_f32(out.ctypes.data, bits.ctypes.data, dt, n)
    return out.reshape(bits.shape) if dt != Q8_0 else out


def from_f32(a, dt):
    a = f32(a)
    out = np.empty(a.shape, np.uint16)
    lib().orc_from_f32(out.ctypes.data, a.ctypes.data, dt, a.size)
    return out


def round_to(a, dt):
    return to_f32(from_f32(a, dt), dt)


def build_sin_cos(nctx, dh, theta):
    s = np.empty((nctx, dh // 2), np.float32)
    c = np.empty((nctx, dh // 2), np.float32)
    lib().orc_build_sin_cos(nctx, dh, theta, s.ctypes.data, c.ctypes.data)
    return s, c


def rms_norm(x, w, eps, dt):
    x, w = f32(x), f32(w)
    y = np.empty_like(x)
    lib().orc_rms_norm(y.ctypes.data, x.ctypes.data, w.ctypes.data, x.shape[0], x.shape[1], eps, dt)
    return y


def linear(x, w, residual, dt):
    x, w = f32(x), f32(w)
    n, k = x.shape
    out = w.shape[0]
    y = np.empty((n, out), np.float32)
    r = None if residual is None else f32(residual)
    lib().orc_linear(y.ctypes.data, x.ctypes.data, w.ctypes.data, None if r is None else r.ctypes.data, n, k, out, dt)
    return y


def rope(x, nheads, dh, pos, sin_t, cos_t, dt):
    """x [n, nheads*dh] -> rotated copy."""
    y = f32(x).copy()
    pos = np.ascontiguousarray(pos, dtype=np.uint32)
    lib().orc_rope(y.ctypes.data, y.shape[0], nheads, dh, y.shape[1], pos.ctypes.data, f32(sin_t).ctypes.data,
                   f32(cos_t).ctypes.data, dt)
    return y


def swiglu(gate, up, dt):
    gate, up = f32(gate), f32(up)
    out = np.empty_like(gate)
    n, di = gate.shape
    lib().orc_swiglu(out.ctypes.data, di, gate.ctypes.data, di, up.ctypes.data, di, n, di, dt)
    return out


def attention(q, kc, vc, nh, nkvh, dh, pos, dt):
    """q [seq, nh*dh]; kc, vc [pos+seq, nkvh*dh] -> o [seq, nh*dh]."""
    q, kc, vc = f32(q), f32(kc), f32(vc)
    o = np.empty_like(q)
    lib().orc_attention(o.ctypes.data, nh * dh, q.ctypes.data, nh * dh, kc.ctypes.data, vc.ctypes.data, nh, nkvh, dh,
                        pos, q.shape[0], dt)
    return o


def argmax(logits):
    logits = f32(logits)
    i, v = C.c_uint32(), C.c_float()
    lib().orc_argmax(logits.ctypes.data, logits.size, C.byref(i), C.byref(v))
    return i.value, v.value


def sample(logits, random, temperature, topp, topk):
    logits = f32(logits)
    v = C.c_float()
    i = lib().orc_sample(logits.ctypes.data, logits.size, random, temperature, topp, min(topk, 2**63), C.byref(v))
    return int(i), v.value


class Model:
    """Whole-model oracle: weights converted to f32 once, one KV cache per sequence."""

    def __init__(self, cfg, weights, act_dtype=None, fill_seed=0):
        """cfg: a ModelConfig-like object; weights: {(layer, kind): uint16 bits | Q8_0 dict},
        or None to fill the model with cheap seeded values (timing only)."""
        self.cfg = cfg
        self.dt = cfg.act_dtype if act_dtype is None else act_dtype
        d = Desc(cfg.n_layers, cfg.d, cfg.nh, cfg.nkvh, cfg.dh, cfg.di, cfg.vocab, cfg.nctx, cfg.eps, cfg.theta, self.dt)
        self.m = lib().orc_model_new(C.byref(d))
        if weights is None:
            assert lib().orc_model_fill_synthetic(self.m, fill_seed) == 0
            return
        for (layer, kind), w in weights.items():
            if isinstance(w, dict):
                data, dt, count = w["blocks"], Q8_0, w["q"].size
            else:
                data, dt, count = np.ascontiguousarray(w), cfg.act_dtype, w.size
            rc = lib().orc_model_set_weight(self.m, max(layer, 0), kind, data.ctypes.data, dt, count)
            assert rc == 0, (layer, kind, rc)

    def __del__(self):
        if getattr(self, "m", None):
            lib().orc_model_free(self.m)
            self.m = None

    def seq_new(self):
        return lib().orc_seq_new(self.m)

    def seq_free(self, s):
        lib().orc_seq_free(self.m, s)

    def forward(self, reqs, tokens):
        """reqs: [(seq, pos, len)] -> (logits [n_req, vocab] f32, ids [n_req])."""
        n = len(reqs)
        seqs = np.array([r[0] for r in reqs], np.int32)
        pos0 = np.array([r[1] for r in reqs], np.uint32)
        lens = np.array([r[2] for r in reqs], np.uint32)
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        assert tokens.size == lens.sum()
        logits = np.empty((n, self.cfg.vocab), np.float32)
        ids = np.empty(n, np.uint32)
        rc = lib().orc_forward(self.m, n, seqs.ctypes.data, tokens.ctypes.data, lens.ctypes.data, pos0.ctypes.data,
                               logits.ctypes.data, ids.ctypes.data)
        if rc != 0:
            raise RuntimeError(f"orc_forward failed: {rc}")
        return logits, ids

    def last_times(self):
        """(seconds in the layers, seconds in the head) of the last forward."""
        a, b = C.c_double(), C.c_double()
        lib().orc_last_times(self.m, C.byref(a), C.byref(b))
        return a.value, b.value

    def last_hidden(self, n_tok):
        out = np.empty((self.cfg.n_layers + 1, n_tok, self.cfg.d), np.float32)
        assert lib().orc_last_hidden(self.m, out.ctypes.data, out.size) == n_tok
        return out

    def generate(self, prompts, steps):
        """Greedy decode mirroring llama_cu_b200.generate: staged prefill, then batched decode.
        Returns (ids [n][steps], logits [n][steps][vocab])."""
        seqs = [self.seq_new() for _ in prompts]
        ids = [[] for _ in prompts]
        lgs = [[] for _ in prompts]
        for i, p in enumerate(prompts):
            lg, t = self.forward([(seqs[i], 0, len(p))], p)
            ids[i].append(int(t[0]))
            lgs[i].append(lg[0])
        pos = [len(p) for p in prompts]
        for _ in range(steps - 1):
            reqs = [(seqs[i], pos[i], 1) for i in range(len(prompts))]
            lg, t = self.forward(reqs, [ids[i][-1] for i in range(len(prompts))])
            for i in range(len(prompts)):
                ids[i].append(int(t[i]))
                lgs[i].append(lg[i])
                pos[i] += 1
        for s in seqs:
            self.seq_free(s)
        return ids, lgs


# ------------------------------------------------------------------ reference kernels (GPU)
_ref = None


def ref_lib():
    """The reference's own kernels behind C entry points, or None when not built."""
    global _ref
    if _ref is None:
        if not os.path.exists(REF_LIB):
            return None
        R = C.CDLL(REF_LIB)
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        R.ref_rms_norm_f16.argtypes = [vp, i, vp, i, vp, i, f, i, i, vp]
        R.ref_rope_f16.argtypes = [vp, i, i, vp, i, i, vp, vp, vp, i, i, i, vp]
        R.ref_swiglu_f16.argtypes = [vp, i, vp, i, vp, i, i, i, vp]
        R.ref_embedding.argtypes = [vp, vp, vp, i, i, vp]
        R.ref_fast_embedding.argtypes = [vp, vp, vp, i, vp]
        R.calculate_workspace_size_half.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_size_t]
        R.argmax_half.argtypes = [vp, vp, C.c_size_t, vp, C.c_size_t, vp]
        R.sample_half.argtypes = [vp, vp, vp, C.c_size_t, f, f, f, C.c_size_t, vp, C.c_size_t, vp]
        _ref = R
    return _ref


def set_threads(n):
    """Sets the OpenMP thread count of the oracle (0 = leave as is); returns the count in effect."""
    return int(lib().orc_set_threads(int(n)))
