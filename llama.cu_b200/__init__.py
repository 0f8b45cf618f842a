"""ctypes binding of liblcu.so — the B200 decode token loop behind a C-ABI.

The directory name contains a dot, so load this package by path (see `llama_cu_b200.py`
at the repository root) rather than with a plain import statement.

Nothing here computes: every call goes to the CUDA library, and loading fails loudly
when the library has not been built (`python llama.cu_b200/build.py`).  PyTorch is used
only to own device memory and streams.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblcu.so")

F16, BF16, F32, Q8_0, U32 = 0, 1, 2, 3, 4
W_EMBD, W_ATTN_NORM, W_QKV, W_O, W_FFN_NORM, W_GATE_UP, W_DOWN, W_OUT_NORM, W_LM_HEAD = range(9)
LINEAR_KINDS = (W_QKV, W_O, W_GATE_UP, W_DOWN)
NO_OUTPUT = 2**64 - 1  # LCU_ENGINE_NO_OUTPUT: a prefill chunk that samples nothing
OK, ERR_INVALID, ERR_CUDA, ERR_OVERFLOW, ERR_NO_PAGES, ERR_STATE, ERR_COMM, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7


class LcuError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"liblcu error {code}: {msg}")
        self.code = code


class ModelDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d", "nh", "nkvh", "dh", "di", "vocab", "nctx")] + [
        ("eps", C.c_float), ("theta", C.c_float)] + [
        (n, C.c_int32) for n in ("act_dtype", "weight_dtype", "norm_dtype", "page_tokens", "max_tokens", "max_seqs")]


class KVPair(C.Structure):
    _fields_ = [("idx", C.c_uint32), ("val", C.c_uint16), ("pad", C.c_uint16)]


class SampleArgs(C.Structure):
    """Mirror of `SampleArgs` (llama.cu/src/op/random_sample/mod.rs:38-83)."""
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_uint64)]

    @classmethod
    def arg_max(cls):
        return cls(0.0, 1.0, 2**64 - 1)

    @classmethod
    def new(cls, temperature, top_p, top_k):
        if temperature < 0:
            raise ValueError("NegativeTemperature")
        if top_k == 0 or top_p <= 0:
            raise ValueError("NonPositiveTop")
        return cls(temperature, min(top_p, 1.0), top_k)

    def is_argmax(self):
        return self.temperature == 0.0 or self.top_k == 1


class Req(C.Structure):
    _fields_ = [("seq", C.c_int32), ("pos", C.c_uint32), ("len", C.c_uint32)]


class RoundInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_tok", "n_req", "n_fast", "n_finished", "n_overflow")]


_lib = None


def _p(*a):
    return list(a)


_SIGNATURES = {
    "lcu_last_error_string": (C.c_char_p, []),
    "lcu_version": (C.c_int, []),
    "lcu_ctx_create": (C.c_int, [C.POINTER(ModelDesc), C.c_int, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "lcu_ctx_destroy": (C.c_int, [C.c_void_p]),
    "lcu_set_weight": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t]),
    "lcu_weight_bytes": (C.c_size_t, [C.c_void_p, C.c_int]),
    "lcu_set_rope_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "lcu_build_sin_cos": (C.c_int, [C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]),
    "lcu_q8_0_repacked_bytes": (C.c_size_t, [C.c_size_t, C.c_size_t]),
    "lcu_repack_q8_0": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "lcu_tp_slice_weight": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lcu_kv_pool_create": (C.c_int, [C.c_void_p, C.c_size_t]),
    "lcu_kv_pool_attach": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "lcu_kv_page_tokens": (C.c_int, [C.c_void_p]),
    "lcu_kv_page_bytes": (C.c_size_t, [C.c_void_p]),
    "lcu_kv_pages_total": (C.c_int, [C.c_void_p]),
    "lcu_kv_pages_free": (C.c_int, [C.c_void_p]),
    "lcu_seq_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "lcu_seq_resize": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32]),
    "lcu_seq_len": (C.c_int, [C.c_void_p, C.c_int]),
    "lcu_seq_free": (C.c_int, [C.c_void_p, C.c_int]),
    "lcu_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(Req), C.c_void_p, C.POINTER(SampleArgs),
                           C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "lcu_logits": (C.c_void_p, [C.c_void_p]),
    "lcu_hidden": (C.c_void_p, [C.c_void_p]),
    "lcu_device_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)]),
    "lcu_set_tuning": (C.c_int, [C.c_void_p, C.c_char_p, C.c_longlong]),
    "lcu_reset_status": (C.c_int, [C.c_void_p]),
    "lcu_set_wait_limit_us": (C.c_int, [C.c_void_p, C.c_longlong]),
    "lcu_set_head_sharding": (C.c_int, [C.c_void_p, C.c_int]),
    "lcu_set_cuda_graph": (C.c_int, [C.c_void_p, C.c_int]),
    "lcu_last_launch_count": (C.c_int, [C.c_void_p]),
    "lcu_last_step_bytes": (C.c_double, [C.c_void_p]),
    "lcu_engine_create": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(C.c_void_p)]),
    "lcu_engine_destroy": (C.c_int, [C.c_void_p]),
    "lcu_engine_session_new": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(SampleArgs), C.POINTER(C.c_uint64)]),
    "lcu_engine_start": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint32, C.c_int]),
    "lcu_engine_remove": (C.c_int, [C.c_void_p, C.c_uint64]),
    "lcu_engine_session_pos": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32)]),
    "lcu_engine_session_set_pos": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32]),
    "lcu_engine_prepare": (C.c_int, [C.c_void_p, C.POINTER(RoundInfo)]),
    "lcu_engine_round_tokens": (C.POINTER(C.c_uint32), [C.c_void_p]),
    "lcu_engine_round_reqs": (C.POINTER(Req), [C.c_void_p]),
    "lcu_engine_round_fast_map": (C.POINTER(C.c_uint32), [C.c_void_p]),
    "lcu_engine_round_sample_args": (C.POINTER(SampleArgs), [C.c_void_p]),
    "lcu_engine_round_output": (C.POINTER(C.c_uint64), [C.c_void_p]),
    "lcu_engine_round_finished": (C.POINTER(C.c_uint64), [C.c_void_p]),
    "lcu_engine_round_overflow": (C.POINTER(C.c_uint64), [C.c_void_p]),
    "lcu_engine_round_positions": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "lcu_engine_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(RoundInfo)]),
    "lcu_engine_set_budget": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32]),
    "lcu_engine_cache_insert": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint32]),
    "lcu_engine_cache_send": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(SampleArgs), C.c_int,
                                        C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]),
    "lcu_engine_cache_count": (C.c_int, [C.c_void_p]),
    "lcu_engine_set_seed": (C.c_int, [C.c_void_p, C.c_uint64]),
    "lcu_engine_draw_randoms": (C.c_int, [C.c_void_p]),
    "lcu_engine_round_randoms": (C.POINTER(C.c_float), [C.c_void_p]),
    "lcu_gguf_open": (C.c_int, [C.POINTER(C.c_char_p), C.c_int, C.POINTER(C.c_void_p)]),
    "lcu_gguf_close": (C.c_int, [C.c_void_p]),
    "lcu_gguf_n_tensors": (C.c_int, [C.c_void_p]),
    "lcu_gguf_tensor_info": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_uint64),
                                       C.POINTER(C.c_int), C.POINTER(C.c_size_t)]),
    "lcu_gguf_meta_u64": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "lcu_gguf_meta_f32": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_float)]),
    "lcu_gguf_meta_str": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "lcu_gguf_model_desc": (C.c_int, [C.c_void_p, C.POINTER(ModelDesc)]),
    "lcu_gguf_load": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "lcu_op_embedding": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "lcu_op_fast_embedding": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "lcu_op_rms_norm": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_int,
                                  C.c_int, C.c_int, C.c_void_p]),
    "lcu_op_linear": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "lcu_op_rope": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                              C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "lcu_op_swiglu": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                C.c_int, C.c_void_p]),
    "lcu_op_add": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int,
                             C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "lcu_op_attention_kv_cached": (C.c_int, [C.c_void_p, C.c_int, C.c_int] * 6 + [C.c_int] * 6 + [C.c_void_p]),
    "lcu_op_all_reduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "lcu_calculate_workspace_size_half": (C.c_int, [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_size_t]),
    "lcu_argmax_half": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lcu_sample_half": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_float,
                                  C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lcu_sample_rows_workspace_size": (C.c_size_t, [C.c_int, C.c_size_t]),
    "lcu_op_sample_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p, C.c_void_p,
                                     C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lcu_argmax_rows_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_void_p]),
    "lcu_comm_unique_id": (C.c_int, [C.c_void_p]),
    "lcu_comm_init_rank": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "lcu_comm_destroy": (C.c_int, [C.c_void_p]),
    "lcu_p2p_create": (C.c_int, [C.c_void_p, C.c_void_p]),
    "lcu_p2p_attach": (C.c_int, [C.c_void_p, C.c_void_p]),
    "lcu_p2p_enabled": (C.c_int, [C.c_void_p]),
}


def load_library():
    """Loads liblcu.so once; raises if it has not been built — there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python llama.cu_b200/build.py` "
                           "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def exported_symbols():
    return sorted(_SIGNATURES)


def last_error():
    return load_library().lcu_last_error_string().decode()


def check(rc):
    if rc != 0:
        raise LcuError(rc, last_error())


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array, or None."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


TORCH_DT = None


def torch_dtype(dt):
    import torch
    return {F16: torch.float16, BF16: torch.bfloat16, F32: torch.float32}[dt]


def set_tuning(key, value, ctx=None):
    """Process-wide tuning value (lcu_set_tuning); `ctx` drops its captured rounds."""
    check(load_library().lcu_set_tuning(ctx.h if ctx is not None else None, key.encode(), int(value)))


def build_sin_cos(nctx, dh, theta):
    """Host tables [nctx, dh/2] exactly as `build_sin_cos` (llama.cu/src/model/mod.rs:186-220)."""
    sin = np.empty((nctx, dh // 2), np.float32)
    cos = np.empty((nctx, dh // 2), np.float32)
    check(load_library().lcu_build_sin_cos(nctx, dh, theta, sin.ctypes.data, cos.ctypes.data))
    return sin, cos


class Context:
    """One GPU's share of a model: weights, KV pages, activation arena, step graphs.

    Mirrors what `Handle` + `ModelGroup` + `OutputHead` hold in the reference
    (llama.cu/src/handle.rs, exec/group.rs, exec/output_head.rs).
    """

    def __init__(self, desc: ModelDesc, device=0, tp_rank=0, tp_size=1, comm=None):
        self.lib = load_library()
        self.desc = desc
        self.device = device
        self.tp_rank, self.tp_size = tp_rank, tp_size
        h = C.c_void_p()
        check(self.lib.lcu_ctx_create(C.byref(desc), device, tp_rank, tp_size, comm, C.byref(h)))
        self.h = h
        self._keep = []  # tensors registered with the library stay alive here

    def close(self):
        if self.h:
            self.lib.lcu_ctx_destroy(self.h)
            self.h = None
            self._keep.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights
    def weight_bytes(self, kind):
        return self.lib.lcu_weight_bytes(self.h, kind)

    def set_weight(self, layer, kind, tensor):
        nbytes = tensor.numel() * tensor.element_size()
        check(self.lib.lcu_set_weight(self.h, layer, kind, tensor.data_ptr(), nbytes))
        self._keep.append(tensor)

    def set_rope_tables(self, sin_dev, cos_dev):
        check(self.lib.lcu_set_rope_tables(self.h, sin_dev.data_ptr(), cos_dev.data_ptr()))
        self._keep += [sin_dev, cos_dev]

    def tp_slice(self, kind, full, stream=None):
        import torch
        out = torch.empty(self.weight_bytes(kind), dtype=torch.uint8, device=full.device)
        check(self.lib.lcu_tp_slice_weight(self.h, kind, out.data_ptr(), full.data_ptr(), stream_ptr(stream)))
        return out

    # ---- KV pages
    def kv_pool_create(self, nbytes):
        check(self.lib.lcu_kv_pool_create(self.h, nbytes))

    def kv_pool_attach(self, tensor):
        check(self.lib.lcu_kv_pool_attach(self.h, tensor.data_ptr(), tensor.numel() * tensor.element_size()))
        self._keep.append(tensor)

    @property
    def page_tokens(self):
        return self.lib.lcu_kv_page_tokens(self.h)

    @property
    def page_bytes(self):
        return self.lib.lcu_kv_page_bytes(self.h)

    @property
    def pages_free(self):
        return self.lib.lcu_kv_pages_free(self.h)

    @property
    def pages_total(self):
        return self.lib.lcu_kv_pages_total(self.h)

    def seq_create(self):
        s = C.c_int()
        check(self.lib.lcu_seq_create(self.h, C.byref(s)))
        return s.value

    def seq_resize(self, seq, length):
        check(self.lib.lcu_seq_resize(self.h, seq, length))

    def seq_len(self, seq):
        return self.lib.lcu_seq_len(self.h, seq)

    def seq_free(self, seq):
        check(self.lib.lcu_seq_free(self.h, seq))

    # ---- the round
    def step(self, reqs, tokens, out, args=None, randoms=None, fast_map=None, stream=None):
        """reqs: [(seq, pos, len)]; tokens: flat uint32 host array; out: device tensor of
        n_req KVPair (8 bytes each).  Returns without synchronising."""
        n = len(reqs)
        creqs = (Req * n)(*[Req(*r) for r in reqs])
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        cargs = None
        if args is not None:
            cargs = (SampleArgs * n)(*args)
        rnd = None if randoms is None else np.ascontiguousarray(randoms, dtype=np.float32)
        fm = None if fast_map is None else np.ascontiguousarray(fast_map, dtype=np.uint32).reshape(-1, 2)
        check(self.lib.lcu_step(self.h, stream_ptr(stream), n, creqs, tokens.ctypes.data, cargs, ptr(rnd), ptr(fm),
                                0 if fm is None else len(fm), ptr(out)))

    def logits(self, n_req):
        """The last round's logits [n_req, vocab] (a copy, after synchronising)."""
        import torch
        torch.cuda.synchronize(self.device)
        return _view(self.lib.lcu_logits(self.h), n_req * self.desc.vocab, self.desc.act_dtype,
                     self.device).view(n_req, self.desc.vocab).clone()

    def hidden(self, n_tok):
        """The residual stream after the last layer of the last round, [n_tok, d] (a copy)."""
        import torch
        torch.cuda.synchronize(self.device)
        return _view(self.lib.lcu_hidden(self.h), n_tok * self.desc.d, self.desc.act_dtype,
                     self.device).view(n_tok, self.desc.d).clone()

    def device_status(self, stream=None):
        v = C.c_uint32()
        check(self.lib.lcu_device_status(self.h, stream_ptr(stream), C.byref(v)))
        return v.value

    def reset_status(self):
        check(self.lib.lcu_reset_status(self.h))

    def set_wait_limit_us(self, us):
        check(self.lib.lcu_set_wait_limit_us(self.h, int(us)))

    def set_head_sharding(self, enabled):
        check(self.lib.lcu_set_head_sharding(self.h, int(enabled)))

    def set_cuda_graph(self, enabled):
        check(self.lib.lcu_set_cuda_graph(self.h, int(enabled)))

    def p2p_connect(self, all_gather_bytes):
        """Switches tensor parallelism from NCCL to NVLink peer memory.  `all_gather_bytes(b)` must return
        the list of every rank's 64-byte `b` in rank order (e.g. built on `torch.distributed.all_gather_object`);
        all ranks call this together."""
        buf = (C.c_ubyte * 64)()
        check(self.lib.lcu_p2p_create(self.h, buf))
        handles = all_gather_bytes(bytes(buf))
        blob = b"".join(handles)
        check(self.lib.lcu_p2p_attach(self.h, C.c_char_p(blob)))

    @property
    def p2p_enabled(self):
        return bool(self.lib.lcu_p2p_enabled(self.h))

    @property
    def last_launch_count(self):
        return self.lib.lcu_last_launch_count(self.h)

    @property
    def last_step_bytes(self):
        return self.lib.lcu_last_step_bytes(self.h)


class GGuf:
    """A (possibly split) GGUF model: metadata, tensor table, upload into a Context (`lcu_gguf_*`)."""

    def __init__(self, paths):
        self.lib = load_library()
        paths = [paths] if isinstance(paths, (str, bytes, os.PathLike)) else list(paths)
        arr = (C.c_char_p * len(paths))(*[os.fsencode(p) for p in paths])
        h = C.c_void_p()
        check(self.lib.lcu_gguf_open(arr, len(paths), C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.lib.lcu_gguf_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensors(self):
        """[(name, lcu dtype, dims outermost first, bytes)] in file order."""
        out = []
        for i in range(self.lib.lcu_gguf_n_tensors(self.h)):
            name, dt, nd, nb = C.c_char_p(), C.c_int(), C.c_int(), C.c_size_t()
            dims = (C.c_uint64 * 4)()
            check(self.lib.lcu_gguf_tensor_info(self.h, i, C.byref(name), C.byref(dt), dims, C.byref(nd), C.byref(nb)))
            out.append((name.value.decode(), dt.value, tuple(dims[:nd.value]), nb.value))
        return out

    def meta_u64(self, key):
        v = C.c_uint64()
        check(self.lib.lcu_gguf_meta_u64(self.h, key.encode(), C.byref(v)))
        return v.value

    def meta_f32(self, key):
        v = C.c_float()
        check(self.lib.lcu_gguf_meta_f32(self.h, key.encode(), C.byref(v)))
        return v.value

    def meta_str(self, key):
        n = C.c_size_t()
        check(self.lib.lcu_gguf_meta_str(self.h, key.encode(), None, 0, C.byref(n)))
        buf = C.create_string_buffer(n.value + 1)
        check(self.lib.lcu_gguf_meta_str(self.h, key.encode(), buf, n.value + 1, None))
        return buf.value.decode()

    def model_desc(self, nctx=0, page_tokens=0, max_tokens=0, max_seqs=0):
        d = ModelDesc()
        d.nctx, d.page_tokens, d.max_tokens, d.max_seqs = nctx, page_tokens, max_tokens, max_seqs
        check(self.lib.lcu_gguf_model_desc(self.h, C.byref(d)))
        return d

    def load(self, ctx, stream=None):
        """Uploads this rank's weights into `ctx` (the handle owns the device memory: keep it alive)."""
        import torch
        with torch.cuda.device(ctx.device):
            check(self.lib.lcu_gguf_load(self.h, ctx.h, stream_ptr(stream)))
        ctx._keep.append(self)


class _RawDevice:
    """Zero-copy view of library-owned device memory through __cuda_array_interface__."""

    def __init__(self, address, n_elems):
        self.__cuda_array_interface__ = {"shape": (n_elems,), "typestr": "<i2", "data": (address, False),
                                         "version": 2}


def _view(address, n_elems, dt, device):
    import torch
    t = torch.as_tensor(_RawDevice(address, n_elems), device=f"cuda:{device}")
    return t.view(torch_dtype(dt))


from .model import (CONFIGS, ModelConfig, iter_synth_weights_torch, load_model, synth_weights_numpy,  # noqa: E402,F401
                    synth_weights_torch, tp_slice_numpy)
from .host import Service, Session, StepRendezvous, generate, generate_continuous  # noqa: E402,F401
