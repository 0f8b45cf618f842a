"""Model shapes of the benchmark configurations and seeded synthetic weights.

Tensor names, shapes and fused row orders follow llama.cu/src/model/mod.rs:61-182
(attn_qkv rows q|k|v, ffn_gate_up rows gate|up, weights [out, in] row-major).
Synthetic weights stand in for GGUF files: N(0, 0.02) linear/embedding weights, norm
weights 1.0, Q8_0 blocks of int8 ~U{-127..127} with an f16 scale ~U(1e-4, 4e-4).
"""
from dataclasses import dataclass, replace

import numpy as np

from . import (BF16, F16, F32, LINEAR_KINDS, Q8_0, W_ATTN_NORM, W_DOWN, W_EMBD, W_FFN_NORM, W_GATE_UP, W_LM_HEAD,
               W_O, W_OUT_NORM, W_QKV, Context, ModelDesc, check, load_library, stream_ptr)


@dataclass(frozen=True)
class ModelConfig:
    name: str
    n_layers: int
    d: int
    nh: int
    nkvh: int
    dh: int
    di: int
    vocab: int
    theta: float
    act_dtype: int = F16
    weight_dtype: int = -1  # -1: same as activations
    eps: float = 1e-5
    nctx: int = 2048

    @property
    def wdt(self):
        return self.act_dtype if self.weight_dtype < 0 else self.weight_dtype

    def desc(self, page_tokens=0, max_tokens=0, max_seqs=0, nctx=None):
        return ModelDesc(self.n_layers, self.d, self.nh, self.nkvh, self.dh, self.di, self.vocab,
                         nctx or self.nctx, self.eps, self.theta, self.act_dtype, self.wdt, self.act_dtype,
                         page_tokens, max_tokens, max_seqs)

    def shapes(self, tp=1):
        """(rows, cols) of every weight kind for one rank."""
        qd, kvd, di = self.nh // tp * self.dh, self.nkvh // tp * self.dh, self.di // tp
        return {W_EMBD: (self.vocab, self.d), W_ATTN_NORM: (self.d,), W_QKV: (qd + 2 * kvd, self.d),
                W_O: (self.d, qd), W_FFN_NORM: (self.d,), W_GATE_UP: (2 * di, self.d), W_DOWN: (self.d, di),
                W_OUT_NORM: (self.d,), W_LM_HEAD: (self.vocab, self.d)}

    def weight_bytes_per_step(self, tp=1):
        """Linear weights of every layer + LM head: the bytes one decode step must stream."""
        sh = self.shapes(tp)
        wb = 34.0 / 32.0 if self.wdt == Q8_0 else 2.0
        per_layer = sum(sh[k][0] * sh[k][1] for k in LINEAR_KINDS) * wb
        return per_layer * self.n_layers + self.vocab * self.d * 2.0

    def kv_bytes_per_token(self, tp=1):
        return self.n_layers * 2 * (self.nkvh // tp) * self.dh * 2


CONFIGS = {
    # BASELINE.json configs[0..4]
    "tiny": ModelConfig("tiny", 2, 256, 4, 4, 64, 688, 2048, 1e4, F16, nctx=1024),
    "llama1b": ModelConfig("llama1b", 16, 2048, 32, 8, 64, 8192, 128256, 5e5, BF16, nctx=2048),
    "llama8b": ModelConfig("llama8b", 32, 4096, 32, 8, 128, 14336, 128256, 5e5, F16, nctx=2048),
    "llama8b_q8": ModelConfig("llama8b_q8", 32, 4096, 32, 8, 128, 14336, 128256, 5e5, F16, Q8_0, nctx=2048),
    "llama70b": ModelConfig("llama70b", 80, 8192, 64, 8, 128, 28672, 32000, 1e4, F16, nctx=2048),
    # what ONE rank of the 70B shape computes under 8-way tensor parallelism (8 query heads, 1 KV head, 3584 FFN
    # columns; no all-reduce): a single-GPU stand-in for profiling the per-rank kernels
    "llama70b_tp8shard": ModelConfig("llama70b_tp8shard", 80, 8192, 8, 1, 128, 3584, 32000, 1e4, F16, nctx=2048),
}


def reduced(cfg, n_layers, vocab=None, name=None):
    """The same layer shape with fewer layers (and optionally a smaller vocabulary)."""
    return replace(cfg, n_layers=n_layers, vocab=vocab or cfg.vocab, name=name or f"{cfg.name}-L{n_layers}")


def f32_to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def q8_0_blocks(q, scales):
    """ggml Q8_0 byte layout (f16 scale then 32 int8) from planes q [rows, cols], scales [rows, cols/32]."""
    rows, cols = q.shape
    out = np.empty((rows * cols // 32, 34), np.uint8)
    out[:, :2] = scales.reshape(-1, 1).view(np.uint8)
    out[:, 2:] = q.reshape(-1, 32).view(np.uint8)
    return out.reshape(-1)


def synth_weights_numpy(cfg, seed=0):
    """Seeded weights as host arrays: {(layer, kind): array}.  Linear/embedding weights are
    uint16 bit patterns of the activation dtype; Q8_0 weights are dicts with `q`, `scales`
    (planes) and `blocks` (ggml bytes); norm weights are ones."""
    rng = np.random.default_rng(seed)
    sh = cfg.shapes()

    def dense(shape):
        w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        return w.astype(np.float16).view(np.uint16) if cfg.act_dtype == F16 else f32_to_bf16_bits(w)

    def linear(shape):
        if cfg.wdt != Q8_0:
            return dense(shape)
        q = rng.integers(-127, 128, size=shape, dtype=np.int8)
        sc = rng.uniform(1e-4, 4e-4, size=(shape[0], shape[1] // 32)).astype(np.float16)
        return {"q": q, "scales": sc, "blocks": q8_0_blocks(q, sc)}

    one = np.float16(1.0).view(np.uint16) if cfg.act_dtype == F16 else np.uint16(0x3F80)
    w = {(-1, W_EMBD): dense(sh[W_EMBD])}
    for l in range(cfg.n_layers):
        w[(l, W_ATTN_NORM)] = np.full(cfg.d, one, np.uint16)
        w[(l, W_QKV)] = linear(sh[W_QKV])
        w[(l, W_O)] = linear(sh[W_O])
        w[(l, W_FFN_NORM)] = np.full(cfg.d, one, np.uint16)
        w[(l, W_GATE_UP)] = linear(sh[W_GATE_UP])
        w[(l, W_DOWN)] = linear(sh[W_DOWN])
    w[(-1, W_OUT_NORM)] = np.full(cfg.d, one, np.uint16)
    w[(-1, W_LM_HEAD)] = dense(sh[W_LM_HEAD])
    return w


def synth_weights_torch(cfg, seed=0, device="cuda:0"):
    """Same distribution generated on the device (Philox), for shapes too large to draw on the host.
    Returns {(layer, kind): tensor}; Q8_0 weights come as one uint8 tensor in the plane layout."""
    return dict(iter_synth_weights_torch(cfg, seed, device))


def iter_synth_weights_torch(cfg, seed=0, device="cuda:0"):
    """Generator form of synth_weights_torch: yields ((layer, kind), tensor) one tensor at a time, so a
    tensor-parallel rank can slice each full tensor and drop it before the next one is drawn."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    tdt = torch.float16 if cfg.act_dtype == F16 else torch.bfloat16
    sh = cfg.shapes()

    def dense(shape):
        w = torch.empty(shape, dtype=tdt, device=device)
        w.normal_(0.0, 0.02, generator=g)
        return w

    def linear(shape):
        if cfg.wdt != Q8_0:
            return dense(shape)
        rows, cols = shape
        buf = torch.empty(rows * cols + rows * cols // 32 * 2, dtype=torch.uint8, device=device)
        q = torch.randint(-127, 128, (rows * cols,), dtype=torch.int8, device=device, generator=g)
        buf[:rows * cols] = q.view(torch.uint8)
        sc = torch.empty(rows * cols // 32, dtype=torch.float32, device=device).uniform_(1e-4, 4e-4, generator=g)
        buf[rows * cols:] = sc.to(torch.float16).view(torch.uint8)
        return buf

    yield (-1, W_EMBD), dense(sh[W_EMBD])
    for l in range(cfg.n_layers):
        yield (l, W_ATTN_NORM), torch.ones(cfg.d, dtype=tdt, device=device)
        yield (l, W_QKV), linear(sh[W_QKV])
        yield (l, W_O), linear(sh[W_O])
        yield (l, W_FFN_NORM), torch.ones(cfg.d, dtype=tdt, device=device)
        yield (l, W_GATE_UP), linear(sh[W_GATE_UP])
        yield (l, W_DOWN), linear(sh[W_DOWN])
    yield (-1, W_OUT_NORM), torch.ones(cfg.d, dtype=tdt, device=device)
    yield (-1, W_LM_HEAD), dense(sh[W_LM_HEAD])


def tp_slice_numpy(cfg, kind, full, rank, tp):
    """This rank's part of a full weight, as `TPAction::move_data` cuts it (llama.cu/src/load/mod.rs:86-99)
    with `Distribution{start=rank, len=1, total=tp}`: q, k, v row blocks by heads; O and down input columns;
    gate and up row blocks.  Other kinds are replicated."""
    dh, nh_l, nkvh_l, di_l = cfg.dh, cfg.nh // tp, cfg.nkvh // tp, cfg.di // tp
    if kind == W_QKV:
        q0, k0, v0 = 0, cfg.nh * dh, (cfg.nh + cfg.nkvh) * dh
        return np.concatenate([full[q0 + rank * nh_l * dh:q0 + (rank + 1) * nh_l * dh],
                               full[k0 + rank * nkvh_l * dh:k0 + (rank + 1) * nkvh_l * dh],
                               full[v0 + rank * nkvh_l * dh:v0 + (rank + 1) * nkvh_l * dh]])
    if kind == W_O:
        return np.ascontiguousarray(full[:, rank * nh_l * dh:(rank + 1) * nh_l * dh])
    if kind == W_GATE_UP:
        return np.concatenate([full[rank * di_l:(rank + 1) * di_l], full[cfg.di + rank * di_l:cfg.di + (rank + 1) * di_l]])
    if kind == W_DOWN:
        return np.ascontiguousarray(full[:, rank * di_l:(rank + 1) * di_l])
    return full


def load_model(cfg, weights, device=0, kv_bytes=None, tp_rank=0, tp_size=1, comm=None, page_tokens=0,
               max_tokens=0, max_seqs=0, nctx=None):
    """Creates a Context, uploads / registers `weights` (numpy from synth_weights_numpy or
    torch from synth_weights_torch; under TP the FULL tensors, sliced here per rank) and
    creates the KV pool."""
    import torch
    dev = f"cuda:{device}"
    ctx = Context(cfg.desc(page_tokens, max_tokens, max_seqs, nctx), device, tp_rank, tp_size, comm)
    lib = load_library()
    items = weights.items() if isinstance(weights, dict) else weights
    for (layer, kind), w in items:
        if isinstance(w, dict):  # Q8_0 from numpy: upload ggml blocks, repack on the device
            rows, cols = w["q"].shape
            blocks = torch.from_numpy(w["blocks"]).to(dev)
            t = torch.empty(lib.lcu_q8_0_repacked_bytes(rows, cols), dtype=torch.uint8, device=dev)
            check(lib.lcu_repack_q8_0(t.data_ptr(), blocks.data_ptr(), rows, cols, stream_ptr()))
            torch.cuda.synchronize(device)
        elif isinstance(w, np.ndarray):
            t = torch.from_numpy(w.view(np.int16)).to(dev)
        else:
            t = w
        # linear weights are cut per rank; the LM head stays whole on the lead rank and is cut by vocabulary rows on
        # the others (used when arg-max rounds shard the head, see lcu_set_head_sharding)
        if tp_size > 1 and (kind in LINEAR_KINDS or (kind == W_LM_HEAD and tp_rank != 0)):
            t = ctx.tp_slice(kind, t)
            torch.cuda.synchronize(device)
        ctx.set_weight(max(layer, 0), kind, t)
    if kv_bytes is None:
        kv_bytes = 64 * ctx.page_bytes
    ctx.kv_pool_create(int(kv_bytes))
    return ctx
