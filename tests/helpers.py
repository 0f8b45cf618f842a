"""Shared helpers of the parity tests."""
import numpy as np
import torch


def bits_to_torch(bits, dt, device="cuda:0"):
    """uint16 bit patterns -> torch tensor of the activation dtype on the device."""
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device)
    return t.view(torch.float16 if dt == 0 else torch.bfloat16)


def torch_to_f32(t):
    return t.detach().float().cpu().numpy()


def prompts_for(cfg, lengths, seed=1):
    """Token ids drawn uniformly from [3, vocab) as the benchmark configurations specify."""
    rng = np.random.default_rng(seed)
    return [rng.integers(3, cfg.vocab, int(n)).astype(np.uint32) for n in lengths]


def greedy_parity(gpu_ids, orc_ids, orc_logits, tol):
    """Compares greedy ids step by step.  Returns (n_equal_prefix, margin_at_divergence).
    A divergence counts as a failure only when the oracle's top-2 margin at that step
    exceeds `tol` (f16/bf16 ties between near-equal logits are legitimate)."""
    for i, (a, b) in enumerate(zip(gpu_ids, orc_ids)):
        if a != b:
            lg = np.sort(orc_logits[i])
            return i, float(lg[-1] - lg[-2])
    return len(orc_ids), None


class _LazyHostWeights:
    """dict-like view over device weights whose .items() yields host copies one tensor at a time,
    so that a full-size model never has a second complete host copy beside the oracle's f32 one."""

    def __init__(self, dev_weights, cfg):
        self.dev, self.cfg = dev_weights, cfg

    def items(self):
        for key, t in self.dev.items():
            yield key, host_weight(self.cfg, key[1], t)


def host_weight(cfg, kind, t):
    """Host form of one device weight as the oracle takes it: uint16 bit patterns, or for a Q8_0
    linear weight (plane layout on the device) the dict with the ggml 34-byte blocks."""
    from llama_cu_b200 import LINEAR_KINDS, Q8_0
    if cfg.wdt == Q8_0 and kind in LINEAR_KINDS:
        rows, cols = cfg.shapes()[kind]
        n = rows * cols
        q = t[:n].view(torch.int8).view(-1, 32)
        sc = t[n:].view(-1, 2)
        blocks = torch.cat([sc, q.view(torch.uint8)], dim=1).reshape(-1).cpu().numpy()
        return {"q": q.view(rows, cols).cpu().numpy(), "scales": sc.reshape(-1).cpu().numpy().view(np.float16).reshape(rows, cols // 32),
                "blocks": blocks}
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def device_weights(L, cfg, seed=0, device="cuda:0"):
    """Seeded synthetic weights drawn on the GPU (seconds even for the 8B shape, where the numpy
    generator needs minutes).  Returns (device dict for load_model, lazy host view for the oracle)."""
    dev = L.synth_weights_torch(cfg, seed, device)
    return dev, _LazyHostWeights(dev, cfg)


def teacher_forced_decode(ctx, prompts, o_ids, steps, stream=None):
    """Prefills every prompt alone, then decodes all sequences together for steps-1 rounds feeding the
    ORACLE's ids.  Returns (logits [n][steps][vocab] f32, ids the GPU picked [n][steps])."""
    n = len(prompts)
    dev = f"cuda:{ctx.device}"
    out = torch.zeros(max(n, 1), 2, dtype=torch.int32, device=dev)
    seqs = [ctx.seq_create() for _ in prompts]
    lgs = [[] for _ in prompts]
    ids = [[] for _ in prompts]

    def sync():
        if stream is not None:
            stream.synchronize()
        torch.cuda.synchronize(ctx.device)

    for i, p in enumerate(prompts):
        ctx.step([(seqs[i], 0, len(p))], p, out, stream=stream)
        sync()
        lgs[i].append(ctx.logits(1)[0].float().cpu().numpy())
        ids[i].append(int(out[0, 0].item()))
    pos = [len(p) for p in prompts]
    for s in range(steps - 1):
        reqs = [(seqs[i], pos[i], 1) for i in range(n)]
        ctx.step(reqs, np.array([o_ids[i][s] for i in range(n)], np.uint32), out, stream=stream)
        sync()
        lg = ctx.logits(n).float().cpu().numpy()
        got = out[:n, 0].cpu().numpy().view(np.uint32)
        for i in range(n):
            lgs[i].append(lg[i])
            ids[i].append(int(got[i]))
            pos[i] += 1
    for s in seqs:
        ctx.seq_free(s)
    return lgs, ids


def parity_report(g_lgs, g_ids, o_lgs, o_ids, tol):
    """Teacher-forced comparison.  Returns (worst |logit difference|, steps whose arg-max equals the
    oracle's, all steps, list of (seq, step, oracle margin) where it does not)."""
    worst, exact, total, off = 0.0, 0, 0, []
    for i in range(len(o_ids)):
        for s in range(len(o_ids[i])):
            worst = max(worst, float(np.abs(g_lgs[i][s] - o_lgs[i][s]).max()))
            total += 1
            if g_ids[i][s] == o_ids[i][s]:
                exact += 1
            else:
                lg = np.sort(o_lgs[i][s])
                off.append((i, s, float(lg[-1] - lg[-2])))
    return worst, exact, total, off


def write_gguf(paths, cfg, weights, norm_f32=True, tied=False, extra_meta=None):
    """Writes the model as GGUF with the reference's tensor naming (fused attn_qkv / ffn_gate_up) using the `gguf`
    package; `paths` with several entries splits the tensors round-robin over shards (metadata in the first shard,
    `general.architecture` — which the writer always emits — in all of them).  `weights` as from synth_weights_numpy."""
    import gguf
    from llama_cu_b200 import (F16, Q8_0, W_ATTN_NORM, W_DOWN, W_EMBD, W_FFN_NORM, W_GATE_UP, W_LM_HEAD, W_O, W_OUT_NORM,
                               W_QKV)
    paths = [paths] if isinstance(paths, str) else list(paths)
    writers = [gguf.GGUFWriter(p, "llama") for p in paths]
    w0 = writers[0]
    w0.add_block_count(cfg.n_layers)
    w0.add_context_length(cfg.nctx)
    w0.add_embedding_length(cfg.d)
    w0.add_head_count(cfg.nh)
    w0.add_head_count_kv(cfg.nkvh)
    w0.add_rope_dimension_count(cfg.dh)
    w0.add_feed_forward_length(cfg.di)
    w0.add_layer_norm_rms_eps(cfg.eps)
    w0.add_rope_freq_base(cfg.theta)
    w0.add_token_list([f"t{i}" for i in range(cfg.vocab)])
    for k, v in (extra_meta or {}).items():
        w0.add_uint32(k, v)
    for i, w in enumerate(writers[1:], 1):
        w.add_uint16("split.no", i)

    def dense(bits):
        if cfg.act_dtype == F16:
            return bits.view(np.float16), None
        return bits.view(np.uint8).reshape(bits.shape[0], -1), gguf.GGMLQuantizationType.BF16

    def norm(bits):
        if norm_f32:
            f = bits.view(np.float16).astype(np.float32) if cfg.act_dtype == F16 else (bits.astype(np.uint32) << 16).view(np.float32)
            return f, None
        return dense(bits.reshape(1, -1))[0].reshape(-1), (None if cfg.act_dtype == F16 else gguf.GGMLQuantizationType.BF16)

    def linear(w):
        if isinstance(w, dict):
            rows, cols = w["q"].shape
            return w["blocks"].reshape(rows, cols // 32 * 34), gguf.GGMLQuantizationType.Q8_0
        return dense(w)

    items = [("token_embd.weight", dense(weights[(-1, W_EMBD)]))]
    for l in range(cfg.n_layers):
        items += [(f"blk.{l}.attn_norm.weight", norm(weights[(l, W_ATTN_NORM)])),
                  (f"blk.{l}.attn_qkv.weight", linear(weights[(l, W_QKV)])),
                  (f"blk.{l}.attn_output.weight", linear(weights[(l, W_O)])),
                  (f"blk.{l}.ffn_norm.weight", norm(weights[(l, W_FFN_NORM)])),
                  (f"blk.{l}.ffn_gate_up.weight", linear(weights[(l, W_GATE_UP)])),
                  (f"blk.{l}.ffn_down.weight", linear(weights[(l, W_DOWN)]))]
    items.append(("output_norm.weight", norm(weights[(-1, W_OUT_NORM)])))
    if not tied:
        items.append(("output.weight", dense(weights[(-1, W_LM_HEAD)])))
    for i, (name, (arr, raw)) in enumerate(items):
        writers[i % len(writers)].add_tensor(name, np.ascontiguousarray(arr), raw_dtype=raw)
    for w in writers:
        w.write_header_to_file()
        w.write_kv_data_to_file()
        w.write_tensors_to_file()
        w.close()
