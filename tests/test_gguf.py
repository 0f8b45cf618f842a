"""GGUF files -> model description and tensor table (CPU) and -> device weights (GPU), against files written
with the `gguf` package in the reference's tensor naming (llama.cu/src/model/mod.rs:61-182)."""
import numpy as np
import pytest

from helpers import prompts_for, write_gguf


def small_cfg(L, q8=False, bf16=False):
    from llama_cu_b200.model import ModelConfig
    return ModelConfig("gg", 2, 128, 4, 2, 64, 256, 512, 5e5, L.BF16 if bf16 else L.F16, L.Q8_0 if q8 else -1, eps=1e-6, nctx=96)


@pytest.mark.parametrize("q8,bf16,shards,norm_f32", [(False, False, 1, True), (True, False, 2, True), (False, True, 3, False)])
def test_metadata_and_tensor_table(L, tmp_path, q8, bf16, shards, norm_f32):
    cfg = small_cfg(L, q8, bf16)
    w = L.synth_weights_numpy(cfg, 1)
    paths = [str(tmp_path / f"m-{i}.gguf") for i in range(shards)]
    write_gguf(paths, cfg, w, norm_f32=norm_f32)
    g = L.GGuf(paths)
    d = g.model_desc()
    assert (d.n_layers, d.d, d.nh, d.nkvh, d.dh, d.di, d.vocab, d.nctx) == (2, 128, 4, 2, 64, 256, 512, 96)
    assert abs(d.eps - 1e-6) < 1e-12 and d.theta == 5e5
    assert d.act_dtype == cfg.act_dtype and d.weight_dtype == cfg.wdt and d.norm_dtype == (L.F32 if norm_f32 else cfg.act_dtype)
    assert g.model_desc(nctx=40, max_seqs=3).nctx == 40           # the caller's context length wins
    assert g.meta_str("general.architecture") == "llama" and g.meta_u64("llama.block_count") == 2
    t = {name: (dt, dims, nb) for name, dt, dims, nb in g.tensors()}
    assert len(t) == 3 + 6 * 2
    assert t["token_embd.weight"][1] == (512, 128)                 # outermost first: [vocab, d]
    dt, dims, nb = t["blk.1.attn_qkv.weight"]
    assert dims == ((4 + 2 + 2) * 64, 128) and dt == cfg.wdt
    assert nb == (dims[0] * dims[1] // 32 * 34 if q8 else dims[0] * dims[1] * 2)
    assert t["blk.0.ffn_gate_up.weight"][1] == (512, 128) and t["blk.0.ffn_down.weight"][1] == (128, 256)
    assert t["output_norm.weight"][0] == (L.F32 if norm_f32 else cfg.act_dtype)
    g.close()


def test_rejects_what_the_reference_rejects(L, tmp_path):
    cfg = small_cfg(L)
    w = L.synth_weights_numpy(cfg, 1)
    a, b = str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")
    write_gguf(a, cfg, w)
    write_gguf(b, cfg, w)
    with pytest.raises(L.LcuError, match="appears twice"):         # DuplicateTensorName (model/gguf.rs:49-51)
        L.GGuf([a, b])
    write_gguf(b, cfg, w, extra_meta={"llama.block_count": 3})
    with pytest.raises(L.LcuError):                                # a key repeating with ANOTHER value
        L.GGuf([a, b])
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + bytes(64))
    with pytest.raises(L.LcuError, match="not a GGUF file"):
        L.GGuf(str(bad))
    with pytest.raises(L.LcuError, match="cannot read"):
        L.GGuf(str(tmp_path / "missing.gguf"))


@pytest.mark.gpu
@pytest.mark.parametrize("q8,shards,tied", [(False, 1, False), (True, 2, False), (False, 2, True)])
def test_loaded_model_generates_like_directly_registered_weights(L, O, tmp_path, q8, shards, tied):
    """lcu_gguf_load (pinned-slab upload, Q8_0 repack, registration) == registering the same arrays by hand."""
    cfg = small_cfg(L, q8)
    w = L.synth_weights_numpy(cfg, 1)
    if tied:
        w[(-1, L.W_LM_HEAD)] = w[(-1, L.W_EMBD)]
    paths = [str(tmp_path / f"m-{i}.gguf") for i in range(shards)]
    write_gguf(paths, cfg, w, tied=tied)
    prompts = prompts_for(cfg, [9, 30])
    ref = L.load_model(cfg, w)
    want = L.generate(ref, prompts, 10)
    ref.close()
    g = L.GGuf(paths)
    ctx = L.Context(g.model_desc(), 0)
    g.load(ctx)
    ctx.kv_pool_create(64 * ctx.page_bytes)
    got = L.generate(ctx, prompts, 10)
    assert got == want
    o_ids, _ = O.Model(cfg, w).generate(prompts, 10)
    assert got[0][:3] == o_ids[0][:3]
    ctx.close()
    g.close()


@pytest.mark.gpu
@pytest.mark.parametrize("kind_name", ["W_QKV", "W_O", "W_GATE_UP", "W_DOWN"])
def test_q8_0_planes_are_sliced_per_rank_like_the_dense_cut(L, kind_name):
    """lcu_tp_slice_weight on Q8_0 planes == tp_slice_numpy (TPAction::move_data) applied to quants and scales."""
    import ctypes as C
    import torch
    cfg = small_cfg(L, q8=True)
    kind = getattr(L, kind_name)
    w = L.synth_weights_numpy(cfg, 2)[(0, kind)]
    rows, cols = w["q"].shape
    planes = torch.from_numpy(np.concatenate([w["q"].reshape(-1).view(np.uint8), w["scales"].reshape(-1).view(np.uint8)])).cuda()
    for rank in range(2):
        ctx = L.Context(cfg.desc(), 0, rank, 2, C.c_void_p(1))     # the communicator is not touched by slicing
        got = ctx.tp_slice(kind, planes).cpu().numpy()
        q = L.tp_slice_numpy(cfg, kind, w["q"], rank, 2)
        sc = L.tp_slice_numpy(cfg.__class__(**{**cfg.__dict__, "dh": cfg.dh // 32, "di": cfg.di // 32}) if kind in (L.W_O, L.W_DOWN) else cfg,
                              kind, w["scales"], rank, 2)
        want = np.concatenate([np.ascontiguousarray(q).reshape(-1).view(np.uint8), np.ascontiguousarray(sc).reshape(-1).view(np.uint8)])
        assert got.size == want.size == ctx.weight_bytes(kind)
        assert np.array_equal(got, want)
        ctx.close()
