"""Step-level parity of BATCHED decode rounds against the CPU oracle (needs a B200).

Rounds of 9..64 sequences take the tcgen05 kernels (stream-K and cluster split-K forms),
the scratch-merge split-KV attention, the 64-row LM-head GEMM and one arg-max launch pair
for all rows, replayed from a CUDA graph — none of which a round of one to three sequences
reaches.  Every case is teacher-forced (the oracle's ids are fed back), so each step is an
independent comparison: logits within the stated tolerance, the GPU's own arg-max equal to
the oracle's (counted; a difference is accepted only where the oracle's top-2 margin is
inside the measured logit error), device status word zero.
"""
import numpy as np
import pytest
import torch

from helpers import device_weights, parity_report, teacher_forced_decode

pytestmark = pytest.mark.gpu

TOL = {0: 2e-2, 1: 8e-2}  # max-abs logits: f16 (north-star figure), bf16 (8 mantissa bits: 4x)


def ragged_lengths(n, long_ones, lo=4, hi=48, seed=7):
    """n prompt lengths: a few long contexts (so split-KV attention really merges) among short ones."""
    rng = np.random.default_rng(seed)
    ls = [int(x) for x in rng.integers(lo, hi + 1, n)]
    for k, v in enumerate(long_ones):
        ls[(k * 5 + 1) % n] = v
    return ls


def run_case(L, O, cfg, lengths, steps, graph, free_running=True, seed=0, **kw):
    dev_w, host_w = device_weights(L, cfg, seed)
    rng = np.random.default_rng(11)
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in lengths]
    orc = O.Model(cfg, host_w)
    o_ids, o_lgs = orc.generate(prompts, steps)
    del orc
    kv = (sum(lengths) + len(lengths) * (steps + 64)) * cfg.kv_bytes_per_token() + (8 << 20)
    ctx = L.load_model(cfg, dev_w, kv_bytes=kv, max_seqs=max(len(lengths), 1), **kw)
    ctx.set_cuda_graph(graph)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        g_lgs, g_ids = teacher_forced_decode(ctx, prompts, o_ids, steps, stream=stream)
    tol = TOL[cfg.act_dtype]
    worst, exact, total, off = parity_report(g_lgs, g_ids, o_lgs, o_ids, tol)
    print(f"[parity] {cfg.name} seqs={len(lengths)} steps={steps} graph={graph}: max|dlogit|={worst:.4g} "
          f"argmax equal {exact}/{total}, launches/step={ctx.last_launch_count}")
    assert worst <= tol, f"logits differ by {worst} (> {tol})"
    for i, s, margin in off:
        assert margin <= 2 * worst + 1e-6, f"seq {i} step {s}: arg-max differs where the oracle's margin is {margin}"
    assert ctx.device_status() == 0
    if free_running:  # device-side token feedback (fast_map) through the session layer
        ids = L.generate(ctx, prompts, steps)
        for i in range(len(prompts)):
            for s in range(steps):
                if ids[i][s] != o_ids[i][s]:
                    lg = np.sort(o_lgs[i][s])
                    assert lg[-1] - lg[-2] <= 2 * worst + 1e-6, (i, s, float(lg[-1] - lg[-2]))
                    break
        assert ctx.device_status() == 0
    ctx.close()
    return worst, exact, total


@pytest.mark.parametrize("graph", [True, False])
def test_8b_cut_32_sequences_ragged(L, O, graph):
    """8B f16 widths, 2 layers, vocab 4096: 32 sequences, contexts 4..1000 -> stream-K tcgen05 GEMMs,
    split-KV attention merging through scratch (contexts beyond 256 positions), 32-row head."""
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS["llama8b"], 2, 4096)
    lengths = ragged_lengths(32, [1000, 520, 300, 129])
    run_case(L, O, cfg, lengths, 8, graph, free_running=graph)


@pytest.mark.parametrize("n", [12, 40])
def test_8b_cut_12_and_40_sequences(L, O, n):
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS["llama8b"], 2, 4096)
    run_case(L, O, cfg, ragged_lengths(n, [270, 70], seed=n), 8, True)


def test_8b_q8_cut_16_sequences(L, O):
    """Q8_0 weights, 16 sequences: the mma.sync kernel's Q8_0 form in every projection."""
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS["llama8b_q8"], 2, 4096)
    run_case(L, O, cfg, ragged_lengths(16, [300, 130]), 8, True)


def test_1b_cut_bf16_24_sequences(L, O):
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS["llama1b"], 2, 4096)
    run_case(L, O, cfg, ragged_lengths(24, [400, 200]), 8, True)


def test_70b_rank_widths_64_sequences(L, O):
    """One rank's widths of the 70B shape under 8-way tensor parallelism (d 8192, 8 query heads, 1 KV head,
    3584 FFN columns), 2 layers, vocab 4096, 64 sequences: the cluster split-K form of the tcgen05 kernel."""
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS["llama70b_tp8shard"], 2, 4096)
    run_case(L, O, cfg, ragged_lengths(64, [600, 260], hi=24), 6, True)


def test_70b_full_widths_cut(L, O):
    """Config 5 widths (d 8192, 64 heads, FFN 28672, vocab 32000), 2 layers, 20 sequences on one GPU."""
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS["llama70b"], 2, 32000)
    run_case(L, O, cfg, ragged_lengths(20, [280], hi=16), 5, True, free_running=False)
