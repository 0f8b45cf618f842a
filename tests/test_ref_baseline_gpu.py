"""Second witness of whole-step parity (needs a B200 and oracle/_ref built from the reference tree).

The reference-kernel baseline (oracle/ref_step.cu: the reference's own kernels + cuBLAS + a restated attention,
launched the way the reference launches a round) runs the same seeded model and prompts as the CUDA library and
the CPU oracle; the three sets of logits must agree within the f16 tolerance at every teacher-forced step.
"""
import numpy as np
import pytest
import torch

from helpers import device_weights, parity_report, teacher_forced_decode

pytestmark = pytest.mark.gpu
TOL = 2e-2


def ref_teacher_forced(m, prompts, o_ids, steps):
    with torch.cuda.stream(torch.cuda.Stream()):  # the round captures graphs: not possible on the legacy default stream
        return _ref_teacher_forced(m, prompts, o_ids, steps)


def _ref_teacher_forced(m, prompts, o_ids, steps):
    n = len(prompts)
    out = torch.zeros(max(n, 1), 2, dtype=torch.int32, device="cuda:0")
    seqs = [m.seq_new() for _ in prompts]
    lgs, ids = [[] for _ in prompts], [[] for _ in prompts]
    for i, p in enumerate(prompts):
        m.round([(seqs[i], 0, len(p))], p, out)
        lgs[i].append(m.logits(1)[0].float().cpu().numpy())
        ids[i].append(int(out[0, 0].item()))
    pos = [len(p) for p in prompts]
    for s in range(steps - 1):
        m.round([(seqs[i], pos[i], 1) for i in range(n)], np.array([o_ids[i][s] for i in range(n)], np.uint32), out)
        lg = m.logits(n).float().cpu().numpy()
        got = out[:n, 0].cpu().numpy().view(np.uint32)
        for i in range(n):
            lgs[i].append(lg[i])
            ids[i].append(int(got[i]))
            pos[i] += 1
    return lgs, ids


@pytest.mark.parametrize("name,layers,vocab,lengths,steps", [
    ("tiny", 2, 2048, [16], 32),                # config 1 at its full shape
    ("tiny", 2, 2048, [5, 40, 70, 9], 8),       # several requests per round: bucket padding 4 -> 8
    ("llama8b", 2, 4096, [20, 70, 129], 8),     # config 3 widths
    ("llama8b", 2, 4096, [12] * 12, 4),         # a 12-request round in the 32 bucket
])
def test_reference_kernel_baseline_agrees_with_oracle_and_library(L, O, name, layers, vocab, lengths, steps):
    from oracle import ref_baseline as RB
    if RB.lib() is None:
        pytest.skip("oracle/_ref is not built (reference tree absent at build time)")
    from llama_cu_b200.model import reduced
    cfg = reduced(L.CONFIGS[name], layers, vocab)
    dev_w, host_w = device_weights(L, cfg, seed=0)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in lengths]
    o_ids, o_lgs = O.Model(cfg, host_w).generate(prompts, steps)
    m = RB.RefModel(cfg, dev_w)
    r_lgs, r_ids = ref_teacher_forced(m, prompts, o_ids, steps)
    m.close()
    ctx = L.load_model(cfg, dev_w, max_seqs=len(prompts))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        g_lgs, g_ids = teacher_forced_decode(ctx, prompts, o_ids, steps, stream=stream)
    assert ctx.device_status() == 0
    ctx.close()
    w_ro, ex_ro, total, off_ro = parity_report(r_lgs, r_ids, o_lgs, o_ids, TOL)
    w_go, ex_go, _, off_go = parity_report(g_lgs, g_ids, o_lgs, o_ids, TOL)
    w_gr = max(float(np.abs(g_lgs[i][s] - r_lgs[i][s]).max()) for i in range(len(prompts)) for s in range(steps))
    print(f"[ref-kernel witness] {cfg.name} {lengths}: |ref-oracle|={w_ro:.4g} ({ex_ro}/{total} ids), "
          f"|lib-oracle|={w_go:.4g} ({ex_go}/{total} ids), |lib-ref|={w_gr:.4g}")
    assert w_ro <= TOL and w_go <= TOL and w_gr <= TOL
    for i, s, margin in off_ro + off_go:
        assert margin <= 2 * max(w_ro, w_go) + 1e-6, (i, s, margin)
