"""Generates the golden vectors in this directory.

The reference ships no golden vectors for the decode path and its binary cannot be built
here, so these are produced by the independent PyTorch fp32 restatement in
tests/torch_ref.py (NOT by the C oracle they are used to check) on the seeded synthetic
models and prompts of the benchmark configurations.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

import llama_cu_b200 as L  # noqa: E402
from llama_cu_b200.model import reduced  # noqa: E402
from torch_ref import TorchModel  # noqa: E402

CASES = {
    # name: (config, layers/vocab override, prompt lengths, steps, weight seed, prompt seed)
    "tiny": ("tiny", None, [16], 32, 0, 1),
    "tiny_batch": ("tiny", None, [5, 16, 33], 8, 0, 2),
    "llama1b_L1": ("llama1b", (1, 2048), [12], 4, 3, 4),
    "llama8b_q8_L1": ("llama8b_q8", (1, 1024), [9], 3, 5, 6),
    # the reduced shape bench.py checks its tensor-parallel transports on before timing (8 KV heads: TP 2/4/8)
    "llama8b_L2_tp": ("llama8b", (2, 2048), [5, 9, 40], 8, 7, 8),
}


def run_case(name):
    cname, red, lengths, steps, wseed, pseed = CASES[name]
    cfg = L.CONFIGS[cname]
    if red:
        cfg = reduced(cfg, red[0], red[1])
    w = L.synth_weights_numpy(cfg, wseed)
    rng = np.random.default_rng(pseed)
    prompts = [rng.integers(3, cfg.vocab, n).astype(np.uint32) for n in lengths]
    m = TorchModel(cfg, w)
    ids = [[] for _ in prompts]
    margins = [[] for _ in prompts]
    probes = [[] for _ in prompts]
    pos = []
    for i, p in enumerate(prompts):
        lg, t = m.forward([(i, 0, len(p))], p)
        ids[i].append(int(t[0]))
        s = np.sort(lg[0])
        margins[i].append(float(s[-1] - s[-2]))
        probes[i].append([float(lg[0][j]) for j in (0, 1, cfg.vocab // 2, cfg.vocab - 1, int(t[0]))])
        pos.append(len(p))
    for _ in range(steps - 1):
        reqs = [(i, pos[i], 1) for i in range(len(prompts))]
        lg, t = m.forward(reqs, [ids[i][-1] for i in range(len(prompts))])
        for i in range(len(prompts)):
            ids[i].append(int(t[i]))
            s = np.sort(lg[i])
            margins[i].append(float(s[-1] - s[-2]))
            probes[i].append([float(lg[i][j]) for j in (0, 1, cfg.vocab // 2, cfg.vocab - 1, int(t[i]))])
            pos[i] += 1
    return {"config": cname, "reduced": red, "lengths": lengths, "steps": steps, "weight_seed": wseed,
            "prompt_seed": pseed, "ids": ids, "top2_margin": margins, "logit_probes": probes}


if __name__ == "__main__":
    out = {name: run_case(name) for name in CASES}
    with open(os.path.join(HERE, "decode_golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", os.path.join(HERE, "decode_golden.json"))
