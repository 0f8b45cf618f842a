"""Noise floor of the logits between two independent CPU restatements of the same forward pass as depth grows.

Both the C oracle (oracle/lcu_oracle.c) and the PyTorch restatement (tests/torch_ref.py) accumulate in f32 and
round to the activation dtype at every operator boundary; they differ only in summation order.  A flipped
rounding early in the network perturbs everything after it, so their max-abs logit difference grows with
depth.  That difference is the floor below which no implementation with its own summation order (cuBLAS, the
kernels here) can be expected to agree, and it is what the full-depth GPU test's tolerance is derived from.

    python tests/golden/noise_floor.py llama8b 2,8,16      (from the repository root; minutes on 8 cores)

Prints one line per depth and a JSON summary; the committed results are in tests/golden/noise_floor.json.
Case: the named shape cut to the given number of layers, vocabulary 4096, one 32-token prompt, 4 greedy steps."""
import sys, time, json
import numpy as np
import os
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, 'tests')]
import llama_cu_b200 as L
from llama_cu_b200.model import reduced
from oracle import oracle as O
from torch_ref import TorchModel
name = sys.argv[1]
res = {}
for layers in [int(x) for x in sys.argv[2].split(',')]:
    cfg = reduced(L.CONFIGS[name], layers, 4096)
    t = time.time()
    w = L.synth_weights_numpy(cfg, 0)
    prompt = np.random.default_rng(5).integers(3, cfg.vocab, 32).astype(np.uint32)
    ids, lgs = O.Model(cfg, w).generate([prompt], 4)
    m = TorchModel(cfg, w)
    worst = 0.0
    lg, tk = m.forward([(0, 0, len(prompt))], prompt)
    worst = max(worst, float(np.abs(lg[0] - lgs[0][0]).max()))
    pos = len(prompt)
    for s in range(3):
        lg, tk = m.forward([(0, pos, 1)], [ids[0][s]])
        worst = max(worst, float(np.abs(lg[0] - lgs[0][s + 1]).max()))
        pos += 1
    res[layers] = worst
    print(name, layers, worst, "absmax logit", float(np.abs(lgs[0][0]).max()), "t=%.0fs" % (time.time() - t), flush=True)
print(json.dumps(res))
