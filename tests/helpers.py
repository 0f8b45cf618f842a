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
