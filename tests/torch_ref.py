"""An independent PyTorch (CPU, fp32) restatement of the forward pass, used to cross-check
the C oracle.  Written against the same reference sources (llama.cu/src/op/*.cuh,
op/linear.rs, model/mod.rs, exec/output_head.rs) but sharing no code with the oracle."""
import numpy as np
import torch

W_EMBD, W_ATTN_NORM, W_QKV, W_O, W_FFN_NORM, W_GATE_UP, W_DOWN, W_OUT_NORM, W_LM_HEAD = range(9)


def rnd(t, dt):
    if dt == 0:
        return t.half().float()
    if dt == 1:
        return t.bfloat16().float()
    return t


def bits_to_f32(bits, dt):
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16))
    return t.view(torch.float16 if dt == 0 else torch.bfloat16).float()


class TorchModel:
    def __init__(self, cfg, weights, act_dtype=None):
        self.cfg = cfg
        self.dt = cfg.act_dtype if act_dtype is None else act_dtype
        self.w = {}
        for key, w in weights.items():
            if isinstance(w, dict):
                q = torch.from_numpy(w["q"].astype(np.float32))
                sc = torch.from_numpy(w["scales"].astype(np.float32)).repeat_interleave(32, dim=1)
                self.w[key] = q * sc
            else:
                self.w[key] = bits_to_f32(w, cfg.act_dtype)
        half = cfg.dh // 2
        # f32 throughout, as build_sin_cos does
        i = torch.arange(half, dtype=torch.float32)
        inv = torch.pow(torch.tensor(cfg.theta, dtype=torch.float32), -(2 * i) / cfg.dh)
        ang = torch.arange(cfg.nctx, dtype=torch.float32)[:, None] * inv[None, :]
        self.sin, self.cos = torch.sin(ang), torch.cos(ang)
        self.cache = {}

    def norm(self, x, w):
        rms = torch.rsqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + self.cfg.eps)
        return rnd(rms * x * w, self.dt)

    def rope(self, x, pos):
        n, hd = x.shape
        dh = self.cfg.dh
        x = x.view(n, hd // dh, dh // 2, 2)
        s, c = self.sin[pos][:, None, :], self.cos[pos][:, None, :]
        a, b = x[..., 0], x[..., 1]
        return rnd(torch.stack([a * c - b * s, a * s + b * c], -1).reshape(n, hd), self.dt)

    def forward(self, reqs, tokens):
        cfg, dt = self.cfg, self.dt
        toks = torch.as_tensor(np.asarray(tokens, dtype=np.int64))
        pos = torch.cat([torch.arange(p, p + l) for _, p, l in reqs])
        x = self.w[(-1, W_EMBD)][toks]
        qd, kvd, g = cfg.nh * cfg.dh, cfg.nkvh * cfg.dh, cfg.nh // cfg.nkvh
        for l in range(cfg.n_layers):
            h = self.norm(x, self.w[(l, W_ATTN_NORM)])
            qkv = rnd(h @ self.w[(l, W_QKV)].T, dt)
            q, k, v = qkv[:, :qd], qkv[:, qd:qd + kvd], qkv[:, qd + kvd:]
            q, k = self.rope(q, pos), self.rope(k, pos)
            att = torch.empty_like(q)
            t0 = 0
            for seq, p, n in reqs:
                kc, vc = self.cache.setdefault((seq, l), (torch.zeros(cfg.nctx, kvd), torch.zeros(cfg.nctx, kvd)))
                kc[p:p + n], vc[p:p + n] = k[t0:t0 + n], v[t0:t0 + n]
                K = kc[:p + n].view(p + n, cfg.nkvh, cfg.dh).repeat_interleave(g, dim=1)   # [ctx, nh, dh]
                V = vc[:p + n].view(p + n, cfg.nkvh, cfg.dh).repeat_interleave(g, dim=1)
                Q = q[t0:t0 + n].view(n, cfg.nh, cfg.dh)
                s = torch.einsum("thd,chd->htc", Q, K) / np.sqrt(np.float32(cfg.dh))
                mask = torch.arange(p + n)[None, :] > (p + torch.arange(n))[:, None]
                s = s.masked_fill(mask[None], float("-inf"))
                pr = torch.softmax(s, -1)
                att[t0:t0 + n] = rnd(torch.einsum("htc,chd->thd", pr, V).reshape(n, qd), dt)
                t0 += n
            x = rnd(att @ self.w[(l, W_O)].T + x, dt)
            h = self.norm(x, self.w[(l, W_FFN_NORM)])
            gu = rnd(h @ self.w[(l, W_GATE_UP)].T, dt)
            gate, up = gu[:, :cfg.di], gu[:, cfg.di:]
            act = rnd(gate * torch.sigmoid(gate) * up, dt)
            x = rnd(act @ self.w[(l, W_DOWN)].T + x, dt)
        last = torch.tensor([sum(r[2] for r in reqs[:i + 1]) - 1 for i in range(len(reqs))])
        xo = self.norm(x[last], self.w[(-1, W_OUT_NORM)])
        logits = rnd(xo @ self.w[(-1, W_LM_HEAD)].T, dt)
        return logits.numpy(), logits.argmax(-1).numpy()
