"""Host-side session layer above the C-ABI, named after the reference's public API
(llama.cu/src/lib.rs: `Service`, `Session`, `SessionId`; exec/engine_manager.rs:
`EngineManager::prepare` -> `Round`).  It decides what goes into each round and calls
`lcu_step`; all arithmetic happens in the CUDA library.
"""
from dataclasses import dataclass, field

import numpy as np

from . import KVPair, SampleArgs


@dataclass
class Session:
    """== `Session{id, sample_args, cache}` (lib.rs / exec/mod.rs:61-69); `pos` is `cache.pos`."""
    id: int
    seq: int
    sample_args: SampleArgs = field(default_factory=SampleArgs.arg_max)
    pos: int = 0


@dataclass
class _Stub:  # == SessionStub (exec/engine.rs:33-66)
    session: Session
    seq_len: int
    remain_steps: int
    prompt: object


@dataclass
class Round:  # == Round (exec/engine_manager.rs:22-31)
    overflow: list
    tokens: list
    reqs: list
    sample: list
    output: list
    fast_map: list
    finished: list


class Service:
    """Continuous batching over one Context: every live session takes part in every round,
    a new session contributes its whole prompt, a running one a placeholder token that the
    device overwrites with its previous sample (exec/engine_manager.rs:72-130)."""

    def __init__(self, ctx, stream=None):
        import torch
        self.ctx = ctx
        self.stream = stream or torch.cuda.Stream(device=ctx.device)
        self.sess = {}        # id -> _Stub, iterated in id order like the reference's BTreeMap
        self.pre_output = {}  # id -> index of its pair in the previous round's output
        self._next_id = 0
        self._outs = [torch.zeros(ctx.desc.max_seqs or 64, 2, dtype=torch.int32, device=f"cuda:{ctx.device}")
                      for _ in range(4)]
        self._round = 0
        self.nctx = ctx.desc.nctx

    def new_session(self, sample_args=None):
        s = Session(self._next_id, self.ctx.seq_create(), sample_args or SampleArgs.arg_max())
        self._next_id += 1
        return s

    def start(self, session, prompt, max_steps):
        """== `Terminal::start` (lib.rs:233-243)."""
        self.sess[session.id] = _Stub(session, len(prompt), max_steps, np.asarray(prompt, dtype=np.uint32))

    def stop(self, session_id):
        stub = self.sess.pop(session_id, None)
        self.pre_output.pop(session_id, None)
        return stub.session if stub else None

    def prepare(self):
        """== `EngineManager::prepare`."""
        r = Round([], [], [], [], [], [], [])
        out_idx = 0
        pre_output, self.pre_output = self.pre_output, {}
        sess, self.sess = self.sess, {}
        for sid in sorted(sess):
            stub = sess[sid]
            s = stub.session
            end = s.pos + stub.seq_len
            if end > self.nctx:
                r.overflow.append(s)
                continue
            pos = s.pos
            s.pos = end
            r.sample.append(s.sample_args)
            r.output.append((sid, 1))
            r.reqs.append((s.seq, pos, stub.seq_len))
            if stub.prompt is not None:
                r.tokens.extend(int(t) for t in stub.prompt)
                stub.prompt = None
                stub.seq_len = 1
            else:
                r.fast_map.append((pre_output[sid], len(r.tokens)))
                r.tokens.append(0)
            stub.remain_steps -= 1
            if stub.remain_steps == 0:
                r.finished.append(s)
            else:
                self.sess[sid] = stub
                self.pre_output[sid] = out_idx
            out_idx += 1
        return r

    def step(self, randoms=None):
        """One round; returns (Round, device tensor of its KVPairs) without synchronising."""
        r = self.prepare()
        if not r.tokens:
            return r, None
        out = self._outs[self._round % len(self._outs)]
        self._round += 1
        any_sampling = any(not a.is_argmax() for a in r.sample)
        if any_sampling and randoms is None:
            randoms = np.random.random(len(r.reqs)).astype(np.float32)
        self.ctx.step(r.reqs, np.asarray(r.tokens, dtype=np.uint32), out,
                      args=r.sample if any_sampling else None, randoms=randoms if any_sampling else None,
                      fast_map=np.asarray(r.fast_map, dtype=np.uint32) if r.fast_map else None, stream=self.stream)
        return r, out

    @staticmethod
    def decode(round_, out):
        """== `exec::decode` (exec/mod.rs:91-115): D2H of the pairs, split per session."""
        host = out[:len(round_.output)].cpu().numpy().view(np.uint32)
        return {sid: int(host[i, 0]) for i, (sid, _) in enumerate(round_.output)}


def generate(ctx, prompts, steps, sample_args=None, read_every_step=False, randoms=None):
    """Greedy (or sampled) generation of `steps` tokens for each prompt, all sequences batched
    — the loop of xtask/src/generate.rs:41-68 and bench.rs:47-80.  Prompts are prefilled one
    sequence per round (the reference admits at most 1024 tokens per round), then every
    session decodes together.  Returns [n_prompts][steps] token ids."""
    import torch
    svc = Service(ctx)
    with torch.cuda.stream(svc.stream):
        return _generate(svc, ctx, prompts, steps, sample_args, read_every_step, randoms)


def _generate(svc, ctx, prompts, steps, sample_args, read_every_step, randoms):
    import torch
    sessions = [svc.new_session(sample_args) for _ in prompts]
    first = {}
    # staged prefill: each prompt alone for one step, then resume all together
    for s, p in zip(sessions, prompts):
        svc.start(s, p, 1)
        r, out = svc.step(randoms)
        svc.stream.synchronize()
        first[s.id] = Service.decode(r, out)[s.id]
    toks = {s.id: [first[s.id]] for s in sessions}
    if steps > 1:
        for s in sessions:
            svc.start(s, [first[s.id]], steps - 1)
        pending = []
        for _ in range(steps - 1):
            r, out = svc.step(randoms)
            if read_every_step:
                svc.stream.synchronize()
                for sid, t in Service.decode(r, out).items():
                    toks[sid].append(t)
            else:
                pending.append((r, out.clone()))
        svc.stream.synchronize()
        torch.cuda.synchronize(ctx.device)
        for r, out in pending:
            for sid, t in Service.decode(r, out).items():
                toks[sid].append(t)
    for s in sessions:
        ctx.seq_free(s.seq)
    return [toks[s.id] for s in sessions]
