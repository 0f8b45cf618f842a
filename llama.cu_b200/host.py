"""Session layer above the C-ABI, named after the reference's public API (llama.cu/src/lib.rs:
`Service`, `Session`; exec/engine_manager.rs: `EngineManager::prepare` -> `Round`).

The round logic itself is the C++ engine inside liblcu.so (csrc/engine.cpp, `lcu_engine_*`); this
module only wraps it for Python callers.  All arithmetic happens in the CUDA library.
"""
import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import NO_OUTPUT, RoundInfo, SampleArgs, check, load_library, stream_ptr


@dataclass
class Session:
    """== `Session{id, sample_args, cache}` (lib.rs / exec/mod.rs:61-69)."""
    id: int
    seq: int
    sample_args: SampleArgs = field(default_factory=SampleArgs.arg_max)
    _svc: object = None

    @property
    def pos(self):
        """== `cache.pos`: tokens of this session already in its KV cache."""
        v = C.c_uint32()
        check(self._svc.lib.lcu_engine_session_pos(self._svc.e, self.id, C.byref(v)))
        return v.value

    @pos.setter
    def pos(self, value):
        check(self._svc.lib.lcu_engine_session_set_pos(self._svc.e, self.id, value))


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
    """Continuous batching over one Context: every live session takes part in every round, a new
    session contributes its whole prompt, a running one a placeholder token that the device
    overwrites with its previous sample (exec/engine_manager.rs:72-130)."""

    def __init__(self, ctx, stream=None, nctx=None):
        self.lib = load_library()
        self.ctx = ctx
        self.nctx = nctx if nctx is not None else ctx.desc.nctx
        e = C.c_void_p()
        check(self.lib.lcu_engine_create(ctx.h if ctx is not None else None, self.nctx, C.byref(e)))
        self.e = e
        self.sessions = {}
        self.stream = stream
        self._outs = None
        self._round = 0
        self._next_fake_seq = 0
        if ctx is not None:
            import torch
            self.stream = stream or torch.cuda.Stream(device=ctx.device)
            self._outs = [torch.zeros(ctx.desc.max_seqs or 64, 2, dtype=torch.int32, device=f"cuda:{ctx.device}")
                          for _ in range(4)]

    def __del__(self):
        try:
            if self.e:
                self.lib.lcu_engine_destroy(self.e)
                self.e = None
        except Exception:
            pass

    def new_session(self, sample_args=None):
        if self.ctx is not None:
            seq = self.ctx.seq_create()
        else:  # host-only use (planning, tests): sequence handles are just labels
            seq = self._next_fake_seq
            self._next_fake_seq += 1
        sid = C.c_uint64()
        args = sample_args or SampleArgs.arg_max()
        check(self.lib.lcu_engine_session_new(self.e, seq, C.byref(args), C.byref(sid)))
        s = Session(sid.value, seq, args, self)
        self.sessions[s.id] = s
        return s

    def start(self, session, prompt, max_steps):
        """== `Terminal::start` (lib.rs:233-243)."""
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        check(self.lib.lcu_engine_start(self.e, session.id, p.ctypes.data, len(p), max_steps))

    def set_budget(self, max_round_tokens=0, prefill_chunk=0):
        """Token budget of a round and largest prefill chunk (chunked prefill; 0 / 0 = whole prompts as the reference)."""
        check(self.lib.lcu_engine_set_budget(self.e, max_round_tokens, prefill_chunk))

    def set_seed(self, seed):
        """Reproducible sampling: the engine draws the random numbers itself from (seed, session, draw index)."""
        check(self.lib.lcu_engine_set_seed(self.e, seed))

    def draw_randoms(self, n_req):
        """The seeded random numbers of the round just prepared (advances the sessions' draw counters)."""
        check(self.lib.lcu_engine_draw_randoms(self.e))
        p = self.lib.lcu_engine_round_randoms(self.e)
        return [p[i] for i in range(n_req)]

    def park(self, session, tokens):
        """== `CacheManager::insert`: park a finished session's history and cache for prefix reuse."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        check(self.lib.lcu_engine_cache_insert(self.e, session.id, t.ctypes.data, len(t)))
        self.sessions.pop(session.id, None)

    def send(self, tokens, sample_args=None, max_steps=1):
        """== `CacheManager::send`: start `tokens` on the parked cache with the longest common prefix (or a fresh one).
        Returns (session, tokens reused from the cache)."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        args = sample_args or SampleArgs.arg_max()
        sid, reused = C.c_uint64(), C.c_uint32()
        check(self.lib.lcu_engine_cache_send(self.e, t.ctypes.data, len(t), C.byref(args), max_steps, C.byref(sid),
                                             C.byref(reused)))
        s = Session(sid.value, -1, args, self)
        self.sessions[s.id] = s
        return s, reused.value

    @property
    def parked(self):
        return self.lib.lcu_engine_cache_count(self.e)

    def stop(self, session_id):
        check(self.lib.lcu_engine_remove(self.e, session_id))
        return self.sessions.get(session_id)

    def _round_from(self, info):
        lib, e = self.lib, self.e
        tokens = [lib.lcu_engine_round_tokens(e)[i] for i in range(info.n_tok)]
        reqs_p = lib.lcu_engine_round_reqs(e)
        reqs = [(reqs_p[i].seq, reqs_p[i].pos, reqs_p[i].len) for i in range(info.n_req)]
        fm_p = lib.lcu_engine_round_fast_map(e)
        fast_map = [(fm_p[2 * i], fm_p[2 * i + 1]) for i in range(info.n_fast)]
        sa_p = lib.lcu_engine_round_sample_args(e)
        sample = [SampleArgs(sa_p[i].temperature, sa_p[i].top_p, sa_p[i].top_k) for i in range(info.n_req)]
        out_p = lib.lcu_engine_round_output(e)
        output = [(out_p[i], 1) for i in range(info.n_req)]
        fin_p = lib.lcu_engine_round_finished(e)
        finished = [self.sessions[fin_p[i]] for i in range(info.n_finished)]
        output = [(sid, n) if sid != NO_OUTPUT else (None, 0) for sid, n in output]  # unfinished prefill chunks sample nothing
        ov_p = lib.lcu_engine_round_overflow(e)
        overflow = [self.sessions[ov_p[i]] for i in range(info.n_overflow)]
        return Round(overflow, tokens, reqs, sample, output, fast_map, finished)

    def prepare(self):
        """== `EngineManager::prepare`: builds the next round without running it."""
        info = RoundInfo()
        check(self.lib.lcu_engine_prepare(self.e, C.byref(info)))
        return self._round_from(info)

    def positions(self, round_):
        """(`pos()`, `out_idx()`) of the round just prepared (exec/engine.rs:352-371)."""
        pos = np.zeros(len(round_.tokens), np.uint32)
        out_idx = np.zeros(len(round_.reqs), np.uint32)
        check(self.lib.lcu_engine_round_positions(self.e, pos.ctypes.data, out_idx.ctypes.data))
        return pos, out_idx

    def step(self, randoms=None):
        """One round (`Worker::lead` loop body): returns (Round, device tensor of its KVPairs)
        without synchronising; (Round, None) when there was nothing to run."""
        out = self._outs[self._round % len(self._outs)]
        info = RoundInfo()
        rnd = None
        if randoms is not None:
            rnd = np.ascontiguousarray(randoms, dtype=np.float32)
        else:
            rnd = np.random.random(max(len(self.sessions), 1)).astype(np.float32)
        check(self.lib.lcu_engine_step(self.e, stream_ptr(self.stream), rnd.ctypes.data, out.data_ptr(), C.byref(info)))
        r = self._round_from(info)
        if info.n_tok == 0:
            return r, None
        self._round += 1
        return r, out

    @staticmethod
    def decode(round_, out):
        """== `exec::decode` (exec/mod.rs:91-115): D2H of the pairs, split per session."""
        host = out[:len(round_.output)].cpu().numpy().view(np.uint32)
        return {sid: int(host[i, 0]) for i, (sid, _) in enumerate(round_.output) if sid is not None}


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


class StepRendezvous:
    """Host-side roll call of the tensor-parallel ranks before a round is launched.

    The reference keeps its per-GPU worker threads in step with a `Barrier` (llama.cu/src/exec/engine.rs:272,339),
    which blocks for ever when a worker has died.  With one process per GPU the ranks meet through a key-value
    store (`torch.distributed.TCPStore` / `FileStore` / the store of an initialised process group): every rank
    marks its arrival at round `step`, then waits until all have — or until `timeout_s` has passed, in which case
    it raises LcuError(ERR_TIMEOUT) naming the ranks that never arrived, BEFORE anything is launched on the GPU.
    (The kernels' own bounded waits are the second line of defence, see lcu_device_status.)"""

    def __init__(self, store, rank, world, timeout_s=5.0, prefix="lcu/round"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, step, rank):
        return f"{self.prefix}/{step}/{rank}"

    def arrive(self, step):
        self.store.set(self._key(step, self.rank), b"1")

    def missing(self, step):
        """Ranks that have not arrived at `step` (non-blocking)."""
        return [r for r in range(self.world) if not self.store.check([self._key(step, r)])]

    def wait(self, step, timeout_s=None):
        import time
        from . import ERR_TIMEOUT, LcuError
        limit = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)
        self.arrive(step)
        while True:
            gone = self.missing(step)
            if not gone:
                return
            if time.monotonic() > limit:
                raise LcuError(ERR_TIMEOUT, f"round {step}: rank(s) {gone} never arrived")
            time.sleep(0.002)


def generate_continuous(ctx, prompts, steps, max_round_tokens=0, prefill_chunk=0, sample_args=None, seed=None):
    """All prompts enter the batch together and run under a token budget with chunked prefill (`Service.set_budget`):
    long prompts are fed a chunk per round while sessions that have finished theirs already decode.  Returns
    [n_prompts][steps] token ids.  (The reference admits whole prompts only, at most 1024 tokens per round.)"""
    import torch
    svc = Service(ctx)
    svc.set_budget(max_round_tokens, prefill_chunk)
    if seed is not None:
        svc.set_seed(seed)
    with torch.cuda.stream(svc.stream):
        sessions = [svc.new_session(sample_args) for _ in prompts]
        for s, p in zip(sessions, prompts):
            svc.start(s, p, steps)
        toks = {s.id: [] for s in sessions}
        pending = []
        while True:
            r, out = svc.step()
            if out is None:
                break
            pending.append((r, out.clone()))
        svc.stream.synchronize()
        torch.cuda.synchronize(ctx.device)
        for r, out in pending:
            for sid, t in Service.decode(r, out).items():
                toks[sid].append(t)
    for s in sessions:
        ctx.seq_free(s.seq)
    return [toks[s.id] for s in sessions]
