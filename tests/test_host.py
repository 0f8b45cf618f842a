"""CPU tests of the session layer: `Service.prepare` against the behaviour of
`EngineManager::prepare` (llama.cu/src/exec/engine_manager.rs:72-130)."""
import numpy as np
import pytest


class FakeDesc:
    nctx = 32
    max_seqs = 8


class FakeCtx:
    """Stands in for the CUDA context: records the rounds it is asked to run."""
    device = 0

    def __init__(self):
        self.desc = FakeDesc()
        self.calls = []
        self._seq = 0

    def seq_create(self):
        self._seq += 1
        return self._seq - 1

    def step(self, reqs, tokens, out, args=None, randoms=None, fast_map=None, stream=None):
        self.calls.append((list(reqs), np.array(tokens), None if fast_map is None else np.array(fast_map), args))


@pytest.fixture
def svc(L, monkeypatch):
    import torch
    from llama_cu_b200 import host

    class S(host.Service):
        def __init__(self, ctx):
            self.ctx, self.stream = ctx, None
            self.sess, self.pre_output, self._next_id = {}, {}, 0
            self._outs = [torch.zeros(8, 2, dtype=torch.int32)]
            self._round = 0
            self.nctx = ctx.desc.nctx
    return S(FakeCtx())


def test_prefill_then_decode_rounds(svc):
    a, b = svc.new_session(), svc.new_session()
    svc.start(b, [7, 8, 9], 3)
    svc.start(a, [5, 6], 2)
    r = svc.prepare()
    # BTreeMap order: session id 0 (a) first, whatever the insertion order
    assert r.tokens == [5, 6, 7, 8, 9]
    assert r.reqs == [(a.seq, 0, 2), (b.seq, 0, 3)]
    assert r.output == [(a.id, 1), (b.id, 1)] and r.fast_map == [] and r.finished == []
    assert (a.pos, b.pos) == (2, 3)
    r = svc.prepare()
    # decode: one placeholder token per session, replaced on the device by the previous sample
    assert r.tokens == [0, 0] and r.fast_map == [(0, 0), (1, 1)]
    assert r.reqs == [(a.seq, 2, 1), (b.seq, 3, 1)]
    assert [s.id for s in r.finished] == [a.id]          # a had max_steps = 2
    r = svc.prepare()
    # only b is left; its previous output sat at index 1 of the last round
    assert r.tokens == [0] and r.fast_map == [(1, 0)] and [s.id for s in r.finished] == [b.id]
    assert svc.prepare().tokens == []


def test_overflow_returns_the_session(svc):
    a = svc.new_session()
    svc.start(a, list(range(3, 3 + 33)), 4)           # 33 tokens > nctx = 32
    r = svc.prepare()
    assert [s.id for s in r.overflow] == [a.id] and r.tokens == [] and a.pos == 0


def test_sessions_resume_at_their_position(svc):
    """A returned session restarts with new tokens at cache.pos (lib.rs:233-243)."""
    a = svc.new_session()
    svc.start(a, [5, 6, 7], 1)
    r = svc.prepare()
    assert [s.id for s in r.finished] == [a.id] and a.pos == 3
    svc.start(a, [11], 2)
    r = svc.prepare()
    assert r.reqs == [(a.seq, 3, 1)] and r.tokens == [11] and r.fast_map == []
    a.pos = 2                                          # prefix reuse: roll the cache back
    svc.start(a, [12, 13], 1)
    assert svc.prepare().reqs == [(a.seq, 2, 2)]


def test_step_passes_the_round_to_the_context(svc):
    a = svc.new_session()
    svc.start(a, [5, 6], 2)
    svc.step()
    svc.step()
    (reqs0, tok0, fm0, _), (reqs1, tok1, fm1, _) = svc.ctx.calls
    assert reqs0 == [(a.seq, 0, 2)] and tok0.tolist() == [5, 6] and fm0 is None
    assert reqs1 == [(a.seq, 2, 1)] and tok1.tolist() == [0] and fm1.tolist() == [[0, 0]]
    assert svc.stop(a.id) is None                      # finished sessions are gone
