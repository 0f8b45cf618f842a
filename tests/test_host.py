"""CPU tests of the round builder (C++ `lcu_engine_*` through the Python `Service` wrapper)
against the behaviour of `EngineManager::prepare` (llama.cu/src/exec/engine_manager.rs:72-130)
and of `pos()` / `out_idx()` (exec/engine.rs:352-371).  No GPU is involved."""
import pytest


@pytest.fixture
def svc(L):
    from llama_cu_b200 import host
    return host.Service(None, nctx=32)


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
    pos, out_idx = svc.positions(r)
    assert pos.tolist() == [0, 1, 0, 1, 2] and out_idx.tolist() == [1, 4]
    r = svc.prepare()
    # decode: one placeholder token per session, replaced on the device by the previous sample
    assert r.tokens == [0, 0] and r.fast_map == [(0, 0), (1, 1)]
    assert r.reqs == [(a.seq, 2, 1), (b.seq, 3, 1)]
    assert [s.id for s in r.finished] == [a.id]          # a had max_steps = 2
    pos, out_idx = svc.positions(r)
    assert pos.tolist() == [2, 3] and out_idx.tolist() == [0, 1]
    r = svc.prepare()
    # only b is left; its previous output sat at index 1 of the last round
    assert r.tokens == [0] and r.fast_map == [(1, 0)] and [s.id for s in r.finished] == [b.id]
    assert svc.prepare().tokens == []


def test_overflow_returns_the_session(svc):
    a = svc.new_session()
    svc.start(a, list(range(3, 3 + 33)), 4)           # 33 tokens > nctx = 32
    r = svc.prepare()
    assert [s.id for s in r.overflow] == [a.id] and r.tokens == [] and a.pos == 0
    assert svc.prepare().tokens == []                  # an overflowed session is out of the batch


def test_sessions_resume_at_their_position(svc):
    """A returned session restarts with new tokens at cache.pos (lib.rs:233-243)."""
    a = svc.new_session()
    svc.start(a, [5, 6, 7], 1)
    r = svc.prepare()
    assert [s.id for s in r.finished] == [a.id] and a.pos == 3
    svc.start(a, [11], 2)
    r = svc.prepare()
    assert r.reqs == [(a.seq, 3, 1)] and r.tokens == [11] and r.fast_map == []
    svc.stop(a.id)
    a.pos = 2                                          # prefix reuse: roll the cache back
    svc.start(a, [12, 13], 1)
    assert svc.prepare().reqs == [(a.seq, 2, 2)]


def test_remove_takes_a_session_out_of_the_batch(svc):
    a, b = svc.new_session(), svc.new_session()
    svc.start(a, [5], 5)
    svc.start(b, [6], 5)
    assert len(svc.prepare().reqs) == 2
    svc.stop(a.id)
    r = svc.prepare()
    assert r.reqs == [(b.seq, 1, 1)] and r.fast_map == [(1, 0)]


def test_sample_args_are_validated_like_the_reference(L, svc):
    import ctypes as C
    lib = L.load_library()
    sid = C.c_uint64()
    bad = L.SampleArgs(-1.0, 0.5, 10)
    assert lib.lcu_engine_session_new(svc.e, 0, C.byref(bad), C.byref(sid)) == L.ERR_INVALID
    assert b"NegativeTemperature" in lib.lcu_last_error_string()
    bad = L.SampleArgs(1.0, 0.5, 0)
    assert lib.lcu_engine_session_new(svc.e, 0, C.byref(bad), C.byref(sid)) == L.ERR_INVALID
    s = svc.new_session(L.SampleArgs(0.7, 3.0, 40))
    svc.start(s, [5], 1)
    assert svc.prepare().sample[0].top_p == 1.0       # top_p is clamped to 1
