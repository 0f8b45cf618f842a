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


def test_chunked_prefill_and_token_budget(L):
    """What the reference leaves as `TODO: chunked prefill` (exec/engine_manager.rs:83): with a budget of 8 tokens per
    round and chunks of at most 5, decoding sessions always get their token, prompts share the rest in session
    order, an unfinished prompt samples nothing and uses no step."""
    from llama_cu_b200 import host
    svc = host.Service(None, nctx=64)
    svc.set_budget(max_round_tokens=8, prefill_chunk=5)
    a, b = svc.new_session(), svc.new_session()
    svc.start(a, list(range(10, 22)), 2)      # 12-token prompt
    svc.start(b, [3, 4, 5], 4)                # 3-token prompt
    r = svc.prepare()                         # a: chunk of 5 (cap), b: its whole prompt (3 of the 3 left)
    assert r.reqs == [(a.seq, 0, 5), (b.seq, 0, 3)] and r.tokens == list(range(10, 15)) + [3, 4, 5]
    assert r.output == [(None, 0), (b.id, 1)] and r.finished == []
    r = svc.prepare()                         # b decodes (1 token, slot 5), a: next chunk of 5 out of the 7 left
    assert r.reqs == [(a.seq, 5, 5), (b.seq, 3, 1)] and r.tokens == list(range(15, 20)) + [0]
    assert r.fast_map == [(1, 5)] and r.output == [(None, 0), (b.id, 1)]
    r = svc.prepare()                         # a finishes its prompt (2 tokens) and samples its first token
    assert r.reqs == [(a.seq, 10, 2), (b.seq, 4, 1)] and r.tokens == [20, 21, 0]
    assert r.output == [(a.id, 1), (b.id, 1)] and r.fast_map == [(1, 2)]
    assert a.pos == 12
    r = svc.prepare()                         # both decode; a finishes (max_steps 2), b finishes (max_steps 4)
    assert r.reqs == [(a.seq, 12, 1), (b.seq, 5, 1)] and r.fast_map == [(0, 0), (1, 1)]
    assert sorted(s.id for s in r.finished) == [a.id, b.id]
    assert svc.prepare().tokens == []


def test_budget_makes_a_prompt_wait(L):
    from llama_cu_b200 import host
    svc = host.Service(None, nctx=64)
    svc.set_budget(max_round_tokens=4, prefill_chunk=0)
    a, b = svc.new_session(), svc.new_session()
    svc.start(a, [5, 6, 7, 8], 2)
    svc.start(b, [9, 10], 2)
    r = svc.prepare()                         # a takes the whole budget, b waits
    assert r.reqs == [(a.seq, 0, 4)] and r.output == [(a.id, 1)]
    r = svc.prepare()                         # a decodes (1), b gets its 2 tokens
    assert r.reqs == [(a.seq, 4, 1), (b.seq, 0, 2)] and r.tokens == [0, 9, 10]


def test_prefix_reuse_manager(L):
    """== CacheManager::send / insert (xtask/src/service/cache_manager.rs:22-66)."""
    from llama_cu_b200 import host
    svc = host.Service(None, nctx=64)
    s1, reused = svc.send([1, 2, 3, 4, 5], max_steps=1)
    assert reused == 0 and svc.prepare().reqs == [(0, 0, 5)]       # nothing parked: a fresh sequence, the whole prompt
    svc.park(s1, [1, 2, 3, 4, 5, 6])                                # history = prompt + the generated token
    s2, _ = svc.send([9, 9, 9], max_steps=1)                        # no common prefix: the parked cache is STILL taken, at 0
    assert svc.parked == 0 and svc.prepare().reqs == [(0, 0, 3)]
    svc.park(s2, [9, 9, 9, 7])
    s3, _ = svc.send([8, 8], max_steps=1)                           # takes s2's cache; a second one must be created next
    svc.prepare()
    s4, reused = svc.send([1, 2], max_steps=1)
    assert reused == 0 and svc.prepare().reqs == [(1, 0, 2)]       # fresh sequence label 1
    svc.park(s3, [8, 8, 3])
    svc.park(s4, [1, 2, 3, 4])
    # longest common prefix with tokens[:-1] wins: [1, 2, 3] of s4's history, not the last token (it must be run)
    s5, reused = svc.send([1, 2, 3, 4], max_steps=1)
    assert reused == 3
    r = svc.prepare()
    assert r.reqs == [(1, 3, 1)] and r.tokens == [4] and svc.parked == 1
    # among equally good caches the most recently parked one is taken
    svc.park(s5, [1, 2, 3, 4, 0])
    s6, reused = svc.send([5, 5, 5], max_steps=1)
    assert reused == 0 and svc.prepare().reqs == [(1, 0, 3)]


def test_seeded_sampling_is_reproducible_and_batch_independent(L):
    """The k-th random number of a session depends only on (seed, session id, k): the same conversation draws the
    same numbers whether another session joins the batch early, late or never; arg-max rows draw nothing."""
    from llama_cu_b200 import host

    def draws(seed, b_joins_at):
        svc = host.Service(None, nctx=64)
        svc.set_seed(seed)
        a = svc.new_session(L.SampleArgs.new(0.8, 0.9, 40))
        b = svc.new_session(L.SampleArgs.new(1.2, 1.0, 10))
        g = svc.new_session()                                  # greedy: never draws
        out = {a.id: [], b.id: [], g.id: []}
        svc.start(a, [3, 4], 6)
        svc.start(g, [6], 6)
        for step in range(8):
            if step == b_joins_at:
                svc.start(b, [5], 4)
            r = svc.prepare()
            if not r.reqs:
                break
            rnd = svc.draw_randoms(len(r.reqs))
            for (sid, _), x in zip(r.output, rnd):
                out[sid].append(x)
        return out, (a.id, b.id, g.id)
    x, (a, b, g) = draws(7, 0)
    y, _ = draws(7, 3)
    z, _ = draws(8, 0)
    assert x[a] == y[a] and x[b] == y[b] and len(x[a]) == 6 and len(x[b]) == 4
    assert all(0.0 <= v < 1.0 for v in x[a] + x[b]) and len(set(x[a])) == 6
    assert x[g] == [0.0] * 6
    assert x[a] != z[a] and x[a] != x[b][:4] + x[a][4:]
