"""Operator-level parity through the C-ABI (needs a B200): each lcu_op_* against the CPU
oracle and, where the reference ships a kernel for it, against that kernel compiled from
the reference's own sources (oracle/_ref)."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import bits_to_torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def sp():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def rand_act(rng, shape, dt, O, scale=1.0):
    """Random activations already representable in the activation dtype: (f32 values, device tensor)."""
    a = (rng.standard_normal(shape).astype(np.float32) * scale)
    bits = O.from_f32(a, dt)
    return O.to_f32(bits, dt), bits_to_torch(bits, dt, DEV)


def as_f32(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("n,d", [(1, 256), (3, 2048), (5, 4096), (2, 8192), (4, 688)])
def test_rms_norm(L, O, dt, n, d):
    rng = np.random.default_rng(d + n)
    x, xt = rand_act(rng, (n, d), dt, O)
    w, wt = rand_act(rng, (d,), dt, O)
    yt = torch.empty_like(xt)
    lib = L.load_library()
    L.check(lib.lcu_op_rms_norm(yt.data_ptr(), d, xt.data_ptr(), d, wt.data_ptr(), dt, 1e-5, n, d, dt, sp()))
    want = O.rms_norm(x, w, 1e-5, dt)
    got = as_f32(yt)
    # one rounding each; sums differ in order, so allow 1 ulp of the activation dtype
    ulp = 2.0 ** (-10 if dt == 0 else -7)
    assert np.all(np.abs(got - want) <= ulp * np.maximum(np.abs(want), 1e-3) + 1e-7)
    # f32 norm weights
    wf = torch.from_numpy(w).to(DEV)
    y2 = torch.empty_like(xt)
    L.check(lib.lcu_op_rms_norm(y2.data_ptr(), d, xt.data_ptr(), d, wf.data_ptr(), 2, 1e-5, n, d, dt, sp()))
    assert torch.equal(y2, yt)
    R = O.ref_lib()
    if R is not None and dt == 0 and d != 688:
        yr = torch.empty_like(xt)
        assert R.ref_rms_norm_f16(yr.data_ptr(), d, xt.data_ptr(), d, wt.data_ptr(), 0, 1e-5, n, d, sp()) == 0
        torch.cuda.synchronize()
        diff = np.abs(as_f32(yr) - got)
        assert np.all(diff <= ulp * np.maximum(np.abs(got), 1e-3) + 1e-7)
        assert (diff == 0).mean() > 0.99


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("nh,dh", [(4, 64), (32, 128), (8, 128)])
def test_rope(L, O, dt, nh, dh):
    rng = np.random.default_rng(nh)
    n, nctx = 7, 300
    x, xt = rand_act(rng, (n, nh * dh), dt, O)
    pos = rng.integers(0, nctx, n).astype(np.uint32)
    sin, cos = L.build_sin_cos(nctx, dh, 5e5)
    s2, c2 = O.build_sin_cos(nctx, dh, 5e5)
    assert np.array_equal(sin, s2) and np.array_equal(cos, c2)
    st, ct, pt = (torch.from_numpy(a).to(DEV) for a in (sin, cos, pos.view(np.int32)))
    yt = torch.empty_like(xt)
    lib = L.load_library()
    L.check(lib.lcu_op_rope(yt.data_ptr(), nh * dh, dh, xt.data_ptr(), nh * dh, dh, pt.data_ptr(), st.data_ptr(),
                            ct.data_ptr(), n, nh, dh, dt, sp()))
    want = O.rope(x, nh, dh, pos, sin, cos, dt)
    # the device contracts a*cos - b*sin into an fma, the host does not: at most 1 ulp apart
    got = as_f32(yt)
    ulp = 2.0 ** (-10 if dt == 0 else -7)
    assert np.all(np.abs(got - want) <= ulp * np.maximum(np.abs(want), 1e-2))
    R = O.ref_lib()
    if R is not None and dt == 0:
        yr = torch.empty_like(xt)
        assert R.ref_rope_f16(yr.data_ptr(), nh * dh, dh, xt.data_ptr(), nh * dh, dh, pt.data_ptr(), st.data_ptr(),
                              ct.data_ptr(), n, nh, dh, sp()) == 0
        torch.cuda.synchronize()
        assert torch.equal(yr, yt), "bit-exact against the reference's rope kernel"


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("di", [688, 8192, 14336])
def test_swiglu(L, O, dt, di):
    rng = np.random.default_rng(di)
    n = 3
    g, gt = rand_act(rng, (n, di), dt, O, 2.0)
    u, ut = rand_act(rng, (n, di), dt, O, 2.0)
    ot = torch.empty_like(gt)
    lib = L.load_library()
    L.check(lib.lcu_op_swiglu(ot.data_ptr(), di, gt.data_ptr(), di, ut.data_ptr(), di, n, di, dt, sp()))
    want = O.swiglu(g, u, dt)
    got = as_f32(ot)
    ulp = 2.0 ** (-10 if dt == 0 else -7)
    assert np.all(np.abs(got - want) <= ulp * np.maximum(np.abs(want), 1e-3) + 1e-6)
    R = O.ref_lib()
    if R is not None and dt == 0:
        orf = torch.empty_like(gt)
        assert R.ref_swiglu_f16(orf.data_ptr(), di, gt.data_ptr(), di, ut.data_ptr(), di, n, di, sp()) == 0
        torch.cuda.synchronize()
        assert torch.equal(orf, ot), "bit-exact against the reference's swiglu kernel"


def test_embedding_and_fast_embedding(L, O):
    rng = np.random.default_rng(3)
    vocab, d, n = 500, 256, 9
    tab, tt = rand_act(rng, (vocab, d), 0, O)
    idx = rng.integers(0, vocab, n).astype(np.uint32)
    it = torch.from_numpy(idx.view(np.int32)).to(DEV)
    out = torch.empty(n, d, dtype=torch.float16, device=DEV)
    lib = L.load_library()
    L.check(lib.lcu_op_embedding(out.data_ptr(), tt.data_ptr(), it.data_ptr(), n, d * 2, sp()))
    assert torch.equal(out, tt[torch.from_numpy(idx.astype(np.int64)).to(DEV)])
    R = O.ref_lib()
    if R is not None:
        o2 = torch.empty_like(out)
        assert R.ref_embedding(o2.data_ptr(), tt.data_ptr(), it.data_ptr(), n, d * 2, sp()) == 0
        torch.cuda.synchronize()
        assert torch.equal(o2, out)
    # fast embedding: tokens[map[i][1]] = pairs[map[i][0]].idx
    pairs = torch.tensor([[11, 0], [22, 0], [33, 0]], dtype=torch.int32, device=DEV)
    fmap = torch.tensor([[2, 0], [0, 3]], dtype=torch.int32, device=DEV)
    toks = torch.zeros(5, dtype=torch.int32, device=DEV)
    L.check(lib.lcu_op_fast_embedding(toks.data_ptr(), pairs.data_ptr(), fmap.data_ptr(), 2, sp()))
    assert toks.tolist() == [33, 0, 0, 11, 0]
    if R is not None:
        t2 = torch.zeros(5, dtype=torch.int32, device=DEV)
        assert R.ref_fast_embedding(t2.data_ptr(), pairs.data_ptr(), fmap.data_ptr(), 2, sp()) == 0
        torch.cuda.synchronize()
        assert torch.equal(t2, toks)


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("n,k,out,res", [(1, 256, 768, False), (1, 4096, 512, True), (2, 688, 256, True),
                                         (4, 2048, 1024, False), (7, 14336, 256, True), (1, 8192, 130, False),
                                         (3, 28672, 64, True)])
def test_linear(L, O, dt, n, k, out, res):
    rng = np.random.default_rng(k + out)
    x, xt = rand_act(rng, (n, k), dt, O)
    w, wt = rand_act(rng, (out, k), dt, O, 0.02)
    r, rt = rand_act(rng, (n, out), dt, O)
    yt = torch.empty(n, out, dtype=xt.dtype, device=DEV)
    lib = L.load_library()
    L.check(lib.lcu_op_linear(yt.data_ptr(), out, xt.data_ptr(), k, wt.data_ptr(), dt, rt.data_ptr() if res else None,
                              out, n, k, out, dt, sp()))
    want = O.linear(x, w, r if res else None, dt)
    got = as_f32(yt)
    ulp = 2.0 ** (-10 if dt == 0 else -7)
    # one rounding apart at most; below 0.25 the f32 accumulation order over up to 28672 terms
    # (tensor cores truncate their partial sums) dominates, so the bound has an absolute floor
    diff = np.abs(got - want)
    assert np.all(diff <= ulp * np.maximum(np.abs(want), 0.25)), diff.max()
    exact = x.astype(np.float64) @ w.astype(np.float64).T + (r if res else 0)
    assert np.all(np.abs(got - exact) <= ulp * np.maximum(np.abs(exact), 0.25))


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("n,k,out,res", [(5, 256, 768, False), (16, 4096, 512, True), (33, 2048, 1024, True),
                                         (64, 14336, 256, False), (100, 8192, 130, True), (7, 28672, 64, False),
                                         (40, 4096, 6144, False)])
def test_linear_batched_tensor_core(L, O, dt, n, k, out, res):
    """More than 4 rows take the tensor-core kernel (blocks of up to 64 rows)."""
    rng = np.random.default_rng(n * 7 + k)
    x, xt = rand_act(rng, (n, k), dt, O)
    w, wt = rand_act(rng, (out, k), dt, O, 0.02)
    r, rt = rand_act(rng, (n, out), dt, O)
    yt = torch.empty(n, out, dtype=xt.dtype, device=DEV)
    lib = L.load_library()
    L.check(lib.lcu_op_linear(yt.data_ptr(), out, xt.data_ptr(), k, wt.data_ptr(), dt, rt.data_ptr() if res else None,
                              out, n, k, out, dt, sp()))
    got = as_f32(yt)
    ulp = 2.0 ** (-10 if dt == 0 else -7)
    exact = x.astype(np.float64) @ w.astype(np.float64).T + (r if res else 0)
    assert np.all(np.abs(got - exact) <= ulp * np.maximum(np.abs(exact), 0.25)), np.abs(got - exact).max()
    want = O.linear(x, w, r if res else None, dt)
    assert (got == want).mean() > 0.85  # same value except where the summation order flips a rounding


@pytest.mark.parametrize("n,k,out", [(1, 4096, 256), (2, 14336, 64), (4, 256, 128), (1, 1024, 6144),
                                     (5, 256, 128), (16, 4096, 512), (33, 14336, 256), (64, 1024, 640), (100, 2048, 130)])
def test_linear_q8_0(L, O, n, k, out):
    """1..4 rows: GEMV with in-register dequantisation; more: the mma.sync kernel with per-block scaling."""
    from llama_cu_b200.model import q8_0_blocks
    rng = np.random.default_rng(k)
    x, xt = rand_act(rng, (n, k), 0, O)
    q = rng.integers(-127, 128, (out, k), dtype=np.int8)
    sc = rng.uniform(1e-4, 4e-4, (out, k // 32)).astype(np.float16)
    blocks = q8_0_blocks(q, sc)
    lib = L.load_library()
    bt = torch.from_numpy(blocks).to(DEV)
    planes = torch.empty(lib.lcu_q8_0_repacked_bytes(out, k), dtype=torch.uint8, device=DEV)
    L.check(lib.lcu_repack_q8_0(planes.data_ptr(), bt.data_ptr(), out, k, sp()))
    assert np.array_equal(planes[:out * k].cpu().numpy().view(np.int8).reshape(out, k), q)
    assert np.array_equal(planes[out * k:].cpu().numpy().view(np.float16).reshape(out, k // 32), sc)
    yt = torch.empty(n, out, dtype=torch.float16, device=DEV)
    L.check(lib.lcu_op_linear(yt.data_ptr(), out, xt.data_ptr(), k, planes.data_ptr(), 3, None, 0, n, k, out, 0, sp()))
    w = O.to_f32(blocks, 3).reshape(out, k)
    # independent dequantisation (the published ggml definition): scale * q
    assert np.array_equal(w, np.repeat(sc.astype(np.float32), 32, axis=1) * q.astype(np.float32))
    want = O.linear(x, w, None, 0)
    got = as_f32(yt)
    assert np.all(np.abs(got - want) <= 2.0 ** -10 * np.maximum(np.abs(want), 1e-2) + 1e-6), np.abs(got - want).max()


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("nh,nkvh,dh,pos,seq", [(4, 4, 64, 0, 5), (32, 8, 128, 37, 1), (32, 8, 64, 100, 3),
                                                (8, 1, 128, 63, 2), (8, 8, 128, 200, 1)])
def test_attention_kv_cached(L, O, dt, nh, nkvh, dh, pos, seq):
    """The per-request operator with strided linear caches laid out as the reference's
    [nkvh, nblk, 2, nctx, dh] view: token stride = 2*nkvh*dh (one layer), head stride = dh."""
    rng = np.random.default_rng(pos + seq)
    nctx = 256
    q, qt = rand_act(rng, (seq, nh * dh), dt, O)
    k, kt = rand_act(rng, (seq, nkvh * dh), dt, O)
    v, vt = rand_act(rng, (seq, nkvh * dh), dt, O)
    kc, _ = rand_act(rng, (nctx, nkvh * dh), dt, O)
    vc, _ = rand_act(rng, (nctx, nkvh * dh), dt, O)
    cache = torch.zeros(nctx, 2, nkvh * dh, dtype=qt.dtype, device=DEV)
    cache[:, 0] = bits_to_torch(O.from_f32(kc, dt), dt, DEV)
    cache[:, 1] = bits_to_torch(O.from_f32(vc, dt), dt, DEV)
    ot = torch.empty_like(qt)
    tok_stride = 2 * nkvh * dh
    lib = L.load_library()
    L.check(lib.lcu_op_attention_kv_cached(
        ot.data_ptr(), nh * dh, dh, qt.data_ptr(), nh * dh, dh, kt.data_ptr(), nkvh * dh, dh, vt.data_ptr(), nkvh * dh, dh,
        cache[:, 0].data_ptr(), tok_stride, dh, cache[:, 1].data_ptr(), tok_stride, dh, nh, nkvh, dh, seq, pos, dt, sp()))
    kc[pos:pos + seq] = k
    vc[pos:pos + seq] = v
    want = O.attention(q, kc[:pos + seq], vc[:pos + seq], nh, nkvh, dh, pos, dt)
    got = as_f32(ot)
    # The kernel rounds the probabilities to the activation dtype before the P.V product (tensor-core operands,
    # as a GEMM-based operator that keeps the attention matrix in f16 does); that adds at most ulp/2 * sum p|v|
    # to an output element, which matters where the output itself is close to zero: hence the 0.25 floor.
    ulp = 2.0 ** (-10 if dt == 0 else -7)
    assert np.all(np.abs(got - want) <= 2 * ulp * np.maximum(np.abs(want), 0.25)), np.abs(got - want).max()
    # the append half
    assert np.array_equal(as_f32(cache[pos:pos + seq, 0]), k) and np.array_equal(as_f32(cache[pos:pos + seq, 1]), v)


@pytest.mark.parametrize("n", [1, 2048, 32000, 128256])
def test_argmax_half(L, O, n):
    rng = np.random.default_rng(n)
    lg, lt = rand_act(rng, (n,), 0, O, 0.5)
    if n > 100:  # force an exact tie between two far-apart positions: the lower index must win
        top = np.float32(lg.max() + 1.0)
        lg[n // 2] = lg[n - 3] = O.round_to(np.array([top]), 0)[0]
        lt = bits_to_torch(O.from_f32(lg, 0), 0, DEV)
    lib = L.load_library()
    a, s = C.c_size_t(), C.c_size_t()
    assert lib.lcu_calculate_workspace_size_half(C.byref(a), C.byref(s), n) == 0
    ws = torch.empty(max(a.value, s.value), dtype=torch.uint8, device=DEV)
    pair = torch.zeros(2, dtype=torch.int32, device=DEV)
    assert lib.lcu_argmax_half(pair.data_ptr(), lt.data_ptr(), n, ws.data_ptr(), ws.numel(), sp()) == 0
    idx, val = O.argmax(lg)
    got = pair.cpu().numpy().view(np.uint32)
    assert got[0] == idx
    assert np.array([got[1] & 0xFFFF], np.uint16).view(np.float16)[0] == np.float16(val)
    R = O.ref_lib()
    if R is not None:
        ra, rs = C.c_size_t(), C.c_size_t()
        assert R.calculate_workspace_size_half(C.byref(ra), C.byref(rs), n) == 0
        rws = torch.empty(max(ra.value, rs.value), dtype=torch.uint8, device=DEV)
        rp = torch.zeros(2, dtype=torch.int32, device=DEV)
        assert R.argmax_half(rp.data_ptr(), lt.data_ptr(), n, rws.data_ptr(), rws.numel(), sp()) == 0
        torch.cuda.synchronize()
        rgot = rp.cpu().numpy().view(np.uint32)
        assert rgot[0] == got[0] and (rgot[1] & 0xFFFF) == (got[1] & 0xFFFF), "same pair as the reference's CUB arg-max"


@pytest.mark.parametrize("n,temp,topp,topk", [(2048, 1.0, 1.0, 2048), (32000, 0.7, 0.9, 50), (128256, 1.3, 0.95, 1000),
                                              (4096, 0.5, 0.5, 3), (4096, 1.0, 1.0, 2**40)])
def test_sample_half(L, O, n, temp, topp, topk):
    rng = np.random.default_rng(n + topk % 1000)
    lg, lt = rand_act(rng, (n,), 0, O, 1.5)
    lib = L.load_library()
    a, s = C.c_size_t(), C.c_size_t()
    assert lib.lcu_calculate_workspace_size_half(C.byref(a), C.byref(s), n) == 0
    ws = torch.empty(max(a.value, s.value), dtype=torch.uint8, device=DEV)
    pair = torch.zeros(2, dtype=torch.int32, device=DEV)
    hits = 0
    rnds = [0.0, 0.999, 0.5] + list(rng.random(9))
    for r in rnds:
        assert lib.lcu_sample_half(pair.data_ptr(), lt.data_ptr(), None, n, r, temp, topp, min(topk, 2**63), ws.data_ptr(),
                                   ws.numel(), sp()) == 0
        got = pair.cpu().numpy().view(np.uint32)
        idx, val = O.sample(lg, r, temp, topp, topk)
        if got[0] == idx:
            hits += 1
            assert np.array([got[1] & 0xFFFF], np.uint16).view(np.float16)[0] == np.float16(val)
        else:
            # device and host expf may differ in the last bit, which can move a threshold
            # across one entry: accept a neighbour of equal or adjacent value
            assert abs(float(lg[got[0]]) - val) <= 2e-3 * max(1.0, abs(val))
    assert hits >= len(rnds) - 1


def test_sample_rows_mixed(L, O):
    """One launch set for a batch where some rows are arg-max and some sample."""
    rng = np.random.default_rng(5)
    rows, n = 6, 32000
    lg, lt = rand_act(rng, (rows, n), 0, O, 1.0)
    lib = L.load_library()
    args = (L.SampleArgs * rows)(*[L.SampleArgs.arg_max() if i % 2 == 0 else L.SampleArgs.new(0.8, 0.9, 40)
                                   for i in range(rows)])
    at = torch.from_numpy(np.frombuffer(bytes(args), np.uint8).copy()).to(DEV)
    rnd = rng.random(rows).astype(np.float32)
    rt = torch.from_numpy(rnd).to(DEV)
    ws = torch.empty(lib.lcu_sample_rows_workspace_size(rows, n), dtype=torch.uint8, device=DEV)
    out = torch.zeros(rows, 2, dtype=torch.int32, device=DEV)
    cp = torch.zeros(rows, 2, dtype=torch.int32, device=DEV)
    L.check(lib.lcu_op_sample_rows(out.data_ptr(), cp.data_ptr(), lt.data_ptr(), rows, n, at.data_ptr(), rt.data_ptr(), 0,
                                   ws.data_ptr(), ws.numel(), sp()))
    got = out.cpu().numpy().view(np.uint32)
    assert torch.equal(out, cp)
    for i in range(rows):
        if i % 2 == 0:
            assert got[i, 0] == O.argmax(lg[i])[0]
        else:
            idx, val = O.sample(lg[i], float(rnd[i]), 0.8, 0.9, 40)
            assert got[i, 0] == idx or abs(float(lg[i][got[i, 0]]) - val) <= 2e-3
