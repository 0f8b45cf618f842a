"""The allocation-free arg-max entry point (needs a B200).

`lcu_argmax_rows_noalloc` serves hosts that may not allocate device memory on the path that
samples — for example a serving loop that keeps cudaMalloc, which synchronises the whole
device, away from its token loop, or a host whose memory is owned by an external pool —
by keeping its partial results in a fixed array inside the library.  This file is collected
last on purpose, so a run that stops at the first failure has already run everything else.
It checks the new entry point against the existing workspace-taking one, twice in a row,
and that oversize problems are refused with a message.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _reference_pairs(L, logits, dt):
    lib = L.load_library()
    rows, n = logits.shape
    ws = torch.empty(lib.lcu_sample_rows_workspace_size(rows, n), dtype=torch.uint8, device=DEV)
    out = torch.zeros(rows, 2, dtype=torch.int32, device=DEV)
    L.check(lib.lcu_op_sample_rows(out.data_ptr(), None, logits.data_ptr(), rows, n, None, None, dt, ws.data_ptr(),
                                   ws.numel(), _stream()))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("rows,n,dt", [(1, 128256, 0), (32, 32000, 0), (5, 2048, 1), (64, 128256, 0), (300, 128256, 0)])
def test_noalloc_argmax_matches_workspace_version_twice(L, rows, n, dt):
    lib = L.load_library()
    tdt = torch.float16 if dt == 0 else torch.bfloat16
    g = torch.Generator(device=DEV)
    g.manual_seed(rows * 1000 + n)
    slots = rows * ((n + 4095) // 4096)
    for call in range(2):  # two calls in a row share the built-in scratch
        logits = torch.randn(rows, n, device=DEV, generator=g).to(tdt)
        if n > 100:
            logits[:, n // 3] = logits[:, n - 2] = 9.0  # an exact tie: the lower index must win
        out = torch.zeros(rows, 2, dtype=torch.int32, device=DEV)
        rc = lib.lcu_argmax_rows_noalloc(out.data_ptr(), logits.data_ptr(), rows, n, dt, _stream())
        if slots > 8192:
            assert rc == L.ERR_INVALID and b"scratch holds" in lib.lcu_last_error_string()
            return
        L.check(rc)
        torch.cuda.synchronize()
        want = _reference_pairs(L, logits, dt)
        assert torch.equal(out, want), f"call {call}"
        if n > 100:
            assert (out[:, 0] == n // 3).all()


def test_noalloc_rejects_bad_arguments(L):
    lib = L.load_library()
    out = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    lg = torch.zeros(16, dtype=torch.float16, device=DEV)
    assert lib.lcu_argmax_rows_noalloc(None, lg.data_ptr(), 1, 16, 0, _stream()) == L.ERR_INVALID
    assert lib.lcu_argmax_rows_noalloc(out.data_ptr(), lg.data_ptr(), 0, 16, 0, _stream()) == L.ERR_INVALID
    assert lib.lcu_argmax_rows_noalloc(out.data_ptr(), lg.data_ptr(), 1, 16, 2, _stream()) == L.ERR_INVALID
