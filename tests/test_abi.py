"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header
declares, and refuses to compute without a GPU (no fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "lcu.h")).read()
    return sorted(set(re.findall(r"LCU_API[^;(]*?\b(lcu_\w+)\s*\(", text)))


def test_header_declares_what_the_binding_binds(L):
    syms = header_symbols()
    assert len(syms) >= 40
    assert syms == L.exported_symbols()


def test_library_exports_every_declared_symbol(L):
    lib = C.CDLL(L.LIB_PATH)
    for s in header_symbols():
        assert hasattr(lib, s), s
    assert L.load_library().lcu_version() >= 100


def test_header_cites_the_reference_for_every_entry_point():
    text = open(os.path.join(ROOT, "include", "lcu.h")).read()
    for needle in ["op/rms_norm", "op/rope", "op/swiglu", "op/linear.rs", "op/embedding", "op/fast_embedding",
                   "random_sample/sample.h", "exec/kv_cache.rs", "exec/engine.rs", "exec/step.rs", "op/all_reduce.rs",
                   "exec/output_head.rs", "memory.rs", "handle.rs"]:
        assert needle in text, needle


def test_header_is_plain_c():
    import subprocess
    src = '#include "lcu.h"\nint main(void){lcu_model_desc d; lcu_kv_pair p; (void)d; (void)p; return sizeof(lcu_kv_pair)==8 && sizeof(lcu_sample_args)==16 && sizeof(lcu_req)==12 ? 0 : 1;}\n'
    exe = "/tmp/lcu_header_check"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-x", "c", "-", "-o", exe],
                   input=src.encode(), check=True)
    assert subprocess.run([exe]).returncode == 0


def test_struct_layouts_match(L):
    assert C.sizeof(L.KVPair) == 8 and C.sizeof(L.SampleArgs) == 16 and C.sizeof(L.Req) == 12
    assert C.sizeof(L.ModelDesc) == 16 * 4


def test_sample_args_rules(L):
    """== SampleArgs::new / is_argmax (llama.cu/src/op/random_sample/mod.rs:58-82)."""
    assert L.SampleArgs.arg_max().is_argmax()
    assert L.SampleArgs.new(0.0, 0.5, 10).is_argmax()
    assert L.SampleArgs.new(0.7, 0.5, 1).is_argmax()
    assert not L.SampleArgs.new(0.7, 2.0, 10).is_argmax()
    assert L.SampleArgs.new(0.7, 2.0, 10).top_p == 1.0
    with pytest.raises(ValueError):
        L.SampleArgs.new(-1.0, 0.5, 10)
    with pytest.raises(ValueError):
        L.SampleArgs.new(1.0, 0.0, 10)
    with pytest.raises(ValueError):
        L.SampleArgs.new(1.0, 0.5, 0)


def test_host_helpers_need_no_gpu(L):
    lib = L.load_library()
    assert lib.lcu_q8_0_repacked_bytes(4096, 4096) == 4096 * 4096 + 4096 * 128 * 2
    a, s = C.c_size_t(), C.c_size_t()
    assert lib.lcu_calculate_workspace_size_half(C.byref(a), C.byref(s), 128256) == 0
    assert 0 < a.value < s.value
    assert lib.lcu_sample_rows_workspace_size(4, 32000) > 4 * 65536 * 4
    sin, cos = L.build_sin_cos(8, 64, 1e4)
    assert sin.shape == (8, 32) and cos[0, 0] == 1.0
    assert lib.lcu_build_sin_cos(0, 64, 1e4, None, None) == L.ERR_INVALID
    assert b"build_sin_cos" in lib.lcu_last_error_string()


def test_invalid_descriptions_are_rejected(L):
    cfg = L.CONFIGS["tiny"]
    for field, bad in [("dh", 48), ("nkvh", 3), ("act_dtype", 2), ("d", 0)]:
        d = cfg.desc()
        setattr(d, field, bad)
        with pytest.raises(L.LcuError) as e:
            L.Context(d)
        assert e.value.code == L.ERR_INVALID
    with pytest.raises(L.LcuError):
        L.Context(cfg.desc(), tp_rank=0, tp_size=3)   # nkvh = 4 does not divide by 3
    with pytest.raises(L.LcuError):
        L.Context(cfg.desc(), tp_rank=0, tp_size=2)   # tensor parallelism needs a communicator


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_tuning_keys_are_validated(L):
    """lcu_set_tuning accepts the documented keys (restoring their defaults here) and refuses anything else; it needs
    neither a context nor a GPU."""
    defaults = {"pdl_edges": -1, "gemv_ctas_per_sm": 2, "q8_rows": 4, "gemv_lean_norm": 1, "rms_pdl": 1, "tc": 1,
                "tc_block": 256, "tc_cluster": 1, "p2p_scatter_ranks": 8, "p2p_scatter_min": 131072}
    for key, value in defaults.items():
        L.set_tuning(key, value)
    with pytest.raises(L.LcuError):
        L.set_tuning("no_such_key", 1)
    with pytest.raises(L.LcuError):
        L.set_tuning("tc_block", 96)
    with pytest.raises(L.LcuError):
        L.set_tuning("gemv_ctas_per_sm", 3)


def test_no_cpu_fallback(L):
    """Without a device the product path fails loudly instead of computing on the host."""
    with pytest.raises(L.LcuError) as e:
        L.Context(L.CONFIGS["tiny"].desc())
    assert e.value.code == L.ERR_CUDA
    assert "CUDA" in str(e.value)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "llama.cu_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "__init__.py" and "oracle" not in text, (dirpath, f)


def test_model_shapes_and_bytes(L):
    c = L.CONFIGS["llama8b"]
    assert abs(c.weight_bytes_per_step() - 15.0104e9) / 15.0104e9 < 1e-3
    assert c.kv_bytes_per_token() == 128 * 1024
    assert abs(L.CONFIGS["llama1b"].weight_bytes_per_step() - 2.4718e9) / 2.4718e9 < 1e-3
    assert L.CONFIGS["llama1b"].kv_bytes_per_token() == 32 * 1024
    assert abs(L.CONFIGS["llama8b_q8"].weight_bytes_per_step() - 8.4673e9) / 8.4673e9 < 1e-3
    c70 = L.CONFIGS["llama70b"]
    assert abs(c70.weight_bytes_per_step() - 137.43e9) / 137.43e9 < 1e-3 and c70.kv_bytes_per_token() == 320 * 1024
    assert abs(c70.weight_bytes_per_step(8) - 17.64e9) / 17.64e9 < 2e-3
    assert L.CONFIGS["tiny"].kv_bytes_per_token() == 2048


def test_synthetic_weights_are_seeded(L):
    cfg = L.CONFIGS["tiny"]
    a, b, c = L.synth_weights_numpy(cfg, 0), L.synth_weights_numpy(cfg, 0), L.synth_weights_numpy(cfg, 1)
    k = (0, L.W_QKV)
    assert np.array_equal(a[k], b[k]) and not np.array_equal(a[k], c[k])
    assert a[k].shape == (768, 256) and a[(1, L.W_GATE_UP)].shape == (1376, 256) and a[(0, L.W_DOWN)].shape == (256, 688)
    w = a[k].view(np.float16).astype(np.float32)
    assert abs(w.std() - 0.02) < 1e-3 and abs(w.mean()) < 1e-3
    assert (a[(0, L.W_ATTN_NORM)].view(np.float16) == 1).all()
