"""CPU-only checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments with status codes before touching a device."""
import ctypes
import os
import re

import pytest

from proteusai_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(pai_\w+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_status_strings(lib):
    assert lib.pai_abi_version() >= 1
    assert lib.pai_status_str(0) == b"ok"
    for code in range(-9, 0):
        assert lib.pai_status_str(code) not in (b"", b"unknown status")


def test_we_fwd_argument_errors(lib):
    p = ctypes.c_void_p(0x1000)  # never dereferenced: validation fails first
    null = None
    f = lib.pai_we_fwd
    assert f(null, null, p, p, p, p, 1, 8, 4, 0, 8, 1, 0.0, 0, 0, None) == -1
    assert f(p, null, p, p, p, p, 0, 8, 4, 0, 8, 1, 0.0, 0, 0, None) == -2
    assert f(p, null, p, p, p, p, 1, 0, 4, 0, 0, 1, 0.0, 0, 0, None) == -2
    assert f(p, null, p, p, p, p, 1, 8, 0, 0, 8, 1, 0.0, 0, 0, None) == -2
    assert f(p, null, p, p, p, p, 1, 8, 4, 5, 4, 1, 0.0, 0, 0, None) == -6
    assert f(p, null, p, p, p, p, 1, 8, 4, 0, 9, 1, 0.0, 0, 0, None) == -6
    assert f(p, null, p, p, p, p, 1, 8, 4, 0, 8, 7, 0.0, 0, 0, None) == -4
    assert f(p, null, p, p, p, p, 1, 8, 4, 0, 8, 1, 1.0, 0, 0, None) == -4   # dropout_p must be in [0, 1)
    assert f(p, null, p, p, p, p, 1, 8, 4, 0, 8, 1, -0.1, 0, 0, None) == -4
    assert f(p, null, p, p, p, p, 1, 8, 4, 0, 8, 1, float("nan"), 0, 0, None) == -4
    assert f(p, null, p, ctypes.c_void_p(0x1004), p, p, 1, 8, 4, 0, 8, 1, 0.0, 0, 0, None) == -3
    assert f(p, null, p, p, p, p, 1, 8, 4, 0, 8, 1, 0.0, 0, 2, None) == -4       # unknown flag bit


def test_we_bwd_argument_errors(lib):
    p = ctypes.c_void_p(0x1000)
    f = lib.pai_we_bwd_dk
    need = lib.pai_we_bwd_dk_workspace_bytes(2, 16, 8)
    assert need >= 8 * 4
    assert f(None, p, p, p, p, need, 2, 16, 8, 0, 16, None) == -1
    assert f(p, p, p, p, p, need, 2, 16, 0, 0, 16, None) == -2
    assert f(p, p, p, p, p, need, 2, 16, 8, 3, 2, None) == -6
    assert f(p, p, p, p, p, need - 1, 2, 16, 8, 0, 16, None) == -5
    assert f(p, p, p, p, ctypes.c_void_p(0x1008), need, 2, 16, 8, 0, 16, None) == -3


def test_no_cpu_fallback():
    import torch
    from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import wf_embedding
    with pytest.raises(RuntimeError):
        wf_embedding(torch.zeros(1, 4, 3), torch.ones(2), mask=None)


def test_dropin_aliases():
    import sys

    import proteusai_b200
    proteusai_b200.install_dropin(force=True)
    mod = sys.modules["utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding"]
    assert hasattr(mod, "wf_embedding") and hasattr(mod, "_wf_embedding")


def test_geoattn_argument_errors(lib):
    p = ctypes.c_void_p(0x1000)
    f = lib.pai_geoattn_fwd
    args = lambda **kw: [kw.get("Q", p), p, p, p, p, kw.get("betas", p), kw.get("valid", None), kw.get("plan", None),
                         kw.get("sched", None), kw.get("bins", 0), p, p,
                         kw.get("Z", 2), kw.get("H", 2), kw.get("N", 256), kw.get("d", 64), 0.125, kw.get("lo", 0.0), kw.get("hi", 1.0),
                         kw.get("form", 0), kw.get("zb", 0), kw.get("ze", 4), kw.get("qb", 0), kw.get("qe", 256), None]
    assert f(*args(Q=None)) == -1
    assert f(*args(Z=0)) == -2
    assert f(*args(d=32)) == -4           # only d_head = 64 is built
    assert f(*args(form=2)) == -4
    assert f(*args(form=1, betas=None)) == -1
    assert f(*args(form=1, lo=1.0, hi=1.0)) == -2
    assert f(*args(zb=3, ze=2)) == -6
    assert f(*args(ze=5)) == -6
    assert f(*args(qb=64)) == -6          # query ranges start on a tile of 128 ...
    assert f(*args(qe=200)) == -6         # ... and end on one, or at N
    assert f(*args(qb=128, qe=0)) == -6
    assert f(*args(qe=257)) == -6
    assert f(*args(Q=ctypes.c_void_p(0x1008))) == -3
    assert f(*args(valid=p)) == -1        # a mask needs the plan made from it
    assert f(*args(valid=p, plan=ctypes.c_void_p(0x1004))) == -3
    assert f(*args(valid=p, plan=p, sched=p, bins=0)) == -2              # a schedule names its number of CTAs
    assert f(*args(valid=p, plan=p, sched=p, bins=296, qe=128)) == -6    # ... and covers the whole problem
    assert f(*args(valid=p, plan=p, sched=ctypes.c_void_p(0x1004), bins=296)) == -3
    g = lib.pai_geoattn_bwd
    need = lib.pai_geoattn_bwd_workspace_bytes(2, 2, 64, 64)
    assert need == 2 * 2 * 64 * 4
    base = [p] * 8 + [p, None, None, None, 0] + [p] * 5 + [p, need, 2, 2, 64, 64, 0.125, 0.0, 1.0, 0, 0, 4, 0, 64, None]
    bad = list(base)
    bad[19] = need - 1
    assert g(*bad) == -5
    bad = list(base)
    bad[0] = None
    assert g(*bad) == -1
    bad = list(base)
    bad[27] = 1      # logit form 1 ...
    bad[17] = None   # ... without a dbetas buffer
    assert g(*bad) == -1
    bad = list(base)
    bad[30] = 32     # query range off the tile grid
    assert g(*bad) == -6
    # the batch plan
    nbytes = lib.pai_geoattn_plan_bytes(4, 1000)
    assert nbytes == 4 * (4 + 3 * 4 + 2 * 4 * 8)
    assert lib.pai_geoattn_plan_bytes(0, 10) == 0
    h = lib.pai_geoattn_plan
    assert h(None, 4, 1000, p, nbytes, None) == -1
    assert h(p, 4, 1000, p, nbytes - 1, None) == -5
    assert h(p, 0, 1000, p, nbytes, None) == -2
    assert h(p, 4, 1000, ctypes.c_void_p(0x1004), nbytes, None) == -3
    assert lib.pai_tune_set(999, 1) == -4
    # the balanced schedule
    sbytes = lib.pai_geoattn_schedule_bytes(4, 1000, 8, 296)
    assert sbytes == 4 * (8 + 296 + 296 * (4 * ((4 * 8 * 8 + 295) // 296) + 8) + 4 * 8 * 8)
    assert lib.pai_geoattn_schedule_bytes(4, 1000, 8, 2000) == 0
    k = lib.pai_geoattn_schedule
    assert k(None, 4, 1000, 8, 296, 0, p, sbytes, None) == -1
    assert k(p, 4, 1000, 8, 0, 0, p, sbytes, None) == -2
    assert k(p, 4, 1000, 8, 296, 0, p, sbytes - 1, None) == -5
    assert k(p, 4, 1000, 8, 296, 0, ctypes.c_void_p(0x1004), sbytes, None) == -3


def test_strided_attention_and_row_op_argument_errors(lib):
    p = ctypes.c_void_p(0x1000)
    i64 = lambda *v: (ctypes.c_int64 * 3)(*v)
    ok = i64(2 * 64 * 64, 64 * 64, 64)
    f = lib.pai_geoattn_fwd_strided
    call = lambda **kw: f(p, kw.get("qs", ok), p, ok, p, ok, p, p, None, None, None, None, 0, p, kw.get("os", ok), p, 2, 2, 64,
                          kw.get("d", 64), 0.125, 0.0, 1.0, 0, 0, kw.get("ze", 4), 0, 64, None)
    assert call(qs=None) == -1
    assert call(d=32) == -4
    assert call(ze=5) == -6
    assert call(qs=i64(2 * 64 * 64, 64 * 64, 68)) == -3     # rows off the 16-byte grid
    assert call(os=i64(2 * 64 * 64, 64 * 64, 32)) == -2     # overlapping rows
    assert call(qs=i64(-8, 64 * 64, 64)) == -2
    g = lib.pai_add_layernorm_bf16
    assert g(None, p, p, p, 0, p, 4, 512, 1e-5, None) == -1
    assert g(p, p, p, p, 0, p, 4, 516, 1e-5, None) == -2      # D must be a multiple of 8
    assert g(p, p, p, p, 0, p, 4, 8192, 1e-5, None) == -2     # ... and at most 4096
    assert g(p, ctypes.c_void_p(0x1008), p, p, 0, p, 4, 512, 1e-5, None) == -3
    h = lib.pai_gelu_bf16
    assert h(p, None, 64, None) == -1
    assert h(p, p, 60, None) == -2
    assert h(ctypes.c_void_p(0x1004), p, 64, None) == -3


def test_neighbour_and_edge_argument_errors(lib):
    p = ctypes.c_void_p(0x1000)
    f = lib.pai_knn_neighbors
    assert f(None, None, p, p, 1, 64, 30, 12.0, None) == -1
    assert f(p, None, p, p, 1, 20, 30, 12.0, None) == -2     # K <= N, as the reference asserts
    assert f(p, None, p, p, 1, 128, 65, 12.0, None) == -4    # at most 64 neighbours
    assert f(p, None, ctypes.c_void_p(0x1004), p, 1, 64, 30, 12.0, None) == -3
    g = lib.pai_edge_rbf
    assert g(p, p, None, 1.25, None, None, 0.0, p, 1, 64, 30, 4, 16, None) == -1
    assert g(p, p, p, 0.0, None, None, 0.0, p, 1, 64, 30, 4, 16, None) == -2
    assert g(p, p, p, 1.25, None, None, 0.0, ctypes.c_void_p(0x1008), 1, 64, 30, 4, 16, None) == -3
    assert g(p, p, p, 1.25, p, None, 1e-5, p, 1, 64, 30, 4, 16, None) == -1      # gamma without beta
    assert g(p, p, p, 1.25, p, p, 1e-5, p, 1, 64, 30, 3, 16, None) == -4         # fused LayerNorm: 4 x 4 x 16 only
