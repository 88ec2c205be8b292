"""The allocation-free WE backward entry point against the workspace one.

Some callers cannot allocate GPU memory when they call into the library (a server that gave all of
the device to its own pool at start-up and forbids cudaMalloc afterwards, for instance), so they have
no scratch buffer to hand to ``pai_we_bwd_dk``.  ``pai_we_bwd_dk_static`` keeps its scratch inside the
library instead.  Both entry points run the same two kernels on the same partition of the rows, so
their results must agree; this file checks that through the C ABI on two calls in a row (the second
with different data and a different shape, so anything left in the shared scratch by the first call
would show), and that a wavenumber count beyond the built-in limit is refused.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DK_TOL = 1e-3  # relative L2, the tolerance of the other wavenumber-gradient tests


def _rel(a, b):
    return float(torch.norm(a.double() - b.double()) / torch.norm(a.double()).clamp_min(1e-30))


def _both(lib, z, n, k, rows, seed):
    from proteusai_b200 import _lib
    g = torch.Generator().manual_seed(seed)
    d_out = torch.randn(z, n, 2 * k, generator=g).cuda()
    cs = torch.randn(z, n, k, generator=g).cuda()
    sn = torch.randn(z, n, k, generator=g).cuda()
    r0, r1 = rows
    # existing entry point, caller-provided workspace
    ws_bytes = lib.pai_we_bwd_dk_workspace_bytes(z, n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    dk_ws = torch.full((k,), float("nan"), device="cuda")
    _lib.check(lib.pai_we_bwd_dk(_lib.ptr(d_out), _lib.ptr(cs), _lib.ptr(sn), _lib.ptr(dk_ws), _lib.ptr(ws), ws_bytes,
                                 z, n, k, r0, r1, _lib.current_stream()), "pai_we_bwd_dk")
    # allocation-free entry point: inputs and the output only
    dk_st = torch.full((k,), float("nan"), device="cuda")
    _lib.check(lib.pai_we_bwd_dk_static(_lib.ptr(d_out), _lib.ptr(cs), _lib.ptr(sn), _lib.ptr(dk_st),
                                        z, n, k, r0, r1, _lib.current_stream()), "pai_we_bwd_dk_static")
    torch.cuda.synchronize()
    ref = ((d_out[:, r0:r1, 1::2].double() * cs[:, r0:r1].double())
           - (d_out[:, r0:r1, 0::2].double() * sn[:, r0:r1].double())).sum(dim=(0, 1))
    return dk_ws, dk_st, ref


def test_static_scratch_matches_workspace_entry_point_twice():
    from proteusai_b200 import _lib
    assert torch.cuda.is_available()
    lib = _lib.lib()
    assert lib.pai_we_bwd_dk_static_max_k() == 1024
    # two calls in a row; the second is smaller, so stale partial rows of the first stay in the scratch
    for z, n, k, rows, seed in ((8, 1024, 256, (0, 1024), 1), (2, 300, 96, (10, 250), 2), (1, 64, 1024, (0, 64), 3)):
        dk_ws, dk_st, ref = _both(lib, z, n, k, rows, seed)
        assert torch.isfinite(dk_st).all()
        assert _rel(dk_ws, dk_st) < DK_TOL, (z, n, k)
        assert torch.equal(dk_ws, dk_st), "same kernels, same row partition: the two results are identical"
        assert _rel(ref, dk_st) < DK_TOL, (z, n, k)
    # an empty row range gives zeros
    d_out = torch.randn(1, 16, 8, device="cuda")
    cs = torch.randn(1, 16, 4, device="cuda")
    dk = torch.full((4,), float("nan"), device="cuda")
    _lib.check(lib.pai_we_bwd_dk_static(_lib.ptr(d_out), _lib.ptr(cs), _lib.ptr(cs), _lib.ptr(dk), 1, 16, 4, 5, 5,
                                        _lib.current_stream()), "pai_we_bwd_dk_static")
    assert torch.all(dk == 0)


def test_static_scratch_rejects_too_many_wavenumbers():
    from proteusai_b200 import _lib
    lib = _lib.lib()
    p = ctypes.c_void_p(0x1000)  # never dereferenced: the size check comes first
    status = lib.pai_we_bwd_dk_static(p, p, p, p, 1, 8, 1025, 0, 8, None)
    assert status == -9
    assert b"1024" in lib.pai_status_str(status)


def test_static_entry_point_allocates_nothing_and_keeps_one_scratch_per_device():
    """What the entry point exists for: once the first call on a device has looked the scratch up, further calls leave
    the amount of free device memory exactly where it was (cudaMemGetInfo), whatever K they use.  With a second GPU
    visible the same holds there, and the results are right on both: the address kept per device is that device's own."""
    from proteusai_b200 import _lib
    lib = _lib.lib()
    for dev in range(min(torch.cuda.device_count(), 2)):
        with torch.cuda.device(dev):
            g = torch.Generator().manual_seed(40 + dev)
            shapes = ((2, 128, 64), (1, 77, 200), (3, 50, 1024))
            data = [(torch.randn(z, n, 2 * k, generator=g).cuda(), torch.randn(z, n, k, generator=g).cuda(),
                     torch.randn(z, n, k, generator=g).cuda(), torch.empty(k, device="cuda")) for z, n, k in shapes]
            call = lambda d_out, cs, sn, dk: _lib.check(lib.pai_we_bwd_dk_static(
                _lib.ptr(d_out), _lib.ptr(cs), _lib.ptr(sn), _lib.ptr(dk), cs.shape[0], cs.shape[1], cs.shape[2], 0, cs.shape[1],
                _lib.current_stream()), "pai_we_bwd_dk_static")
            call(*data[0])                       # first call on this device: looks the scratch address up
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            for _ in range(3):
                for item in data:
                    call(*item)
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, (dev, free_before, free_after)
            for d_out, cs, sn, dk in data:
                ref = (d_out[:, :, 1::2].double() * cs.double() - d_out[:, :, 0::2].double() * sn.double()).sum(dim=(0, 1))
                assert _rel(ref, dk) < DK_TOL, dev
