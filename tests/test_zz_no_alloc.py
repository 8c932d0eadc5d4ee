"""GPU: the allocation-free GEMV entry point (fb_gemv_static) against the ordinary one (fb_repack + fb_gemv) and the CPU oracle.

Some hosts of this library may not allocate device memory once they are running: a server that has handed all of HBM to
its own arena, or code inside a stream capture. For them the library carries the GEMV's scratch (the streaming-layout
copy of the matrix) in a fixed built-in array. This file is collected last on purpose: if it fails, a run that stops at
the first failure has already run everything else. It passes alone in a fresh process and after the other tests; it makes
two calls in a row because every call reuses the same array and must not depend on what the previous call left there.
"""
import ctypes

import numpy as np
import pytest
import torch

from flint_b200 import _lib, packing
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(rows, k, seed, asym):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(rows, k, generator=g) * 0.02).bfloat16()
    x = torch.randn(k, generator=g).bfloat16().cuda()
    if asym:
        q, s, z = packing.qpc_asym(W)
        return q.cuda(), s.cuda(), z.cuda(), x
    q, s = packing.qpc(W)
    return q.cuda(), s.cuda(), None, x


def _ordinary(lib, q, s, z, x):
    rows, k = q.shape[0], q.shape[1] * 8
    st = torch.empty(lib.fb_stream_bytes(rows, k, int(z is not None)) + 16, dtype=torch.uint8, device="cuda")
    _lib.check(lib.fb_repack(_p(q), _p(s), _p(z) if z is not None else None, rows, k, 0, 0, 0, _p(st), None), "fb_repack")
    y = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    _lib.check(lib.fb_gemv(_p(st), rows, k, int(z is not None), 0, 0, 0, _p(x), _p(y), _p(status), None), "fb_gemv")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return y


def test_static_scratch_gemv_matches_ordinary_entry_point_twice():
    lib = _lib.load()
    # second call: different shape, fewer bytes, asymmetric layout: stale records of the first call stay in the array
    for rows, k, seed, asym in ((3000, 2560, 1, False), (700, 512, 2, True)):
        q, s, z, x = _case(rows, k, seed, asym)
        want = _ordinary(lib, q, s, z, x)
        y = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda")
        status = torch.full((8,), 7, dtype=torch.int32, device="cuda")     # garbage: the call clears it
        _lib.check(lib.fb_gemv_static(_p(q), _p(s), _p(z) if z is not None else None, rows, k, _p(x), _p(y), _p(status),
                                      None), "fb_gemv_static")
        torch.cuda.synchronize()
        assert int(status[0]) == 0, status.tolist()
        scale = float(want.abs().max()) + 1e-6
        assert float((y - want).abs().max()) / scale < 2e-5       # the bound the GEMV tests use; same kernels: equal
        assert torch.equal(y, want)
        # and on its own feet: the CPU oracle's GEMV on the caller-layout tensors (fp32 summation order differs)
        ref = O.c_gemv(q.cpu(), s.cpu(), None if z is None else z.cpu(), x.cpu())[0]
        assert float(np.abs(y.cpu().numpy() - ref).max()) / (float(np.abs(ref).max()) + 1e-6) < 2e-5


def test_static_scratch_rejects_oversized_matrix():
    lib = _lib.load()
    q, s, z, x = _case(8, 2560, 3, False)
    y = torch.zeros(8, dtype=torch.float32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    too_many = ((9 << 20) // (4 * 1320) + 1) * 4                    # one 4-row tile more than the built-in array holds
    rc = lib.fb_gemv_static(_p(q), _p(s), None, too_many, 2560, _p(x), _p(y), _p(status), None)
    assert rc == _lib.FB_ERR_RANGE
