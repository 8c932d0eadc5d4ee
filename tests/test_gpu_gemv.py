"""GPU parity of the streaming layout and the stand-alone int4 GEMV, through the C ABI, against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

from flint_b200 import _lib, packing
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _repack(lib, q, s, z, order=0, arg=0, orows=0):
    rows, k = q.shape[0], q.shape[1] * 8
    nbytes = lib.fb_stream_bytes(rows, k, int(z is not None))
    assert nbytes > 0
    out = torch.empty(nbytes + 16, dtype=torch.uint8, device="cuda")
    _lib.check(lib.fb_repack(_p(q), _p(s), _p(z) if z is not None else None, rows, k, order, arg, orows, _p(out), None),
               "fb_repack")
    return out


def _mat(rows, k, seed, asym):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(rows, k, generator=g) * 0.02).bfloat16()
    W[0, :128] = 0                      # an all-zero group rides along
    if asym:
        q, s, z = packing.qpc_asym(W)
    else:
        (q, s), z = packing.qpc(W), None
    return q, s, z


@pytest.mark.parametrize("asym", [False, True])
@pytest.mark.parametrize("order", [0, 1, 2])
def test_streaming_layout_dequant_bit_exact(asym, order):
    lib = _lib.load()
    rows, k = 384, 512
    q, s, z = _mat(rows, k, 1, asym)
    arg, orows = (0, 0) if order == 0 else ((64, 256) if order == 1 else (rows // 2, 0))
    dq, ds, dz = q.cuda(), s.cuda(), (z.cuda() if z is not None else None)
    st = _repack(lib, dq, ds, dz, order, arg, orows)
    out = torch.empty(rows, k, dtype=torch.float32, device="cuda")
    _lib.check(lib.fb_dequant(_p(st), rows, k, int(asym), order, arg, orows, _p(out), None), "fb_dequant")
    torch.cuda.synchronize()
    ref = O.c_dequant(q, s, z)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("k", [512, 640, 1280, 14336])          # tile heights 4, 16, 8, 2
@pytest.mark.parametrize("asym", [False, True])
def test_streaming_layout_every_tile_height(k, asym):
    """Rows that do not fill the last tile: the padding rows must not leak into the rows that exist."""
    lib = _lib.load()
    rows = 37
    q, s, z = _mat(rows, k, 11, asym)
    st = _repack(lib, q.cuda(), s.cuda(), z.cuda() if z is not None else None)
    out = torch.empty(rows, k, dtype=torch.float32, device="cuda")
    _lib.check(lib.fb_dequant(_p(st), rows, k, int(asym), 0, 0, 0, _p(out), None), "fb_dequant")
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), O.c_dequant(q, s, z).view(np.uint32))


@pytest.mark.parametrize("k", [512, 640, 1024, 1280, 1408, 1792, 2048, 2560, 3584, 4096, 7168, 8192, 14336])
@pytest.mark.parametrize("asym", [False, True])
def test_gemv_vs_oracle(k, asym):
    """Every K the decode kernels are built for (tensor-parallel slices included); row counts that are ragged against
    148 CTAs and the tile sizes.
    Same criterion family as the reference's GEMV check (reference: bench/int4_kernel_test.py:80-91), tightened:
    the reference accepts rel-L2 < 0.02, fp32 accumulation over identical dequantised weights gives < 1e-5."""
    lib = _lib.load()
    for rows in (1, 149, 1000):
        q, s, z = _mat(rows, k, 7 + rows, asym)
        g = torch.Generator().manual_seed(5)
        x = torch.randn(k, generator=g).bfloat16()
        dq, ds, dz, dx = q.cuda(), s.cuda(), (z.cuda() if z is not None else None), x.cuda()
        st = _repack(lib, dq, ds, dz)
        y = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda")
        status = torch.zeros(8, dtype=torch.int32, device="cuda")
        _lib.check(lib.fb_gemv(_p(st), rows, k, int(asym), 0, 0, 0, _p(dx), _p(y), _p(status), None), "fb_gemv")
        torch.cuda.synchronize()
        assert int(status[0]) == 0, status.tolist()
        ref = O.c_gemv(q, s, z, x)[0]
        got = y.cpu().numpy()
        scale = np.abs(ref).max() + 1e-6
        assert np.abs(got - ref).max() / scale < 2e-5, (k, rows, np.abs(got - ref).max(), scale)


@pytest.mark.parametrize("e", [-100, 60, 100])
def test_gemv_power_of_two_activations_are_exact(e):
    """The kernel multiplies fp16 copies of the activations; a power of two per group of 128 columns keeps that exact
    over the whole bf16 range: scaling x by 2^e (one group by a different power) scales y by exactly 2^e."""
    lib = _lib.load()
    rows, k = 300, 2560
    q, s, z = _mat(rows, k, 21, True)
    x = torch.randn(k, generator=torch.Generator().manual_seed(6)).bfloat16()
    x[128:256] *= 2.0 ** -20            # one group far below the others
    x[512:640] = 0                      # and an all-zero group
    st = _repack(lib, q.cuda(), s.cuda(), z.cuda())
    ys = []
    for f in (1.0, 2.0 ** e):
        dx = (x.float() * f).bfloat16().cuda()
        y = torch.zeros(rows, dtype=torch.float32, device="cuda")
        status = torch.zeros(8, dtype=torch.int32, device="cuda")
        _lib.check(lib.fb_gemv(_p(st), rows, k, 1, 0, 0, 0, _p(dx), _p(y), _p(status), None), "fb_gemv")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        ys.append(y.cpu().numpy().astype(np.float64))
    assert np.array_equal(ys[0] * 2.0 ** e, ys[1])
    ref = O.c_gemv(q, s, z, x)[0]
    assert np.abs(ys[0] - ref).max() < 2e-5 * (np.abs(ref).max() + 1e-6)


def test_gemv_permuted_rows_land_in_source_order():
    lib = _lib.load()
    rows, k = 768, 512           # tiny-config QKV: 8 q + 2 k heads of 64 paired, 2 v heads plain
    q, s, z = _mat(rows, k, 3, False)
    x = torch.randn(k, generator=torch.Generator().manual_seed(9)).bfloat16()
    st = _repack(lib, q.cuda(), s.cuda(), None, 1, 64, 640)
    y = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    _lib.check(lib.fb_gemv(_p(st), rows, k, 0, 1, 64, 640, _p(x.cuda()), _p(y), _p(status), None), "fb_gemv")
    torch.cuda.synchronize()
    ref = O.c_gemv(q, s, None, x)[0]
    assert np.abs(y.cpu().numpy() - ref).max() < 2e-5 * (np.abs(ref).max() + 1e-6)


def test_gemv_linearity_full_size():
    """Full-size matrix (gate/up of the 3B-class model: 16384 x 2560): W(a) + W(b) == W(a+b) up to bf16 rounding of
    the inputs is not exact, so use the exact property W(2x) == 2 W(x) (scaling by 2 is exact in bf16 and fp32)."""
    lib = _lib.load()
    rows, k = 16384, 2560
    g = torch.Generator(device="cuda").manual_seed(0)
    W = (torch.randn(rows, k, generator=g, device="cuda") * 0.02).bfloat16()
    q, s = packing.qpc(W)
    x = torch.randn(k, generator=g, device="cuda").bfloat16()
    st = _repack(lib, q, s, None)
    ys = []
    for xx in (x, (x.float() * 2).bfloat16()):
        y = torch.zeros(rows, dtype=torch.float32, device="cuda")
        status = torch.zeros(8, dtype=torch.int32, device="cuda")
        _lib.check(lib.fb_gemv(_p(st), rows, k, 0, 0, 0, 0, _p(xx), _p(y), _p(status), None), "fb_gemv")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        ys.append(y)
    assert torch.equal(ys[0] * 2, ys[1])
    ref = (packing.dequant(q, s).double() @ x.double()).float()
    assert (ys[0] - ref).abs().max() / ref.abs().max() < 2e-5
