"""Kernel-level parity on the GPU: every C-ABI entry point against the CPU oracle (evaluated in
fp64 on the same seeded inputs).  Tolerances: factors 1e-5 relative Frobenius, inverses /
preconditioned updates / Cholesky factors 1e-4."""
import math

import numpy as np
import pytest
import torch

import cases
from oracle import kfac_oracle as ko

pytestmark = pytest.mark.gpu

FACTOR_TOL = 1e-5
INV_TOL = 1e-4


@pytest.fixture(scope='module')
def nat():
    from torchsso import _native
    _native.lib()
    return _native


def rel(a, b):
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-300)).item()


def dev(t):
    return t.cuda()


# ------------------------------------------------------------------------------------ factors
@pytest.mark.parametrize('rows,cols,bias', [(128, 784, True), (128, 1000, True), (128, 10, False),
                                            (32, 2048, True), (300, 147, False), (5000, 64, False),
                                            (9000, 129, True), (1, 7, True)])
def test_factor_rows_matches_oracle(nat, rows, cols, bias):
    x = cases.make_normal((rows, cols), 10 + rows + cols)
    d = cols + int(bias)
    out = torch.full((d, d), float('nan'), device='cuda')
    nat.factor_rows(dev(x), bias, None, 1.0 / rows, 0.0, out, nat.IMPL_SIMT)
    ref = ko.linear_factor_A(x.double(), bias)
    assert rel(out, ref) < FACTOR_TOL
    assert torch.equal(out, out.t())


def test_factor_rows_weighted_accumulate_and_strides(nat):
    rows, cols = 200, 96
    g = cases.make_normal((rows, cols), 3)
    p = torch.rand(rows, generator=torch.Generator().manual_seed(5))
    ref = ko.linear_factor_G(g.double(), p.double())
    out = torch.zeros((cols, cols), device='cuda')
    nat.factor_rows(dev(g), False, dev(p), 0.5 / rows, 0.0, out, nat.IMPL_SIMT)
    nat.factor_rows(dev(g), False, dev(p), 0.5 / rows, 1.0, out, nat.IMPL_SIMT)   # accumulate
    assert rel(out, ref) < FACTOR_TOL
    # column-major view of the same matrix (rows contiguous)
    gt = dev(g).t().contiguous().t()
    assert gt.stride() == (1, rows)
    out2 = torch.empty((cols, cols), device='cuda')
    nat.factor_rows(gt, False, dev(p), 1.0 / rows, 0.0, out2, nat.IMPL_SIMT)
    assert rel(out2, ref) < FACTOR_TOL


def test_factor_rows_bf16_input(nat):
    x = cases.make_normal((512, 200), 8).bfloat16()
    out = torch.empty((201, 201), device='cuda')
    nat.factor_rows(dev(x), True, None, 1.0 / 512, 0.0, out, nat.IMPL_SIMT)
    assert rel(out, ko.linear_factor_A(x.double(), True)) < FACTOR_TOL


CONVS = [
    # n, c, h, w, k, stride, pad, dil, bias
    (4, 3, 12, 12, (5, 5), (1, 1), (2, 2), (1, 1), True),
    (3, 8, 9, 7, (3, 3), (2, 2), (1, 1), (1, 1), False),
    (2, 5, 10, 10, (3, 2), (1, 2), (0, 1), (2, 1), True),
    (2, 64, 14, 14, (1, 1), (1, 1), (0, 0), (1, 1), False),
    (2, 3, 30, 30, (7, 7), (2, 2), (3, 3), (1, 1), False),
    (8, 16, 32, 32, (3, 3), (1, 1), (1, 1), (1, 1), True),      # 8192 rows: split path
    (2, 130, 6, 6, (3, 3), (1, 1), (1, 1), (1, 1), False),      # d = 1170: many tiles
]


@pytest.mark.parametrize('cfg', CONVS)
@pytest.mark.parametrize('channels_last', [False, True])
def test_factor_conv_A_matches_oracle(nat, cfg, channels_last):
    n, c, h, w, k, s, p, d, bias = cfg
    x = cases.make_normal((n, c, h, w), 21 + c + h)
    ref = ko.conv_factor_A(x.double(), k, s, p, d, bias)
    xd = dev(x)
    if channels_last:
        xd = xd.contiguous(memory_format=torch.channels_last)
    out = torch.full(tuple(ref.shape), float('nan'), device='cuda')
    nat.factor_im2col(xd, k, s, p, d, bias, None, 1.0 / n, 0.0, out, nat.IMPL_SIMT)
    assert rel(out, ref) < FACTOR_TOL
    assert torch.equal(out, out.t())


@pytest.mark.parametrize('channels_last', [False, True])
def test_factor_conv_G_weighted(nat, channels_last):
    n, c, h, w = 6, 40, 7, 7
    g = cases.make_normal((n, c, h, w), 77)
    p = torch.rand(n, generator=torch.Generator().manual_seed(1))
    ref = ko.conv_factor_G(g.double(), p.double()) * (n * n)
    gd = dev(g)
    if channels_last:
        gd = gd.contiguous(memory_format=torch.channels_last)
    out = torch.empty((c, c), device='cuda')
    nat.factor_im2col(gd, (1, 1), (1, 1), (0, 0), (1, 1), False, dev(p), n * n / (n * h * w), 0.0, out,
                      nat.IMPL_SIMT)
    assert rel(out, ref) < FACTOR_TOL


def test_factor_conv_bf16_channels_last(nat):
    n, c, h, w = 4, 32, 14, 14
    x = cases.make_normal((n, c, h, w), 5).bfloat16()
    ref = ko.conv_factor_A(x.double(), (3, 3), (1, 1), (1, 1), (1, 1), False)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    out = torch.empty(tuple(ref.shape), device='cuda')
    nat.factor_im2col(xd, (3, 3), (1, 1), (1, 1), (1, 1), False, None, 1.0 / n, 0.0, out, nat.IMPL_SIMT)
    assert rel(out, ref) < FACTOR_TOL


# tensor-core (tcgen05) path: channels-contiguous inputs, bf16 single pass and fp32 as 3xTF32
TC_CONVS = [
    # n, c, h, w, k, stride, pad, dil, bias
    (2, 8, 6, 6, (3, 3), (1, 1), (1, 1), (1, 1), False),
    (4, 64, 14, 14, (3, 3), (1, 1), (1, 1), (1, 1), True),
    (4, 64, 14, 14, (3, 3), (2, 2), (1, 1), (1, 1), False),
    (3, 16, 9, 11, (5, 3), (1, 2), (2, 0), (1, 2), True),
    (4, 256, 14, 14, (1, 1), (1, 1), (0, 0), (1, 1), False),
    (16, 32, 32, 32, (3, 3), (1, 1), (1, 1), (1, 1), True),      # 16384 rows: several splits
    (2, 136, 6, 6, (3, 3), (1, 1), (1, 1), (1, 1), False),       # d = 1224: 10 x 10 tiles, ragged edge
    (32, 128, 16, 16, (3, 3), (1, 1), (1, 1), (1, 1), False),    # d = 1152 from 8192 rows: several splits, row-wise finish
]


@pytest.mark.parametrize('cfg', TC_CONVS)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32, torch.float16])
def test_factor_tcgen05_conv_matches_oracle(nat, cfg, dtype):
    n, c, h, w, k, s, p, d, bias = cfg
    x = cases.make_normal((n, c, h, w), 91 + c + h).to(dtype)
    ref = ko.conv_factor_A(x.double(), k, s, p, d, bias)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    out = torch.full(tuple(ref.shape), float('nan'), device='cuda')
    nat.factor_im2col(xd, k, s, p, d, bias, None, 1.0 / n, 0.0, out, nat.IMPL_TCGEN05)
    assert rel(out, ref) < FACTOR_TOL
    assert torch.equal(out, out.t())
    # accumulate on top (beta = 1) and compare with the fp32 SIMT kernel doing the same
    simt = torch.empty_like(out)
    nat.factor_im2col(xd, k, s, p, d, bias, None, 1.0 / n, 0.0, simt, nat.IMPL_SIMT)
    nat.factor_im2col(xd, k, s, p, d, bias, None, 1.0 / n, 1.0, out, nat.IMPL_TCGEN05)
    assert rel(out, 2 * simt) < FACTOR_TOL


@pytest.mark.parametrize('rows,cols,bias,dtype', [(128, 784, True, torch.float32), (128, 1000, True, torch.float32),
                                                  (4096, 256, True, torch.bfloat16), (1000, 2048, True, torch.bfloat16),
                                                  (100352, 64, False, torch.bfloat16), (32768, 512, False, torch.float32),
                                                  (77, 8, False, torch.float32)])
def test_factor_tcgen05_rows_matches_oracle(nat, rows, cols, bias, dtype):
    x = cases.make_normal((rows, cols), 7 + rows).clamp_min(-0.5).to(dtype)     # positive mean: long sums
    d = cols + int(bias)
    out = torch.full((d, d), float('nan'), device='cuda')
    nat.factor_rows(dev(x), bias, None, 1.0 / rows, 0.0, out, nat.IMPL_TCGEN05)
    assert rel(out, ko.linear_factor_A(x.double(), bias)) < FACTOR_TOL
    again = torch.empty_like(out)
    nat.factor_rows(dev(x), bias, None, 1.0 / rows, 0.0, again, nat.IMPL_TCGEN05)
    assert torch.equal(out, again)                                                  # deterministic


# TMA-fed tensor-core path: 16-bit channels-contiguous inputs with a multiple of 64 channels
TMA_CONVS = [
    # n, c, h, w, k, stride, pad, dil
    (2, 64, 6, 6, (1, 1), (1, 1), (0, 0), (1, 1)),
    (2, 64, 6, 6, (3, 3), (1, 1), (1, 1), (1, 1)),
    (3, 128, 9, 7, (3, 3), (1, 1), (1, 1), (1, 1)),
    (4, 64, 14, 14, (3, 3), (2, 2), (1, 1), (1, 1)),
    (4, 64, 14, 14, (1, 1), (2, 2), (0, 0), (1, 1)),
    (2, 192, 20, 20, (3, 3), (1, 1), (1, 1), (1, 1)),       # d = 1728: ragged last tile
    (2, 64, 12, 12, (5, 3), (1, 1), (2, 1), (1, 2)),        # rectangular kernel, dilation
    (5, 64, 7, 7, (3, 3), (1, 1), (1, 1), (1, 1)),          # whole images per box, ragged image count
    (6, 64, 30, 30, (3, 3), (1, 1), (1, 1), (1, 1)),        # 5400 rows: several splits
    (3, 64, 14, 14, (3, 3), (1, 1), (1, 1), (1, 1)),        # 196 pixels per image: box rows must divide 14
    (2, 64, 13, 13, (3, 3), (1, 1), (1, 1), (1, 1)),        # prime height: one output row per box
]


@pytest.mark.parametrize('cfg', TMA_CONVS)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_factor_tma_conv_matches_oracle(nat, cfg, dtype):
    n, c, h, w, k, s, p, d = cfg
    x = cases.make_normal((n, c, h, w), 191 + c + h).to(dtype)
    ref = ko.conv_factor_A(x.double(), k, s, p, d, False)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    out = torch.full(tuple(ref.shape), float('nan'), device='cuda')
    nat.factor_im2col(xd, k, s, p, d, False, None, 1.0 / n, 0.0, out, nat.IMPL_TMA)
    assert rel(out, ref) < FACTOR_TOL
    assert torch.equal(out, out.t())
    again = torch.empty_like(out)
    nat.factor_im2col(xd, k, s, p, d, False, None, 1.0 / n, 0.0, again, nat.IMPL_TMA)
    assert torch.equal(out, again)


@pytest.mark.parametrize('cfg', TMA_CONVS)
@pytest.mark.parametrize('pair_min_d', [64, 0])
def test_factor_tma_pair_and_single_kernels(nat, cfg, pair_min_d):
    """The CTA-pair kernel (tcgen05.mma.cta_group::2, forced for every width) and the single-CTA
    kernel (pair kernel switched off) both match the oracle, bitwise symmetric and reproducible."""
    n, c, h, w, k, s, p, d = cfg
    x = cases.make_normal((n, c, h, w), 291 + c + h).bfloat16()
    ref = ko.conv_factor_A(x.double(), k, s, p, d, False)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    nat.configure('tma_pair_min_d', pair_min_d)
    try:
        out = torch.full(tuple(ref.shape), float('nan'), device='cuda')
        nat.factor_im2col(xd, k, s, p, d, False, None, 1.0 / n, 0.0, out, nat.IMPL_TMA)
        again = torch.full_like(out, float('nan'))
        nat.factor_im2col(xd, k, s, p, d, False, None, 1.0 / n, 0.0, again, nat.IMPL_TMA)
    finally:
        nat.configure('tma_pair_min_d', 512)
    assert rel(out, ref) < FACTOR_TOL
    assert torch.equal(out, out.t())
    assert torch.equal(out, again)


def test_factor_tma_pair_accumulates_with_beta(nat):
    """alpha / beta epilogue through both finishing kernels (d = 1152 is wide enough for the
    row-wise one when there are few splits)."""
    n, c, h, w = 4, 128, 10, 10
    x = cases.make_normal((n, c, h, w), 77).bfloat16()
    ref = ko.conv_factor_A(x.double(), (3, 3), (1, 1), (1, 1), (1, 1), False)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    base = cases.make_normal(tuple(ref.shape), 78)
    out = dev(base).clone()
    nat.factor_im2col(xd, (3, 3), (1, 1), (1, 1), (1, 1), False, None, 0.5 / n, 0.25, out, nat.IMPL_TMA)
    assert rel(out, 0.5 * ref + 0.25 * base.double()) < FACTOR_TOL


@pytest.mark.parametrize('cfg', [
    (2, 32, 6, 6, (1, 1), (1, 1), (0, 0), (1, 1)),
    (2, 64, 6, 6, (3, 3), (1, 1), (1, 1), (1, 1)),
    (3, 128, 9, 7, (3, 3), (1, 1), (1, 1), (1, 1)),
    (4, 64, 14, 14, (3, 3), (2, 2), (1, 1), (1, 1)),
    (2, 96, 20, 20, (3, 3), (1, 1), (1, 1), (1, 1)),
    (2, 64, 12, 12, (5, 3), (1, 1), (2, 1), (1, 2)),
    (6, 64, 30, 30, (3, 3), (1, 1), (1, 1), (1, 1)),
])
def test_factor_tma_fp32_matches_oracle(nat, cfg):
    """Opt-in TMA-fed 3xTF32 kernel for fp32 channels-contiguous inputs (MN-major tf32 operands in
    the 32-byte-chunk swizzle, split into hi / lo in shared memory)."""
    n, c, h, w, k, s, p, d = cfg
    x = cases.make_normal((n, c, h, w), 391 + c + h)
    ref = ko.conv_factor_A(x.double(), k, s, p, d, False)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    nat.configure('tma_f32', 1)
    try:
        out = torch.full(tuple(ref.shape), float('nan'), device='cuda')
        nat.factor_im2col(xd, k, s, p, d, False, None, 1.0 / n, 0.0, out, nat.IMPL_TMA)
        again = torch.full_like(out, float('nan'))
        nat.factor_im2col(xd, k, s, p, d, False, None, 1.0 / n, 0.0, again, nat.IMPL_TMA)
    finally:
        nat.configure('tma_f32', 0)
    assert rel(out, ref) < FACTOR_TOL
    assert torch.equal(out, out.t())
    assert torch.equal(out, again)


@pytest.mark.parametrize('engine_tma', [0, 1])
def test_precondition_kernel_variants_agree(nat, engine_tma):
    """k-contiguous tile tasks fed by TMA (tensor maps per task) or by cp.async give the oracle's
    preconditioned gradient."""
    da, dg = 1152, 256
    Ai, Gi = spd_pair(da, dg, 160)
    gw = cases.make_normal((dg, da), 161) * 0.1
    rw, _ = ko.kron_precondition(Ai.double(), Gi.double(), gw.double(), None)
    nat.configure('engine_tma', engine_tma)
    try:
        dgw = dev(gw)
        tmp = torch.empty(dg * da, device='cuda')
        plan = nat.precond_plan([da], [dg], [dev(Ai)], [dev(Gi)], [dgw], [None], [tmp], torch.device('cuda'))
        kinds = [k for k, _, _ in plan.phases()]
        nat.precond_plan_run(plan)
        torch.cuda.synchronize()
    finally:
        nat.configure('engine_tma', 1)
    assert 4 in kinds            # both products run as k-contiguous phases
    assert rel(dgw, rw) < INV_TOL


@pytest.mark.parametrize('rows,cols', [(300, 64), (1000, 2048), (100352, 64), (77, 128)])
def test_factor_tma_rows_matches_oracle(nat, rows, cols):
    x = cases.make_normal((rows, cols), 5 + rows).clamp_min(-0.5).bfloat16()
    out = torch.full((cols, cols), float('nan'), device='cuda')
    nat.factor_rows(dev(x), False, None, 1.0 / rows, 0.0, out, nat.IMPL_TMA)
    assert rel(out, ko.linear_factor_A(x.double(), False)) < FACTOR_TOL
    # not eligible: ones column, fp32, channel count not a multiple of 64
    with pytest.raises(RuntimeError):
        nat.factor_rows(dev(x), True, None, 1.0 / rows, 0.0, torch.empty((cols + 1, cols + 1), device='cuda'),
                        nat.IMPL_TMA)
    with pytest.raises(RuntimeError):
        nat.factor_rows(dev(x).float(), False, None, 1.0 / rows, 0.0, out, nat.IMPL_TMA)


def test_factor_tcgen05_weighted_fp32_and_dispatch(nat):
    rows, cols = 300, 96
    g = cases.make_normal((rows, cols), 3)
    p = torch.rand(rows, generator=torch.Generator().manual_seed(5))
    ref = ko.linear_factor_G(g.double(), p.double())
    out = torch.empty((cols, cols), device='cuda')
    nat.factor_rows(dev(g), False, dev(p), 1.0 / rows, 0.0, out, nat.IMPL_TCGEN05)
    assert rel(out, ref) < FACTOR_TOL
    # 16-bit inputs with per-sample weights are not eligible (weights would be rounded into the
    # operands): asking for the tensor-core kernel explicitly is an error, AUTO falls back
    with pytest.raises(RuntimeError):
        nat.factor_rows(dev(g).bfloat16(), False, dev(p), 1.0 / rows, 0.0, out, nat.IMPL_TCGEN05)
    nat.factor_rows(dev(g).bfloat16(), False, dev(p), 1.0 / rows, 0.0, out, nat.IMPL_AUTO)
    assert rel(out, ko.linear_factor_G(g.bfloat16().double(), p.double())) < FACTOR_TOL
    # NCHW input is not channels-contiguous: explicit request fails, AUTO uses the SIMT kernel
    x = dev(cases.make_normal((2, 8, 6, 6), 4))
    o = torch.empty((72, 72), device='cuda')
    with pytest.raises(RuntimeError):
        nat.factor_im2col(x, (3, 3), (1, 1), (1, 1), (1, 1), False, None, 0.5, 0.0, o, nat.IMPL_TCGEN05)
    nat.factor_im2col(x, (3, 3), (1, 1), (1, 1), (1, 1), False, None, 0.5, 0.0, o, nat.IMPL_AUTO)
    assert rel(o, ko.conv_factor_A(x.cpu().double(), (3, 3), (1, 1), (1, 1), (1, 1), False)) < FACTOR_TOL


def test_factor_is_deterministic(nat):
    x = dev(cases.make_normal((8, 16, 32, 32), 3))
    a = torch.empty((144, 144), device='cuda')
    b = torch.empty((144, 144), device='cuda')
    for o in (a, b):
        nat.factor_im2col(x, (3, 3), (1, 1), (1, 1), (1, 1), False, None, 1.0 / 8, 0.0, o, nat.IMPL_SIMT)
    assert torch.equal(a, b)


def test_factor_rejects_bad_arguments(nat):
    x = dev(cases.make_normal((4, 4), 1))
    out = torch.empty((4, 4), device='cuda')
    with pytest.raises(RuntimeError):
        nat._check(nat.lib().sso_factor_syrk(x.data_ptr(), 0, 4, 4, 4, 1, 0, None, 1.0, 0.0,
                                             out.data_ptr(), 2, None, 0, 1, None))   # ldo < d
    with pytest.raises(RuntimeError):
        nat._check(nat.lib().sso_factor_syrk(None, 0, 4, 4, 4, 1, 0, None, 1.0, 0.0,
                                             out.data_ptr(), 4, None, 0, 1, None))


# ------------------------------------------------------------------------------------ batch norm
@pytest.mark.parametrize('shape', [(6, 5, 4, 4), (4, 70, 7, 7), (8, 33), (3, 64, 1, 1), (4, 64, 56, 56),
                                   (2, 2048, 7, 7), (3, 24, 20, 20)])
@pytest.mark.parametrize('channels_last', [False, True])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_bn_diag_matches_oracle(nat, shape, channels_last, dtype):
    if channels_last and len(shape) != 4:
        pytest.skip('2-D input has no channels_last form')
    y = cases.make_normal(shape, 31).to(dtype)
    g = cases.make_normal(shape, 32).to(dtype)
    c = shape[1]
    gamma = 1.0 + 0.1 * cases.make_normal((c,), 33)
    beta = 0.1 * cases.make_normal((c,), 34)
    p = torch.rand(shape[0], generator=torch.Generator().manual_seed(2))
    xhat = ko.bn_restore_input(y.double(), gamma.double(), beta.double())
    ref = ko.bn_diag(xhat, g.double(), p.double(), True)
    n = shape[0]
    yd, gd = dev(y), dev(g)
    if channels_last:
        yd = yd.contiguous(memory_format=torch.channels_last)
        gd = gd.contiguous(memory_format=torch.channels_last)
    sx = torch.full((n * c * 64,), float('nan'), device='cuda')
    sg = torch.full((n * c * 64,), float('nan'), device='cuda')
    kx = nat.bn_plane_sums(yd, True, dev(gamma), dev(beta), sx)
    kg = nat.bn_plane_sums(gd, False, None, None, sg)
    w_out = torch.empty(c, device='cuda')
    b_out = torch.empty(c, device='cuda')
    nat.bn_diag_finish(sx, sg, dev(p), n, c, kx, kg, 1.0, 0.0, w_out, b_out)
    assert rel(w_out, ref[0]) < 2e-5
    assert rel(b_out, ref[1]) < 2e-5


# ------------------------------------------------------------------------------------ streaming
def test_ema_axpby_diag(nat):
    n = 100003
    data = dev(cases.make_normal((n,), 1))
    ema = dev(cases.make_normal((n,), 2)).abs_()
    ref = ko.ema_update(data.cpu(), ema.cpu(), 0.95)
    nat.ema_update(data, ema, 0.95, False)
    assert rel(ema, ref) < 1e-6
    first = torch.empty_like(ema)
    nat.ema_update(data, first, 0.95, True)
    assert torch.equal(first, data)
    # unaligned views
    a, b = data[1:5001], ema[3:5003].clone()
    exp = 2.0 * a + 0.5 * b
    nat.axpby(a, b, 2.0, 0.5)
    assert rel(b, exp) < 1e-6
    e = dev(cases.make_normal((999,), 4)).abs_()
    inv = torch.empty_like(e)
    grad = dev(cases.make_normal((999,), 5))
    g0 = grad.clone()
    nat.diag_inv_precondition(e, inv, grad, 1e-3, False, True)
    ref_inv = ko.diag_inverse(e.cpu().double(), 1e-3)
    assert rel(inv, ref_inv) < 1e-6
    assert rel(grad, g0.cpu().double() * ref_inv) < 1e-6


@pytest.mark.parametrize('rows', [0, 32, 7])
def test_tri_pack_unpack_roundtrip(nat, rows):
    """rows: rows per record of the unpack table (0: long records, element-wise path; <= 32: bands whose
    part below the diagonal is transposed through shared memory, as the communicator unpacks)."""
    mats, packed_ref, offs, off = [], [], [], 0
    for i, n in enumerate([1, 7, 64, 129, 300, 1000]):
        m = cases.make_normal((n, n), 40 + i)
        m = m + m.t()
        mats.append(dev(m))
        packed_ref.append(ko.tri_pack(m))
        offs.append(off)
        off += n * (n + 1) // 2
    buf = torch.full((off,), float('nan'), device='cuda')
    table = nat.tri_records(mats, buf, offs)
    nat.tri_pack(table, 0.5)
    assert torch.equal(buf.cpu(), 0.5 * torch.cat(packed_ref))
    outs = [torch.full_like(m, float('nan')) for m in mats]
    nat.tri_unpack(nat.tri_records(outs, buf, offs, rows), 2.0, True)
    for o, m in zip(outs, mats):
        assert torch.equal(o, m)
    up = [torch.full_like(m, float('nan')) for m in mats]
    nat.tri_unpack(nat.tri_records(up, buf, offs, rows), 2.0, False)
    for o, m in zip(up, mats):
        assert torch.equal(o, torch.triu(m))


# ------------------------------------------------------------------------------------ engine
def spd_pair(da, dg, seed):
    xa = cases.make_normal((max(4 * da, 64), da), seed)
    xg = cases.make_normal((max(4 * dg, 64), dg), seed + 1) * 0.1
    return (xa.t() @ xa) / xa.shape[0], (xg.t() @ xg) / xg.shape[0]


@pytest.mark.parametrize('dims', [[(10, 28)], [(64, 65), (147, 10)], [(513, 130), (785, 1000)],
                                  [(1601, 128)]])
def test_kron_inverse_and_std_match_oracle(nat, dims):
    damping = 1e-3
    src, dst, work, std, sizes, partner, role = [], [], [], [], [], [], []
    refs = []
    for i, (da, dg) in enumerate(dims):
        A, G = spd_pair(da, dg, 50 + 2 * i)
        refs.append((A, G))
        for which, m in enumerate((A, G)):
            sizes.append(m.shape[0])
            src.append(dev(m))
            dst.append(torch.full_like(src[-1], float('nan')))
            work.append(torch.full_like(src[-1], float('nan')))
            std.append(torch.full_like(src[-1], float('nan')))
            partner.append(2 * i + 1 - which)
            role.append(which)
    plan = nat.kron_plan(sizes, src, dst, work, std, partner, role, torch.device('cuda'))
    damp = torch.full((len(sizes),), math.sqrt(damping), device='cuda')
    info = torch.zeros(2 * len(sizes), dtype=torch.int32, device='cuda')
    nat.kron_plan_run(plan, damp, info, True, True)
    assert int(info.abs().sum()) == 0
    for i, (A, G) in enumerate(refs):
        Ai, Gi = ko.kron_damped_inverse(A.double(), G.double(), damping)
        for got, ref in ((dst[2 * i], Ai), (dst[2 * i + 1], Gi)):
            assert rel(got, ref) < INV_TOL
            assert torch.equal(got, got.t())
        for got, ref in ((std[2 * i], Ai), (std[2 * i + 1], Gi)):
            assert rel(got, ko.cholesky_upper(ref)) < INV_TOL
            assert torch.equal(got, torch.triu(got))
    # second run on the same buffers gives the same bits (no atomics, fixed order)
    first = [d.clone() for d in dst]
    nat.kron_plan_run(plan, damp, info, True, False)
    for a, b in zip(first, dst):
        assert torch.equal(a, b)


def test_kron_inverse_reports_non_spd(nat):
    d = 70
    A, _ = spd_pair(d, 8, 3)
    A[66, 66] = -5.0
    src = dev(A)
    dst, work = torch.empty_like(src), torch.empty_like(src)
    plan = nat.kron_plan([d], [src], [dst], [work], None, [-1], [0], torch.device('cuda'))
    info = torch.zeros(2, dtype=torch.int32, device='cuda')
    nat.kron_plan_run(plan, torch.zeros(1, device='cuda'), info, True, False)
    assert int(info[0]) == 67          # 1-based index of the failing pivot
    assert int(info[1]) == 0


@pytest.mark.parametrize('panel', [1, 0])
def test_kron_inverse_block_sizes_and_pivot_positions(nat, panel):
    """One launch factorises a whole 128-column panel's diagonal block in panels of 16 columns (or, with
    "chol_panel" 0, two 64-wide halves): sizes on both sides of every internal boundary, all in one plan,
    against the fp64 oracle; then a non-positive pivot at several positions, reported LAPACK style."""
    nat.configure('chol_panel', panel)
    try:
        dims = [1, 2, 15, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 143, 144, 145, 255, 257, 300]
        mats = [spd_pair(d, 8, 700 + d)[0] + 1e-2 * torch.eye(d) for d in dims]
        src = [dev(m) for m in mats]
        dst = [torch.full_like(m, float('nan')) for m in src]
        work = [torch.full_like(m, float('nan')) for m in src]
        std = [torch.full_like(m, float('nan')) for m in src]
        plan = nat.kron_plan(dims, src, dst, work, std, [-1] * len(dims), [0] * len(dims), torch.device('cuda'))
        info = torch.zeros(2 * len(dims), dtype=torch.int32, device='cuda')
        nat.kron_plan_run(plan, torch.zeros(len(dims), device='cuda'), info, True, True)
        assert int(info.abs().sum()) == 0
        for d, m, got, u in zip(dims, mats, dst, std):
            ref = ko.spd_inverse(m.double())
            assert rel(got, ref) < INV_TOL, d
            assert torch.equal(got, got.t()), d
            assert rel(u, ko.cholesky_upper(ref)) < INV_TOL, d
        for d, bad in ((40, 0), (40, 15), (40, 16), (130, 70), (130, 127), (130, 128), (300, 299)):
            A = spd_pair(d, 8, 900 + d)[0] + 1e-2 * torch.eye(d)
            A[bad, bad] = -1.0
            s1 = dev(A)
            d1, w1 = torch.empty_like(s1), torch.empty_like(s1)
            plan = nat.kron_plan([d], [s1], [d1], [w1], None, [-1], [0], torch.device('cuda'))
            info = torch.zeros(2, dtype=torch.int32, device='cuda')
            nat.kron_plan_run(plan, torch.zeros(1, device='cuda'), info, True, False)
            assert int(info[0]) == bad + 1, (d, bad, int(info[0]))
    finally:
        nat.configure('chol_panel', 1)


def test_utils_inv_and_cholesky(nat):
    import torchsso
    A, _ = spd_pair(200, 8, 9)
    A = A + 0.1 * torch.eye(200)
    got = torchsso.utils.inv(dev(A))
    assert rel(got, ko.spd_inverse(A.double())) < INV_TOL
    U = torchsso.utils.cholesky(dev(A))
    assert rel(U, ko.cholesky_upper(A.double())) < INV_TOL
    with pytest.raises(RuntimeError):
        torchsso.utils.inv(A)          # CPU tensor: no fallback


@pytest.mark.parametrize('da,dg,bias', [(21, 16, True), (785, 1000, True), (1001, 10, True),
                                        (576, 64, False), (1153, 256, True)])
def test_precondition_matches_oracle(nat, da, dg, bias):
    Ai, Gi = spd_pair(da, dg, 60)
    wc = da - 1 if bias else da
    gw = cases.make_normal((dg, wc), 61) * 0.1
    gb = cases.make_normal((dg,), 62) * 0.1 if bias else None
    rw, rb = ko.kron_precondition(Ai.double(), Gi.double(), gw.double(), None if gb is None else gb.double())
    dgw, dgb = dev(gw), None if gb is None else dev(gb)
    tmp = torch.empty(dg * da, device='cuda')
    plan = nat.precond_plan([da], [dg], [dev(Ai)], [dev(Gi)], [dgw], [dgb], [tmp], torch.device('cuda'))
    nat.precond_plan_run(plan)
    assert rel(dgw, rw) < INV_TOL
    if bias:
        assert rel(dgb, rb) < INV_TOL


@pytest.mark.parametrize('da,dg,bias', [(28, 6, True), (577, 64, True), (300, 129, False)])
def test_sample_matches_oracle(nat, da, dg, bias):
    UA = torch.triu(cases.make_normal((da, da), 70))
    UG = torch.triu(cases.make_normal((dg, dg), 71))
    wc = da - 1 if bias else da
    mw = cases.make_normal((dg, wc), 72)
    mb = cases.make_normal((dg,), 73) if bias else None
    E = cases.make_normal((dg, da), 74)
    s = 0.0123
    rw, rb = ko.kron_sample(mw.double(), None if mb is None else mb.double(), UA.double(), UG.double(),
                            E.double(), s)
    w, b = dev(mw), None if mb is None else dev(mb)
    tmp = torch.empty(dg * da, device='cuda')
    plan = nat.sample_plan([da], [dg], [dev(UA)], [dev(UG)], [dev(E)], [w], [b], [tmp], torch.device('cuda'))
    nat.sample_plan_run(plan, s)
    assert rel(w, rw) < 1e-5
    if bias:
        assert rel(b, rb) < 1e-5


def test_optimizer_tail_matches_torch(nat):
    """sso_optimizer_tail against the chain of multi-tensor torch ops it replaces
    (torchsso/optim/secondorder.py:225-283): l2 / weight decay, momentum, gradient moving average,
    bias-correction scale, update."""
    torch.manual_seed(3)
    shapes = [(70000,), (33,), (128, 65)]
    items, ref = [], []
    for i, shp in enumerate(shapes):
        p, g = torch.randn(shp, device='cuda'), torch.randn(shp, device='cuda')
        m, e = torch.randn(shp, device='cuda'), torch.randn(shp, device='cuda')
        use_m, use_e = i != 1, i != 0
        add, mom, ema, scale, lr = 1e-2 * (i + 1), 0.9, 0.3, 1.5, 0.05 if i != 2 else 0.0
        rp, rg, rm, re = p.double(), g.double(), m.double(), e.double()
        rg = rg + add * rp
        if use_m:
            rm = mom * rm + rg
            rg = rm
        if use_e:
            re = (1 - ema) * re + ema * rg
            rg = re
        rg = rg * scale
        rp = rp - lr * rg
        ref.append((rp, rg, rm, re))
        items.append((p, g, m if use_m else None, e if use_e else None, add, mom, ema, scale, lr))
    table = nat.tail_records([(p.view(-1), g.view(-1), None if m is None else m.view(-1),
                               None if e is None else e.view(-1), a, mo, em, sc, lr)
                              for p, g, m, e, a, mo, em, sc, lr in items], torch.device('cuda'))
    untouched = [(None if it[2] is None else it[2].clone(), None if it[3] is None else it[3].clone()) for it in items]
    nat.optimizer_tail(table)
    torch.cuda.synchronize()
    for (p, g, m, e, *_), (rp, rg, rm, re) in zip(items, ref):
        assert rel(p, rp) < 1e-6 and rel(g, rg) < 1e-6
        if m is not None:
            assert rel(m, rm) < 1e-6
        if e is not None:
            assert rel(e, re) < 1e-6


# ------------------------------------------------------------------ diagonal Linear / Conv2d
@pytest.mark.parametrize('n,fi,fo,weighted', [(12, 37, 10, False), (128, 200, 130, True), (5, 64, 64, False)])
def test_diag_sq_linear_matches_oracle(nat, n, fi, fo, weighted):
    x = cases.make_normal((n, fi), 801)
    g = cases.make_normal((n, fo), 802) * 0.1
    prob = cases.make_uniform((n,), 803).float() if weighted else None
    rw, rb = ko.diag_linear(x.double(), g.double(), None if prob is None else prob.double())
    out_w = torch.full((fo, fi), float('nan'), device='cuda')
    out_b = torch.full((fo,), float('nan'), device='cuda')
    nat.diag_sq(dev(x), dev(g), None, None, None, None, None if prob is None else dev(prob), 1.0 / n, 0.0, out_w, out_b)
    assert rel(out_w, rw) < FACTOR_TOL and rel(out_b, rb) < FACTOR_TOL
    # accumulate (beta = 1) doubles the result
    nat.diag_sq(dev(x), dev(g), None, None, None, None, None if prob is None else dev(prob), 1.0 / n, 1.0, out_w, out_b)
    assert rel(out_w, 2 * rw) < FACTOR_TOL and rel(out_b, 2 * rb) < FACTOR_TOL


@pytest.mark.parametrize('cfg', [
    (4, 3, 8, 8, 6, (3, 3), (1, 1), (1, 1), (1, 1)),
    (3, 16, 9, 7, 70, (3, 3), (2, 2), (1, 1), (1, 1)),
    (2, 8, 12, 12, 5, (5, 3), (1, 1), (2, 1), (1, 2)),
    (6, 32, 6, 6, 33, (1, 1), (1, 1), (0, 0), (1, 1)),
])
@pytest.mark.parametrize('channels_last,dtype', [(False, torch.float32), (True, torch.float32), (True, torch.bfloat16)])
def test_diag_sq_conv_matches_oracle(nat, cfg, channels_last, dtype):
    n, c, h, w, oc, k, s, p, d = cfg
    x = cases.make_normal((n, c, h, w), 811 + c).to(dtype)
    ho = (h + 2 * p[0] - d[0] * (k[0] - 1) - 1) // s[0] + 1
    wo = (w + 2 * p[1] - d[1] * (k[1] - 1) - 1) // s[1] + 1
    g = (cases.make_normal((n, oc, ho, wo), 812 + oc) * 0.1).to(dtype)
    prob = cases.make_uniform((n,), 813).float()
    rw, rb = ko.diag_conv(x.double(), g.double(), k, s, p, d, prob.double())
    xd, gd = dev(x), dev(g)
    if channels_last:
        xd, gd = xd.contiguous(memory_format=torch.channels_last), gd.contiguous(memory_format=torch.channels_last)
    out_w = torch.full((oc, c, k[0], k[1]), float('nan'), device='cuda')
    out_b = torch.full((oc,), float('nan'), device='cuda')
    nat.diag_sq(xd, gd, k, s, p, d, dev(prob), 1.0 / n, 0.0, out_w, out_b)
    assert rel(out_w, rw) < FACTOR_TOL and rel(out_b, rb) < FACTOR_TOL


# ------------------------------------------------------------------------------------ batched factors
def _desc_array(nat, items):
    arr = (nat.FactorDesc * len(items))()
    for d, (x, geo, alpha, beta, out) in zip(arr, items):
        n, c, h, w = x.shape
        (kh, kw), (sh, sw), (ph, pw), (dh, dw) = geo
        d.x, d.dtype, d.append_ones = x.data_ptr(), nat._dtype_code(x), 0
        d.n, d.c, d.h, d.w = n, c, h, w
        d.sn, d.sc, d.sh, d.sw = x.stride()
        d.kh, d.kw, d.stride_h, d.stride_w, d.pad_h, d.pad_w, d.dil_h, d.dil_w = kh, kw, sh, sw, ph, pw, dh, dw
        d.sample_weight, d.alpha, d.beta, d.out, d.ldo = None, alpha, beta, out.data_ptr(), out.stride(0)
    return arr


def test_factor_batch_matches_oracle(nat):
    """Several factor problems of different geometry in ONE call (persistent CTA-pair kernel over all
    of them + one finishing launch): 3x3 / 1x1 / strided windows, channel counts 64 ... 384, a single
    image plane smaller than a stage, accumulation onto existing contents, and one fp32 problem that
    the batched kernel does not take (it runs behind the batch through the single-problem path)."""
    cl = torch.channels_last
    specs = [  # (n, c, h, w), geometry, dtype, alpha, beta
        ((6, 64, 12, 12), ((3, 3), (1, 1), (1, 1), (1, 1)), torch.bfloat16, 1.0 / 6, 0.0),
        ((5, 128, 14, 14), ((1, 1), (1, 1), (0, 0), (1, 1)), torch.bfloat16, 0.5, 1.0),
        ((4, 256, 7, 7), ((3, 3), (1, 1), (1, 1), (1, 1)), torch.float16, 0.25, 0.0),
        ((3, 64, 16, 16), ((3, 3), (2, 2), (1, 1), (1, 1)), torch.bfloat16, 1.0, 0.0),
        ((9, 384, 5, 5), ((1, 1), (1, 1), (0, 0), (1, 1)), torch.bfloat16, 2.0, 0.5),
        ((40, 64, 28, 28), ((1, 1), (1, 1), (0, 0), (1, 1)), torch.bfloat16, 1.0 / 40, 0.0),
        ((2, 8, 9, 9), ((3, 3), (1, 1), (1, 1), (1, 1)), torch.float32, 1.0, 0.0),
    ]
    items, news = [], []
    for i, (shape, geo, dt, alpha, beta) in enumerate(specs):
        x = cases.make_normal(shape, 300 + i).to(dt).cuda().contiguous(memory_format=cl)
        d = shape[1] * geo[0][0] * geo[0][1]
        init = cases.make_normal((d, d), 400 + i)
        out = (init + init.t()).cuda()
        items.append((x, geo, alpha, beta, out))
        news.append(alpha * ko.conv_factor_A(x.double().cpu(), *geo, False) * shape[0])    # alpha * sum_r u u^T
    arr = _desc_array(nat, items)
    L = nat.lib()
    nbytes = L.sso_factor_batch_workspace_bytes(len(items), arr)
    assert nbytes > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    for rep in range(2):     # twice on the same scratch: stale partial tiles must not leak
        before = [it[4].double().cpu() for it in items]
        nat._check(L.sso_factor_batch(len(items), arr, ws.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        for (x, geo, alpha, beta, out), new, old in zip(items, news, before):
            assert rel(out, new + beta * old) < 1e-5, (rep, tuple(x.shape), geo)
            assert torch.equal(out, out.t())
    with pytest.raises(RuntimeError, match='write the same matrix'):
        bad = _desc_array(nat, [items[0], items[0]])
        nat._check(L.sso_factor_batch(2, bad, ws.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream))
