"""Failure detection on the device without a fault: every wait inside the tensor-core kernels is
bounded; when one runs out the kernel records a code, winds down normally (barriers released, tensor
memory freed) and its result is NaN instead of a stale or partial matrix.

The waits are made to run out by two library controls, not by breaking anything: the limit is
lowered to ~1 ms (`wait_kcycles`) and the TMA producer warps are told to issue no loads
(`inject_stall`), so the consumers wait for data that never arrives.  Afterwards the same calls
must work again in the same process."""
import math

import pytest
import torch

import cases
from oracle import kfac_oracle as ko

pytestmark = pytest.mark.gpu


@pytest.fixture
def nat():
    from torchsso import _native
    _native.lib()
    yield _native
    _native.configure('inject_stall', 0)
    _native.configure('wait_kcycles', 0)


def _rel(a, b):
    a, b = a.detach().double().cpu(), b.double()
    return ((a - b).norm() / b.norm()).item()


@pytest.mark.parametrize('channels', [64, 512])      # single-CTA kernel / CTA-pair kernel
def test_factor_kernel_wait_runs_out(nat, channels):
    x = cases.make_normal((4, channels, 6, 6), 5).cuda().to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    geo = ((1, 1), (1, 1), (0, 0), (1, 1))
    out = torch.zeros((channels, channels), device='cuda')
    nat.configure('wait_kcycles', 2000)       # ~2e6 clocks: about a millisecond
    nat.configure('inject_stall', 1)
    nat.factor_im2col(x, *geo, False, None, 1.0 / 4, 0.0, out, impl=nat.IMPL_TMA)
    torch.cuda.synchronize()                  # the kernel returned by itself
    ws = nat._workspaces[('cuda', x.device.index)]
    assert int(ws[:4].view(torch.int32).item()) != 0, 'the status word must carry the code of the wait that gave up'
    assert bool(torch.isnan(out).all()), 'the result of a kernel whose wait gave up must be NaN'
    nat.configure('inject_stall', 0)
    nat.configure('wait_kcycles', 0)
    nat.factor_im2col(x, *geo, False, None, 1.0 / 4, 0.0, out, impl=nat.IMPL_TMA)
    ref = ko.conv_factor_A(x.double().cpu(), *geo, False)
    assert _rel(out, ref) < 1e-5
    assert int(ws[:4].view(torch.int32).item()) == 0


def test_batched_factor_kernel_wait_runs_out(nat):
    """The persistent kernel of sso_factor_batch: with its producers stalled, every role's wait runs out,
    the kernel returns, and the finishing kernel writes NaN for every problem of the batch."""
    xs = [cases.make_normal((4, c, 6, 6), 5 + c).cuda().to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
          for c in (64, 320)]
    outs = [torch.zeros((x.shape[1], x.shape[1]), device='cuda') for x in xs]
    arr = (nat.FactorDesc * 2)()
    for d, x, out in zip(arr, xs, outs):
        d.x, d.dtype, d.append_ones = x.data_ptr(), nat._dtype_code(x), 0
        d.n, d.c, d.h, d.w = x.shape
        d.sn, d.sc, d.sh, d.sw = x.stride()
        d.kh = d.kw = d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1
        d.pad_h = d.pad_w = 0
        d.sample_weight, d.alpha, d.beta, d.out, d.ldo = None, 0.25, 0.0, out.data_ptr(), out.stride(0)
    L = nat.lib()
    nbytes = L.sso_factor_batch_workspace_bytes(2, arr)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    nat.configure('wait_kcycles', 2000)
    nat.configure('inject_stall', 1)
    nat._check(L.sso_factor_batch(2, arr, ws.data_ptr(), nbytes, stream))
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) != 0
    assert all(bool(torch.isnan(o).all()) for o in outs)
    nat.configure('inject_stall', 0)
    nat.configure('wait_kcycles', 0)
    nat._check(L.sso_factor_batch(2, arr, ws.data_ptr(), nbytes, stream))
    for x, out in zip(xs, outs):
        ref = ko.conv_factor_A(x.double().cpu(), (1, 1), (1, 1), (0, 0), (1, 1), False)
        assert _rel(out, ref) < 1e-5
    assert int(ws[:4].view(torch.int32).item()) == 0


def test_engine_tile_task_wait_runs_out(nat):
    d = 384
    xa = cases.make_normal((4 * d, d), 7)
    A = ((xa.t() @ xa) / xa.shape[0]).cuda()

    def run(stall):
        src = [A.clone()]
        dst = [torch.zeros_like(A)]
        work = [torch.zeros_like(A)]
        plan = nat.kron_plan([d], src, dst, work, None, [-1], [0], torch.device('cuda'))
        damp = torch.full((1,), math.sqrt(1e-3), device='cuda')
        info = torch.zeros(2, dtype=torch.int32, device='cuda')
        if stall:
            nat.configure('wait_kcycles', 2000)
            nat.configure('inject_stall', 1)
        try:
            nat.kron_plan_run(plan, damp, info, True, False)
            torch.cuda.synchronize()
        finally:
            nat.configure('inject_stall', 0)
            nat.configure('wait_kcycles', 0)
        return plan, dst[0], info

    plan, inv, info = run(True)
    assert plan.status() != 0
    assert int(info[0]) == -(1000 + plan.status()), info
    assert bool(torch.isnan(inv).any()), 'tiles of a task whose wait gave up must be NaN'
    plan, inv, info = run(False)
    assert plan.status() == 0 and int(info.abs().sum()) == 0
    ref = torch.linalg.inv(A.double().cpu() + math.sqrt(1e-3) * torch.eye(d, dtype=torch.float64))
    assert _rel(inv, ref) < 1e-4


def test_pool_check_info_reports_a_wait_that_gave_up(nat):
    import torch.nn as nn
    import torchsso
    lin = nn.Linear(300, 200).cuda()
    curv = torchsso.KronCovLinear(lin, ema_decay=1.0, damping=1e-3)
    x = cases.make_normal((64, 300), 9).cuda()
    lin(x).square().mean().backward()
    nat.configure('wait_kcycles', 2000)
    nat.configure('inject_stall', 1)
    try:
        curv.update_ema()
        curv.update_inv()
        torch.cuda.synchronize()
    finally:
        nat.configure('inject_stall', 0)
        nat.configure('wait_kcycles', 0)
    with pytest.raises(RuntimeError, match='wait of the inverse plan gave up'):
        curv.pool.check_info()
