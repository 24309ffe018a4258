"""Full-size checks (the ResNet-50 / batch 32 shapes of the benchmark configuration) through
properties that need no full-size oracle: the CPU restatement would take minutes on these sizes, so
the CUDA path is checked against identities that hold for any input.

* factors: symmetric bit for bit; trace(A) equals the mean squared norm of the im2col rows, which a
  box filter over x^2 gives independently; a column block of A equals the small-case kernel run on a
  channel slice (linearity in the column set); two halves of the batch add up (linearity in rows);
* damped inverse at d = 4608: (M + vI) M^-1 = I to fp32 accuracy, M^-1 symmetric bit for bit;
* precondition at (4608, 512): G (G^-1 dW A^-1) A = dW.
"""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def nat():
    from torchsso import _native
    _native.lib()
    return _native


def rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-300)).item()


# (c, h, w, k, stride, pad) at batch 32: the wide 3x3 layers of ResNet-50 and one 1x1
FULL = [(64, 56, 56, 3, 1, 1), (128, 28, 28, 3, 1, 1), (256, 14, 14, 3, 1, 1), (512, 7, 7, 3, 1, 1),
        (512, 14, 14, 3, 2, 1), (1024, 14, 14, 1, 1, 0)]


@pytest.mark.parametrize('cfg', FULL)
def test_full_size_factor_properties(nat, cfg):
    c, h, w, k, s, p = cfg
    n = 32
    g = torch.Generator(device='cuda').manual_seed(c + h)
    x = torch.randn((n, c, h, w), device='cuda', generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    d = c * k * k
    geo = ((k, k), (s, s), (p, p), (1, 1))
    A = torch.full((d, d), float('nan'), device='cuda')
    nat.factor_im2col(x, *geo, False, None, 1.0 / n, 0.0, A)
    assert torch.isfinite(A).all()
    assert torch.equal(A, A.t())
    # trace: sum over output pixels and kernel offsets of x^2 = box filter of x^2, summed
    x2 = (x.float() ** 2).sum(dim=1, keepdim=True)
    box = F.conv2d(x2, torch.ones((1, 1, k, k), device='cuda'), stride=s, padding=p)
    assert abs(A.trace().item() / (box.sum().item() / n) - 1.0) < 1e-5
    # diagonal entries per (channel, offset): column (ch, ky, kx) has energy sum_pixels x[ch, ...]^2
    ch = c // 3
    xs = (x[:, ch:ch + 1].float() ** 2)
    per = F.conv2d(xs, torch.eye(k * k, device='cuda').reshape(k * k, 1, k, k), stride=s, padding=p).sum(dim=(0, 2, 3)) / n
    assert rel(A.diagonal()[ch * k * k:(ch + 1) * k * k], per) < 1e-5
    # linearity in the rows: the two halves of the batch add up to the whole
    H0 = torch.empty_like(A)
    nat.factor_im2col(x[:n // 2], *geo, False, None, 1.0 / n, 0.0, H0)
    nat.factor_im2col(x[n // 2:], *geo, False, None, 1.0 / n, 1.0, H0)       # beta = 1 accumulates
    assert rel(H0, A) < 1e-5
    # a 64-channel slice through the small-shape kernel reproduces its diagonal block
    xs64 = x[:, :64].contiguous(memory_format=torch.channels_last)
    B = torch.empty((64 * k * k, 64 * k * k), device='cuda')
    nat.factor_im2col(xs64, *geo, False, None, 1.0 / n, 0.0, B)
    assert rel(A[:64 * k * k, :64 * k * k], B) < 1e-5


def _spd(d, seed):
    g = torch.Generator(device='cuda').manual_seed(seed)
    x = torch.randn((2 * d, d), device='cuda', generator=g)
    return (x.t() @ x) / x.shape[0]


def test_full_size_inverse_identity(nat):
    dA, dG = 4608, 512
    A, G = _spd(dA, 1), _spd(dG, 2)
    src = [A, G]
    dst = [torch.full_like(m, float('nan')) for m in src]
    work = [torch.empty_like(m) for m in src]
    plan = nat.kron_plan([dA, dG], src, dst, work, None, [1, 0], [0, 1], torch.device('cuda'))
    damping = 1e-3
    r = math.sqrt(damping)
    damp = torch.full((2,), r, device='cuda')
    info = torch.zeros(4, dtype=torch.int32, device='cuda')
    nat.kron_plan_run(plan, damp, info, True, False)
    assert int(info.abs().sum()) == 0
    pi = math.sqrt((A.trace().item() / dA) / (G.trace().item() / dG))
    for M, Mi, v, d in ((A, dst[0], r * pi, dA), (G, dst[1], r / pi, dG)):
        assert torch.equal(Mi, Mi.t())
        eye = torch.eye(d, device='cuda', dtype=torch.float64)
        resid = ((M.double() + v * eye) @ Mi.double() - eye).norm().item() / math.sqrt(d)
        assert resid < 1e-4, resid


def test_full_size_precondition_round_trip(nat):
    dA, dG = 4608, 512
    # well conditioned symmetric factors so that the round trip itself is accurate
    Ai = _spd(dA, 3) + torch.eye(dA, device='cuda')
    Gi = _spd(dG, 4) + torch.eye(dG, device='cuda')
    Ai = (Ai + Ai.t()) / 2
    Gi = (Gi + Gi.t()) / 2
    g = torch.Generator(device='cuda').manual_seed(5)
    dW = torch.randn((dG, dA), device='cuda', generator=g) * 0.1
    out = dW.clone()
    tmp = torch.empty(dG * dA, device='cuda')
    plan = nat.precond_plan([dA], [dG], [Ai], [Gi], [out], [None], [tmp], torch.device('cuda'))
    nat.precond_plan_run(plan)
    ref = Gi.double() @ dW.double() @ Ai.double()
    assert rel(out, ref) < 1e-5
