"""Step-level parity on the GPU: the torchsso optimizers of this repository, driven exactly like
the reference's (same constructor arguments, same closure protocol), against golden vectors
produced by the unmodified reference on CPU (tests/golden/make_golden.py).

Random draws are aligned by substituting the Fisher target draw and ``torch.randn_like`` with
the same seeded numpy streams the generator used.  Tolerances: factors 1e-5, inverses and
updates 1e-4 on the first step (growing slowly afterwards, because parameters that differ in
the 5th digit feed the next step), loss trajectories |dloss| <= 1e-3 * max(1, |loss|)."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import cases
from oracle.kfac_step import inverse_cdf_targets

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), 'golden')
KRON = {'Linear': 'Kron', 'Conv2d': 'Kron', 'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'}


def load(name):
    return np.load(os.path.join(GOLD, name + '.npz'))


def rel(a, b, floor=1e-30):
    a = torch.as_tensor(np.asarray(a.detach().cpu() if torch.is_tensor(a) else a)).double()
    b = torch.as_tensor(np.asarray(b)).double()
    return ((a - b).norm() / b.norm().clamp_min(floor)).item()


@pytest.fixture
def torchsso_mod():
    import torchsso
    return torchsso


def patch_targets(monkeypatch, torchsso, state):
    def fake(prob, num_mc):
        return inverse_cdf_targets(prob.detach().float().cpu(), state['u']).to(prob.device)
    monkeypatch.setattr(torchsso.curv.fisher, 'sample_targets', fake)


def check(gold, tag, opt, f_tol, i_tol, with_std=False, grad_floor=1e-30):
    for gi, group in enumerate(opt.param_groups):
        curv = group['curv']
        for j, e in enumerate(curv.ema):
            assert rel(e, gold['%s/g%d/ema%d' % (tag, gi, j)]) < f_tol, (tag, gi, 'ema', j)
        for j, e in enumerate(curv.inv):
            assert rel(e, gold['%s/g%d/inv%d' % (tag, gi, j)]) < i_tol, (tag, gi, 'inv', j)
        if with_std:
            for j, e in enumerate(curv.std):
                assert rel(e, gold['%s/g%d/std%d' % (tag, gi, j)]) < i_tol, (tag, gi, 'std', j)
        for j, p in enumerate(group['params']):
            assert rel(p, gold['%s/g%d/param%d' % (tag, gi, j)]) < f_tol * 10, (tag, gi, 'param', j)
            assert rel(p.grad, gold['%s/g%d/grad%d' % (tag, gi, j)], grad_floor) < i_tol * 3, (tag, gi, 'grad', j)


@pytest.mark.parametrize('prune,batched', [(True, True), (True, False), (False, False)])
def test_tiny_convnet_fisher_mc(torchsso_mod, monkeypatch, prune, batched):
    """prune: the sampling passes ask autograd for the hooked output gradients only (default) or
    run the reference's full backward with frozen parameters; batched: the two Monte Carlo targets
    share one walk of the graph or take one each (default), as in the reference
    (torchsso/curv/fisher/__init__.py:65-72); same vectors every way."""
    torchsso = torchsso_mod
    gold = load('tiny_convnet_fisher')
    state = {}
    patch_targets(monkeypatch, torchsso, state)
    model = cases.make_model('tiny_convnet', seed=1).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON,
                                              {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2)
    for t in range(4):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100 + t)
        state['u'] = cases.make_uniform((2, 6), seed=200 + t)
        opt.update_inv = (t != 2)
        closure = torchsso.get_closure_for_fisher(opt, model, x.cuda(), y.cuda(), approx_type='mc', num_mc=2,
                                                  prune_sampling_pass=prune, batch_mc_passes=batched)
        loss, _ = opt.step(closure=closure)
        for group in opt.param_groups:
            assert 'output_edge' not in group['curv'].module.__dict__ or not prune
        opt.pool.check_info()
        g = float(gold['step%d/loss' % t])
        assert abs(loss.item() - g) <= 1e-3 * max(1.0, abs(g))
        for gi, group in enumerate(opt.param_groups):
            for j, d in enumerate(group['curv'].data):
                assert rel(d, gold['step%d/g%d/data%d' % (t, gi, j)]) < 1e-5 * (1 + 3 * t), (t, gi, j)
        check(gold, 'step%d' % t, opt, 1e-5 * (1 + 3 * t), 1e-4 * (1 + 3 * t))


def test_tiny_convnet_diag_fisher_and_cov(torchsso_mod, monkeypatch):
    """Every layer with the diagonal curvature (the squared per-sample gradient kernel for
    Linear / Conv2d), against the unmodified reference's vectors."""
    torchsso = torchsso_mod
    gold = load('tiny_convnet_diag')
    state = {}
    patch_targets(monkeypatch, torchsso, state)
    diag = {'Linear': 'Diag', 'Conv2d': 'Diag', 'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'}
    model = cases.make_model('tiny_convnet', seed=4).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', diag, {'ema_decay': 0.9, 'damping': 1e-3}, lr=1e-2)
    for t in range(2):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=500 + t)
        state['u'] = cases.make_uniform((2, 6), seed=600 + t)
        # (second step: both targets in one batched walk of the graph, whose slices then feed the
        # BatchNorm and squared-gradient kernels)
        closure = torchsso.get_closure_for_fisher(opt, model, x.cuda(), y.cuda(), approx_type='mc', num_mc=2,
                                                  batch_mc_passes=(t == 1))
        loss, _ = opt.step(closure=closure)
        assert abs(loss.item() - float(gold['fisher%d/loss' % t])) < 1e-4
        # the bias of a convolution that feeds a BatchNorm has a gradient of pure rounding noise
        # (1e-7): a floor on the denominator keeps the relative error meaningful
        check(gold, 'fisher%d' % t, opt, 2e-5, 1e-4, grad_floor=1e-2)
    model = cases.make_model('tiny_convnet', seed=5).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Cov', diag, {'ema_decay': 0.9, 'damping': 1e-3}, lr=1e-2)
    for t in range(2):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=700 + t)
        x, y = x.cuda(), y.cuda()

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, _ = opt.step(closure=closure)
        assert abs(loss.item() - float(gold['cov%d/loss' % t])) < 1e-4
        check(gold, 'cov%d' % t, opt, 2e-5, 1e-4, grad_floor=1e-2)


def test_tiny_convnet_fisher_exact(torchsso_mod):
    torchsso = torchsso_mod
    gold = load('tiny_convnet_fisher_exact')
    model = cases.make_model('tiny_convnet', seed=2).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON,
                                              {'ema_decay': 1.0, 'damping': 1e-3}, lr=1e-2)
    x, y = cases.make_batch((6, 3, 8, 8), 5, seed=300)
    closure = torchsso.get_closure_for_fisher(opt, model, x.cuda(), y.cuda(), approx_type=None)
    loss, _ = opt.step(closure=closure)
    assert abs(loss.item() - float(gold['step0/loss'])) < 1e-4
    check(gold, 'step0', opt, 1e-5, 1e-4)


def test_tiny_convnet_fisher_exact_on_curvature_stream(torchsso_mod):
    """Exact Fisher with the hooks' kernels on the side stream: the per-class weight vector is rebound
    for every class while kernels of the previous class may still read the old one."""
    torchsso = torchsso_mod
    gold = load('tiny_convnet_fisher_exact')
    model = cases.make_model('tiny_convnet', seed=2).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON,
                                              {'ema_decay': 1.0, 'damping': 1e-3}, lr=1e-2)
    x, y = cases.make_batch((6, 3, 8, 8), 5, seed=300)
    closure = torchsso.get_closure_for_fisher(opt, model, x.cuda(), y.cuda(), approx_type=None)
    torchsso.utils.set_curvature_stream(True)
    try:
        loss, _ = opt.step(closure=closure)
    finally:
        torchsso.utils.set_curvature_stream(False)
    assert abs(loss.item() - float(gold['step0/loss'])) < 1e-4
    check(gold, 'step0', opt, 1e-5, 1e-4)


def test_small_mlp_lars_and_weight_normalisation(torchsso_mod):
    """LARS (on the preconditioned and on the raw gradient) and weight normalisation
    (torchsso/optim/secondorder.py:282-330) against the unmodified reference's vectors."""
    torchsso = torchsso_mod
    gold = load('small_mlp_lars_wnorm')
    for tag, kw in (('pre', dict(lars=True, lars_type='preconditioned', normalizing_weights=True)),
                    ('raw', dict(lars=True, lars_type='raw', normalizing_weights=True, weight_scale=1.5,
                                 momentum=0.9, momentum_type='raw'))):
        model = cases.make_model('small_mlp', seed=6).cuda()
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Cov', KRON, {'ema_decay': 0.9, 'damping': 1e-2},
                                                  lr=5e-2, **kw)
        for t in range(3):
            x, y = cases.make_batch((8, 20), 4, seed=800 + t)
            x, y = x.cuda(), y.cuda()

            def closure():
                opt.zero_grad()
                o = model(x)
                loss = F.cross_entropy(o, y)
                loss.backward()
                return loss, o
            loss, _ = opt.step(closure=closure)
            assert abs(loss.item() - float(gold['%s%d/loss' % (tag, t)])) < 1e-4
            check(gold, '%s%d' % (tag, t), opt, 1e-5 * (1 + 3 * t), 1e-4 * (1 + 3 * t))


def test_tiny_convnet_max_ema(torchsso_mod):
    """use_max_ema: BatchNorm curvatures invert the running maximum of the EMA, Kronecker ones the
    EMA itself, as the reference does (torchsso/curv/curvature.py:193-195 against :302-312)."""
    torchsso = torchsso_mod
    gold = load('tiny_convnet_max_ema')
    model = cases.make_model('tiny_convnet', seed=7).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Cov', KRON,
                                              {'ema_decay': 0.5, 'damping': 1e-2, 'use_max_ema': True}, lr=1e-2)
    for t in range(3):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=900 + t)
        if t == 1:
            x = x * 0.3
        x, y = x.cuda(), y.cuda()

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, _ = opt.step(closure=closure)
        assert abs(loss.item() - float(gold['step%d/loss' % t])) < 1e-4
        check(gold, 'step%d' % t, opt, 1e-5 * (1 + 3 * t), 1e-4 * (1 + 3 * t))
        for gi, group in enumerate(opt.param_groups):
            for j, e in enumerate(group['curv'].ema_max):
                assert rel(e, gold['step%d/g%d/ema_max%d' % (t, gi, j)]) < 1e-5 * (1 + 3 * t)


def test_full_matrix_curvature_classes(torchsso_mod):
    """CovLinear builds the reference's full per-sample-gradient covariance with torch ops; the
    classes the reference ships as empty stubs refuse construction with the reason."""
    import torch.nn as nn
    torchsso = torchsso_mod
    lin = nn.Linear(5, 3).cuda()
    curv = torchsso.CovLinear(lin, ema_decay=1.0, damping=1e-2)
    x = cases.make_normal((7, 5), 3).cuda()
    out = lin(x)
    g = cases.make_normal((7, 3), 4).cuda()
    out.backward(g)
    xb = torch.cat([x, torch.ones(7, 1, device='cuda')], 1)
    per = torch.einsum('bi,bj->bij', g, xb).reshape(7, -1)
    assert rel(curv.data[0], (per.t() @ per).cpu().numpy()) < 1e-5
    curv.step()
    ref = torch.linalg.inv((per.t() @ per).double() + 1e-2 * torch.eye(18, device='cuda', dtype=torch.float64))
    assert rel(curv.inv[0], ref.cpu().numpy()) < 1e-4
    for cls, mod in ((torchsso.CovConv2d, nn.Conv2d(2, 2, 3)), (torchsso.CovBatchNorm2d, nn.BatchNorm2d(2)),
                     (torchsso.CovBatchNorm1d, nn.BatchNorm1d(2))):
        with pytest.raises(NotImplementedError, match='full-matrix curvature'):
            cls(mod.cuda())


def test_small_mlp_cov_momentum_l2_accsteps(torchsso_mod):
    torchsso = torchsso_mod
    gold = load('small_mlp_cov')
    model = cases.make_model('small_mlp', seed=3).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Cov', KRON, {'ema_decay': 0.9, 'damping': 1e-2},
                                              lr=5e-2, momentum=0.9, l2_reg=1e-3, weight_decay=1e-4,
                                              acc_steps=2)
    upd = 0
    for t in range(6):
        x, y = cases.make_batch((8, 20), 4, seed=400 + t)
        x, y = x.cuda(), y.cuda()

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, _ = opt.step(closure=closure)
        assert abs(loss.item() - float(gold['micro%d/loss' % t])) < 1e-4
        if t % 2 == 1:
            check(gold, 'step%d' % upd, opt, 1e-5 * (1 + 3 * upd), 1e-4 * (1 + 3 * upd))
            upd += 1


def test_tiny_vgg_vi(torchsso_mod, monkeypatch):
    torchsso = torchsso_mod
    gold = load('tiny_vgg_vi')
    model = cases.make_model('tiny_vgg', seed=4).cuda()
    state = {'seed': 0, 'count': 0}

    def fake_randn_like(t, **kw):
        s = state['seed'] * 1000 + state['count']
        state['count'] += 1
        return cases.make_normal(tuple(t.shape), s).to(device=t.device, dtype=t.dtype)

    opt = torchsso.optim.VIOptimizer(model, 1000, 'Cov', KRON, {'ema_decay': 0.95, 'damping': 1e-3},
                                     lr=1e-2, num_mc_samples=2, val_num_mc_samples=2, kl_weighting=1,
                                     prior_variance=1)
    monkeypatch.setattr(torch, 'randn_like', fake_randn_like)
    for t in range(3):
        x, y = cases.make_batch((8, 3, 8, 8), 6, seed=600 + t)
        x, y = x.cuda(), y.cuda()
        state['seed'], state['count'] = 700 + t, 0

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, prob = opt.step(closure=closure)
        opt.pool.check_info()
        assert abs(loss.item() - float(gold['step%d/loss' % t])) < 1e-4
        assert rel(prob, gold['step%d/prob' % t]) < 1e-4
        check(gold, 'step%d' % t, opt, 2e-5 * (1 + 3 * t), 2e-4 * (1 + 3 * t), with_std=True)
        for gi, group in enumerate(opt.param_groups):
            for j, m in enumerate(group['mean']):
                assert rel(m, gold['step%d/g%d/mean%d' % (t, gi, j)]) < 1e-4


def test_mnist_mlp_100_step_trajectory(torchsso_mod, monkeypatch):
    """784-1000-1000-10 MLP, batch 128, Fisher MC(1), EMA 0.95, damping 1e-3, lr 1e-2, inverse
    every step, one fixed batch: the loss trajectory must follow the reference's CPU run."""
    torchsso = torchsso_mod
    gold = load('mnist_mlp_fisher')['losses']
    state = {}
    patch_targets(monkeypatch, torchsso, state)
    model = cases.make_model('mnist_mlp', seed=0).cuda()
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON,
                                              {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2)
    x, y = cases.make_batch((128, 1, 28, 28), 10, seed=0)
    x, y = x.cuda(), y.cuda()
    losses = []
    for t in range(100):
        state['u'] = cases.make_uniform((1, 128), seed=5000 + t)
        closure = torchsso.get_closure_for_fisher(opt, model, x, y, approx_type='mc', num_mc=1)
        loss, _ = opt.step(closure=closure)
        losses.append(loss.item())
    opt.pool.check_info()
    worst = max(abs(a - b) / max(1.0, abs(b)) for a, b in zip(losses, gold))
    assert worst <= 1e-3, (worst, losses[:5], gold[:5])


def test_standalone_curvature_objects(torchsso_mod):
    """Curvature classes are usable without an optimizer (private pool of one layer)."""
    import torch.nn as nn
    from oracle import kfac_oracle as ko
    torchsso = torchsso_mod
    lin = nn.Linear(12, 7).cuda()
    curv = torchsso.KronCovLinear(lin, ema_decay=1.0, damping=1e-2)
    x = cases.make_normal((9, 12), 1).cuda()
    out = lin(x)
    out.square().mean().backward()
    A, G = curv.data
    assert rel(A, ko.linear_factor_A(x.cpu().double(), True)) < 1e-5
    curv.step()
    Ai, Gi = ko.kron_damped_inverse(curv.ema[0].cpu().double(), curv.ema[1].cpu().double(), 1e-2)
    assert rel(curv.inv[0], Ai) < 1e-4 and rel(curv.inv[1], Gi) < 1e-4
    gw, gb = lin.weight.grad.clone(), lin.bias.grad.clone()
    curv.precondition_grad([lin.weight, lin.bias])
    rw, rb = ko.kron_precondition(Ai, Gi, gw.cpu().double(), gb.cpu().double())
    assert rel(lin.weight.grad, rw) < 1e-4 and rel(lin.bias.grad, rb) < 1e-4


def test_constructor_validation_matches_reference(torchsso_mod):
    import torch.nn as nn
    torchsso = torchsso_mod
    model = nn.Sequential(nn.Linear(4, 3)).cuda()
    with pytest.raises(ValueError, match='Invalid learning rate'):
        torchsso.optim.SecondOrderOptimizer(model, 'Cov', KRON, {}, lr=-1)
    with pytest.raises(ValueError, match='Invalid ema_decay'):
        torchsso.optim.SecondOrderOptimizer(model, 'Cov', KRON, {'ema_decay': 2.0})
    with pytest.raises(AssertionError, match='Failed to lookup Curvature class'):
        torchsso.optim.SecondOrderOptimizer(model, 'Nope', KRON, {})


def test_conv_stem_with_three_channels_channels_last(torchsso_mod):
    """3-channel channels_last input (image stem): channels are zero-padded to a 16-byte chunk for the
    tensor-core kernel and the padding rows / columns dropped again; with and without bias."""
    import torch.nn as nn
    from oracle import kfac_oracle as ko
    torchsso = torchsso_mod
    for bias in (False, True):
        conv = nn.Conv2d(3, 8, 7, stride=2, padding=3, bias=bias).cuda().to(memory_format=torch.channels_last)
        curv = torchsso.KronCovConv2d(conv, ema_decay=1.0, damping=1e-3)
        x = cases.make_normal((4, 3, 20, 20), 17).cuda().contiguous(memory_format=torch.channels_last)
        conv(x).square().mean().backward()
        ref = ko.conv_factor_A(x.cpu().double(), (7, 7), (2, 2), (3, 3), (1, 1), bias)
        assert rel(curv.data[0], ref) < 1e-5


@pytest.mark.parametrize('side_stream', [False, True])
def test_graphed_closure_equals_eager(torchsso_mod, side_stream):
    """Replaying the closure from a CUDA graph (hooks' curvature kernels included, on the main
    stream or forked to the curvature side stream) must give the same parameters as issuing it
    eagerly."""
    torchsso = torchsso_mod

    def run(graphed):
        model = cases.make_model('tiny_convnet', seed=1).cuda()
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Cov', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2)
        xs = torch.empty((6, 3, 8, 8), device='cuda')
        ys = torch.empty((6,), dtype=torch.int64, device='cuda')

        def closure():
            opt.zero_grad()
            o = model(xs)
            loss = F.cross_entropy(o, ys)
            loss.backward()
            return loss, o
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100)
        xs.copy_(x); ys.copy_(y)
        step_closure = closure
        if graphed:
            # batch-norm running statistics advance during warm-up and capture: snapshot / restore
            state = {k: v.clone() for k, v in model.state_dict().items()}
            step_closure = torchsso.utils.GraphedClosure(opt, closure)
            model.load_state_dict(state)
            assert step_closure.library_kernels_per_replay > 0
        losses = []
        for t in range(3):
            x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100 + t)
            xs.copy_(x); ys.copy_(y)
            loss, _ = opt.step(closure=step_closure)
            losses.append(loss.item())
        return losses, [p.detach().clone() for p in model.parameters()]

    l0, p0 = run(False)
    torchsso.utils.set_curvature_stream(side_stream)
    try:
        l1, p1 = run(True)
        if side_stream:          # eager launches through the side stream as well
            l2, p2 = run(False)
            assert max(abs(a - b) for a, b in zip(l0, l2)) < 1e-5
    finally:
        torchsso.utils.set_curvature_stream(False)
    assert max(abs(a - b) for a, b in zip(l0, l1)) < 1e-5
    for a, b in zip(p0, p1):
        assert rel(b, a.cpu().numpy()) < 1e-5


@pytest.mark.parametrize('graphed', [False, True])
def test_fused_ema_equals_separate_pass(torchsso_mod, monkeypatch, graphed):
    """optimizer.fuse_ema: the running average written by the epilogue of the factor / BatchNorm
    kernels equals the separate data -> ema pass (eagerly and from a replayed graph, whose warm-up
    executions must leave the averages untouched)."""
    torchsso = torchsso_mod
    state = {}

    def run(fuse):
        patch_targets(monkeypatch, torchsso, state)      # (the graphed variant swaps in fixed targets below)
        model = cases.make_model('tiny_convnet', seed=1).cuda()
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON, {'ema_decay': 0.9, 'damping': 1e-3}, lr=1e-2)
        xs = torch.empty((6, 3, 8, 8), device='cuda')
        ys = torch.empty((6,), dtype=torch.int64, device='cuda')
        closure = torchsso.get_closure_for_fisher(opt, model, xs, ys, approx_type='mc', num_mc=2)
        step_closure = closure
        for t in range(4):
            x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100 + t)
            xs.copy_(x); ys.copy_(y)
            state['u'] = cases.make_uniform((2, 6), seed=200 + t)
            if t == 1:
                opt.fuse_ema = fuse
                if graphed:
                    with torch.no_grad():
                        fixed = inverse_cdf_targets(torch.softmax(model(xs), dim=1).float().cpu(), state['u']).cuda()
                    monkeypatch.setattr(torchsso.curv.fisher, 'sample_targets', lambda prob, num_mc: fixed)
                    bn = {k: v.clone() for k, v in model.state_dict().items()}
                    step_closure = torchsso.utils.GraphedClosure(opt, closure)
                    model.load_state_dict(bn)
            if graphed and t >= 1:      # the captured targets are those of step 1: keep its batch too
                x, y = cases.make_batch((6, 3, 8, 8), 5, seed=101)
                xs.copy_(x); ys.copy_(y)
            opt.update_inv = (t != 2)
            opt.step(closure=step_closure)
        emas = [e.clone() for g in opt.param_groups for e in g['curv'].ema]
        if fuse:
            assert all(g['curv'].data is None for g in opt.param_groups)
        return emas, [p.detach().clone() for p in model.parameters()]

    e0, p0 = run(False)
    e1, p1 = run(True)
    for a, b in zip(e0 + p0, e1 + p1):
        assert rel(b, a.cpu().numpy()) < 3e-5        # one fused multiply-add instead of two rounded steps, over four updates


@pytest.mark.parametrize('graphed', [False, True])
def test_early_inverse_equals_inverse_after_closure(torchsso_mod, monkeypatch, graphed):
    """optimizer.early_inverse: the round of inverses issued inside the closure (after the sampling
    passes, on the curvature stream, beside the real backward pass) gives the same parameters as
    the round issued after the closure; from a replayed graph there is one graph per kind of step."""
    torchsso = torchsso_mod
    state = {}

    def run(early):
        patch_targets(monkeypatch, torchsso, state)
        model = cases.make_model('tiny_convnet', seed=1).cuda()
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON, {'ema_decay': 0.9, 'damping': 1e-3}, lr=1e-2)
        opt.fuse_ema = True
        opt.early_inverse = early
        xs = torch.empty((6, 3, 8, 8), device='cuda')
        ys = torch.empty((6,), dtype=torch.int64, device='cuda')
        closure = torchsso.get_closure_for_fisher(opt, model, xs, ys, approx_type='mc', num_mc=2)
        step_closure = closure
        torchsso.utils.set_curvature_stream(True)
        try:
            for t in range(5):
                x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100 + min(t, 1) if graphed else 100 + t)
                xs.copy_(x); ys.copy_(y)
                state['u'] = cases.make_uniform((2, 6), seed=200 + t)
                if t == 1 and graphed:
                    with torch.no_grad():
                        fixed = inverse_cdf_targets(torch.softmax(model(xs), dim=1).float().cpu(), state['u']).cuda()
                    monkeypatch.setattr(torchsso.curv.fisher, 'sample_targets', lambda prob, num_mc: fixed)
                    bn = {k: v.clone() for k, v in model.state_dict().items()}
                    step_closure = torchsso.utils.GraphedClosure(opt, closure)
                    model.load_state_dict(bn)
                opt.update_inv = t in (0, 2, 3)
                opt.step(closure=step_closure)
                opt.pool.check_info()
        finally:
            torchsso.utils.set_curvature_stream(False)
        invs = [e.clone() for g in opt.param_groups for e in g['curv'].inv]
        return invs + [p.detach().clone() for p in model.parameters()]

    a, b = run(False), run(True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_fisher_sampling_survives_nan_probabilities(torchsso_mod):
    """NaN / zero rows in the predictive distribution (a diverged model) must not reach the
    sampling kernel's device-side assertion."""
    from torchsso.curv import fisher
    prob = torch.tensor([[float('nan'), 0.5, 0.5], [0.0, 0.0, 0.0], [0.2, 0.3, 0.5]], device='cuda')
    torch.manual_seed(1234)
    t = fisher.sample_targets(prob, 4)
    torch.cuda.synchronize()
    assert t.shape == (4, 3), t.shape
    assert int(t.min()) >= 0 and int(t.max()) <= 2, t
    assert int(t[:, 0].min()) >= 1, t       # the NaN class is never drawn


def test_zero_grad_to_none_same_step(torchsso_mod, monkeypatch):
    """Both gradient protocols of zero_grad() (bind to the flat buffer / set to None and harvest)
    give the same update."""
    torchsso = torchsso_mod
    state = {}
    patch_targets(monkeypatch, torchsso, state)
    outs = []
    for to_none in (False, True):
        model = cases.make_model('tiny_convnet', seed=1).cuda()
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON, {'ema_decay': 0.95, 'damping': 1e-3},
                                                  lr=1e-2, momentum=0.9, weight_decay=1e-4)
        opt.zero_grad_to_none = to_none
        for t in range(3):
            x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100 + t)
            state['u'] = cases.make_uniform((2, 6), seed=200 + t)
            closure = torchsso.get_closure_for_fisher(opt, model, x.cuda(), y.cuda(), approx_type='mc', num_mc=2)
            opt.step(closure=closure)
        outs.append([p.detach().clone() for p in model.parameters()])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_batch_prefetcher_delivers_every_batch_in_order(torchsso_mod):
    """The double-buffered input pipeline: the fixed device tensors hold batch i during iteration i, for
    more batches than staging buffers, while a kernel on the compute stream keeps the consumer busy."""
    torchsso = torchsso_mod
    batches = [(torch.full((64, 3, 8, 8), float(i)).pin_memory(), torch.full((64,), i, dtype=torch.int64).pin_memory())
               for i in range(7)]
    x = torch.empty((64, 3, 8, 8), device='cuda')
    y = torch.empty((64,), dtype=torch.int64, device='cuda')
    seen = []
    sink = torch.zeros((), device='cuda')
    for i in torchsso.utils.BatchPrefetcher(iter(batches), (x, y)):
        torch.cuda._sleep(2_000_000)            # ~1 ms of "step" between the copy in and the read below
        sink += x.sum() * 0 + y.float().mean()
        seen.append((i, x.clone(), y.clone()))
    torch.cuda.synchronize()
    assert [i for i, _, _ in seen] == list(range(7))
    for i, xv, yv in seen:
        assert torch.equal(xv.cpu(), batches[i][0]) and torch.equal(yv.cpu(), batches[i][1])
    assert float(sink) == sum(range(7))
