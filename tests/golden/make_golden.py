"""Generate golden vectors by running the UNMODIFIED reference library on CPU.

Usage (only where the reference source tree is available):
    python tests/golden/make_golden.py /path/to/reference [case ...]

The reference is imported from the given path with three harness-side shims and no
edits to its files:
  * empty ``chainer`` / ``chainer.backends`` / ``chainer.backends.cuda`` modules and
    an empty ``chainermn`` tree, because the communicator module imports them at load;
  * the step-hook dictionaries torch >= 2 expects on an Optimizer, which the
    reference's constructor never creates;
  * ``torchsso.utils.cholesky`` pointed at a CPU Cholesky (lower factor, transposed),
    because the reference only ships a CuPy implementation of it.
Random draws are made reproducible on both sides of a parity test by replacing
``Categorical.sample`` (Fisher MC targets) and ``torch.randn_like`` (VI noise) with
draws derived from seeded numpy streams (see ``cases.py``).

Outputs: ``tests/golden/<case>.npz``.
"""
from __future__ import annotations

import os
import sys
import types
from collections import OrderedDict

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from oracle.kfac_step import inverse_cdf_targets  # noqa: E402

STATE = {'u': None, 'noise_seed': None, 'noise_count': 0}


def import_reference(path: str):
    os.environ['CUDA_VISIBLE_DEVICES'] = ''
    for name in ['chainer', 'chainer.backends', 'chainer.backends.cuda', 'chainermn',
                 'chainermn.communicators', 'chainermn.communicators.mpi_communicator_base',
                 'chainermn.communicators._memory_utility',
                 'chainermn.communicators._communication_utility', 'chainermn.nccl']:
        mod = types.ModuleType(name)
        sys.modules[name] = mod
    sys.modules['chainer'].cuda = types.SimpleNamespace(Stream=types.SimpleNamespace(null=None))
    sys.modules['chainermn.communicators.mpi_communicator_base'].MpiCommunicatorBase = object
    sys.modules['chainermn.communicators']._memory_utility = sys.modules[
        'chainermn.communicators._memory_utility']
    sys.modules['chainermn.communicators']._communication_utility = sys.modules[
        'chainermn.communicators._communication_utility']
    sys.modules['chainermn'].nccl = sys.modules['chainermn.nccl']
    sys.path.insert(0, path)
    import torchsso
    assert os.path.abspath(torchsso.__file__).startswith(os.path.abspath(path))
    torchsso.utils.cholesky = lambda m, upper=True: (
        torch.linalg.cholesky(m).t() if upper else torch.linalg.cholesky(m))

    def fake_sample(self, sample_shape=torch.Size()):
        return inverse_cdf_targets(self.probs, STATE['u'])
    torch.distributions.Categorical.sample = fake_sample
    return torchsso


def fake_randn_like(t, **kw):
    seed = STATE['noise_seed'] * 1000 + STATE['noise_count']
    STATE['noise_count'] += 1
    return cases.make_normal(tuple(t.shape), seed).to(t.dtype)


def fix_hooks(opt):
    opt._optimizer_step_pre_hooks = OrderedDict()
    opt._optimizer_step_post_hooks = OrderedDict()
    return opt


def dump_groups(out, tag, opt, with_std=False):
    for gi, group in enumerate(opt.param_groups):
        curv = group['curv']
        for j, e in enumerate(curv.ema):
            out['%s/g%d/ema%d' % (tag, gi, j)] = e.numpy().copy()
        for j, e in enumerate(curv.inv):
            out['%s/g%d/inv%d' % (tag, gi, j)] = e.numpy().copy()
        if with_std and curv.std is not None:
            for j, e in enumerate(curv.std):
                out['%s/g%d/std%d' % (tag, gi, j)] = e.numpy().copy()
        for j, p in enumerate(group['params']):
            out['%s/g%d/param%d' % (tag, gi, j)] = p.detach().numpy().copy()
            out['%s/g%d/grad%d' % (tag, gi, j)] = p.grad.detach().numpy().copy()


KRON = {'Linear': 'Kron', 'Conv2d': 'Kron', 'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'}


def case_tiny_convnet_fisher(torchsso):
    model = cases.make_model('tiny_convnet', seed=1)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Fisher', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2))
    out = {}
    for t in range(4):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=100 + t)
        STATE['u'] = cases.make_uniform((2, 6), seed=200 + t)
        opt.update_inv = (t != 2)
        closure = torchsso.get_closure_for_fisher(opt, model, x, y, approx_type='mc', num_mc=2)
        loss, _ = opt.step(closure=closure)
        out['step%d/loss' % t] = np.float64(loss.item())
        for gi, group in enumerate(opt.param_groups):
            for j, d in enumerate(group['curv'].data):
                out['step%d/g%d/data%d' % (t, gi, j)] = d.numpy().copy()
        dump_groups(out, 'step%d' % t, opt)
    return out


def case_tiny_convnet_fisher_exact(torchsso):
    """Exact Fisher: one backward per class with prob[:, i] row weights."""
    model = cases.make_model('tiny_convnet', seed=2)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Fisher', KRON, {'ema_decay': 1.0, 'damping': 1e-3}, lr=1e-2))
    out = {}
    x, y = cases.make_batch((6, 3, 8, 8), 5, seed=300)
    closure = torchsso.get_closure_for_fisher(opt, model, x, y, approx_type=None)
    loss, _ = opt.step(closure=closure)
    out['step0/loss'] = np.float64(loss.item())
    dump_groups(out, 'step0', opt)
    return out


DIAG = {'Linear': 'Diag', 'Conv2d': 'Diag', 'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'}


def case_tiny_convnet_diag(torchsso):
    """Diagonal curvature for every layer: two Fisher (MC) steps, then on a fresh model two
    empirical-covariance steps."""
    out = {}
    model = cases.make_model('tiny_convnet', seed=4)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Fisher', DIAG, {'ema_decay': 0.9, 'damping': 1e-3}, lr=1e-2))
    for t in range(2):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=500 + t)
        STATE['u'] = cases.make_uniform((2, 6), seed=600 + t)
        closure = torchsso.get_closure_for_fisher(opt, model, x, y, approx_type='mc', num_mc=2)
        loss, _ = opt.step(closure=closure)
        out['fisher%d/loss' % t] = np.float64(loss.item())
        dump_groups(out, 'fisher%d' % t, opt)
    model = cases.make_model('tiny_convnet', seed=5)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Cov', DIAG, {'ema_decay': 0.9, 'damping': 1e-3}, lr=1e-2))
    for t in range(2):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=700 + t)

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, _ = opt.step(closure=closure)
        out['cov%d/loss' % t] = np.float64(loss.item())
        dump_groups(out, 'cov%d' % t, opt)
    return out


def case_small_mlp_cov(torchsso):
    model = cases.make_model('small_mlp', seed=3)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Cov', KRON, {'ema_decay': 0.9, 'damping': 1e-2}, lr=5e-2, momentum=0.9,
        l2_reg=1e-3, weight_decay=1e-4, acc_steps=2))
    out = {}
    upd = 0
    for t in range(6):
        x, y = cases.make_batch((8, 20), 4, seed=400 + t)

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, _ = opt.step(closure=closure)
        out['micro%d/loss' % t] = np.float64(loss.item())
        if t % 2 == 1:
            dump_groups(out, 'step%d' % upd, opt)
            upd += 1
    return out


def case_mnist_mlp_fisher(torchsso):
    """Single-process CPU configuration: 100 steps on one fixed batch, inverse every step."""
    model = cases.make_model('mnist_mlp', seed=0)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Fisher', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2))
    x, y = cases.make_batch((128, 1, 28, 28), 10, seed=0)
    losses = []
    for t in range(100):
        STATE['u'] = cases.make_uniform((1, 128), seed=5000 + t)
        closure = torchsso.get_closure_for_fisher(opt, model, x, y, approx_type='mc', num_mc=1)
        loss, _ = opt.step(closure=closure)
        losses.append(loss.item())
    out = {'losses': np.array(losses, dtype=np.float64)}
    for gi, group in enumerate(opt.param_groups):
        for j, p in enumerate(group['params']):
            out['final/g%d/param%d_norm' % (gi, j)] = np.float64(p.detach().double().norm().item())
    return out


def case_tiny_vgg_vi(torchsso):
    model = cases.make_model('tiny_vgg', seed=4)
    opt = fix_hooks(torchsso.optim.VIOptimizer(
        model, 1000, 'Cov', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2,
        num_mc_samples=2, val_num_mc_samples=2, kl_weighting=1, prior_variance=1))
    real_randn_like = torch.randn_like
    torch.randn_like = fake_randn_like
    out = {}
    try:
        for t in range(3):
            x, y = cases.make_batch((8, 3, 8, 8), 6, seed=600 + t)
            STATE['noise_seed'], STATE['noise_count'] = 700 + t, 0

            def closure():
                opt.zero_grad()
                o = model(x)
                loss = F.cross_entropy(o, y)
                loss.backward()
                return loss, o
            loss, prob = opt.step(closure=closure)
            out['step%d/loss' % t] = np.float64(loss.item())
            out['step%d/prob' % t] = prob.detach().numpy().copy()
            dump_groups(out, 'step%d' % t, opt, with_std=True)
            for gi, group in enumerate(opt.param_groups):
                for j, m in enumerate(group['mean']):
                    out['step%d/g%d/mean%d' % (t, gi, j)] = m.detach().numpy().copy()
    finally:
        torch.randn_like = real_randn_like
    return out


def dump_summary(out, tag, opt, with_std=False):
    """Fingerprints (cases.summarize) instead of whole tensors, for the full-size models."""
    for gi, group in enumerate(opt.param_groups):
        curv = group['curv']
        items = [('ema%d' % j, e) for j, e in enumerate(curv.ema)]
        items += [('inv%d' % j, e) for j, e in enumerate(curv.inv)]
        if with_std and curv.std is not None:
            items += [('std%d' % j, e) for j, e in enumerate(curv.std)]
        for j, p in enumerate(group['params']):
            items += [('param%d' % j, p), ('grad%d' % j, p.grad)]
        if 'mean' in group:
            items += [('mean%d' % j, m) for j, m in enumerate(group['mean'])]
        for name, t in items:
            for k, v in cases.summarize(t).items():
                out['%s/g%d/%s/%s' % (tag, gi, name, k)] = v


def _convnet_b256_run(torchsso, dtype, out, prefix):
    model = cases.make_model('convnet_b256', seed=11).to(dtype)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Fisher', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2))
    for t in range(3):
        x, y = cases.make_batch((256, 3, 32, 32), 10, seed=1000 + t)
        STATE['u'] = cases.make_uniform((1, 256), seed=2000 + t)
        opt.update_inv = (t == 0)
        closure = torchsso.get_closure_for_fisher(opt, model, x.to(dtype), y, approx_type='mc', num_mc=1)
        loss, _ = opt.step(closure=closure)
        out['%sstep%d/loss' % (prefix, t)] = np.float64(loss.item())
        dump_summary(out, '%sstep%d' % (prefix, t), opt)


def case_convnet_b256_fisher(torchsso):
    """The single-GPU ConvNet configuration at its real shapes: batch 256 of 3x32x32, a fresh batch
    every step (a fixed batch with stale inverses diverges in the reference itself), Fisher MC(1),
    inverse on the first step only (the configuration inverts every 5th step).  The reference is
    run twice: in fp32 as shipped (keys ``step*``) and with model and inputs in fp64 (keys
    ``f64/step*``): the distance between the two is the reference's own rounding noise at these
    sizes, the yardstick for any other fp32 implementation."""
    out = {}
    _convnet_b256_run(torchsso, torch.float32, out, '')
    _convnet_b256_run(torchsso, torch.float64, out, 'f64/')
    return out


def case_vgg16_vi(torchsso):
    """The variational-inference configuration at its real shapes: VGG-16-style stack, batch 128 of
    3x32x32, dataset size 50000, prior variance 1, one weight sample per step, two steps (the
    first step draws no noise because there is no posterior scale yet; the second one does)."""
    model = cases.make_model('vgg16_style', seed=12).to(VGG_DTYPE)
    opt = fix_hooks(torchsso.optim.VIOptimizer(
        model, 50000, 'Cov', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-3,
        num_mc_samples=1, val_num_mc_samples=1, kl_weighting=VGG_KL, prior_variance=1))
    real_randn_like = torch.randn_like
    torch.randn_like = fake_randn_like
    out = {}
    try:
        for t in range(2):
            x, y = cases.make_batch((128, 3, 32, 32), 100, seed=3000 + t)
            x = x.to(VGG_DTYPE)
            STATE['noise_seed'], STATE['noise_count'] = 3100 + t, 0

            def closure():
                opt.zero_grad()
                o = model(x)
                loss = F.cross_entropy(o, y)
                loss.backward()
                return loss, o
            loss, prob = opt.step(closure=closure)
            out['step%d/loss' % t] = np.float64(loss.item())
            out['step%d/prob_rows' % t] = prob.detach()[:4].numpy().copy()
            dump_summary(out, 'step%d' % t, opt, with_std=True)
    finally:
        torch.randn_like = real_randn_like
    return out


# with 1.0 the posterior noise of the untrained network (its G factors are tiny, so their damped
# inverses are huge) blows the second step's loss up to 1e6 in the reference itself
VGG_KL = 0.01
# fp64: in fp32 the reference's CPU inverse (LU) of the 4609-dimensional damped factors is not
# numerically positive definite and its own update_std (Cholesky of that inverse) fails
VGG_DTYPE = torch.float64


def case_small_mlp_lars_wnorm(torchsso):
    """LARS on the preconditioned gradient and weight normalisation after the update
    (torchsso/optim/secondorder.py:282-330), then the same with LARS on the raw gradient."""
    out = {}
    for tag, kw in (('pre', dict(lars=True, lars_type='preconditioned', normalizing_weights=True)),
                    ('raw', dict(lars=True, lars_type='raw', normalizing_weights=True, weight_scale=1.5,
                                 momentum=0.9, momentum_type='raw'))):
        model = cases.make_model('small_mlp', seed=6)
        opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
            model, 'Cov', KRON, {'ema_decay': 0.9, 'damping': 1e-2}, lr=5e-2, **kw))
        for t in range(3):
            x, y = cases.make_batch((8, 20), 4, seed=800 + t)

            def closure():
                opt.zero_grad()
                o = model(x)
                loss = F.cross_entropy(o, y)
                loss.backward()
                return loss, o
            loss, _ = opt.step(closure=closure)
            out['%s%d/loss' % (tag, t)] = np.float64(loss.item())
            dump_groups(out, '%s%d' % (tag, t), opt)
    return out


def case_tiny_convnet_max_ema(torchsso):
    """use_max_ema=True: the diagonal (BatchNorm) curvatures invert the running element-wise maximum
    of the EMA, the Kronecker ones keep inverting the EMA itself (torchsso/curv/curvature.py:193-195
    against :302-312)."""
    model = cases.make_model('tiny_convnet', seed=7)
    opt = fix_hooks(torchsso.optim.SecondOrderOptimizer(
        model, 'Cov', KRON, {'ema_decay': 0.5, 'damping': 1e-2, 'use_max_ema': True}, lr=1e-2))
    out = {}
    for t in range(3):
        x, y = cases.make_batch((6, 3, 8, 8), 5, seed=900 + t)
        if t == 1:
            x = x * 0.3        # smaller curvature on the middle step: EMA and its maximum part ways

        def closure():
            opt.zero_grad()
            o = model(x)
            loss = F.cross_entropy(o, y)
            loss.backward()
            return loss, o
        loss, _ = opt.step(closure=closure)
        out['step%d/loss' % t] = np.float64(loss.item())
        dump_groups(out, 'step%d' % t, opt)
        for gi, group in enumerate(opt.param_groups):
            for j, e in enumerate(group['curv'].ema_max):
                out['step%d/g%d/ema_max%d' % (t, gi, j)] = e.numpy().copy()
    return out


CASES = OrderedDict([
    ('tiny_convnet_fisher', case_tiny_convnet_fisher),
    ('tiny_convnet_fisher_exact', case_tiny_convnet_fisher_exact),
    ('small_mlp_cov', case_small_mlp_cov),
    ('tiny_convnet_diag', case_tiny_convnet_diag),
    ('tiny_vgg_vi', case_tiny_vgg_vi),
    ('mnist_mlp_fisher', case_mnist_mlp_fisher),
    ('small_mlp_lars_wnorm', case_small_mlp_lars_wnorm),
    ('tiny_convnet_max_ema', case_tiny_convnet_max_ema),
    ('convnet_b256_fisher', case_convnet_b256_fisher),
    ('vgg16_vi', case_vgg16_vi),
])


def main():
    ref = sys.argv[1]
    names = sys.argv[2:] or list(CASES)
    torchsso = import_reference(ref)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name in names:
        out = CASES[name](torchsso)
        path = os.path.join(HERE, name + '.npz')
        np.savez_compressed(path, **out)
        print(name, len(out), 'arrays ->', path, os.path.getsize(path), 'bytes')


if __name__ == '__main__':
    main()
