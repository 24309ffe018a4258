"""Whole-step CPU oracle: a K-FAC optimizer step restated with torch CPU autograd and
the op-level oracle in ``kfac_oracle``.  TEST INFRASTRUCTURE ONLY (see that module's
header): used to check loss/parameter trajectories of the CUDA path and as the timed
CPU baseline; the product never imports it.

It follows the control flow of torchsso/optim/secondorder.py:158-231 (step),
torchsso/curv/fisher/__init__.py:50-88 (Fisher closure), torchsso/curv/curvature.py
:118-172 (hooks, step) and torchsso/optim/vi.py:174-258 (VI step), but is organised as
one flat class with per-layer records instead of the reference's class hierarchy.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kfac_oracle as ko


def inverse_cdf_targets(prob: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Deterministic categorical draw shared by both sides of a parity run:
    target[s, i] = first class whose cumulative probability exceeds u[s, i]."""
    cdf = prob.double().cumsum(dim=1)
    cdf = cdf / cdf[:, -1:].clone()
    idx = torch.searchsorted(cdf.unsqueeze(0).expand(u.shape[0], -1, -1).contiguous(),
                             u.double().unsqueeze(-1)).squeeze(-1)
    return idx.clamp_(max=prob.shape[1] - 1)


class _Layer:
    def __init__(self, module: nn.Module):
        self.module = module
        self.params = list(module.parameters())
        self.is_bn = isinstance(module, (nn.BatchNorm1d, nn.BatchNorm2d))
        self.is_conv = isinstance(module, nn.Conv2d)
        self.is_diag = self.is_bn    # BatchNorm is always diagonal; Linear / Conv2d on request
        self.x = None
        self.has_bias = getattr(module, 'bias', None) is not None
        self.data: Optional[List[torch.Tensor]] = None      # Kron: [A, G]; Diag: [w(, b)]
        self.A = None
        self.xhat = None
        self.acc = None          # Fisher accumulation over sampling passes
        self.ema = None
        self.inv = None
        self.std = None
        self.l2_reg = 0.0
        self.l2_reg_ema = 0.0
        self.momentum_buf = [torch.zeros_like(p) for p in self.params]
        self.mean = None


class OracleKFAC:
    """K-FAC ('Cov' or 'Fisher' curvature; Kron for Linear/Conv2d, Diag for BatchNorm)."""

    def __init__(self, model: nn.Module, curv_type: str = 'Fisher', ema_decay: float = 1.0,
                 damping: float = 1e-7, lr: float = 0.01, momentum: float = 0.0,
                 l2_reg: float = 0.0, weight_decay: float = 0.0, acc_steps: int = 1,
                 diag: tuple = (), momentum_type: str = 'preconditioned', lars: bool = False,
                 lars_type: str = 'preconditioned', normalizing_weights: bool = False,
                 weight_scale: Optional[float] = None, use_max_ema: bool = False):
        """``diag``: class names ('Linear', 'Conv2d') that get the diagonal curvature of
        torchsso/curv/cov/linear.py:28-45 / cov/conv.py:15-42 instead of the Kronecker one."""
        assert curv_type in ('Cov', 'Fisher')
        self.model = model
        self.curv_type = curv_type
        self.beta = ema_decay
        self.damping = damping
        self.lr, self.momentum = lr, momentum
        self.l2_reg, self.weight_decay = l2_reg, weight_decay
        self.acc_steps = acc_steps
        self.momentum_type, self.lars, self.lars_type = momentum_type, lars, lars_type
        self.normalizing_weights, self.weight_scale = normalizing_weights, weight_scale
        self.use_max_ema = use_max_ema
        self.acc_step = 0
        self.steps = 0
        self.update_inv = True
        self.sampling = False      # inside a Fisher sampling backward pass
        self.prob = None           # per-sample weight for the current sampling pass
        self.layers: List[_Layer] = []
        self._acc_grads = None
        self._acc_curv = None
        for m in model.modules():
            if len(list(m.children())) > 0 or len(list(m.parameters())) == 0:
                continue
            if not isinstance(m, (nn.Linear, nn.Conv2d, nn.BatchNorm1d, nn.BatchNorm2d)):
                raise AssertionError('no curvature for %s' % type(m).__name__)
            L = _Layer(m)
            L.is_diag = L.is_bn or type(m).__name__ in diag
            self.layers.append(L)
            m.register_forward_hook(self._make_fwd(L))

    # -- hooks ---------------------------------------------------------------
    def _make_fwd(self, L: _Layer):
        def fwd(module, inputs, output):
            x = inputs[0].detach()
            if L.is_bn:
                # curvature.py:123-134
                L.xhat = ko.bn_restore_input(output.detach(), module.weight.detach(),
                                             module.bias.detach())
            elif L.is_diag:
                L.x = x
            elif L.is_conv:
                L.A = ko.conv_factor_A(x, module.kernel_size, module.stride, module.padding,
                                       module.dilation, L.has_bias)
            else:
                L.A = ko.linear_factor_A(x, L.has_bias)
            if output.requires_grad:
                output.register_hook(lambda g, L=L: self._bwd(L, g))
        return fwd

    def _bwd(self, L: _Layer, g: torch.Tensor):
        g = g.detach()
        n = g.shape[0]
        fisher = self.curv_type == 'Fisher'
        if fisher and not self.sampling:
            # real backward: take what the sampling passes accumulated
            # (fisher/linear.py:56-57) and apply the n^2 rescale (curvature.py:151-155)
            new = [t.clone() for t in L.acc]
            L.acc = None
        else:
            p = self.prob if fisher else None
            if L.is_bn:
                new = ko.bn_diag(L.xhat, g, p, L.has_bias)
            elif L.is_diag:
                m = L.module
                if L.is_conv:
                    new = list(ko.diag_conv(L.x, g, m.kernel_size, m.stride, m.padding, m.dilation, p))
                else:
                    new = list(ko.diag_linear(L.x, g, p))
                    new[0] = new[0].reshape(m.weight.shape)
                new = new if L.has_bias else new[:1]
            elif L.is_conv:
                new = [ko.conv_factor_G(g, p)]
            else:
                new = [ko.linear_factor_G(g, p)]
            if fisher:
                # accumulate UNSCALED; the scale below touches only the per-pass copy
                L.acc = new if L.acc is None else [a + b for a, b in zip(L.acc, new)]
        scale = float(n * n)
        if L.is_diag:
            L.data = [d * scale for d in new]
        else:
            L.data = [L.A, new[0] * scale]

    # -- closure (fisher/__init__.py:50-88) ----------------------------------
    def _closure(self, data, target, mc_targets=None, approx='mc'):
        for L in self.layers:
            for p in L.params:
                p.grad = None
        out = self.model(data)
        if self.curv_type == 'Fisher':
            prob = F.softmax(out, dim=1)
            for L in self.layers:
                for p in L.params:
                    p.requires_grad = False
            self.sampling = True
            if approx == 'mc':
                num_mc = mc_targets.shape[0]
                self.prob = torch.ones_like(prob[:, 0]) / num_mc
                for i in range(num_mc):
                    F.cross_entropy(out, mc_targets[i]).backward(retain_graph=True)
            else:
                for i in range(out.shape[1]):
                    self.prob = prob[:, i].detach()
                    F.cross_entropy(out, torch.full_like(target, i)).backward(retain_graph=True)
            self.sampling = False
            for L in self.layers:
                for p in L.params:
                    p.requires_grad = True
        loss = F.cross_entropy(out, target)
        loss.backward()
        return loss.detach(), out.detach()

    # -- step (secondorder.py:158-231) ---------------------------------------
    def step(self, data, target, mc_targets=None, approx='mc'):
        loss, out = self._closure(data, target, mc_targets, approx)
        n = self.acc_steps
        grads = [[p.grad.detach() / n for p in L.params] for L in self.layers]
        curv = [[d / n for d in L.data] for L in self.layers]
        if self._acc_grads is None:
            self._acc_grads, self._acc_curv = grads, curv
        else:
            self._acc_grads = [[a + b for a, b in zip(x, y)] for x, y in zip(self._acc_grads, grads)]
            self._acc_curv = [[a + b for a, b in zip(x, y)] for x, y in zip(self._acc_curv, curv)]
        self.acc_step += 1
        if self.acc_step < n:
            return loss, out
        self.acc_step = 0
        for L, g, c in zip(self.layers, self._acc_grads, self._acc_curv):
            for p, gi in zip(L.params, g):
                p.grad = gi.clone()
            L.data = c
        self._acc_grads = self._acc_curv = None
        self.apply_update()
        return loss, out

    def apply_update(self, layer_filter: Optional[Callable[[int], bool]] = None):
        """Curvature step + precondition + parameter update for every (owned) layer."""
        self.steps += 1
        for idx, L in enumerate(self.layers):
            if layer_filter is not None and not layer_filter(idx):
                continue
            with torch.no_grad():
                # secondorder.py:233-307: raw stage, curvature step, preconditioned stage, update
                self._preprocess(L, 'raw')
                self.curvature_step(L)
                self.precondition(L)
                self._preprocess(L, 'preconditioned')
                for p in L.params:
                    p.data.add_(p.grad, alpha=-self.lr)
                if self.normalizing_weights:
                    # secondorder.py:309-330: the module's ``weight`` only, rescaled to a fixed norm
                    w = getattr(L.module, 'weight', None)
                    for p in L.params:
                        if w is not None and p is w and p.data.norm() > 1e-2:
                            scale = self.weight_scale
                            if scale is None:
                                scale = math.sqrt(2.0 * w.shape[0])
                            p.data.div_(p.data.norm() + 1e-9).mul_(scale)

    def _preprocess(self, L: _Layer, stage: str):
        """secondorder.py:233-307 for one stage ('raw' before the curvature step, 'preconditioned'
        after): l2 / weight decay, momentum, LARS, in the reference's order."""
        for p, buf in zip(L.params, L.momentum_buf):
            if stage == 'raw' and self.l2_reg != 0:
                p.grad.add_(p.data, alpha=self.l2_reg)
                L.l2_reg = self.l2_reg
            if stage == 'preconditioned' and self.weight_decay != 0:
                p.grad.add_(p.data, alpha=self.weight_decay)
            if self.momentum_type == stage and self.momentum != 0:
                buf.mul_(self.momentum).add_(p.grad)
                p.grad.copy_(buf)
            if self.lars and self.lars_type == stage:
                d_norm = p.data.norm()
                if d_norm > 1e-2:
                    p.grad.mul_(d_norm / (p.grad.norm() + 1e-9))

    def curvature_step(self, L: _Layer):
        """curvature.py:166-191 (EMA incl. the l2 term) then :302-312 / :226-232."""
        first = L.ema is None
        L.ema = [ko.ema_update(d, None if first else e, self.beta)
                 for d, e in zip(L.data, L.ema or [None] * len(L.data))]
        if first or self.beta == 1:
            L.l2_reg_ema = L.l2_reg
        else:
            L.l2_reg_ema = L.l2_reg * self.beta + L.l2_reg_ema * (1 - self.beta)
        if self.use_max_ema:
            # curvature.py:180-191: running element-wise maximum of the EMA
            if getattr(L, 'ema_max', None) is None:
                L.ema_max = [e.clone() for e in L.ema]
            L.ema_max = [torch.maximum(e, m) for e, m in zip(L.ema, L.ema_max)]
        if not self.update_inv:
            return
        damping = self.damping + L.l2_reg_ema
        if L.is_diag:
            # curvature.py:193-195: the diagonal classes invert the maximum when asked to; the
            # Kronecker update_inv (:302-312) always reads the EMA itself
            src = L.ema_max if self.use_max_ema else L.ema
            L.inv = [ko.diag_inverse(e, damping) for e in src]
        else:
            L.inv = list(ko.kron_damped_inverse(L.ema[0], L.ema[1], damping))

    def precondition(self, L: _Layer):
        if L.is_diag:
            for p, inv in zip(L.params, L.inv):
                p.grad.copy_(inv * p.grad)
            return
        gw = L.params[0].grad
        gb = L.params[1].grad if L.has_bias else None
        pw, pb = ko.kron_precondition(L.inv[0], L.inv[1], gw, gb)
        gw.copy_(pw)
        if gb is not None:
            gb.copy_(pb)


class OracleVI(OracleKFAC):
    """Noisy-K-FAC variational step, torchsso/optim/vi.py:50-258: a Gaussian posterior whose
    mean is updated with the preconditioned gradient averaged over ``num_mc_samples`` weight
    draws  theta = mean + s * U_G E U_A  (Kron) or  mean + s * e * sigma  (Diag).
    ``noise_fn(shape)`` supplies the standard-normal draws in call order."""

    def __init__(self, model, dataset_size, noise_fn, num_mc_samples=10, kl_weighting=1.0,
                 prior_variance=1.0, **kw):
        l2 = kl_weighting / dataset_size / prior_variance if prior_variance != 0 else 0
        super().__init__(model, l2_reg=l2, **kw)
        self.std_scale = math.sqrt(kl_weighting / dataset_size) if l2 != 0 else 0.0
        self.num_mc = num_mc_samples
        self.noise_fn = noise_fn
        for L in self.layers:
            L.mean = [p.detach().clone() for p in L.params]

    def sample_params(self):
        with torch.no_grad():
            for L in self.layers:
                if L.std is None:
                    for p, m in zip(L.params, L.mean):
                        p.copy_(m)
                elif L.is_bn:
                    for p, m, s in zip(L.params, L.mean, L.std):
                        p.copy_(ko.diag_sample(m, s, self.noise_fn(tuple(m.shape)), self.std_scale))
                else:
                    mw = L.mean[0]
                    mb = L.mean[1] if L.has_bias else None
                    cols = mw[0].numel() + (1 if L.has_bias else 0)
                    noise = self.noise_fn((mw.shape[0], cols))
                    w, b = ko.kron_sample(mw, mb, L.std[0], L.std[1], noise, self.std_scale)
                    L.params[0].copy_(w)
                    if b is not None:
                        L.params[1].copy_(b)

    def step(self, data, target):
        m = self.num_mc
        loss_acc, prob_acc = 0.0, 0.0
        grads = curv = None
        for _ in range(m):
            self.sample_params()
            loss, out = self._closure(data, target)
            loss_acc = loss_acc + loss / m
            prob_acc = prob_acc + F.softmax(out, dim=1)
            g = [[p.grad.detach() / m for p in L.params] for L in self.layers]
            c = [[d / m for d in L.data] for L in self.layers]
            if grads is None:
                grads, curv = g, c
            else:
                grads = [[a + b for a, b in zip(x, y)] for x, y in zip(grads, g)]
                curv = [[a + b for a, b in zip(x, y)] for x, y in zip(curv, c)]
        self.steps += 1
        with torch.no_grad():
            for L, g, c in zip(self.layers, grads, curv):
                L.data = c
                g = [gi.clone() for gi in g]
                if self.l2_reg != 0:
                    for gi, mu in zip(g, L.mean):
                        gi.add_(mu, alpha=self.l2_reg)
                    L.l2_reg = self.l2_reg
                self.update_inv = True
                self.curvature_step(L)
                if self.std_scale > 0:
                    # curvature.py:240-241 (Diag: sqrt of inverse) and :317-321 (Kron: upper
                    # Cholesky factor of each inverse)
                    L.std = ([i.sqrt() for i in L.inv] if L.is_bn
                             else [ko.cholesky_upper(i) for i in L.inv])
                if L.is_bn:
                    g = [inv * gi for inv, gi in zip(L.inv, g)]
                else:
                    pw, pb = ko.kron_precondition(L.inv[0], L.inv[1], g[0],
                                                  g[1] if L.has_bias else None)
                    g = [pw] + ([pb] if L.has_bias else [])
                for mu, gi, buf, p in zip(L.mean, g, L.momentum_buf, L.params):
                    if self.weight_decay != 0:
                        gi = gi + self.weight_decay * mu
                    if self.momentum != 0:
                        buf.mul_(self.momentum).add_(gi)
                        gi = buf.clone()
                    mu.add_(gi, alpha=-self.lr)
                    p.copy_(mu)
                    p.grad = gi.clone()
        return loss_acc, prob_acc
