"""SecondOrderOptimizer / DistributedSecondOrderOptimizer with the constructor, attributes and
step protocol of torchsso/optim/secondorder.py:15-392, re-organised around flat device pools:

* all gradients live in one fp32 buffer (``p.grad`` are views into it), all curvature tensors in
  the FactorPool, so accumulation, EMA, inversion and preconditioning are a handful of launches
  per step instead of a Python loop over ~100 layers with several small kernels each;
* the per-group hyper-parameter logic (l2 / weight decay / momentum / gradient EMA / bias
  correction / LARS / weight normalisation) is unchanged in meaning and applied with
  multi-tensor ops over groups that share the same settings.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import List

import numpy as np
import torch
import torch.nn as nn
from torch.optim import Optimizer

import torchsso
from torchsso import _native as nat
from torchsso.curv.layers import _KronFactors, _DiagBatchNorm
from torchsso.curv.pool import FactorPool
from torchsso.utils import TensorAccumulator

_NORM_TYPES = (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)


def _is_pooled(curv) -> bool:
    return isinstance(curv, (_KronFactors, _DiagBatchNorm)) and not curv.use_max_ema


class SecondOrderOptimizer(Optimizer):
    r"""Second-order optimizer: one param_group per leaf module that has parameters, each with a
    ``torchsso.Curvature`` looked up as ``curv_shapes[module class] + curv_type + module class``.

    Arguments are those of the reference class (same names, defaults and validation).

    Example:
        >>> curv_shapes = {"Conv2d": "Kron", "Linear": "Kron", "BatchNorm2d": "Diag"}
        >>> curv_kwargs = {"damping": 1e-3, "ema_decay": 0.999}
        >>> optimizer = torchsso.optim.SecondOrderOptimizer(model, "Cov", curv_shapes, curv_kwargs)
        >>> def closure():
        >>>    optimizer.zero_grad()
        >>>    output = model(data)
        >>>    loss = F.cross_entropy(output, target)
        >>>    loss.backward()
        >>>    return loss, output
        >>> optimizer.step(closure=closure)
    """

    def __init__(self, model: nn.Module, curv_type: str, curv_shapes: dict, curv_kwargs: dict,
                 lr=0.01, momentum=0., momentum_type='preconditioned',
                 grad_ema_decay=1., grad_ema_type='raw', l2_reg=0., weight_decay=0.,
                 normalizing_weights=False, weight_scale=None,
                 acc_steps=1, non_reg_for_bn=False, bias_correction=False,
                 lars=False, lars_type='preconditioned', update_inv=True, precondition_grad=True):

        if lr < 0:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if momentum < 0:
            raise ValueError("Invalid momentum: {}".format(momentum))
        if momentum > 0 and momentum_type not in ['raw', 'preconditioned']:
            raise ValueError("Invalid momentum type: {}".format(momentum_type))
        if grad_ema_decay < 0 or 1 < grad_ema_decay:
            raise ValueError("Invalid grad_ema value: {}".format(grad_ema_decay))
        if grad_ema_decay > 0 and grad_ema_type not in ['raw', 'preconditioned']:
            raise ValueError("Invalid grad_ema type: {}".format(grad_ema_type))
        if l2_reg < 0:
            raise ValueError("Invalid l2_reg value: {}".format(l2_reg))
        if weight_decay < 0:
            raise ValueError("Invalid weight_decay value: {}".format(weight_decay))
        if acc_steps < 1:
            raise ValueError("Invalid acc_steps: {}".format(acc_steps))
        if lars and lars_type not in ['raw', 'preconditioned']:
            raise ValueError("Invalid LARS type: {}".format(lars_type))
        if normalizing_weights and weight_scale is not None and weight_scale <= 0:
            raise ValueError("Invalid weight scale for LARS: {}".format(weight_scale))

        self.model = model
        defaults = {'lr': lr, 'momentum': momentum, 'momentum_type': momentum_type,
                    'grad_ema_decay': grad_ema_decay, 'grad_ema_type': grad_ema_type,
                    'l2_reg': l2_reg, 'weight_decay': weight_decay,
                    'normalizing_weights': normalizing_weights, 'weight_scale': weight_scale,
                    'acc_steps': acc_steps, 'bias_correction': bias_correction,
                    'lars': lars, 'lars_type': lars_type}
        defaults.update(curv_kwargs)
        self.curv_type = curv_type
        self.curv_shapes = {} if curv_shapes is None else curv_shapes
        self.update_inv = update_inv
        self.precondition_grad = precondition_grad
        self.optim_state = {'step': 0, 'acc_step': 0}

        groups = []
        for module in model.modules():
            if len(list(module.children())) > 0:
                continue
            params = list(module.parameters())
            if len(params) == 0:
                continue
            curvature = self.get_curv_class(module)(module, **curv_kwargs)
            group = {'params': params, 'curv': curvature,
                     'acc_curv': TensorAccumulator(), 'acc_grads': TensorAccumulator()}
            if non_reg_for_bn and isinstance(module, _NORM_TYPES):
                group['l2_reg'] = 0
                group['weight_decay'] = 0
                group['normalizing_weights'] = False
            groups.append(group)
        if not groups:
            raise ValueError('model has no parameters')
        super(SecondOrderOptimizer, self).__init__(groups, defaults)
        for group in self.param_groups:
            self.init_buffer(group['params'])
        self._build_storage()

    # ------------------------------------------------------------------ construction helpers
    def init_buffer(self, params):
        for p in params:
            state = self.state[p]
            state['momentum_buffer'] = torch.zeros_like(p.data)
            state['grad_ema_buffer'] = torch.zeros_like(p.data)

    def get_curv_class(self, module):
        module_name = module.__class__.__name__
        curv_shape = self.curv_shapes.get(module_name, '')
        curv_name = curv_shape + self.curv_type + module_name
        curv_class = getattr(torchsso, curv_name, None)
        assert curv_class is not None, f"Failed to lookup Curvature class {curv_name} for {module}."
        return curv_class

    def _group_order(self) -> List[int]:
        """Order in which groups are laid out in the pools (owner-major when distributed)."""
        return list(range(len(self.param_groups)))

    def _build_storage(self):
        groups = [self.param_groups[i] for i in self._group_order()]
        device = groups[0]['params'][0].device
        kron = [g for g in groups if isinstance(g['curv'], _KronFactors) and _is_pooled(g['curv'])]
        diag = [g for g in groups if isinstance(g['curv'], _DiagBatchNorm) and _is_pooled(g['curv'])]
        taken = {id(g) for g in kron} | {id(g) for g in diag}
        rest = [g for g in groups if id(g) not in taken]
        self.pool = FactorPool([g['curv'] for g in kron], [g['curv'] for g in diag], device)
        # flat fp32 gradient buffer: Kronecker layers, then diagonal layers in the diagonal
        # pool's own element order, then everything else
        views, off = OrderedDict(), 0
        for g in kron:
            for p in g['params']:
                views[p] = (off, p.numel())
                off += p.numel()
        self._diag_grad_base = off
        for g in diag:
            for p in g['params']:
                views[p] = (off, p.numel())
                off += p.numel()
        for g in rest:
            for p in g['params']:
                views[p] = (off, p.numel())
                off += p.numel()
        self._grad_flat = torch.zeros(off, dtype=torch.float32, device=device)
        self._grad_acc = None
        self._grad_view = {p: self._grad_flat[o:o + n].view(p.shape) for p, (o, n) in views.items()}
        self._grad_slot = views
        self._acc_first = True

    # ------------------------------------------------------------------ gradients
    @property
    def local_param_groups(self):
        return self.param_groups

    @property
    def fuse_ema(self):
        """Write ``ema <- decay * new + (1 - decay) * ema`` in the epilogue of the kernels that build
        the curvature (factor, BatchNorm), instead of storing ``data`` and streaming ``data -> ema``
        over all factors once per step (torchsso/curv/curvature.py:174-191).  Off by default because
        it changes the hooks' contract: ``curv.data`` is no longer produced, and every closure call
        that runs a backward pass must be followed by exactly one ``step()`` (evaluation forwards under
        ``no_grad`` are ignored).  Needs ``acc_steps == 1``, a single process, and curvatures that
        share one ``ema_decay``."""
        return self.__dict__.get('_fuse_ema', False)

    @fuse_ema.setter
    def fuse_ema(self, on):
        curvs = [g['curv'] for g in self.param_groups]
        if on:
            if self.defaults['acc_steps'] != 1 or type(self).backward_postprocess is not SecondOrderOptimizer.backward_postprocess:
                raise ValueError('fuse_ema needs acc_steps == 1 and a single process: accumulation and the '
                                 'owner-rank exchange carry curv.data')
            if not all(c is not None and _is_pooled(c) for c in curvs) or len({c.ema_decay for c in curvs}) > 1:
                raise ValueError('fuse_ema needs Kronecker / BatchNorm curvatures with one common ema_decay')
        nat.join_curvature_stream(None)
        for c in curvs:
            if c is not None:
                c._fuse_ema = bool(on)
                if on:
                    c._have.discard('data')
        self.__dict__['_fuse_ema'] = bool(on)

    @property
    def early_inverse(self):
        """Start the round of damped inverses inside the Fisher closure, as soon as its sampling passes
        have finished: with ``fuse_ema`` the running averages of A and G are complete at that point and
        the real backward pass that follows only produces gradients, so the inverses (issued on the
        curvature stream when that is enabled) run beside it instead of after it.  Same matrices, same
        step as ``torchsso/optim/secondorder.py:195-209`` inverts; only the place in the stream
        changes.  Needs ``fuse_ema`` and ``l2_reg == 0`` (the damping must not depend on this step's
        bookkeeping).  Closures not built by ``get_closure_for_fisher`` are unaffected."""
        return self.__dict__.get('_early_inverse', False)

    @early_inverse.setter
    def early_inverse(self, on):
        if on:
            if not self.fuse_ema:
                raise ValueError('early_inverse needs fuse_ema: the running averages must be complete inside the closure')
            if any(g['l2_reg'] != 0 for g in self.param_groups):
                raise ValueError('early_inverse needs l2_reg == 0')
        self.__dict__['_early_inverse'] = bool(on)

    def _after_sampling_passes(self):
        if not (self.early_inverse and self.update_inv):
            return
        kc = [g['curv'] for g in self.local_param_groups
              if isinstance(g['curv'], _KronFactors) and _is_pooled(g['curv'])]
        if not kc:
            return
        nat.flush_factors()
        nat.run_on_curvature_stream(lambda _: self.pool.update_inv(kc, with_std=False), self._grad_flat)
        self.__dict__['_early_inverse_done'] = True

    #: what ``zero_grad()`` does when called without an argument (as the closures do).  True (torch's
    #: own default): set every ``p.grad`` to None, autograd assigns its own tensors and one
    #: multi-tensor copy after the closure brings them into the flat buffer (100 MB more memory for
    #: ResNet-50).  False: zero the flat buffer and bind every ``p.grad`` to its view of it, autograd
    #: accumulates in place (one small add kernel per parameter in every backward pass; ResNet-50:
    #: 0.3 ms per step slower).
    zero_grad_to_none = True

    def zero_grad(self, set_to_none=None):
        """Zero the flat gradient buffer.  Parameters that are fp32 and contiguous get ``p.grad``
        bound to their view of it, so autograd accumulates in place; others (channels_last
        weights, 16-bit parameters) get ``None`` and are copied in after the backward pass.
        With ``set_to_none`` every parameter is treated like the latter."""
        if set_to_none is None:
            set_to_none = self.zero_grad_to_none
        if set_to_none:
            for p in self._grad_view:
                if p.grad is not None:
                    p.grad = None
            return
        self._grad_flat.zero_()
        for p, v in self._grad_view.items():
            if p.dtype == torch.float32 and p.is_contiguous():
                if p.grad is not v:
                    p.grad = v
            elif p.grad is not None:
                p.grad = None

    def _harvest_grads(self):
        """Make sure the flat buffer holds this closure's gradients and that every ``p.grad`` is
        its view of the buffer (one multi-tensor copy for gradients that live elsewhere)."""
        dsts, srcs = [], []
        for p, v in self._grad_view.items():
            g = p.grad
            if g is None:
                v.zero_()
            elif g.data_ptr() != v.data_ptr() or g.dtype != torch.float32:
                dsts.append(v)
                srcs.append(g)
            if g is not v:
                p.grad = None
        if dsts:
            torch._foreach_copy_(dsts, srcs)
        for p, v in self._grad_view.items():
            if p.grad is None:
                p.grad = v

    def _accumulate(self, scale: float):
        if self._grad_acc is None:
            self._grad_acc = torch.zeros_like(self._grad_flat)
        first = self._acc_first
        nat.axpby(self._grad_flat, self._grad_acc, scale, 0.0 if first else 1.0)
        self.pool.accumulate(scale, first)
        for group in self.param_groups:
            curv = group['curv']
            if curv is not None and not _is_pooled(curv) and curv.data is not None:
                group['acc_curv'].update(curv.data, scale=scale)
        self._acc_first = False

    def _take_accumulated(self, target='params'):
        nat.axpby(self._grad_acc, self._grad_flat, 1.0, 0.0)
        self.pool.take_accumulated()
        for group in self.param_groups:
            curv = group['curv']
            if curv is not None and not _is_pooled(curv):
                acc = group['acc_curv'].get()
                if acc is not None:
                    curv.data = acc
        self._acc_first = True

    # ------------------------------------------------------------------ step
    def step(self, closure=None):
        """One optimisation step.  ``closure`` does forward + backward and returns
        ``(loss, output)``; its return value is passed through."""
        n = self.defaults['acc_steps']
        loss = None
        if closure is not None:
            loss = closure()
            nat.join_curvature_stream(None)
            self._harvest_grads()
            if n > 1:
                self._accumulate(1.0 / n)
            self.optim_state['acc_step'] += 1
            if self.optim_state['acc_step'] < n:
                return loss
            self.optim_state['acc_step'] = 0
            self.backward_postprocess()

        self.optim_state['step'] += 1
        self._update_groups(self.local_param_groups, 'params', self.update_inv, None)
        return loss

    def backward_postprocess(self, target='params'):
        if self.defaults['acc_steps'] > 1 or not self._acc_first:
            self._take_accumulated(target)
        self._bind_grads(target)

    def _bind_grads(self, target):
        if target == 'params':
            return
        for group in self.param_groups:
            for p, t in zip(group['params'], group[target]):
                t.grad = self._grad_view[p]

    def _update_groups(self, groups, target, update_inv, update_std):
        """raw preprocess -> curvature step -> precondition -> preconditioned preprocess -> update.
        Groups whose tensors are flat fp32 run each of the two preprocess stages (and the update) as
        one launch of the fused tail kernel; the others take the per-group multi-tensor path."""
        fused = self._fused_tail(groups, target, 'raw')
        for group in groups:
            if id(group) not in fused:
                self.update_preprocess(group, target=target, grad_type='raw')
        self._curvature_step(groups, target, update_inv, update_std)
        fused = self._fused_tail(groups, target, 'preconditioned')
        rest = [g for g in groups if id(g) not in fused]
        for group in rest:
            self.update_preprocess(group, target=target, grad_type='preconditioned')
        self._apply_update(rest, target)
        for group in groups:
            self.update_postprocess(group, target=target)

    def _fused_tail(self, groups, target, stage):
        """torchsso/optim/secondorder.py:225-283 for all eligible groups in one kernel launch.
        Returns the ids of the groups it handled."""
        raw = stage == 'raw'
        items, key, handled = [], [], set()
        for group in groups:
            if group['lars']:
                continue                      # needs per-tensor norms: multi-tensor path
            params = [p for p in group[target] if p.grad is not None]
            if not params or any(p.dtype != torch.float32 or p.grad.dtype != torch.float32 or
                                 not p.data.is_contiguous() or not p.grad.is_contiguous() for p in params):
                continue
            add = group['l2_reg'] if raw else group['weight_decay']
            use_m = group['momentum'] != 0 and group['momentum_type'] == stage
            use_e = group['grad_ema_decay'] != 1 and group['grad_ema_type'] == stage
            scale = 1.0
            if not raw and group['bias_correction']:
                curv = group['curv']
                bc1 = 1 - (1 - group['grad_ema_decay']) ** self.optim_state['step']
                bc2 = 1 - (1 - curv.ema_decay) ** self.optim_state['step']
                if getattr(curv, 'use_sqrt_ema', False):
                    bc2 = math.sqrt(bc2)
                scale = bc2 / bc1
            lr = 0.0 if raw else group['lr']
            handled.add(id(group))
            if raw and group['l2_reg'] != 0 and group['curv'] is not None:
                group['curv'].l2_reg = group['l2_reg']
            if raw and add == 0 and not use_m and not use_e:
                continue                      # nothing to apply at this stage
            for p in params:
                st = self.state[p]
                items.append((p.data, p.grad, st['momentum_buffer'] if use_m else None,
                              st['grad_ema_buffer'] if use_e else None, float(add), float(group['momentum']),
                              float(group['grad_ema_decay']), float(scale), float(lr)))
                key.append((p.data.data_ptr(), p.grad.data_ptr(), use_m, use_e, add, group['momentum'],
                            group['grad_ema_decay'], scale, lr))
        if items:
            cache = self.__dict__.setdefault('_tail_tables', {})
            ent = cache.get((target, stage))
            key = tuple(key)
            if ent is None or ent[0] != key:
                ent = (key, nat.tail_records(items, items[0][0].device))
                cache[(target, stage)] = ent
            nat.optimizer_tail(ent[1])
        return handled

    def _curvature_step(self, groups, target, update_inv, update_std):
        pooled = [g for g in groups if g['curv'] is not None and _is_pooled(g['curv'])]
        kron = [g for g in pooled if isinstance(g['curv'], _KronFactors)]
        diag = [g for g in pooled if isinstance(g['curv'], _DiagBatchNorm)]
        curvs = [g['curv'] for g in pooled]
        uniform = len({(c.ema_decay, 'ema' in c._have) for c in curvs}) <= 1
        if pooled and uniform:
            firsts = [c._ema_bookkeeping() for c in curvs]
            if not self.fuse_ema:        # else the hooks' kernels have already written the average
                self.pool.update_ema(curvs[0].ema_decay, firsts[0], [g['curv'] for g in kron],
                                     [g['curv'] for g in diag])
            for c in curvs:
                c._have.add('ema')
        else:
            for c in curvs:
                c.update_ema()
        early = self.__dict__.pop('_early_inverse_done', False)     # consumed by this step whatever it does
        kc = [g['curv'] for g in kron]
        if kc:
            want_std = [bool(update_std(g)) if update_std else False for g in kron]
            if update_inv:
                if not (early and not any(want_std)):      # else: issued inside the closure already
                    self.pool.update_inv(kc, with_std=any(want_std))
                for c in kc:
                    c._have.add('inv')
                    if any(want_std):
                        c._have.add('std')
            if self.precondition_grad or target != 'params':
                grads = [[self._grad_view[p] for p in g['params']] for g in kron]
                self.pool.precondition(kc, grads)
        if diag:
            dc = [g['curv'] for g in diag]
            lo, hi = self.pool.diag_range(dc)
            gflat = None
            if self.precondition_grad or target != 'params':
                gflat = self._grad_flat[self._diag_grad_base + lo: self._diag_grad_base + hi]
            uniform_d = len({(c.damping, c.use_sqrt_ema) for c in dc}) <= 1
            if uniform_d:
                self.pool.diag_step(dc, gflat, bool(update_inv))
            else:
                for c in dc:
                    l, h = self.pool.diag_range([c])
                    gf = None if gflat is None else self._grad_flat[self._diag_grad_base + l:
                                                                     self._diag_grad_base + h]
                    self.pool.diag_step([c], gf, bool(update_inv))
            for g in diag:
                c = g['curv']
                if update_inv:
                    c._have.add('inv')
                    if update_std and update_std(g):
                        c.update_std()
        for g in groups:
            curv = g['curv']
            if curv is None or _is_pooled(curv):
                continue
            curv.step(update_inv=bool(update_inv),
                      update_std=bool(update_std(g)) if update_std else False)
            if self.precondition_grad or target != 'params':
                curv.precondition_grad(g[target])

    def _apply_update(self, groups, target):
        by_lr = {}
        for group in groups:
            ts, gs = by_lr.setdefault(group['lr'], ([], []))
            for p in group[target]:
                if p.grad is None:
                    continue
                ts.append(p.data)
                gs.append(p.grad if p.grad.dtype == p.dtype else p.grad.to(p.dtype))
        for lr, (ts, gs) in by_lr.items():
            if ts:
                torch._foreach_add_(ts, gs, alpha=-lr)

    def update(self, group, target='params'):
        for p in group[target]:
            if p.grad is None:
                continue
            p.data.add_(p.grad.to(p.dtype), alpha=-group['lr'])

    def update_preprocess(self, group, target='params', grad_type='raw'):
        assert grad_type in ['raw', 'preconditioned'], 'Invalid grad type: {}.'.format(grad_type)
        raw = grad_type == 'raw'
        if not ((raw and group['l2_reg'] != 0) or (not raw and group['weight_decay'] != 0) or
                (group['momentum'] != 0 and group['momentum_type'] == grad_type) or
                (group['grad_ema_decay'] != 1 and group['grad_ema_type'] == grad_type) or
                (not raw and group['bias_correction']) or (group['lars'] and group['lars_type'] == grad_type)):
            return      # nothing to apply for this group at this stage
        params = [p for p in group[target] if p.grad is not None]
        if not params:
            return
        state = self.state
        grads = [p.grad for p in params]
        datas = [p.data for p in params]

        if grad_type == 'raw' and group['l2_reg'] != 0:
            torch._foreach_add_(grads, datas, alpha=group['l2_reg'])
            if group['curv'] is not None:
                group['curv'].l2_reg = group['l2_reg']

        if grad_type == 'preconditioned' and group['weight_decay'] != 0:
            torch._foreach_add_(grads, datas, alpha=group['weight_decay'])

        if group['momentum_type'] == grad_type and group['momentum'] != 0:
            bufs = [state[p]['momentum_buffer'] for p in params]
            torch._foreach_mul_(bufs, group['momentum'])
            torch._foreach_add_(bufs, grads)
            torch._foreach_copy_(grads, bufs)

        if group['grad_ema_type'] == grad_type and group['grad_ema_decay'] != 1:
            d = group['grad_ema_decay']
            bufs = [state[p]['grad_ema_buffer'] for p in params]
            torch._foreach_mul_(bufs, 1 - d)
            torch._foreach_add_(bufs, grads, alpha=d)
            torch._foreach_copy_(grads, bufs)

        if grad_type == 'preconditioned' and group['bias_correction']:
            curv = group['curv']
            beta1 = 1 - group['grad_ema_decay']
            beta2 = 1 - curv.ema_decay
            bc1 = 1 - beta1 ** self.optim_state['step']
            bc2 = 1 - beta2 ** self.optim_state['step']
            if getattr(curv, 'use_sqrt_ema', False):
                bc2 = math.sqrt(bc2)
            torch._foreach_mul_(grads, bc2 / bc1)

        if group['lars_type'] == grad_type and group['lars']:
            for p, g in zip(params, grads):
                d_norm = p.data.norm()
                if d_norm > 1e-2:
                    g.mul_(d_norm / (g.norm() + 1e-9))

    def update_postprocess(self, group, target='params'):
        if not group['normalizing_weights']:
            return
        curv = group['curv']
        w = getattr(curv.module, 'weight', None) if curv is not None else None
        for p, _p in zip(group[target], group['params']):
            if w is not None and w is _p:
                d_norm = p.data.norm()
                if d_norm > 1e-2:
                    scale = group['weight_scale']
                    if scale is None:
                        scale = np.sqrt(2.0 * w.data.shape[0])
                    p.data.div_(d_norm + 1e-9).mul_(scale)


class DistributedSecondOrderOptimizer(SecondOrderOptimizer):
    """Data-parallel K-FAC (torchsso/optim/secondorder.py:333-392): every rank builds factors and
    gradients on its batch shard; ``reduce_scatterv_data`` delivers their world mean to each
    layer's owner rank; only the owner runs EMA / inverse / precondition / update for its layers;
    ``allgatherv_data`` returns the updated parameters to everyone.

    ``comm`` (keyword, optional): a torchsso.utils.KFACCommunicator; default wraps the default
    torch.distributed process group.  ``balance`` (keyword): 'contiguous' reproduces the
    reference's numpy.array_split ownership, 'inverse_cost' (default) balances sum(d_A^3 + d_G^3)
    per rank."""

    def __init__(self, *args, comm=None, balance='inverse_cost', **kwargs):
        from torchsso.utils.communicator import create_communicator, assign_owners
        self.comm = comm if comm is not None else create_communicator()
        self._balance = balance
        self._assign_owners = assign_owners
        self.actual_optimizer.__init__(self, *args, **kwargs)
        self.comm.setup(self)

    @property
    def actual_optimizer(self):
        return SecondOrderOptimizer

    def _group_order(self):
        costs = []
        for g in self.param_groups:
            shp = g['curv']._get_shape() if isinstance(g['curv'], _KronFactors) else None
            costs.append(0 if shp is None else shp[0][0] ** 3 + shp[1][0] ** 3)
        indices = self._assign_owners(costs, self.comm.size, self._balance)
        self.indices = indices
        self.local_indices = indices[self.comm.rank]
        self._local_param_groups = [self.param_groups[i] for i in self.local_indices]
        setattr(self.comm, 'indices', indices)
        return [i for part in indices for i in part]

    @property
    def local_param_groups(self):
        return self._local_param_groups

    def extractors_for_rsv(self):
        return ['grad', 'curv.data']

    def extractors_for_agv(self):
        return ['param.data']

    def backward_postprocess(self, target='params'):
        self.actual_optimizer.backward_postprocess(self, target)
        self.comm.reduce_scatterv_data(self.param_groups, self.extractors_for_rsv())

    def is_updated(self):
        return self.optim_state['acc_step'] == 0

    def step(self, closure=None):
        ret = self.actual_optimizer.step(self, closure)
        if self.is_updated():
            self.comm.allgatherv_data(self.param_groups, self.extractors_for_agv())
        return ret
