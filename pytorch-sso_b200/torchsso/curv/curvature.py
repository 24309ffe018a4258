"""Per-layer curvature objects: data -> ema -> inv (-> std).

Same public contract as the reference base classes (torchsso/curv/curvature.py:10-331):
constructor ``cls(module, ema_decay, damping, use_max_ema, use_sqrt_ema, pi_type)``,
attributes ``data / ema / inv / std / module / bias / damping / l2_reg / shape / device`` and
methods ``step / update_ema / update_inv / update_std / precondition_grad / sample_params /
std_norm / element_wise_init / adjust_data_scale``.  The storage and the arithmetic are not
the reference's: tensors are views into a FactorPool and every update is a launch of the
sm_100a kernels in libsso_b200 (no torch linear algebra, no CPU path).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import _native as nat
from .pool import FactorPool

PI_TYPE_TRACENORM = 'tracenorm'
_NORM_TYPES = (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)


class Curvature(object):
    """Curvature of one leaf module.  Hooks the module: the forward hook sees the layer input
    (and output), a tensor hook on the output delivers the output gradient during backward
    (torchsso/curv/curvature.py:55-56,118-155 use a module backward hook for the same value)."""

    def __init__(self, module: nn.Module, ema_decay=1., damping=1e-7,
                 use_max_ema=False, use_sqrt_ema=False, pi_type=PI_TYPE_TRACENORM):
        if ema_decay < 0 or 1 < ema_decay:
            raise ValueError("Invalid ema_decay: {}".format(ema_decay))
        if damping < 0:
            raise ValueError("Invalid damping: {}".format(damping))
        if pi_type not in [PI_TYPE_TRACENORM]:
            raise ValueError("Invalid pi_type: {}".format(pi_type))
        self._module = module
        self.ema_decay = ema_decay
        self._damping = damping
        self._l2_reg = 0
        self._l2_reg_ema = 0
        self.use_sqrt_ema = use_sqrt_ema
        self.use_max_ema = use_max_ema
        self.pi_type = pi_type
        self._pool = None
        self._fuse_ema = False      # hooks write the running average themselves (optimizer.fuse_ema)
        self._have = set()          # which of data / ema / inv / std hold values
        self._generic = {}          # storage for curvature shapes the pool does not manage
        self._is_norm = isinstance(module, _NORM_TYPES)
        module.register_forward_hook(self.forward_postprocess)

    # ---- identity ---------------------------------------------------------------
    @property
    def module(self):
        return self._module

    @property
    def device(self):
        return next(self._module.parameters()).device

    @property
    def bias(self):
        return getattr(self._module, 'bias', None) is not None

    @property
    def damping(self):
        return self._damping + self._l2_reg_ema

    @property
    def l2_reg(self):
        return self._l2_reg

    @l2_reg.setter
    def l2_reg(self, value):
        self._l2_reg = value

    @property
    def l2_reg_ema(self):
        return self._l2_reg_ema

    @property
    def shape(self):
        return self._get_shape()

    def _get_shape(self):
        size = sum(p.numel() for p in self._module.parameters())
        return ((size, size),)

    # ---- storage ----------------------------------------------------------------
    @property
    def pool(self) -> FactorPool:
        if self._pool is None:
            self._make_private_pool()
        return self._pool

    def _make_private_pool(self):
        raise NotImplementedError

    def _views(self, role):
        raise NotImplementedError

    def _get(self, role):
        nat.join_curvature_stream(None)
        if role in self._generic:
            return self._generic[role]
        return self._views(role) if role in self._have else None

    def _set(self, role, value):
        if value is None:
            self._have.discard(role)
            self._generic.pop(role, None)
            return
        for dst, src in zip(self._views(role), value):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        self._have.add(role)

    data = property(lambda self: self._get('data'), lambda self, v: self._set('data', v))
    ema = property(lambda self: self._get('ema'), lambda self, v: self._set('ema', v))
    ema_max = property(lambda self: self._get('ema_max'), lambda self, v: self._set('ema_max', v))
    inv = property(lambda self: self._get('inv'), lambda self, v: self._set('inv', v))
    std = property(lambda self: self._get('std'), lambda self, v: self._set('std', v))

    # ---- hooks ------------------------------------------------------------------
    def forward_postprocess(self, module, input, output):
        assert self._module is module
        x = input[0].detach()
        d = module.__dict__          # plain attributes; nn.Module.__setattr__ is slow on this hot path
        d['data_input'] = x
        d['data_output'] = output.detach()   # detached: keeping the graph alive between steps would
                                             # pin last step's activations and autograd nodes
        if self._fuse_ema and not (output.requires_grad and torch.is_grad_enabled()):
            return      # an evaluation forward must not advance a running average the hooks own
        if nat._batching:
            nat.note_phase('forward')
        nat.run_on_curvature_stream(self.update_in_forward, output.detach() if self._is_norm else x)
        d.pop('output_edge', None)
        if output.requires_grad and torch.is_grad_enabled():
            output.register_hook(self._backward_hook)
            if getattr(self, '_keep_output_edge', False):
                # where the output gradient enters the autograd graph (taken now: a later
                # in-place op would move the tensor to another node); the Fisher sampling passes
                # ask for exactly these gradients and nothing else.  The closure takes it away
                # again, so no graph stays alive between steps.
                d['output_edge'] = torch.autograd.graph.get_gradient_edge(output)

    def _backward_hook(self, grad_output):
        if self.__dict__.get('_mute_hook'):
            return      # a batched walk of the graph: its caller feeds the kernels slice by slice afterwards
        self.backward_postprocess(self._module, None, (grad_output,))

    def backward_postprocess(self, module, grad_input, grad_output):
        g = grad_output[0].detach()
        module.__dict__['grad_output'] = g
        if nat._batching:
            nat.note_phase('backward')
        # the n^2 rescale that undoes the mean reduction of the loss
        # (torchsso/curv/curvature.py:151-155) is folded into the kernels' alpha
        nat.run_on_curvature_stream(self.update_in_backward, g)

    def update_in_forward(self, data_input):
        pass

    def update_in_backward(self, grad_output):
        raise NotImplementedError

    def adjust_data_scale(self, scale):
        for d in self.data:
            d.mul_(scale)

    def element_wise_init(self, value):
        for d in self._views('data'):
            d.zero_()
            if d.dim() == 2:
                d.diagonal().fill_(value)
            else:
                d.fill_(value)
        self._have.add('data')

    # ---- data -> ema -> inv -> std ------------------------------------------------
    def step(self, update_std=False, update_inv=True):
        nat.join_curvature_stream(None)
        self.update_ema()
        if update_inv:
            self.update_inv()
        if update_std:
            self.update_std()

    def _ema_bookkeeping(self):
        """Scalar part of the EMA (the l2 term that later joins the damping,
        torchsso/curv/curvature.py:183,187).  Returns True if this is a (re)initialisation."""
        first = 'ema' not in self._have or self.ema_decay == 1
        beta = self.ema_decay
        if first:
            self._l2_reg_ema = self._l2_reg
        else:
            self._l2_reg_ema = self._l2_reg * beta + self._l2_reg_ema * (1 - beta)
        return first

    def update_ema(self):
        first = self._ema_bookkeeping()
        for d, e in zip(self._views('data'), self._views('ema')):
            nat.ema_update(d, e, self.ema_decay, first)
        self._have.add('ema')
        self._update_ema_max()

    def _update_ema_max(self):
        if not self.use_max_ema:
            return
        if 'ema_max' not in self._have:
            for e, m in zip(self._views('ema'), self._views('ema_max')):
                m.copy_(e)
            self._have.add('ema_max')
        else:
            for e, m in zip(self._views('ema'), self._views('ema_max')):
                torch.max(e, m, out=m)

    def update_inv(self):
        raise NotImplementedError

    def update_std(self):
        raise NotImplementedError

    def precondition_grad(self, params):
        raise NotImplementedError

    def sample_params(self, params, mean, std_scale):
        raise NotImplementedError

    def std_norm(self):
        raise NotImplementedError


class DiagCurvature(Curvature):
    """Diagonal curvature: one vector per parameter tensor."""

    def _get_shape(self):
        return tuple(p.shape for p in self.module.parameters())

    def _make_private_pool(self):
        FactorPool([], [self], self.device)

    def _views(self, role):
        return [self.pool.vec(role, self, j) for j in range(len(self._get_shape()))]

    def update_inv(self):
        self.pool.diag_step([self], None, True)
        self._have.add('inv')

    def precondition_grad(self, params):
        for p, inv in zip(params, self.inv):
            p.grad.mul_(inv)

    def update_std(self):
        for i, s in zip(self._views('inv'), self._views('std')):
            torch.sqrt(i, out=s)
        self._have.add('std')

    def sample_params(self, params, mean, std_scale):
        for p, m, std in zip(params, mean, self.std):
            noise = torch.randn_like(m)
            p.data.copy_(torch.addcmul(m, noise, std, value=std_scale))

    def std_norm(self):
        if self.std is None:
            return 0
        return sum(std.norm().item() for std in self.std)


class KronCurvature(Curvature):
    """Kronecker-factored curvature: data = [A, G]."""

    def __init__(self, *args, **kwargs):
        super(KronCurvature, self).__init__(*args, **kwargs)
        self._g_passes = 0      # backward passes accumulated into G since the last finalize

    def _make_private_pool(self):
        FactorPool([self], [], self.device)

    def _views(self, role):
        return [self.pool.mat(role, self, 0), self.pool.mat(role, self, 1)]

    @property
    def A(self):
        d = self.data
        return None if d is None else d[0]

    @property
    def G(self):
        d = self.data
        return None if d is None else d[1]

    def element_wise_init(self, value):
        super(KronCurvature, self).element_wise_init(math.sqrt(value))

    def adjust_data_scale(self, scale):
        self._views('data')[1].mul_(scale)

    def update_ema(self):
        first = self._ema_bookkeeping()
        lo, hi = self.pool.kron_range([self])
        nat.ema_update(self.pool.buf('data')[lo:hi], self.pool.buf('ema')[lo:hi], self.ema_decay, first)
        self._have.add('ema')
        self._update_ema_max()

    def update_inv(self):
        # always from the EMA: the reference's Kronecker update_inv ignores use_max_ema
        # (torchsso/curv/curvature.py:302-312 reads self.ema; only the base / diagonal classes
        # switch to ema_max, :193-195)
        self.pool.update_inv([self], with_std=False)
        self._have.add('inv')

    def update_std(self):
        self.pool.update_inv([self], with_std=True, do_inverse=False)
        self._have.add('std')

    def _grads_2d(self, params):
        """[dW (, db)] as fp32 contiguous tensors plus a flag telling whether they alias
        the parameters' .grad storage (so that no copy back is needed)."""
        out, alias = [], True
        for p in params:
            g = p.grad
            if g.dtype != torch.float32 or not g.is_contiguous():
                g = g.float().contiguous()
                alias = False
            out.append(g)
        return out, alias

    def precondition_grad(self, params):
        grads, alias = self._grads_2d(params)
        self.pool.precondition([self], [grads])
        if not alias:
            for p, g in zip(params, grads):
                p.grad.copy_(g)

    def sample_params(self, params, mean, std_scale):
        oc = mean[0].shape[0]
        cols = mean[0].numel() // oc + (1 if len(mean) > 1 else 0)
        noise = torch.randn_like(mean[0].new_empty((oc, cols)))
        tgt = []
        for p, m in zip(params, mean):
            p.data.copy_(m)
            assert p.data.is_contiguous() and p.data.dtype == torch.float32
            tgt.append(p.data)
        self.pool.sample([self], [tgt], [noise], float(std_scale))

    def std_norm(self):
        if self.std is None:
            return 0
        A_ic, G_ic = self.std
        return A_ic.norm().item() * G_ic.norm().item()
