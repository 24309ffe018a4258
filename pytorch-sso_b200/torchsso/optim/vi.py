"""VIOptimizer / VOGN / DistributedVIOptimizer with the interface of torchsso/optim/vi.py:11-351:
natural-gradient variational inference with a Gaussian posterior whose per-layer covariance is
the (Kronecker-factored or diagonal) inverse curvature.  Each step draws ``num_mc_samples``
weight samples  theta = mean + s * U_G E U_A,  accumulates gradients and curvature over them,
then updates the mean with the preconditioned gradient and refreshes inverse and Cholesky
factors.  Sampling for all Kronecker layers is one engine plan; accumulation runs on the flat
pools."""
from __future__ import annotations

import math

import torch

from torchsso import _native as nat
import torch.nn as nn
import torch.nn.functional as F

from torchsso.curv.layers import _KronFactors
from torchsso.optim.secondorder import (SecondOrderOptimizer, DistributedSecondOrderOptimizer,
                                        _is_pooled)
from torchsso.utils import TensorAccumulator


def _probabilities(output):
    if output.ndim == 2:
        return F.softmax(output, dim=1)
    if output.ndim == 1:
        return torch.sigmoid(output)
    raise ValueError(f'Invalid ndim {output.ndim}')


class VIOptimizer(SecondOrderOptimizer):
    r"""Variational-inference optimizer.  Arguments as in the reference class: ``dataset_size``
    scales the KL term (l2_reg = kl_weighting / dataset_size / prior_variance, sampling scale
    s = sqrt(kl_weighting / dataset_size)); ``num_mc_samples`` weight draws per step;
    ``init_precision`` optionally initialises the curvature to a multiple of the identity."""

    def __init__(self, model: nn.Module, dataset_size: float, curv_type: str, curv_shapes: dict,
                 curv_kwargs: dict, lr=0.01, momentum=0., momentum_type='preconditioned',
                 grad_ema_decay=1., grad_ema_type='raw', weight_decay=0.,
                 normalizing_weights=False, weight_scale=None,
                 acc_steps=1, non_reg_for_bn=False, bias_correction=False,
                 lars=False, lars_type='preconditioned',
                 num_mc_samples=10, val_num_mc_samples=10,
                 kl_weighting=1, warmup_kl_weighting_init=0.01, warmup_kl_weighting_steps=None,
                 prior_variance=1, init_precision=None,
                 seed=1, total_steps=1000):

        if dataset_size < 0:
            raise ValueError("Invalid dataset size: {}".format(dataset_size))
        if num_mc_samples < 1:
            raise ValueError("Invalid number of MC samples: {}".format(num_mc_samples))
        if val_num_mc_samples < 0:
            raise ValueError("Invalid number of MC samples for validation: {}".format(val_num_mc_samples))
        if kl_weighting < 0:
            raise ValueError("Invalid KL weighting: {}".format(kl_weighting))
        if warmup_kl_weighting_steps is not None and warmup_kl_weighting_init < 0:
            raise ValueError("Invalid initial KL weighting: {}".format(warmup_kl_weighting_init))
        if prior_variance < 0:
            raise ValueError("Invalid prior variance: {}".format(prior_variance))
        if init_precision is not None and init_precision < 0:
            raise ValueError("Invalid initial precision: {}".format(init_precision))

        init_kl = kl_weighting if warmup_kl_weighting_steps is None else warmup_kl_weighting_init
        l2_reg = init_kl / dataset_size / prior_variance if prior_variance != 0 else 0
        std_scale = math.sqrt(init_kl / dataset_size)

        super(VIOptimizer, self).__init__(model, curv_type, curv_shapes, curv_kwargs,
                                          lr=lr, momentum=momentum, momentum_type=momentum_type,
                                          grad_ema_decay=grad_ema_decay, grad_ema_type=grad_ema_type,
                                          l2_reg=l2_reg, weight_decay=weight_decay,
                                          normalizing_weights=normalizing_weights, weight_scale=weight_scale,
                                          acc_steps=acc_steps, non_reg_for_bn=non_reg_for_bn,
                                          bias_correction=bias_correction,
                                          lars=lars, lars_type=lars_type)

        self.defaults['std_scale'] = std_scale
        self.defaults['kl_weighting'] = kl_weighting
        self.defaults['warmup_kl_weighting_init'] = warmup_kl_weighting_init
        self.defaults['warmup_kl_weighting_steps'] = warmup_kl_weighting_steps
        self.defaults['num_mc_samples'] = num_mc_samples
        self.defaults['val_num_mc_samples'] = val_num_mc_samples
        self.defaults['total_steps'] = total_steps
        self.defaults['seed_base'] = seed
        self._noise = {}

        for group in self.param_groups:
            group['std_scale'] = 0 if group['l2_reg'] == 0 else std_scale
            group['mean'] = [p.data.detach().clone() for p in group['params']]
            self.init_buffer(group['mean'])
            if init_precision is not None:
                curv = group['curv']
                curv.element_wise_init(init_precision)
                curv.step(update_std=(group['std_scale'] > 0))

    def zero_grad(self, set_to_none=None):
        super(VIOptimizer, self).zero_grad(set_to_none)
        for group in self.param_groups:
            for m, p in zip(group['mean'], group['params']):
                if m.grad is not None and m.grad.data_ptr() != self._grad_view[p].data_ptr():
                    m.grad.detach_()
                    m.grad.zero_()

    @property
    def seed(self):
        return self.optim_state['step'] + self.defaults['seed_base']

    def set_random_seed(self, seed=None):
        if seed is None:
            seed = self.seed
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    def _noise_buf(self, group):
        key = id(group['curv'])
        buf = self._noise.get(key)
        if buf is None:
            mean = group['mean']
            oc = mean[0].shape[0]
            cols = mean[0].numel() // oc + (1 if len(mean) > 1 else 0)
            buf = torch.empty((oc, cols), dtype=torch.float32, device=mean[0].device)
            self._noise[key] = buf
        return buf

    def sample_params(self):
        """params <- a draw from the posterior (mean where a layer has no std yet).  Noise is
        drawn layer by layer in param_group order; all Kronecker layers are then transformed in
        one batched plan."""
        batches = {}
        for group in self.param_groups:
            params, mean, curv = group['params'], group['mean'], group['curv']
            if curv is None or curv.std is None:
                torch._foreach_copy_([p.data for p in params], mean)
                continue
            fast = (isinstance(curv, _KronFactors) and _is_pooled(curv) and
                    all(p.data.is_contiguous() and p.dtype == torch.float32 for p in params))
            if not fast:
                curv.sample_params(params, mean, group['std_scale'])
                continue
            buf = self._noise_buf(group)
            buf.copy_(torch.randn_like(buf))
            torch._foreach_copy_([p.data for p in params], mean)
            c, t, nz = batches.setdefault(float(group['std_scale']), ([], [], []))
            c.append(curv)
            t.append([p.data for p in params])
            nz.append(buf)
        for scale, (c, t, nz) in batches.items():
            self.pool.sample(c, t, nz, scale)

    def copy_mean_to_params(self):
        for group in self.param_groups:
            for p, m in zip(group['params'], group['mean']):
                p.data.copy_(m.data)
                if getattr(p, 'grad', None) is not None and getattr(m, 'grad', None) is not None \
                        and p.grad.data_ptr() != m.grad.data_ptr():
                    p.grad.copy_(m.grad)

    def adjust_kl_weighting(self):
        warmup_steps = self.defaults['warmup_kl_weighting_steps']
        if warmup_steps is None:
            return
        current_step = self.optim_state['step']
        if warmup_steps < current_step:
            return
        target_kl = self.defaults['kl_weighting']
        init_kl = self.defaults['warmup_kl_weighting_init']
        rate = current_step / warmup_steps
        kl_weighting = init_kl + rate * (target_kl - init_kl)
        rate = kl_weighting / init_kl
        l2_reg = rate * self.defaults['l2_reg']
        std_scale = math.sqrt(rate) * self.defaults['std_scale']
        for group in self.param_groups:
            if group['l2_reg'] > 0:
                group['l2_reg'] = l2_reg
            if group['std_scale'] > 0:
                group['std_scale'] = std_scale

    def step(self, closure=None):
        """closure() -> (loss, output); returns (mean loss over the MC samples, summed probabilities)."""
        m = self.defaults['num_mc_samples']
        n = self.defaults['acc_steps']
        acc_loss = TensorAccumulator()
        acc_prob = TensorAccumulator()
        self.set_random_seed()

        for _ in range(m):
            self.sample_params()
            loss, output = closure()
            nat.join_curvature_stream(None)
            acc_loss.update(loss.detach(), scale=1 / m)
            acc_prob.update(_probabilities(output.detach()), scale=1 / n)
            self._harvest_grads()
            self._accumulate(1 / m / n)

        loss, prob = acc_loss.get(), acc_prob.get()
        self.optim_state['acc_step'] += 1
        if self.optim_state['acc_step'] < n:
            return loss, prob
        self.optim_state['acc_step'] = 0

        self.backward_postprocess(target='mean')
        self.optim_state['step'] += 1
        groups = self.local_param_groups
        self._update_groups(groups, 'mean', True, lambda g: g['std_scale'] > 0)
        for group in groups:
            torch._foreach_copy_([p.data for p in group['params']], group['mean'])
        self.adjust_kl_weighting()
        return loss, prob

    def prediction(self, data, mc=None, keep_probs=False):
        self.set_random_seed(self.optim_state['step'])
        acc_prob = TensorAccumulator()
        probs = []
        mc_samples = self.defaults['val_num_mc_samples'] if mc is None else mc
        use_mean = mc_samples == 0
        n = 1 if use_mean else mc_samples
        for _ in range(n):
            if use_mean:
                self.copy_mean_to_params()
            else:
                self.sample_params()
            prob = _probabilities(self.model(data))
            acc_prob.update(prob, scale=1 / n)
            if keep_probs:
                probs.append(prob)
        self.copy_mean_to_params()
        prob = acc_prob.get()
        return (prob, probs) if keep_probs else prob


class VOGN(VIOptimizer):
    """VIOptimizer with the diagonal-curvature defaults of the reference (vi.py:302-319)."""

    def __init__(self, *args, **kwargs):
        default_kwargs = dict(lr=1e-3, curv_type='Cov',
                              curv_shapes={'Linear': 'Diag', 'Conv2d': 'Diag',
                                           'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'},
                              curv_kwargs={'ema_decay': 0.01, 'damping': 1e-7},
                              warmup_kl_weighting_init=0.01, warmup_kl_weighting_steps=1000,
                              grad_ema_decay=0.1, num_mc_samples=50, val_num_mc_samples=100)
        default_kwargs.update(kwargs)
        super(VOGN, self).__init__(*args, **default_kwargs)


class DistributedVIOptimizer(DistributedSecondOrderOptimizer, VIOptimizer):
    """MC-sample / data parallel VI: ranks of different ``mc_group_id`` use different seeds and
    therefore different weight draws; the factor exchange averages over data shards and MC
    samples alike (torchsso/optim/vi.py:322-351)."""

    def __init__(self, *args, mc_group_id=0, **kwargs):
        super(DistributedVIOptimizer, self).__init__(*args, **kwargs)
        self.defaults['seed_base'] += mc_group_id * self.defaults['total_steps']

    @property
    def actual_optimizer(self):
        return VIOptimizer

    def zero_grad(self, set_to_none=None):
        self.actual_optimizer.zero_grad(self, set_to_none)

    def extractors_for_rsv(self):
        return ['grad', 'curv.data']

    def extractors_for_agv(self):
        return ['mean.data', 'curv.std']

    def step(self, closure=None):
        ret = super(DistributedVIOptimizer, self).step(closure)
        if self.is_updated():
            self.copy_mean_to_params()
        return ret
