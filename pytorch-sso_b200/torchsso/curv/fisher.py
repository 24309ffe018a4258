"""Closure factory for Fisher curvatures (same protocol as
torchsso/curv/fisher/__init__.py:34-90): forward once, then one extra backward pass per Monte
Carlo target (or per class for the exact Fisher) that only the curvature hooks see, then the
real backward for the loss gradient.

The reference freezes the parameters for the sampling passes (requires_grad = False after the
forward), which still computes every weight gradient and drops it at the accumulation node.
Here a sampling pass asks autograd for the output gradients of the hooked modules only
(``prune_sampling_pass=True``, the default): the hooks see the same values, the weight-gradient
kernels of those passes never run.  ``prune_sampling_pass=False`` is the reference's protocol."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as nat
from .layers import Fisher

_APPROX_TYPE_MC = 'mc'


def sample_targets(prob: torch.Tensor, num_mc: int) -> torch.Tensor:
    """[num_mc, n] class indices drawn from the model's predictive distribution.
    A module-level function so that a parity harness can substitute a deterministic draw."""
    # same draw as torch.distributions.Categorical(prob).sample((num_mc,)) without the argument
    # validation, which synchronises with the host (and so cannot be captured in a CUDA graph).
    # A diverged model produces NaN / all-zero rows, on which the sampling kernel would fail a
    # device-side assertion and take the CUDA context with it: such rows are sampled uniformly
    # instead (the loss is already NaN and says so).
    prob = torch.nan_to_num(prob, nan=0.0, posinf=0.0, neginf=0.0).clamp_min(0.0)
    dead = prob.sum(dim=1, keepdim=True) <= 0
    prob = torch.where(dead, torch.ones_like(prob), prob)
    return torch.multinomial(prob, num_mc, replacement=True).t()


def get_closure_for_fisher(optimizer, model, data, target, approx_type=None, num_mc=1,
                           prune_sampling_pass=True):

    def set_sampling(on: bool):
        for group in optimizer.param_groups:
            curv = group['curv']
            if on:
                curv.turn_on_backward()
            else:
                curv.turn_off_backward()
            if not prune_sampling_pass:
                for param in group['params']:
                    param.requires_grad = not on

    def sampling_backward(loss, edges):
        if prune_sampling_pass:
            torch.autograd.grad(loss, edges, retain_graph=True, allow_unused=True)
        else:
            loss.backward(retain_graph=True)
        # with batched factor construction: this pass's G factors go to the device now, in one launch,
        # beside whatever the closure does next (the next pass accumulates onto them)
        nat.flush_factors()

    def closure():
        for group in optimizer.param_groups:
            assert isinstance(group['curv'], Fisher), f"Invalid Curvature type: {type(group['curv'])}."
        if approx_type is not None and approx_type != _APPROX_TYPE_MC:
            raise ValueError('Invalid approx type: {}'.format(approx_type))

        optimizer.zero_grad()
        output = model(data)
        nat.flush_factors()          # batched factor construction: all A factors of the forward pass
        prob = F.softmax(output, dim=1)

        edges = []
        if prune_sampling_pass:
            for group in optimizer.param_groups:
                edge = group['curv'].module.__dict__.pop('output_edge', None)
                if edge is not None:
                    edges.append(edge)
            if not edges:
                raise RuntimeError('no hooked module produced an output that requires grad')

        set_sampling(True)
        if approx_type == _APPROX_TYPE_MC:
            mc_targets = sample_targets(prob.detach(), num_mc)
            weight = torch.full_like(prob[:, 0], 1.0 / num_mc).detach()
            for group in optimizer.param_groups:
                group['curv'].prob = weight
                group['curv'].prob_scale = 1.0 / num_mc
            for i in range(num_mc):
                sampling_backward(F.cross_entropy(output, mc_targets[i]), edges)
        else:
            for i in range(model.num_classes):
                weight = prob[:, i].detach().float().contiguous()
                for group in optimizer.param_groups:
                    group['curv'].prob = weight
                    group['curv'].prob_scale = None
                sampling_backward(F.cross_entropy(output, torch.full_like(target, i)), edges)
        set_sampling(False)
        del edges
        # every G factor is complete now; the real backward below only produces gradients.  An optimizer
        # with early_inverse set starts its round of inverses here, beside that backward pass.
        after_sampling = getattr(optimizer, '_after_sampling_passes', None)
        if after_sampling is not None:
            after_sampling()

        loss = F.cross_entropy(output, target)
        loss.backward()
        return loss, output

    return closure
