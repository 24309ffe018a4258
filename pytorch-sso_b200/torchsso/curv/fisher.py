"""Closure factory for Fisher curvatures (same protocol as
torchsso/curv/fisher/__init__.py:34-90): forward once, then one extra backward pass per Monte
Carlo target (or per class for the exact Fisher) that only the curvature hooks see, then the
real backward for the loss gradient.

The reference freezes the parameters for the sampling passes (requires_grad = False after the
forward), which still computes every weight gradient and drops it at the accumulation node.
Here a sampling pass asks autograd for the output gradients of the hooked modules only
(``prune_sampling_pass=True``, the default): the hooks see the same values, the weight-gradient
kernels of those passes never run.  ``prune_sampling_pass=False`` is the reference's protocol.

With several Monte Carlo targets the reference walks the graph once per target
(torchsso/curv/fisher/__init__.py:65-72).  A backward pass is linear in the gradient it starts
from, so the ``num_mc`` walks can be one (``batch_mc_passes=True``, needs the pruned pass): autograd
is asked for the output gradients of all targets at once
(``torch.autograd.grad(..., is_grads_batched=True)``: every backward op runs once on tensors with a
leading target dimension), the hooks stay silent during that walk (they would be handed batched
tensors that have no address), and the curvature kernels are then fed target by target with the
slices of the returned gradients, exactly as the hooks would have been.  Off by default, by
measurement (ResNet-50, batch 32, bf16, 4 targets, B200): issued eagerly the single walk saves host
time (47.4 against 52.1 ms per step), but replayed from a CUDA graph, where launches are free, the
batched backward kernels that vmap selects are slower than four plain walks (40.5 against 30.7 ms);
the 5x5 ConvNet at batch 256: 9.7 against 9.2 ms."""
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
                           prune_sampling_pass=True, batch_mc_passes=False):

    if batch_mc_passes and not prune_sampling_pass:
        raise ValueError('batch_mc_passes needs prune_sampling_pass: the batched walk returns the output '
                         'gradients of the hooked modules instead of running their hooks')

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

    def batched_sampling_backward(output, mc_targets, curvs, edges):
        """All Monte Carlo targets in one walk of the graph, then the hooks' work target by target."""
        losses = torch.stack([F.cross_entropy(output, mc_targets[i]) for i in range(num_mc)])
        seeds = torch.eye(num_mc, device=losses.device, dtype=losses.dtype)
        for curv in curvs:
            curv.__dict__['_mute_hook'] = True
        try:
            grads = torch.autograd.grad(losses, edges, grad_outputs=seeds, is_grads_batched=True,
                                        retain_graph=True, allow_unused=True)
        finally:
            for curv in curvs:
                curv.__dict__['_mute_hook'] = False
        for i in range(num_mc):
            for curv, g in zip(curvs, grads):
                if g is not None:
                    curv.backward_postprocess(curv.module, None, (g[i],))
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

        edges, edge_curvs = [], []
        if prune_sampling_pass:
            for group in optimizer.param_groups:
                edge = group['curv'].module.__dict__.pop('output_edge', None)
                if edge is not None:
                    edges.append(edge)
                    edge_curvs.append(group['curv'])
            if not edges:
                raise RuntimeError('no hooked module produced an output that requires grad')

        set_sampling(True)
        if approx_type == _APPROX_TYPE_MC:
            mc_targets = sample_targets(prob.detach(), num_mc)
            weight = torch.full_like(prob[:, 0], 1.0 / num_mc).detach()
            for group in optimizer.param_groups:
                group['curv'].prob = weight
                group['curv'].prob_scale = 1.0 / num_mc
            if batch_mc_passes and prune_sampling_pass and num_mc > 1:
                batched_sampling_backward(output, mc_targets, edge_curvs, edges)
            else:
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
        del edges, edge_curvs
        # every G factor is complete now; the real backward below only produces gradients.  An optimizer
        # with early_inverse set starts its round of inverses here, beside that backward pass.
        after_sampling = getattr(optimizer, '_after_sampling_passes', None)
        if after_sampling is not None:
            after_sampling()

        loss = F.cross_entropy(output, target)
        loss.backward()
        return loss, output

    return closure
