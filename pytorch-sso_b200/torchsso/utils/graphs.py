"""CUDA-graph capture of a training closure.

A K-FAC step launches ~2000 kernels (forward, sampling backward, loss backward, ~200 curvature
kernels in the hooks); issued eagerly the host cannot keep a B200 busy.  ``GraphedClosure`` runs
the closure a few times on a side stream, captures one execution into a CUDA graph and replays it:
the hooks' kernels (all launched on the current stream through the C ABI, no synchronisation, no
allocation after warm-up) are part of the graph.  The closure must read its batch from fixed
tensors (copy every new batch into them before calling).
"""
from __future__ import annotations

import torch


class GraphedClosure:
    """``graphed = GraphedClosure(optimizer, closure); optimizer.step(closure=graphed)``.

    ``closure`` takes no arguments, calls ``optimizer.zero_grad()``, does forward / backward and
    returns tensors (e.g. ``(loss, output)``); the same tensor objects are returned by every replay.
    Gradients that autograd allocates during capture (parameters whose ``.grad`` the optimizer does
    not bind to its flat buffer, e.g. channels_last weights) live in the graph's memory pool; they
    are re-attached to the parameters after each replay so the optimizer finds them."""

    def __init__(self, optimizer, closure, warmup: int = 3):
        self.optimizer = optimizer
        params = [p for g in optimizer.param_groups for p in g['params']]
        # Warm up and capture on ONE side stream: autograd's gradient-accumulation nodes run on the
        # stream they were created on, so they must be (re)created on the stream that captures.
        torch.cuda.synchronize()
        # high priority: the model's own kernels (the critical path) go before the curvature kernels
        # that the hooks fork to the (default-priority) curvature stream
        side = torch.cuda.Stream(priority=-1)
        side.wait_stream(torch.cuda.current_stream())
        from torchsso import _native as nat
        # with optimizer.fuse_ema the hooks advance the running averages: the executions below (warm-up
        # and the capture itself) are not optimisation steps, so the averages are put back afterwards
        saved = []
        if getattr(optimizer, 'fuse_ema', False):
            pool = optimizer.pool
            saved = [(pool.buf('ema', k), pool.buf('ema', k).clone()) for k in ('k', 'd') if pool.has('ema', k)]
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                closure()
                nat.join_curvature_stream(None)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        before = nat.launch_count()
        with torch.cuda.graph(self.graph, stream=side):
            self.result = closure()
            nat.join_curvature_stream(None)      # forked curvature kernels rejoin inside the capture
        torch.cuda.synchronize()
        for buf, copy in saved:
            buf.copy_(copy)
        #: kernels of libsso_b200 inside the graph, i.e. launched by every replay
        self.library_kernels_per_replay = nat.launch_count() - before
        self.replays = 0
        self._params = params
        self._grads = [p.grad for p in params]

    def __call__(self):
        self.graph.replay()
        self.replays += 1
        for p, g in zip(self._params, self._grads):
            if p.grad is not g:
                p.grad = g
        return self.result
