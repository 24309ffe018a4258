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
        # with optimizer.fuse_ema the hooks advance the running averages (and with early_inverse the
        # closure rewrites the inverses): the executions below (warm-up and the captures themselves) are
        # not optimisation steps, so those buffers are put back afterwards
        saved = []
        if getattr(optimizer, 'fuse_ema', False):
            pool = optimizer.pool
            roles = ('ema', 'inv') if getattr(optimizer, 'early_inverse', False) else ('ema',)
            saved = [(pool.buf(r, k), pool.buf(r, k).clone()) for r in roles for k in ('k', 'd') if pool.has(r, k)]
        # an optimizer that starts its inverses inside the closure needs one graph per kind of step
        variants = [False, True] if getattr(optimizer, 'early_inverse', False) else [None]
        keep_update_inv = optimizer.update_inv
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                if variants[0] is not None:
                    optimizer.update_inv = False
                closure()
                nat.join_curvature_stream(None)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graphs, self._results, self._grads, self._launches = {}, {}, {}, {}
        mem_pool = None
        for v in variants:
            if v is not None:
                optimizer.update_inv = v
            graph = torch.cuda.CUDAGraph()
            before = nat.launch_count()
            with torch.cuda.graph(graph, stream=side, pool=mem_pool):
                result = closure()
                nat.join_curvature_stream(None)      # forked curvature kernels rejoin inside the capture
            optimizer.__dict__.pop('_early_inverse_done', None)
            mem_pool = graph.pool()
            self._graphs[v], self._results[v] = graph, result
            self._grads[v] = [p.grad for p in params]
            self._launches[v] = nat.launch_count() - before
        optimizer.update_inv = keep_update_inv
        torch.cuda.synchronize()
        for buf, copy in saved:
            buf.copy_(copy)
        self.graph = self._graphs[variants[0]]
        self.result = self._results[variants[0]]
        #: kernels of libsso_b200 inside the graph, i.e. launched by every replay (of a step without
        #: inverses when there are two graphs)
        self.library_kernels_per_replay = self._launches[variants[0]]
        #: kernels of libsso_b200 launched by all replays so far
        self.library_launches = 0
        self.replays = 0
        self._params = params
        self._two = variants[0] is not None

    def __call__(self):
        v = bool(self.optimizer.update_inv) if self._two else None
        self._graphs[v].replay()
        self.replays += 1
        self.library_launches += self._launches[v]
        if v:
            self.optimizer.__dict__['_early_inverse_done'] = True
        for p, g in zip(self._params, self._grads[v]):
            if p.grad is not g:
                p.grad = g
        return self._results[v]
