"""Flat device storage and batched execution for the curvatures of a set of layers.

Every Kronecker factor (A and G of each layer) and every diagonal curvature vector lives in
one contiguous fp32 buffer per role -- ``data`` (this step's estimate), ``ema``, ``inv``,
``std`` (VI), ``work`` (scratch of the inverse) and ``acc`` (accumulation over micro-steps /
MC samples) -- with the same element layout in each.  That turns the per-layer loops of the
reference (torchsso/optim/secondorder.py:195-209: EMA, inverse, precondition one layer at a
time, a handful of small launches each) into a few launches per step:

  EMA / accumulation   one streaming kernel over the whole pool
  pi-damped inverse    one engine plan over all matrices (torchsso/curv/curvature.py:302-312)
  precondition         two engine phases over all layers (torchsso/curv/cov/linear.py:69-84)
  diagonal curvatures  one streaming kernel (torchsso/curv/curvature.py:226-238)

A curvature object that is used on its own gets a private pool of size one, so there is a
single code path.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

from .. import _native as nat

_ALIGN = 64  # elements; keeps every matrix 256-byte aligned inside the pool


def _round_up(v: int, a: int = _ALIGN) -> int:
    return (v + a - 1) // a * a


def _ld(d: int) -> int:
    """Leading dimension of a d x d factor inside the pool: rows padded to a multiple of four floats,
    so that every row starts on 16 bytes and the tile tasks that read the factor (inverse, std,
    precondition, sampling) can fetch it with TMA / 16-byte loads even when d is odd (layers with a
    bias).  The padding columns are zero and stay zero."""
    return (d + 3) // 4 * 4


class FactorPool:

    def __init__(self, kron: Sequence, diag: Sequence, device):
        self.device = torch.device(device)
        self.kron = list(kron)
        self.diag = list(diag)
        self._bufs: Dict[str, torch.Tensor] = {}
        # --- Kronecker layout: [A_0 | G_0 | A_1 | G_1 | ...]
        self.k_off = {}
        off = 0
        for c in self.kron:
            (da, _), (dg, _) = c._get_shape()
            a_off = off
            off = _round_up(off + da * _ld(da))
            g_off = off
            off = _round_up(off + dg * _ld(dg))
            self.k_off[id(c)] = (a_off, da, g_off, dg)
        self.k_total = off
        # --- diagonal layout: parameters of each layer back to back, layers back to back
        self.d_off = {}
        off = 0
        for c in self.diag:
            offs = []
            for p in c.module.parameters():
                offs.append((off, tuple(p.shape)))
                off += p.numel()
            self.d_off[id(c)] = offs
        self.d_total = off
        self._plans = {}
        self._damp = {}
        self.last_info: Optional[torch.Tensor] = None
        for c in list(self.kron) + list(self.diag):
            c._pool = self

    # ------------------------------------------------------------------ storage
    def buf(self, role: str, kind: str = 'k') -> torch.Tensor:
        key = role + ':' + kind
        b = self._bufs.get(key)
        if b is None:
            total = self.k_total if kind == 'k' else self.d_total
            b = torch.zeros(max(total, 1), dtype=torch.float32, device=self.device)
            self._bufs[key] = b
        return b

    def has(self, role: str, kind: str = 'k') -> bool:
        return (role + ':' + kind) in self._bufs

    def mat(self, role: str, curv, which: int) -> torch.Tensor:
        a_off, da, g_off, dg = self.k_off[id(curv)]
        off, d = (a_off, da) if which == 0 else (g_off, dg)
        ld = _ld(d)
        m = self.buf(role)[off: off + d * ld].view(d, ld)
        return m if ld == d else m[:, :d]

    def vec(self, role: str, curv, j: int) -> torch.Tensor:
        off, shape = self.d_off[id(curv)][j]
        return self.buf(role, 'd')[off: off + int(math.prod(shape))].view(shape)

    def kron_range(self, curvs: Sequence):
        """[lo, hi) element range of the pool covered by `curvs` (must be contiguous in layout)."""
        if not curvs:
            return 0, 0
        idx = sorted(self.kron.index(c) for c in curvs)
        assert idx == list(range(idx[0], idx[-1] + 1)), 'curvatures are not contiguous in the pool'
        lo = self.k_off[id(self.kron[idx[0]])][0]
        hi = self.k_off[id(self.kron[idx[-1] + 1])][0] if idx[-1] + 1 < len(self.kron) else self.k_total
        return lo, hi

    def diag_range(self, curvs: Sequence):
        if not curvs:
            return 0, 0
        idx = sorted(self.diag.index(c) for c in curvs)
        assert idx == list(range(idx[0], idx[-1] + 1)), 'curvatures are not contiguous in the pool'
        lo = self.d_off[id(self.diag[idx[0]])][0][0]
        hi = self.d_off[id(self.diag[idx[-1] + 1])][0][0] if idx[-1] + 1 < len(self.diag) else self.d_total
        return lo, hi

    # ------------------------------------------------------------------ streaming ops
    def _flat(self, src_role, dst_role, a, b, kron, diag):
        lo, hi = self.kron_range(kron)
        if hi > lo:
            nat.axpby(self.buf(src_role)[lo:hi], self.buf(dst_role)[lo:hi], a, b)
        lo, hi = self.diag_range(diag)
        if hi > lo:
            nat.axpby(self.buf(src_role, 'd')[lo:hi], self.buf(dst_role, 'd')[lo:hi], a, b)

    def accumulate(self, scale: float, first: bool, kron=None, diag=None):
        """acc <- scale*data (first) or acc + scale*data."""
        kron = self.kron if kron is None else kron
        diag = self.diag if diag is None else diag
        self._flat('data', 'acc', scale, 0.0 if first else 1.0, kron, diag)

    def take_accumulated(self, kron=None, diag=None):
        """data <- acc."""
        kron = self.kron if kron is None else kron
        diag = self.diag if diag is None else diag
        self._flat('acc', 'data', 1.0, 0.0, kron, diag)

    def update_ema(self, beta: float, first: bool, kron=None, diag=None):
        """ema <- data (first use, or beta == 1), else beta*data + (1-beta)*ema, for all given
        layers in one launch per pool (torchsso/curv/curvature.py:174-191)."""
        kron = self.kron if kron is None else kron
        diag = self.diag if diag is None else diag
        if first or beta == 1:
            self._flat('data', 'ema', 1.0, 0.0, kron, diag)
        else:
            self._flat('data', 'ema', beta, 1.0 - beta, kron, diag)

    # ------------------------------------------------------------------ engine plans
    def _kron_plan(self, curvs: Sequence, with_std: bool, src_role: str):
        key = ('inv', tuple(id(c) for c in curvs), with_std, src_role)
        ent = self._plans.get(key)
        if ent is None:
            dims, src, dst, work, std, partner, role = [], [], [], [], [], [], []
            for c in curvs:
                base = len(dims)
                for which in (0, 1):
                    m = self.mat(src_role, c, which)
                    dims.append(m.shape[0])
                    src.append(m)
                    dst.append(self.mat('inv', c, which))
                    work.append(self.mat('work', c, which))
                    if with_std:
                        std.append(self.mat('std', c, which))
                    tracenorm = getattr(c, 'pi_type', 'tracenorm') == 'tracenorm'
                    partner.append(base + (1 - which) if tracenorm else -1)
                    role.append(which)
            plan = nat.kron_plan(dims, src, dst, work, std if with_std else None, partner, role, self.device)
            damp = torch.zeros(len(dims), dtype=torch.float32, device=self.device)
            info = torch.zeros(2 * len(dims), dtype=torch.int32, device=self.device)
            ent = (plan, damp, info)
            self._plans[key] = ent
        return ent

    def update_inv(self, curvs: Optional[Sequence] = None, with_std: bool = False,
                   do_inverse: bool = True, use_max_ema: bool = False):
        """inv <- [ (A + r*pi*I)^-1, (G + r/pi*I)^-1 ] for every layer in one plan; with_std also
        std <- upper Cholesky factors of the inverses (torchsso/curv/curvature.py:302-321)."""
        curvs = self.kron if curvs is None else list(curvs)
        if not curvs:
            return
        plan, damp, info = self._kron_plan(curvs, with_std, 'ema_max' if use_max_ema else 'ema')
        r = []
        for c in curvs:
            v = math.sqrt(c.damping)
            r += [v, v]
        key = id(plan)
        if self._damp.get(key) != r:
            damp.copy_(torch.tensor(r, dtype=torch.float32), non_blocking=False)
            self._damp[key] = r
        nat.kron_plan_run(plan, damp, info, do_inverse, with_std)
        self.last_info = info

    def _trim_plans(self, limit: int = 32):
        """Plans bake buffer addresses in; callers with unstable addresses would grow the cache."""
        if len(self._plans) > limit:
            for k in [k for k in self._plans if k[0] in ('pre', 'smp')]:
                del self._plans[k]

    def check_info(self):
        """Raise if the last factorisation met a non-positive pivot, or if a bounded device-side wait of
        any engine plan of this pool ever gave up (its tiles were written as NaN).  Synchronises."""
        for key, ent in self._plans.items():
            plan = ent[0] if isinstance(ent, tuple) else ent
            code = plan.status()
            if code:
                raise RuntimeError('a device-side wait of the %s plan gave up (code %d): its results are NaN'
                                   % ({'inv': 'inverse', 'pre': 'precondition', 'smp': 'sampling'}[key[0]], code))
        if self.last_info is None:
            return
        info = self.last_info.cpu()
        if int(info[0]) <= -1000:
            raise RuntimeError('a device-side wait of the inverse plan gave up (code %d): its results are NaN'
                               % (-int(info[0]) - 1000))
        bad = torch.nonzero(info).flatten()
        if bad.numel():
            i = int(bad[0])
            raise RuntimeError('curvature matrix %d (%s pass) is not positive definite at row %d'
                               % (i // 2, 'inverse' if i % 2 == 0 else 'cholesky', int(info[i])))

    def precondition(self, curvs: Sequence, grads: Sequence[Sequence[torch.Tensor]]):
        """grads[i] = [dW (, db)] of layer i, fp32 contiguous; replaced by G^-1 [dW|db] A^-1."""
        if not curvs:
            return
        key = ('pre', tuple(id(c) for c in curvs), tuple(g.data_ptr() for gs in grads for g in gs))
        plan = self._plans.get(key)
        if plan is None:
            dA, dG, A_inv, G_inv, gw, gb, tmp = [], [], [], [], [], [], []
            for c, gs in zip(curvs, grads):
                a, g = self.mat('inv', c, 0), self.mat('inv', c, 1)
                assert gs[0].is_contiguous() and gs[0].dtype == torch.float32
                wcols = gs[0].numel() // gs[0].shape[0]
                has_b = len(gs) > 1
                assert a.shape[0] == wcols + (1 if has_b else 0) and g.shape[0] == gs[0].shape[0]
                dA.append(a.shape[0]); dG.append(g.shape[0])
                A_inv.append(a); G_inv.append(g)
                gw.append(gs[0]); gb.append(gs[1] if has_b else None)
                # scratch: the A-slot of `work` is dA*dA >= ... not always >= dG*dA; own buffer
                # [d_A x d_G] with the leading dimension of G_inv
                tmp.append(torch.empty(a.shape[0] * max(g.stride(0), g.shape[0]), dtype=torch.float32, device=self.device))
            plan = nat.precond_plan(dA, dG, A_inv, G_inv, gw, gb, tmp, self.device)
            self._trim_plans()
            self._plans[key] = plan
        nat.precond_plan_run(plan)

    def sample(self, curvs: Sequence, params: Sequence[Sequence[torch.Tensor]],
               noises: Sequence[torch.Tensor], std_scale: float):
        """params[i] (pre-loaded with the mean) += s * U_G E U_A (torchsso/curv/cov/linear.py:86-100)."""
        if not curvs:
            return
        key = ('smp', tuple(id(c) for c in curvs), tuple(p.data_ptr() for ps in params for p in ps),
               tuple(n.data_ptr() for n in noises))
        plan = self._plans.get(key)
        if plan is None:
            dA, dG, UA, UG, w, b, tmp = [], [], [], [], [], [], []
            for c, ps in zip(curvs, params):
                ua, ug = self.mat('std', c, 0), self.mat('std', c, 1)
                dA.append(ua.shape[0]); dG.append(ug.shape[0])
                UA.append(ua); UG.append(ug)
                assert ps[0].is_contiguous() and ps[0].dtype == torch.float32
                w.append(ps[0]); b.append(ps[1] if len(ps) > 1 else None)
                tmp.append(torch.empty(ug.shape[0] * ua.shape[0], dtype=torch.float32, device=self.device))
            plan = nat.sample_plan(dA, dG, UA, UG, list(noises), w, b, tmp, self.device)
            self._trim_plans()
            self._plans[key] = plan
        nat.sample_plan_run(plan, std_scale)

    # ------------------------------------------------------------------ diagonal curvatures
    def diag_step(self, curvs: Sequence, grad_flat: Optional[torch.Tensor], update_inv: bool):
        """inv <- 1/(ema + damping) (if update_inv) and grad <- grad*inv over a contiguous run of
        diagonal curvatures that share damping / sqrt settings; grad_flat has the pool's layout."""
        lo, hi = self.diag_range(curvs)
        if hi <= lo:
            return
        c0 = curvs[0]
        ema = self.buf('ema_max' if c0.use_max_ema else 'ema', 'd')[lo:hi]
        inv = self.buf('inv', 'd')[lo:hi]
        nat.diag_inv_precondition(ema, inv, grad_flat, float(c0.damping), bool(c0.use_sqrt_ema), update_inv)
