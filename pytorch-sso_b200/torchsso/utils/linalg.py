"""``inv`` and ``cholesky`` with the signatures of torchsso/utils/inv_cupy.py:27-34 and
torchsso/utils/cholesky_cupy.py:9-14, executed by the tile-task engine of libsso_b200.

``inv(m)`` returns a new tensor holding the inverse of the SPD matrix ``m`` (input untouched);
``cholesky(m, upper=True)`` returns the upper factor U with U^T U = m (or the lower factor).
Both are one-matrix conveniences; the optimizers invert all layers in one batched plan."""
from __future__ import annotations

import torch

from .. import _native as nat

_cache = {}


def _solo(d: int, device):
    key = (d, device.index)
    ent = _cache.get(key)
    if ent is None:
        bufs = [torch.empty((d, d), dtype=torch.float32, device=device) for _ in range(4)]
        src, dst, work, std = bufs
        plan = nat.kron_plan([d], [src], [dst], [work], [std], [-1], [0], device)
        zero = torch.zeros(1, dtype=torch.float32, device=device)
        info = torch.zeros(2, dtype=torch.int32, device=device)
        ent = (plan, src, dst, work, std, zero, info)
        if len(_cache) > 16:
            _cache.clear()
        _cache[key] = ent
    return ent


def inv(m: torch.Tensor) -> torch.Tensor:
    if not m.is_cuda:
        raise RuntimeError('torchsso.utils.inv needs a CUDA tensor (no CPU path in this build)')
    assert m.dim() == 2 and m.shape[0] == m.shape[1]
    plan, src, dst, work, std, zero, info = _solo(m.shape[0], m.device)
    src.copy_(m)
    nat.kron_plan_run(plan, zero, info, True, False)
    return dst.clone()


def cholesky(m: torch.Tensor, upper: bool = True) -> torch.Tensor:
    if not m.is_cuda:
        raise RuntimeError('torchsso.utils.cholesky needs a CUDA tensor (no CPU path in this build)')
    assert m.dim() == 2 and m.shape[0] == m.shape[1]
    plan, src, dst, work, std, zero, info = _solo(m.shape[0], m.device)
    dst.copy_(m)           # the factorisation stage reads the "inverse" slot
    nat.kron_plan_run(plan, zero, info, False, True)
    out = std.clone()
    return out if upper else out.t()
