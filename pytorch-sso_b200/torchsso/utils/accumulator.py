"""Running weighted sum of a tensor or a list of tensors (same role as
torchsso/utils/accumulator.py:4-57 in the reference; used by the public API for loss /
probability averaging -- the factor and gradient accumulation of the optimizers runs on the
flat pools with one kernel launch instead)."""
from __future__ import annotations

import torch


class TensorAccumulator(object):

    def __init__(self):
        self._accumulation = None

    def _validate(self, data):
        sample = data[0] if isinstance(data, list) else data
        assert isinstance(sample, torch.Tensor), \
            'the type of data has to be list of torch.Tensor or torch.Tensor'
        if self._accumulation is not None:
            assert isinstance(data, list) == isinstance(self._accumulation, list), \
                'cannot mix tensors and lists of tensors in one accumulator'

    def update(self, data, scale=1.):
        self._validate(data)
        acc = self._accumulation
        if isinstance(data, list):
            if acc is None:
                self._accumulation = [d * scale for d in data]
            else:
                self._accumulation = [torch.add(a, d, alpha=scale) for a, d in zip(acc, data)]
        elif acc is None:
            self._accumulation = data * scale
        else:
            self._accumulation = torch.add(acc, data, alpha=scale)

    def get(self, clear=True):
        acc = self._accumulation
        if acc is None:
            return None
        out = [a.clone() for a in acc] if isinstance(acc, list) else acc.clone()
        if clear:
            self.clear()
        return out

    def clear(self):
        self._accumulation = None
