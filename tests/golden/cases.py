"""Seeded model/input builders shared by the golden-vector generator and the tests.

All randomness comes from numpy's PCG64 (stable across numpy/torch versions and
machines); nothing here depends on torch's global RNG.  Data are synthetic: shapes
are borrowed from MNIST / CIFAR-style inputs, values are N(0,1), labels uniform.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F


def _fill_params(model: nn.Module, seed: int, scale: float = 1.0):
    rng = np.random.default_rng(seed)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            if p.dim() > 1:
                fan_in = int(np.prod(p.shape[1:]))
                v = rng.standard_normal(p.shape).astype(np.float32) * (scale / np.sqrt(fan_in))
            elif name.endswith('weight'):      # norm scale: away from zero
                v = (1.0 + 0.1 * rng.standard_normal(p.shape)).astype(np.float32)
            else:
                v = (0.1 * rng.standard_normal(p.shape)).astype(np.float32)
            p.copy_(torch.from_numpy(v))
    return model


class TinyConvNet(nn.Module):
    """conv(s2,p1,bias) - bn - relu - conv(no bias) - bn - relu - fc(bias); functional relu."""
    num_classes = 5

    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 4, 3, stride=2, padding=1, bias=True)
        self.bn1 = nn.BatchNorm2d(4)
        self.conv2 = nn.Conv2d(4, 6, 3, stride=1, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(6)
        self.fc = nn.Linear(6 * 4 * 4, 5)

    def forward(self, x):
        x = F.relu(self.bn1(self.conv1(x)))
        x = F.relu(self.bn2(self.conv2(x)))
        return self.fc(x.reshape(x.shape[0], -1))


class SmallMLP(nn.Module):
    num_classes = 4

    def __init__(self, d_in=20, d_hid=16, d_out=4):
        super().__init__()
        self.l1 = nn.Linear(d_in, d_hid)
        self.l2 = nn.Linear(d_hid, d_hid)
        self.l3 = nn.Linear(d_hid, d_out)

    def forward(self, x):
        x = x.reshape(x.shape[0], -1)
        return self.l3(F.relu(self.l2(F.relu(self.l1(x)))))


class MnistMLP(nn.Module):
    """784-1000-1000-10 with functional relu (the single-process CPU configuration)."""
    num_classes = 10

    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(784, 1000)
        self.l2 = nn.Linear(1000, 1000)
        self.l3 = nn.Linear(1000, 10)

    def forward(self, x):
        x = x.reshape(-1, 784)
        return self.l3(F.relu(self.l2(F.relu(self.l1(x)))))


class TinyVGG(nn.Module):
    """Two biased convs + fc, no norm layers (shape of the VI configuration, shrunk)."""
    num_classes = 6

    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(3, 5, 3, padding=1)
        self.c2 = nn.Conv2d(5, 7, 3, padding=1)
        self.fc = nn.Linear(7 * 2 * 2, 6)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        return self.fc(x.reshape(x.shape[0], -1))


def make_model(name: str, seed: int = 0) -> nn.Module:
    cls = {'tiny_convnet': TinyConvNet, 'small_mlp': SmallMLP, 'mnist_mlp': MnistMLP,
           'tiny_vgg': TinyVGG}[name]
    return _fill_params(cls(), seed)


def make_batch(shape, num_classes: int, seed: int):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal(shape).astype(np.float32))
    y = torch.from_numpy(rng.integers(0, num_classes, size=(shape[0],)).astype(np.int64))
    return x, y


def make_uniform(shape, seed: int) -> torch.Tensor:
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.random(shape))          # float64 in [0, 1)


def make_normal(shape, seed: int) -> torch.Tensor:
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.standard_normal(shape).astype(np.float32))
