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


class ConvNetB256(nn.Module):
    """conv 3->64 5x5 p2, pool, conv 64->128 5x5 p2, pool, conv 128->256 3x3 p1, pool, fc 4096->512->10
    (functional relu / max_pool2d; every layer has a bias): the single-GPU ConvNet configuration,
    factor dimensions 76 / 1601 / 1153 / 4097 / 513."""
    num_classes = 10

    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(3, 64, 5, padding=2)
        self.c2 = nn.Conv2d(64, 128, 5, padding=2)
        self.c3 = nn.Conv2d(128, 256, 3, padding=1)
        self.f1 = nn.Linear(4096, 512)
        self.f2 = nn.Linear(512, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        x = F.max_pool2d(F.relu(self.c3(x)), 2)
        return self.f2(F.relu(self.f1(x.reshape(x.shape[0], -1))))


class VGG16Style(nn.Module):
    """64-64-M-128-128-M-256x3-M-512x3-M-512x3-M conv stack (3x3, pad 1, bias, no norm layers)
    then linear 512->100: the variational-inference configuration (factor dimensions up to 4609)."""
    num_classes = 100
    CFG = (64, 64, 'M', 128, 128, 'M', 256, 256, 256, 'M', 512, 512, 512, 'M', 512, 512, 512, 'M')

    def __init__(self):
        super().__init__()
        convs, cin = [], 3
        for v in self.CFG:
            if v != 'M':
                convs.append(nn.Conv2d(cin, v, 3, padding=1))
                cin = v
        self.convs = nn.ModuleList(convs)
        self.fc = nn.Linear(512, 100)

    def forward(self, x):
        it = iter(self.convs)
        for v in self.CFG:
            x = F.max_pool2d(x, 2) if v == 'M' else F.relu(next(it)(x))
        return self.fc(x.reshape(x.shape[0], -1))


class UnevenNet(nn.Module):
    """Nine convolutions and four linear layers of very different sizes (factor dimensions 19 ... 361),
    with and without bias, three BatchNorm layers: owner assignment by inverse cost and by contiguous
    ranges give different, unbalanced partitions on 2, 4 and 8 ranks.  Smooth throughout (tanh, average
    pooling): it is compared between runs whose parameters differ by one rounding, and with ReLU and
    max pooling such a difference now and then flips a unit, which moves every gradient below it by
    ~1e-2 (seen on 4 GPUs: 7.7e-4 in the parameters after two steps in some runs, 3e-6 in others)."""
    num_classes = 7
    WIDTHS = (6, 24, 8, 40, 12, 12, 32, 6, 16)

    def __init__(self):
        super().__init__()
        convs, bns, cin = [], {}, 2
        for i, w in enumerate(self.WIDTHS):
            convs.append(nn.Conv2d(cin, w, 3 if i % 3 else 1, padding=1 if i % 3 else 0, bias=(i % 2 == 0)))
            if i in (1, 4, 7):
                bns[str(i)] = nn.BatchNorm2d(w)
            cin = w
        self.convs = nn.ModuleList(convs)
        self.bns = nn.ModuleDict(bns)
        self.f1 = nn.Linear(cin * 4, 48)
        self.f2 = nn.Linear(48, 20, bias=False)
        self.f3 = nn.Linear(20, 30)
        self.f4 = nn.Linear(30, 7)

    def forward(self, x):
        for i, conv in enumerate(self.convs):
            x = conv(x)
            if str(i) in self.bns:
                x = self.bns[str(i)](x)
            x = torch.tanh(x)
            if i in (2, 5):
                x = F.avg_pool2d(x, 2)
        x = x.reshape(x.shape[0], -1)
        return self.f4(torch.tanh(self.f3(torch.tanh(self.f2(torch.tanh(self.f1(x)))))))


def make_model(name: str, seed: int = 0) -> nn.Module:
    cls = {'tiny_convnet': TinyConvNet, 'small_mlp': SmallMLP, 'mnist_mlp': MnistMLP,
           'tiny_vgg': TinyVGG, 'convnet_b256': ConvNetB256, 'vgg16_style': VGG16Style, 'uneven_net': UnevenNet}[name]
    return _fill_params(cls(), seed, scale=_INIT_SCALE.get(name, 1.0))


# He-style gain for the deep ReLU stacks, so that activations neither vanish nor explode at depth
_INIT_SCALE = {'vgg16_style': 2.0 ** 0.5}


def summary_rows(d: int):
    """Rows of a d x d (or length-d leading dimension) tensor kept by the large-model fixtures."""
    return sorted({d // 2, d - 1})


def summarize(t: torch.Tensor) -> dict:
    """Compact fingerprint of a tensor too large to commit: Frobenius norm, sum, the diagonal of a
    square matrix and a few full rows (a wrong scale, permutation or transpose changes them)."""
    t = t.detach().cpu()
    m = t.reshape(t.shape[0], -1) if t.dim() > 1 else t.reshape(1, -1)
    out = {'norm': np.float64(m.double().norm().item()), 'sum': np.float64(m.double().sum().item())}
    rows = summary_rows(m.shape[0])
    out['rows'] = m[rows].numpy().astype(np.float32).copy()
    if m.dim() == 2 and m.shape[0] == m.shape[1]:
        out['diag'] = m.diagonal().numpy().astype(np.float32).copy()
    return out


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


def summary_error(gold, prefix: str, t: torch.Tensor) -> float:
    """Worst relative deviation of tensor ``t`` from the fingerprint stored under ``prefix`` in a
    fixture written with ``summarize``: Frobenius norm, the kept rows and the diagonal."""
    got = summarize(t)
    worst = abs(float(got['norm']) - float(gold[prefix + '/norm'])) / max(float(gold[prefix + '/norm']), 1e-30)
    for key in ('rows', 'diag'):
        if key in got:
            a = np.asarray(got[key], dtype=np.float64)
            b = np.asarray(gold[prefix + '/' + key], dtype=np.float64)
            assert a.shape == b.shape, (prefix, key, a.shape, b.shape)
            worst = max(worst, float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)))
    return worst
