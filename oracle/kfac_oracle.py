"""CPU oracle for the K-FAC curvature path of PyTorch-SSO.  TEST INFRASTRUCTURE ONLY.

This module restates, op by op, what the reference library computes on the
K-FAC hot path, using plain torch CPU tensor algebra (fp32 or fp64, chosen by
the dtype of the inputs).  It exists so that the CUDA kernels can be checked
against it and so that a CPU baseline can be timed.  Nothing in the product
package may import it; only the tests, the smoke check and the CPU arms of the
benchmark do.

Parity pin: the functions below are compared with outputs of the unmodified
reference (imported from its source tree in the build container) by
``tests/golden/make_golden.py``; the resulting vectors are committed under
``tests/golden/`` and re-checked by ``tests/test_oracle_golden.py``.

Every function names the reference file:line it follows (paths are relative
to the reference project root).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------
# im2col
# --------------------------------------------------------------------------
def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def unfold_rows(x: Tensor, kernel_size, stride=1, padding=0, dilation=1) -> Tensor:
    """im2col with one row per output pixel.

    Returns ``[n*ho*wo, c*kh*kw]`` whose column order is (c, kh, kw) and whose
    row order is (n, ho, wo) -- the transpose of the ``m`` matrix built at
    torchsso/curv/cov/conv.py:51-58 (F.unfold + transpose + reshape).
    Written with explicit slicing so it does not depend on F.unfold.
    """
    kh, kw = _pair(kernel_size)
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    dh, dw = _pair(dilation)
    n, c, h, w = x.shape
    ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    xp = torch.zeros((n, c, h + 2 * ph, w + 2 * pw), dtype=x.dtype)
    xp[:, :, ph:ph + h, pw:pw + w] = x
    cols = torch.empty((n, ho, wo, c, kh, kw), dtype=x.dtype)
    for i in range(kh):
        for j in range(kw):
            patch = xp[:, :, i * dh: i * dh + (ho - 1) * sh + 1: sh,
                       j * dw: j * dw + (wo - 1) * sw + 1: sw]      # n c ho wo
            cols[:, :, :, :, i, j] = patch.permute(0, 2, 3, 1)
    return cols.reshape(n * ho * wo, c * kh * kw)


# --------------------------------------------------------------------------
# Kronecker factors
# --------------------------------------------------------------------------
def linear_factor_A(x: Tensor, bias: bool) -> Tensor:
    """A = [x 1]^T [x 1] / n.   torchsso/curv/cov/linear.py:50-59."""
    n = x.shape[0]
    if bias:
        x = torch.cat([x, torch.ones((n, 1), dtype=x.dtype)], dim=1)
    return (x.t() @ x) / n


def linear_factor_G(g: Tensor, prob: Optional[Tensor] = None) -> Tensor:
    """G = (p*g)^T g / n.  torchsso/curv/cov/linear.py:61-67 (p = 1) and
    torchsso/curv/fisher/linear.py:44-53 (p = per-sample weight)."""
    n = g.shape[0]
    left = g if prob is None else g * prob.reshape(n, 1)
    return (left.t() @ g) / n


def conv_factor_A(x: Tensor, kernel_size, stride, padding, dilation, bias: bool) -> Tensor:
    """A = m m^T / n with m the (c*kh*kw [+1]) x (n*ho*wo) im2col matrix; note the
    divisor is the batch size, not the row count.  torchsso/curv/cov/conv.py:47-67."""
    n = x.shape[0]
    rows = unfold_rows(x, kernel_size, stride, padding, dilation)
    if bias:
        rows = torch.cat([rows, torch.ones((rows.shape[0], 1), dtype=x.dtype)], dim=1)
    return (rows.t() @ rows) / n


def conv_factor_G(g: Tensor, prob: Optional[Tensor] = None) -> Tensor:
    """G = (p*g) g^T / (n*h*w), g viewed [c_out, n*h*w].
    torchsso/curv/cov/conv.py:69-74, torchsso/curv/fisher/conv.py:56-66."""
    n, c, h, w = g.shape
    rows = g.permute(0, 2, 3, 1).reshape(n * h * w, c)
    left = rows
    if prob is not None:
        left = (g * prob.reshape(n, 1, 1, 1)).permute(0, 2, 3, 1).reshape(n * h * w, c)
    return (left.t() @ rows) / (n * h * w)


def bn_restore_input(out: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
    """x_hat = (out - beta) / gamma, broadcast over channel dim 1.
    torchsso/curv/curvature.py:123-134."""
    shape = [1, -1] + [1] * (out.dim() - 2)
    return (out - bias.reshape(shape)) / weight.reshape(shape)


def bn_diag(xhat: Tensor, g: Tensor, prob: Optional[Tensor] = None,
            bias: bool = True) -> List[Tensor]:
    """Diagonal curvature of BatchNorm scale/shift.

    2-D input [n, f]  (torchsso/curv/cov/batchnorm.py:12-26):
        w = mean_n(x^2 * g^2),             b = mean_n(g^2)
    4-D input [n, c, h, w] (torchsso/curv/cov/batchnorm.py:36-49 and
    torchsso/curv/fisher/batchnorm.py:17-29):
        w = mean_n( (sum_hw x^2) * (sum_hw p g^2) ),  b = mean_n(sum_hw p g^2)
    i.e. a product of sums, not a sum of products.
    """
    n = g.shape[0]
    gg = g * g
    if prob is not None:
        gg = gg * prob.reshape([n] + [1] * (g.dim() - 1))
    xx = xhat * xhat
    if g.dim() == 4:
        gg = gg.sum(dim=(2, 3))
        xx = xx.sum(dim=(2, 3))
    out = [(xx * gg).mean(dim=0)]
    if bias:
        out.append(gg.mean(dim=0))
    return out


# --------------------------------------------------------------------------
# EMA, damping, inverse
# --------------------------------------------------------------------------
def diag_linear(x: Tensor, g: Tensor, prob: Optional[Tensor] = None):
    """Diagonal curvature of a Linear layer (torchsso/curv/cov/linear.py:28-45; with `prob` the
    Fisher weighting of torchsso/curv/fisher/linear.py:11-32): mean over samples of g^2 (x) x^2 and
    of g^2.  Returns (weight part [f_out, f_in], bias part [f_out]), before the n^2 rescale."""
    n = x.shape[0]
    gg = g * g if prob is None else g * g * prob.reshape(n, 1)
    return gg.t() @ (x * x) / n, gg.mean(dim=0)


def diag_conv(x: Tensor, g: Tensor, kernel_size, stride, padding, dilation, prob: Optional[Tensor] = None):
    """Diagonal curvature of a Conv2d layer (torchsso/curv/cov/conv.py:15-42): mean over samples of
    the squared per-sample weight gradient; bias part: mean over samples of the pixel sum of g^2.
    Returns (weight part [c_out, c_in, kh, kw], bias part [c_out]), before the n^2 rescale."""
    n, c_out = g.shape[0], g.shape[1]
    g2 = g.reshape(n, c_out, -1)
    rows = unfold_rows(x, kernel_size, stride, padding, dilation).reshape(n, g2.shape[2], -1)  # n, L, c_in*kh*kw
    per = torch.einsum('bik,bkj->bij', g2, rows)                          # per-sample gradients
    sq = per * per if prob is None else per * per * prob.reshape(n, 1, 1)
    gg = g2 * g2 if prob is None else g2 * g2 * prob.reshape(n, 1, 1)
    kh, kw = _pair(kernel_size)
    return sq.mean(dim=0).reshape(c_out, -1, kh, kw), gg.sum(dim=2).mean(dim=0)


def ema_update(data: Tensor, ema: Optional[Tensor], beta: float) -> Tensor:
    """ema <- data on the first call or when beta == 1, else beta*data + (1-beta)*ema
    (beta weights the NEW data).  torchsso/curv/curvature.py:174-191."""
    if ema is None or beta == 1:
        return data.clone()
    return data * beta + ema * (1 - beta)


def spd_inverse(m: Tensor) -> Tensor:
    """Dense inverse as the reference's CPU branch does it: LAPACK LU inverse of the
    (already damped) matrix.  torchsso/utils/inv_cupy.py:32-34."""
    import scipy.linalg
    return torch.from_numpy(scipy.linalg.inv(m.numpy()))


def kron_pi(A: Tensor, G: Tensor) -> Tensor:
    """pi = sqrt((tr A / d_A) / (tr G / d_G)).  torchsso/curv/curvature.py:305-306."""
    return torch.sqrt((A.trace() / A.shape[0]) / (G.trace() / G.shape[0]))


def kron_damped_inverse(A: Tensor, G: Tensor, damping: float) -> Tuple[Tensor, Tensor]:
    """[inv(A + r*pi*I), inv(G + (r/pi)*I)], r = sqrt(damping).
    torchsso/curv/curvature.py:302-312 with add_value_to_diagonal at :334-340."""
    pi = kron_pi(A, G)
    r = damping ** 0.5
    Ad = A + torch.eye(A.shape[0], dtype=A.dtype) * (r * pi)
    Gd = G + torch.eye(G.shape[0], dtype=G.dtype) * (r / pi)
    return spd_inverse(Ad), spd_inverse(Gd)


def diag_inverse(ema: Tensor, damping: float, use_sqrt: bool = False) -> Tensor:
    """1 / (ema [sqrt] + damping).  torchsso/curv/curvature.py:226-232."""
    x = ema.sqrt() if use_sqrt else ema
    return 1.0 / (x + damping)


# --------------------------------------------------------------------------
# precondition, std, sampling
# --------------------------------------------------------------------------
def kron_precondition(A_inv: Tensor, G_inv: Tensor, grad_w: Tensor,
                      grad_b: Optional[Tensor]) -> Tuple[Tensor, Optional[Tensor]]:
    """G^-1 [dW | db] A^-1 split back into weight and bias parts; dW is viewed
    [c_out, everything else].  torchsso/curv/cov/linear.py:69-84,
    torchsso/curv/cov/conv.py:76-92."""
    oc = grad_w.shape[0]
    g2d = grad_w.reshape(oc, -1)
    if grad_b is not None:
        g2d = torch.cat([g2d, grad_b.reshape(oc, 1)], dim=1)
    p = G_inv @ g2d @ A_inv
    if grad_b is not None:
        return p[:, :-1].reshape(grad_w.shape), p[:, -1].clone()
    return p.reshape(grad_w.shape), None


def cholesky_upper(m: Tensor) -> Tensor:
    """Upper factor U = L^T of m = L L^T.  torchsso/utils/cholesky_cupy.py:9-14
    (lower Cholesky, transposed when upper=True)."""
    return torch.linalg.cholesky(m).t().contiguous()


def kron_sample(mean_w: Tensor, mean_b: Optional[Tensor], U_A: Tensor, U_G: Tensor,
                noise: Tensor, std_scale: float) -> Tuple[Tensor, Optional[Tensor]]:
    """theta = [W | b] + s * U_G @ E @ U_A with E the supplied standard-normal matrix
    (the reference draws it with randn_like).  torchsso/curv/cov/linear.py:86-100,
    torchsso/curv/cov/conv.py:94-108."""
    oc = mean_w.shape[0]
    m = mean_w.reshape(oc, -1)
    if mean_b is not None:
        m = torch.cat([m, mean_b.reshape(oc, 1)], dim=1)
    p = m + std_scale * (U_G @ noise @ U_A)
    if mean_b is not None:
        return p[:, :-1].reshape(mean_w.shape), p[:, -1].clone()
    return p.reshape(mean_w.shape), None


def diag_sample(mean: Tensor, std: Tensor, noise: Tensor, std_scale: float) -> Tensor:
    """mean + s * noise * std.  torchsso/curv/curvature.py:243-246."""
    return mean + std_scale * noise * std


# --------------------------------------------------------------------------
# communicator semantics
# --------------------------------------------------------------------------
def tri_pack(m: Tensor) -> Tensor:
    """Row-major upper triangle (diagonal included) flattened row by row: element
    (y, x), x >= y, lands at  n*y - y*(y+1)/2 + x.  This is what cuBLAS trttp(LOWER)
    on the column-major view produces at
    torchsso/utils/chainer_communicators/_utility.py:59-86 and what the unpack index
    formula at :19-33 reads."""
    n = m.shape[0]
    iu = torch.triu_indices(n, n)
    return m[iu[0], iu[1]].clone()


def tri_unpack(v: Tensor, n: int) -> Tensor:
    """Symmetric matrix whose (y, x) and (x, y) both read packed element
    n*min - min*(min+1)/2 + max.  torchsso/utils/chainer_communicators/_utility.py:19-33."""
    out = torch.empty((n, n), dtype=v.dtype)
    iu = torch.triu_indices(n, n)
    out[iu[0], iu[1]] = v
    out[iu[1], iu[0]] = v
    return out


def reduce_scatterv_mean(per_rank_arrays: Sequence[Sequence[Tensor]]) -> List[Tensor]:
    """World mean of every array (what owners receive).
    torchsso/utils/chainer_communicators/pure_nccl_communicator.py:114-213:
    allReduce(SUM) of the packed buffer followed by a multiply with 1/size."""
    world = len(per_rank_arrays)
    out = []
    for arrs in zip(*per_rank_arrays):
        acc = arrs[0].clone()
        for a in arrs[1:]:
            acc = acc + a
        out.append(acc * (1.0 / world))
    return out


def owner_partition(num_groups: int, world: int) -> List[List[int]]:
    """Contiguous split of group indices over ranks (numpy.array_split rule: the first
    num_groups % world ranks get one extra).  torchsso/optim/secondorder.py:341-346."""
    return [part.tolist() for part in np.array_split(np.arange(num_groups), world)]
