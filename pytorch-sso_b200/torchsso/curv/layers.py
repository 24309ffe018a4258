"""Curvature classes per layer type, resolved by name (``shape + type + module class``) exactly
as torchsso/optim/secondorder.py:148-156 does: Kron{Cov,Fisher}{Linear,Conv2d},
Diag{Cov,Fisher}{Linear,Conv2d}, DiagCovBatchNorm{1d,2d}, DiagFisherBatchNorm2d and the full
Cov* placeholders.

Hot classes (Kron Linear/Conv2d, Diag BatchNorm) run on libsso_b200 kernels.  The diagonal
Linear/Conv2d curvatures (per-sample squared gradients, torchsso/curv/cov/linear.py:28-45,
torchsso/curv/cov/conv.py:15-42) are outside the accelerated path and are computed with plain
torch ops on the device.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as nat
from ..utils.accumulator import TensorAccumulator
from .curvature import Curvature, DiagCurvature, KronCurvature


class Fisher(object):
    """Mixin for Fisher curvatures: the closure built by get_closure_for_fisher runs extra
    backward passes ("sampling passes", do_backward True) weighted by ``prob`` and then the real
    backward (do_backward False), which finalises the accumulated curvature
    (torchsso/curv/fisher/__init__.py:7-31)."""

    def __init__(self):
        self.prob = None
        # set together with ``prob`` when every sample has the same weight (Monte Carlo Fisher:
        # 1/num_mc): the kernels then take the weight as part of their scalar alpha, which keeps
        # 16-bit inputs on the tensor-core path (per-sample weights would have to be rounded
        # into the operands)
        self.prob_scale = None
        self._do_backward = True
        self._acc_cov = TensorAccumulator()
        self._keep_output_edge = True     # the sampling passes ask autograd for the output gradient

    @property
    def do_backward(self):
        return self._do_backward

    def turn_on_backward(self):
        self._do_backward = True

    def turn_off_backward(self):
        self._do_backward = False

    def accumulate_cov(self, cov):
        self._acc_cov.update(cov)

    def finalize(self):
        return self._acc_cov.get()

    def update_as_presoftmax(self, prob):
        raise NotImplementedError('This method supports only torchsso.KronFisherLinear.')


def _weights(curv, n, device):
    """(per-sample weight vector or None, scalar weight) of the current sampling pass."""
    if not isinstance(curv, Fisher):
        return None, 1.0
    if curv.prob_scale is not None:
        return None, float(curv.prob_scale)
    assert curv.prob is not None
    w = curv.prob.detach().reshape(n)
    if w.dtype != torch.float32 or not w.is_contiguous():
        w = w.float().contiguous()
    if nat.curvature_stream_enabled() and w.is_cuda:
        # the hook's kernels run on the curvature stream while the closure, on its own stream, goes
        # on to rebind ``prob`` for the next class: without this the caching allocator could hand the
        # weight's block to the next allocation while a kernel here still reads it
        w.record_stream(torch.cuda.current_stream(w.device))
    return w, 1.0


def _fused_ema_coefficients(curv):
    """(scale of the new estimate, weight of the old average) when a hook writes the running
    average itself (torchsso/curv/curvature.py:174-191: ema <- data on first use or with decay 1,
    else decay * data + (1 - decay) * ema)."""
    b = curv.ema_decay
    if 'ema' not in curv._have or b == 1:
        return 1.0, 0.0
    return float(b), float(1.0 - b)


# ---------------------------------------------------------------------------------------------
# Kronecker-factored
# ---------------------------------------------------------------------------------------------
def _channels_last_if_worthwhile(t, d):
    """NCHW activations (channel stride != 1) can only use the exact-fp32 SIMT factor kernel; the
    tensor-core kernels gather whole 16-byte runs of channels.  For anything but tiny problems one
    extra pass over the activation (a layout copy to channels_last) is far cheaper than that."""
    if t.dim() != 4 or t.stride(1) == 1 or t.shape[1] == 1:
        return t
    rows = t.shape[0] * t.shape[2] * t.shape[3]
    if 2.0 * rows * d * d < 5e8:
        return t
    return t.contiguous(memory_format=torch.channels_last)


class _KronFactors(KronCurvature):
    """Shared driver: A in the forward hook, G (optionally prob-weighted and accumulated over
    sampling passes) in the backward hook, both by the fused factor kernel."""

    def _factor_A(self, x, out, scale=1.0, beta=0.0):
        raise NotImplementedError

    def _factor_G(self, g, weight, alpha_scale, beta, out):
        raise NotImplementedError

    def _op(self, x, geometry, append_ones, out):
        """Prepared factor call for this input layout (built on first sight of a shape/stride/dtype)."""
        ops = self.__dict__.setdefault('_ops', {})
        key = (x.shape, x.stride(), x.dtype, out.data_ptr())
        op = ops.get(key)
        if op is None:
            while len(ops) >= 16:          # oldest first: a second input shape must not evict the first
                ops.pop(next(iter(ops)))
            op = nat.FactorOp(x, *geometry, append_ones, out)
            ops[key] = op
        return op

    def _data_views(self):
        v = self.__dict__.get('_dv')
        if v is None or v[0] is not self._pool:
            v = (self._pool if self._pool is not None else self.pool, self._views('data'))
            self.__dict__['_dv'] = v
        return v[1]

    def _ema_views(self):
        v = self.__dict__.get('_ev')
        if v is None or v[0] is not self._pool:
            v = (self._pool if self._pool is not None else self.pool, self._views('ema'))
            self.__dict__['_ev'] = v
        return v[1]

    def update_in_forward(self, x):
        if self._fuse_ema:
            # the kernel's epilogue is the running average: ema <- b * A + (1 - b) * ema
            scale, beta = _fused_ema_coefficients(self)
            self._factor_A(x, self._ema_views()[0], scale, beta)
        else:
            self._factor_A(x, self._data_views()[0])

    def update_in_backward(self, g):
        fisher = isinstance(self, Fisher)
        if fisher and not self.do_backward:
            # real backward: the sampling passes already left  n^2 * sum_pass G_pass  in place
            self._g_passes = 0
            if not self._fuse_ema:
                self._have.add('data')
            return
        n = g.shape[0]
        later_pass = fisher and self._g_passes > 0
        w, ws = _weights(self, n, g.device)
        if self._fuse_ema:
            scale, beta = _fused_ema_coefficients(self)
            self._factor_G(g, w, scale * ws * float(n) * float(n), 1.0 if later_pass else beta, self._ema_views()[1])
        else:
            self._factor_G(g, w, ws * float(n) * float(n), 1.0 if later_pass else 0.0, self._data_views()[1])
            self._have.add('data')
        if fisher:
            self._g_passes += 1


class KronCovLinear(_KronFactors):
    """A = [x 1]^T [x 1] / n, G = g^T g / n (then * n^2).  torchsso/curv/cov/linear.py:48-115."""

    def _get_shape(self):
        f_out, f_in = self._module.weight.shape
        da = f_in + 1 if self.bias else f_in
        return (da, da), (f_out, f_out)

    _PLAIN = ((1, 1), (1, 1), (0, 0), (1, 1))

    def _factor_A(self, x, out, scale=1.0, beta=0.0):
        x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
        self._op(x2, self._PLAIN, self.bias, out).run(x2, None, scale / x2.shape[0], beta)

    def _factor_G(self, g, weight, scale, beta, out):
        g2 = g if g.dim() == 2 else g.reshape(-1, g.shape[-1])
        self._op(g2, self._PLAIN, False, out).run(g2, weight, scale / g2.shape[0], beta)


class KronCovConv2d(_KronFactors):
    """A = U^T U / n over the im2col rows U of the input (never materialised), G = g g^T / (n h w)
    with g viewed [c_out, n h w] (then * n^2).  torchsso/curv/cov/conv.py:45-124."""

    def _get_shape(self):
        c_out, c_in, kh, kw = self._module.weight.shape
        da = c_in * kh * kw + (1 if self.bias else 0)
        return (da, da), (c_out, c_out)

    def _factor_A(self, x, out, scale=1.0, beta=0.0):
        m = self._module
        if m.groups != 1 or isinstance(m.padding, str):
            raise NotImplementedError('grouped / string-padded convolutions have no Kronecker curvature here')
        n, c = x.shape[0], x.shape[1]
        vec = 4 if x.dtype == torch.float32 else 8
        x = _channels_last_if_worthwhile(x, c * m.kernel_size[0] * m.kernel_size[1])
        if x.stride(1) == 1 and c % vec != 0 and c < 64:
            # Channels-last input whose channel count is not a whole number of 16-byte chunks (the
            # 3-channel stem): zero-pad the channels so the tensor-core kernel applies, then keep
            # the rows / columns of the real channels.  Columns are ordered (c, kh, kw), so the
            # padding channels are a trailing block (followed by the ones column when there is a bias).
            cp = (c + vec - 1) // vec * vec
            kk = m.kernel_size[0] * m.kernel_size[1]
            xp = torch.empty((n, cp, x.shape[2], x.shape[3]), dtype=x.dtype, device=x.device,
                             memory_format=torch.channels_last)
            xp[:, c:].zero_()
            xp[:, :c] = x
            dp = cp * kk + (1 if self.bias else 0)
            if getattr(self, '_pad_buf', None) is None or self._pad_buf.shape[0] != dp:
                self._pad_buf = torch.empty((dp, dp), dtype=torch.float32, device=x.device)
            self._op(xp, (m.kernel_size, m.stride, m.padding, m.dilation), self.bias,
                     self._pad_buf).run(xp, None, 1.0 / n, 0.0, defer=False)      # read back right below
            d = c * kk

            def merge(dst, src):
                if beta == 0.0 and scale == 1.0:
                    dst.copy_(src)
                else:
                    dst.mul_(beta).add_(src, alpha=scale)
            merge(out[:d, :d], self._pad_buf[:d, :d])
            if self.bias:
                merge(out[:d, d], self._pad_buf[:d, dp - 1])
                merge(out[d, :d], self._pad_buf[dp - 1, :d])
                merge(out[d, d], self._pad_buf[dp - 1, dp - 1])
            return
        geometry = (m.kernel_size, m.stride, m.padding, m.dilation)
        self._op(x, geometry, self.bias, out).run(x, None, scale / n, beta)

    _PLAIN = ((1, 1), (1, 1), (0, 0), (1, 1))

    def _factor_G(self, g, weight, scale, beta, out):
        n, c, h, w = g.shape
        if c % (4 if g.dtype == torch.float32 else 8) == 0:
            g = _channels_last_if_worthwhile(g, c)
        self._op(g, self._PLAIN, False, out).run(g, weight, scale / (n * h * w), beta)


class KronFisherLinear(KronCovLinear, Fisher):

    def __init__(self, *args, **kwargs):
        KronCovLinear.__init__(self, *args, **kwargs)
        Fisher.__init__(self)

    def update_as_presoftmax(self, prob):
        # G = (diag(sum_n p) - p^T p / n) / n   (torchsso/curv/fisher/linear.py:59-63)
        n = prob.shape[0]
        G = self._views('data')[1]
        nat.factor_rows(prob.detach(), False, None, -1.0 / (n * n), 0.0, G)
        G.diagonal().add_(prob.detach().float().sum(dim=0) / n)
        self._have.add('data')


class KronFisherConv2d(KronCovConv2d, Fisher):

    def __init__(self, *args, **kwargs):
        KronCovConv2d.__init__(self, *args, **kwargs)
        Fisher.__init__(self)


# ---------------------------------------------------------------------------------------------
# diagonal BatchNorm (accelerated)
# ---------------------------------------------------------------------------------------------
class _DiagBatchNorm(DiagCurvature):
    """w = mean_n[(sum_hw xhat^2)(sum_hw p g^2)], b = mean_n[sum_hw p g^2], scaled by n^2, where
    xhat = (out - beta)/gamma is recovered from the layer OUTPUT (torchsso/curv/curvature.py:123-134,
    torchsso/curv/cov/batchnorm.py:10-49).  The per-(n,c) sums of xhat^2 are taken in the forward
    hook, so later in-place edits of the output (ReLU, residual add) cannot disturb them."""

    def __init__(self, *args, **kwargs):
        super(_DiagBatchNorm, self).__init__(*args, **kwargs)
        self._sx = None
        self._sg = None
        self._splits_x = 1
        self._passes = 0

    @staticmethod
    def _buffer(buf, numel, device):
        if buf is None or buf.numel() < numel or buf.device != device:
            buf = torch.empty(numel, dtype=torch.float32, device=device)
        return buf

    def _layout(self, t):
        """(strides, splits) of the plane-sum kernel for this tensor layout, cached."""
        cache = self.__dict__.setdefault('_layouts', {})
        key = (t.shape, t.stride(), t.dtype, t.data_ptr() % 16)
        ent = cache.get(key)
        if ent is None:
            while len(cache) >= 16:
                cache.pop(next(iter(cache)))
            t2, st, splits = nat.bn_plane_layout(t)
            ent = (st, splits, t2 is t)
            cache[key] = ent
        if not ent[2]:
            t = t.contiguous()
        return (t, ent[0], ent[1])

    def update_in_forward(self, out):
        bn = self._module
        if bn.weight is None:
            raise NotImplementedError('affine=False normalisation has no parameters to precondition')
        layout = self._layout(out)
        self._sx = self._buffer(self._sx, out.shape[0] * layout[2] * out.shape[1], out.device)
        self._splits_x = nat.bn_plane_sums(layout[0], True, bn.weight.detach(), bn.bias.detach(), self._sx, layout)

    def update_in_backward(self, g):
        fisher = isinstance(self, Fisher)
        if fisher and not self.do_backward:
            self._passes = 0
            if not self._fuse_ema:
                self._have.add('data')
            return
        n, c = g.shape[0], g.shape[1]
        layout = self._layout(g)
        self._sg = self._buffer(self._sg, n * layout[2] * c, g.device)
        splits_g = nat.bn_plane_sums(layout[0], False, None, None, self._sg, layout)
        later_pass = fisher and self._passes > 0
        role = 'ema' if self._fuse_ema else 'data'
        views = self.__dict__.get('_bnv')
        if views is None or views[0] is not self._pool or views[2] != role:
            views = (self._pool if self._pool is not None else self.pool, self._views(role), role)
            self.__dict__['_bnv'] = views
        views = views[1]
        w, ws = _weights(self, n, g.device)
        scale, beta = _fused_ema_coefficients(self) if self._fuse_ema else (1.0, 0.0)
        nat.bn_diag_finish(self._sx, self._sg, w, n, c, self._splits_x, splits_g, scale * ws * float(n) * float(n),
                           1.0 if later_pass else beta, views[0], views[1] if len(views) > 1 else None)
        if fisher:
            self._passes += 1
        if not self._fuse_ema:
            self._have.add('data')


class DiagCovBatchNorm1d(_DiagBatchNorm):
    pass


class DiagCovBatchNorm2d(_DiagBatchNorm):
    pass


class DiagFisherBatchNorm2d(DiagCovBatchNorm2d, Fisher):

    def __init__(self, *args, **kwargs):
        DiagCovBatchNorm2d.__init__(self, *args, **kwargs)
        Fisher.__init__(self)


# ---------------------------------------------------------------------------------------------
# diagonal Linear / Conv2d: mean over samples of the squared per-sample gradient
# ---------------------------------------------------------------------------------------------
class _DiagSq(DiagCurvature):
    """torchsso/curv/cov/linear.py:28-45 and torchsso/curv/cov/conv.py:15-42 (the Fisher variants
    weight each sample by its probability, torchsso/curv/fisher/linear.py:11-32): one launch of
    the fused kernel per backward pass; the im2col matrix and the per-sample gradients are never
    materialised."""

    def _geometry(self):
        raise NotImplementedError

    def _operands(self, x, g):
        return x, g

    def update_in_backward(self, g):
        fisher = isinstance(self, Fisher)
        if not hasattr(self, '_passes'):
            self._passes = 0
        if fisher and not self.do_backward:
            self._passes = 0
            return
        x, g = self._operands(self._module.data_input, g)
        n = g.shape[0]
        p, ws = _weights(self, n, g.device)
        views = self._views('data')
        first = not (fisher and self._passes > 0)
        # mean over samples, then the n^2 that undoes the mean reduction of the loss
        nat.diag_sq(x, g, *self._geometry(), p, ws * float(n), 0.0 if first else 1.0,
                    views[0], views[1] if self.bias else None)
        if fisher:
            self._passes += 1
        self._have.add('data')


class DiagCovLinear(_DiagSq):

    def _geometry(self):
        return (1, 1), (1, 1), (0, 0), (1, 1)

    def _operands(self, x, g):
        if x.dim() != 2:        # [.., f_in]: every leading index is a sample
            x, g = x.reshape(-1, x.shape[-1]), g.reshape(-1, g.shape[-1])
        return x, g


class DiagCovConv2d(_DiagSq):

    def _geometry(self):
        m = self._module
        if m.groups != 1 or isinstance(m.padding, str):
            raise NotImplementedError('grouped / string-padded convolutions have no diagonal curvature here')
        return m.kernel_size, m.stride, m.padding, m.dilation


class DiagFisherLinear(DiagCovLinear, Fisher):

    def __init__(self, *args, **kwargs):
        DiagCovLinear.__init__(self, *args, **kwargs)
        Fisher.__init__(self)


class DiagFisherConv2d(DiagCovConv2d, Fisher):

    def __init__(self, *args, **kwargs):
        DiagCovConv2d.__init__(self, *args, **kwargs)
        Fisher.__init__(self)


# ---------------------------------------------------------------------------------------------
# full-matrix curvatures: outside the accelerated path
# ---------------------------------------------------------------------------------------------
class CovLinear(Curvature):
    """Full covariance of the per-sample gradients of a Linear layer, [(f_out (f_in+1))^2]
    (torchsso/curv/cov/linear.py:5-25).  Not part of the accelerated path: built with plain torch
    ops on the device, as the reference does; like the reference's, ``precondition_grad`` leaves
    the gradient untouched."""

    def update_in_backward(self, grad_output):
        x = self._module.__dict__.get('data_input')
        assert x is not None
        n = x.shape[0]
        x, g = x.float(), grad_output.float()
        if self.bias:
            x = torch.cat((x, x.new_ones((n, 1))), 1)
        per_sample = torch.einsum('bi,bj->bij', g, x).reshape(n, -1)
        self._generic['data'] = [per_sample.t() @ per_sample]

    def update_ema(self):
        first = self._ema_bookkeeping() or 'ema' not in self._generic
        data, beta = self._generic['data'], self.ema_decay
        if first:
            self._generic['ema'] = [d.clone() for d in data]
        else:
            self._generic['ema'] = [d.mul(beta).add_(e, alpha=1 - beta) for d, e in zip(data, self._generic['ema'])]
        self._have.add('ema')

    def update_inv(self):
        from ..utils import linalg
        out = []
        for e in self._generic['ema']:
            m = e.clone()
            m.diagonal().add_(self.damping)
            out.append(linalg.inv(m))
        self._generic['inv'] = out

    def precondition_grad(self, params):
        pass


class _NoFullCurvature(Curvature):
    """The reference ships these classes as stubs (``update_in_backward`` is ``pass``,
    torchsso/curv/cov/conv.py:6-13, torchsso/curv/cov/batchnorm.py:4-7,28-31) whose first ``step()``
    fails on the missing data.  Fail at construction instead, with the reason."""

    def __init__(self, module, *args, **kwargs):
        raise NotImplementedError(
            '%s: a full-matrix curvature for %s does not exist (a stub in the reference as well); '
            "use the 'Kron' or 'Diag' shape for this module" % (type(self).__name__, type(module).__name__))


class CovConv2d(_NoFullCurvature):
    pass


class CovBatchNorm1d(_NoFullCurvature):
    pass


class CovBatchNorm2d(_NoFullCurvature):
    pass
