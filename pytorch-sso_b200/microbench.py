"""Operator-level microbenchmarks of libsso_b200 (one JSON line per case).

    python pytorch-sso_b200/microbench.py factor   [--dtype bf16|fp32] [--case I] [--iters K]
    python pytorch-sso_b200/microbench.py batch    [--case 0|1]    all ResNet-50 A / G factors: one batched call vs one call each
    python pytorch-sso_b200/microbench.py rows     [--case I]      fp32 X^T X, d in 64..4608
    python pytorch-sso_b200/microbench.py inverse  [--case I]      damped SPD inverse, d in 64..4608
    python pytorch-sso_b200/microbench.py precond  [--case I]      G^-1 dW A^-1
    python pytorch-sso_b200/microbench.py stream                   EMA / axpby / BN plane sums / triangular pack and unpack
    python pytorch-sso_b200/microbench.py steps    [--case 0..3]   whole steps of the smaller reference configurations
    python pytorch-sso_b200/microbench.py peaks                    cuBLAS bf16 / TF32 GEMM and copy, for reference
    torchrun ... pytorch-sso_b200/microbench.py collective         factor exchange sweep (N > 1)

Inputs are seeded N(0,1) tensors created on the device; every case moves more bytes than the
L2 holds or is timed over launches on rotating buffers, and times are CUDA-event times on
the launching stream after warm-up.  ``--case I`` runs a single case (what a profiler capture
wants); without it the whole suite runs.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

from torchsso import _native as nat  # noqa: E402

# (c, h, w, k, stride, pad) of the distinct ResNet-50 convolutions' A factors at 224x224 input
R50_CONVS = [
    (64, 56, 56, 1, 1, 0), (64, 56, 56, 3, 1, 1), (256, 56, 56, 1, 1, 0), (128, 56, 56, 3, 2, 1),
    (128, 28, 28, 3, 1, 1), (512, 28, 28, 1, 1, 0), (256, 28, 28, 3, 2, 1), (256, 14, 14, 3, 1, 1),
    (1024, 14, 14, 1, 1, 0), (512, 14, 14, 3, 2, 1), (512, 7, 7, 3, 1, 1), (2048, 7, 7, 1, 1, 0),
]
DIMS = [64, 256, 576, 1152, 2304, 4608]
# (d_A, d_G) of representative ResNet-50 layers
R50_PAIRS = [(576, 64), (256, 64), (1152, 128), (2304, 256), (1024, 256), (4608, 512), (2048, 512), (2049, 1000)]


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def emit(**kw):
    print(json.dumps(kw), flush=True)


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', 'MEASURED_PEAKS.json')
    try:
        p = json.load(open(path))
        return float(p['hbm_gbs']), float(p['bf16_tflops'])
    except Exception:
        return 6650.0, 1590.0


def select(cases, idx):
    return list(enumerate(cases)) if idx is None else [(idx, cases[idx])]


def suite_factor(args):
    dt = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp32': torch.float32}[args.dtype]
    n = args.batch
    _, tf_peak = peaks()
    for i, (c, h, w, k, s, p) in select(R50_CONVS, args.case):
        g = torch.Generator(device='cuda').manual_seed(i)
        xs = [torch.randn((n, c, h, w), device='cuda', generator=g).to(dt).contiguous(
            memory_format=torch.channels_last) for _ in range(args.rotate)]
        d = c * k * k
        out = torch.empty((d, d), device='cuda')
        ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        rows = n * ho * wo
        state = {'i': 0}

        def run():
            x = xs[state['i'] % len(xs)]
            state['i'] += 1
            nat.factor_im2col(x, (k, k), (s, s), (p, p), (1, 1), False, None, 1.0 / n, 0.0, out, args.impl)
        ms = timeit(run, args.iters)
        tf = 2.0 * rows * d * d / ms / 1e9
        emit(suite='factor', case=i, dtype=args.dtype, conv=dict(n=n, c=c, h=h, w=w, k=k, stride=s, pad=p),
             rows=rows, d=d, ms=round(ms, 4), tflops=round(tf, 1), frac_of_measured_bf16=round(tf / tf_peak, 3),
             input_gbs=round(xs[0].numel() * xs[0].element_size() / ms / 1e6, 1))


def suite_rows(args):
    _, tf_peak = peaks()
    for i, d in select(DIMS, args.case):
        rows = args.rows if args.rows else max(8192, min(802816, (1 << 31) // (4 * d)))
        g = torch.Generator(device='cuda').manual_seed(i)
        x = torch.randn((rows, d), device='cuda', generator=g)
        out = torch.empty((d, d), device='cuda')
        ms = timeit(lambda: nat.factor_rows(x, False, None, 1.0 / rows, 0.0, out, args.impl), args.iters)
        tf = 2.0 * rows * d * d / ms / 1e9
        emit(suite='rows', case=i, dtype='fp32 (3xTF32)', rows=rows, d=d, ms=round(ms, 4), tflops=round(tf, 1),
             tensor_tflops=round(3 * tf, 1), frac_of_measured_bf16=round(3 * tf / tf_peak, 3),
             input_gbs=round(4.0 * rows * d / ms / 1e6, 1))


# (n, c, h, w, oc, k, stride, pad): convolutions of the VGG / ResNet configurations, and two Linear
# layers written as 1x1 convolutions over one pixel
DIAG_CASES = [(128, 64, 32, 32, 64, 3, 1, 1), (128, 256, 8, 8, 256, 3, 1, 1), (32, 64, 56, 56, 64, 3, 1, 1),
              (32, 256, 14, 14, 256, 3, 1, 1), (128, 512, 1, 1, 10, 1, 1, 0), (128, 4096, 1, 1, 1000, 1, 1, 0)]


def suite_diag(args):
    """Squared per-sample gradient kernel (diagonal curvature of Linear / Conv2d): exact fp32 FFMA,
    2 * n * L * oc * d flops per launch."""
    for i, (n, c, h, w, oc, k, s, p) in select(DIAG_CASES, args.case):
        g = torch.Generator(device='cuda').manual_seed(i)
        ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        x = torch.randn((n, c, h, w), device='cuda', generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
        go = torch.randn((n, oc, ho, wo), device='cuda', generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
        d = c * k * k
        ow, ob = torch.empty((oc, d), device='cuda'), torch.empty((oc,), device='cuda')
        ms = timeit(lambda: nat.diag_sq(x, go, (k, k), (s, s), (p, p), (1, 1), None, 1.0 / n, 0.0, ow, ob), args.iters)
        fl = 2.0 * n * ho * wo * oc * d
        emit(suite='diag', case=i, dtype='bf16 in, fp32 math', n=n, c=c, hw=[h, w], oc=oc, k=k, ms=round(ms, 4),
             tflops=round(fl / ms / 1e9, 2))


def spd(d, seed):
    g = torch.Generator(device='cuda').manual_seed(seed)
    x = torch.randn((4 * d, d), device='cuda', generator=g)
    return (x.t() @ x) / x.shape[0]


def suite_inverse(args):
    for i, d in select(DIMS, args.case):
        A, G = spd(d, 2 * i), spd(d, 2 * i + 1)
        src = [A, G]
        dst = [torch.empty_like(m) for m in src]
        work = [torch.empty_like(m) for m in src]
        plan = nat.kron_plan([d, d], src, dst, work, None, [1, 0], [0, 1], torch.device('cuda'))
        damp = torch.full((2,), math.sqrt(1e-3), device='cuda')
        info = torch.zeros(4, dtype=torch.int32, device='cuda')
        ms = timeit(lambda: nat.kron_plan_run(plan, damp, info, True, False), args.iters)
        assert int(info.abs().sum()) == 0
        eye = torch.eye(d, device='cuda')
        r = math.sqrt(1e-3)
        pi = math.sqrt((A.trace() / d / (G.trace() / d)).item())
        resid = ((A + r * pi * eye) @ dst[0] - eye).norm().item() / math.sqrt(d)
        emit(suite='inverse', case=i, d=d, matrices=2, ms=round(ms, 4),
             gflops=round(2 * d ** 3 / ms / 1e6, 1), residual=float('%.3g' % resid))


def suite_precond(args):
    for i, (da, dg) in select(R50_PAIRS, args.case):
        Ai, Gi = spd(da, 50 + i), spd(dg, 80 + i)
        g = torch.Generator(device='cuda').manual_seed(i)
        gw = torch.randn((dg, da), device='cuda', generator=g) * 0.1
        tmp = torch.empty(dg * da, device='cuda')
        plan = nat.precond_plan([da], [dg], [Ai], [Gi], [gw], [None], [tmp], torch.device('cuda'))
        ms = timeit(lambda: nat.precond_plan_run(plan), args.iters)
        fl = 2.0 * dg * da * (da + dg)
        emit(suite='precond', case=i, dA=da, dG=dg, ms=round(ms, 4), tflops=round(fl / ms / 1e9, 2))


def suite_stream(args):
    hbm, _ = peaks()
    n = 1 << 27                                # 512 MiB per fp32 array
    a = torch.randn(n, device='cuda')
    b = torch.randn(n, device='cuda')
    ms = timeit(lambda: nat.ema_update(a, b, 0.95, False), args.iters)
    emit(suite='stream', kernel='ema_update', bytes=12 * n, ms=round(ms, 4), gbs=round(12.0 * n / ms / 1e6, 1),
         frac_of_measured_hbm=round(12.0 * n / ms / 1e6 / hbm, 3))
    # triangular pack / unpack of the exchange (two 4608^2 and eight 1152^2 factors, as the communicator does it)
    mats = [torch.randn((4608, 4608), device='cuda') for _ in range(2)] + [torch.randn((1152, 1152), device='cuda') for _ in range(8)]
    offs, off = [], 0
    for m in mats:
        offs.append(off)
        off += m.shape[0] * (m.shape[0] + 1) // 2
    buf = torch.empty(off, device='cuda')
    t_pack, t_unpack = nat.tri_records(mats, buf, offs), nat.tri_records(mats, buf, offs, 32)
    full = sum(m.numel() for m in mats) * 4
    ms = timeit(lambda: nat.tri_pack(t_pack, 0.5), args.iters)
    emit(suite='stream', kernel='tri_pack', bytes=2 * off * 4, ms=round(ms, 4), gbs=round(2 * off * 4 / ms / 1e6, 1),
         frac_of_measured_hbm=round(2 * off * 4 / ms / 1e6 / hbm, 3))
    ms = timeit(lambda: nat.tri_unpack(t_unpack, 1.0, True), args.iters)
    emit(suite='stream', kernel='tri_unpack (symmetric)', bytes=off * 4 + full, ms=round(ms, 4),
         gbs=round((off * 4 + full) / ms / 1e6, 1), frac_of_measured_hbm=round((off * 4 + full) / ms / 1e6 / hbm, 3))
    ms = timeit(lambda: nat.axpby(a, b, 0.5, 0.5), args.iters)
    emit(suite='stream', kernel='axpby', bytes=12 * n, ms=round(ms, 4), gbs=round(12.0 * n / ms / 1e6, 1),
         frac_of_measured_hbm=round(12.0 * n / ms / 1e6 / hbm, 3))
    x = torch.randn((128, 256, 56, 56), device='cuda').to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    layout = nat.bn_plane_layout(x)
    out = torch.empty((layout[2] * 128 * 256,), device='cuda')
    ms = timeit(lambda: nat.bn_plane_sums(x, False, None, None, out, layout), args.iters)
    nb = x.numel() * 2
    emit(suite='stream', kernel='bn_plane_sums', bytes=nb, ms=round(ms, 4), gbs=round(nb / ms / 1e6, 1),
         frac_of_measured_hbm=round(nb / ms / 1e6 / hbm, 3))


def suite_peaks(args):
    """Library peaks on this GPU, timed like the other suites: cuBLAS bf16 and TF32 GEMM (the
    3xTF32 kernels spend three TF32 MMAs per product, so their ceiling is a third of the TF32
    figure) and a device-to-device copy."""
    n = 8192
    for name, dt, tf32 in (('bf16', torch.bfloat16, False), ('tf32', torch.float32, True)):
        torch.backends.cuda.matmul.allow_tf32 = tf32
        a = torch.randn((n, n), device='cuda', dtype=dt)
        b = torch.randn((n, n), device='cuda', dtype=dt)
        c = torch.empty((n, n), device='cuda', dtype=dt)
        ms = timeit(lambda: torch.matmul(a, b, out=c), args.iters)
        emit(suite='peaks', kernel='cuBLAS %s gemm %d^3' % (name, n), ms=round(ms, 4),
             tflops=round(2.0 * n ** 3 / ms / 1e9, 1))
    torch.backends.cuda.matmul.allow_tf32 = False
    x = torch.empty(1 << 28, device='cuda')
    y = torch.empty(1 << 28, device='cuda')
    ms = timeit(lambda: y.copy_(x), args.iters)
    emit(suite='peaks', kernel='copy 1 GiB', ms=round(ms, 4), gbs=round(2.0 * 4 * (1 << 28) / ms / 1e6, 1))


def suite_steps(args):
    """Whole optimizer steps of the smaller reference configurations (fp32, eager launches, a fresh
    seeded batch every step): the 784-1000-1000-10 MLP at batch 128 with inverses every step, the
    5x5/5x5/3x3 ConvNet at batch 256 with inverses every 5 steps (also with four Monte Carlo targets per
    step, as one batched sampling pass and as one pass per target), and the VGG-16-style network under
    VIOptimizer with 4 weight samples per step at batch 128."""
    import torch.nn as nn
    import torch.nn.functional as F
    import torchsso

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.f1, self.f2, self.f3 = nn.Linear(784, 1000), nn.Linear(1000, 1000), nn.Linear(1000, 10)

        def forward(self, x):
            return self.f3(F.relu(self.f2(F.relu(self.f1(x.flatten(1))))))

    class ConvNet(nn.Module):
        def __init__(self):
            super().__init__()
            self.c1, self.c2 = nn.Conv2d(3, 64, 5, padding=2), nn.Conv2d(64, 128, 5, padding=2)
            self.c3 = nn.Conv2d(128, 256, 3, padding=1)
            self.f1, self.f2 = nn.Linear(4096, 512), nn.Linear(512, 10)

        def forward(self, x):
            x = F.max_pool2d(F.relu(self.c1(x)), 2)
            x = F.max_pool2d(F.relu(self.c2(x)), 2)
            x = F.max_pool2d(F.relu(self.c3(x)), 2)
            return self.f2(F.relu(self.f1(x.flatten(1))))

    class VGG(nn.Module):
        def __init__(self):
            super().__init__()
            cfg = [64, 64, 'M', 128, 128, 'M', 256, 256, 256, 'M', 512, 512, 512, 'M', 512, 512, 512, 'M']
            layers, c = [], 3
            for v in cfg:
                if v == 'M':
                    layers.append(None)
                else:
                    layers.append(nn.Conv2d(c, v, 3, padding=1))
                    c = v
            self.convs = nn.ModuleList([l for l in layers if l is not None])
            self.plan = [l is not None for l in layers]
            self.fc = nn.Linear(512, 100)

        def forward(self, x):
            it = iter(self.convs)
            for is_conv in self.plan:
                x = F.relu(next(it)(x)) if is_conv else F.max_pool2d(x, 2)
            return self.fc(x.flatten(1))

    kron = {'Conv2d': 'Kron', 'Linear': 'Kron'}
    kw = {'ema_decay': 0.95, 'damping': 1e-3}
    dev = torch.device('cuda')

    def batches(shape, classes, count=8):
        g = torch.Generator(device='cuda').manual_seed(11)
        xs = [torch.randn(shape, device='cuda', generator=g) for _ in range(count)]
        ys = [torch.randint(0, classes, (shape[0],), device='cuda', generator=g) for _ in range(count)]
        return xs, ys

    def run(name, step, batch, iters):
        for i in range(3):
            step(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            loss = step(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        emit(suite='steps', config=name, batch=batch, ms_per_step=round(ms, 3),
             images_per_sec=round(batch / ms * 1e3, 1), last_loss=round(float(loss), 4))

    torch.manual_seed(0)
    want = lambda k: args.case is None or args.case == k      # --case: 0 MLP, 1 ConvNet, 2 ConvNet with 4 targets, 3 VGG / VI
    if want(0):
        # MLP, inverse every step
        model = MLP().to(dev)
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', kron, kw, lr=1e-2)
        xs, ys = batches((128, 1, 28, 28), 10)
        x, y = xs[0].clone(), ys[0].clone()
        closure = torchsso.get_closure_for_fisher(opt, model, x, y, approx_type='mc', num_mc=1)

        def step_mlp(i):
            x.copy_(xs[i % 8]); y.copy_(ys[i % 8])
            opt.update_inv = True
            return opt.step(closure=closure)[0]
        run('mlp 784-1000-1000-10, Fisher MC, inverse every step', step_mlp, 128, args.iters * 3)

    if want(1) or want(2):
        # ConvNet (NCHW, as a reference user would run it), inverse every 5 steps
        model2 = ConvNet().to(dev)
        opt2 = torchsso.optim.SecondOrderOptimizer(model2, 'Fisher', kron, kw, lr=1e-3)
        xs2, ys2 = batches((256, 3, 32, 32), 10)
        x2, y2 = xs2[0].clone(), ys2[0].clone()
    if want(1):
        closure2 = torchsso.get_closure_for_fisher(opt2, model2, x2, y2, approx_type='mc', num_mc=1)

        def step_conv(i):
            x2.copy_(xs2[i % 8]); y2.copy_(ys2[i % 8])
            opt2.update_inv = (i % 5 == 0)
            return opt2.step(closure=closure2)[0]
        run('convnet 5x5-5x5-3x3 + 4096-512-10, Fisher MC, inverse every 5', step_conv, 256, args.iters * 2)

    if want(2):
        # the same ConvNet with four Monte Carlo targets per step: one walk of the graph for all of them
        # against one walk per target (the reference's loop, torchsso/curv/fisher/__init__.py:65-72)
        for batched in (True, False):
            model4 = ConvNet().to(dev)
            opt4 = torchsso.optim.SecondOrderOptimizer(model4, 'Fisher', kron, kw, lr=1e-3)
            closure4 = torchsso.get_closure_for_fisher(opt4, model4, x2, y2, approx_type='mc', num_mc=4,
                                                       batch_mc_passes=batched)

            def step_mc(i):
                x2.copy_(xs2[i % 8]); y2.copy_(ys2[i % 8])
                opt4.update_inv = (i % 5 == 0)
                return opt4.step(closure=closure4)[0]
            run('convnet, Fisher MC with 4 targets, %s' % ('one batched sampling pass' if batched else 'one pass per target'),
                step_mc, 256, args.iters * 2)

    if want(3):
        # VGG-16-style under VIOptimizer, 4 weight samples per step
        model3 = VGG().to(dev)
        # kl_weighting 0.01 (the start value of the reference's warm-up, vi.py:302-319): with 1.0 the weight
        # noise of the untrained network overflows the activations on N(0,1) inputs within two steps
        opt3 = torchsso.optim.VIOptimizer(model3, 50000, 'Cov', kron, kw, lr=1e-3, num_mc_samples=4,
                                          kl_weighting=0.01, prior_variance=1)
        xs3, ys3 = batches((128, 3, 32, 32), 100, count=4)
        x3, y3 = xs3[0].clone(), ys3[0].clone()

        def closure3():
            opt3.zero_grad()
            o = model3(x3)
            loss = F.cross_entropy(o, y3)
            loss.backward()
            return loss, o

        def step_vi(i):
            x3.copy_(xs3[i % 4]); y3.copy_(ys3[i % 4])
            return opt3.step(closure=closure3)[0]
        run('vgg16-style, VIOptimizer, 4 MC samples, inverse + std every step', step_vi, 128, max(3, args.iters // 2))


def suite_collective(args):
    """Reduce-scatter of the tri-packed ResNet-50 factors to owner ranks and all-gather of the
    parameter-sized updates, as the distributed optimizer issues them (padded equal segments)."""
    import torch.distributed as dist
    from torchsso.utils.communicator import assign_owners
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', 0)))
    dist.init_process_group('nccl', device_id=torch.device('cuda', torch.cuda.current_device()))
    layers = []
    for (c, h, w, k, s, p), reps, oc in zip(R50_CONVS, [1, 3, 2, 1, 3, 3, 1, 5, 5, 1, 2, 2],
                                            [64, 64, 64, 128, 128, 128, 256, 256, 256, 512, 512, 512]):
        layers += [(c * k * k, oc)] * reps
    layers.append((2049, 1000))
    owners = assign_owners([a ** 3 + g ** 3 for a, g in layers], world)
    tri = lambda d: d * (d + 1) // 2
    seg = max(sum(tri(layers[i][0]) + tri(layers[i][1]) + layers[i][0] * layers[i][1] for i in own)
              for own in owners)
    seg = (seg + 255) // 256 * 256
    send = torch.randn(seg * world, device='cuda')
    recv = torch.empty(seg, device='cuda')
    pseg = max(sum(layers[i][0] * layers[i][1] for i in own) for own in owners)
    pseg = (pseg + 255) // 256 * 256
    psend = torch.randn(pseg, device='cuda')
    precv = torch.empty(pseg * world, device='cuda')

    def timed(fn):
        dist.barrier()
        ms = torch.tensor([timeit(fn, args.iters)], device='cuda')
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()
    ms_rs = timed(lambda: dist.reduce_scatter_tensor(recv, send, op=dist.ReduceOp.SUM))
    ms_ag = timed(lambda: dist.all_gather_into_tensor(precv, psend))
    if rank == 0:
        f = (world - 1) / world
        emit(suite='collective', op='reduce_scatter(factors+grads)', world=world, bytes=4 * seg * world,
             ms=round(ms_rs, 4), bus_gbs=round(4.0 * seg * world * f / ms_rs / 1e6, 1), nominal_gbs=900)
        emit(suite='collective', op='all_gather(updates)', world=world, bytes=4 * pseg * world,
             ms=round(ms_ag, 4), bus_gbs=round(4.0 * pseg * world * f / ms_ag / 1e6, 1), nominal_gbs=900)
    # sweep over the distinct (d_A, d_G) pairs of the model: the exchange of ONE layer (packed A and G
    # plus the gradient), cut into `world` equal segments, reduce-scattered and all-gathered; bus
    # bandwidth against bytes shows where the collectives leave the latency-bound regime
    for a, g in sorted(set(layers), key=lambda ag: tri(ag[0]) + tri(ag[1]) + ag[0] * ag[1]):
        n = tri(a) + tri(g) + a * g
        sg = (n + world - 1) // world
        sg = (sg + 63) // 64 * 64
        s_buf = torch.randn(sg * world, device='cuda')
        r_buf = torch.empty(sg, device='cuda')
        t_rs = timed(lambda: dist.reduce_scatter_tensor(r_buf, s_buf, op=dist.ReduceOp.SUM))
        t_ag = timed(lambda: dist.all_gather_into_tensor(s_buf, r_buf))
        if rank == 0:
            f = (world - 1) / world
            emit(suite='collective_sweep', dA=a, dG=g, world=world, bytes=4 * sg * world,
                 reduce_scatter_ms=round(t_rs, 4), reduce_scatter_bus_gbs=round(4.0 * sg * world * f / t_rs / 1e6, 1),
                 all_gather_ms=round(t_ag, 4), all_gather_bus_gbs=round(4.0 * sg * world * f / t_ag / 1e6, 1),
                 nominal_gbs=900)
    dist.barrier()
    dist.destroy_process_group()


def r50_convs(batch):
    """(c_in, h, w, kernel, stride, pad, c_out, h_out, w_out) of every convolution of the benchmark's
    ResNet-50 at 224x224, taken from a shape-only forward pass of the model itself."""
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), '..')
    if root not in sys.path:
        sys.path.insert(0, root)
    import bench
    with torch.device('meta'):
        model = bench.ResNet50()
    out = []

    def hook(m, inp, res):
        x = inp[0]
        out.append((x.shape[1], x.shape[2], x.shape[3], m.kernel_size[0], m.stride[0], m.padding[0],
                    res.shape[1], res.shape[2], res.shape[3]))
    for m in model.modules():
        if isinstance(m, torch.nn.Conv2d):
            m.register_forward_hook(hook)
    model(torch.empty((batch, 3, 224, 224), device='meta'))
    return out


def suite_batch(args):
    """All A factors (or all G factors) of ResNet-50's convolutions, bf16, as ONE sso_factor_batch call,
    against the same problems issued one sso_factor_syrk_im2col call at a time (the 3-channel stem is
    left out of both: its input is the fp32 image)."""
    n = args.batch
    convs = [c for c in r50_convs(n) if c[0] % 64 == 0]
    cl = torch.channels_last
    g = torch.Generator(device='cuda').manual_seed(0)
    for which in ('A', 'G'):
        items, flops, nbytes_in = [], 0.0, 0
        for (cin, h, w, k, st, pad, cout, ho, wo) in convs:
            if which == 'A':
                x = torch.randn((n, cin, h, w), device='cuda', generator=g).bfloat16().contiguous(memory_format=cl)
                geo, d, rows = ((k, k), (st, st), (pad, pad), (1, 1)), cin * k * k, n * ho * wo
            else:
                x = torch.randn((n, cout, ho, wo), device='cuda', generator=g).bfloat16().contiguous(memory_format=cl)
                geo, d, rows = ((1, 1), (1, 1), (0, 0), (1, 1)), cout, n * ho * wo
            items.append((x, geo, torch.empty((d, d), device='cuda')))
            flops += 2.0 * rows * d * d
            nbytes_in += x.numel() * 2
        arr = (nat.FactorDesc * len(items))()
        for dsc, (x, geo, out) in zip(arr, items):
            dsc.x, dsc.dtype, dsc.append_ones = x.data_ptr(), nat.BF16, 0
            dsc.n, dsc.c, dsc.h, dsc.w = x.shape
            dsc.sn, dsc.sc, dsc.sh, dsc.sw = x.stride()
            (dsc.kh, dsc.kw), (dsc.stride_h, dsc.stride_w), (dsc.pad_h, dsc.pad_w), (dsc.dil_h, dsc.dil_w) = geo
            dsc.sample_weight, dsc.alpha, dsc.beta, dsc.out, dsc.ldo = None, 1.0 / n, 0.0, out.data_ptr(), out.stride(0)
        L = nat.lib()
        nb = L.sso_factor_batch_workspace_bytes(len(items), arr)
        ws = torch.empty(nb, dtype=torch.uint8, device='cuda')

        def batched():
            nat._check(L.sso_factor_batch(len(items), arr, ws.data_ptr(), nb, torch.cuda.current_stream().cuda_stream))

        def one_by_one():
            for x, geo, out in items:
                nat.factor_im2col(x, *geo, False, None, 1.0 / n, 0.0, out)
        if args.case in (None, 0):
            ms_b = timeit(batched, args.iters)
            emit(suite='batch', which=which, mode='one sso_factor_batch call', problems=len(items), ms=round(ms_b, 4),
                 tflops_algorithmic=round(flops / ms_b / 1e9, 1), input_mb=round(nbytes_in / 1e6, 1),
                 scratch_mb=round(nb / 1e6, 1))
        if args.case in (None, 1):
            ms_s = timeit(one_by_one, args.iters)
            emit(suite='batch', which=which, mode='one call per problem', problems=len(items), ms=round(ms_s, 4),
                 tflops_algorithmic=round(flops / ms_s / 1e9, 1))
        del items, ws


SUITES = {'batch': suite_batch, 'diag': suite_diag, 'peaks': suite_peaks, 'steps': suite_steps, 'factor': suite_factor, 'rows': suite_rows, 'inverse': suite_inverse, 'precond': suite_precond,
          'stream': suite_stream, 'collective': suite_collective}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('suite', choices=sorted(SUITES))
    ap.add_argument('--case', type=int, default=None)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--dtype', default='bf16', choices=['bf16', 'fp16', 'fp32'])
    ap.add_argument('--batch', type=int, default=32)
    ap.add_argument('--rows', type=int, default=0)
    ap.add_argument('--rotate', type=int, default=4, help='input buffers rotated between launches')
    ap.add_argument('--impl', type=int, default=nat.IMPL_AUTO, help='0 auto, 1 SIMT, 2 tcgen05 gather, 3 TMA')
    ap.add_argument('--configure', action='append', default=[], metavar='KEY=VALUE',
                    help='library switches (sso_configure), e.g. chol_ksplit=0')
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit('microbench needs a CUDA device: there is no CPU path')
    nat.lib()
    for kv in args.configure:
        k, v = kv.split('=')
        nat.configure(k, int(v))
    SUITES[args.suite](args)


if __name__ == '__main__':
    main()
