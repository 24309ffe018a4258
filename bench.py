#!/usr/bin/env python
"""Benchmark of the K-FAC curvature hot path:  ResNet-50 K-FAC images/sec.

Workload ("resnet50_kfac_b32"): ResNet-50 (bottleneck [3,4,6,3], width 64), K-FAC (Fisher, 1 MC
sample) on every Conv2d/Linear (Kronecker factors, largest A is 4608^2) and diagonal curvature
on every BatchNorm2d; synthetic inputs N(0,1) of shape 3x224x224, 32 per GPU, uniform labels;
bf16 activations (autocast) with fp32 factors; factors every step, inverses every 10 steps.
One "step" = closure (forward, sampling backward, loss backward, with the factor kernels in the
hooks) + optimizer step.  N > 1: data parallel, factors reduce-scattered to owner ranks,
updated parameters all-gathered (launch with torch.distributed.run, one rank per GPU).

  python bench.py [--gpus N] [--steps K] [--warmup W]            # this repository's CUDA path
  python bench.py --impl reference [...]                          # the CPU restatement of the
        reference's path (oracle/), timed on the host cores on a bounded sample of the workload

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, 'pytorch-sso_b200'))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.nn as nn  # noqa: E402
import torch.nn.functional as F  # noqa: E402

KRON = {'Linear': 'Kron', 'Conv2d': 'Kron', 'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'}
CURV_KW = {'ema_decay': 0.95, 'damping': 1e-3}
INV_INTERVAL = 10
METRIC = 'ResNet-50 K-FAC images/sec'


# ---------------------------------------------------------------------------------------------
# model: ResNet-50, ImageNet stem, functional relu (no in-place module activations needed)
# ---------------------------------------------------------------------------------------------
class Bottleneck(nn.Module):
    def __init__(self, cin, width, stride, downsample):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, width * 4, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(width * 4)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = F.relu(self.bn1(self.conv1(x)))
        out = F.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return F.relu(out + idt)


class ResNet50(nn.Module):
    def __init__(self, num_classes=1000, layers=(3, 4, 6, 3), width=64):
        super().__init__()
        self.num_classes = num_classes
        self.conv1 = nn.Conv2d(3, width, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        cin, stages = width, []
        for i, nblk in enumerate(layers):
            w = width * 2 ** i
            for b in range(nblk):
                stride = 2 if (b == 0 and i > 0) else 1
                ds = None
                if b == 0:
                    ds = nn.Sequential(nn.Conv2d(cin, w * 4, 1, stride=stride, bias=False),
                                       nn.BatchNorm2d(w * 4))
                stages.append(Bottleneck(cin, w, stride, ds))
                cin = w * 4
        self.blocks = nn.Sequential(*stages)
        self.fc = nn.Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.bn1(self.conv1(x))), 3, stride=2, padding=1)
        x = self.blocks(x)
        x = F.adaptive_avg_pool2d(x, 1).flatten(1)
        return self.fc(x)


def synthetic_batch(batch, num_classes, seed, device='cpu', pin=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((batch, 3, 224, 224), generator=g)
    y = torch.randint(0, num_classes, (batch,), generator=g)
    if pin:
        x, y = x.contiguous(memory_format=torch.channels_last).pin_memory(), y.pin_memory()
    return x.to(device), y.to(device)


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(['nvidia-smi', '-i', str(self.index), '--query-gpu=' + self.Q,
                                      '--format=csv,noheader,nounits'], capture_output=True, text=True,
                                     timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(',')])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = max(mx, float(s[1]))
                for nm, v in zip(names, s[2:6]):
                    if v.lower().startswith('active'):
                        reasons.add(nm)
            except Exception:
                continue
        mhz.sort()
        return {'sm_mhz': mhz[len(mhz) // 2] if mhz else None, 'sm_max_mhz': mx or None,
                'reasons': sorted(reasons), 'samples': len(mhz)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference path on the host cores
# ---------------------------------------------------------------------------------------------
class CpuPort:
    """oracle.kfac_step.OracleKFAC (torch CPU ops, all host threads) on the benchmark's own
    configuration: ResNet-50, `batch` images of the rank-0 stream (seed = step index), fp32, Fisher
    MC(1), inverses on every INV_INTERVAL-th step starting with the first."""

    def __init__(self, batch):
        from oracle.kfac_step import OracleKFAC
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        torch.manual_seed(0)
        self.batch = batch
        self.model = ResNet50()
        self.opt = OracleKFAC(self.model, 'Fisher', ema_decay=CURV_KW['ema_decay'], damping=CURV_KW['damping'], lr=1e-3)
        self.step_index = 0
        self.first = None

    def step(self):
        """One optimizer step; returns its wall time in seconds."""
        i = self.step_index
        x, y = synthetic_batch(self.batch, 1000, i)
        mc = torch.randint(0, 1000, (1, self.batch), generator=torch.Generator().manual_seed(50000 + i))
        self.opt.update_inv = (i % INV_INTERVAL == 0)
        t0 = time.perf_counter()
        loss, _ = self.opt.step(x, y, mc)
        dt = time.perf_counter() - t0
        if self.first is None:
            self.first = {'loss': float(loss), 'stem_A_norm': float(self.opt.layers[0].ema[0].double().norm()),
                          'layer1_conv1_A_norm': float(self.opt.layers[2].ema[0].double().norm())}
        self.step_index += 1
        return dt


def cpu_port_sample(batch, budget_s=25.0):
    """Bounded sample for the GPU arm's `cpu_baseline`: the first step (with inverses) and as many
    plain steps as fit in the budget (at least one), combined with the 1-in-INV_INTERVAL schedule."""
    port = CpuPort(batch)
    t_inv = port.step()
    ts = []
    while not ts or (sum(ts) + t_inv + ts[-1] < budget_s and len(ts) < 4):
        ts.append(port.step())
    t_plain = sorted(ts)[len(ts) // 2]
    per_step = t_plain + max(0.0, t_inv - t_plain) / INV_INTERVAL
    sample = ('ResNet-50 K-FAC steps at batch %d (the benchmark\'s configuration, full model, 107 curvature '
              'groups): 1 step with inverses (%.1f s) + %d without (median %.1f s), combined 1-in-%d'
              % (batch, t_inv, len(ts), t_plain, INV_INTERVAL))
    return batch / per_step, port.cores, sample, port.first


def sgd_images_per_sec(batch, dev, world, rank, steps=20):
    """Stock torch SGD (momentum 0.9) on the same ResNet-50, bf16 autocast, channels_last inputs: the
    denominator of the "fraction of SGD" figure, whole job over `world` GPUs.  Forward + backward are
    replayed from one CUDA graph and the update from another; between them, on more than one GPU,
    the flat gradient buffer is all-reduced (what DistributedDataParallel does, in one bucket)."""
    import torch.distributed as dist
    torch.manual_seed(0)
    model = ResNet50().to(dev)
    opt = torch.optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)
    x, y = synthetic_batch(batch, 1000, 7 + 1000 * rank)
    x = x.to(dev).contiguous(memory_format=torch.channels_last)
    y = y.to(dev)
    params = list(model.parameters())
    flat = torch.zeros(sum(p.numel() for p in params), device=dev)
    off = 0
    for p in params:
        p.grad = flat[off:off + p.numel()].view_as(p)
        off += p.numel()

    def fwd_bwd():
        flat.zero_()
        with torch.autocast('cuda', dtype=torch.bfloat16):
            loss = F.cross_entropy(model(x).float(), y)
        loss.backward()

    def update():
        if world > 1:
            flat.mul_(1.0 / world)
        opt.step()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fwd_bwd()
            update()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g1, g2 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g1):
        fwd_bwd()
    with torch.cuda.graph(g2):
        update()

    def step():
        g1.replay()
        if world > 1:
            dist.all_reduce(flat)
        g2.replay()
    for _ in range(3):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return world * batch * steps / (ms / 1e3)


def run_reference_arm(args):
    """CPU arm: the oracle port of the reference path on all host cores, same configuration as the GPU
    arm (batch 32 per step, inverses every INV_INTERVAL-th step).  The reference itself is Python
    over CuPy / ChainerMN and cannot be installed here, and its sources do not travel to the
    benchmark machine; the port is bit-identical to the reference's CPU run on the committed fixtures.
    W warm-up steps and K timed steps are executed as asked as long as they fit a wall-clock budget;
    the JSON line reports the steps that were actually run and timed."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    t_start = time.perf_counter()
    budget = args.cpu_budget
    port = CpuPort(args.batch)
    warm = 0
    for _ in range(args.warmup):
        if warm >= 1 and time.perf_counter() - t_start > 0.2 * budget:
            break
        port.step()
        warm += 1
    # keep the timed window on the schedule's phase: it starts on a step with inverses
    port.step_index = 0
    ts = []
    for _ in range(args.steps):
        if ts and time.perf_counter() - t_start + max(ts) > budget:
            break
        ts.append(port.step())
    steps = len(ts)
    total = sum(ts)
    val = args.batch * steps / total
    n_inv = sum(1 for i in range(steps) if i % INV_INTERVAL == 0)
    sample = ('%d consecutive optimizer steps at batch %d (%d with inverses), %.1f s; asked for %d steps / %d warm-up, '
              'budget %.0f s' % (steps, args.batch, n_inv, total, args.steps, args.warmup, budget))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': 'images/sec', 'n_gpus': args.gpus,
        'steps': steps, 'warmup': warm, 'ms_per_step': total / steps * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic',
        'config': {'workload': 'resnet50_kfac_b32', 'batch_per_gpu': args.batch, 'global_batch': args.batch,
                   'image': '3x224x224', 'curvature': 'Fisher MC(1): Kron conv/linear + diag BN',
                   'factors_every': 1, 'inverse_every': INV_INTERVAL,
                   'steps_requested': args.steps, 'warmup_requested': args.warmup,
                   'note': 'CPU restatement (oracle/) of the reference path on the host cores; the reference '
                           'needs CuPy/ChainerMN for its GPU path and is Python, so it neither installs nor travels'},
        'cpu_baseline': {'value': val, 'unit': 'images/sec', 'cores': port.cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': val, 'unit': 'images/sec', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'first_step': port.first,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get('hbm_gbs', 6650.0), d.get('bf16_tflops_sustained', 1400.0), 'measured'
    return 6650.0, 1400.0, 'fallback'


def run_gpu_arm(args):
    import torch.distributed as dist
    import torchsso
    from torchsso import _native as nat

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise RuntimeError('bench.py needs a CUDA device (use --impl reference for the CPU arm)')
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)
    nat.lib()
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(0)
    model = ResNet50().to(dev)
    if args.weights == 'channels_last':
        model = model.to(memory_format=torch.channels_last)
    kw = dict(lr=1e-3)
    if world > 1:
        opt = torchsso.optim.DistributedSecondOrderOptimizer(model, 'Fisher', KRON, CURV_KW, **kw)
    else:
        opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON, CURV_KW, **kw)
    B = args.batch
    # A fresh synthetic batch for every step (rank r, step i: seed 1000*r + i), generated and pinned
    # before anything is timed: one fixed batch is memorised within a few steps, the loss and with it
    # the G factors collapse, and stale inverses then blow the loss up.
    W = max(args.warmup, 3)
    NB = 1 + W + 2 * args.steps
    pinned = [synthetic_batch(B, 1000, 1000 * rank + i, pin=True) for i in range(NB)]
    x_pin, y_pin = pinned[0]
    resident = [(xp.to(dev), yp.to(dev)) for xp, yp in pinned[:1 + W + args.steps]]
    state = {'step': 0, 'batch': 0}

    # The closure reads its batch from fixed device tensors so that it can be captured once into a
    # CUDA graph (forward, sampling backward, loss backward and all curvature kernels of the hooks)
    # and replayed; every step first copies its batch into them.
    x_static = torch.empty_like(resident[0][0])
    y_static = torch.empty_like(resident[0][1])
    x_static.copy_(resident[0][0]); y_static.copy_(resident[0][1])
    state['batch'] = 1
    # autograd assigns fresh gradient tensors instead of accumulating into the optimizer's flat buffer
    # (one add kernel per parameter per backward pass); one multi-tensor copy harvests them
    opt.zero_grad_to_none = (args.grads == 'assign')
    # all factors of a pass go to the device in one persistent launch instead of one launch pair per layer
    torchsso.utils.set_factor_batching(args.batching)
    if args.batch_pairs:
        nat.configure('batch_pairs', args.batch_pairs)
    if args.fuse_ema and world == 1:
        # the kernels that build the curvature write the running average in their epilogue
        # (one closure call per step, which is how this loop drives the optimizer)
        opt.fuse_ema = True
        # ... and the round of inverses starts inside the closure, beside the real backward pass
        opt.early_inverse = args.early_inverse
    closure = fisher_closure(torchsso, opt, model, x_static, y_static)
    eager_closure = closure
    first = None
    if args.graph:
        opt.update_inv = True
        # eager first step: builds pools, plans, scratch.  Only the value of the loss is kept: a live loss
        # tensor would pin this step's autograd graph, whose gradient-accumulation nodes belong to the
        # default stream and would then break the capture below
        loss0 = float(opt.step(closure=closure)[0].detach())
        if world == 1:
            kron_groups = [g for g in opt.param_groups if isinstance(g['curv'], torchsso.KronCurvature)]
            first = {'loss': loss0, 'stem_A_norm': float(kron_groups[0]['curv'].ema[0].double().norm()),
                     'layer1_conv1_A_norm': float(kron_groups[1]['curv'].ema[0].double().norm())}
        # the model has no in-place activations, so the hooks' kernels may run beside it
        torchsso.utils.set_curvature_stream(args.side_stream)
        closure = torchsso.utils.GraphedClosure(opt, closure)
        state['step'] = 1

    def run_step():
        opt.update_inv = (state['step'] % INV_INTERVAL == 0)
        loss, _ = opt.step(closure=closure)
        state['step'] += 1
        return loss

    def one_step(x, y):
        x_static.copy_(x, non_blocking=True)
        y_static.copy_(y, non_blocking=True)
        return run_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def next_batch(pool):
        b = pool[state['batch'] % len(pool)]
        state['batch'] += 1
        return b

    def timed(nsteps, e2e):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = nat.launch_count()
        r0 = closure.library_launches if args.graph else 0
        ev0.record()
        last = None
        if e2e:
            # every batch comes from pinned host memory inside the timed region, through the package's
            # double-buffered input pipeline (the copy of batch i + 1 runs beside step i), and every
            # step's loss is copied to the host and read there (checked for NaN) one step later
            feed = torchsso.utils.BatchPrefetcher((next_batch(pinned) for _ in range(nsteps)), (x_static, y_static))
            host_loss = torch.empty(nsteps, dtype=torch.float32).pin_memory()
            copied = [torch.cuda.Event() for _ in range(nsteps)]
            for i in feed:
                host_loss[i:i + 1].copy_(run_step().detach().reshape(1), non_blocking=True)
                copied[i].record()
                if i > 0:               # read one step behind, so the host keeps the device fed
                    copied[i - 1].synchronize()
                    last = float(host_loss[i - 1])
                    if last != last:
                        raise RuntimeError('loss is NaN at e2e step %d' % (i - 1))
            copied[nsteps - 1].synchronize()
            last = float(host_loss[nsteps - 1])
        else:
            for i in range(nsteps):
                last = one_step(*next_batch(resident))
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        launches = nat.launch_count() - l0
        if args.graph:      # kernels inside the replayed graph are not seen by the host-side counter
            launches += closure.library_launches - r0
        return ms, launches, float(last.detach()) if torch.is_tensor(last) else float(last)

    # warm-up (also builds plans and cuDNN algorithm choices); first step inverts
    for i in range(W):
        one_step(*next_batch(resident))
    # align the inverse schedule so that every timed window of K steps sees K/10 inverses
    state['step'] = 1
    with ClockSampler(local_rank) as clocks:
        ms, launches, last_loss = timed(args.steps, e2e=False)
    torch.cuda.synchronize()
    state['step'] = 1
    ms_e2e, _, last_e2e = timed(args.steps, e2e=True)
    # The metric's second figure, "K-FAC optimizer step ms": what optimizer.step() adds to its closure
    # (EMA, exchange on N > 1, precondition, update; plus the round of inverses on every 10th step) =
    # step time minus the time of the closure alone, CUDA events, same for every rank.
    def avg_ms(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / n

    def closure_only():
        closure()
        nat.join_curvature_stream(None)

    def step_with(inv):
        opt.update_inv = inv
        opt.step(closure=closure)
    opt.update_inv = False
    closure_ms = avg_ms(closure_only, 5)
    step_noinv_ms = avg_ms(lambda: step_with(False), 5)
    step_inv_ms = avg_ms(lambda: step_with(True), 3)
    # Per-kernel timing of the dominant kernel (factor construction): CUDA events around every
    # factor launch, on the launching stream, over a few more steps of the same workload issued
    # eagerly (a replayed graph has no host-side call to bracket).
    # The probe launches the hooks' kernels on the main stream: beside the model's kernels (side
    # stream) a factor kernel's elapsed time includes waiting for SMs, which says nothing about it.
    torchsso.utils.set_curvature_stream(False)
    nat.FACTOR_TIMING = []
    probe_steps = 3
    for i in range(probe_steps):
        # hold the stream back ~25 ms so that the host runs ahead and the step's kernels execute
        # back to back, as they do inside the replayed graph, instead of each starting on an idle GPU
        torch.cuda._sleep(int(5e7))
        x_static.copy_(resident[i][0]); y_static.copy_(resident[i][1])
        opt.update_inv = False
        opt.step(closure=eager_closure)
    torch.cuda.synchronize()
    ft = nat.FACTOR_TIMING
    nat.FACTOR_TIMING = None
    f_ms = sum(a.elapsed_time(b) for a, b, _, _ in ft)
    f_flops = sum(f for _, _, f, _ in ft)
    f_bytes = sum(nb for _, _, _, nb in ft)

    # data-parallel correctness bit: after the all-gather every rank must hold the same parameters
    rank_diff = None
    if world > 1:
        flat_p = torch.cat([p.detach().flatten().float() for p in model.parameters()])
        hi, lo = flat_p.clone(), flat_p.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        rank_diff = float((hi - lo).abs().max().item())
        del flat_p, hi, lo
    sgd = None
    if not args.no_sgd_baseline:
        del closure, eager_closure, opt
        torch.cuda.empty_cache()
        sgd = sgd_images_per_sec(B, dev, world, rank)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    hbm_peak, tf_peak, peak_src = measured_peaks()
    ips = world * B * args.steps / (ms / 1e3)
    ips_e2e = world * B * args.steps / (ms_e2e / 1e3)
    achieved_tf = f_flops / (f_ms / 1e3) / 1e12 if f_ms > 0 else 0.0
    line = {
        'metric': METRIC, 'value': ips, 'unit': 'images/sec', 'n_gpus': world, 'steps': args.steps,
        'warmup': max(args.warmup, 3), 'ms_per_step': ms / args.steps, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16 activations, f32 factors', 'data': 'synthetic',
        'config': {'workload': 'resnet50_kfac_b32', 'batch_per_gpu': B, 'global_batch': B * world,
                   'image': '3x224x224', 'curvature': 'Fisher MC(1): Kron conv/linear + diag BN',
                   'factors_every': 1, 'inverse_every': INV_INTERVAL,
                   'closure': 'CUDA graph replay' if args.graph else 'eager',
                   'curvature_stream': bool(args.graph and args.side_stream),
                   'factor_launches': 'batched per pass' if args.batching else 'per layer',
                   'inverses': 'started inside the closure, beside the real backward' if (args.early_inverse and args.fuse_ema and world == 1) else 'after the closure',
                   'ema': 'fused into the factor / BatchNorm epilogues' if (args.fuse_ema and world == 1) else 'separate pass',
                   'parallelism': 'dp%d, factors reduce-scattered to owners' % world if world > 1 else 'single',
                   'l2_policy': 'per-step inputs (%.0f MB activations + 615 MB factor pools) exceed the 126 MB L2'
                                % (B * 3 * 224 * 224 * 2 / 1e6),
                   'final_loss': float(last_loss)},
        'clocks': clocks.summary(),
        'e2e': {'value': ips_e2e, 'unit': 'images/sec',
                'h2d_bytes_per_step': int(x_pin.numel() * 4 + y_pin.numel() * 8), 'd2h_bytes_per_step': 4,
                'input_pipeline': 'pinned host batches through torchsso.utils.BatchPrefetcher (copy of batch i+1 beside step i)',
                'final_loss': float(last_e2e)},
        'gpu_launches': int(launches),
        'optimizer_step_ms': {'closure': closure_ms, 'without_inverses': step_noinv_ms - closure_ms,
                              'with_inverses': step_inv_ms - closure_ms,
                              'note': 'optimizer.step() minus its closure (forward, sampling pass, backward, '
                                      'curvature hooks); inverses run on every %dth step' % INV_INTERVAL},
        'roofline': {'bound': 'tensor', 'kernel': 'factor construction (all Kron layers, A and G)',
                     'achieved': achieved_tf, 'peak': tf_peak, 'unit': 'TFLOP/s',
                     'frac': achieved_tf / tf_peak if tf_peak else None,
                     # measured DRAM bytes exist per kernel and shape only (ncu captures summarised under
                     # profiles/: they equal the algorithmic bytes, the input read once); a step's 108
                     # launches are all different, so the line carries the algorithmic figure
                     'traffic': None,
                     'algorithmic_bytes_per_launch': (f_bytes / len(ft)) if ft else None,
                     'peak_source': peak_src + ' (bf16 dense, sustained)',
                     'launches': len(ft), 'total_ms': f_ms, 'measured_over_steps': probe_steps,
                     'flops_rule': '2*rows*d^2 per factor (what the reference einsum performs)'},
    }
    if rank_diff is not None:
        line['config']['max_param_difference_across_ranks'] = rank_diff
    if sgd is not None:
        line['sgd_baseline'] = {'value': sgd, 'unit': 'images/sec', 'frac_of_sgd': ips / sgd, 'n_gpus': world,
                                'note': 'stock torch SGD+momentum, same model / per-GPU batch / bf16 autocast, '
                                        'CUDA-graph replay, flat-gradient all-reduce on N > 1, measured in this run'}
    if world == 1 and not args.no_cpu_baseline:
        val, cores, sample, cpu_first = cpu_port_sample(B)
        line['cpu_baseline'] = {'value': val, 'unit': 'images/sec', 'cores': cores, 'kind': 'port',
                                'sample': sample}
        if first is not None:
            # same initial weights and first batch on both arms: the stem factor sees the fp32 image on
            # both (1e-6 class agreement); the loss and the next layer go through bf16 activations here
            line['parity'] = {'first_step_gpu': first, 'first_step_cpu_port': cpu_first,
                              'rel_diff': {k: abs(first[k] - cpu_first[k]) / max(abs(cpu_first[k]), 1e-30)
                                           for k in first}}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def fisher_closure(torchsso, opt, model, x, y):
    """torchsso.get_closure_for_fisher with the forward pass under bf16 autocast."""
    class _AutocastModel:
        num_classes = getattr(model, 'num_classes', None)

        def __call__(self, inp):
            with torch.autocast('cuda', dtype=torch.bfloat16):
                return model(inp).float()
    return torchsso.get_closure_for_fisher(opt, _AutocastModel(), x, y, approx_type='mc', num_mc=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--batch', type=int, default=32, help='images per GPU')
    ap.add_argument('--cpu-budget', type=float, default=240.0,
                    help='wall-clock budget in seconds of the CPU arm (--impl reference)')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-sgd-baseline', action='store_true')
    ap.add_argument('--weights', default='contiguous', choices=['channels_last', 'contiguous'],
                    help='memory format of the convolution weights (activations are channels_last)')
    ap.add_argument('--grads', default='assign', choices=['assign', 'accumulate'],
                    help="zero_grad(): 'assign' sets .grad to None (autograd assigns, one harvest copy), "
                         "'accumulate' binds .grad to the flat buffer (autograd adds in place)")
    ap.add_argument('--no-side-stream', dest='side_stream', action='store_false',
                    help='launch the curvature kernels of the hooks on the main stream')
    ap.add_argument('--no-batching', dest='batching', action='store_false',
                    help='one factor launch per layer and pass instead of one batched launch per pass')
    ap.add_argument('--batch-pairs', type=int, default=0,
                    help='CTA pairs of the batched factor kernel (0 = one per two SMs); fewer leave SMs to the '
                         'model kernels that run beside it')
    ap.add_argument('--no-fuse-ema', dest='fuse_ema', action='store_false',
                    help='keep curv.data and the separate data -> ema pass (single GPU only; N > 1 always does)')
    ap.add_argument('--no-early-inverse', dest='early_inverse', action='store_false',
                    help='run the round of inverses after the closure instead of beside its real backward pass')
    ap.add_argument('--no-graph', dest='graph', action='store_false',
                    help='issue the closure eagerly instead of replaying a captured CUDA graph')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == '__main__':
    main()
