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
def cpu_port_images_per_sec(batch, steps, seed=0):
    """Times oracle.kfac_step.OracleKFAC (torch CPU ops, all host threads) on ResNet-50 with a
    reduced batch: `steps` steps without inverse + one step with the inverses, combined as the
    workload's 1-in-10 inverse schedule.  Returns (images/sec, cores, sample description)."""
    from oracle.kfac_step import OracleKFAC
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    torch.manual_seed(seed)
    model = ResNet50()
    opt = OracleKFAC(model, 'Fisher', ema_decay=CURV_KW['ema_decay'], damping=CURV_KW['damping'], lr=1e-3)
    x, y = synthetic_batch(batch, 1000, seed)
    mc = torch.randint(0, 1000, (1, batch), generator=torch.Generator().manual_seed(seed + 1))
    t0 = time.perf_counter()
    opt.update_inv = True
    opt.step(x, y, mc)
    t_inv = time.perf_counter() - t0
    opt.update_inv = False
    ts = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        opt.step(x, y, mc)
        ts.append(time.perf_counter() - t0)
    t_plain = sorted(ts)[len(ts) // 2]
    per_step = t_plain + max(0.0, t_inv - t_plain) / INV_INTERVAL
    sample = ('ResNet-50 K-FAC step at batch %d (full model, all 107 curvature groups): 1 step with '
              'inverses (%.1f s) + %d without (median %.1f s), combined 1-in-%d'
              % (batch, t_inv, len(ts), t_plain, INV_INTERVAL))
    return batch / per_step, cores, sample, per_step


def sgd_images_per_sec(batch, dev, steps=20):
    """Stock torch SGD (momentum 0.9) on the same ResNet-50, bf16 autocast, channels_last inputs,
    the whole step replayed from a CUDA graph: the denominator of the "fraction of SGD" figure."""
    model = ResNet50().to(dev)
    opt = torch.optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)
    x, y = synthetic_batch(batch, 1000, 7)
    x = x.to(dev).contiguous(memory_format=torch.channels_last)
    y = y.to(dev)

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast('cuda', dtype=torch.bfloat16):
            loss = F.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return batch * steps / (e0.elapsed_time(e1) / 1e3)


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    val, cores, sample, per_step = cpu_port_images_per_sec(args.cpu_batch, max(1, min(args.steps, 2)))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': 'images/sec', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': per_step * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic',
        'config': {'workload': 'resnet50_kfac_b32', 'batch_per_gpu': 32, 'inverse_every': INV_INTERVAL,
                   'note': 'CPU restatement of the reference path (the reference GPU path needs '
                           'CuPy/ChainerMN, absent here); bounded sample at batch %d' % args.cpu_batch},
        'cpu_baseline': {'value': val, 'unit': 'images/sec', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': val, 'unit': 'images/sec', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
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
    # a small pool of different synthetic batches, cycled: fresh data every step keeps the loss
    # (and with it the curvature) stationary instead of memorising one batch
    NB = 4
    pinned = [synthetic_batch(B, 1000, 1000 * rank + i, pin=True) for i in range(NB)]
    resident = [(xp.to(dev).contiguous(memory_format=torch.channels_last), yp.to(dev)) for xp, yp in pinned]
    x_pin, y_pin = pinned[0]
    state = {'step': 0}

    # The closure reads its batch from fixed device tensors so that it can be captured once into a
    # CUDA graph (forward, sampling backward, loss backward and all curvature kernels of the hooks)
    # and replayed; every step first copies its batch into them.
    x_static = torch.empty_like(resident[0][0])
    y_static = torch.empty_like(resident[0][1])
    x_static.copy_(resident[0][0]); y_static.copy_(resident[0][1])
    # autograd assigns fresh gradient tensors instead of accumulating into the optimizer's flat buffer
    # (one add kernel per parameter per backward pass); one multi-tensor copy harvests them
    opt.zero_grad_to_none = (args.grads == 'assign')
    closure = fisher_closure(torchsso, opt, model, x_static, y_static)
    eager_closure = closure
    if args.graph:
        opt.update_inv = True
        opt.step(closure=closure)            # eager first step: builds pools, plans, scratch
        # the model has no in-place activations, so the hooks' kernels may run beside it
        torchsso.utils.set_curvature_stream(args.side_stream)
        closure = torchsso.utils.GraphedClosure(opt, closure)
        state['step'] = 1

    def one_step(x, y):
        x_static.copy_(x, non_blocking=True)
        y_static.copy_(y, non_blocking=True)
        opt.update_inv = (state['step'] % INV_INTERVAL == 0)
        loss, _ = opt.step(closure=closure)
        state['step'] += 1
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(nsteps, e2e):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = nat.launch_count()
        r0 = closure.replays if args.graph else 0
        ev0.record()
        last = None
        for i in range(nsteps):
            if e2e:
                last = one_step(*pinned[i % NB]).item()      # host -> device copy inside one_step
            else:
                last = one_step(*resident[i % NB])
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        launches = nat.launch_count() - l0
        if args.graph:      # kernels inside the replayed graph are not seen by the host-side counter
            launches += (closure.replays - r0) * closure.library_kernels_per_replay
        return ms, launches, float(last)

    # warm-up (also builds plans and cuDNN algorithm choices); first step inverts
    for i in range(max(args.warmup, 3)):
        one_step(*resident[i % NB])
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
        x_static.copy_(resident[i % NB][0]); y_static.copy_(resident[i % NB][1])
        opt.update_inv = False
        opt.step(closure=eager_closure)
    torch.cuda.synchronize()
    ft = nat.FACTOR_TIMING
    nat.FACTOR_TIMING = None
    f_ms = sum(a.elapsed_time(b) for a, b, _, _ in ft)
    f_flops = sum(f for _, _, f, _ in ft)
    f_bytes = sum(nb for _, _, _, nb in ft)

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
                   'parallelism': 'dp%d, factors reduce-scattered to owners' % world if world > 1 else 'single',
                   'l2_policy': 'per-step inputs (%.0f MB activations + 615 MB factor pools) exceed the 126 MB L2'
                                % (B * 3 * 224 * 224 * 2 / 1e6),
                   'final_loss': float(last_loss)},
        'clocks': clocks.summary(),
        'e2e': {'value': ips_e2e, 'unit': 'images/sec',
                'h2d_bytes_per_step': int(x_pin.numel() * 4 + y_pin.numel() * 8), 'd2h_bytes_per_step': 4,
                'final_loss': float(last_e2e)},
        'gpu_launches': int(launches),
        'optimizer_step_ms': {'closure': closure_ms, 'without_inverses': step_noinv_ms - closure_ms,
                              'with_inverses': step_inv_ms - closure_ms,
                              'note': 'optimizer.step() minus its closure (forward, sampling pass, backward, '
                                      'curvature hooks); inverses run on every %dth step' % INV_INTERVAL},
        'roofline': {'bound': 'tensor', 'kernel': 'factor construction (all Kron layers, A and G)',
                     'achieved': achieved_tf, 'peak': tf_peak, 'unit': 'TFLOP/s',
                     'frac': achieved_tf / tf_peak if tf_peak else None,
                     # DRAM bytes per launch: algorithmic bytes (input once + d*d*4 output) averaged over
                     # the factor launches, times the measured/algorithmic ratio of the ncu capture of one
                     # launch (profiles/factor_tma_pair_kernel_*: 55.4 MB measured for 56.7 MB algorithmic)
                     'traffic': (f_bytes / len(ft)) * (55.4 / 56.7) if ft else None,
                     'traffic_unit': 'bytes per launch (average over the launches of a step)',
                     'peak_source': peak_src + ' (bf16 dense, sustained)',
                     'launches': len(ft), 'total_ms': f_ms, 'measured_over_steps': probe_steps,
                     'flops_rule': '2*rows*d^2 per factor (what the reference einsum performs)'},
    }
    if world == 1 and not args.no_sgd_baseline:
        del closure, eager_closure, opt
        sgd = sgd_images_per_sec(B, dev)
        line['sgd_baseline'] = {'value': sgd, 'unit': 'images/sec', 'frac_of_sgd': ips / sgd,
                                'note': 'stock torch SGD+momentum, same model / batch / bf16 autocast, '
                                        'CUDA-graph replay, measured in this run'}
    if world == 1 and not args.no_cpu_baseline:
        val, cores, sample, _ = cpu_port_images_per_sec(args.cpu_batch, 2)
        line['cpu_baseline'] = {'value': val, 'unit': 'images/sec', 'cores': cores, 'kind': 'port',
                                'sample': sample}
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
    ap.add_argument('--cpu-batch', type=int, default=16, help='batch of the bounded CPU sample')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-sgd-baseline', action='store_true')
    ap.add_argument('--weights', default='contiguous', choices=['channels_last', 'contiguous'],
                    help='memory format of the convolution weights (activations are channels_last)')
    ap.add_argument('--grads', default='assign', choices=['assign', 'accumulate'],
                    help="zero_grad(): 'assign' sets .grad to None (autograd assigns, one harvest copy), "
                         "'accumulate' binds .grad to the flat buffer (autograd adds in place)")
    ap.add_argument('--no-side-stream', dest='side_stream', action='store_false',
                    help='launch the curvature kernels of the hooks on the main stream')
    ap.add_argument('--no-graph', dest='graph', action='store_false',
                    help='issue the closure eagerly instead of replaying a captured CUDA graph')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == '__main__':
    main()
