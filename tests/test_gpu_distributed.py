"""Two-GPU data-parallel K-FAC against its single-process equivalent.

Grads and curvature data are averaged over ranks with equal weights, so N-rank data parallel
training equals one process with ``acc_steps = N`` fed the N shards in rank order (batch-norm
statistics are per shard in both).  Needs two GPUs; skipped otherwise."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

import cases
from oracle.kfac_step import inverse_cdf_targets

pytestmark = pytest.mark.gpu

KRON = {'Linear': 'Kron', 'Conv2d': 'Kron', 'BatchNorm1d': 'Diag', 'BatchNorm2d': 'Diag'}
KW = {'ema_decay': 0.95, 'damping': 1e-3}
STEPS = 3


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _shard(step, rank):
    x, y = cases.make_batch((6, 3, 8, 8), 5, seed=900 + 10 * step + rank)
    u = cases.make_uniform((1, 6), seed=950 + 10 * step + rank)
    return x, y, u


def _run_single(device):
    import torchsso
    model = cases.make_model('tiny_convnet', seed=1).to(device)
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON, KW, lr=1e-2, acc_steps=2)
    state = {}
    torchsso.curv.fisher.sample_targets = \
        lambda prob, num_mc: inverse_cdf_targets(prob.detach().float().cpu(), state['u']).to(prob.device)
    for step in range(STEPS):
        for rank in range(2):
            x, y, state['u'] = _shard(step, rank)
            closure = torchsso.get_closure_for_fisher(opt, model, x.to(device), y.to(device),
                                                      approx_type='mc', num_mc=1)
            opt.step(closure=closure)
    return [p.detach().cpu().clone() for p in model.parameters()]


def _worker(rank, world, port, balance, ret):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    device = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    try:
        import torchsso
        model = cases.make_model('tiny_convnet', seed=1).to(device)
        opt = torchsso.optim.DistributedSecondOrderOptimizer(model, 'Fisher', KRON, KW, lr=1e-2,
                                                             balance=balance)
        state = {}
        torchsso.curv.fisher.sample_targets = \
            lambda prob, num_mc: inverse_cdf_targets(prob.detach().float().cpu(), state['u']).to(prob.device)
        for step in range(STEPS):
            x, y, state['u'] = _shard(step, rank)
            closure = torchsso.get_closure_for_fisher(opt, model, x.to(device), y.to(device),
                                                      approx_type='mc', num_mc=1)
            opt.step(closure=closure)
        opt.pool.check_info()
        assert sorted(i for part in opt.indices for i in part) == list(range(len(opt.param_groups)))
        ret[rank] = [p.detach().cpu().clone() for p in model.parameters()]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('balance', ['inverse_cost', 'contiguous'])
def test_two_gpu_data_parallel_equals_accumulation(balance):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    ref = _run_single(torch.device('cuda', 0))
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), balance, ret), nprocs=2, join=True)
    for rank in range(2):
        for got, exp in zip(ret[rank], ref):
            err = ((got - exp).norm() / exp.norm().clamp_min(1e-12)).item()
            assert err < 2e-5, (rank, err)
    for a, b in zip(ret[0], ret[1]):
        assert torch.equal(a, b), 'ranks disagree after the all-gather'
