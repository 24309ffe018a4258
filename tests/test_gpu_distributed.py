"""Data-parallel K-FAC on 2, 4 and 8 GPUs against its single-process equivalent.

Grads and curvature data are averaged over ranks with equal weights, so N-rank data parallel
training equals one process with ``acc_steps = N`` fed the N shards in rank order (batch-norm
statistics are per shard in both).  The model has 13 Kronecker layers of very different sizes, so the
two ownership rules give different, unbalanced partitions with padded segments.

Two ways of running the ranks: over NCCL with one GPU per rank (each case needs as many GPUs as ranks
and is skipped otherwise), and over gloo with all ranks sharing GPU 0 (runs anywhere there is one GPU:
same optimizer, ownership, device packer and exchange logic; only the collective's transport differs).
Two steps: the preconditioned update multiplies a difference of one rounding by ~30 per step on this
net (measured), so longer runs only test that amplification.  The net is smooth and the convolutions
run in full fp32 (TF32 off): TF32 rounds the weights to 10 bits, so a last-bit difference in one of
them becomes a 1e-3 step in what the convolution sees, and with ReLU units that moved the
parameters of some 4-GPU runs by 7.7e-4 after two steps and of others by 3e-6."""
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
STEPS = 2
LR = 1e-3


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _shard(step, rank):
    x, y = cases.make_batch((6, 2, 8, 8), 7, seed=900 + 10 * step + rank)
    u = cases.make_uniform((1, 6), seed=950 + 10 * step + rank)
    return x, y, u


def _run_single(device, world):
    import torchsso
    model = cases.make_model('uneven_net', seed=1).to(device)
    opt = torchsso.optim.SecondOrderOptimizer(model, 'Fisher', KRON, KW, lr=LR, acc_steps=world)
    state = {}
    original = torchsso.curv.fisher.sample_targets
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    torchsso.curv.fisher.sample_targets = \
        lambda prob, num_mc: inverse_cdf_targets(prob.detach().float().cpu(), state['u']).to(prob.device)
    try:
        for step in range(STEPS):
            for rank in range(world):
                x, y, state['u'] = _shard(step, rank)
                closure = torchsso.get_closure_for_fisher(opt, model, x.to(device), y.to(device),
                                                          approx_type='mc', num_mc=1)
                opt.step(closure=closure)
    finally:
        torchsso.curv.fisher.sample_targets = original       # this runs in the test process itself
        torch.backends.cudnn.allow_tf32 = tf32
    return [p.detach().cpu().clone() for p in model.parameters()]


def _worker(rank, world, port, balance, ret, wire=None, scaling=True, backend='nccl'):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    index = rank if backend == 'nccl' else 0           # gloo ranks share GPU 0
    torch.cuda.set_device(index)
    device = torch.device('cuda', index)
    if backend == 'nccl':
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    else:
        dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        import torchsso
        torch.backends.cudnn.allow_tf32 = False
        model = cases.make_model('uneven_net', seed=1).to(device)
        comm = torchsso.utils.create_communicator(wire_dtype=wire, wire_scaling=scaling)
        opt = torchsso.optim.DistributedSecondOrderOptimizer(model, 'Fisher', KRON, KW, lr=LR,
                                                             balance=balance, comm=comm)
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
        ret['indices'] = [list(p) for p in opt.indices]
    finally:
        dist.destroy_process_group()


def _worst(got, ref):
    return max(((g - e).norm() / e.norm().clamp_min(1e-12)).item() for g, e in zip(got, ref))


@pytest.mark.parametrize('world', [2, 4, 8])
@pytest.mark.parametrize('balance', ['inverse_cost', 'contiguous'])
def test_data_parallel_equals_accumulation(world, balance):
    if torch.cuda.device_count() < world:
        pytest.skip('needs %d GPUs' % world)
    ref = _run_single(torch.device('cuda', 0), world)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), balance, ret), nprocs=world, join=True)
    sizes = [len(p) for p in ret['indices']]
    assert sum(sizes) == 16
    # the ranks' shards are summed by the collective, the accumulation adds them one after the other:
    # differences of one rounding, carried through two preconditioned updates
    for rank in range(world):
        assert _worst(ret[rank], ref) < 1e-4, (rank, _worst(ret[rank], ref))
    for rank in range(1, world):
        for a, b in zip(ret[0], ret[rank]):
            assert torch.equal(a, b), 'ranks disagree after the all-gather'


def _wire_worker(rank, world, port, ret):
    """Arrays from 1e-6 (a gradient vector) to 1e+5 (a factor) through the device packer and the
    sso_wire_* kernels: owner `rank` must receive the world mean of its arrays to fp16 rounding with the
    per-array scaling, and must NOT with the plain cast (underflow / overflow)."""
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    device = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    try:
        from torchsso.utils.communicator import KFACCommunicator
        dims = [37, 130]

        def arrays_of(r):
            out = []
            for owner in range(world):
                g = torch.Generator().manual_seed(1000 * r + owner)
                n = dims[owner]
                grad = torch.randn(n + 3, generator=g) * 1e-6
                m = torch.randn(n, n, generator=g) * 1e5
                out.append([grad, m + m.t()])
            return out
        mine = [[(t.to(device), t.dim() == 2) for t in local] for local in arrays_of(rank)]
        expect = [sum(arrays_of(r)[rank][j] for r in range(world)) / world for j in range(2)]
        result = {}
        for scaling in (True, False):
            arrays = [[(t.clone(), tri) for t, tri in local] for local in mine]
            comm = KFACCommunicator(wire_dtype=torch.float16, wire_scaling=scaling)
            comm.reduce_scatterv_arrays(arrays)
            torch.cuda.synchronize()
            errs = []
            for (got, _), exp in zip(arrays[rank], expect):
                e = ((got.cpu().double() - exp.double()).norm() / exp.double().norm()).item()
                errs.append(e if e == e else float('inf'))
            result[scaling] = errs
            if scaling:
                comm.allgatherv_arrays(arrays)       # the owners' values, again to fp16 rounding
                torch.cuda.synchronize()
                for owner in range(world):
                    exp_o = [sum(arrays_of(r)[owner][j] for r in range(world)) / world for j in range(2)]
                    for (got, _), exp in zip(arrays[owner], exp_o):
                        e = ((got.cpu().double() - exp.double()).norm() / exp.double().norm()).item()
                        assert e < 4e-3, ('all-gather', owner, e)
        ret[rank] = result
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4])
@pytest.mark.parametrize('balance', ['inverse_cost', 'contiguous'])
def test_data_parallel_equals_accumulation_ranks_sharing_one_gpu(world, balance):
    """The same equivalence with gloo ranks that all use GPU 0."""
    ref = _run_single(torch.device('cuda', 0), world)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), balance, ret, None, True, 'gloo'), nprocs=world, join=True)
    assert sum(len(p) for p in ret['indices']) == 16
    for rank in range(world):
        assert _worst(ret[rank], ref) < 2e-5, (rank, _worst(ret[rank], ref))
    for rank in range(1, world):
        for a, b in zip(ret[0], ret[rank]):
            assert torch.equal(a, b), 'ranks disagree after the all-gather'


def test_two_gpu_half_precision_wire_needs_its_scaling():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_wire_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for rank in range(2):
        scaled, plain = ret[rank][True], ret[rank][False]
        assert max(scaled) < 2e-3, (rank, scaled)
        assert max(plain) > 1e-2, (rank, plain)      # 1e-6 underflows fp16's 11 bits, 1e5 overflows its range


def test_two_gpu_half_precision_wire_in_the_optimizer():
    """The distributed optimizer with fp16 on the wire (per-array scaling on): two steps stay within
    fp16 rounding, amplified by the preconditioner, of the fp32 exchange."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    ref = _run_single(torch.device('cuda', 0), 2)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), 'inverse_cost', ret, torch.float16, True), nprocs=2, join=True)
    assert _worst(ret[0], ref) < 5e-2, _worst(ret[0], ref)
    for a, b in zip(ret[0], ret[1]):
        assert torch.equal(a, b)


# ---------------------------------------------------------------------------------------------
# MC-sample parallel VI: two ranks with one weight sample each on the SAME batch equal one process
# with two samples, when rank r draws the noise the single process draws for its sample r.
# ---------------------------------------------------------------------------------------------
VI_STEPS = 2
LR = 1e-3


def _vi_setup(device, num_mc, distributed):
    import torchsso
    model = cases.make_model('tiny_vgg', seed=4).to(device)
    cls = torchsso.optim.DistributedVIOptimizer if distributed else torchsso.optim.VIOptimizer
    opt = cls(model, 1000, 'Cov', KRON, {'ema_decay': 0.95, 'damping': 1e-3}, lr=1e-2,
              num_mc_samples=num_mc, val_num_mc_samples=2, kl_weighting=1, prior_variance=1)
    return model, opt


def _vi_noise_patch(state):
    def fake_randn_like(t, **kw):
        s = state['seed'] * 1000 + state['count']
        state['count'] += 1
        return cases.make_normal(tuple(t.shape), s).to(device=t.device, dtype=t.dtype)
    torch.randn_like = fake_randn_like


def _vi_closure(model, opt, x, y):
    import torch.nn.functional as F

    def closure():
        opt.zero_grad()
        o = model(x)
        loss = F.cross_entropy(o, y)
        loss.backward()
        return loss, o
    return closure


def _run_vi_single(device):
    model, opt = _vi_setup(device, 2, False)
    state = {'seed': 0, 'count': 0}
    _vi_noise_patch(state)
    per_sample = None
    for t in range(VI_STEPS):
        x, y = cases.make_batch((8, 3, 8, 8), 6, seed=600 + t)
        state['seed'], state['count'] = 700 + t, 0
        opt.step(closure=_vi_closure(model, opt, x.to(device), y.to(device)))
        per_sample = state['count'] // 2
    means = [m.detach().cpu().clone() for g in opt.param_groups for m in g['mean']]
    return means, per_sample


def _vi_worker(rank, world, port, per_sample, ret):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    device = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    try:
        model, opt = _vi_setup(device, 1, True)
        state = {'seed': 0, 'count': 0}
        _vi_noise_patch(state)
        for t in range(VI_STEPS):
            x, y = cases.make_batch((8, 3, 8, 8), 6, seed=600 + t)     # same batch on both ranks
            state['seed'], state['count'] = 700 + t, rank * per_sample
            opt.step(closure=_vi_closure(model, opt, x.to(device), y.to(device)))
        opt.pool.check_info()
        ret[rank] = [m.detach().cpu().clone() for g in opt.param_groups for m in g['mean']]
    finally:
        dist.destroy_process_group()


def test_two_gpu_vi_mc_parallel_equals_two_samples():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    real = torch.randn_like
    try:
        ref, per_sample = _run_vi_single(torch.device('cuda', 0))
    finally:
        torch.randn_like = real
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_vi_worker, args=(2, _free_port(), per_sample, ret), nprocs=2, join=True)
    for rank in range(2):
        for got, exp in zip(ret[rank], ref):
            err = ((got - exp).norm() / exp.norm().clamp_min(1e-12)).item()
            assert err < 5e-5, (rank, err)
    for a, b in zip(ret[0], ret[1]):
        assert torch.equal(a, b), 'ranks disagree after the all-gather'
