"""Host-side logic of the data-parallel factor exchange, run as two gloo ranks on the CPU:
owner assignment, equal padded segments, reduce-scatter of the world mean to owners, all-gather
of the owners' values.  The packer used here is a plain torch restatement of the pack / unpack
kernels (the product packs with its CUDA kernels; only the collective plumbing is under test)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kfac_oracle as ko


class TorchPacker:
    def pack(self, arrays, buf, offset, scale):
        off = offset
        for t, tri in arrays:
            v = ko.tri_pack(t) if tri else t.reshape(-1)
            buf[off: off + v.numel()] = v * scale
            off += v.numel()

    def unpack(self, arrays, buf, offset, symmetric=True):
        off = offset
        for t, tri in arrays:
            if tri:
                n = t.shape[0]
                k = n * (n + 1) // 2
                full = ko.tri_unpack(buf[off: off + k].clone(), n)
                t.copy_(full if symmetric else torch.triu(full))
            else:
                k = t.numel()
                t.copy_(buf[off: off + k].reshape(t.shape))
            off += k


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _make_arrays(rank, world, dims):
    """Every rank holds its own version of every owner's arrays: a gradient vector and a symmetric
    factor per owner, values depending on (rank, owner)."""
    arrays = []
    for owner in range(world):
        g = torch.Generator().manual_seed(1000 * rank + owner)
        n = dims[owner]
        grad = torch.randn(n + 3, generator=g)
        m = torch.randn(n, n, generator=g)
        arrays.append([(grad, False), (m + m.t(), True)])
    return arrays


def _worker(rank, world, port, dims, ret, wire_dtype=None, atol=1e-6):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from torchsso.utils.communicator import KFACCommunicator
        comm = KFACCommunicator(packer=TorchPacker(), wire_dtype=wire_dtype)
        arrays = _make_arrays(rank, world, dims)
        expect = ko.reduce_scatterv_mean([[t for t, _ in _make_arrays(r, world, dims)[rank]]
                                          for r in range(world)])
        comm.reduce_scatterv_arrays(arrays)
        for (got, _), exp in zip(arrays[rank], expect):
            assert torch.allclose(got, exp, atol=atol), 'owner did not receive the world mean'
        # arrays owned by other ranks are untouched
        other = (rank + 1) % world
        for (got, _), (orig, _) in zip(arrays[other], _make_arrays(rank, world, dims)[other]):
            assert torch.equal(got, orig)
        # all-gather: every rank ends with the owners' (averaged) values
        comm.allgatherv_arrays(arrays)
        for owner in range(world):
            exp = ko.reduce_scatterv_mean([[t for t, _ in _make_arrays(r, world, dims)[owner]]
                                           for r in range(world)])
            for (got, _), e in zip(arrays[owner], exp):
                assert torch.allclose(got, e, atol=atol)
        sizes, seg = comm.segment_sizes(arrays)
        assert seg % 64 == 0 and seg >= max(sizes)
        ret[rank] = 'ok'
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_gloo():
    world, dims = 2, [5, 9]
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, dims, ret), nprocs=world, join=True)
    assert dict(ret) == {0: 'ok', 1: 'ok'}


def test_two_rank_exchange_gloo_half_wire():
    """Optional 16-bit wire format: same exchange, values rounded to fp16 on the way."""
    world, dims = 2, [5, 9]
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, dims, ret, torch.float16, 2e-2), nprocs=world, join=True)
    assert dict(ret) == {0: 'ok', 1: 'ok'}


def test_owner_assignment_rules():
    from torchsso.utils.communicator import assign_owners
    assert assign_owners([0] * 7, 3, 'contiguous') == ko.owner_partition(7, 3)
    costs = [100, 1, 1, 50, 50, 0, 0, 0]
    parts = assign_owners(costs, 2, 'inverse_cost')
    assert sorted(i for p in parts for i in p) == list(range(8))
    loads = [sum(costs[i] for i in p) for p in parts]
    assert max(loads) - min(loads) <= 2
    assert abs(len(parts[0]) - len(parts[1])) <= 2
    # a single dominant layer cannot be split: the best possible maximum is that layer's cost
    parts = assign_owners([98, 10, 10, 10, 10], 4, 'inverse_cost')
    assert max(sum([98, 10, 10, 10, 10][i] for i in p) for p in parts) == 98
    with pytest.raises(ValueError):
        assign_owners([1], 1, 'nope')
