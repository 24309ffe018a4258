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


    # torch restatement of the sso_wire_* kernels (tables are plain lists here)
    def wire_table(self, offsets, counts, ids, device):
        return list(zip(offsets, counts, ids))

    def wire_absmax(self, buf, table, maxima):
        for off, n, i in table:
            maxima[i] = torch.maximum(maxima[i], buf[off: off + n].abs().max())

    def wire_encode(self, buf, table, sums, out16):
        for off, n, i in table:
            s = float(sums[i])
            out16[off: off + n] = (buf[off: off + n] * (65000.0 / s if s > 0 else 1.0)).to(out16.dtype)

    def wire_decode(self, in16, table, sums, out32):
        for off, n, i in table:
            s = float(sums[i])
            out32[off: off + n] = in16[off: off + n].float() * (s / 65000.0 if s > 0 else 1.0)


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _make_arrays(rank, world, dims, spread=False):
    """Every rank holds its own version of every owner's arrays: a gradient vector and a symmetric
    factor per owner, values depending on (rank, owner).  `spread`: magnitudes from 1e-6 (gradients)
    to 1e+5 (factors), which a plain fp16 cast flushes to zero / overflows."""
    arrays = []
    for owner in range(world):
        g = torch.Generator().manual_seed(1000 * rank + owner)
        n = dims[owner]
        grad = torch.randn(n + 3, generator=g) * (1e-6 if spread else 1.0)
        m = torch.randn(n, n, generator=g) * (1e5 if spread else 1.0)
        arrays.append([(grad, False), (m + m.t(), True)])
    return arrays


def _close(got, exp, rtol):
    return ((got - exp).norm() <= rtol * exp.norm()).item()


def _worker(rank, world, port, dims, ret, wire_dtype=None, rtol=1e-6, spread=False, scaling=True, expect_ok=True):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from torchsso.utils.communicator import KFACCommunicator
        comm = KFACCommunicator(packer=TorchPacker(), wire_dtype=wire_dtype, wire_scaling=scaling)
        arrays = _make_arrays(rank, world, dims, spread)
        expect = ko.reduce_scatterv_mean([[t for t, _ in _make_arrays(r, world, dims, spread)[rank]]
                                          for r in range(world)])
        comm.reduce_scatterv_arrays(arrays)
        ok = all(_close(got, exp, rtol) for (got, _), exp in zip(arrays[rank], expect))
        if not expect_ok:
            assert not ok, 'the plain 16-bit cast was expected to lose these arrays'
            ret[rank] = 'ok'
            return
        assert ok, 'owner did not receive the world mean'
        # arrays owned by other ranks are untouched
        other = (rank + 1) % world
        for (got, _), (orig, _) in zip(arrays[other], _make_arrays(rank, world, dims, spread)[other]):
            assert torch.equal(got, orig)
        # all-gather: every rank ends with the owners' (averaged) values
        comm.allgatherv_arrays(arrays)
        for owner in range(world):
            exp = ko.reduce_scatterv_mean([[t for t, _ in _make_arrays(r, world, dims, spread)[owner]]
                                           for r in range(world)])
            for (got, _), e in zip(arrays[owner], exp):
                assert _close(got, e, 2 * rtol)
        # the replicas hold the same bits (with a 16-bit wire the owner takes the rounded values too)
        flat = torch.cat([t.reshape(-1) for local in arrays for t, _ in local]).clone()
        lo, hi = flat.clone(), flat.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), 'ranks disagree after the all-gather'
        sizes, seg = comm.segment_sizes(arrays)
        assert seg % 64 == 0 and seg >= max(sizes)
        # the layout of a list is remembered while the list comes back unchanged, recomputed when it grew
        assert comm._layout(arrays)[:2] == (sizes, seg)
        arrays[rank].append((torch.zeros(3 * seg), False))
        grown, seg2, _ = comm._layout(arrays)
        assert grown[rank] == sizes[rank] + 3 * seg and seg2 > seg
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


@pytest.mark.parametrize('wire', [torch.float16, torch.bfloat16])
def test_two_rank_exchange_gloo_half_wire(wire):
    """Optional 16-bit wire format: same exchange, values rounded to 11 / 8 mantissa bits on the way."""
    world, dims = 2, [5, 9]
    mgr = mp.Manager()
    ret = mgr.dict()
    rtol = 2e-3 if wire == torch.float16 else 1.5e-2
    mp.spawn(_worker, args=(world, _free_port(), dims, ret, wire, rtol), nprocs=world, join=True)
    assert dict(ret) == {0: 'ok', 1: 'ok'}


def test_half_wire_needs_its_per_array_scaling():
    """Arrays from 1e-6 to 1e+5: with the per-array scaling of the reference
    (pure_nccl_communicator.py:359-412) the fp16 exchange keeps 11 bits of every array; the plain
    cast underflows the small ones and overflows the large ones."""
    world, dims = 2, [5, 9]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), dims, ret, torch.float16, 2e-3, True, True, True), nprocs=world, join=True)
    assert dict(ret) == {0: 'ok', 1: 'ok'}
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), dims, ret, torch.float16, 2e-3, True, False, False), nprocs=world, join=True)
    assert dict(ret) == {0: 'ok', 1: 'ok'}


def test_three_rank_exchange_gloo():
    """Three ranks with unequal owner sizes: padded equal segments, every owner's offsets."""
    world, dims = 3, [4, 11, 7]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), dims, ret), nprocs=world, join=True)
    assert dict(ret) == {0: 'ok', 1: 'ok', 2: 'ok'}


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


def test_host_side_argument_checks():
    """Switches that are refused before anything touches a device."""
    import torchsso
    with pytest.raises(ValueError, match='prune_sampling_pass'):
        torchsso.get_closure_for_fisher(None, None, None, None, approx_type='mc', num_mc=2,
                                        prune_sampling_pass=False, batch_mc_passes=True)
    from torchsso.utils.communicator import KFACCommunicator
    assert not dist.is_initialized()
    with pytest.raises(RuntimeError, match='not initialised'):
        KFACCommunicator()
