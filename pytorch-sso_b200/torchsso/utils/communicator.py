"""Factor / update exchange for data-parallel K-FAC over torch.distributed (NCCL on NVLink).

Replaces the ChainerMN communicator of the reference
(torchsso/utils/chainer_communicators/pure_nccl_communicator.py:114-309 with the Packer of
_utility.py:16-104).  Semantics kept: after ``reduce_scatterv_data`` the owner rank of every
layer holds the WORLD MEAN of that layer's gradients and curvature data (symmetric factors
travel as packed upper triangles); after ``allgatherv_data`` every rank holds the owners'
values.  What differs is the mechanism: the reference all-reduces the whole buffer twice
(every rank receives everything); here the first exchange is a true reduce-scatter over
equal, padded per-owner segments and the second a true all-gather, so each rank moves
(N-1)/N of ONE segment set instead of two full buffers, and pack / scale / unpack are one
kernel launch each over a device-side table.

The class works on "arrays": for every rank a list of ``(tensor, triangular)`` pairs in a
fixed order, where ``triangular`` means "square matrix, send the upper triangle".
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

Arrays = List[List[Tuple[torch.Tensor, bool]]]


def assign_owners(costs: Sequence[float], world: int, mode: str = 'inverse_cost') -> List[List[int]]:
    """Partition group indices over ranks.

    'contiguous'   : numpy.array_split of the index range (torchsso/optim/secondorder.py:341-346).
    'inverse_cost' : longest-processing-time greedy on ``costs`` (d_A^3 + d_G^3 per layer), ties
                     and zero-cost groups going to the rank with the fewest groups; each rank's
                     list is returned in ascending index order."""
    n = len(costs)
    if mode == 'contiguous':
        return [part.tolist() for part in np.array_split(np.arange(n), world)]
    if mode != 'inverse_cost':
        raise ValueError('unknown balance mode: %s' % mode)
    load = [0.0] * world
    count = [0] * world
    parts = [[] for _ in range(world)]
    for i in sorted(range(n), key=lambda i: (-costs[i], i)):
        r = min(range(world), key=lambda r: (load[r], count[r], r))
        parts[r].append(i)
        load[r] += costs[i]
        count[r] += 1
    return [sorted(p) for p in parts]


def packed_numel(t: torch.Tensor, triangular: bool) -> int:
    if triangular:
        n = t.shape[0]
        return n * (n + 1) // 2
    return t.numel()


class DevicePacker:
    """Pack / unpack with the sm_100a kernels (one launch per direction per table)."""

    def __init__(self):
        self._tables = {}
        self._by_list = {}

    def _table(self, arrays, buf, offset, direction):
        from torchsso import _native as nat
        # A list that comes back unchanged (the communicator caches the lists it extracts) is recognised by
        # identity, length and its first and last tensor: asking every tensor of a ResNet-50 for its
        # address on every call costs more host time than the kernels take on the device.
        quick = (direction, buf.data_ptr(), offset, id(arrays))
        hit = self._by_list.get(quick)
        if (hit is not None and hit[0] is arrays and hit[1] == len(arrays) and arrays and
                hit[2] == (arrays[0][0].data_ptr(), arrays[-1][0].data_ptr())):
            return hit[3]
        key = (direction, buf.data_ptr(), offset, tuple((t.data_ptr(), tri) for t, tri in arrays))
        ent = self._tables.get(key)
        if ent is None:
            flat_pairs, tri_mats, tri_offs, strided, off = [], [], [], ([], []), offset
            for t, tri in arrays:
                k = packed_numel(t, tri)
                if tri:
                    tri_mats.append(t)
                    tri_offs.append(off)
                elif t.is_contiguous() and t.dtype == torch.float32:
                    seg = buf[off: off + k]
                    flat_pairs.append((t.reshape(-1), seg) if direction == 'pack' else (seg, t.reshape(-1)))
                else:
                    # e.g. channels_last convolution weights: multi-tensor strided copy
                    strided[0].append(t)
                    strided[1].append(buf[off: off + k].view(t.shape))
                off += k
            seg_tab = nat.seg_records(flat_pairs, buf.device) if flat_pairs else None
            # unpacking goes in bands of 32 rows (the kernel transposes 32 x 32 tiles below the diagonal)
            tri_tab = nat.tri_records(tri_mats, buf, tri_offs, 32 if direction == 'unpack' else 0) if tri_mats else None
            while len(self._tables) >= 256:      # oldest first; one model needs 2 x world entries
                self._tables.pop(next(iter(self._tables)))
            ent = (seg_tab, tri_tab, strided)
            self._tables[key] = ent
        if arrays:
            while len(self._by_list) >= 256:
                self._by_list.pop(next(iter(self._by_list)))
            # (the entry keeps the list alive, so its id cannot be handed to another list meanwhile)
            self._by_list[quick] = (arrays, len(arrays), (arrays[0][0].data_ptr(), arrays[-1][0].data_ptr()), ent)
        return ent

    # ---- 16-bit wire format (per-array scaling fused into the casts) ---------------------------
    def wire_table(self, offsets, counts, ids, device):
        from torchsso import _native as nat
        return nat.wire_records(offsets, counts, device, ids=ids)

    def wire_absmax(self, buf, table, maxima):
        from torchsso import _native as nat
        nat.wire_absmax(buf, table, maxima)

    def wire_encode(self, buf, table, sums, out16):
        from torchsso import _native as nat
        nat.wire_encode(buf, table, sums, out16)

    def wire_decode(self, in16, table, sums, out32):
        from torchsso import _native as nat
        nat.wire_decode(in16, table, sums, out32)

    def pack(self, arrays, buf, offset, scale):
        from torchsso import _native as nat
        seg_tab, tri_tab, (tensors, views) = self._table(arrays, buf, offset, 'pack')
        if seg_tab is not None:
            nat.copy_segments(seg_tab, scale)
        if tri_tab is not None:
            nat.tri_pack(tri_tab, scale)
        if tensors:
            torch._foreach_copy_(views, tensors)
            if scale != 1.0:
                torch._foreach_mul_(views, scale)

    def unpack(self, arrays, buf, offset, symmetric=True):
        from torchsso import _native as nat
        seg_tab, tri_tab, (tensors, views) = self._table(arrays, buf, offset, 'unpack')
        if seg_tab is not None:
            nat.copy_segments(seg_tab, 1.0)
        if tri_tab is not None:
            nat.tri_unpack(tri_tab, 1.0, symmetric)
        if tensors:
            torch._foreach_copy_(tensors, views)


class KFACCommunicator:

    def __init__(self, group=None, packer=None, wire_dtype=None, wire_scaling=True):
        """``wire_dtype`` (torch.bfloat16 / torch.float16, default None = fp32): the packed buffers
        cross the links in that type (half the bytes), as the reference's ``allreduce_grad_dtype``
        option does, with its per-array scaling (pure_nccl_communicator.py:359-412): the maximum
        magnitude of every array is taken on each rank, the maxima are summed over the ranks (one small
        all-reduce), every array is scaled to 65000 / sum on the way into the 16-bit buffer and scaled
        back on the way out, so arrays of very different magnitude (G factors carry an n^2, late-layer
        gradients are tiny) neither overflow nor underflow.  ``wire_scaling=False`` is the plain cast.
        It still rounds factors and gradients to 8 / 11 mantissa bits, so it is off in every parity
        configuration."""
        if not dist.is_initialized():
            raise RuntimeError('torch.distributed is not initialised')
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.packer = packer if packer is not None else DevicePacker()
        if wire_dtype not in (None, torch.float32, torch.bfloat16, torch.float16):
            raise ValueError('wire_dtype must be None, torch.bfloat16 or torch.float16')
        self.wire_dtype = None if wire_dtype == torch.float32 else wire_dtype
        self.wire_scaling = bool(wire_scaling)
        self._wire_layouts = {}
        self._extract_cache = {}
        self._layouts = {}
        self.indices = None
        self._optimizer = None
        self._bufs = {}
        self.last_bytes = {'rsv': 0, 'agv': 0}

    # ---- wiring ----------------------------------------------------------------------------
    def setup(self, optimizer):
        self._optimizer = optimizer

    def _buffer(self, name, numel, device):
        b = self._bufs.get(name)
        if b is None or b.numel() < numel or b.device != device:
            b = torch.zeros(numel, dtype=torch.float32, device=device)
            self._bufs[name] = b
        return b[:numel]

    @staticmethod
    def segment_sizes(arrays: Arrays):
        sizes = [sum(packed_numel(t, tri) for t, tri in local) for local in arrays]
        seg = max(sizes) if sizes else 0
        seg = (seg + 63) // 64 * 64       # equal, 256-byte aligned segments
        return sizes, seg

    def _layout(self, arrays: Arrays):
        """(sizes, segment length, device) of a list of arrays; remembered for lists that come back
        unchanged (same object, same lengths), like the ones ``extract`` caches."""
        lens = tuple(len(local) for local in arrays)
        hit = self._layouts.get(id(arrays))
        if hit is not None and hit[0] is arrays and hit[1] == lens:
            return hit[2]
        sizes, seg = self.segment_sizes(arrays)
        device = next((t.device for local in arrays for t, _ in local), None)
        while len(self._layouts) >= 16:
            self._layouts.pop(next(iter(self._layouts)))
        self._layouts[id(arrays)] = (arrays, lens, (sizes, seg, device))
        return sizes, seg, device

    # ---- the two collectives -----------------------------------------------------------------
    def reduce_scatterv_arrays(self, arrays: Arrays):
        """Owner r ends up with the world mean of every array in arrays[r]."""
        sizes, seg, device = self._layout(arrays)
        if seg == 0:
            return
        send = self._buffer('rsv_send', seg * self.size, device)
        recv = self._buffer('rsv_recv', seg, device)
        for r, local in enumerate(arrays):
            if local:
                self.packer.pack(local, send, r * seg, 1.0 / self.size)
        if self.size > 1:
            self._reduce_scatter(recv, send, seg, arrays)
        else:
            recv = send[:seg]
        if arrays[self.rank]:
            self.packer.unpack(arrays[self.rank], recv, 0, True)
        self.last_bytes['rsv'] = (4 if self.wire_dtype is None else 2) * seg * self.size

    def allgatherv_arrays(self, arrays: Arrays, symmetric=True):
        """Every rank ends up with rank r's values of every array in arrays[r]."""
        sizes, seg, device = self._layout(arrays)
        if seg == 0:
            return
        send = self._buffer('agv_send', seg, device)
        recv = self._buffer('agv_recv', seg * self.size, device)
        if arrays[self.rank]:
            self.packer.pack(arrays[self.rank], send, 0, 1.0)
        if self.size > 1:
            self._all_gather(recv, send, seg, arrays)
        else:
            recv = send
        # with a 16-bit wire the owner takes the rounded values back too: every rank must hold the same
        # bits, or the replicas drift apart by one wire rounding per step
        rounded = self.wire_dtype is not None and self.size > 1
        for r, local in enumerate(arrays):
            if local and (r != self.rank or rounded):
                self.packer.unpack(local, recv, r * seg, symmetric)
        self.last_bytes['agv'] = (4 if self.wire_dtype is None else 2) * seg * self.size

    def _wire(self, name, like):
        b = self._bufs.get(name)
        if b is None or b.numel() < like.numel() or b.device != like.device or b.dtype != self.wire_dtype:
            b = torch.zeros(like.numel(), dtype=self.wire_dtype, device=like.device)
            self._bufs[name] = b
        return b[:like.numel()]

    def _wire_layout(self, arrays: Arrays, seg: int, device):
        """(table over the whole [world x seg] buffer, table over this rank's segment alone, maxima
        vector): array i of the flattened per-owner lists has index i in the maxima."""
        key = (seg, tuple((t.data_ptr(), tri) for local in arrays for t, tri in local))
        ent = self._wire_layouts.get(key)
        if ent is None:
            offs, cnts, ids, l_offs, l_cnts, l_ids = [], [], [], [], [], []
            i = 0
            for r, local in enumerate(arrays):
                off = 0
                for t, tri in local:
                    k = packed_numel(t, tri)
                    offs.append(r * seg + off); cnts.append(k); ids.append(i)
                    if r == self.rank:
                        l_offs.append(off); l_cnts.append(k); l_ids.append(i)
                    off += k
                    i += 1
            whole = self.packer.wire_table(offs, cnts, ids, device)
            own = self.packer.wire_table(l_offs, l_cnts, l_ids, device) if l_ids else None
            maxima = torch.zeros(max(i, 1), dtype=torch.float32, device=device)
            while len(self._wire_layouts) >= 8:
                self._wire_layouts.pop(next(iter(self._wire_layouts)))
            ent = (whole, own, maxima)
            self._wire_layouts[key] = ent
        return ent

    def _reduce_scatter(self, recv, send, seg, arrays=None):
        if self.wire_dtype is None:
            self._reduce_scatter_raw(recv, send, seg)
            return
        send16, recv16 = self._wire('rsv_send16', send), self._wire('rsv_recv16', recv)
        if self.wire_scaling and arrays is not None:
            whole, own, maxima = self._wire_layout(arrays, seg, send.device)
            maxima.zero_()
            self.packer.wire_absmax(send, whole, maxima)
            dist.all_reduce(maxima, op=dist.ReduceOp.SUM, group=self.group)
            self.packer.wire_encode(send, whole, maxima, send16)
            self._reduce_scatter_raw(recv16, send16, seg)
            if own is not None:
                self.packer.wire_decode(recv16, own, maxima, recv)
            return
        send16.copy_(send)
        self._reduce_scatter_raw(recv16, send16, seg)
        recv.copy_(recv16)

    def _all_gather(self, recv, send, seg, arrays=None):
        if self.wire_dtype is None:
            self._all_gather_raw(recv, send, seg)
            return
        send16, recv16 = self._wire('agv_send16', send), self._wire('agv_recv16', recv)
        if self.wire_scaling and arrays is not None:
            whole, own, maxima = self._wire_layout(arrays, seg, send.device)
            maxima.zero_()
            if own is not None:
                self.packer.wire_absmax(send, own, maxima)
            # only the owner contributes a non-zero maximum for an array, so the sum is the owner's value
            dist.all_reduce(maxima, op=dist.ReduceOp.SUM, group=self.group)
            if own is not None:
                self.packer.wire_encode(send, own, maxima, send16)
            self._all_gather_raw(recv16, send16, seg)
            self.packer.wire_decode(recv16, whole, maxima, recv)
            return
        send16.copy_(send)
        self._all_gather_raw(recv16, send16, seg)
        recv.copy_(recv16)

    def _reduce_scatter_raw(self, recv, send, seg):
        backend = dist.get_backend(self.group)
        if backend == 'nccl':
            dist.reduce_scatter_tensor(recv, send, op=dist.ReduceOp.SUM, group=self.group)
        else:   # gloo has no reduce-scatter: reduce everything, keep the own segment
            dist.all_reduce(send, op=dist.ReduceOp.SUM, group=self.group)
            recv.copy_(send[self.rank * seg:(self.rank + 1) * seg])

    def _all_gather_raw(self, recv, send, seg):
        backend = dist.get_backend(self.group)
        if backend == 'nccl':
            dist.all_gather_into_tensor(recv, send, group=self.group)
        elif send.is_cuda:
            # gloo carries device tensors through the host and implements all_reduce for them: place the
            # own segment into a zeroed buffer and sum (ranks that share one GPU in tests take this path)
            recv.zero_()
            recv[self.rank * seg:(self.rank + 1) * seg].copy_(send)
            dist.all_reduce(recv, op=dist.ReduceOp.SUM, group=self.group)
        else:
            parts = [recv[r * seg:(r + 1) * seg] for r in range(self.size)]
            dist.all_gather(parts, send, group=self.group)

    # ---- optimizer-facing API (names of the reference communicator) ------------------------------
    def extract(self, param_groups, extractors) -> Arrays:
        """Arrays per owner rank: for every owned group, in order, what each extractor names:
        'grad' (flat-pool gradient views), 'param.data', 'mean.data', 'curv.data', 'curv.std'."""
        opt = self._optimizer
        # the lists depend on which tensors exist, not on their values: rebuild only when the groups'
        # storage changes (the pools and the flat gradient buffer are allocated once)
        # (lists that name parameter storage are rebuilt every time: a caller may swap ``p.data``)
        cacheable = not any(ex in ('param.data', 'mean.data', 'curv.std') for ex in extractors)
        key = (id(param_groups), tuple(extractors), id(getattr(opt, 'pool', None)), id(getattr(opt, '_grad_flat', None)))
        hit = self._extract_cache.get(key) if cacheable else None
        if hit is not None and hit[0] is param_groups:
            return hit[1]
        arrays = []
        for local_indices in self.indices:
            local = []
            for i in local_indices:
                group = param_groups[i]
                for ex in extractors:
                    if ex == 'grad':
                        local += [(opt._grad_view[p], False) for p in group['params']]
                    elif ex == 'param.data':
                        local += [(p.data, False) for p in group['params']]
                    elif ex == 'mean.data':
                        local += [(m.data, False) for m in group['mean']]
                    elif ex in ('curv.data', 'curv.std'):
                        curv = group['curv']
                        if curv is None:
                            continue
                        role = ex.split('.')[1]
                        if role == 'std' and group.get('std_scale', 0) <= 0:
                            continue
                        for x in curv._views(role):
                            tri = x.dim() == 2 and x.shape[0] == x.shape[1]
                            local.append((x, tri))
                    else:
                        raise ValueError('unknown extractor %r' % (ex,))
            arrays.append(local)
        if cacheable:
            while len(self._extract_cache) >= 16:
                self._extract_cache.pop(next(iter(self._extract_cache)))
            self._extract_cache[key] = (param_groups, arrays)
        return arrays

    def reduce_scatterv_data(self, param_groups, extractors):
        self.reduce_scatterv_arrays(self.extract(param_groups, extractors))
        # the owner now holds averaged curvature data for its groups
        for i in self.indices[self.rank]:
            curv = param_groups[i]['curv']
            if curv is not None:
                curv._have.add('data')

    def allgatherv_data(self, param_groups, extractors):
        has_std = 'curv.std' in extractors
        self.allgatherv_arrays(self.extract(param_groups, extractors), symmetric=not has_std)
        if has_std:
            for group in param_groups:
                curv = group['curv']
                if curv is not None and group.get('std_scale', 0) > 0:
                    curv._have.add('std')


def create_communicator(group=None, packer=None, wire_dtype=None, wire_scaling=True, **unused):
    """Communicator over the default (or given) process group; one process per GPU, NCCL backend."""
    return KFACCommunicator(group=group, packer=packer, wire_dtype=wire_dtype, wire_scaling=wire_scaling)
