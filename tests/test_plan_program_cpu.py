"""The engine's task programs (blocked Cholesky -> triangular inverse -> L^-T L^-1, Cholesky of
the inverse, precondition, sampling) are plain data: lists of tile tasks, diagonal-block records
and copy records.  Here the programs are built host-only over numpy buffers and interpreted by a
small numpy executor, which checks the planning logic without a GPU.  (The interpreter exists
only in this test; the product has no CPU execution path.)"""
import ctypes as C

import numpy as np
import pytest

from torchsso import _native as nat


class Mem:
    """Maps raw addresses back to the numpy buffers that own them."""

    def __init__(self):
        self.bufs = []

    def new(self, n, fill=None):
        a = np.full(n, np.nan, dtype=np.float32) if fill is None else np.full(n, fill, dtype=np.float32)
        self.bufs.append(a)
        return a

    def at(self, ptr):
        for a in self.bufs:
            base = a.ctypes.data
            if base <= ptr < base + a.nbytes:
                return a, (ptr - base) // 4
        raise KeyError(hex(ptr))

    def view(self, ptr, rows, cols, ld):
        a, off = self.at(ptr)
        assert off + (rows - 1) * ld + cols <= a.size, 'tile outside its buffer'
        return np.lib.stride_tricks.as_strided(a[off:], shape=(rows, cols), strides=(4 * ld, 4))


def run_program(plan, mem, shift=None, scale_alpha=None):
    tasks, _ = plan.tasks()
    diags, _ = plan.diag_recs()
    copies, _ = plan.copy_recs()
    info = {}
    for kind, first, count in plan.phases():
        if kind in (0, 1, 4):
            tile = 64 if kind == 0 else 128
            results = []
            for t in [tasks[i] for i in range(first, first + count)]:
                assert 0 < t.m <= tile and 0 < t.n <= tile and t.k > 0
                A = mem.view(t.A, t.k, t.m, t.lda).T if t.flags & 1 else mem.view(t.A, t.m, t.k, t.lda)
                B = mem.view(t.B, t.n, t.k, t.ldb).T if t.flags & 2 else mem.view(t.B, t.k, t.n, t.ldb)
                Cv = mem.view(t.C, t.m, t.n, t.ldc)
                alpha = t.alpha if scale_alpha is None or t.beta != 1.0 else scale_alpha * t.alpha
                val = alpha * (A.astype(np.float64) @ B.astype(np.float64))
                if t.beta != 0:
                    val = val + t.beta * Cv
                if t.flags & 4:
                    val = np.tril(val) + np.tril(val, -1).T
                results.append((t, val.astype(np.float32)))
            # tasks of one phase are independent: apply all writes after all reads
            for t, val in results:
                assert not np.isnan(val).any(), 'task read uninitialised memory'
                mem.view(t.C, t.m, t.n, t.ldc)[...] = val
                if t.C2:
                    mem.view(t.C2, t.n, t.m, t.ldc2)[...] = val.T
        elif kind in (2, 5):    # diagonal block: 64-wide, or a whole 128-column panel's
            assert all(diags[i].size <= (64 if kind == 2 else 128) for i in range(first, first + count))
            for r in [diags[i] for i in range(first, first + count)]:
                Lv = mem.view(r.L, r.size, r.size, r.ld_l)
                blk = np.tril(Lv).astype(np.float64)
                blk = blk + np.tril(blk, -1).T
                try:
                    L = np.linalg.cholesky(blk)
                except np.linalg.LinAlgError:
                    # LAPACK numbering, as the kernels report it: the first pivot that is not positive
                    bad = next(j for j in range(r.size) if np.linalg.eigvalsh(blk[:j + 1, :j + 1]).min() <= 0)
                    info[(r.mat, r.info_slot)] = r.row0 + bad + 1
                    L = np.eye(r.size)
                Lv[...] = L.astype(np.float32)
                Linv = np.linalg.inv(L).astype(np.float32)
                mem.view(r.Linv, r.size, r.size, r.ld_inv)[...] = Linv
                if r.LinvT:
                    mem.view(r.LinvT, r.size, r.size, r.ld_invt)[...] = Linv.T
        elif kind == 3:
            for r in [copies[i] for i in range(first, first + count)]:
                if r.mode == 3:     # tile += its partial products (128 columns apart, from src on)
                    tile = mem.view(r.dst, r.nrows, r.d, r.ld)
                    assert r.mat >= 1
                    for q in range(r.mat):
                        part = mem.view(r.src + 4 * 128 * q, r.nrows, r.d, r.ld)
                        assert not np.isnan(part).any(), 'partial product was never written'
                        tile += part
                    continue
                dst = mem.view(r.dst, r.d, r.d, r.ld)
                rows = slice(r.row0, r.row0 + r.nrows)
                if r.mode == 2:
                    dst[rows] = 0
                elif r.mode == 1:
                    src = mem.view(r.src, r.d, r.d, r.ld)
                    dst[rows] = np.triu(np.tril(src).T)[rows]
                else:
                    src = mem.view(r.src, r.d, r.d, r.ld)
                    dst[rows] = src[rows]
                    if r.mat >= 0:
                        for i in range(r.row0, r.row0 + r.nrows):
                            dst[i, i] += shift[r.mat]
        else:
            raise AssertionError(kind)
    return info


def spd(d, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((4 * d + 8, d)).astype(np.float32)
    return (x.T @ x / x.shape[0]).astype(np.float32)


@pytest.mark.parametrize('dims', [[10, 28], [64, 65], [130, 200], [257, 64, 1, 513], [1100, 700]])
def test_kron_inverse_and_std_program(dims):
    # cut the panel updates along K from the fourth panel on (default: the sixth), so that the small
    # matrices of this test exercise the partial-product tasks and the summing copies
    nat.configure('chol_ksplit', 4)
    try:
        _kron_inverse_and_std_program(dims)
    finally:
        nat.configure('chol_ksplit', 6)


def _kron_inverse_and_std_program(dims):
    mem = Mem()
    n = len(dims)
    src = [mem.new(d * d) for d in dims]
    dst = [mem.new(d * d) for d in dims]
    work = [mem.new(d * d) for d in dims]
    std = [mem.new(d * d) for d in dims]
    for i, d in enumerate(dims):
        src[i][:] = spd(d, 100 + i).ravel()
    partner = [i ^ 1 if (i ^ 1) < n else -1 for i in range(n)]
    role = [i & 1 for i in range(n)]
    plan = nat.kron_plan(dims, [a.ctypes.data for a in src], [a.ctypes.data for a in dst],
                         [a.ctypes.data for a in work], [a.ctypes.data for a in std],
                         partner, role, device=None, host_only=True)
    mem.bufs.append(plan.host_mem)
    r = np.sqrt(1e-3)
    shift = []
    for i, d in enumerate(dims):
        if partner[i] < 0:
            pi = 1.0
        else:
            a, g = (i, partner[i]) if role[i] == 0 else (partner[i], i)
            ta = np.trace(src[a].reshape(dims[a], dims[a])) / dims[a]
            tg = np.trace(src[g].reshape(dims[g], dims[g])) / dims[g]
            pi = np.sqrt(ta / tg)
        shift.append(r * pi if role[i] == 0 else r / pi)
    info = run_program(plan, mem, shift=shift)
    assert not info
    for i, d in enumerate(dims):
        M = src[i].reshape(d, d).astype(np.float64) + shift[i] * np.eye(d)
        inv = dst[i].reshape(d, d)
        ref = np.linalg.inv(M)
        assert np.linalg.norm(inv - ref) / np.linalg.norm(ref) < 1e-4, (d, 'inverse')
        assert np.array_equal(inv, inv.T)
        U = std[i].reshape(d, d)
        assert np.array_equal(U, np.triu(U))
        refU = np.linalg.cholesky(ref).T
        assert np.linalg.norm(U - refU) / np.linalg.norm(refU) < 1e-3, (d, 'std')


def test_kron_program_with_padded_leading_dimension():
    """Matrices whose rows are padded to a multiple of four floats (what the factor pool does for
    odd dimensions, so that every row starts on 16 bytes)."""
    mem = Mem()
    dims = [65, 201]
    lds = [(d + 3) // 4 * 4 for d in dims]
    src = [mem.new(d * l) for d, l in zip(dims, lds)]
    dst = [mem.new(d * l) for d, l in zip(dims, lds)]
    work = [mem.new(d * l) for d, l in zip(dims, lds)]
    std = [mem.new(d * l) for d, l in zip(dims, lds)]
    mats = []
    for i, (d, l) in enumerate(zip(dims, lds)):
        m = spd(d, 300 + i)
        mats.append(m)
        np.lib.stride_tricks.as_strided(src[i], shape=(d, d), strides=(4 * l, 4))[...] = m
    plan = nat.kron_plan(dims, [a.ctypes.data for a in src], [a.ctypes.data for a in dst],
                         [a.ctypes.data for a in work], [a.ctypes.data for a in std],
                         [1, 0], [0, 1], device=None, host_only=True, lds=lds)
    mem.bufs.append(plan.host_mem)
    r = np.sqrt(1e-3)
    ta, tg = np.trace(mats[0]) / dims[0], np.trace(mats[1]) / dims[1]
    pi = np.sqrt(ta / tg)
    shift = [r * pi, r / pi]
    assert not run_program(plan, mem, shift=shift)
    for i, (d, l) in enumerate(zip(dims, lds)):
        inv = np.lib.stride_tricks.as_strided(dst[i], shape=(d, d), strides=(4 * l, 4))
        ref = np.linalg.inv(mats[i].astype(np.float64) + shift[i] * np.eye(d))
        assert np.linalg.norm(inv - ref) / np.linalg.norm(ref) < 1e-4
        assert np.array_equal(inv, inv.T)
        U = np.lib.stride_tricks.as_strided(std[i], shape=(d, d), strides=(4 * l, 4))
        refU = np.linalg.cholesky(ref).T
        assert np.linalg.norm(U - refU) / np.linalg.norm(refU) < 1e-3


def test_kron_program_reports_bad_pivot():
    mem = Mem()
    d = 70
    src, dst, work = mem.new(d * d), mem.new(d * d), mem.new(d * d)
    m = spd(d, 3)
    m[66, 66] = -5.0
    src[:] = m.ravel()
    plan = nat.kron_plan([d], [src.ctypes.data], [dst.ctypes.data], [work.ctypes.data], None,
                         [-1], [0], device=None, host_only=True)
    mem.bufs.append(plan.host_mem)
    info = run_program(plan, mem, shift=[0.0])
    assert info == {(0, 0): 67}          # the failing pivot (row 66), 1-based


@pytest.mark.parametrize('dA,dG,bias', [(21, 16, True), (130, 70, True), (300, 129, False), (64, 1, True)])
def test_precondition_program(dA, dG, bias):
    mem = Mem()
    rng = np.random.default_rng(7)
    wc = dA - 1 if bias else dA
    Ainv, Ginv = mem.new(dA * dA), mem.new(dG * dG)
    gw, gb, tmp = mem.new(dG * wc), mem.new(dG), mem.new(dG * dA)
    Ainv[:] = spd(dA, 1).ravel()
    Ginv[:] = spd(dG, 2).ravel()
    gw[:] = rng.standard_normal(dG * wc).astype(np.float32)
    gb[:] = rng.standard_normal(dG).astype(np.float32)
    g2d = gw.reshape(dG, wc).copy()
    if bias:
        g2d = np.concatenate([g2d, gb.reshape(dG, 1)], axis=1)
    ref = Ginv.reshape(dG, dG).astype(np.float64) @ g2d @ Ainv.reshape(dA, dA).astype(np.float64)
    plan = nat.precond_plan([dA], [dG], [Ainv.ctypes.data], [Ginv.ctypes.data], [gw.ctypes.data],
                            [gb.ctypes.data if bias else None], [tmp.ctypes.data], device=None,
                            host_only=True)
    run_program(plan, mem)
    got = gw.reshape(dG, wc)
    if bias:
        got = np.concatenate([got, gb.reshape(dG, 1)], axis=1)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-5


@pytest.mark.parametrize('dA,dG,bias', [(21, 16, True), (200, 150, True), (129, 130, False)])
def test_sample_program(dA, dG, bias):
    mem = Mem()
    rng = np.random.default_rng(9)
    wc = dA - 1 if bias else dA
    UA, UG = mem.new(dA * dA), mem.new(dG * dG)
    noise, w, b, tmp = mem.new(dG * dA), mem.new(dG * wc), mem.new(dG), mem.new(dG * dA)
    UA[:] = np.triu(rng.standard_normal((dA, dA))).astype(np.float32).ravel()
    UG[:] = np.triu(rng.standard_normal((dG, dG))).astype(np.float32).ravel()
    noise[:] = rng.standard_normal(dG * dA).astype(np.float32)
    w[:] = rng.standard_normal(dG * wc).astype(np.float32)
    b[:] = rng.standard_normal(dG).astype(np.float32)
    mean = w.reshape(dG, wc).copy()
    if bias:
        mean = np.concatenate([mean, b.reshape(dG, 1)], axis=1)
    s = 0.37
    ref = mean + s * (UG.reshape(dG, dG).astype(np.float64) @ noise.reshape(dG, dA) @ UA.reshape(dA, dA))
    plan = nat.sample_plan([dA], [dG], [UA.ctypes.data], [UG.ctypes.data], [noise.ctypes.data],
                           [w.ctypes.data], [b.ctypes.data if bias else None], [tmp.ctypes.data],
                           device=None, host_only=True)
    run_program(plan, mem, scale_alpha=s)
    got = w.reshape(dG, wc)
    if bias:
        got = np.concatenate([got, b.reshape(dG, 1)], axis=1)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-5


def test_library_exports_every_declared_symbol():
    import os
    import re
    hdr = open(os.path.join(os.path.dirname(__file__), '..', 'include', 'sso_b200.h')).read()
    names = set(re.findall(r'\b(sso_[a-z0-9_]+)\s*\(', hdr))
    assert names, 'no declarations found'
    lib = nat.lib()
    for name in sorted(names):
        assert hasattr(lib, name), name
    assert names == set(nat.SIGNATURES), names ^ set(nat.SIGNATURES)
    assert lib.sso_version() == 100
