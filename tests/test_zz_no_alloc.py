"""The allocation-free factor entry point (for hosts that may not call cudaMalloc once they are
running: all device memory owned by their own pool, or a fixed budget after start-up) must give
the same matrix as the ordinary entry point, which is handed scratch by the caller.

It works out of one fixed 16 MiB array inside the library that every call on a device shares and
that keeps whatever the previous call left in it, so the check is made on two different problems
in a row: stale partial tiles from the first must not leak into the second.  This file sorts
last so that the rest of the suite has run before it; it also passes on its own."""
import pytest
import torch

pytestmark = pytest.mark.gpu

_PRIMED = []


def _both(nat, x, bias, alpha, beta, impl, seed_out):
    rows, cols = x.shape
    d = cols + int(bias)
    L = nat.lib()
    stream = torch.cuda.current_stream().cuda_stream
    init = torch.randn((d, d), device='cuda', generator=torch.Generator(device='cuda').manual_seed(seed_out))
    ref, got = init.clone(), init.clone()
    nbytes = L.sso_factor_workspace_bytes(rows, d, impl)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device='cuda')
    nat._check(L.sso_factor_syrk(x.data_ptr(), nat._dtype_code(x), rows, cols, x.stride(0), x.stride(1),
                                 int(bias), None, alpha, beta, ref.data_ptr(), d, ws.data_ptr(), nbytes,
                                 impl, stream))
    if not _PRIMED:
        # The very first use of the entry point on a device resolves the address of its built-in
        # scratch array; with CUDA's lazy module loading that is also the moment the driver sets the
        # array's 16 MiB aside.  From then on no call changes the amount of free device memory.
        tmp = torch.zeros((d, d), device='cuda')
        nat._check(L.sso_factor_syrk_noalloc(x.data_ptr(), nat._dtype_code(x), rows, cols, x.stride(0),
                                             x.stride(1), int(bias), None, alpha, 0.0, tmp.data_ptr(), d,
                                             impl, stream))
        _PRIMED.append(True)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]     # sees allocations made behind torch's back as well
    nat._check(L.sso_factor_syrk_noalloc(x.data_ptr(), nat._dtype_code(x), rows, cols, x.stride(0),
                                         x.stride(1), int(bias), None, alpha, beta, got.data_ptr(), d,
                                         impl, stream))
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before, 'the call took device memory'
    # and against the CPU oracle, so that two wrong-but-equal results cannot pass
    from oracle import kfac_oracle as ko
    exact = ko.linear_factor_A(x.double().cpu(), bias) * (alpha * rows) + beta * init.double().cpu()
    err = ((got.double().cpu() - exact).norm() / exact.norm()).item()
    assert err < 1e-5, err
    return ref, got


@pytest.mark.parametrize('impl_name', ['IMPL_SIMT', 'IMPL_TCGEN05', 'IMPL_AUTO', 'IMPL_TMA'])
def test_noalloc_entry_matches_regular_entry_twice(impl_name):
    from torchsso import _native as nat
    impl = getattr(nat, impl_name)
    g = torch.Generator(device='cuda').manual_seed(11)
    # first problem: many row splits, so the shared scratch is left full of partial tiles
    x1 = torch.randn((20000, 96), device='cuda', generator=g)
    bias1 = True
    if impl == nat.IMPL_TMA:      # the TMA-fed kernel takes 16-bit rows of a multiple of 64 columns, no ones column
        x1, bias1 = torch.randn((20000, 128), device='cuda', generator=g).bfloat16(), False
    ref1, got1 = _both(nat, x1, bias1, 1.0 / 20000, 0.0, impl, 1)
    # second problem, different shape and an accumulate (beta = 1) on top of existing contents; 192 bf16
    # columns take the automatic choice to the TMA-fed kernel
    cols2 = 200 if impl in (nat.IMPL_SIMT, nat.IMPL_TCGEN05) else 192
    x2 = (torch.randn((3000, cols2), device='cuda', generator=g) + 0.5).bfloat16()
    ref2, got2 = _both(nat, x2, False, 1.0 / 3000, 1.0, impl, 2)
    for ref, got in ((ref1, got1), (ref2, got2)):
        assert torch.isfinite(got).all()
        err = ((got.double() - ref.double()).norm() / ref.double().norm()).item()
        assert err < 1e-6, err            # same kernels, same split schedule: expected to be identical


def test_noalloc_entry_rejects_problems_beyond_its_scratch():
    from torchsso import _native as nat
    L = nat.lib()
    rows, cols = 400000, 1024               # needs far more than 16 MiB of partial tiles
    assert L.sso_factor_workspace_bytes(rows, cols, nat.IMPL_SIMT) > (16 << 20)
    x = torch.zeros((8, 8), device='cuda')  # never read: the call must fail before launching
    out = torch.zeros((cols, cols), device='cuda')
    rc = L.sso_factor_syrk_noalloc(x.data_ptr(), 0, rows, cols, cols, 1, 0, None, 1.0, 0.0, out.data_ptr(),
                                   cols, nat.IMPL_SIMT, torch.cuda.current_stream().cuda_stream)
    assert rc < 0
    assert b'built-in' in L.sso_last_error()
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
