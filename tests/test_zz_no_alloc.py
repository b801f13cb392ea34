"""The allocation-free LayerNorm backward (bb_layernorm_bwd_static) against the regular entry
point.  It is for hosts that may not allocate GPU memory after start-up; its scratch is an
array inside the library, shared by every call on the device, so the test calls it twice in a
row (the second call meets the first call's leftovers) and compares both results with
bb_layernorm_bwd on the same inputs.  Collected last on purpose: a failure here cannot hide
another test's result when the run stops at the first failure."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(rows, h, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, h, device="cuda", generator=g).bfloat16()
    dy = torch.randn(rows, h, device="cuda", generator=g).bfloat16()
    dres = torch.randn(rows, h, device="cuda", generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(h, device="cuda", generator=g)).bfloat16()
    beta = torch.zeros(h, device="cuda").bfloat16()
    return x, dy, dres, gamma, beta


def _run(fn, L, x, dy, dres, gamma, beta):
    rows, h = x.shape
    y = torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    L.layernorm_fwd(x, gamma, beta, y, mean, rstd, 1e-5)
    dx = torch.empty_like(x)
    dg, db = torch.zeros(h, device="cuda"), torch.zeros(h, device="cuda")
    fn(dy, x, gamma, mean, rstd, dres, dx, dg, db)
    torch.cuda.synchronize()
    return dx, dg, db


def test_static_scratch_entry_point_matches_regular_one():
    from bamboo_b200 import lib as L
    L.load()
    # different problems back to back: each reuses scratch the previous one dirtied.  Hidden
    # sizes that are multiples of 256 take the column-owner kernel, 1000 the generic
    # row kernel, 512 and 768 the register-resident row kernels
    for rows, h, seed in ((4096, 1024, 1), (1000, 768, 2), (777, 1000, 3), (2048, 512, 4)):
        args = _inputs(rows, h, seed)
        want = _run(L.layernorm_bwd, L, *args)
        got = _run(L.layernorm_bwd_static, L, *args)
        for a, b in zip(got, want):
            # same kernels, same grid, same summation order: bit-identical
            assert torch.equal(a, b)
    assert L.read_status() == 0


def test_static_scratch_entry_point_allocates_nothing():
    """The entry point's defining property: with outputs allocated beforehand, a call changes
    neither the driver's free-memory figure nor the caching allocator's reservation."""
    from bamboo_b200 import lib as L
    L.load()
    x, dy, dres, gamma, beta = _inputs(4096, 1024, 5)
    rows, h = x.shape
    y = torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    L.layernorm_fwd(x, gamma, beta, y, mean, rstd, 1e-5)
    dx = torch.empty_like(x)
    dg, db = torch.zeros(h, device="cuda"), torch.zeros(h, device="cuda")
    for _ in range(2):                                     # the first call on a device looks the array up
        L.layernorm_bwd_static(dy, x, gamma, mean, rstd, dres, dx, dg, db)
    torch.cuda.synchronize()
    free0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
    L.layernorm_bwd_static(dy, x, gamma, mean, rstd, dres, dx, dg, db)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_reserved() == reserved0


def test_static_scratch_entry_point_rejects_oversized_problems():
    from bamboo_b200 import lib as L
    handle = L.load()
    handle.bb_layernorm_bwd_static_capacity_bytes.restype = ctypes.c_longlong
    handle.bb_layernorm_bwd_workspace_bytes.restype = ctypes.c_longlong
    cap = handle.bb_layernorm_bwd_static_capacity_bytes()
    assert cap == 8 << 20
    rows, h = 8192, 8192
    assert handle.bb_layernorm_bwd_workspace_bytes(rows, h) > cap
    x, dy, dres, gamma, beta = _inputs(64, h, 3)          # pointers only need to be valid
    dx = torch.empty_like(x)
    mean, rstd = torch.zeros(rows, device="cuda"), torch.ones(rows, device="cuda")
    dg, db = torch.zeros(h, device="cuda"), torch.zeros(h, device="cuda")
    rc = handle.bb_layernorm_bwd_static(ctypes.c_void_p(dy.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                        ctypes.c_void_p(gamma.data_ptr()), ctypes.c_void_p(mean.data_ptr()),
                                        ctypes.c_void_p(rstd.data_ptr()), None, ctypes.c_void_p(dx.data_ptr()),
                                        ctypes.c_void_p(dg.data_ptr()), ctypes.c_void_p(db.data_ptr()),
                                        ctypes.c_int(rows), ctypes.c_int(h), None)
    assert rc == -4 and b"needs" in handle.bb_last_error()
