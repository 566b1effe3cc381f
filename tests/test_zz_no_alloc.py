"""The allocation-free prefill entry point (lbk_ternary_linear_prefill_static).

Some callers may not allocate device memory at all: a serving loop that forbids allocator calls
once it is running, a plug-in living inside somebody else's CUDA heap budget. For them the
library keeps the prefill path's quantised activations in a fixed array of its own instead of
cudaMalloc'd scratch. This file checks, through the C ABI, that the entry point gives the same
bits as the regular one (lbk_ternary_linear_n) on two calls in a row that share the array -- the
second smaller than the first, so stale bytes from the first call would show -- and that a
request beyond the array's size is refused with a clear message. It is named to be collected
last, so a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _group(ctx, oracle, cols, shapes, seed):
    import torch
    from lemonade_burn_b200 import ops
    rng = np.random.default_rng(seed)
    lins = []
    for rows, sc in shapes:
        t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
        lins.append(ops.TernaryLinear(torch.from_numpy(oracle.pack_matrix(t)).cuda(), sc, cols, ctx))
    return lins


def _call(ctx, name, x, lins):
    import torch
    from lemonade_burn_b200 import _lib
    m = x.shape[0]
    outs = [torch.full((m, l.rows), float("nan"), device="cuda") for l in lins]
    iouts = [torch.full((m, l.rows), -7, dtype=torch.int32, device="cuda") for l in lins]
    wp, k1 = _lib.ptr_array([l.weight.handle.value for l in lins])
    op, k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    ip, k3 = _lib.ptr_array([o.data_ptr() for o in iouts])
    st = getattr(ctx._lib, name)(ctx.handle, C.c_void_p(x.data_ptr()), m, wp, len(lins), op, ip,
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return st, outs, iouts


def _call_into(ctx, name, x, lins, outs, iouts):
    """The same call into buffers that already exist: nothing in the test allocates around it."""
    import torch
    from lemonade_burn_b200 import _lib
    wp, k1 = _lib.ptr_array([l.weight.handle.value for l in lins])
    op, k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    ip, k3 = _lib.ptr_array([o.data_ptr() for o in iouts])
    st = getattr(ctx._lib, name)(ctx.handle, C.c_void_p(x.data_ptr()), x.shape[0], wp, len(lins), op, ip,
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return st, outs, iouts


def test_static_scratch_matches_regular_entry_twice(oracle, ctx):
    import torch
    cols = 640
    lins = _group(ctx, oracle, cols, [(300, 41.0), (96, 57.5)], 5)
    g = torch.Generator().manual_seed(9)
    # 70 then 33 rows: the second call is smaller, so anything left over from the first must not matter.
    # 8, 4 and 1 rows: the regular entry point takes its fused few-row kernel there, this one still
    # quantises and runs the GEMM; the bits must be the same.
    for m in (70, 33, 8, 4, 1):
        x = torch.randn(m, cols, generator=g).cuda()
        st_a, out_a, iout_a = _call(ctx, "lbk_ternary_linear_n", x, lins)
        st_b, out_b, iout_b = _call(ctx, "lbk_ternary_linear_prefill_static", x, lins)
        assert st_a == 0 and st_b == 0, ctx._lib.lbk_last_error()
        # the property the entry point exists for: the call takes no device memory (measured after the
        # outputs are allocated, around the call alone; cudaMemGetInfo would show any cudaMalloc)
        free_before = torch.cuda.mem_get_info()[0]
        st_c, out_c, iout_c = _call_into(ctx, "lbk_ternary_linear_prefill_static", x, lins, out_b, iout_b)
        assert st_c == 0 and torch.cuda.mem_get_info()[0] == free_before
        for a, b in zip(iout_a, iout_b):
            assert torch.equal(a, b)                      # int32 accumulators: bit exact
        for a, b in zip(out_a, out_b):
            assert torch.equal(a.view(torch.int32), b.view(torch.int32))  # f32 outputs: same bits
        # and both agree with the CPU oracle
        q, s, ssum = oracle.quantize_acts(x.cpu().numpy())
        for l, b in zip(lins, iout_b):
            want = oracle.ternary_gemm_i32(l.packed.cpu().numpy(), cols, q, ssum)
            assert np.array_equal(b.cpu().numpy(), want)
    ctx.check_device_error()


def test_static_scratch_refuses_oversize(oracle, ctx):
    import torch
    cols = 8192
    lins = _group(ctx, oracle, cols, [(32, 1.0)], 6)
    m = 1025  # 1025 * 8192 bytes > 8 MiB
    x = torch.zeros(m, cols, device="cuda")
    st, _, _ = _call(ctx, "lbk_ternary_linear_prefill_static", x, lins)
    assert st == 4  # LBK_ERR_UNSUPPORTED
    msg = ctx._lib.lbk_last_error().decode()
    assert "static scratch too small" in msg and "8388608" in msg
    st, _, _ = _call(ctx, "lbk_ternary_linear_prefill_static", torch.zeros(1024, cols, device="cuda"), lins)
    assert st == 0, ctx._lib.lbk_last_error()
