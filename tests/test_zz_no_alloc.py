"""The allocation-free norm backward (``pf_norm_bwd_static``), called through its exported C
symbol the way an embedding application would, against the regular entry point that takes a
caller-provided scratch buffer.

Who needs it: code that may not call cudaMalloc where it runs, e.g. a plugin confined to a
workspace its host handed it, or a loop that cannot afford an allocation.  The test makes two
calls in a row (the built-in scratch keeps the first call's contents, so the second call checks
that stale partial sums do not leak into the result) and checks the size limit is enforced.
This file sorts last so that a failure here cannot hide the other tests under ``-x``.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(L, fn_name, scratch, dy, h, gamma, mean, rstd, dx, dg, db, rows, N, sm):
    vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fn = getattr(L, fn_name)
    args = [vp(dy), vp(h), vp(gamma), vp(mean), vp(rstd), vp(None), vp(dx), vp(dg), vp(db)]
    if scratch is not None:
        args.append(vp(scratch))
    args += [ctypes.c_longlong(rows), N, 0, 0, 2, sm, stream]       # LayerNorm, bf16
    return fn(*args)


def test_static_scratch_entry_matches_regular_entry_twice():
    from pfeife_b200.ops import _lib
    from pfeife_b200.ops import kernels as kx
    L = _lib.lib()
    _lib.bind_thread(torch.cuda.current_device())
    sm = _lib.sm_count()
    for call, (rows, N) in enumerate([(4000, 1408), (777, 1024)]):
        g = torch.Generator(device="cuda").manual_seed(call)
        x = torch.randn(rows, N, device="cuda", generator=g).to(torch.bfloat16)
        dy = torch.randn(rows, N, device="cuda", generator=g).to(torch.bfloat16)
        gamma = torch.randn(N, device="cuda", generator=g)
        beta = torch.zeros(N, device="cuda")
        _, _, mean, rstd = kx.norm_fwd(x, gamma, beta, 1e-5, False)
        outs = []
        for name in ("pf_norm_bwd", "pf_norm_bwd_static"):
            dx = torch.empty_like(x)
            dg = torch.empty(N, device="cuda")
            db = torch.empty(N, device="cuda")
            scratch = None
            if name == "pf_norm_bwd":
                ctas = L.pf_norm_bwd_ctas(ctypes.c_longlong(rows), sm)
                scratch = torch.empty(ctas * 2 * N, device="cuda")
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0]
            code = _call(L, name, scratch, dy, x, gamma, mean, rstd, dx, dg, db, rows, N, sm)
            assert code == 0, f"{name} returned {code}"
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            if name == "pf_norm_bwd_static" and call > 0:
                # the device's free memory as the driver counts it: a cudaMalloc inside the
                # entry point would show here even though torch's allocator never saw it.  The
                # first call is exempt: it may load the module image.
                assert torch.cuda.mem_get_info()[0] == free_before
            outs.append((dx, dg, db))
        (dx0, dg0, db0), (dx1, dg1, db1) = outs
        assert torch.equal(dx0, dx1)
        assert torch.allclose(dg0, dg1, rtol=1e-5, atol=1e-4)
        assert torch.allclose(db0, db1, rtol=1e-5, atol=1e-4)
    kx.check_status()


def test_static_scratch_entry_rejects_oversized_problems():
    from pfeife_b200.ops import _lib
    L = _lib.lib()
    _lib.bind_thread(torch.cuda.current_device())
    sm = _lib.sm_count()
    rows, N = 100000, 4096          # ctas * 2 * N floats is far beyond the 1 Mi built-in floats
    x = torch.zeros(8, N, device="cuda", dtype=torch.bfloat16)
    v = torch.zeros(N, device="cuda")
    code = _call(L, "pf_norm_bwd_static", None, x, x, v, v, v, x, v, v, rows, N, sm)
    assert code == -3
