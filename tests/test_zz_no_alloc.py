"""The allocation-free routing entry point (orome_cuda_moe_route_static) against the regular one.

Some callers cannot let the library allocate: the per-token loop of an engine that reserved
all of its device memory at start-up (cudaMalloc synchronises the device and can fail once
the model fills HBM), or a host whose device memory is owned by another allocator.  For
them the router logits live in a fixed 64 KiB array inside the library image.  This file is
named so that pytest collects it last: a failure here cannot hide other tests in a run that
stops at the first failure.  It must pass alone in a fresh process and after the other tests.
"""
import numpy as np
import pytest

from orome_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_routing_matches_regular_entry_point_twice():
    import torch
    from orome_b200 import format as F

    ctx = F.Context(0)
    try:
        n_experts, hidden, K = 128, 2048, 8
        W = synth.host_router(n_experts, hidden, seed=41)
        wt = torch.from_numpy(W.view(np.uint8).reshape(-1).copy()).cuda()
        router = F.tensor_ref(wt.data_ptr(), 0, synth.F32, n_experts, hidden)
        stream = torch.cuda.current_stream().cuda_stream
        # two calls in a row with different inputs and token counts: the second must not see the first's logits
        for call, T in enumerate((32, 5)):
            x = torch.from_numpy(np.atleast_2d(synth.host_x(hidden, T, seed=50 + call))).cuda()
            idx_a = torch.full((T, 8), -1, device="cuda", dtype=torch.int32)
            idx_b = torch.full((T, 8), -1, device="cuda", dtype=torch.int32)
            w_a = torch.full((T, 8), float("nan"), device="cuda")
            w_b = torch.full((T, 8), float("nan"), device="cuda")
            logits = torch.empty((T, n_experts), device="cuda")
            ctx.moe_route(router, x.data_ptr(), T, hidden, K, idx_a.data_ptr(), w_a.data_ptr(), logits.data_ptr(), stream)
            ctx.moe_route_static(router, x.data_ptr(), T, hidden, K, idx_b.data_ptr(), w_b.data_ptr(), stream)
            torch.cuda.synchronize()
            assert torch.equal(idx_a, idx_b)                                   # indices exact
            assert float((w_a - w_b).abs().max()) <= 1e-6                       # weights: the tolerance of the routing tests
            assert abs(float(w_b.sum(1).mean()) - 1.0) < 1e-5

        # beyond the fixed scratch: a clear refusal, nothing launched
        T = F.ROUTE_STATIC_MAX_LOGITS // n_experts + 1
        x = torch.zeros((T, hidden), device="cuda")
        idx = torch.zeros((T, 8), device="cuda", dtype=torch.int32)
        w = torch.zeros((T, 8), device="cuda")
        before = ctx.launch_count
        with pytest.raises(F.OromeError) as e:
            ctx.moe_route_static(router, x.data_ptr(), T, hidden, K, idx.data_ptr(), w.data_ptr(), stream)
        assert e.value.code == F.EINVAL and "exceed" in str(e.value)
        assert ctx.launch_count == before
        assert ctx.status() == 0
    finally:
        ctx.close()


def test_static_routing_allocates_no_device_memory():
    """Free device memory (cudaMemGetInfo) is the same before and after a run of static routing calls: every buffer
    the calls touch was there beforehand, the library adds none.  The regular entry point without a logits buffer
    is the contrast: its first call grows the context's scratch."""
    import torch
    from orome_b200 import format as F

    ctx = F.Context(0)
    try:
        n_experts, hidden, K, T = 128, 2048, 8, 32
        wt = torch.from_numpy(synth.host_router(n_experts, hidden, seed=43).view(np.uint8).reshape(-1).copy()).cuda()
        router = F.tensor_ref(wt.data_ptr(), 0, synth.F32, n_experts, hidden)
        x = torch.from_numpy(np.atleast_2d(synth.host_x(hidden, T, seed=60))).cuda()
        idx = torch.zeros((T, 8), device="cuda", dtype=torch.int32)
        w = torch.zeros((T, 8), device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        ctx.moe_route_static(router, x.data_ptr(), T, hidden, K, idx.data_ptr(), w.data_ptr(), stream)    # loads the kernels
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(0)[0]
        for n in (T, 5, 1, T):
            ctx.moe_route_static(router, x.data_ptr(), n, hidden, K, idx.data_ptr(), w.data_ptr(), stream)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(0)[0] == free_before
        assert ctx.status() == 0
        # contrast: the regular entry point, given no logits buffer, allocates its scratch on first use
        ctx.moe_route(router, x.data_ptr(), T, hidden, K, idx.data_ptr(), w.data_ptr(), 0, stream)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(0)[0] <= free_before
    finally:
        ctx.close()
