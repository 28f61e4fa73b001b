"""kronos_cuda_linear_noalloc against kronos_cuda_linear.

The no-allocation entry point serves hosts that may not call cudaMalloc while decoding (fixed memory
plan, real-time loop, memory cap): it must give exactly what the allocating entry point gives, also
when its shared static scratch still holds the previous call's activations.  Collected last on purpose
(file name), so a failure here cannot hide any other test in a stop-at-first-failure run.
"""
import numpy as np
import pytest

from k2t_rng import normal

pytestmark = pytest.mark.gpu


def test_linear_noalloc_matches_linear_on_two_calls_in_a_row(oracle):
    import torch

    import kronos_2t_b200 as k2

    ctx = k2.Context(0)
    try:
        big = oracle.bipolar_quantize_rtn(normal(1, (320, 1536), 0.02), 5)
        small = oracle.nf_quantize_rtn(normal(2, (96, 576), 0.02), 4, 2)
        d_big = ctx.upload_bipolar(big.rows, big.cols, big.planes, big.data, big.scales)
        d_small = ctx.upload_nf(small.rows, small.cols, small.bits, small.sgc, small.codebook, small.pair, small.tail)
        # first call: 6 tokens (two passes through the scratch); second call: fewer, narrower tokens,
        # so most of the scratch still holds the first call's bytes
        for mat, dm, x in ((big, d_big, normal(3, (6, 1536))), (small, d_small, normal(4, (2, 576)))):
            want = ctx.linear(dm, x)                      # allocating entry point, host buffers
            d_x = torch.from_numpy(x).cuda()
            d_out = torch.full((x.shape[0], mat.rows), float("nan"), device="cuda")
            torch.cuda.synchronize()
            ctx.linear_noalloc_dev(dm, d_x.data_ptr(), x.shape[0], d_out.data_ptr())
            ctx.synchronize()
            got = d_out.cpu().numpy()
            assert np.array_equal(got, want)              # same kernels, same order: bit-identical
            assert np.array_equal(got, oracle.gemv(mat, oracle.act_populate_fwht(x)))
        # sizes beyond the static scratch are refused with a message, not truncated
        wide_cols = 32768 + 64
        rng = np.random.Generator(np.random.PCG64(5))
        u = rng.integers(0, 16, (8, wide_cols), dtype=np.uint8)
        sc = rng.integers(0x3800, 0x3C00, (8, wide_cols // 64)).astype(np.uint16)
        wide = oracle.bipolar_from_codes(u, sc, 4)
        d_wide = ctx.upload_bipolar(wide.rows, wide.cols, 4, wide.data, wide.scales)
        d_x = torch.zeros(wide_cols, device="cuda")
        d_out = torch.zeros(8, device="cuda")
        with pytest.raises(k2.KronosCudaError, match="at most 32768"):
            ctx.linear_noalloc_dev(d_wide, d_x.data_ptr(), 1, d_out.data_ptr())
        for m in (d_big, d_small, d_wide):
            m.free()
    finally:
        ctx.close()
