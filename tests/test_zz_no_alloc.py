"""The allocation-free GEMM entry point against the regular one.

Collected last on purpose: a run that stops at the first failure has already run every other
test by the time it gets here.  The entry point exists for callers that cannot reach the CUDA
allocator in the middle of a step: a host runtime whose own pool already owns the free device
memory, or a loop with overlapped compute and collective streams that an allocator call could
stall.  Its split-K partial sums live in a fixed 32 MiB array inside the library.
"""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu


def _case(rng, m, n, k):
    a = ho.bf16_round(rng.standard_normal((m, k)))
    b = ho.bf16_round(rng.standard_normal((k, n)))
    # both operands stored contraction-major-last, as a weight gradient sees them
    return a, b, dev(a.T.copy(), torch.bfloat16), dev(b.copy(), torch.bfloat16)


def test_static_scratch_gemm_matches_the_allocating_entry_point_twice_in_a_row():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(21)
    # the second call is smaller, so stale partial sums of the first one sit right behind its own
    for m, n, k, split in ((384, 520, 4096, 4), (256, 264, 2048, 0)):
        a, b, da, db = _case(rng, m, n, k)
        want = cuda.gemm_bf16(c, da, db, m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR, out_dtype=torch.float32, split_k=split)
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        c.sync()
        before = c.counters()
        got = cuda.gemm_bf16_static_scratch(c, da, db, out, m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR, split_k=split)
        after = c.counters()
        # the one promise of the entry point: the library allocated nothing on the way
        assert (after.allocations, after.allocated_bytes) == (before.allocations, before.allocated_bytes)
        assert_close("static scratch vs regular", host(got), host(want), atol=1e-2, rtol=1e-5)
        assert_close("static scratch vs oracle", host(got), a @ b, atol=1e-2, rtol=1e-5)


def test_static_scratch_gemm_with_dealt_k_blocks_twice_in_a_row():
    """80 output tiles with a contraction of 12288 on 148 SMs: the automatic work split deals the tiles' k blocks out
    over the CTAs, the only path that uses the per-CTA slots and the flag array of the fixed scratch.  The second call
    finds the first one's slots and flags in place."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(22)
    m, n, k = 1280, 2048, 12288
    splits, dealt, need = cuda.gemm_bf16_plan(c, m, n, k)
    assert dealt > 0 and 0 < need <= (32 << 20)
    for _ in range(2):
        a, b, da, db = _case(rng, m, n, k)
        want = cuda.gemm_bf16(c, da, db, m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR, out_dtype=torch.float32, split_k=0)
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        c.sync()
        before = c.counters()
        got = cuda.gemm_bf16_static_scratch(c, da, db, out, m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR, split_k=0)
        after = c.counters()
        assert (after.allocations, after.allocated_bytes) == (before.allocations, before.allocated_bytes)
        assert np.array_equal(host(got), host(want))  # same kernel, same split, same summation order
        assert_close("static scratch vs oracle", host(got), a @ b, atol=2e-2, rtol=1e-5)


def test_static_scratch_gemm_rejects_shapes_beyond_its_fixed_array():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    m, n, k = 2048, 2048, 4096  # 4 splits x 2048 x 2048 x 4 bytes = 64 MiB > 32 MiB
    a = c.zeros((k, m), torch.bfloat16)
    b = c.zeros((k, n), torch.bfloat16)
    out = c.zeros((m, n), torch.float32)
    with pytest.raises(HeirloomError, match="more than the fixed"):
        cuda.gemm_bf16_static_scratch(c, a, b, out, m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR, split_k=4)
