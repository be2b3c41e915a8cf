"""The instruction-cost figures behind the choice of mma.sync for the 16-head attention, measured by
the library's self-test entry (one CTA on all-zero operands): a tcgen05.mma with N = 16 costs about
as much for M = 128 as for M = 64 and several times a warp-level m16n8k16 per row of work, and its
cost grows with N beyond that floor.  Ranges are wide: they pin the shape of the cost curve, not a
clock-exact value."""
import pytest
import torch

from auto_gpu_kernel_b200.run_case import measure_mma_rate

pytestmark = pytest.mark.gpu


def test_tcgen05_cost_has_a_floor_independent_of_m(cuda):
    _, m64 = measure_mma_rate(cuda, 0, 64, 16)
    _, m128 = measure_mma_rate(cuda, 0, 128, 16)
    _, wide = measure_mma_rate(cuda, 0, 128, 256)
    assert 25 < m64 < 80 and 25 < m128 < 80, (m64, m128)        # the floor: tens of cycles at N = 16
    assert abs(m128 - m64) < 0.35 * m64, (m64, m128)             # about the same for 64 and 128 rows
    assert 90 < wide < 200 and wide > 1.8 * m128, (wide, m128)   # grows with N: about N / 2 cycles


def test_fp8_scorer_shape_and_warp_level_mma(cuda):
    _, scorer = measure_mma_rate(cuda, 1, 128, 64)               # the scorer's product: M=128, N=64, K=32 e4m3
    assert 25 < scorer < 90, scorer
    _, warp8 = measure_mma_rate(cuda, 2, 8, 0, iters=2000)       # cycles per m16n8k16 per SM from 8 warps
    assert 1.0 < warp8 < 4.5, warp8
    # a 64-row attention tile: 544 warp-level products against 68 tcgen05 products
    _, t64 = measure_mma_rate(cuda, 0, 64, 16)
    assert 544 * warp8 < 68 * t64, (warp8, t64)
