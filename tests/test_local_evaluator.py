"""The packed solution directory run the way the reference's evaluator runs a solution: entry file
imported by path, `kernel` called positionally with pre-allocated outputs, checked against the
definition's reference, timed with CUDA events."""
import pytest
import torch

from auto_gpu_kernel_b200 import pack
import local_evaluator as ev

pytestmark = pytest.mark.gpu

# Shapes in the regime the reference reports for its contest workloads (batch 1..31, contexts up
# to a few thousand tokens, attention rows with tens to 2048 valid ids); values are synthetic.
INDEXER_WORKLOADS = {
    "b1_short": ([700], 1),
    "b4_mixed": ([1024, 2048, 3000, 4096], 2),
    "b8_ragged": ([5806, 12, 0, 2049, 4000, 333, 2048, 5000], 3),
    "b31": ([1500 + 137 * i for i in range(31)], 4),
}
ATTENTION_WORKLOADS = {
    "t1_few_valid": ([40], 5, 0),
    "t8_padded": ([3000] * 8, 6, 2015),
    "t16_full": ([4000 + 100 * i for i in range(16)], 7, 0),
    "t31": ([2100 + 50 * i for i in range(31)], 8, 0),
}


@pytest.fixture(scope="module")
def solution(tmp_path_factory):
    dest = tmp_path_factory.mktemp("solution")
    pack.pack(dest)
    return dest


def test_indexer_entry_under_the_local_evaluator(solution):
    kernel = ev.load_entry(solution, "indexer.py::kernel")
    results = ev.evaluate_indexer(kernel, INDEXER_WORKLOADS, torch.device("cuda", 0))
    assert [r.workload_id for r in results] == list(INDEXER_WORKLOADS)
    for r in results:
        assert r.status == "passed", (r.workload_id, r.log)
        assert r.latency_ms is not None and 0 < r.latency_ms < 5


def test_attention_entry_under_the_local_evaluator(solution):
    kernel = ev.load_entry(solution, "attention.py::kernel")
    results = ev.evaluate_attention(kernel, ATTENTION_WORKLOADS, torch.device("cuda", 0))
    for r in results:
        assert r.status == "passed", (r.workload_id, r.log, r.max_abs_error)
        assert r.latency_ms is not None and 0 < r.latency_ms < 5


def test_errors_are_recorded_not_raised(solution):
    def broken(*args):
        raise RuntimeError("boom")
    results = ev.evaluate_indexer(broken, {"w": ([100], 0)}, torch.device("cuda", 0))
    assert results[0].status == "error" and "boom" in results[0].log
