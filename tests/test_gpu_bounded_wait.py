"""A device-side wait that runs out: the kernel returns, the status word says so, the context
lives on.  Uses the library's self-test entry (one thread, a barrier nothing arrives on, a limit of
a millisecond) -- nothing faults, traps or spins past the limit."""
import pytest
import torch

from auto_gpu_kernel_b200 import _lib, indexer, inputs as wl, workspace

pytestmark = pytest.mark.gpu

WAIT_TIMEOUT = 0x1


def test_expired_wait_sets_status_and_returns(cuda):
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    waited = torch.zeros(1, dtype=torch.int64, device=cuda)
    limit_ns = 1_000_000
    with torch.cuda.device(cuda):
        rc = lib.dsa_selftest_wait_expiry(limit_ns, status.data_ptr(), waited.data_ptr(),
                                          torch.cuda.current_stream(cuda).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(cuda)
    assert int(status.item()) == WAIT_TIMEOUT
    assert limit_ns <= int(waited.item()) < 50 * limit_ns      # gave up soon after the limit
    # the shim turns the bit into an error, once
    word = workspace.status_word(cuda)
    word.copy_(status)
    with pytest.raises(RuntimeError, match="wait timed out"):
        workspace.check_status(cuda)
    assert workspace.check_status(cuda) == 0
    # and the context is as usable as before
    inp = wl.make_indexer_inputs([3000, 100], seed=1, device=cuda)
    out = indexer.run(*inp.args())
    workspace.check_status(cuda)
    assert int((out[0] >= 0).sum()) == 2048 and int((out[1] >= 0).sum()) == 100


def test_selftest_rejects_limits_beyond_a_second(cuda):
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    assert lib.dsa_selftest_wait_expiry(2_000_000_000, status.data_ptr(), None, None) == -2
    assert lib.dsa_selftest_wait_expiry(0, status.data_ptr(), None, None) == -2
    assert lib.dsa_selftest_wait_expiry(1000, None, None, None) == -1
