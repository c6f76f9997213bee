"""A bounded device wait that nobody answers: it gives up by design, reports through the status word, and the
context stays usable.  (The wait RETURNS after its clock budget - no fault, no hang.)"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_barrier_gives_up_and_reports():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from chitudiffusion_b200 import _lib, ops

    dev = torch.device("cuda", torch.cuda.current_device())
    # two "ranks" whose flag arrays both live on this GPU; rank 1 never enqueues its side of the barrier
    flags = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(2)]
    old = ops.set_flag_wait_cycles(2_000_000)  # about a millisecond instead of a second
    try:
        assert ops.set_flag_wait_cycles(0) == 2_000_000  # query form
        torch.cuda.synchronize()
        ops.peer_barrier([f.data_ptr() for f in flags], rank=0, world=2, device=dev)
        torch.cuda.synchronize()  # returns: the wait ran out
        assert int(ops.status_word(dev).item()) == 5
        # rank 0 did post its own arrival to "rank 1" before it started waiting
        assert int(flags[1][0].item()) == 1
        with pytest.raises(_lib.ChituB200Error, match="flag wait"):
            ops.check_status(dev)
        ops.check_status(dev)  # the word was cleared by the raise
        # the deferred form used on the product path: the poll after the failing launch enqueues a copy of
        # the word, a later poll sees it
        ops.peer_barrier([f.data_ptr() for f in flags], rank=0, world=2, device=dev)
        ops.poll_status(dev)
        torch.cuda.synchronize()
        with pytest.raises(_lib.ChituB200Error, match="flag wait"):
            ops.poll_status(dev)
        torch.cuda.synchronize()
        ops.check_status(dev)
        # a barrier that IS answered (one rank) still passes and the device still computes
        solo = torch.zeros(2, dtype=torch.int32, device=dev)
        ops.peer_barrier([solo.data_ptr()], rank=0, world=1, device=dev)
        torch.cuda.synchronize()
        ops.check_status(dev)
        assert float((torch.ones(8, device=dev) * 2).sum().item()) == 16.0
    finally:
        ops.set_flag_wait_cycles(old)
