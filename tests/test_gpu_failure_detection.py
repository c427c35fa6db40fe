"""Failure detection without a GPU fault: a rank that never joins is noticed by the bounded wait of the peer barrier.

The barrier kernel stores its epoch into every rank's flag array and waits (about a second and a half at most) until
all slots of its own array have reached the epoch.  Here a second "rank" exists only as a flag slot that nothing ever
sets: the wait runs out, the kernel records the time-out in the context's status word and returns, the host reads it
through ``xfold_check_status`` as an error, and the context stays usable for the next call.  Nothing is trapped,
faulted or left spinning."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_barrier_times_out_on_a_missing_rank(ops, pkg):
    from distributed_xfold_b200 import peer_ops
    from distributed_xfold_b200._cabi import XfoldError
    flags_me = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags_absent = torch.zeros(8, dtype=torch.int32, device="cuda")
    ops.synchronize_and_check()
    t0 = time.time()
    peer_ops.peer_barrier([flags_me.data_ptr(), flags_absent.data_ptr()], 0, 2, 1, "cuda:0")
    with pytest.raises(XfoldError) as err:
        ops.synchronize_and_check()
    dt = time.time() - t0
    assert "wait ran out" in str(err.value)
    assert 0.3 < dt < 10.0, dt                       # bounded: it neither returns at once nor hangs
    assert flags_me.cpu().tolist()[:2] == [1, 0]     # this rank signalled; the absent one never did
    assert flags_absent.cpu().tolist()[0] == 1
    # the status word is cleared by the read and the context keeps working
    ops.synchronize_and_check()
    x = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
    y = ops.layernorm(x, None, None)
    ops.synchronize_and_check()
    ref = torch.nn.functional.layer_norm(x.float(), (128,))
    assert float((y.float() - ref).abs().max()) < 5e-2


def test_peer_barrier_completes_when_every_rank_arrives(ops, pkg):
    """Two ranks emulated by two flag arrays on one GPU, arriving one after the other in ONE stream would wait on each
    other; so the second rank's arrival is written by the host first, and the kernel only has to observe it."""
    from distributed_xfold_b200 import peer_ops
    flags_me = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags_other = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags_me[1] = 1                                    # "rank 1 has arrived at epoch 1"
    torch.cuda.synchronize()
    t0 = time.time()
    peer_ops.peer_barrier([flags_me.data_ptr(), flags_other.data_ptr()], 0, 2, 1, "cuda:0")
    ops.synchronize_and_check()
    assert time.time() - t0 < 1.0
    assert flags_other.cpu().tolist()[0] == 1
