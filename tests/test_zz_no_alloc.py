"""The Transition entry point that needs no caller workspace (``xfold_transition_static_fwd``).

Some hosts of this library are given device buffers for inputs and outputs but are not allowed to
allocate device memory of their own: a plugin living inside another runtime's arena, or a serving
path where allocation is off limits.  For them the library keeps the Transition's scratch in a
fixed array of its own.  This test calls that entry point through the C ABI twice in a row (the
second call finds the first call's leftovers in the shared scratch) and requires the results to be
identical to the regular entry point, which runs the same kernels on a caller workspace; it also
checks that a request beyond the array's size is refused with a clear message instead of running.
The file name sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _call_static(ops, cabi, x, w):
    dev = x.device.index or 0
    rc = cabi.load().xfold_transition_static_fwd(cabi.ctx(dev), x.data_ptr(), x.numel() // w.C, w.C, w.F, C.byref(w.c),
                                                 torch.cuda.current_stream(dev).cuda_stream)
    return rc


@pytest.mark.parametrize("rows,c", [((40, 37), 128), ((1000,), 384)])
def test_static_scratch_transition_matches_workspace_version(ops, oracle, rows, c):
    from distributed_xfold_b200 import _cabi
    g = torch.Generator().manual_seed(77 + c)
    st = oracle.make_transition_state(g, "", c)
    w = ops.PackedTransition(st, "", "cuda")
    for call in range(2):  # two calls in a row: the second one starts from a dirty shared scratch
        x = (torch.randn(*rows, c, generator=g) * (1 + call)).to(BF)
        ref = x.cuda().contiguous()
        ops.transition_(ref, w)                       # existing entry point, caller workspace
        got = x.cuda().contiguous()
        assert _call_static(ops, _cabi, got, w) == 0, _cabi.load().xfold_last_error(_cabi.ctx(0))
        ops.synchronize_and_check()
        assert torch.equal(got, ref)                  # same kernels, same inputs: bit-identical
        # and right, not merely equal: against the CPU oracle within the bf16 tolerance of the other tests
        want = x.float() + oracle.transition({k: v.to(BF).float() for k, v in st.items()}, "", x.float())
        err = float((got.float().cpu() - want).norm() / want.norm())
        assert err < 2e-2


def test_static_scratch_rejects_oversize(ops, oracle):
    from distributed_xfold_b200 import _cabi
    lib = _cabi.load()
    g = torch.Generator().manual_seed(3)
    w = ops.PackedTransition(oracle.make_transition_state(g, "", 128), "", "cuda")
    limit = lib.xfold_transition_static_max_bytes()
    rows = limit // (2 * (128 + 512)) + 4096          # scratch need clearly above the limit
    assert lib.xfold_transition_workspace_bytes(rows, 128, 512) > limit
    x = torch.zeros(8, 128, dtype=BF, device="cuda")  # never touched: the call must be refused before any launch
    rc = lib.xfold_transition_static_fwd(_cabi.ctx(0), x.data_ptr(), rows, 128, 512, C.byref(w.c),
                                         torch.cuda.current_stream(0).cuda_stream)
    assert rc == _cabi.XFOLD_ERR_ARG
    msg = lib.xfold_last_error(_cabi.ctx(0)).decode()
    assert "static scratch" in msg and "workspace" in msg


@pytest.mark.parametrize("c,f,last_ok", [(128, 512, 13105), (384, 1536, 4368)])
def test_static_scratch_edge_of_limit(ops, oracle, c, f, last_ok):
    """The documented capacity is exact: `last_ok` rows run (and match the workspace version), one row more is refused."""
    from distributed_xfold_b200 import _cabi
    lib = _cabi.load()
    limit = lib.xfold_transition_static_max_bytes()
    assert lib.xfold_transition_workspace_bytes(last_ok, c, f) <= limit < lib.xfold_transition_workspace_bytes(last_ok + 1, c, f)
    g = torch.Generator().manual_seed(5 + c)
    w = ops.PackedTransition(oracle.make_transition_state(g, "", c), "", "cuda")
    x = torch.randn(last_ok + 1, c, generator=g).to(BF)
    ref = x[:last_ok].cuda().contiguous()
    ops.transition_(ref, w)
    got = x.cuda().contiguous()
    st = torch.cuda.current_stream(0).cuda_stream
    assert lib.xfold_transition_static_fwd(_cabi.ctx(0), got.data_ptr(), last_ok, c, f, C.byref(w.c), st) == 0
    ops.synchronize_and_check()
    assert torch.equal(got[:last_ok], ref) and torch.equal(got[last_ok], x[last_ok].cuda())   # the extra row is untouched
    assert lib.xfold_transition_static_fwd(_cabi.ctx(0), got.data_ptr(), last_ok + 1, c, f, C.byref(w.c), st) == _cabi.XFOLD_ERR_ARG
    # a row count whose byte size would wrap around is refused as well, before any launch
    assert lib.xfold_transition_static_fwd(_cabi.ctx(0), got.data_ptr(), 1 << 62, c, f, C.byref(w.c), st) == _cabi.XFOLD_ERR_ARG
    ops.synchronize_and_check()
