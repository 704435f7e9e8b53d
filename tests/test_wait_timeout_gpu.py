"""A bounded wait that actually runs out, without faulting or hanging anything: the all-reduce
kernel is given a second "rank" whose workspace is an ordinary local buffer that nobody ever
writes a flag into, and a wait limit of 50 ms.  The kernel must return by itself, the status word
must say that a wait gave up, the output must be untouched, and the next ordinary call on the
same context must work."""
import ctypes
import time

import pytest
import torch

from relax_b200 import _lib

pytestmark = pytest.mark.gpu


def test_allreduce_wait_runs_out_and_the_context_survives():
    lib = _lib.load()
    count, max_count = 4096, 4096
    nbytes = lib.rb200_allreduce_workspace_bytes(max_count)
    own = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    absent_peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")  # its flags stay zero for good
    ws2 = (ctypes.c_void_p * 2)(own.data_ptr(), absent_peer.data_ptr())
    inp = torch.randn(count, device="cuda").half()
    out = torch.full((count,), 7.0, dtype=torch.float16, device="cuda")
    st = ctypes.c_int(0)
    assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0 and st.value == 0
    _lib.check(lib.rb200_set_wait_limit_ms(50))
    try:
        t0 = time.perf_counter()
        _lib.check(lib.rb200_allreduce_oneshot(ws2, 0, 2, ctypes.c_void_p(inp.data_ptr()),
                                               ctypes.c_void_p(out.data_ptr()), count, max_count, None))
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert waited < 1.5, "the wait was not bounded by the limit (%.2f s)" % waited
        assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0
        assert st.value == 1, "expected the wait-timeout status, got %d" % st.value
        assert torch.all(out == 7.0), "a call whose wait gave up must leave its output unwritten"
        # reading the status cleared it
        assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0 and st.value == 0
    finally:
        _lib.check(lib.rb200_set_wait_limit_ms(0))
    # the context is intact: an ordinary single-rank call on the same workspace gives the input back
    ws1 = (ctypes.c_void_p * 1)(own.data_ptr())
    _lib.check(lib.rb200_allreduce_oneshot(ws1, 0, 1, ctypes.c_void_p(inp.data_ptr()),
                                           ctypes.c_void_p(out.data_ptr()), count, max_count, None))
    torch.cuda.synchronize()
    assert torch.equal(out, inp)
    assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0 and st.value == 0
