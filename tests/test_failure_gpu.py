"""Failure detection on the device without faulting it: a cross-GPU wait that nobody answers
must run out within its limit, leave an error code for the host, and leave the context usable.

The all-reduce kernel is launched for rank 0 of a two-rank group whose second rank does not
exist: both ranks' data and flag pointers are ordinary buffers of this one GPU (no multicast
object, no peer mapping), and nothing ever signals for the absent rank."""
import ctypes

import pytest
import torch

from sharq_b200 import _lib
from tests.gpu_util import call, dptr, stream_ptr

pytestmark = pytest.mark.gpu


def test_all_reduce_wait_runs_out_and_reports():
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    nbytes = 64 * 1024
    flag_bytes = int(lib.sharq_allreduce_flag_bytes())
    data = [torch.ones(nbytes // 2, dtype=torch.bfloat16, device=dev) * (r + 1) for r in range(2)]
    flags = [torch.zeros(flag_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    call("sharq_set_wait_limit_cycles", 2_000_000)  # about a millisecond per wait
    try:
        data_ptrs = (ctypes.c_void_p * 2)(data[0].data_ptr(), data[1].data_ptr())
        flag_ptrs = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call("sharq_allreduce_bf16_peer", data_ptrs, flag_ptrs, 0, 2, nbytes, 0, dptr(err), stream_ptr())
        e1.record()
        torch.cuda.synchronize()  # returns: the kernel gave up instead of spinning on
        assert e0.elapsed_time(e1) < 500.0
        assert int(err.item()) in (0x201, 0x202), hex(int(err.item()))  # one of the two barriers of the peer-copy kernel
    finally:
        call("sharq_set_wait_limit_cycles", 0)
    # the context is still usable: a complete single-rank group works and reports nothing
    err.zero_()
    fresh = torch.zeros(flag_bytes, dtype=torch.uint8, device=dev)
    solo = torch.full((nbytes // 2,), 3.0, dtype=torch.bfloat16, device=dev)
    call("sharq_allreduce_bf16_peer", (ctypes.c_void_p * 1)(solo.data_ptr()), (ctypes.c_void_p * 1)(fresh.data_ptr()), 0, 1,
         nbytes, 0, dptr(err), stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert bool((solo == 3.0).all())
