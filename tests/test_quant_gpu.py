"""Bit-exact parity of the weight / dense quantisation kernels with the CPU oracle."""
import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k", [(1, 32), (130, 256), (256, 4096), (384, 3584)])
def test_quantize_w32_shared(oracle, n, k):
    from tests.gpu_util import Buf, call, dptr, stream_ptr

    w = H.config0_w(n, k, seed=n)
    w = (w.float() / (w.float().abs().max() / 2688.0)).to(torch.bfloat16)
    wd = w.cuda()
    sf = (n // 128 + 1) * 128 * k // 16
    bufs = [Buf(n * k // 2), Buf(sf), Buf(sf)]
    call("sharq_quantize_w32_shared", dptr(wd), n, k, *[b.ptr for b in bufs], stream_ptr())
    got = [b.get() for b in bufs]
    want = oracle.quantize_w32_shared(H.bits(w))
    for name, g, wv in zip(("qw", "sfw_sparse", "sfw_dense"), got, want):
        assert np.array_equal(g, np.asarray(wv).reshape(-1)), name
    # duplicate op reproduces the dense view from the sparse one
    dup = Buf(sf)
    call("sharq_duplicate_sfa32_to_sfa16", bufs[1].ptr, n, 64, k, dup.ptr, stream_ptr())
    assert np.array_equal(dup.get(), want[2])


@pytest.mark.parametrize("rows,k", [(1, 16), (33, 128), (130, 2048), (64, 14336), (16, 3584)])
def test_quantize_dense_nvfp4(oracle, rows, k):
    from tests.gpu_util import Buf, SENTINEL, call, dptr, stream_ptr

    x = H.config0_x(rows, k, seed=rows + 1)
    x = (x.float() / (x.float().abs().max() / 2688.0)).to(torch.bfloat16)
    xd = x.cuda()
    sf = (rows // 128 + 1) * 128 * k // 16
    bufs = [Buf(rows * k // 2), Buf(sf)]
    call("sharq_quantize_nvfp4", dptr(xd), rows, k, *[b.ptr for b in bufs], stream_ptr())
    q, s = [b.get() for b in bufs]
    wq, ws = oracle.quantize_dense_nvfp4(H.bits(x), fill=SENTINEL)  # unwritten bytes stay as they were
    assert np.array_equal(q, wq.reshape(-1))
    assert np.array_equal(s, ws)


def test_compress_sparse_a(oracle):
    from tests.gpu_util import Buf, call, dptr, stream_ptr

    m, k, n = 70, 512, 128
    x = H.outlier_rich_x(m, k, 11)
    dense = oracle.prepare(H.bits(x), debug=True)[0]
    # add corner cases: empty chunks, single survivors at each position, minus zeros
    dense[0, :8] = 0
    dense[1, :4] = [0, 0, 0, 0x23]
    dense[1, 4:8] = [0, 0x51, 0, 0]
    dense[2, :4] = [0x88, 0x08, 0x33, 0x80]
    dd = torch.from_numpy(dense).cuda()
    bufs = [Buf(m * k // 4), Buf(((m + 127) // 128 * 128) * k // 16)]
    call("sharq_compress_sparse_a", dptr(dd), m, n, k, *[b.ptr for b in bufs], stream_ptr())
    got = [b.get() for b in bufs]
    want = oracle.compress_sparse_a(dense)
    assert np.array_equal(got[0], want[0])
    assert np.array_equal(got[1], want[1])
