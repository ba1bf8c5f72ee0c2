"""sharq_b200: B200 (sm_100a) kernels for the SharQ quantized-linear hot path.

`sharq_b200.ops` exposes the reference's `sharq_ops` operator names on top of the
C ABI in include/sharq_b200.h; `sharq_b200.quantize` and `sharq_b200.qlinear` mirror
the reference's host-side helpers and its QLinearLayer.
"""
__version__ = "0.1.0"
