"""The reference's UNMODIFIED Python host code running on this project's kernels.

oracle/build_ref.py --stage-python copies the reference's loader, its QLinearLayer, its
quantize glue and its matrix-suite correctness script into the git-ignored oracle/_ref/py/
(nothing of it is in the repository).  Here SHARQ_KERNEL_BUILD points the reference's loader at
sharq_b200/dropin, so `load_sharq_ops()` imports this project's `sharq_ops` module, and

  * the reference's QLinearLayer (model/qLinearLayer.py:21-202) in SHARQ and NVFP4 mode must give,
    bit for bit, the output of sharq_b200.qlinear.QLinearLayer with the reference's two-launch
    GEMM composition (fused_gemm=False) - which runs the scaling, statistics and prepare inside
    one kernel where the reference uses ATen passes;
  * the invariants of benchmarks/correctness/example_fused_pairtop2_matrix_suite.py:169-208 hold
    on its own input families: at most two non-zero bytes per four in the sparse payload, the sparse
    GEMM equals the dense GEMM on the decoded payload, kernel results track its pseudo-quantised
    model.
The tests skip when the staging is absent."""
import contextlib
import importlib
import io
import os
import re
import sys
from pathlib import Path

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
STAGE = ROOT / "oracle" / "_ref" / "py"


@pytest.fixture(scope="module")
def ref_modules():
    if not (STAGE / "model" / "qLinearLayer.py").exists():
        pytest.skip("oracle/_ref/py not staged (python oracle/build_ref.py --stage-python)")
    os.environ["SHARQ_KERNEL_BUILD"] = str(ROOT / "sharq_b200" / "dropin")
    for p in (STAGE / "model", STAGE / "benchmarks" / "correctness"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    qll = importlib.import_module("qLinearLayer")
    suite = importlib.import_module("example_fused_pairtop2_matrix_suite")
    ops_mod = importlib.import_module("quantize").load_sharq_ops()
    assert Path(ops_mod.__file__).resolve() == (ROOT / "sharq_b200" / "dropin" / "sharq_ops.py").resolve()
    return qll, suite


def _linear(n, k, bias, seed):
    lin = torch.nn.Linear(k, n, bias=bias, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(H.config0_w(n, k, seed))
        if bias:
            lin.bias.copy_((0.1 * torch.randn(n, generator=torch.Generator().manual_seed(seed))).to(torch.bfloat16))
    return lin


@pytest.mark.parametrize("quant_type", ["SHARQ", "NVFP4"])
@pytest.mark.parametrize("m,n,k,bias", [(64, 256, 512, True), (300, 384, 1024, False), (2048, 4096, 4096, False)])
def test_reference_qlinear_runs_on_the_dropin_bit_exact(ref_modules, quant_type, m, n, k, bias):
    from sharq_b200.qlinear import QLinearLayer

    qll, _ = ref_modules
    lin = _linear(n, k, bias, m)
    theirs = qll.QLinearLayer(lin, quant_type=quant_type)
    mine = QLinearLayer(lin, quant_type=quant_type, fused_gemm=False)
    x = H.config0_x(m, k, m + 1).cuda()
    y_ref = theirs(x)
    y = mine(x)
    torch.cuda.synchronize()
    assert y_ref.dtype == torch.bfloat16 and tuple(y_ref.shape) == (m, n)
    assert torch.equal(y, y_ref), float((y.float() - y_ref.float()).abs().max())
    if quant_type == "SHARQ":
        gamma = H.config0_gamma(k, 3).cuda()
        y_ref = theirs.apply_prepared(theirs.prepare_input_rmsnorm(x, gamma, 1e-6))
        y = mine.apply_prepared(mine.prepare_input_rmsnorm(x, gamma, 1e-6))
        assert torch.equal(y, y_ref)
        # the single-launch GEMM of this project stays within the GEMM tolerance of the reference composition
        fused = QLinearLayer(lin, quant_type="SHARQ", fused_gemm=True)
        y_fused = fused.apply_prepared(fused.prepare_input_rmsnorm(x, gamma, 1e-6))
        rel = float((y_fused.float() - y_ref.float()).norm() / y_ref.float().norm())
        assert rel <= 1e-2, rel


def test_reference_matrix_suite_invariants(ref_modules):
    """Runs the reference script's own run_case on its own input families and checks the numbers it prints."""
    _, suite = ref_modules
    dev = torch.device("cuda")
    torch.manual_seed(0)
    torch.cuda.manual_seed_all(0)
    backend = suite.load_sharq_ops()
    m, n, k = 8, 1024, 1024
    cases = [
        ("zero x eye", suite.make_zero_x(m, k, dev), suite.make_eye_w(n, k, dev)),
        ("ones x ones", suite.make_one_x(m, k, dev), suite.make_ones_w(n, k, dev)),
        ("pair-friendly x random_w", suite.make_pair_friendly_x(m, k, dev), suite.make_random_w(n, k, dev)),
        ("alternating-pair x block-repeat_w", suite.make_alternating_pair_x(m, k, dev), suite.make_block_repeat_w(n, k, dev)),
        ("outlier-rich x random_w", suite.make_outlier_rich_x(m, k, dev), suite.make_random_w(n, k, dev)),
    ]
    for name, x, w in cases:
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            suite.run_case(name, x, w, backend)
        text = buf.getvalue()
        viol = float(re.search(r"raw-byte violation\s*:\s*([0-9.eE+-]+)", text).group(1))
        assert viol == 0.0, (name, viol)

        def rel_rmse(title):
            block = text[text.index(title):]
            return float(re.search(r"rel_rmse\s*:\s*([0-9.eE+-]+|nan)", block).group(1))

        # the sparse GEMM on (A_comp, E) and the dense GEMM on the decoded payload see the same numbers
        dd = rel_rmse("sparse_gemm vs dense_decode")
        assert dd != dd or dd <= 1e-2, (name, dd)  # nan only for the all-zero case (0 / 0)
        if name != "zero x eye":
            assert rel_rmse("kernel_total vs pseudo_total") <= 0.08, (name, text)
