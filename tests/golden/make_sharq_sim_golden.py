"""Generates tests/golden/sharq_sim_*.npz by importing the reference's SHARQ_SIM path.

Run in the build container, where the reference checkout is mounted:

    python tests/golden/make_sharq_sim_golden.py /path/to/reference

It imports model/qLinearLayer.py and model/quantize.py of the reference unmodified
(via sys.path, not as a package), runs QLinearLayer(quant_type="SHARQ_SIM") on small
seeded inputs on CPU and stores inputs and every intermediate as raw bf16 bit patterns.
The tests read only the committed .npz files.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

CASES = {
    # name: (M, K, N, with_bias, with_rmsnorm, seed)
    "small": (8, 256, 128, False, False, 0),
    "bias": (16, 256, 64, True, False, 1),
    "rmsnorm": (32, 512, 128, False, True, 2),
    "outlier": (24, 384, 96, True, True, 3),
}


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy().copy()


def make_inputs(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    cols = torch.randperm(k, generator=g)[: max(1, k // 100)]
    x[:, cols] *= 20.0
    w = torch.randn(n, k, generator=g) * 0.02
    b = torch.randn(n, generator=g) * 0.1
    gamma = 1.0 + torch.randn(k, generator=g) * 0.1
    return x.to(torch.bfloat16), w.to(torch.bfloat16), b.to(torch.bfloat16), gamma.to(torch.bfloat16)


def main() -> None:
    import os

    default = os.environ.get("SHARQ_REFERENCE_DIR") or str(Path(__file__).resolve().parents[3] / "reference")
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else default)
    sys.path.insert(0, str(ref / "model"))
    from qLinearLayer import QLinearLayer  # noqa: E402  (the reference's own module)
    import quantize as refq  # noqa: E402

    out_dir = Path(__file__).resolve().parent
    torch.set_num_threads(1)
    for name, (m, k, n, with_bias, with_norm, seed) in CASES.items():
        x, w, b, gamma = make_inputs(m, k, n, seed)
        lin = torch.nn.Linear(k, n, bias=with_bias, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(w)
            if with_bias:
                lin.bias.copy_(b)
        layer = QLinearLayer(lin, quant_type="SHARQ_SIM")
        eps = 1e-6
        if with_norm:
            prepared = layer.prepare_input_rmsnorm(x, gamma, eps)
            x_norm = refq.apply_rmsnorm(x, gamma, eps)
        else:
            prepared = layer.prepare_input(x)
            x_norm = x
        y = layer.apply_prepared(prepared)
        _, main_q, res_q, scale_x = prepared
        np.savez_compressed(
            out_dir / f"sharq_sim_{name}.npz",
            x=bits(x), w=bits(w), bias=bits(b), gamma=bits(gamma),
            with_bias=np.array(with_bias), with_norm=np.array(with_norm), eps=np.float32(eps),
            x_norm=bits(x_norm), main_q=bits(main_q), res_q=bits(res_q),
            scale_x=np.float32(scale_x.item()), w_q=bits(layer.weight_sim_q32),
            scale_w=np.float32(layer.weight_scale.item()), y=bits(y),
        )
        print(name, "y abs mean", y.float().abs().mean().item(), file=sys.stderr)


if __name__ == "__main__":
    main()
