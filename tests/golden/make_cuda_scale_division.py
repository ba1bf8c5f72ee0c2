"""Generates tests/golden/cuda_scale_division.npz ON A CUDA DEVICE: what torch itself returns
for the reference's activation pre-scaling expression `(x / scale).to(torch.bfloat16)`
(model/quantize.py:43-44,179-183 of the reference: x a bf16 CUDA tensor, scale the 0-dim
float32 CUDA tensor clamp(amax / 2688, 1e-9)).  The CPU oracle's cuda_mode is pinned to it.

    python tests/golden/make_cuda_scale_division.py [output.npz]

Inputs: for several absmax caps, every finite bf16 value up to the cap (a few hundred thousand
values in total), so that rounding ties, subnormals and both ends of the exponent range occur.
"""
import sys
from pathlib import Path

import numpy as np
import torch


def main() -> None:
    out = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent / "cuda_scale_division.npz"
    assert torch.cuda.is_available(), "this fixture records the behaviour of torch on a CUDA device"
    allv = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    finite = torch.isfinite(allv.float())
    data = {}
    for i, cap in enumerate((64.0, 38.0, 1.0, 224.0, 3.0e38, 1.0e-30, 7.0e-37)):
        x = allv[finite & (allv.float().abs() <= cap)].cuda()
        scale = torch.clamp(x.abs().max().float() / (448.0 * 6.0), min=1e-9)
        q = (x / scale).to(torch.bfloat16)
        data[f"x{i}"] = x.cpu().view(torch.int16).numpy().view(np.uint16)
        data[f"scale{i}"] = np.float32(scale.item())
        data[f"q{i}"] = q.cpu().view(torch.int16).numpy().view(np.uint16)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 4096, generator=g).to(torch.bfloat16).cuda()
    scale = torch.clamp(x.abs().max().float() / (448.0 * 6.0), min=1e-9)
    data["x7"] = x.cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    data["scale7"] = np.float32(scale.item())
    data["q7"] = (x / scale).to(torch.bfloat16).cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    np.savez_compressed(out, **data)
    print(out, {k: (v.shape if hasattr(v, "shape") else v) for k, v in data.items()})


if __name__ == "__main__":
    main()
