"""Generates tests/golden/converter_tables.npz.

The reference's kernels convert with cutlass::NumericConverter<..., round_to_nearest>
(kernels/src/fused_sparse_prepare.cu:113-116).  CUTLASS is an un-vendored submodule of
the reference, so its published host implementation of those converters is compiled
here (CUTLASS 4.5.0 headers shipped inside the flashinfer wheel, host code path, no GPU)
and run on a probe set of floats.  The resulting tables pin the oracle's scalar
converters.  Run once in the build container:

    python tests/golden/make_converter_tables.py

Needs nvcc and the CUTLASS headers; the tests only read the committed .npz.
"""
from __future__ import annotations

import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

PROBE = r"""
#include <cstdio>
#include <cstdint>
#include <cstring>
#include "cutlass/numeric_conversion.h"
#include "cutlass/float_subbyte.h"
#include "cutlass/float8.h"
#include "cutlass/bfloat16.h"
int main() {
  cutlass::NumericConverter<cutlass::float_e2m1_t, float, cutlass::FloatRoundStyle::round_to_nearest> to_fp4;
  cutlass::NumericConverter<cutlass::float_ue4m3_t, float, cutlass::FloatRoundStyle::round_to_nearest> to_sf;
  cutlass::NumericConverter<cutlass::bfloat16_t, float, cutlass::FloatRoundStyle::round_to_nearest> to_bf;
  cutlass::NumericConverter<float, cutlass::float_e2m1_t, cutlass::FloatRoundStyle::round_to_nearest> fp4_to_f;
  cutlass::NumericConverter<float, cutlass::float_ue4m3_t, cutlass::FloatRoundStyle::round_to_nearest> sf_to_f;
  float v;
  while (fread(&v, 4, 1, stdin) == 1) {
    auto a = to_fp4(v); auto b = to_sf(v); auto c = to_bf(v);
    uint8_t ab = a.storage & 0xF; uint8_t bb = b.storage; uint16_t cb; memcpy(&cb, &c, 2);
    float af = fp4_to_f(a), bf = sf_to_f(b);
    fwrite(&ab,1,1,stdout); fwrite(&bb,1,1,stdout); fwrite(&cb,2,1,stdout);
    fwrite(&af,4,1,stdout); fwrite(&bf,4,1,stdout);
  }
  return 0;
}
"""


def find_cutlass() -> Path:
    import flashinfer  # noqa: F401  (only to locate the vendored headers)

    inc = Path(flashinfer.__file__).parent / "data" / "cutlass" / "include"
    if not (inc / "cutlass" / "numeric_conversion.h").exists():
        raise SystemExit("CUTLASS headers not found")
    return inc


def probe_values() -> np.ndarray:
    rng = np.random.default_rng(0)
    vals = []
    # e2m1: every rounding boundary and representable value, +-1/2 ulp neighbours, both signs
    e2m1_pts = [0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, 7.0, 100.0]
    for p in e2m1_pts:
        f = np.float32(p)
        for s in (1.0, -1.0):
            v = np.float32(s) * f
            vals += [v, np.nextafter(v, np.float32(np.inf)), np.nextafter(v, np.float32(-np.inf))]
    vals += list(rng.uniform(-6.5, 6.5, 4000).astype(np.float32))
    # ue4m3: every code value, every midpoint between adjacent codes, and neighbours
    codes = []
    for c in range(0x7F):
        e, m = c >> 3, c & 7
        codes.append(m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))
    codes = np.array(codes, np.float64)
    mids = (codes[1:] + codes[:-1]) / 2
    for p in np.concatenate([codes, mids, [460.0, 1000.0]]):
        v = np.float32(p)
        vals += [v, np.nextafter(v, np.float32(np.inf)), np.nextafter(v, np.float32(0))]
    vals += list(np.exp(rng.uniform(np.log(2.0 ** -9), np.log(448.0), 4000)).astype(np.float32))
    # bf16: random values plus exact ties
    r = rng.standard_normal(4000).astype(np.float32) * 5
    vals += list(r)
    ties = (r.view(np.uint32) & 0xFFFF0000 | 0x8000).view(np.float32)
    vals += list(ties)
    return np.array(vals, np.float32)


def main() -> None:
    inc = find_cutlass()
    out = Path(__file__).resolve().parent / "converter_tables.npz"
    vals = probe_values()
    with tempfile.TemporaryDirectory() as td:
        src = Path(td) / "probe.cu"
        src.write_text(PROBE)
        exe = Path(td) / "probe"
        subprocess.run(["nvcc", "-std=c++17", "-O1", "-Wno-deprecated-gpu-targets", f"-I{inc}", str(src), "-o", str(exe)],
                       check=True)
        res = subprocess.run([str(exe)], input=vals.tobytes(), stdout=subprocess.PIPE, check=True).stdout
    rec = np.frombuffer(res, dtype=np.dtype([("e2m1", "u1"), ("ue4m3", "u1"), ("bf16", "<u2"),
                                             ("e2m1_f", "<f4"), ("ue4m3_f", "<f4")]))
    assert rec.shape[0] == vals.shape[0]
    np.savez_compressed(out, values=vals, e2m1=rec["e2m1"], ue4m3=rec["ue4m3"], bf16=rec["bf16"],
                        e2m1_back=rec["e2m1_f"], ue4m3_back=rec["ue4m3_f"],
                        cutlass_version=np.array("4.5.0 (flashinfer wheel)"))
    print(f"wrote {out} with {vals.shape[0]} probes", file=sys.stderr)


if __name__ == "__main__":
    main()
