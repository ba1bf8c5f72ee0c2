"""CPU checks of the oracle itself: converter tables from the CUTLASS host converters,
SHARQ_SIM golden vectors produced by the imported reference, layout/size facts, and the
invariants the reference's correctness scripts print."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import sharq_sim
from tests import helpers as H

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_converters_match_cutlass_tables(oracle):
    d = np.load(GOLDEN / "converter_tables.npz")
    v = d["values"]
    L = oracle.lib()
    e2m1 = np.array([L.sharq_f32_to_e2m1(float(x)) for x in v], np.uint8)
    assert np.array_equal(e2m1, d["e2m1"])
    in_range = (v >= 2.0 ** -9) & (v <= 448.0)  # callers clamp to this range first
    ue = np.array([L.sharq_f32_to_ue4m3(float(x)) for x in v[in_range]], np.uint8)
    assert np.array_equal(ue, d["ue4m3"][in_range])
    assert np.array_equal(oracle.f32_to_bf16_bits(v), d["bf16"])
    back = np.array([L.sharq_e2m1_to_f32(int(c)) for c in d["e2m1"]], np.float32)
    assert np.array_equal(back, d["e2m1_back"])
    ok = d["ue4m3"] != 0x7F
    back = np.array([L.sharq_ue4m3_to_f32(int(c)) for c in d["ue4m3"][ok]], np.float32)
    assert np.array_equal(back, d["ue4m3_back"][ok])


def test_rounding_rules(oracle):
    L = oracle.lib()
    for v, code in [(0.25, 0), (0.75, 2), (1.25, 2), (1.75, 4), (2.5, 4), (3.5, 6), (5.0, 6), (-0.1, 8), (7.0, 7)]:
        assert L.sharq_f32_to_e2m1(v) == code
    for v, code in [(2.0 ** -9, 1), (0.0029, 1), (0.003, 2), (1.0, 0x38), (440.0, 0x7E), (448.0, 0x7E)]:
        assert L.sharq_f32_to_ue4m3(v) == code
    # the dense-quant kernels write the reciprocal as a double division; same float for every scale
    for c in range(1, 0x7F):
        f = np.float32(L.sharq_ue4m3_to_f32(c))
        assert np.float32(1.0) / f == np.float32(1.0 / np.float64(f))


@pytest.mark.parametrize("name", ["small", "bias", "rmsnorm", "outlier"])
def test_sharq_sim_port_matches_reference_golden(name):
    d = np.load(GOLDEN / f"sharq_sim_{name}.npz")
    t = H.from_bits
    x, w = t(d["x"]), t(d["w"])
    bias = t(d["bias"]) if d["with_bias"] else None
    gamma = t(d["gamma"]) if d["with_norm"] else None
    torch.set_num_threads(1)  # the fixtures were made single-threaded; bf16 matmul order matters
    xin = sharq_sim.rmsnorm(x, gamma, float(d["eps"])) if gamma is not None else x
    assert np.array_equal(H.bits(xin), d["x_norm"])
    main, res, s = sharq_sim.quantize_activation(xin)
    assert np.array_equal(H.bits(main), d["main_q"])
    assert np.array_equal(H.bits(res), d["res_q"])
    assert np.float32(s.item()) == d["scale_x"]
    w_q, s_w = sharq_sim.quantize_weight(w)
    assert np.array_equal(H.bits(w_q), d["w_q"])
    assert np.float32(s_w.item()) == d["scale_w"]
    y = sharq_sim.linear(main, res, s, w_q, s_w, bias)
    assert np.array_equal(H.bits(y), d["y"])


@pytest.mark.parametrize("name", ["small", "outlier"])
def test_kernel_oracle_agrees_with_sharq_sim(oracle, name):
    """The bit-exact kernel restatement and the reference's simulation differ only through the
    documented rounding details (ties, subnormal scales, bf16 rounding of x/scale), so the
    dequantised activations must agree closely and the kept pairs almost always coincide."""
    d = np.load(GOLDEN / f"sharq_sim_{name}.npz")
    xin = d["x_norm"]
    m, k = xin.shape
    s = oracle.tensor_scale(oracle.absmax_bf16(xin), cuda_mode=False)
    assert s == d["scale_x"]
    a_comp, e, sfa, q_res, sf_res = oracle.prepare(oracle.scale_bf16(xin, s))
    xs = oracle.dequant_sparse(a_comp, e, sfa, m, k)
    xr = oracle.dequant_dense(q_res, sf_res, 16)
    sim_main = oracle.bf16_bits_to_f32(d["main_q"])
    sim_res = oracle.bf16_bits_to_f32(d["res_q"])
    assert ((xs != 0) == (sim_main != 0)).mean() > 0.99
    total, sim_total = xs + xr, sim_main + sim_res
    assert H.rel_fro(total, sim_total) < 2e-2
    x_true = oracle.bf16_bits_to_f32(xin) / s
    assert H.rel_fro(total, x_true) < 0.05  # sparse + residual reconstructs the scaled activation


def test_sizes_match_reference_layout_probe(oracle):
    """Byte sizes the reference's size helpers report (evaluated once against its headers)."""
    probe = {  # (M, N, K): (A_comp, E, SFA alloc, SFB alloc)
        (512, 4096, 4096): (524288, 131072, 163840, 1081344),
        (16, 4096, 4096): (16384, 32768, 32768, 1081344),
        (2048, 6144, 4096): (2097152, 524288, 557056, 1605632),
        (2048, 4096, 14336): (7340032, 1835008, 1949696, 3784704),
        (130, 256, 512): (16640, 8192, 8192, 12288),
    }
    for (m, n, k), (a, e, sfa, sfb) in probe.items():
        assert oracle.a_comp_bytes(m, k) == a
        assert oracle.e_bytes(m, k) == e
        assert oracle.sf_alloc_bytes(m, k) == sfa
        assert oracle.sf_alloc_bytes(n, k) == sfb


def test_scale_layout_is_a_permutation(oracle):
    for rows, groups in [(130, 4), (256, 32), (1, 128)]:
        off = oracle.sf_offsets(rows, groups)
        assert len(np.unique(off)) == off.size
        assert off.max() < ((rows + 127) // 128) * 128 * groups
        L = oracle.lib()
        for r, g in [(0, 0), (rows - 1, groups - 1), (rows // 2, groups // 3)]:
            assert L.sharq_sf_offset(r, g, groups) == off[r, g]


@pytest.mark.parametrize("case", sorted(H.MATRIX_SUITE))
def test_prepare_invariants(oracle, case):
    m, k = 8, 1024
    x = H.MATRIX_SUITE[case](m, k)
    xb = H.bits(x)
    qs, sfa_dbg, q_res_dbg, sf_res_dbg = oracle.prepare(xb, debug=True)
    a_comp, e, sfa, q_res, sf_res = oracle.prepare(xb)
    # never more than two non-zero bytes per 4-byte chunk of the dense sparse payload
    assert H.raw_violation_rate(qs) == 0.0
    assert np.array_equal(sfa, sfa_dbg) and np.array_equal(q_res, q_res_dbg) and np.array_equal(sf_res, sf_res_dbg)
    # compressed form decodes to the dense form (sparse GEMM == dense GEMM on the raw payload)
    dense_decode = oracle.dequant_dense(qs, oracle.duplicate_sf32_to_sf16(sfa, m, k), 16)
    assert np.array_equal(oracle.dequant_sparse(a_comp, e, sfa, m, k), dense_decode)
    # metadata: ascending distinct pair indices in every nibble of the used region
    nib = np.concatenate([e & 0xF, e >> 4])
    used = e.reshape(k // 256, 128, 16)[:, :m, :].reshape(-1)
    for b in (used & 0xF, used >> 4):
        assert ((b & 3) < (b >> 2)).all()
    assert nib.max() <= 0xE


def test_weight_shared_payload(oracle):
    w = H.config0_w(130, 512, 4)
    wb = oracle.scale_bf16(H.bits(w), oracle.tensor_scale(oracle.absmax_bf16(H.bits(w))))
    qw, sfs, sfd = oracle.quantize_w32_shared(wb)
    assert np.array_equal(oracle.dequant_dense(qw, sfs, 32), oracle.dequant_dense(qw, sfd, 16))
    assert np.array_equal(oracle.duplicate_sf32_to_sf16(sfs, 130, 512), sfd)
    deq = oracle.dequant_dense(qw, sfs, 32)
    assert H.rel_fro(deq, oracle.bf16_bits_to_f32(wb)) < 0.12  # 4-bit quantisation error level


def test_rmsnorm_stats_order_and_scale(oracle):
    x = H.config0_x(5, 256, 9)
    g = H.config0_gamma(256, 9)
    inv, amax, ssq = oracle.rmsnorm_row_stats(H.bits(x), H.bits(g), 1e-6)
    xf = x.float().numpy()
    # group-wise left-to-right float32 summation
    want = np.zeros(5, np.float32)
    for r in range(5):
        tot = np.float32(0)
        for gi in range(8):
            s = np.float32(0)
            for v in xf[r, 32 * gi:32 * gi + 32]:
                s = np.float32(s + np.float32(v * v))
            tot = np.float32(tot + s)
        want[r] = tot
    assert np.array_equal(ssq, want)
    assert np.allclose(inv, 1.0 / np.sqrt(want / 256 + 1e-6), rtol=1e-6)
    assert oracle.tensor_scale(2688.0, True) == np.float32(2688.0) * (np.float32(1.0) / np.float32(2688.0))
    assert oracle.tensor_scale(0.0, True) == np.float32(1e-9)


def test_cuda_mode_scaling_matches_torch_on_a_cuda_device(oracle):
    """tests/golden/cuda_scale_division.npz holds what torch returned on a B200 for the reference's
    `(x / scale).to(bf16)`; the oracle's cuda_mode must reproduce every value, and the fixture
    must really differ from the float32-scale division (else it would pin nothing)."""
    from pathlib import Path

    fix = np.load(Path(__file__).resolve().parent / "golden" / "cuda_scale_division.npz")
    differs = 0
    for i in range(8):
        x, scale, q = fix[f"x{i}"], float(fix[f"scale{i}"]), fix[f"q{i}"]
        assert oracle.tensor_scale(oracle.absmax_bf16(x), cuda_mode=True) == np.float32(scale)
        assert np.array_equal(oracle.scale_bf16(x, scale, cuda_mode=True), q), i
        differs += int((oracle.scale_bf16(x, scale, cuda_mode=False) != q).sum())
    assert differs > 1000
