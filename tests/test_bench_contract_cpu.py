"""The benchmark's reference arm runs on the host and prints one JSON line with the keys the
round-end driver reads."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_contract_line():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1",
                          "--cpu-seconds", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "sharq_linear_tflops" and d["unit"] == "TFLOP/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
                "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["value"] > 0


def test_bench_help_lists_modes():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--shape-sweep", "--kernel-table", "--prefill-model"):
        assert flag in res.stdout


def test_kernel_categories_follow_the_reference_profiler():
    """bench.py --kernel-table sums kernels into the categories of the reference's prefill profiler
    (benchmarks/e2e/profile_prefill_nvtx.py:159-275)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cat = bench.kernel_category
    assert cat("void sharq::(anonymous namespace)::gemm_kernel<256, true, true, true, false>(CUtensorMap_st") == "gemm"
    assert cat("sharq::(anonymous namespace)::gemm_grouped_kernel(sharq::(anonymous namespace)::GroupTable") == "gemm"
    assert cat("nvjet_tst_128x8_64x12_2x1_v_bz_TNT") == "gemm"
    assert cat("void sharq::(anonymous namespace)::prepare_fused_kernel<1, true, 512>(") == "sharq_kernel"
    assert cat("void sharq::(anonymous namespace)::prepare_kernel<2, false, 2>(") == "sharq_kernel"
    assert cat("void sharq::(anonymous namespace)::rms_stats_kernel<true>(") == "sharq_kernel"
    assert cat("sharq::(anonymous namespace)::sp_transition_kernel(sharq::(anonymous namespace)::SpParams)") == "sharq_kernel+collective"
    assert cat("void sharq::(anonymous namespace)::quantize_dense_nvfp4_kernel(") == "quantize_kernel"
    assert cat("cudnn_generated_fort_native_sdpa_sm100_flash_fprop_f16_knob_7_128x128x128") == "attention"
    assert cat("void sharq::(anonymous namespace)::add_rmsnorm_kernel<true>(") == "rmsnorm"
    assert cat("ncclDevKernel_AllReduce_Sum_f32_RING_LL(ncclDevKernelArgsStorage<4096ul>)") == "collective"
    assert cat("sharq::(anonymous namespace)::allreduce_multimem_kernel(") == "collective"
    assert cat("sharq::(anonymous namespace)::rope_kernel(__nv_bfloat16*, long long") == "other"
