"""report.py turns benchmark lines into the documentation's tables; checked on synthetic lines (no GPU)."""
from e5m2effma_b200 import report


def _roof(frac):
    return {"frac": frac, "frac_of_nominal": frac * 0.7, "sustained": {"ms_per_step": 0.4, "frac": 0.8, "clocks": {"sm_mhz": 1400}}}


def test_single_gpu_table_lists_headline_and_workloads():
    d = {"n_gpus": 1, "config": {"workload": "headline"}, "ms_per_step": 0.35, "value": 2800.0, "unit": "TFLOP/s", "roofline": _roof(0.86),
         "clocks": {"sm_mhz": 1965, "reasons": []},
         "cpu_baseline": {"cores": 16, "kind": "port", "value": 1.0, "unit": "TFLOP/s", "sample": "slab",
                          "observed_error": {"accumulation": {"max_error_in_units_of_2^-23_sum_abs_products": 0.5}}},
         "e2e": {"ms_per_step": 3.3, "value": 288.0, "unit": "TFLOP/s", "h2d_bytes_per_step": 176e6, "d2h_bytes_per_step": 33e6},
         "workloads": {"c1": {"workload": "small gemm", "ms_per_step": 0.056, "value": 2400.0, "unit": "TFLOP/s", "roofline": _roof(0.75), "clocks": {}},
                       "c9": {"error": "boom"}}}
    text = report.single_gpu_table(d)
    assert "| headline | 350.0 us | 2800 TFLOP/s | 86.0 %" in text and "| small gemm | 56.0 us" in text and "failed: boom" in text
    assert "End to end" in text and "CPU oracle (16 threads" in text


def test_strong_scaling_table():
    s = {"full_problem_one_gpu_ms": 0.34, "kernel_only": {"ms_per_step": 0.18, "strong_efficiency": 0.93},
         "with_collectives_nccl": {"ms_per_step": 0.24, "strong_efficiency": 0.70}, "with_collectives_fused": {"unavailable": "x"}}
    d = {"n_gpus": 2, "config": {"workload": "headline", "weak": {"ms_per_step": 0.35, "value": 5500.0, "unit": "TFLOP/s"}}, "strong_scaling": s,
         "workloads": {"c4": {"workload": "wgrad", "strong_scaling": {"full_problem_one_gpu_ms": 2.0, "kernel_only": {"ms_per_step": 1.05, "strong_efficiency": 0.96}}}}}
    text = report.strong_table(d)
    assert "| headline | 340.0 us | 180.0 us, 93.0 % | 240.0 us, 70.0 % | unavailable |" in text
    assert "| wgrad | 2000.0 us | 1050.0 us, 96.0 % | - | - |" in text and "Weak scaling" in text


def test_rows_table():
    d = {"gemm_rows": [{"row": "e5ma_gemm NT E5M2 x E5M2 -> BF16", "ms_per_step": 0.06, "value": 2290.0, "unit": "TFLOP/s",
                        "kernel": "tcgen05 one CTA, 256-row tiles", "peak": 3245.6, "peak_source": "measured: 2 x bf16_tflops burst",
                        "frac": 0.7056, "clocks": {"sm_mhz": 1900}},
                       {"row": "e5ma_gemm TN E5M2 x FP32 -> BF16", "error": "boom"}]}
    text = report.rows_table(d)
    assert "| e5ma_gemm NT E5M2 x E5M2 -> BF16 | 60.0 us | 2290 TFLOP/s | tcgen05 one CTA, 256-row tiles | 70.6 % of 3246 (measured: 2 x bf16_tflops burst) | 1900 |" in text
    assert "failed: boom" in text
