"""The byte / flop figures bench.py divides by (the algorithmic bytes per launch of every workload)."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_dense_algorithmic_bytes():
    b = _bench()
    assert b.algorithmic_bytes("u4b8", 4096, 4096, 128) == 8_650_752
    assert b.algorithmic_bytes("u4", 8192, 28672, 128) == 124_780_544
    assert b.algorithmic_bytes("u8b128", 8192, 28672, -1) == 234_938_368
    assert b.algorithmic_bytes("fp8", 5120, 25600, -1) == 131_123_200
    assert b.algorithmic_bytes("mxfp4", 5120, 25600, 32) == 69_632_000
    assert b.algorithmic_bytes("nvfp4", 5120, 25600, 16) == 73_728_004


def test_moe_bytes_per_expert():
    b = _bench()
    assert b.moe_bytes_per_expert("u4b8", 4096, 1536, 128) == 9_732_096
    assert b.moe_bytes_per_expert("mxfp4", 3072, 1024, 32) == 5_013_504


def test_workload_tables_and_selector_names():
    b = _bench()
    assert b.DEFAULT_WORKLOAD in b.WORKLOADS
    assert b.dominant_kernel("dense_u4_g128_bf16_m16", 16, 8192, 28672) == "decode_tc_kernel"
    assert b.dominant_kernel("dense_u4_g128_bf16_m1", 1, 8192, 28672) == "decode_kernel"
    assert b.dominant_kernel("dense_u4_g128_bf16_m4096", 4096, 8192, 28672) == "tc_gemm_kernel"
    assert b.dominant_kernel("dense_u4_g128_bf16_m64", 64, 8192, 28672) == "tc_gemm_kernel"
    # the metric's name follows the row count: weight streaming up to 64 rows, tensor throughput above
    assert b.metric_name("dense_u4_g128_bf16_m16") == b.METRIC
    assert b.metric_name("dense_u4_g128_bf16_m64") == b.METRIC_MID
    assert b.metric_name("dense_u4b8_g128_fp16_m64_k4096") == b.METRIC_MID
    assert b.metric_name("dense_u4_g128_bf16_m4096") == b.METRIC_COMPUTE
    for name, cfg in b.MOE_WORKLOADS.items():
        assert cfg[2] % 8 == 0 and cfg[7] >= 1, name
