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


def test_records_of_the_default_line_and_their_data():
    b = _bench()
    for name in b.ALSO_WORKLOADS + (b.EP_WORKLOAD,):
        assert name in b.WORKLOADS or name in b.MOE_WORKLOADS
    # the streaming layout changes the dominant kernel of the decode sizes, and the traffic figure follows it
    assert b.dominant_kernel("dense_u4_g128_bf16_m16", 16, 8192, 28672, "streaming") == "stream_i8_kernel"
    assert b.dominant_kernel("dense_u8b128_ch_bf16_m16", 16, 8192, 28672, "streaming") == "stream_gemm_kernel"
    # 17-32 rows stay on the integer kernel, 33-64 rows go to the 16-bit streaming kernel
    assert b.dominant_kernel("dense_u4_g128_bf16_m32", 32, 8192, 28672, "streaming") == "stream_i8_kernel"
    assert b.dominant_kernel("dense_u4_g128_bf16_m64", 64, 8192, 28672, "streaming") == "stream_gemm_kernel"
    assert b.dominant_kernel("dense_u4_g128_bf16_m64", 64, 8192, 28672, "reference") == "tc_gemm_kernel"
    traffic = b.ncu_traffic("dense_u4_g128_bf16_m16", "stream_i8_kernel")
    assert traffic is not None and 1.0 <= traffic / b.algorithmic_bytes("u4", 8192, 28672, 128) <= 1.05
    assert b.ncu_traffic("dense_u4_g128_bf16_m16", "decode_tc_kernel") is None     # figure of another kernel
    assert b.ncu_traffic("no_such_workload", "stream_i8_kernel") is None
    from oracle import marlin_oracle as mo
    assert b.type_id_of("u4b8") == mo.TYPE_U4B8 and b.type_id_of("mxfp4") == mo.TYPE_FE2M1
    assert b.type_id_of("fp8") == mo.TYPE_FE4M3 and b.type_id_of("u8") == mo.TYPE_U8


def test_expert_placement_of_the_benchmark_router():
    """The placement the expert-parallel record uses: the busiest rank stays within 1.1x of the mean at 2, 4
    and 8 ranks on the benchmark's Zipf router (contiguous shards: up to 2.2x)."""
    import torch
    from marlin_v100_b200 import parallel
    b = _bench()
    fmt, dtype, e, topk, hidden, inter, group, tokens, zipf = b.MOE_WORKLOADS[b.EP_WORKLOAD]
    g = torch.Generator().manual_seed(3)
    torch.randn(tokens, hidden, generator=g)
    logits = torch.randn(tokens, e, generator=g)
    ranks = torch.randperm(e, generator=g).float() + 1.0
    pe = ranks.pow(-1.1)
    logits = logits + (pe / pe.sum()).log()
    cal = torch.randn(4096, e, generator=torch.Generator().manual_seed(4)) + (pe / pe.sum()).log()
    expected = torch.bincount(torch.topk(cal, topk, dim=-1).indices.reshape(-1), minlength=e).float()
    count = torch.bincount(torch.topk(logits, topk, dim=-1).indices.reshape(-1), minlength=e).float()
    for world in (2, 4, 8):
        slot = parallel.balanced_expert_placement(expected, world)
        load = torch.zeros(world)
        load.index_add_(0, torch.div(slot.long(), e // world, rounding_mode="floor"), count)
        assert float(load.max() / load.mean()) <= 1.1
