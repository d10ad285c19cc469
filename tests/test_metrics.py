"""The MBU / MFU report (crates/luminal_bench/src/metrics.rs:13-60): same arithmetic, same JSON field names."""
import json

import pytest


def test_derived_figures_follow_the_reference_formulas(pkg):
    from oneiron_luminal_b200.metrics import BenchMetrics, BenchMetricsMap, HardwareSpec
    m = BenchMetrics(bytes_loaded=8_000_000_000, bytes_stored=500_000_000, flops=16_000_000_000)
    assert m.bytes == 8_500_000_000
    assert m.throughput_gbps(2000.0) == pytest.approx(4250.0)          # bytes / us / 1000
    assert m.tflops(2000.0) == pytest.approx(8.0)                      # flops / us / 1e6
    assert m.mbu(2000.0, 8000.0) == pytest.approx(53.125)              # percent
    assert m.mfu(2000.0, 2250.0) == pytest.approx(8.0 / 2250.0 * 100)
    assert m.throughput_gbps(0.0) == 0.0 and m.tflops(-1.0) == 0.0
    mm = BenchMetricsMap(HardwareSpec("NVIDIA B200", 180.0, 6540.8, 1646.6))
    mm.add("decode/llama3_8b_q8/p512", m)
    d = json.loads(mm.to_json())
    assert set(d) == {"hardware", "benchmarks"}
    assert set(d["hardware"]) == {"device_name", "memory_gb", "peak_bandwidth_gbps", "peak_tflops"}
    assert set(d["benchmarks"]["decode/llama3_8b_q8/p512"]) == {"bytes", "bytes_loaded", "bytes_stored", "flops"}
    back = BenchMetricsMap.from_json(mm.to_json())
    assert back.summary("decode/llama3_8b_q8/p512", 2000.0)["mbu_pct"] == pytest.approx(4250.0 / 6540.8 * 100)


def test_decode_step_counts_match_the_byte_model(pkg):
    from oneiron_luminal_b200.metrics import decode_step_metrics, linear_params
    d = pkg.CONFIGS["llama3_8b_q8"]
    # 8.03e9 parameters, 7.5e9 of them in linear layers and the head (the embedding table is read one row at a time)
    assert linear_params(d) == 32 * (2 * 4096 * 4096 + 2 * 4096 * 1024 + 3 * 4096 * 14336) + 128256 * 4096
    m = decode_step_metrics(d, 512)
    assert m.bytes == pytest.approx(pkg.decode_bytes_per_token(d, 512), rel=1e-9)
    assert m.flops == 2 * linear_params(d) + 4 * 32 * 32 * 128 * 513
    m32 = decode_step_metrics(d, 512, rows=32)
    assert m32.bytes_stored == 32 * m.bytes_stored and m32.flops == 32 * m.flops
    moe = pkg.CONFIGS["gpt_oss_20b_q8"]
    assert linear_params(moe) < 4e9                                     # 4 of 32 experts per token
