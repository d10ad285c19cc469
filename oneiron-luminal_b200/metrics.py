"""Benchmark metrics in the shape of the reference's bench crate (crates/luminal_bench/src/metrics.rs:13-60, 62-110): constant
per-benchmark byte and flop counts, a hardware description, and the derived figures — GB/s, TFLOP/s, MBU and MFU (both in
percent, as the reference prints them) — once a time is known.  The JSON written by ``BenchMetricsMap.to_json`` has the
reference's field names, so tooling that reads its ``metrics.json`` reads this one.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Dict

from .runtime import ModelDesc, decode_bytes_per_token


@dataclass
class BenchMetrics:
    """Bytes moved and floating-point operations of one benchmark configuration."""
    bytes_loaded: int
    bytes_stored: int
    flops: int
    bytes: int = 0

    def __post_init__(self):
        self.bytes = self.bytes_loaded + self.bytes_stored

    def throughput_gbps(self, time_us: float) -> float:
        return 0.0 if time_us <= 0 else self.bytes / time_us / 1000.0

    def tflops(self, time_us: float) -> float:
        return 0.0 if time_us <= 0 else self.flops / time_us / 1_000_000.0

    def mbu(self, time_us: float, peak_bandwidth_gbps: float) -> float:
        return self.throughput_gbps(time_us) / peak_bandwidth_gbps * 100.0

    def mfu(self, time_us: float, peak_tflops: float) -> float:
        return self.tflops(time_us) / peak_tflops * 100.0


@dataclass
class HardwareSpec:
    device_name: str
    memory_gb: float
    peak_bandwidth_gbps: float
    peak_tflops: float


@dataclass
class BenchMetricsMap:
    hardware: HardwareSpec
    benchmarks: Dict[str, BenchMetrics] = field(default_factory=dict)

    def add(self, name: str, m: BenchMetrics) -> None:
        self.benchmarks[name] = m

    def to_json(self) -> str:
        return json.dumps({"hardware": asdict(self.hardware), "benchmarks": {k: asdict(v) for k, v in self.benchmarks.items()}}, indent=2)

    @staticmethod
    def from_json(text: str) -> "BenchMetricsMap":
        d = json.loads(text)
        m = BenchMetricsMap(HardwareSpec(**d["hardware"]))
        for k, v in d["benchmarks"].items():
            m.add(k, BenchMetrics(v["bytes_loaded"], v["bytes_stored"], v["flops"]))
        return m

    def summary(self, name: str, time_us: float) -> dict:
        """The derived figures of one benchmark at a measured time."""
        b = self.benchmarks[name]
        return {"time_us": time_us, "gbps": b.throughput_gbps(time_us), "tflops": b.tflops(time_us),
                "mbu_pct": b.mbu(time_us, self.hardware.peak_bandwidth_gbps), "mfu_pct": b.mfu(time_us, self.hardware.peak_tflops)}


def linear_params(d: ModelDesc) -> int:
    """Weights of the linear layers one token passes through (a routed FFN counts its top_k experts), head included."""
    hd = d.head_dim
    attn = d.hidden * (d.n_q_heads * hd) * 2 + d.hidden * (d.n_kv_heads * hd) * 2
    if d.n_experts > 0:
        ffn = d.top_k * 3 * d.hidden * d.ffn + d.n_experts * d.hidden
    else:
        ffn = 3 * d.hidden * d.ffn
    return d.n_layers * (attn + ffn) + d.vocab * d.hidden


def decode_step_metrics(d: ModelDesc, context: int, rows: int = 1) -> BenchMetrics:
    """One decode step of `rows` sequences with `context` cached positions each: bytes as decode_bytes_per_token counts them
    (weights once per step, the cache rows per sequence), 2 flops per weight per row plus the attention products."""
    kv_elem = 2 if d.kv_dtype == 2 else 4
    kv_row = 2 * d.n_layers * d.n_kv_heads * d.head_dim * kv_elem
    weights = decode_bytes_per_token(d, 0) - kv_row            # the step's bytes with an empty cache, minus the row it writes
    loaded = int(weights + rows * kv_row * context)
    stored = int(rows * kv_row)
    flops = rows * (2 * linear_params(d) + 4 * d.n_layers * d.n_q_heads * d.head_dim * (context + 1))
    return BenchMetrics(loaded, stored, int(flops))
