"""Observability helpers against fakes (no NVML, no HTTP)."""
import json
import types

from skyrl_b200.utils.monitor import AsyncPhaseGauges, GPUMonitor, ServerMetricsScraper, parse_prometheus_text
from skyrl_b200.utils.trajectory_logging import TrajectoryLogger


class _FakeNVML:
    NVML_CLOCK_SM = 1

    def __init__(self):
        self.t = 0

    def nvmlDeviceGetCount(self):
        return 2

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetUtilizationRates(self, h):
        self.t += 1
        return types.SimpleNamespace(gpu=50 + 10 * h + self.t, memory=0)

    def nvmlDeviceGetMemoryInfo(self, h):
        return types.SimpleNamespace(used=(h + 1) * 2**30, total=180 * 2**30)

    def nvmlDeviceGetClockInfo(self, h, which):
        return 1700

    def nvmlDeviceGetPowerUsage(self, h):
        return 900_000


def test_gpu_monitor_reads_only_and_summarises():
    mon = GPUMonitor(nvml=_FakeNVML())
    assert mon._init()
    mon.sample_once()
    mon.sample_once()
    s = mon.summary()
    assert s["gpu/1/mem_used_gb_max"] == 2.0 and s["gpu/0/sm_mhz_mean"] == 1700 and s["gpu/0/power_w_max"] == 900.0
    assert s["gpu/0/util_max"] > s["gpu/0/util_mean"] - 5
    assert mon.summary() == {}


def test_scraper_rates_between_two_scrapes():
    state = {"n": 0}

    def fetch(url):
        state["n"] += 1
        k = state["n"]
        return (f"# HELP x\nskyrl_b200_generation_tokens_total {1000 * k}\nskyrl_b200_kv_usage 0.5\n"
                f"skyrl_b200_ttft_seconds_sum {0.2 * k}\nskyrl_b200_ttft_seconds_count {2 * k}\n"
                f"skyrl_b200_prefix_cache_queries_total {10 * k}\nskyrl_b200_prefix_cache_hits_total {4 * k}\n")

    sc = ServerMetricsScraper(["http://a"], fetch=fetch)
    first = sc.delta()
    assert first["inference/kv_usage"] == 0.5 and "inference/gen_tokens_per_s" not in first
    second = sc.delta()
    assert second["inference/gen_tokens_per_s"] > 0
    assert abs(second["inference/ttft_s"] - 0.1) < 1e-9 and abs(second["inference/prefix_hit_rate"] - 0.4) < 1e-9
    assert parse_prometheus_text('a{x="1"} 2\na{x="2"} 3\nbad line\n')["a"] == 5.0


def test_gauges_and_trajectory_log(tmp_path):
    g = AsyncPhaseGauges("skyrl_b200_test")
    g.set("staleness_max", 3)
    assert g.values["staleness_max"] == 3.0
    out = {"prompt_token_ids": [[1, 2], [3]], "response_ids": [[4, 5, 6], [7]], "rewards": [[0, 0, 1.0], 0.5],
           "stop_reasons": ["stop", "length"]}
    p = TrajectoryLogger(str(tmp_path), max_rows=1).log(out, 3, uids=["u0", "u1"])
    rows = [json.loads(l) for l in open(p)]
    assert len(rows) == 1 and rows[0]["reward"] == 1.0 and rows[0]["response"] == "4 5 6" and rows[0]["uid"] == "u0"
