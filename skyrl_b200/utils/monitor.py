"""Observability helpers: GPU monitor thread, rollout-server metrics scraper, Prometheus gauges for async phases.

References: skyrl/train/utils/ray_gpu_monitor.py (periodic utilisation / memory sampling per GPU),
skyrl/train/utils/vllm_metrics_scraper.py (Prometheus text scrape of the rollout servers: tokens/s, TTFT, ITL, KV-cache
usage, prefix-cache hit rate, spec-decode acceptance), skyrl/train/utils/metrics.py:19-83 (gauges for the async phases).
NVML is only ever *read* here (utilisation, memory, clocks, power, throttle reasons); nothing is set.
"""

from __future__ import annotations

import re
import threading
import time
from typing import Any, Callable, Dict, List, Optional


class GPUMonitor:
    """Samples NVML in a daemon thread; ``summary()`` gives mean / max per metric since the last call."""

    FIELDS = ("util", "mem_used_gb", "sm_mhz", "power_w")

    def __init__(self, interval_s: float = 1.0, devices: Optional[List[int]] = None, nvml=None):
        self.interval_s, self.devices = interval_s, devices
        self._nvml = nvml  # injectable fake for tests
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()
        self._samples: Dict[int, List[Dict[str, float]]] = {}
        self._handles: Dict[int, Any] = {}

    def _init(self) -> bool:
        if self._nvml is None:
            try:
                import pynvml

                pynvml.nvmlInit()
                self._nvml = pynvml
            except Exception:
                return False
        n = self._nvml.nvmlDeviceGetCount()
        for i in (self.devices if self.devices is not None else range(n)):
            self._handles[i] = self._nvml.nvmlDeviceGetHandleByIndex(i)
        return bool(self._handles)

    def sample_once(self) -> Dict[int, Dict[str, float]]:
        nv, out = self._nvml, {}
        for i, h in self._handles.items():
            u = nv.nvmlDeviceGetUtilizationRates(h)
            m = nv.nvmlDeviceGetMemoryInfo(h)
            s = {"util": float(u.gpu), "mem_used_gb": m.used / 2**30}
            try:
                s["sm_mhz"] = float(nv.nvmlDeviceGetClockInfo(h, getattr(nv, "NVML_CLOCK_SM", 1)))
                s["power_w"] = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
            except Exception:
                pass
            out[i] = s
        with self._lock:
            for i, s in out.items():
                self._samples.setdefault(i, []).append(s)
        return out

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.sample_once()
            except Exception:
                return

    def start(self) -> "GPUMonitor":
        if self._init():
            self._thread = threading.Thread(target=self._run, name="gpu-monitor", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def summary(self, reset: bool = True) -> Dict[str, float]:
        with self._lock:
            snap = {i: list(v) for i, v in self._samples.items()}
            if reset:
                self._samples.clear()
        out: Dict[str, float] = {}
        for i, rows in snap.items():
            for f in self.FIELDS:
                vals = [r[f] for r in rows if f in r]
                if vals:
                    out[f"gpu/{i}/{f}_mean"] = sum(vals) / len(vals)
                    out[f"gpu/{i}/{f}_max"] = max(vals)
        return out


_LINE = re.compile(r"^([a-zA-Z_:][a-zA-Z0-9_:]*)(\{[^}]*\})?\s+([-+0-9.eE]+|NaN|[+-]Inf)\s*$")


def parse_prometheus_text(text: str) -> Dict[str, float]:
    """``name{labels} value`` lines -> ``{name: sum over label sets}`` (histogram ``_sum`` / ``_count`` kept as is)."""
    out: Dict[str, float] = {}
    for line in text.splitlines():
        if not line or line[0] == "#":
            continue
        m = _LINE.match(line.strip())
        if not m:
            continue
        try:
            v = float(m.group(3))
        except ValueError:
            continue
        out[m.group(1)] = out.get(m.group(1), 0.0) + v
    return out


class ServerMetricsScraper:
    """Polls ``/metrics`` of each rollout server; ``delta()`` turns counters into rates between two scrapes."""

    # counter name on the server -> rate reported (both this engine's names and the conventional *_total ones)
    RATES = {"generation_tokens_total": "gen_tokens_per_s", "prompt_tokens_total": "prompt_tokens_per_s",
             "requests_finished_total": "requests_per_s", "decode_tokens": "gen_tokens_per_s",
             "prefill_tokens": "prompt_tokens_per_s", "decode_steps": "decode_steps_per_s"}
    COUNTERS = frozenset(RATES)

    def __init__(self, urls: List[str], fetch: Optional[Callable[[str], str]] = None, prefix: str = "skyrl_b200_"):
        self.urls, self.prefix = [u.rstrip("/") for u in urls], prefix
        self._fetch = fetch or self._http_get
        self._last: Optional[Dict[str, float]] = None
        self._last_t = 0.0

    @staticmethod
    def _http_get(url: str) -> str:
        import requests

        return requests.get(url + "/metrics", timeout=5).text

    def scrape(self) -> Dict[str, float]:
        tot: Dict[str, float] = {}
        for u in self.urls:
            try:
                for k, v in parse_prometheus_text(self._fetch(u)).items():
                    k = k[len(self.prefix):] if k.startswith(self.prefix) else k
                    tot[k] = tot.get(k, 0.0) + v
            except Exception:
                tot["scrape_errors"] = tot.get("scrape_errors", 0.0) + 1
        return tot

    def delta(self) -> Dict[str, float]:
        now, cur = time.time(), self.scrape()
        out = {f"inference/{k}": v for k, v in cur.items() if not k.endswith("_total") and k not in self.COUNTERS}
        if self._last is not None and now > self._last_t:
            dt = now - self._last_t
            for k, name in self.RATES.items():
                if k in cur and k in self._last:
                    out[f"inference/{name}"] = (cur[k] - self._last[k]) / dt
            if cur.get("ttft_seconds_count", 0) > self._last.get("ttft_seconds_count", 0):
                out["inference/ttft_s"] = ((cur["ttft_seconds_sum"] - self._last.get("ttft_seconds_sum", 0.0)) /
                                           (cur["ttft_seconds_count"] - self._last.get("ttft_seconds_count", 0.0)))
            q, h = cur.get("prefix_cache_queries_total"), cur.get("prefix_cache_hits_total")
            if q and h is not None and q > self._last.get("prefix_cache_queries_total", 0):
                out["inference/prefix_hit_rate"] = ((h - self._last.get("prefix_cache_hits_total", 0.0)) /
                                                    (q - self._last.get("prefix_cache_queries_total", 0.0)))
        self._last, self._last_t = cur, now
        return out


class AsyncPhaseGauges:
    """Prometheus gauges of the fully-async trainer's phases (queue depth, staleness, in-flight groups)."""

    def __init__(self, namespace: str = "skyrl_b200"):
        self.values: Dict[str, float] = {}
        self._g = {}
        try:
            from prometheus_client import Gauge

            for n in ("generation_queue_depth", "inflight_groups", "staleness_mean", "staleness_max", "trainer_idle_s",
                      "weight_version"):
                try:
                    self._g[n] = Gauge(f"{namespace}_{n}", n.replace("_", " "))
                except ValueError:  # already registered in this process
                    pass
        except ImportError:
            pass

    def set(self, name: str, value: float) -> None:
        self.values[name] = float(value)
        g = self._g.get(name)
        if g is not None:
            g.set(float(value))
