"""Every environment variable the framework reads, in one place (reference: ``skyrl/env_vars.py:13-106``).

Two families: ``SKYRL_*`` knobs carried over from the reference where the concept still exists in a
one-process-per-GPU runtime, and ``SB_*`` switches of the native kernels (mostly A/B toggles for measurements).
``describe()`` returns the table (name, current value, default, meaning); ``python -m skyrl_b200.env_vars`` prints it.
Variables that configure an actor cluster in the reference (placement-group timeout, LD_LIBRARY_PATH / PYTHONPATH
export to remote workers, data-parallel port offsets of the external engine) have no counterpart here: ranks are local
processes started by ``skyrl_b200.launch`` and inherit the launching environment.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, List


def _flag(v: str) -> bool:
    return str(v).strip().lower() in ("1", "true", "yes", "on")


@dataclass(frozen=True)
class EnvVar:
    name: str
    default: str
    parse: Callable[[str], object]
    doc: str

    def get(self):
        return self.parse(os.environ.get(self.name, self.default))


_VARS: List[EnvVar] = [
    # ---- carried over from the reference
    EnvVar("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", "600", int,
           "timeout of the NCCL / gloo process groups created by the workers (seconds)"),
    EnvVar("SKYRL_WAIT_UNTIL_INFERENCE_SERVER_HEALTHY_TIMEOUT_S", "600", int,
           "how long clients wait for a generation server's /health before giving up (seconds)"),
    EnvVar("SKYRL_HTTP_CONNECTION_LIMIT", "50000", int, "connection-pool limit of the HTTP inference client"),
    EnvVar("SKYRL_GENERATE_CONCURRENCY_PER_ENGINE", "512", int,
           "trajectories a generator keeps in flight per generation engine"),
    EnvVar("SKYRL_DUMP_INFRA_LOG_TO_STDOUT", "False", _flag, "print infrastructure logs of all ranks instead of rank 0 only"),
    EnvVar("SKYRL_LOG_LEVEL", "INFO", str, "log level of the ``skyrl_b200`` logger"),
    # ---- this runtime
    EnvVar("SKYRL_B200_NO_AUTOBUILD", "0", _flag, "do not compile the native libraries on first import (CI images ship them)"),
    EnvVar("SKYRL_B200_NUMA_PIN", "1", _flag, "bind each rank's host threads to the CPUs of its GPU's NUMA node"),
    EnvVar("SKYRL_B200_PEER_WAIT_S", "2.0", float, "upper bound of every wait on a peer flag inside the NVLink kernels (seconds)"),
    # ---- kernel switches (A/B measurements; defaults are the fast paths)
    EnvVar("SB_TP_DECODE_SPLITK", "0", _flag,
           "tensor-parallel engines: split the row-parallel decode GEMMs over k slices (more SMs, more NVLink bytes)"),
    EnvVar("SKYRL_B200_ROLLOUT_BASE_PORT", "", str,
           "disaggregated launch: first port of the rollout-only ranks' servers (default MASTER_PORT + 100)"),
    EnvVar("SKYRL_B200_ROLLOUT_URLS", "", str,
           "disaggregated launch: server URLs of the rollout ranks (written by the role split for the training ranks)"),
    EnvVar("SKYRL_B200_ROLE", "", str, "disaggregated launch: 'train' or 'rollout' once the role split has run"),
    EnvVar("SB_FORCE_CPU", "0", _flag, "tests: run the multi-rank engine check on CPU tensors even when GPUs exist"),
    EnvVar("SB_PDL", "1", _flag, "programmatic dependent launch between the kernels of a decode step / training layer"),
    EnvVar("SB_GEMM_PAIR", "1", _flag, "CTA-pair (cta_group::2) GEMM for large problems"),
    EnvVar("SB_FUSED_MLP", "1", _flag, "SwiGLU inside the gate/up and down-gradient GEMM epilogues (training)"),
    EnvVar("SB_DECODE_FUSED_MLP", "1", _flag, "SwiGLU inside the gate/up GEMM epilogue (decode)"),
    EnvVar("SKYRL_B200_JUDGE_URL", "http://127.0.0.1:8000", str, "llm_judge environment: default base URL of the judge endpoint"),
    EnvVar("SKYRL_B200_REFERENCE_ANCHORS", "1", _flag,
           "bench.py --impl reference: time the reference's own LM-head kernel and flash-attn as phase anchors"),
    EnvVar("SKYRL_B200_DEBUG_BOUNDS", "0", _flag,
           "debug mode: check every index tensor (token ids, cache slots, block tables, targets) before the kernel launch"),
    EnvVar("SB_DECODE_MLP_BLOCK", "0", _flag,
           "decode: o-proj .. down-proj of a layer as one persistent kernel (when EngineConfig.fused_mlp_block is unset)"),
    EnvVar("SB_DECODE_ATTN_PERSIST", "1", _flag, "persistent paged decode attention (one CTA per SM walking a work list)"),
    EnvVar("SB_DECODE_ATTN_SPLITS", "", str, "force the context split count of decode attention (empty = cost model)"),
    EnvVar("SB_BF16_TFLOPS", "1376.9", float, "bf16 GEMM peak used as roofline denominator by the benchmarks (TFLOP/s)"),
    EnvVar("SB_HBM_GBS", "6543.4", float, "HBM copy bandwidth used as roofline denominator by the benchmarks (GB/s)"),
]

_BY_NAME: Dict[str, EnvVar] = {v.name: v for v in _VARS}


def get(name: str):
    """Parsed value of a registered variable (its default when unset)."""
    return _BY_NAME[name].get()


def describe() -> List[Dict[str, str]]:
    return [{"name": v.name, "value": os.environ.get(v.name, v.default), "default": v.default, "doc": v.doc} for v in _VARS]


# module-level constants for the names the reference exposes the same way
SKYRL_WORKER_NCCL_TIMEOUT_IN_S = get("SKYRL_WORKER_NCCL_TIMEOUT_IN_S")
SKYRL_WAIT_UNTIL_INFERENCE_SERVER_HEALTHY_TIMEOUT_S = get("SKYRL_WAIT_UNTIL_INFERENCE_SERVER_HEALTHY_TIMEOUT_S")
SKYRL_HTTP_CONNECTION_LIMIT = get("SKYRL_HTTP_CONNECTION_LIMIT")
SKYRL_GENERATE_CONCURRENCY_PER_ENGINE = get("SKYRL_GENERATE_CONCURRENCY_PER_ENGINE")
SKYRL_DUMP_INFRA_LOG_TO_STDOUT = get("SKYRL_DUMP_INFRA_LOG_TO_STDOUT")


if __name__ == "__main__":
    for row in describe():
        print(f"{row['name']:<52} {row['value']!s:<10} (default {row['default']!s})  {row['doc']}")
