"""Environment-variable knobs (names kept from the reference, skyrl/env_vars.py:13-106)."""

from __future__ import annotations

import os


def _int(name: str, default: int) -> int:
    return int(os.environ.get(name, str(default)))


def _bool(name: str, default: bool = False) -> bool:
    return os.environ.get(name, "1" if default else "0").lower() in ("1", "true", "yes")


SKYRL_RAY_PG_TIMEOUT_IN_S = _int("SKYRL_RAY_PG_TIMEOUT_IN_S", 180)  # kept for launch-time rendezvous timeouts
SKYRL_WORKER_NCCL_TIMEOUT_IN_S = _int("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", 600)
SKYRL_GENERATE_CONCURRENCY_PER_ENGINE = _int("SKYRL_GENERATE_CONCURRENCY_PER_ENGINE", 512)
SKYRL_HTTP_CONNECTION_LIMIT = _int("SKYRL_HTTP_CONNECTION_LIMIT", 4096)
SKYRL_DUMP_INFRA_LOG_TO_STDOUT = _bool("SKYRL_DUMP_INFRA_LOG_TO_STDOUT")
SKYRL_LD_LIBRARY_PATH_EXPORT = _bool("SKYRL_LD_LIBRARY_PATH_EXPORT")
SKYRL_PYTHONPATH_EXPORT = _bool("SKYRL_PYTHONPATH_EXPORT")
SKYRL_WAIT_UNTIL_INFERENCE_SERVER_HEALTHY_TIMEOUT_S = _int("SKYRL_WAIT_UNTIL_INFERENCE_SERVER_HEALTHY_TIMEOUT_S", 600)
SKYRL_INCLUDE_PYTHONPATH_IN_RUNTIME_ENV = _bool("SKYRL_INCLUDE_PYTHONPATH_IN_RUNTIME_ENV")
# knobs of this implementation
SKYRL_B200_NO_AUTOBUILD = _bool("SKYRL_B200_NO_AUTOBUILD")
SKYRL_B200_PEER_WAIT_S = float(os.environ.get("SKYRL_B200_PEER_WAIT_S", "10"))
SKYRL_B200_DISABLE_PEER = _bool("SKYRL_B200_DISABLE_PEER")
