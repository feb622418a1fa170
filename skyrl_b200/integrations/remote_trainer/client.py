"""Blocking client of a Tinker-compatible training service (the verbs of ``skyrl_b200/tinker/api.py``)."""

from __future__ import annotations

import time
from typing import Any, Dict, List, Optional


class ServiceError(RuntimeError):
    pass


class TrainingServiceClient:
    """``transport`` needs ``post(path, json=...)`` and ``get(path)`` returning objects with ``status_code``, ``json()``
    and ``text`` -- a ``requests.Session`` bound to a base URL (the default) or FastAPI's ``TestClient``."""

    def __init__(self, base_url: str = "", transport: Any = None, poll_interval: float = 0.05, timeout: float = 600.0):
        if transport is None:
            import requests

            class _Http:
                def __init__(self, base):
                    self.base, self.s = base.rstrip("/"), requests.Session()

                def post(self, path, json=None):
                    return self.s.post(self.base + path, json=json, timeout=timeout)

                def get(self, path):
                    return self.s.get(self.base + path, timeout=timeout)

            transport = _Http(base_url)
        self.t = transport
        self.poll_interval, self.timeout = poll_interval, timeout
        self.session_id: Optional[str] = None
        self.model_id: Optional[str] = None
        self.sampling_session_id: Optional[str] = None
        self._seq = 0          # per-model request order (the service executes a model's requests in this order)
        self._sampler_seq = 0

    # ------------------------------------------------------------------ plumbing
    def _post(self, path: str, body: Dict[str, Any]) -> Dict[str, Any]:
        r = self.t.post(path, json=body)
        if r.status_code != 200:
            raise ServiceError(f"{path}: HTTP {r.status_code}: {r.text[:500]}")
        return r.json()

    def wait(self, fut: Dict[str, Any]) -> Dict[str, Any]:
        """Result of a future; the service may answer "try again" while the request is still queued."""
        t0 = time.time()
        while True:
            r = self.t.post("/api/v1/retrieve_future", json={"request_id": fut["request_id"]})
            if r.status_code == 200:
                out = r.json()
                if out.get("type") != "try_again":
                    if out.get("error"):
                        raise ServiceError(str(out["error"]))
                    return out
            elif r.status_code not in (408, 425):
                raise ServiceError(f"retrieve_future: HTTP {r.status_code}: {r.text[:500]}")
            if time.time() - t0 > self.timeout:
                raise ServiceError(f"request {fut['request_id']} did not finish within {self.timeout} s")
            time.sleep(self.poll_interval)

    def _next_seq(self) -> int:
        self._seq += 1
        return self._seq

    # ------------------------------------------------------------------ verbs
    def connect(self, base_model: str, lora_rank: int = 0) -> str:
        self.session_id = self._post("/api/v1/create_session", {"tags": ["skyrl_b200"], "sdk_version": "remote_trainer"})["session_id"]
        r = self._post("/api/v1/create_model", {"session_id": self.session_id, "base_model": base_model,
                                               "lora_config": {"rank": int(lora_rank)}})
        self.model_id = r["model_id"]
        self.wait(r)
        return self.model_id

    def forward(self, datums: List[dict], loss_fn: str = "cross_entropy") -> Dict[str, Any]:
        return self.wait(self._post("/api/v1/forward", {"model_id": self.model_id, "seq_id": self._next_seq(),
                                                        "forward_input": {"data": datums, "loss_fn": loss_fn}}))

    def forward_backward_async(self, datums: List[dict], loss_fn: str, loss_fn_config: Optional[dict] = None) -> Dict[str, Any]:
        body = {"data": datums, "loss_fn": loss_fn}
        if loss_fn_config:
            body["loss_fn_config"] = loss_fn_config
        return self._post("/api/v1/forward_backward", {"model_id": self.model_id, "seq_id": self._next_seq(),
                                                       "forward_backward_input": body})

    def optim_step_async(self, learning_rate: float, **adam) -> Dict[str, Any]:
        return self._post("/api/v1/optim_step", {"model_id": self.model_id, "seq_id": self._next_seq(),
                                                 "adam_params": {"learning_rate": float(learning_rate), **adam}})

    def save_weights_for_sampler(self) -> str:
        self._sampler_seq += 1
        out = self.wait(self._post("/api/v1/save_weights_for_sampler", {"model_id": self.model_id, "seq_id": self._next_seq(),
                                                                       "sampling_session_seq_id": self._sampler_seq}))
        self.sampling_session_id = out["sampling_session_id"]
        return self.sampling_session_id

    def sample_async(self, prompt_tokens: List[int], num_samples: int, sampling_params: Dict[str, Any]) -> Dict[str, Any]:
        if self.sampling_session_id is None:
            self.save_weights_for_sampler()
        return self._post("/api/v1/asample", {"sampling_session_id": self.sampling_session_id, "num_samples": int(num_samples),
                                              "prompt": {"chunks": [{"type": "encoded_text", "tokens": list(prompt_tokens)}]},
                                              "sampling_params": sampling_params})

    def save_state(self, name: str) -> str:
        return self.wait(self._post("/api/v1/save_weights", {"model_id": self.model_id, "seq_id": self._next_seq(),
                                                             "path": name}))["path"]

    def load_state(self, path: str) -> None:
        self.wait(self._post("/api/v1/load_weights", {"model_id": self.model_id, "seq_id": self._next_seq(), "path": path}))
