"""HTTP facade of the generation engine (FastAPI), for disaggregated deployments and external clients.

Endpoint set and payload shapes follow the reference server actor and client
(skyrl/backends/skyrl_train/inference_servers/vllm_server_actor.py:340-476, remote_inference_client.py:484-525):
data plane ``/inference/v1/generate`` (token-in / token-out), ``/skyrl/v1/generate``, ``/v1/completions``,
``/v1/chat/completions``, ``/tokenize``, ``/detokenize``; control plane ``/health``, ``/pause``, ``/resume``, ``/sleep``,
``/wake_up``, ``/reset_prefix_cache``, ``/get_world_size``, ``/init_weight_transfer_engine``, ``/collective_rpc``,
``/update_weights``, ``/fetch_weights``, ``/skyrl/v1/load_lora_adapter``, ``/finish_session``, ``/metrics``.
In colocated runs none of this is on the hot path (the trainer talks to the engine in-process).
"""

from __future__ import annotations

from fastapi import FastAPI, HTTPException, Request  # module level: needed to resolve route annotations
from fastapi.responses import JSONResponse, PlainTextResponse

import asyncio
import base64
import math
import threading
import time
from typing import Any, Dict, List, Optional

from . import wire
from .local_client import LocalInferenceClient
from ..utils.tokenizer import chat_template_ids

MISSING_LOGPROB = -9999.0


def clamp_logprobs(lps: Optional[List[Optional[float]]]) -> List[float]:
    """Missing or non-finite log-probabilities are floored (reference: generate_wire.py:22-56)."""
    out = []
    for x in lps or []:
        out.append(float(x) if (x is not None and math.isfinite(x)) else MISSING_LOGPROB)
    return out


def build_app(client: LocalInferenceClient, model_name: str = "policy", weight_loader=None):
    """``weight_loader(kind, payload) -> dict`` handles weight-update verbs (peer / broadcast / delta)."""
    app = FastAPI(title="skyrl_b200 inference server")
    state = {"loras": {}, "started": time.time(), "sessions": set()}

    def _tok():
        if client.tokenizer is None:
            raise HTTPException(400, "this server has no tokenizer; use token-in / token-out endpoints")
        return client.tokenizer

    @app.get("/health")
    async def health():
        return {"status": "ok", "model": model_name, "uptime_s": time.time() - state["started"]}

    @app.get("/get_world_size")
    async def world_size():
        return {"world_size": client.get_world_size()}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model"}] +
                [{"id": n, "object": "model", "parent": model_name} for n in state["loras"]]}

    async def _generate(body: Dict[str, Any], session: Optional[str]):
        ids = body.get("token_ids") or body.get("prompt_token_ids")
        if ids is None:
            raise HTTPException(400, "token_ids is required")
        if ids and isinstance(ids[0], int):
            ids = [ids]
        sp = dict(body.get("sampling_params") or {})
        if sp.get("n", 1) != 1:
            raise HTTPException(400, "n > 1 is not supported; send one request per sample")
        out = await client.generate({"prompt_token_ids": ids, "sampling_params": sp, "session_ids": [session] * len(ids),
                                     "cache_salt": body.get("cache_salt")})
        choices = []
        for i in range(len(ids)):
            lps = clamp_logprobs(out["response_logprobs"][i] if out.get("response_logprobs") else None)
            choices.append({"index": i, "token_ids": out["response_ids"][i], "finish_reason": out["stop_reasons"][i],
                            "text": out["responses"][i],
                            "logprobs": {"content": [{"logprob": lp} for lp in lps]} if lps else None})
            plps = out.get("prompt_logprobs")
            if plps and plps[i] is not None:
                choices[-1]["prompt_logprobs"] = [None if x is None else float(x) for x in plps[i]]
            routes = (out.get("rollout_expert_indices") or [None] * len(ids))[i]
            if routes is not None:  # mixture-of-experts engine started with return_routed_experts
                choices[-1]["routed_experts"] = wire.pack_routed_experts(routes)
        return {"id": f"gen-{int(time.time() * 1e6)}", "model": body.get("model", model_name), "choices": choices,
                "weight_version": client.weight_version}

    @app.post("/inference/v1/generate")
    async def generate(request: Request):
        return await _generate(await request.json(), request.headers.get("X-Session-ID"))

    @app.post("/skyrl/v1/generate")
    async def skyrl_generate(request: Request):
        return await _generate(await request.json(), request.headers.get("X-Session-ID"))

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await request.json()
        prompt = body.get("prompt")
        ids = prompt if (isinstance(prompt, list) and prompt and isinstance(prompt[0], int)) else _tok().encode(str(prompt))
        sp = {k: body[k] for k in ("temperature", "top_p", "top_k", "min_p", "stop") if k in body}
        sp["max_generate_length"] = body.get("max_tokens", 16)
        r = await _generate({"token_ids": ids, "sampling_params": sp}, request.headers.get("X-Session-ID"))
        c = r["choices"][0]
        return {"id": r["id"], "object": "text_completion", "model": model_name,
                "choices": [{"index": 0, "text": c["text"], "finish_reason": c["finish_reason"], "token_ids": c["token_ids"],
                             "logprobs": c["logprobs"]}],
                "prompt_token_ids": list(ids), "usage": {"prompt_tokens": len(ids), "completion_tokens": len(c["token_ids"])}}

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        body = await request.json()
        ids = chat_template_ids(_tok(), body["messages"], add_generation_prompt=True)
        sp = {k: body[k] for k in ("temperature", "top_p", "top_k", "min_p", "stop") if k in body}
        sp["max_generate_length"] = body.get("max_tokens") or body.get("max_completion_tokens") or 256
        r = await _generate({"token_ids": list(ids), "sampling_params": sp}, request.headers.get("X-Session-ID"))
        c = r["choices"][0]
        return {"id": r["id"], "object": "chat.completion", "model": model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": c["text"]},
                             "finish_reason": c["finish_reason"], "token_ids": c["token_ids"], "logprobs": c["logprobs"]}],
                "prompt_token_ids": list(ids), "usage": {"prompt_tokens": len(ids), "completion_tokens": len(c["token_ids"])}}

    @app.post("/tokenize")
    async def tokenize(request: Request):
        body = await request.json()
        if "messages" in body:
            ids = chat_template_ids(_tok(), body["messages"], add_generation_prompt=body.get("add_generation_prompt", True))
        else:
            ids = _tok().encode(body.get("prompt", ""))
        return {"tokens": list(ids), "count": len(ids)}

    @app.post("/detokenize")
    async def detokenize(request: Request):
        body = await request.json()
        return {"prompt": _tok().decode(body["tokens"], skip_special_tokens=body.get("skip_special_tokens", True))}

    @app.post("/pause")
    async def pause(mode: str = "keep", clear_cache: bool = False):
        if mode not in ("keep", "abort", "wait"):
            raise HTTPException(400, f"unknown pause mode '{mode}'")
        await client.pause(mode, clear_cache)
        return {"status": "paused", "mode": mode}

    @app.post("/resume")
    async def resume():
        await client.resume()
        return {"status": "running"}

    @app.post("/sleep")
    async def sleep(level: int = 1, tags: Optional[str] = None):
        await client.sleep(level, tags.split(",") if tags else None)
        return {"status": "sleeping", "level": level}

    @app.post("/wake_up")
    async def wake_up(tags: Optional[str] = None):
        await client.wake_up(tags.split(",") if tags else None)
        return {"status": "awake"}

    @app.post("/reset_prefix_cache")
    async def reset_prefix_cache(reset_running_requests: bool = False):
        await client.reset_prefix_cache(reset_running_requests)
        return {"status": "ok"}

    @app.post("/finish_session")
    async def finish_session(request: Request):
        body = await request.json()
        state["sessions"].discard(body.get("session_id"))
        return {"status": "ok"}

    async def _weights(kind: str, request: Request):
        if weight_loader is None:
            raise HTTPException(501, "this server was started without a weight loader")
        body = await request.json()
        res = await asyncio.to_thread(weight_loader, kind, body)
        if kind in ("update_weights", "fetch_weights", "finish_weight_update"):
            client.increment_weight_version()
        return {"status": "ok", "weight_version": client.weight_version, **(res or {})}

    @app.post("/init_weight_transfer_engine")
    async def init_wte(request: Request):
        return await _weights("init", request)

    @app.post("/update_weights")
    async def update_weights(request: Request):
        return await _weights("update_weights", request)

    @app.post("/fetch_weights")
    async def fetch_weights(request: Request):
        return await _weights("fetch_weights", request)

    @app.post("/collective_rpc")
    async def collective_rpc(request: Request):
        body = await request.json()
        method = body.get("method")
        if method in ("skyrl_sleep_for_weight_sync", "sleep_for_weight_sync"):
            await client.sleep(1, ["kv_cache"] if body.get("kwargs", {}).get("offload_kv", True) else [])
            return {"status": "ok"}
        if method in ("skyrl_wake_for_weight_sync", "wake_for_weight_sync"):
            await client.wake_up(body.get("kwargs", {}).get("tags"))
            return {"status": "ok"}
        if method in ("start_weight_update", "finish_weight_update"):
            return await _weights(method, request)
        raise HTTPException(400, f"unknown collective_rpc method '{method}'")

    @app.post("/skyrl/v1/load_lora_adapter")
    async def load_lora(request: Request):
        body = await request.json()
        if weight_loader is None:
            raise HTTPException(501, "this server was started without a weight loader")
        await asyncio.to_thread(weight_loader, "load_lora", body)
        state["loras"][body.get("lora_name", "skyrl-lora")] = body.get("lora_path")
        client.increment_weight_version()
        return {"status": "ok"}

    @app.post("/skyrl/v1/unload_lora_adapter")
    async def unload_lora(request: Request):
        body = await request.json()
        state["loras"].pop(body.get("lora_name", "skyrl-lora"), None)
        return {"status": "ok"}

    @app.get("/metrics")
    async def metrics():
        m = client.metrics()
        lines = [f"skyrl_b200_{k} {float(v)}" for k, v in sorted(m.items())]
        return PlainTextResponse("\n".join(lines) + "\n")

    return app


class ServerThread:
    """Run the app with uvicorn in a background thread (tests, single-process deployments)."""

    def __init__(self, app, host: str = "127.0.0.1", port: int = 0):
        import socket

        import uvicorn

        if port == 0:
            s = socket.socket()
            s.bind((host, 0))
            port = s.getsockname()[1]
            s.close()
        self.host, self.port = host, port
        self.server = uvicorn.Server(uvicorn.Config(app, host=host, port=port, log_level="warning"))
        self.thread = threading.Thread(target=self.server.run, daemon=True)

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def start(self, timeout: float = 20.0) -> "ServerThread":
        self.thread.start()
        t0 = time.time()
        while not self.server.started:
            if time.time() - t0 > timeout:
                raise TimeoutError("inference server did not start")
            if not self.thread.is_alive():
                raise RuntimeError("inference server crashed during start-up")
            time.sleep(0.02)
        return self

    def stop(self) -> None:
        self.server.should_exit = True
        self.thread.join(timeout=10)
