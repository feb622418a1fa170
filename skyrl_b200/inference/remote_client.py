"""HTTP client for remote inference servers (reference: skyrl/backends/skyrl_train/inference_servers/
remote_inference_client.py:171-1450).

Data plane: one ``POST /inference/v1/generate`` per prompt through the router URL (or directly, round-robin /
session-hashed) carrying ``X-Session-ID`` so that the router can pin a session to one replica; bounded
concurrency; retries with backoff; an ``abort``-paused request is transparently re-submitted with the tokens
accumulated so far.  Control plane: fan-out of pause / resume / sleep / wake_up / reset_prefix_cache / weight
verbs to every server.
"""

from __future__ import annotations

import asyncio
from typing import Any, Dict, List, Optional

import aiohttp

from ..env_vars import SKYRL_GENERATE_CONCURRENCY_PER_ENGINE
from . import wire
from .base import InferenceEngineInput, InferenceEngineInterface, InferenceEngineOutput

_DATA_PLANE_RETRIES = 30


class RemoteInferenceClient(InferenceEngineInterface):
    def __init__(self, server_urls: List[str], router_url: Optional[str] = None, model_name: str = "policy",
                 tokenizer=None, retries: int = _DATA_PLANE_RETRIES, backoff_s: float = 0.2, timeout_s: float = 3600.0):
        if not server_urls:
            raise ValueError("at least one server url is required")
        self.server_urls = [u.rstrip("/") for u in server_urls]
        self.router_url = router_url.rstrip("/") if router_url else None
        self.model_name = model_name
        self.tokenizer = tokenizer
        self.retries, self.backoff_s, self.timeout_s = retries, backoff_s, timeout_s
        self.weight_version = 0
        self._rr = 0
        self._session: Optional[aiohttp.ClientSession] = None
        self._sem: Optional[asyncio.Semaphore] = None
        self._loop = None

    # pickling drops the live session (workers re-create it lazily)
    def __getstate__(self):
        d = dict(self.__dict__)
        d["_session"] = d["_sem"] = d["_loop"] = None
        return d

    async def _http(self) -> aiohttp.ClientSession:
        loop = asyncio.get_running_loop()
        if self._session is None or self._session.closed or self._loop is not loop:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s),
                                                  connector=aiohttp.TCPConnector(limit=0))
            self._sem = asyncio.Semaphore(SKYRL_GENERATE_CONCURRENCY_PER_ENGINE * len(self.server_urls))
            self._loop = loop
        return self._session

    def _target(self, session_id: Any) -> str:
        if self.router_url:
            return self.router_url
        if session_id is None:
            self._rr = (self._rr + 1) % len(self.server_urls)
            return self.server_urls[self._rr]
        return self.server_urls[hash(str(session_id)) % len(self.server_urls)]

    async def _post(self, url: str, json_body: Any = None, params: Optional[dict] = None, headers: Optional[dict] = None,
                    retries: Optional[int] = None) -> Any:
        http = await self._http()
        last: Optional[BaseException] = None
        n = self.retries if retries is None else retries
        for attempt in range(n + 1):
            try:
                async with http.post(url, json=json_body, params=params, headers=headers) as r:
                    if r.status >= 500:
                        raise aiohttp.ClientResponseError(r.request_info, r.history, status=r.status, message=await r.text())
                    if r.status >= 400:
                        raise ValueError(f"{url} -> HTTP {r.status}: {await r.text()}")
                    return await r.json()
            except (aiohttp.ClientConnectionError, aiohttp.ClientResponseError, asyncio.TimeoutError) as e:
                last = e
                await asyncio.sleep(min(5.0, self.backoff_s * (2 ** min(attempt, 5))))
        raise ConnectionError(f"{url}: no success after {n + 1} attempts: {last}")

    # ------------------------------------------------------------------ data plane
    async def _generate_single(self, ids: List[int], sp: Dict[str, Any], session_id: Any, salt: Optional[str]):
        await self._http()
        acc_ids: List[int] = []
        acc_lps: List[float] = []
        budget = sp.get("max_generate_length", sp.get("max_tokens"))
        async with self._sem:
            while True:
                body = {"sampling_params": dict(sp), "model": self.model_name, "token_ids": list(ids) + acc_ids}
                if budget is not None and acc_ids:
                    body["sampling_params"]["max_generate_length"] = max(1, budget - len(acc_ids))
                    body["sampling_params"].pop("max_tokens", None)
                if salt:
                    body["cache_salt"] = salt
                headers = {"X-Session-ID": str(session_id)} if session_id is not None else None
                r = await self._post(self._target(session_id) + "/inference/v1/generate", body, headers=headers)
                c = r["choices"][0]
                acc_ids += list(c["token_ids"])
                lp = c.get("logprobs")
                acc_lps += [x["logprob"] for x in lp["content"]] if lp else []
                # a continuation re-submits everything generated so far, so the newest table covers the whole sequence
                routes = wire.decode_packed_routed_experts(c["routed_experts"]) if c.get("routed_experts") else None
                self.weight_version = max(self.weight_version, int(r.get("weight_version", 0)))
                if c["finish_reason"] != "abort":
                    return acc_ids, acc_lps, c["finish_reason"], routes
                if budget is not None and len(acc_ids) >= budget:
                    return acc_ids, acc_lps, "length", routes
                await asyncio.sleep(self.backoff_s)  # server was paused with mode=abort: continue from what we have

    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput:
        ids = input_batch.get("prompt_token_ids")
        if ids is None:
            raise ValueError("RemoteInferenceClient.generate needs prompt_token_ids (token-in / token-out)")
        sp = dict(input_batch.get("sampling_params") or {})
        if sp.get("n", 1) != 1:
            raise ValueError("n > 1 is not supported; repeat the prompt instead")
        sessions = input_batch.get("session_ids") or [None] * len(ids)
        salt = input_batch.get("cache_salt")
        res = await asyncio.gather(*[self._generate_single(list(p), sp, s, salt) for p, s in zip(ids, sessions)])
        texts = [self.tokenizer.decode(r[0], skip_special_tokens=True) if self.tokenizer is not None else "" for r in res]
        return InferenceEngineOutput(responses=texts, response_ids=[r[0] for r in res], stop_reasons=[r[2] for r in res],
                                     response_logprobs=[r[1] for r in res] if all(len(r[1]) == len(r[0]) for r in res) else None,
                                     prompt_logprobs=None,
                                     rollout_expert_indices=[r[3] for r in res] if any(r[3] is not None for r in res) else None)

    async def chat_completion(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        return await self._post(self._target(request_payload.get("session_id")) + "/v1/chat/completions",
                                request_payload.get("json", request_payload))

    async def completion(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        return await self._post(self._target(request_payload.get("session_id")) + "/v1/completions",
                                request_payload.get("json", request_payload))

    # ------------------------------------------------------------------ control plane (fan-out)
    async def _fanout(self, path: str, json_body: Any = None, params: Optional[dict] = None) -> List[Any]:
        return list(await asyncio.gather(*[self._post(u + path, json_body, params=params, retries=3)
                                           for u in self.server_urls]))

    async def pause(self, mode: str = "keep", clear_cache: bool = False) -> None:
        await self._fanout("/pause", params={"mode": mode, "clear_cache": str(clear_cache).lower()})

    async def resume(self) -> None:
        await self._fanout("/resume")

    async def sleep(self, level: int = 2, tags: Optional[List[str]] = None) -> None:
        p = {"level": level}
        if tags:
            p["tags"] = ",".join(tags)
        await self._fanout("/sleep", params=p)

    async def wake_up(self, tags: Optional[List[str]] = None) -> None:
        await self._fanout("/wake_up", params={"tags": ",".join(tags)} if tags else None)

    async def reset_prefix_cache(self, reset_running_requests: bool = False) -> None:
        await self._fanout("/reset_prefix_cache", params={"reset_running_requests": str(reset_running_requests).lower()})

    async def init_weight_update_communicator(self, init_info: Any) -> None:
        await self._fanout("/init_weight_transfer_engine", init_info)

    async def update_named_weights(self, request: Any) -> None:
        body = request if isinstance(request, dict) else getattr(request, "__dict__", {"request": request})
        res = await self._fanout("/update_weights", body)
        self.weight_version = max([self.weight_version] + [int(r.get("weight_version", 0)) for r in res])

    async def fetch_weights(self, payload: Dict[str, Any]) -> None:
        res = await self._fanout("/fetch_weights", payload)
        self.weight_version = max([self.weight_version] + [int(r.get("weight_version", 0)) for r in res])

    async def collective_rpc(self, method: str, **kwargs) -> List[Any]:
        return await self._fanout("/collective_rpc", {"method": method, "kwargs": kwargs})

    async def sleep_for_weight_sync(self, offload_kv: bool = True) -> None:
        await self.collective_rpc("skyrl_sleep_for_weight_sync", offload_kv=offload_kv)

    async def wake_for_weight_sync(self, tags: Optional[List[str]] = None) -> None:
        await self.collective_rpc("skyrl_wake_for_weight_sync", tags=tags)

    async def load_lora_adapter(self, lora_path: str, lora_name: str = "skyrl-lora") -> None:
        await self._fanout("/skyrl/v1/load_lora_adapter", {"lora_path": lora_path, "lora_name": lora_name})

    def get_endpoint_url(self) -> str:
        """Where OpenAI-protocol clients should connect: the router if there is one, else the first server."""
        return self.router_url or self.server_urls[0]

    async def unload_lora_adapter(self, lora_name: str = "skyrl-lora") -> None:
        await self._fanout("/skyrl/v1/unload_lora_adapter", {"lora_name": lora_name})

    async def pause_generation(self, clear_cache: bool = False) -> None:
        """Freeze in-flight requests with their KV cache (``pause`` in keep mode)."""
        await self.pause("keep", clear_cache)

    async def resume_generation(self) -> None:
        await self.resume()

    # ------------------------------------------------------------------ Tinker-style sampling and text utilities
    async def sample(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        """``{"json": {prompt, num_samples, sampling_params, include_prompt_logprobs | prompt_logprobs, session_id}}``
        -> ``{"type": "sample", "sequences": [{tokens, logprobs, stop_reason}], "prompt_logprobs",
        "topk_prompt_logprobs"}`` through ``/inference/v1/generate`` (reference: remote_inference_client.py:620-728).
        ``prompt`` is a Tinker model input (``{"chunks": [{"tokens": [...]}]}``) or a plain id list; one request per
        sample.  The engine scores each prompt token only, so ``topk_prompt_logprobs`` is always ``None``."""
        body = dict(request_payload.get("json", request_payload))
        session_id = body.get("session_id") or request_payload.get("session_id")
        prompt = body.get("prompt") or {}
        if isinstance(prompt, dict):
            ids: List[int] = []
            for ch in prompt.get("chunks", []):
                if "tokens" not in ch:
                    raise ValueError("sample: only token chunks are supported by this client")
                ids.extend(int(t) for t in ch["tokens"])
        else:
            ids = [int(t) for t in prompt]
        n = max(1, int(body.get("num_samples", 1)))
        tp = body.get("sampling_params") or {}
        want_plp = bool(body.get("include_prompt_logprobs", body.get("prompt_logprobs", False)))
        sp: Dict[str, Any] = {}
        for src, dst in (("max_tokens", "max_tokens"), ("temperature", "temperature"), ("top_p", "top_p"),
                         ("top_k", "top_k"), ("stop", "stop"), ("seed", "seed")):
            if tp.get(src) is not None:
                sp[dst] = tp[src]
        if want_plp:
            sp["prompt_logprobs"] = True
        await self._http()
        headers = {"X-Session-ID": str(session_id)} if session_id else None
        url = self._target(session_id) + "/inference/v1/generate"

        async def one():
            async with self._sem:
                return await self._post(url, {"sampling_params": sp, "model": body.get("model", self.model_name),
                                              "token_ids": ids}, headers=headers)

        res = await asyncio.gather(*[one() for _ in range(n)])
        seqs, plp = [], None
        for r in res:
            c = r["choices"][0]
            lp = c.get("logprobs")
            seqs.append({"tokens": list(c["token_ids"]), "logprobs": [x["logprob"] for x in lp["content"]] if lp else None,
                         "stop_reason": c.get("finish_reason")})
            if want_plp and plp is None:
                plp = c.get("prompt_logprobs")
        return {"type": "sample", "sequences": seqs, "prompt_logprobs": plp, "topk_prompt_logprobs": None}

    async def tokenize(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        return await self._post(self.server_urls[0] + "/tokenize", request_payload.get("json", request_payload))

    async def detokenize(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        return await self._post(self.server_urls[0] + "/detokenize", request_payload.get("json", request_payload))

    async def render_chat_completion(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        """Messages -> token ids without generating (the ``/tokenize`` endpoint applied to ``messages``)."""
        body = dict(request_payload.get("json", request_payload))
        out = await self._post(self.server_urls[0] + "/tokenize", {"messages": body["messages"],
                                                                  "add_generation_prompt": body.get("add_generation_prompt", True)})
        return {"token_ids": out.get("tokens", out.get("token_ids")), "count": out.get("count")}

    async def __aenter__(self) -> "RemoteInferenceClient":
        await self._http()
        return self

    async def __aexit__(self, exc_type, exc, tb) -> None:
        await self.teardown()

    async def aclose(self) -> None:
        await self.teardown()

    async def finish_session(self, session_id: Any) -> None:
        try:
            await self._post(self._target(session_id) + "/finish_session", {"session_id": str(session_id)}, retries=0)
        except Exception:
            pass

    async def health(self) -> bool:
        http = await self._http()
        try:
            for u in self.server_urls:
                async with http.get(u + "/health") as r:
                    if r.status != 200:
                        return False
            return True
        except aiohttp.ClientError:
            return False

    def increment_weight_version(self) -> int:
        self.weight_version += 1
        return self.weight_version

    def get_world_size(self) -> int:
        return len(self.server_urls)

    async def teardown(self) -> None:
        if self._session is not None and not self._session.closed:
            await self._session.close()
