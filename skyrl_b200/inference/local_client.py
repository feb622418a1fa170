"""In-process inference client: drives one or more ``LLMEngine`` replicas living in this process.

This is the colocated data plane: no HTTP, no serialisation -- ``generate`` hands token ids to the
engine and awaits a future that the stepping loop resolves.  Requests from many concurrent
``agent_loop`` coroutines are batched by the engine's continuous batching, sessions are pinned to
a replica by consistent hashing (C++ ring) so multi-turn prefixes hit that replica's prefix cache
(the reference routes on ``X-Session-ID`` for the same reason, remote_inference_client.py:484-503).
"""

from __future__ import annotations

import asyncio
import ctypes
import threading
from typing import Any, Dict, List, Optional, Sequence

from ..engine.llm_engine import LLMEngine, RequestOutput, SamplingParams
from ..ops import _lib
from .base import InferenceEngineInput, InferenceEngineInterface, InferenceEngineOutput
from ..utils.tokenizer import chat_template_ids


class _Ring:
    def __init__(self, n: int, vnodes: int = 64):
        rt = _lib.runtime()
        rt.sbrt_ring_create.restype = ctypes.c_void_p
        rt.sbrt_ring_create.argtypes = [ctypes.c_int]
        rt.sbrt_ring_add.argtypes = [ctypes.c_void_p, ctypes.c_int]
        rt.sbrt_ring_remove.argtypes = [ctypes.c_void_p, ctypes.c_int]
        rt.sbrt_ring_lookup.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
        rt.sbrt_ring_destroy.argtypes = [ctypes.c_void_p]
        self.rt = rt
        self.h = rt.sbrt_ring_create(vnodes)
        for i in range(n):
            rt.sbrt_ring_add(self.h, i)

    def lookup(self, key: str) -> int:
        b = key.encode()
        return int(self.rt.sbrt_ring_lookup(self.h, b, len(b)))

    def __del__(self):
        try:
            self.rt.sbrt_ring_destroy(self.h)
        except Exception:
            pass


class LocalInferenceClient(InferenceEngineInterface):
    def __init__(self, engines: Sequence[LLMEngine], tokenizer=None, model_name: str = "policy"):
        self.engines = list(engines)
        self.tokenizer = tokenizer
        self.model_name = model_name
        self.ring = _Ring(len(self.engines))
        self._rr = 0
        self._futures: List[Dict[str, asyncio.Future]] = [dict() for _ in self.engines]
        self._loops: List[Optional[asyncio.Task]] = [None] * len(self.engines)
        self._locks = [threading.Lock() for _ in self.engines]
        self._next = 0
        self.weight_version = 0

    def get_endpoint_url(self) -> str:
        """Base URL of an OpenAI-compatible HTTP server in front of these engines (``/v1/chat/completions``,
        ``/v1/completions``, ``/inference/v1/generate``, ``/tokenize`` ...), started in a background thread of this
        process on first use.  It lets agent scaffolds that only speak the OpenAI protocol roll out against the
        colocated engines (reference: ``RemoteInferenceClient.get_endpoint_url``; there the servers always exist).
        All requests must then come through the endpoint: the engine loop lives in the server's event loop."""
        if getattr(self, "_endpoint", None) is None:
            from .server import ServerThread, build_app

            self._endpoint = ServerThread(build_app(self, model_name=self.model_name)).start()
        return self._endpoint.url

    def close_endpoint(self) -> None:
        ep = getattr(self, "_endpoint", None)
        if ep is not None:
            ep.stop()
            self._endpoint = None

    # ------------------------------------------------------------------ data plane
    def _route(self, session_id: Any) -> int:
        if session_id is None or len(self.engines) == 1:
            self._rr = (self._rr + 1) % len(self.engines)
            return self._rr
        return self.ring.lookup(str(session_id))

    def _decode(self, ids: List[int]) -> str:
        if self.tokenizer is None:
            return ""
        return self.tokenizer.decode(ids, skip_special_tokens=True)

    async def _engine_loop(self, k: int) -> None:
        eng = self.engines[k]
        futs = self._futures[k]
        try:
            while futs:
                if eng.paused or eng.asleep:
                    await asyncio.sleep(0.002)
                    if not getattr(eng, "lockstep", False):
                        continue  # a tensor-parallel group keeps stepping: the step carries the resume to its ranks

                def _step():
                    with self._locks[k]:
                        return eng.step()

                outs = await asyncio.to_thread(_step)
                for o in outs:
                    f = futs.pop(o.request_id, None)
                    if f is not None and not f.done():
                        f.set_result(o)
                if not outs:
                    await asyncio.sleep(0)
        finally:
            self._loops[k] = None

    async def _submit(self, k: int, prompt: List[int], sp: SamplingParams, salt: Optional[str]) -> RequestOutput:
        rid = f"req-{self._next}"
        self._next += 1
        fut: asyncio.Future = asyncio.get_running_loop().create_future()
        self._futures[k][rid] = fut
        with self._locks[k]:
            self.engines[k].add_request(rid, prompt, sp, salt)
        if self._loops[k] is None:
            self._loops[k] = asyncio.create_task(self._engine_loop(k))
        return await fut

    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput:
        ids = input_batch.get("prompt_token_ids")
        if ids is None:
            prompts = input_batch.get("prompts")
            assert prompts is not None and self.tokenizer is not None, "need prompt_token_ids or (prompts + tokenizer)"
            ids = [chat_template_ids(self.tokenizer, p, add_generation_prompt=True) for p in prompts]
        sp = SamplingParams.from_dict(input_batch.get("sampling_params"))
        sessions = input_batch.get("session_ids") or [None] * len(ids)
        salt = input_batch.get("cache_salt")
        outs = await asyncio.gather(*[self._submit(self._route(s), list(p), sp, salt) for p, s in zip(ids, sessions)])
        return self._to_output(outs)

    def generate_sync(self, prompt_token_ids: Sequence[Sequence[int]], sampling_params,
                      cache_salt: Optional[str] = None) -> InferenceEngineOutput:
        """Blocking batched generation (single-turn batched rollouts; no event loop required)."""
        n = len(self.engines)
        sps = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * len(prompt_token_ids)
        sps = [s if isinstance(s, SamplingParams) else SamplingParams.from_dict(s) for s in sps]
        parts: List[List[int]] = [[] for _ in range(n)]
        for i in range(len(prompt_token_ids)):
            parts[i % n].append(i)
        results: List[Optional[RequestOutput]] = [None] * len(prompt_token_ids)
        for k, idxs in enumerate(parts):
            if not idxs:
                continue
            with self._locks[k]:
                outs = self.engines[k].generate([prompt_token_ids[i] for i in idxs], [sps[i] for i in idxs],
                                                cache_salt=cache_salt)
            for i, o in zip(idxs, outs):
                results[i] = o
        return self._to_output(results)

    def _to_output(self, outs: Sequence[RequestOutput]) -> InferenceEngineOutput:
        return InferenceEngineOutput(
            responses=[self._decode(o.token_ids) for o in outs], response_ids=[o.token_ids for o in outs],
            stop_reasons=[o.finish_reason for o in outs], response_logprobs=[o.logprobs for o in outs],
            prompt_logprobs=[o.prompt_logprobs for o in outs] if any(o.prompt_logprobs for o in outs) else None,
            rollout_expert_indices=([o.routed_experts.numpy() if o.routed_experts is not None else None for o in outs]
                                    if any(o.routed_experts is not None for o in outs) else None),
            weight_versions=[o.weight_version for o in outs])

    # ------------------------------------------------------------------ control plane
    async def pause(self, mode: str = "keep", clear_cache: bool = False) -> None:
        for k, e in enumerate(self.engines):
            with self._locks[k]:
                outs = e.pause(mode, clear_cache)
            for o in outs:
                f = self._futures[k].pop(o.request_id, None)
                if f is not None and not f.done():
                    f.set_result(o)

    async def resume(self) -> None:
        for e in self.engines:
            e.resume()

    async def sleep(self, level: int = 2, tags: Optional[List[str]] = None) -> None:
        for k, e in enumerate(self.engines):
            with self._locks[k]:
                e.sleep(level, tags)

    async def wake_up(self, tags: Optional[List[str]] = None) -> None:
        for k, e in enumerate(self.engines):
            with self._locks[k]:
                e.wake_up(tags)

    async def reset_prefix_cache(self, reset_running_requests: bool = False) -> None:
        for k, e in enumerate(self.engines):
            with self._locks[k]:
                e.reset_prefix_cache(reset_running_requests)

    def increment_weight_version(self) -> int:
        self.weight_version += 1
        for e in self.engines:
            e.on_weights_updated(clear_kv=True)
        return self.weight_version

    def get_world_size(self) -> int:
        return len(self.engines)

    def dp_size(self) -> int:
        return len(self.engines)

    def metrics(self) -> Dict[str, float]:
        agg: Dict[str, float] = {}
        for e in self.engines:
            for k, v in e.metrics().items():
                agg[k] = agg.get(k, 0.0) + float(v)
        return agg
