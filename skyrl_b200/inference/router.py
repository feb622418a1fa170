"""Session-affine HTTP router in front of several inference servers: consistent hashing on ``X-Session-ID``
(C++ hash ring with virtual nodes, ``csrc/runtime/runtime.cpp``) or ``sticky_least_loaded`` (a new session goes to
the server with the fewest open sessions and stays there until ``/finish_session`` closes it), round-robin for
requests without a session, health-based ejection, optional prefill/decode URL lists.  Role of the Rust ``vllm-router`` wheel the reference
launches (skyrl/backends/skyrl_train/inference_servers/vllm_router.py:47-175)."""

from __future__ import annotations

from fastapi import FastAPI, HTTPException, Request  # module level: needed to resolve route annotations
from fastapi.responses import JSONResponse, PlainTextResponse

import asyncio
import itertools
from typing import Dict, List, Optional

import aiohttp

from .local_client import _Ring


class SessionRouter:
    def __init__(self, server_urls: List[str], policy: str = "consistent_hash", vnodes: int = 128,
                 prefill_urls: Optional[List[str]] = None):
        self.urls = [u.rstrip("/") for u in server_urls]
        self.prefill_urls = [u.rstrip("/") for u in (prefill_urls or [])]
        self.policy = policy
        self.ring = _Ring(len(self.urls), vnodes)
        self.healthy = [True] * len(self.urls)
        self._rr = itertools.count()
        self.stats: Dict[str, int] = {u: 0 for u in self.urls}
        if policy not in ("consistent_hash", "round_robin", "sticky_least_loaded"):
            raise ValueError(f"unknown routing policy '{policy}'")
        # sticky_least_loaded: where each open session lives, and how many open sessions each server holds
        self.session_home: Dict[str, int] = {}
        self.open_sessions: List[int] = [0] * len(self.urls)

    def pick(self, session_id: Optional[str]) -> str:
        live = [i for i, ok in enumerate(self.healthy) if ok]
        if not live:
            raise RuntimeError("no healthy inference server")
        if session_id is None or self.policy == "round_robin":
            i = live[next(self._rr) % len(live)]
        elif self.policy == "sticky_least_loaded":
            i = self.session_home.get(session_id, -1)
            if i < 0 or not self.healthy[i]:
                if i >= 0:  # its server went away: the session moves (and loses its cached prefix)
                    self.open_sessions[i] -= 1
                i = min(live, key=lambda k: (self.open_sessions[k], k))
                self.session_home[session_id] = i
                self.open_sessions[i] += 1
        else:
            i = self.ring.lookup(session_id)
            if not self.healthy[i]:  # walk to the next live node deterministically
                i = live[hash(session_id) % len(live)]
        self.stats[self.urls[i]] += 1
        return self.urls[i]

    def finish(self, session_id: Optional[str]) -> Optional[str]:
        """The session is over: free its place (sticky_least_loaded).  Returns the URL it lived on, if any."""
        i = self.session_home.pop(session_id, -1) if session_id is not None else -1
        if i < 0:
            return None
        self.open_sessions[i] -= 1
        return self.urls[i]

    def mark(self, url: str, ok: bool) -> None:
        self.healthy[self.urls.index(url.rstrip("/"))] = ok


def _make_handler(proxy, path: str):
    async def handler(request: Request):
        return await proxy(path, request)

    return handler


def build_router_app(router: SessionRouter):
    app = FastAPI(title="skyrl_b200 router")
    holder: Dict[str, aiohttp.ClientSession] = {}

    async def http() -> aiohttp.ClientSession:
        if "s" not in holder or holder["s"].closed:
            holder["s"] = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=3600),
                                                connector=aiohttp.TCPConnector(limit=0))
        return holder["s"]

    @app.get("/health")
    async def health():
        return {"status": "ok", "servers": router.urls, "healthy": router.healthy}

    @app.get("/stats")
    async def stats():
        return router.stats

    async def proxy(path: str, request: Request):
        sid = request.headers.get("X-Session-ID")
        body = await request.body()
        s = await http()
        headers = {"Content-Type": "application/json"}
        if sid:
            headers["X-Session-ID"] = sid
        if path == "/finish_session" and router.policy == "sticky_least_loaded":
            try:
                sid = sid or (await request.json()).get("session_id")
            except Exception:
                pass
            url = router.finish(sid)
            if url is None:
                return JSONResponse({"status": "ok"})
            try:
                async with s.post(url + path, data=body, headers=headers) as r:
                    return JSONResponse(await r.json(), status_code=r.status)
            except aiohttp.ClientConnectionError:
                return JSONResponse({"status": "ok"})
        for _attempt in range(len(router.urls)):
            url = router.pick(sid)
            try:
                async with s.post(url + path, data=body, headers=headers, params=dict(request.query_params)) as r:
                    return JSONResponse(await r.json(), status_code=r.status)
            except aiohttp.ClientConnectionError:
                router.mark(url, False)
        return JSONResponse({"error": "all inference servers are unreachable"}, status_code=503)

    for p in ("/inference/v1/generate", "/skyrl/v1/generate", "/v1/completions", "/v1/chat/completions", "/tokenize",
              "/detokenize", "/finish_session"):
        app.add_api_route(p, _make_handler(proxy, p), methods=["POST"])

    async def probe_loop():
        s = await http()
        while True:
            for u in router.urls:
                try:
                    async with s.get(u + "/health", timeout=aiohttp.ClientTimeout(total=2)) as r:
                        router.mark(u, r.status == 200)
                except Exception:
                    router.mark(u, False)
            await asyncio.sleep(2.0)

    async def _start():
        holder["probe"] = asyncio.create_task(probe_loop())

    async def _stop():
        holder["probe"].cancel()
        if "s" in holder:
            await holder["s"].close()

    app.router.on_startup.append(_start)
    app.router.on_shutdown.append(_stop)
    return app
