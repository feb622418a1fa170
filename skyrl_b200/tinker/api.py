"""Tinker-compatible REST service (FastAPI).

Route set and payload shapes follow the reference service (skyrl/tinker/api.py:899-1700): every training / sampling
operation inserts a PENDING row and returns a ``future_id``; ``/api/v1/retrieve_future`` long-polls the row until the
engine loop completed it (408 on timeout so the SDK polls again; 400 with the stored message for user errors).
Idempotency: a request that repeats an earlier ``(model_id, seq_id)`` returns the first future, and a different
request under the same pair is rejected with 409.  Checkpoints are addressed as
``tinker://<model_id>/<weights|sampler_weights>/<checkpoint_id>`` and can be listed, downloaded as tar archives and
deleted.  The engine loop runs in a thread of this process (the reference forks a subprocess) because a GPU process
that already owns the model is the unit here; ``build_app`` accepts any backend factory so tests run on CPU.
"""

from __future__ import annotations

from fastapi import FastAPI, HTTPException, Request  # module level: route annotations are resolved against globals
from fastapi.responses import FileResponse, JSONResponse, Response

import asyncio
import json
import os
import re
import time
import uuid
from datetime import datetime, timezone
from typing import Any, Callable, Dict, List, Optional

from . import db as tdb
from . import engine as teng

ID_PATTERN = re.compile(r"^[A-Za-z0-9._-]+$")
ID_MAX_LENGTH = 128
RETRIEVE_FUTURE_TIMEOUT_SECONDS = 30.0
LOSS_FNS = ("cross_entropy", "importance_sampling", "ppo", "gspo", "cispo", "ppo_critic", "dppo")


def _iso(ts: float) -> str:
    return datetime.fromtimestamp(ts, tz=timezone.utc).isoformat()


def _require(body: Dict[str, Any], *keys: str) -> None:
    missing = [k for k in keys if k not in body]
    if missing:
        raise HTTPException(422, f"missing field(s): {missing}")


# what a client may tune per request (the Tinker names; the backend maps them onto the algorithm config)
LOSS_FN_CONFIG_KEYS = {
    "cross_entropy": set(), "importance_sampling": set(),
    "ppo": {"clip_low_threshold", "clip_high_threshold", "value_clip"},
    "gspo": {"clip_low_threshold", "clip_high_threshold"}, "cispo": {"clip_low_threshold", "clip_high_threshold"},
    "ppo_critic": {"value_clip"}, "dppo": {"delta_low", "delta_high"},
}


def _validate_pass_input(inp: Dict[str, Any]) -> None:
    _require(inp, "data", "loss_fn")
    if inp["loss_fn"] not in LOSS_FNS:
        raise HTTPException(422, f"loss_fn must be one of {LOSS_FNS}")
    cfg = inp.get("loss_fn_config")
    if cfg:
        if not isinstance(cfg, dict):
            raise HTTPException(422, "loss_fn_config must be an object of numbers")
        allowed = LOSS_FN_CONFIG_KEYS[inp["loss_fn"]]
        bad = sorted(set(cfg) - allowed)
        if bad and allowed:
            raise HTTPException(422, f"Invalid loss_fn_config keys for loss_fn='{inp['loss_fn']}': {bad}. "
                                     f"Allowed keys: {sorted(allowed)}.")
        if bad:
            raise HTTPException(422, f"loss_fn='{inp['loss_fn']}' does not accept loss_fn_config keys. Received: {bad}.")
        if any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in cfg.values()):
            raise HTTPException(422, "loss_fn_config values must be numbers")
    if not isinstance(inp["data"], list) or not inp["data"]:
        raise HTTPException(422, "data must be a non-empty list of datums")
    for d in inp["data"]:
        if "model_input" not in d or "loss_fn_inputs" not in d:
            raise HTTPException(422, "each datum needs model_input and loss_fn_inputs")
        li = d["loss_fn_inputs"]
        need = {"cross_entropy": ("target_tokens", "weights"), "ppo_critic": ("target_tokens",)}.get(
            inp["loss_fn"], ("target_tokens", "logprobs", "advantages"))
        for k in need:
            if k not in li:
                raise HTTPException(422, f"loss_fn '{inp['loss_fn']}' needs loss_fn_inputs['{k}']")


def build_app(backend_factory: Callable[[str], Any], db_path: str = ":memory:", supported_models: Optional[List[str]] = None,
              poll_interval: float = 0.02, start_engine: bool = True, external_sampler=None) -> FastAPI:
    """``backend_factory(base_model) -> backend`` (see ``tinker.backend.SkyRLTrainBackend``).
    ``external_sampler(body) -> awaitable result`` forwards sample requests to remote rollout servers instead of
    queueing them for the engine loop (non-colocated deployments)."""
    from contextlib import asynccontextmanager

    db = tdb.TinkerDB(db_path)
    engine = teng.TinkerEngine(db, backend_factory, poll_interval=poll_interval)

    @asynccontextmanager
    async def lifespan(_app):
        if start_engine:
            engine.start()
        yield
        engine.stop()

    app = FastAPI(title="skyrl_b200 tinker service", version="0.1", lifespan=lifespan)
    app.state.db, app.state.engine = db, engine

    def future(rid: int) -> Dict[str, Any]:
        return {"future_id": str(rid), "request_id": str(rid), "status": "pending"}

    def need_model(model_id: str):
        m = db.get_model(model_id)
        if m is None:
            raise HTTPException(404, "Model not found")
        return m

    def enqueue(rtype: str, model_id: Optional[str], body: Dict[str, Any], seq_id: Optional[int] = None) -> int:
        try:
            return db.create_future(rtype, model_id, body, seq_id)
        except tdb.SequenceReused:
            raise HTTPException(409, "Training request sequence number was reused")

    # ------------------------------------------------------------------ service
    @app.get("/")
    async def root():
        return {"service": "skyrl_b200 tinker", "docs": "/docs"}

    @app.get("/api/v1/healthz")
    async def healthz():
        return {"status": "ok"}

    @app.post("/api/v1/client/config")
    async def client_config():
        return {"pjwt_auth_enabled": False}

    @app.get("/api/v1/get_server_capabilities")
    async def capabilities():
        return {"supported_models": [{"model_name": m} for m in (supported_models or [])]}

    @app.post("/api/v1/telemetry")
    async def telemetry(request: Request):
        await request.json()
        return {"status": "accepted"}

    # ------------------------------------------------------------------ sessions
    @app.post("/api/v1/create_session")
    async def create_session(request: Request):
        body = await request.json()
        sid = f"session-{uuid.uuid4().hex[:16]}"
        db.create_session(sid, body.get("tags") or [], body.get("user_metadata"), body.get("sdk_version", ""))
        return {"type": "create_session", "session_id": sid, "info_message": None, "warning_message": None, "error_message": None}

    @app.post("/api/v1/session_heartbeat")
    async def heartbeat(request: Request):
        body = await request.json()
        if not db.heartbeat(body.get("session_id", "")):
            raise HTTPException(404, "Session not found")
        return {"type": "session_heartbeat"}

    @app.post("/api/v1/create_sampling_session")
    async def create_sampling_session(request: Request):
        body = await request.json()
        _require(body, "session_id", "sampling_session_seq_id")
        if not body.get("base_model") and not body.get("model_path"):
            raise HTTPException(422, "give base_model or model_path")
        sid = f"sampler-{uuid.uuid4().hex[:16]}"
        db.create_sampling_session(sid, body["session_id"], int(body["sampling_session_seq_id"]), body.get("base_model"),
                                   body.get("model_path"))
        return {"type": "create_sampling_session", "sampling_session_id": sid}

    @app.get("/api/v1/samplers/{sampler_id}")
    async def get_sampler(sampler_id: str):
        s = db.get_sampling_session(sampler_id)
        if s is None:
            raise HTTPException(404, "Sampler not found")
        base = s["base_model"]
        if not base and s["model_path"]:
            m = db.get_model(teng.parse_tinker_path(s["model_path"])[0])
            base = m["base_model"] if m else ""
        return {"sampler_id": sampler_id, "base_model": base or "", "model_path": s["model_path"]}

    # ------------------------------------------------------------------ models
    @app.post("/api/v1/create_model")
    async def create_model(request: Request):
        body = await request.json()
        _require(body, "session_id", "base_model")
        if supported_models and body["base_model"] not in supported_models:
            raise HTTPException(400, f"base_model '{body['base_model']}' is not served here")
        model_id = f"model-{uuid.uuid4().hex[:12]}"
        rid = enqueue(teng.CREATE_MODEL, model_id, {"base_model": body["base_model"], "lora_config": body.get("lora_config"),
                                                    "model_role": body.get("model_role", "policy")})
        db.create_model(model_id, body["base_model"], body.get("lora_config"), body.get("model_role", "policy"),
                        body["session_id"], rid)
        return {"model_id": model_id, "base_model": body["base_model"], "lora_config": body.get("lora_config"),
                "status": "created", "request_id": str(rid)}

    @app.post("/api/v1/unload_model")
    async def unload_model(request: Request):
        body = await request.json()
        need_model(body.get("model_id", ""))
        rid = enqueue(teng.UNLOAD_MODEL, body["model_id"], {})
        return {"request_id": str(rid), "model_id": body["model_id"]}

    @app.post("/api/v1/get_info")
    async def get_info(request: Request):
        body = await request.json()
        m = need_model(body.get("model_id", ""))
        return {"model_id": m["model_id"], "status": m["status"],
                "model_data": {"base_model": m["base_model"], "model_name": m["base_model"],
                               "lora_config": json.loads(m["lora_config"]) if m["lora_config"] else None}}

    def _ckpt_json(model_id: str, c) -> Dict[str, Any]:
        kind = "weights" if c["checkpoint_type"] == "training" else "sampler_weights"
        return {"checkpoint_id": c["checkpoint_id"], "checkpoint_type": c["checkpoint_type"],
                "time": _iso(c["completed_at"] or c["created_at"]), "tinker_path": f"tinker://{model_id}/{kind}/{c['checkpoint_id']}"}

    def _run_json(m) -> Dict[str, Any]:
        cks = db.list_checkpoints(m["model_id"])
        tr = [c for c in cks if c["checkpoint_type"] == "training"]
        sa = [c for c in cks if c["checkpoint_type"] == "sampler"]
        lc = json.loads(m["lora_config"]) if m["lora_config"] else None
        return {"training_run_id": m["model_id"], "base_model": m["base_model"], "model_owner": "default",
                "is_lora": bool(lc and lc.get("rank")), "corrupted": False, "lora_rank": (lc or {}).get("rank"),
                "last_request_time": _iso(m["last_request_at"]),
                "last_checkpoint": _ckpt_json(m["model_id"], tr[-1]) if tr else None,
                "last_sampler_checkpoint": _ckpt_json(m["model_id"], sa[-1]) if sa else None, "user_metadata": None}

    @app.get("/api/v1/training_runs")
    async def training_runs(limit: int = 20, offset: int = 0):
        rows, total = db.list_models(limit, offset)
        return {"training_runs": [_run_json(m) for m in rows], "cursor": {"offset": offset, "limit": limit, "total_count": total}}

    @app.get("/api/v1/training_runs/{model_id}")
    async def training_run(model_id: str):
        return _run_json(need_model(model_id))

    # ------------------------------------------------------------------ training verbs
    @app.post("/api/v1/forward_backward")
    async def forward_backward(request: Request):
        body = await request.json()
        _require(body, "model_id", "forward_backward_input")
        need_model(body["model_id"])
        _validate_pass_input(body["forward_backward_input"])
        return future(enqueue(teng.FORWARD_BACKWARD, body["model_id"],
                              {"forward_backward_input": body["forward_backward_input"]}, body.get("seq_id")))

    @app.post("/api/v1/forward")
    async def forward(request: Request):
        body = await request.json()
        _require(body, "model_id", "forward_input")
        need_model(body["model_id"])
        _validate_pass_input(body["forward_input"])
        return future(enqueue(teng.FORWARD, body["model_id"], {"forward_input": body["forward_input"]}, body.get("seq_id")))

    @app.post("/api/v1/optim_step")
    async def optim_step(request: Request):
        body = await request.json()
        _require(body, "model_id")
        need_model(body["model_id"])
        ap = dict(body.get("adam_params") or {})
        ap.setdefault("learning_rate", 1e-4)
        if ap["learning_rate"] < 0 or ap.get("weight_decay", 0.0) < 0 or ap.get("eps", 1e-12) <= 0:
            raise HTTPException(422, "adam_params out of range")
        return future(enqueue(teng.OPTIM_STEP, body["model_id"], {"adam_params": ap}, body.get("seq_id")))

    def _check_id(cid: Optional[str]) -> None:
        if cid is not None and (not ID_PATTERN.match(cid) or len(cid) > ID_MAX_LENGTH):
            raise HTTPException(422, "checkpoint names may contain letters, digits, '.', '_' and '-' only")

    @app.post("/api/v1/save_weights")
    async def save_weights(request: Request):
        body = await request.json()
        _require(body, "model_id", "path")
        need_model(body["model_id"])
        _check_id(body["path"])
        if not db.create_checkpoint(body["model_id"], body["path"], "training"):
            raise HTTPException(409, f"Checkpoint '{body['path']}' already exists for model '{body['model_id']}'")
        return future(enqueue(teng.SAVE_WEIGHTS, body["model_id"], {"path": body["path"]}, body.get("seq_id")))

    @app.post("/api/v1/load_weights")
    async def load_weights(request: Request):
        body = await request.json()
        _require(body, "model_id", "path")
        need_model(body["model_id"])
        try:
            src, kind, cid = teng.parse_tinker_path(body["path"])
        except ValueError as e:
            raise HTTPException(400, str(e))
        if kind != "weights":
            raise HTTPException(400, "only training checkpoints (…/weights/…) can be loaded for training")
        if db.get_checkpoint(src, cid, "training") is None:
            raise HTTPException(404, f"checkpoint '{body['path']}' not found")
        return future(enqueue(teng.LOAD_WEIGHTS, body["model_id"], {"path": body["path"], "optimizer": body.get("optimizer", True)},
                              body.get("seq_id")))

    @app.post("/api/v1/save_weights_for_sampler")
    async def save_for_sampler(request: Request):
        body = await request.json()
        _require(body, "model_id")
        m = need_model(body["model_id"])
        _check_id(body.get("path"))
        if body.get("path") is None and body.get("sampling_session_seq_id") is None:
            raise HTTPException(422, "give path (persistent) or sampling_session_seq_id (ephemeral)")
        ssid = None
        if body.get("path") is not None:
            if not db.create_checkpoint(body["model_id"], body["path"], "sampler"):
                raise HTTPException(409, f"Checkpoint '{body['path']}' already exists for model '{body['model_id']}'")
        else:  # ephemeral: the sampling session addresses the live weights of this model
            ssid = f"sampler-{uuid.uuid4().hex[:16]}"
            db.create_sampling_session(ssid, m["session_id"] or "", int(body["sampling_session_seq_id"]), m["base_model"],
                                       f"tinker://{body['model_id']}/sampler_weights/live")
        return future(enqueue(teng.SAVE_FOR_SAMPLER, body["model_id"], {"path": body.get("path"), "sampling_session_id": ssid},
                              body.get("seq_id")))

    @app.post("/api/v1/asample")
    async def asample(request: Request):
        body = await request.json()
        _require(body, "prompt", "sampling_params")
        model_id = None
        if body.get("sampling_session_id"):
            s = db.get_sampling_session(body["sampling_session_id"])
            if s is None:
                raise HTTPException(404, "Sampling session not found")
            if s["model_path"]:
                model_id = teng.parse_tinker_path(s["model_path"])[0]
            body.setdefault("base_model", s["base_model"])
        elif body.get("model_path"):
            try:
                model_id = teng.parse_tinker_path(body["model_path"])[0]
            except ValueError as e:
                raise HTTPException(400, str(e))
        elif not body.get("base_model"):
            raise HTTPException(422, "give sampling_session_id, model_path or base_model")
        if model_id is not None and db.get_model(model_id) is None:
            raise HTTPException(404, "Model not found")
        payload = {k: body.get(k) for k in ("prompt", "sampling_params", "num_samples", "base_model", "prompt_logprobs",
                                            "topk_prompt_logprobs")}
        payload["num_samples"] = payload.get("num_samples") or 1
        if external_sampler is not None:
            rid = enqueue(teng.EXTERNAL, model_id, payload)

            async def run():
                try:
                    db.complete_future(rid, await external_sampler(payload))
                except Exception as e:  # noqa: BLE001
                    db.complete_future(rid, {"error": str(e), "category": "server"}, ok=False)

            asyncio.get_running_loop().create_task(run())
            return future(rid)
        return future(enqueue(teng.SAMPLE, model_id, payload))

    # ------------------------------------------------------------------ futures
    @app.post("/api/v1/retrieve_future")
    async def retrieve_future(request: Request):
        body = await request.json()
        try:
            rid = int(body.get("request_id"))
        except (TypeError, ValueError):
            raise HTTPException(422, "request_id must be an integer string")
        t0 = time.time()
        while True:
            row = db.get_future(rid)
            if row is None:
                raise HTTPException(404, "Future not found")
            if row["status"] == tdb.COMPLETED:
                return Response(content=row["result_data"], media_type="application/json")
            if row["status"] == tdb.FAILED:
                try:
                    err = json.loads(row["result_data"])
                except (TypeError, json.JSONDecodeError):
                    raise HTTPException(500, "Unknown error")
                raise HTTPException(400 if err.get("category") == "user" else 500, err.get("error", "Unknown error"))
            if time.time() - t0 > RETRIEVE_FUTURE_TIMEOUT_SECONDS:
                raise HTTPException(408, "Timeout waiting for result")
            await asyncio.sleep(0.01)

    # ------------------------------------------------------------------ checkpoints
    @app.get("/api/v1/training_runs/{model_id}/checkpoints")
    async def list_checkpoints(model_id: str):
        need_model(model_id)
        return {"checkpoints": [_ckpt_json(model_id, c) for c in db.list_checkpoints(model_id)]}

    @app.get("/api/v1/models/{model_id}/checkpoints")
    async def list_checkpoints_alias(model_id: str):
        return await list_checkpoints(model_id)

    def _find_ckpt(model_id: str, checkpoint_id: str):
        need_model(model_id)
        c = db.get_checkpoint(model_id, checkpoint_id)
        if c is None or c["status"] != tdb.COMPLETED or not c["path"] or not os.path.exists(c["path"]):
            raise HTTPException(404, "Checkpoint not found")
        return c

    @app.get("/api/v1/training_runs/{model_id}/checkpoints/{checkpoint_id}/archive")
    async def checkpoint_archive(model_id: str, checkpoint_id: str):
        c = _find_ckpt(model_id, checkpoint_id)
        return FileResponse(c["path"], media_type="application/x-tar", filename=f"{model_id}-{checkpoint_id}.tar")

    @app.get("/api/v1/training_runs/{model_id}/checkpoints/{checkpoint_id}/download")
    async def checkpoint_download(model_id: str, checkpoint_id: str, request: Request):
        _find_ckpt(model_id, checkpoint_id)
        url = str(request.url_for("checkpoint_archive", model_id=model_id, checkpoint_id=checkpoint_id))
        return {"url": url, "expires": _iso(time.time() + 3600)}

    @app.delete("/api/v1/training_runs/{model_id}/checkpoints/{checkpoint_path:path}", status_code=204)
    async def delete_checkpoint(model_id: str, checkpoint_path: str):
        need_model(model_id)
        parts = checkpoint_path.split("/")
        kind, cid = (parts[0], parts[1]) if len(parts) == 2 else ("weights", parts[0])
        ctype = "training" if kind == "weights" else "sampler"
        c = db.get_checkpoint(model_id, cid, ctype)
        if c is None:
            raise HTTPException(404, "Checkpoint not found")
        if c["path"] and os.path.exists(c["path"]):
            os.remove(c["path"])
        db.delete_checkpoint(model_id, cid, ctype)
        return Response(status_code=204)

    @app.post("/api/v1/weights_info")
    async def weights_info(request: Request):
        body = await request.json()
        try:
            model_id, _, _ = teng.parse_tinker_path(body.get("tinker_path", ""))
        except ValueError as e:
            raise HTTPException(400, str(e))
        m = need_model(model_id)
        lc = json.loads(m["lora_config"]) if m["lora_config"] else None
        return {"base_model": m["base_model"], "is_lora": bool(lc and lc.get("rank")), "lora_rank": (lc or {}).get("rank")}

    return app


def main(argv: Optional[List[str]] = None) -> None:
    """``python -m skyrl_b200.tinker.api --base-model NAME [--port 8000] [--db tinker.db] [key=value overrides]``"""
    import argparse

    import uvicorn

    from ..parallel import dist as pdist
    from ..utils.tokenizer import get_tokenizer
    from .backend import SkyRLTrainBackend

    ap = argparse.ArgumentParser()
    ap.add_argument("--base-model", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--db", default="tinker.db")
    ap.add_argument("--checkpoints-base", default=None)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    env = pdist.init_distributed()
    ov = dict(o.split("=", 1) for o in a.overrides)
    tok = get_tokenizer(a.base_model)

    def factory(base_model: str):
        return SkyRLTrainBackend(base_model, ov, env=env, tokenizer=tok, checkpoints_base=a.checkpoints_base)

    uvicorn.run(build_app(factory, a.db, [a.base_model], poll_interval=0.1), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
