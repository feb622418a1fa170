"""Background loop of the Tinker service: turns PENDING rows into results.

Reference: skyrl/tinker/engine.py:212-843.  Every ``poll_interval`` (100 ms) the loop
  1. batches all pending ``forward_backward`` requests -- and separately all ``forward`` requests -- that sit
     *before* their model's next weight-changing request (``optim_step`` / ``load_weights``): gradients accumulate, so
     any number of them may be fused into one pass without changing results (:380-416),
  2. batches pending ``sample`` requests,
  3. executes the remaining single operations in request order,
  4. every ``session_cleanup_interval`` expires sessions without a heartbeat and unloads their models (:700-760).
Failures become FAILED rows carrying ``{"error", "category"}``; the loop itself keeps running.
"""

from __future__ import annotations

import json
import threading
import time
import traceback
from typing import Any, Callable, Dict, List, Optional

from . import db as tdb

FORWARD_BACKWARD, FORWARD, OPTIM_STEP, SAMPLE = "forward_backward", "forward", "optim_step", "sample"
CREATE_MODEL, UNLOAD_MODEL = "create_model", "unload_model"
SAVE_WEIGHTS, LOAD_WEIGHTS, SAVE_FOR_SAMPLER = "save_weights", "load_weights", "save_weights_for_sampler"
BARRIER_TYPES = [OPTIM_STEP, LOAD_WEIGHTS]
EXTERNAL = "external"  # handled outside the loop (sample forwarding to remote rollout servers)


class TinkerEngine:
    def __init__(self, db: tdb.TinkerDB, backend_factory: Callable[[str], Any], poll_interval: float = 0.1,
                 session_timeout_s: float = 300.0, session_cleanup_interval_s: float = 60.0, max_batch_datums: int = 4096):
        self.db = db
        self.backend_factory = backend_factory
        self.backends: Dict[str, Any] = {}  # base_model -> backend
        self.model_backend: Dict[str, Any] = {}  # model_id -> backend
        self.poll_interval = poll_interval
        self.session_timeout_s, self.session_cleanup_interval_s = session_timeout_s, session_cleanup_interval_s
        self.max_batch_datums = max_batch_datums
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_cleanup = time.time()
        self.stats = {"passes": 0, "batched_requests": 0, "failed": 0}

    # ------------------------------------------------------------------ scheduling
    def find_batchable_model_passes(self, request_type: str) -> List[Any]:
        """Pending rows of ``request_type`` that precede every pending barrier of their model."""
        barriers = self.db.barriers(BARRIER_TYPES)
        return [r for r in self.db.pending([request_type])
                if r["model_id"] not in barriers or r["request_id"] < barriers[r["model_id"]]]

    def _fail(self, rid: int, exc: BaseException, category: str = "server") -> None:
        self.stats["failed"] += 1
        if isinstance(exc, (ValueError, KeyError)):
            category = "user"
        self.db.complete_future(rid, {"error": f"{type(exc).__name__}: {exc}", "category": category}, ok=False)

    def _backend_for(self, model_id: str):
        b = self.model_backend.get(model_id)
        if b is None:
            raise KeyError(f"model '{model_id}' is not loaded")
        return b

    # ------------------------------------------------------------------ batched passes
    def process_model_passes(self, request_type: str) -> int:
        rows = self.find_batchable_model_passes(request_type)
        if not rows:
            return 0
        key = "forward_backward_input" if request_type == FORWARD_BACKWARD else "forward_input"
        groups: Dict[Any, List[Any]] = {}
        for r in rows:
            body = json.loads(r["request_data"])[key]
            cfg = json.dumps(body.get("loss_fn_config"), sort_keys=True)
            groups.setdefault((r["model_id"], body["loss_fn"], cfg), []).append((r, body))
        done = 0
        for (model_id, loss_fn, _), items in groups.items():
            # one pass per (model, loss): concatenate datums, split the per-datum outputs back per request
            while items:
                take, count = [], 0
                while items and (not take or count + len(items[0][1]["data"]) <= self.max_batch_datums):
                    take.append(items.pop(0))
                    count += len(take[-1][1]["data"])
                try:
                    be = self._backend_for(model_id)
                    datums = [d for _, b in take for d in b["data"]]
                    res = be.forward_backward(model_id, datums, loss_fn, take[0][1].get("loss_fn_config"),
                                              forward_only=(request_type == FORWARD))
                    outs = res.get("loss_fn_outputs") or []
                    k = 0
                    for r, b in take:
                        n = len(b["data"])
                        part = dict(res, loss_fn_outputs=outs[k : k + n] if outs else [])
                        k += n
                        self.db.complete_future(r["request_id"], part)
                        done += 1
                    self.db.touch_model(model_id)
                    self.stats["passes"] += 1
                    self.stats["batched_requests"] += len(take)
                except Exception as e:  # noqa: BLE001 - the row must leave PENDING whatever happened
                    traceback.print_exc()
                    for r, _ in take:
                        self._fail(r["request_id"], e)
        return done

    def process_samples(self) -> int:
        rows = self.db.pending([SAMPLE])
        if not rows:
            return 0
        by_backend: Dict[int, List[Any]] = {}
        for r in rows:
            body = json.loads(r["request_data"])
            try:
                be = self._sampling_backend(r["model_id"], body)
            except Exception as e:  # noqa: BLE001
                self._fail(r["request_id"], e)
                continue
            by_backend.setdefault(id(be), []).append((r, body, be))
        done = 0
        for items in by_backend.values():
            be = items[0][2]
            try:
                from .backend import flatten_model_input

                prompts = [flatten_model_input(b["prompt"]) for _, b, _ in items]
                res = be.sample(prompts, [b.get("sampling_params") or {} for _, b, _ in items],
                                [int(b.get("num_samples", 1)) for _, b, _ in items],
                                model_id=items[0][0]["model_id"],
                                prompt_logprobs=any(b.get("prompt_logprobs") for _, b, _ in items))
                for (r, _, _), out in zip(items, res):
                    self.db.complete_future(r["request_id"], out)
                    done += 1
            except Exception as e:  # noqa: BLE001
                traceback.print_exc()
                for r, _, _ in items:
                    self._fail(r["request_id"], e)
        return done

    def _sampling_backend(self, model_id: Optional[str], body: Dict[str, Any]):
        if model_id and model_id in self.model_backend:
            return self.model_backend[model_id]
        base = body.get("base_model")
        if base and base in self.backends:
            return self.backends[base]
        if self.backends:
            return next(iter(self.backends.values()))
        raise KeyError("no model is loaded to sample from")

    # ------------------------------------------------------------------ single operations
    def process_single(self, row) -> None:
        rid, rtype, model_id = row["request_id"], row["request_type"], row["model_id"]
        body = json.loads(row["request_data"])
        try:
            if rtype == CREATE_MODEL:
                base = body["base_model"]
                be = self.backends.get(base)
                if be is None:
                    be = self.backends[base] = self.backend_factory(base)
                be.create_model(model_id, body.get("lora_config"), body.get("model_role", "policy"))
                self.model_backend[model_id] = be
                self.db.set_model_status(model_id, "ready")
                out = {"model_id": model_id, "base_model": base, "lora_config": body.get("lora_config"), "status": "created"}
            elif rtype == UNLOAD_MODEL:
                be = self.model_backend.pop(model_id, None)
                if be is not None:
                    be.delete_model(model_id)
                self.db.set_model_status(model_id, "unloaded")
                out = {"model_id": model_id, "status": "unloaded"}
            elif rtype == OPTIM_STEP:
                out = self._backend_for(model_id).optim_step(model_id, body.get("adam_params"))
            elif rtype == SAVE_WEIGHTS:
                cid = body["path"]
                try:
                    path = self._backend_for(model_id).save_checkpoint(model_id, cid)
                    self.db.finish_checkpoint(model_id, cid, "training", path)
                except Exception as e:
                    self.db.finish_checkpoint(model_id, cid, "training", None, str(e))
                    raise
                out = {"path": f"tinker://{model_id}/weights/{cid}", "type": "save_weights"}
            elif rtype == LOAD_WEIGHTS:
                src_model, cid = parse_tinker_path(body["path"])[::2]
                ck = self.db.get_checkpoint(src_model, cid, "training")
                if ck is None or ck["status"] != tdb.COMPLETED:
                    raise ValueError(f"checkpoint '{body['path']}' does not exist")
                self._backend_for(model_id).load_checkpoint(model_id, ck["path"], bool(body.get("optimizer", True)))
                out = {"type": "load_weights"}
            elif rtype == SAVE_FOR_SAMPLER:
                cid = body.get("path")
                be = self._backend_for(model_id)
                try:
                    path = be.save_sampler_checkpoint(model_id, cid, persist=cid is not None)
                    if cid is not None:
                        self.db.finish_checkpoint(model_id, cid, "sampler", path)
                except Exception as e:
                    if cid is not None:
                        self.db.finish_checkpoint(model_id, cid, "sampler", None, str(e))
                    raise
                out = {"path": f"tinker://{model_id}/sampler_weights/{cid}" if cid else None,
                       "sampling_session_id": body.get("sampling_session_id"), "type": "save_weights_for_sampler"}
            else:
                raise ValueError(f"unknown request type '{rtype}'")
            if model_id:
                self.db.touch_model(model_id)
            self.db.complete_future(rid, out)
        except Exception as e:  # noqa: BLE001
            traceback.print_exc()
            self._fail(rid, e)

    def cleanup_stale_sessions(self) -> int:
        n = 0
        for sid in self.db.stale_sessions(self.session_timeout_s):
            for model_id in self.db.expire_session(sid):
                be = self.model_backend.pop(model_id, None)
                if be is not None:
                    be.delete_model(model_id)
                self.db.set_model_status(model_id, "unloaded")
                n += 1
        return n

    # ------------------------------------------------------------------ loop
    def step(self) -> int:
        """One scheduling round; returns the number of requests finished."""
        done = self.process_model_passes(FORWARD_BACKWARD)
        done += self.process_model_passes(FORWARD)
        done += self.process_samples()
        batched = {FORWARD_BACKWARD, FORWARD, SAMPLE, EXTERNAL}
        for row in self.db.pending():
            if row["request_type"] in batched:
                continue
            self.process_single(row)
            done += 1
            if row["request_type"] in BARRIER_TYPES:
                break  # passes queued behind this barrier are now batchable: go round again
        if time.time() - self._last_cleanup > self.session_cleanup_interval_s:
            self._last_cleanup = time.time()
            self.cleanup_stale_sessions()
        return done

    def run(self) -> None:
        while not self._stop.is_set():
            try:
                if self.step() == 0:
                    self._stop.wait(self.poll_interval)
            except Exception:  # noqa: BLE001 - keep serving
                traceback.print_exc()
                self._stop.wait(self.poll_interval)

    def start(self) -> "TinkerEngine":
        self._thread = threading.Thread(target=self.run, name="tinker-engine", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=30)


def parse_tinker_path(path: str):
    """``tinker://<model_id>/<weights|sampler_weights>/<checkpoint_id>`` -> (model_id, kind, checkpoint_id)."""
    if not path.startswith("tinker://"):
        raise ValueError(f"'{path}' is not a tinker:// path")
    parts = path[len("tinker://"):].split("/")
    if len(parts) != 3 or parts[1] not in ("weights", "sampler_weights"):
        raise ValueError(f"malformed tinker path '{path}'")
    return parts[0], parts[1], parts[2]
