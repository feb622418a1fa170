"""Request/response store of the Tinker-compatible service, on the standard library's sqlite3 (WAL mode).

Reference: skyrl/tinker/db_models.py:78-152 (``FutureDB``, ``ModelDB``, ``CheckpointDB``, ``SessionDB``,
``SamplingSessionDB``) which uses sqlmodel/sqlalchemy; the same tables and status values are kept so that the
API process and the engine loop communicate only through rows: the API inserts PENDING futures, the engine turns
them into COMPLETED / FAILED rows, ``retrieve_future`` long-polls on them.
"""

from __future__ import annotations

import json
import sqlite3
import threading
import time
from typing import Any, Dict, List, Optional, Tuple

PENDING, COMPLETED, FAILED = "pending", "completed", "failed"

_SCHEMA = """
CREATE TABLE IF NOT EXISTS futures (
  request_id INTEGER PRIMARY KEY AUTOINCREMENT, request_type TEXT NOT NULL, model_id TEXT, seq_id INTEGER,
  request_data TEXT NOT NULL, result_data TEXT, status TEXT NOT NULL, created_at REAL NOT NULL, completed_at REAL);
CREATE UNIQUE INDEX IF NOT EXISTS futures_model_seq ON futures(model_id, seq_id) WHERE seq_id IS NOT NULL AND model_id IS NOT NULL;
CREATE INDEX IF NOT EXISTS futures_status ON futures(status, request_type, request_id);
CREATE TABLE IF NOT EXISTS models (
  model_id TEXT PRIMARY KEY, base_model TEXT NOT NULL, lora_config TEXT, model_role TEXT, status TEXT NOT NULL,
  request_id INTEGER, session_id TEXT, created_at REAL NOT NULL, last_request_at REAL NOT NULL);
CREATE TABLE IF NOT EXISTS checkpoints (
  model_id TEXT NOT NULL, checkpoint_id TEXT NOT NULL, checkpoint_type TEXT NOT NULL, status TEXT NOT NULL,
  path TEXT, error TEXT, created_at REAL NOT NULL, completed_at REAL, PRIMARY KEY (model_id, checkpoint_id, checkpoint_type));
CREATE TABLE IF NOT EXISTS sessions (
  session_id TEXT PRIMARY KEY, tags TEXT, user_metadata TEXT, sdk_version TEXT, status TEXT NOT NULL,
  created_at REAL NOT NULL, last_heartbeat_at REAL NOT NULL, heartbeat_count INTEGER NOT NULL DEFAULT 0);
CREATE TABLE IF NOT EXISTS sampling_sessions (
  sampling_session_id TEXT PRIMARY KEY, session_id TEXT NOT NULL, sampling_session_seq_id INTEGER NOT NULL,
  base_model TEXT, model_path TEXT, created_at REAL NOT NULL);
"""


class SequenceReused(Exception):
    """A (model_id, seq_id) pair was re-submitted with a different request."""


class TinkerDB:
    def __init__(self, path: str = ":memory:"):
        self.path = path
        self._lock = threading.RLock()
        self._conn = sqlite3.connect(path, check_same_thread=False, isolation_level=None, timeout=30.0)
        self._conn.row_factory = sqlite3.Row
        if path != ":memory:":
            self._conn.execute("PRAGMA journal_mode=WAL")
            self._conn.execute("PRAGMA synchronous=NORMAL")
        self._conn.executescript(_SCHEMA)

    def _x(self, sql: str, args: Tuple = ()) -> sqlite3.Cursor:
        with self._lock:
            return self._conn.execute(sql, args)

    def _all(self, sql: str, args: Tuple = ()) -> List[sqlite3.Row]:
        with self._lock:
            return self._conn.execute(sql, args).fetchall()

    # ------------------------------------------------------------------ futures
    def create_future(self, request_type: str, model_id: Optional[str], request_data: Dict[str, Any],
                      seq_id: Optional[int] = None) -> int:
        """Idempotent on (model_id, seq_id): a retry of the same request returns the first future's id."""
        blob = json.dumps(request_data, sort_keys=True)
        with self._lock:
            if model_id is not None and seq_id is not None:
                row = self._conn.execute("SELECT request_id, request_type, request_data FROM futures WHERE model_id=? AND seq_id=?",
                                         (model_id, seq_id)).fetchone()
                if row is not None:
                    if row["request_type"] != request_type or row["request_data"] != blob:
                        raise SequenceReused(f"seq_id {seq_id} of model {model_id} was reused for a different request")
                    return int(row["request_id"])
            cur = self._conn.execute(
                "INSERT INTO futures(request_type, model_id, seq_id, request_data, status, created_at) VALUES (?,?,?,?,?,?)",
                (request_type, model_id, seq_id, blob, PENDING, time.time()))
            return int(cur.lastrowid)

    def get_future(self, request_id: int) -> Optional[sqlite3.Row]:
        rows = self._all("SELECT * FROM futures WHERE request_id=?", (request_id,))
        return rows[0] if rows else None

    def complete_future(self, request_id: int, result: Dict[str, Any], ok: bool = True) -> None:
        self._x("UPDATE futures SET status=?, result_data=?, completed_at=? WHERE request_id=?",
                (COMPLETED if ok else FAILED, json.dumps(result), time.time(), request_id))

    def pending(self, request_types: Optional[List[str]] = None) -> List[sqlite3.Row]:
        if request_types:
            q = ",".join("?" * len(request_types))
            return self._all(f"SELECT * FROM futures WHERE status=? AND request_type IN ({q}) ORDER BY request_id",
                             (PENDING, *request_types))
        return self._all("SELECT * FROM futures WHERE status=? ORDER BY request_id", (PENDING,))

    def barriers(self, barrier_types: List[str]) -> Dict[str, int]:
        """Per model: the smallest pending request_id that changes the weights (optim_step / load_weights)."""
        q = ",".join("?" * len(barrier_types))
        rows = self._all(f"SELECT model_id, MIN(request_id) AS rid FROM futures WHERE status=? AND request_type IN ({q}) "
                         "GROUP BY model_id", (PENDING, *barrier_types))
        return {r["model_id"]: int(r["rid"]) for r in rows if r["model_id"] is not None}

    # ------------------------------------------------------------------ models / sessions / checkpoints
    def create_model(self, model_id: str, base_model: str, lora_config: Optional[dict], model_role: str, session_id: str,
                     request_id: int) -> None:
        now = time.time()
        self._x("INSERT INTO models VALUES (?,?,?,?,?,?,?,?,?)",
                (model_id, base_model, json.dumps(lora_config) if lora_config else None, model_role, "created", request_id,
                 session_id, now, now))

    def get_model(self, model_id: str) -> Optional[sqlite3.Row]:
        rows = self._all("SELECT * FROM models WHERE model_id=?", (model_id,))
        return rows[0] if rows else None

    def list_models(self, limit: int = 100, offset: int = 0) -> Tuple[List[sqlite3.Row], int]:
        total = self._all("SELECT COUNT(*) AS n FROM models")[0]["n"]
        return self._all("SELECT * FROM models ORDER BY created_at DESC LIMIT ? OFFSET ?", (limit, offset)), int(total)

    def set_model_status(self, model_id: str, status: str) -> None:
        self._x("UPDATE models SET status=? WHERE model_id=?", (status, model_id))

    def touch_model(self, model_id: str) -> None:
        self._x("UPDATE models SET last_request_at=? WHERE model_id=?", (time.time(), model_id))

    def create_session(self, session_id: str, tags: List[str], user_metadata: Optional[dict], sdk_version: str) -> None:
        now = time.time()
        self._x("INSERT INTO sessions VALUES (?,?,?,?,?,?,?,0)",
                (session_id, json.dumps(tags), json.dumps(user_metadata) if user_metadata else None, sdk_version, "active", now, now))

    def heartbeat(self, session_id: str) -> bool:
        cur = self._x("UPDATE sessions SET last_heartbeat_at=?, heartbeat_count=heartbeat_count+1 WHERE session_id=?",
                      (time.time(), session_id))
        return cur.rowcount > 0

    def stale_sessions(self, older_than_s: float) -> List[str]:
        rows = self._all("SELECT session_id FROM sessions WHERE status='active' AND last_heartbeat_at < ?",
                         (time.time() - older_than_s,))
        return [r["session_id"] for r in rows]

    def expire_session(self, session_id: str) -> List[str]:
        self._x("UPDATE sessions SET status='expired' WHERE session_id=?", (session_id,))
        return [r["model_id"] for r in self._all("SELECT model_id FROM models WHERE session_id=? AND status!='unloaded'",
                                                 (session_id,))]

    def create_sampling_session(self, sid: str, session_id: str, seq: int, base_model: Optional[str],
                                model_path: Optional[str]) -> None:
        self._x("INSERT INTO sampling_sessions VALUES (?,?,?,?,?,?)", (sid, session_id, seq, base_model, model_path, time.time()))

    def get_sampling_session(self, sid: str) -> Optional[sqlite3.Row]:
        rows = self._all("SELECT * FROM sampling_sessions WHERE sampling_session_id=?", (sid,))
        return rows[0] if rows else None

    def create_checkpoint(self, model_id: str, checkpoint_id: str, ctype: str) -> bool:
        try:
            self._x("INSERT INTO checkpoints(model_id, checkpoint_id, checkpoint_type, status, created_at) VALUES (?,?,?,?,?)",
                    (model_id, checkpoint_id, ctype, PENDING, time.time()))
            return True
        except sqlite3.IntegrityError:
            return False

    def finish_checkpoint(self, model_id: str, checkpoint_id: str, ctype: str, path: Optional[str], error: Optional[str] = None) -> None:
        self._x("UPDATE checkpoints SET status=?, path=?, error=?, completed_at=? WHERE model_id=? AND checkpoint_id=? AND checkpoint_type=?",
                (FAILED if error else COMPLETED, path, error, time.time(), model_id, checkpoint_id, ctype))

    def get_checkpoint(self, model_id: str, checkpoint_id: str, ctype: Optional[str] = None) -> Optional[sqlite3.Row]:
        if ctype:
            rows = self._all("SELECT * FROM checkpoints WHERE model_id=? AND checkpoint_id=? AND checkpoint_type=?",
                             (model_id, checkpoint_id, ctype))
        else:
            rows = self._all("SELECT * FROM checkpoints WHERE model_id=? AND checkpoint_id=?", (model_id, checkpoint_id))
        return rows[0] if rows else None

    def list_checkpoints(self, model_id: str) -> List[sqlite3.Row]:
        return self._all("SELECT * FROM checkpoints WHERE model_id=? AND status=? ORDER BY created_at", (model_id, COMPLETED))

    def delete_checkpoint(self, model_id: str, checkpoint_id: str, ctype: str) -> bool:
        return self._x("DELETE FROM checkpoints WHERE model_id=? AND checkpoint_id=? AND checkpoint_type=?",
                       (model_id, checkpoint_id, ctype)).rowcount > 0

    def close(self) -> None:
        with self._lock:
            self._conn.close()
