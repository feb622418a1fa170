"""Trajectory tables: a sample of prompts / responses / rewards per step, written as JSONL and (when the tracker
supports tables) as a table (reference: skyrl/train/utils/trajectory_logging.py)."""

from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional


class TrajectoryLogger:
    def __init__(self, log_dir: str, tokenizer=None, max_rows: int = 16, max_chars: int = 4000, tracker=None):
        self.log_dir, self.tokenizer, self.max_rows, self.max_chars, self.tracker = log_dir, tokenizer, max_rows, max_chars, tracker
        os.makedirs(log_dir, exist_ok=True)

    def _text(self, ids: List[int]) -> str:
        if self.tokenizer is None:
            return " ".join(str(i) for i in ids)[: self.max_chars]
        return self.tokenizer.decode(ids, skip_special_tokens=False)[: self.max_chars]

    def rows(self, out: Dict[str, Any], uids: Optional[List[str]] = None) -> List[Dict[str, Any]]:
        n = min(self.max_rows, len(out["response_ids"]))
        rows = []
        for i in range(n):
            r = out["rewards"][i]
            rows.append({"uid": uids[i] if uids else None, "prompt": self._text(out["prompt_token_ids"][i]),
                         "response": self._text(out["response_ids"][i]),
                         "reward": float(sum(r)) if isinstance(r, (list, tuple)) else float(r),
                         "response_length": len(out["response_ids"][i]),
                         "stop_reason": (out.get("stop_reasons") or [None] * n)[i]})
        return rows

    def log(self, out: Dict[str, Any], step: int, split: str = "train", uids: Optional[List[str]] = None) -> str:
        rows = self.rows(out, uids)
        path = os.path.join(self.log_dir, f"{split}_trajectories_step_{step}.jsonl")
        with open(path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        if self.tracker is not None and hasattr(self.tracker, "log_table"):
            self.tracker.log_table(f"{split}/trajectories", rows, step)
        return path
