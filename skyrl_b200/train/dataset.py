"""Prompt datasets and a resumable batch iterator.

``PromptDataset`` reads parquet / json / jsonl files (or an in-memory list) whose rows have a chat
``prompt`` and optional ``env_class`` / ``reward_spec`` / ``extra_info`` fields, drops prompts longer than
``max_prompt_length`` tokens, and yields ``{"prompt", "env_class", "env_extras", "uid"}`` items
(reference: skyrl/train/dataset/dataset.py:16-103).  ``StatefulBatchIterator`` replaces the
torchdata ``StatefulDataLoader``: a seeded permutation per epoch whose position can be saved and
restored exactly (reference: trainer_utils.py:829-876, samplers.py).
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterator, List, Optional, Sequence

import numpy as np
from ..utils.tokenizer import chat_template_ids


def _read_rows(path: str) -> List[Dict[str, Any]]:
    if path.endswith(".parquet"):
        import pandas as pd

        df = pd.read_parquet(path)
        rows = df.to_dict(orient="records")
        for r in rows:  # numpy containers -> python
            for k, v in list(r.items()):
                if isinstance(v, np.ndarray):
                    r[k] = v.tolist()
        return rows
    if path.endswith(".jsonl"):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    if path.endswith(".json"):
        with open(path) as f:
            data = json.load(f)
        return data if isinstance(data, list) else data["data"]
    raise ValueError(f"unsupported dataset file '{path}' (parquet, json, jsonl)")


class PromptDataset:
    def __init__(self, datasets: Sequence[Any], tokenizer=None, max_prompt_length: int = 512, prompt_key: str = "prompt",
                 env_class_key: str = "env_class", num_workers: int = 0):
        rows: List[Dict[str, Any]] = []
        for d in datasets:
            if isinstance(d, str):
                rows.extend(_read_rows(os.path.expanduser(d)))
            elif isinstance(d, dict):
                rows.append(d)
            else:
                rows.extend(list(d))
        self.items: List[Dict[str, Any]] = []
        dropped = 0
        for i, r in enumerate(rows):
            prompt = r[prompt_key]
            if tokenizer is not None and max_prompt_length is not None and r.get("prompt_token_ids") is None:
                n = len(chat_template_ids(tokenizer, prompt, add_generation_prompt=True))
                if n > max_prompt_length:
                    dropped += 1
                    continue
            extras = {k: v for k, v in r.items() if k not in (prompt_key, env_class_key, "uid", "prompt_token_ids")}
            self.items.append({"prompt": prompt, "env_class": r.get(env_class_key), "env_extras": extras,
                               "uid": str(r.get("uid", i)), "prompt_token_ids": r.get("prompt_token_ids")})
        self.num_dropped = dropped

    def __len__(self) -> int:
        return len(self.items)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        return self.items[i]

    def collate_fn(self, batch: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        return list(batch)


class StatefulBatchIterator:
    """Epoch-wise shuffled batches with ``state_dict`` / ``load_state_dict`` (drop_last semantics)."""

    def __init__(self, dataset: PromptDataset, batch_size: int, shuffle: bool = True, seed: int = 42, drop_last: bool = True):
        self.ds, self.bs, self.shuffle, self.seed, self.drop_last = dataset, batch_size, shuffle, seed, drop_last
        self.epoch = 0
        self.cursor = 0

    def __len__(self) -> int:
        n = len(self.ds)
        return n // self.bs if self.drop_last else (n + self.bs - 1) // self.bs

    def _order(self) -> np.ndarray:
        idx = np.arange(len(self.ds))
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(idx)
        return idx

    def __iter__(self) -> Iterator[List[Dict[str, Any]]]:
        order = self._order()
        n_batches = len(self)
        while self.cursor < n_batches:
            b = order[self.cursor * self.bs : (self.cursor + 1) * self.bs]
            self.cursor += 1
            yield [self.ds[int(i)] for i in b]
        self.epoch += 1
        self.cursor = 0

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.epoch, self.cursor = int(sd["epoch"]), int(sd["cursor"])
        self.seed = int(sd.get("seed", self.seed))
