"""SFT data path: example tokenization (chat / alpaca, tool calls), on-disk token cache, padded and packed
collators, sequence bin-packing and samplers.

Reference behaviour: skyrl/train/sft_trainer.py:89-760 (tokenizers, cache, collate), skyrl/train/dataset/collators.py:35-260,
skyrl/train/dataset/bin_packing.py:29-240, skyrl/train/dataset/samplers.py:59-140.  The batch layout is the RL one
(left-padded ``sequences``, right-aligned ``loss_mask`` over the last ``num_actions`` positions) so the policy worker's
``cross_entropy`` branch consumes it unchanged; packing is expressed as bins of row indices because the worker packs
rows into varlen attention calls itself.
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import os
import pickle
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, Iterator, List, Optional, Sequence

import numpy as np
import torch

from .batch import TrainingInputBatch, pad_training_input_batch
from ..utils.tokenizer import chat_template_ids

TRAIN_ON_LAST = "last_assistant_message"
TRAIN_ON_ALL = "all_assistant_messages"


# ----------------------------------------------------------------------------- message normalisation
def _coerce_tools(tools: Any) -> Optional[list]:
    """Tool schemas arrive as a list, a JSON string or null."""
    if tools is None or tools == "" or (isinstance(tools, float) and np.isnan(tools)):
        return None
    if isinstance(tools, str):
        try:
            tools = json.loads(tools)
        except json.JSONDecodeError:
            return None
    if isinstance(tools, np.ndarray):
        tools = tools.tolist()
    return list(tools) if tools else None


def _normalize_tool_calls(tc: Any) -> Optional[list]:
    """``tool_calls`` with ``function.arguments`` given as a JSON string -> dict (what chat templates expect)."""
    if tc is None:
        return None
    if isinstance(tc, str):
        try:
            tc = json.loads(tc)
        except json.JSONDecodeError:
            return None
    if isinstance(tc, np.ndarray):
        tc = tc.tolist()
    out = []
    for c in tc or []:
        c = dict(c)
        fn = dict(c.get("function") or {})
        args = fn.get("arguments")
        if isinstance(args, str):
            try:
                fn["arguments"] = json.loads(args)
            except json.JSONDecodeError:
                pass
        if fn:
            c["function"] = fn
        out.append(c)
    return out or None


def normalize_chat_messages(messages: Sequence[dict]) -> List[dict]:
    out = []
    for m in messages:
        m = {k: v for k, v in dict(m).items() if v is not None}
        if "tool_calls" in m:
            tc = _normalize_tool_calls(m["tool_calls"])
            if tc:
                m["tool_calls"] = tc
            else:
                m.pop("tool_calls")
        m.setdefault("content", "")
        out.append(m)
    return out


# ----------------------------------------------------------------------------- tokenization
def _template(tokenizer, msgs, add_generation_prompt: bool, tools=None) -> List[int]:
    kw = {"tools": tools} if tools else {}
    return chat_template_ids(tokenizer, msgs, add_generation_prompt=add_generation_prompt, **kw)


def tokenize_chat_example(example: dict, tokenizer, max_length: Optional[int] = None, messages_key: str = "messages",
                          tools_key: str = "tools", system_key: str = "system",
                          train_on_what: str = TRAIN_ON_LAST) -> Optional[dict]:
    """Conversation -> ``{input_ids, attention_mask, loss_mask, num_actions}``.

    The loss mask covers the tokens an assistant turn adds on top of its generation prompt (content plus the
    end-of-turn token).  ``num_actions`` counts from the first trained token to the end; the mask is stored over
    exactly that suffix.  Returns ``None`` when there is no assistant turn or the first trained token would be
    truncated away."""
    msgs = normalize_chat_messages(example[messages_key])
    sys_prompt = example.get(system_key)
    if sys_prompt and (not msgs or msgs[0].get("role") != "system"):
        msgs = [{"role": "system", "content": sys_prompt}] + msgs
    tools = _coerce_tools(example.get(tools_key))
    turns = [i for i, m in enumerate(msgs) if m.get("role") == "assistant"]
    if not turns:
        return None
    if train_on_what == TRAIN_ON_LAST:
        msgs = msgs[: turns[-1] + 1]
        turns = [turns[-1]]
    full = _template(tokenizer, msgs, False, tools)
    mask = np.zeros(len(full), dtype=np.int64)
    for i in turns:
        start = len(_template(tokenizer, msgs[:i], True, tools))
        end = len(_template(tokenizer, msgs[: i + 1], False, tools))
        if full[:start] != _template(tokenizer, msgs[:i], True, tools)[:start] or end > len(full):
            # template is not prefix-stable here (e.g. it rewrites history): fall back to the tail span
            if i == turns[-1]:
                end = len(full)
            else:
                continue
        mask[start:end] = 1
    if max_length is not None and len(full) > max_length:
        full, mask = full[:max_length], mask[:max_length]
    nz = np.flatnonzero(mask)
    if nz.size == 0:
        return None
    first = int(nz[0])
    return {"input_ids": full, "attention_mask": [1] * len(full), "loss_mask": mask[first:].tolist(),
            "num_actions": len(full) - first}


def tokenize_sft_example(example: dict, tokenizer, max_length: Optional[int] = 512) -> Optional[dict]:
    """Alpaca-style ``instruction`` / ``input`` / ``output`` rows: prompt rendered as one user message."""
    instr = example.get("instruction") or example.get("prompt") or ""
    inp = example.get("input") or ""
    user = f"{instr}\n\n{inp}" if inp else instr
    out = example.get("output") if example.get("output") is not None else example.get("response", "")
    return tokenize_chat_example({"messages": [{"role": "user", "content": user}, {"role": "assistant", "content": out}]},
                                 tokenizer, max_length)


def _cache_key(source: str, tokenizer, max_length, train_on_what: str, extra: str = "") -> str:
    st = os.stat(source) if os.path.exists(source) else None
    ident = f"{source}|{st.st_size if st else 0}|{st.st_mtime_ns if st else 0}|{getattr(tokenizer, 'name_or_path', type(tokenizer).__name__)}" \
            f"|{getattr(tokenizer, 'vocab_size', 0)}|{max_length}|{train_on_what}|{extra}"
    return hashlib.sha256(ident.encode()).hexdigest()[:24]


def load_and_tokenize(source: str, tokenizer, cfg, split: Optional[str] = None) -> List[dict]:
    """Read ``source`` (jsonl / json / parquet), tokenize with a thread pool, cache the result on disk."""
    from .dataset import _read_rows

    key = _cache_key(source, tokenizer, cfg.max_length, cfg.train_on_what, f"{cfg.messages_key}|{split}")
    path = os.path.join(cfg.cache_dir, f"{key}.pkl")
    if not cfg.disable_cache and not cfg.force_recache and os.path.exists(path):
        try:
            with open(path, "rb") as f:
                return pickle.load(f)
        except Exception:
            pass  # unreadable cache: rebuild
    rows = _read_rows(os.path.expanduser(source))

    def one(r):
        if cfg.messages_key in r:
            return tokenize_chat_example(r, tokenizer, cfg.max_length, cfg.messages_key, cfg.tools_key, cfg.system_key,
                                         cfg.train_on_what)
        return tokenize_sft_example(r, tokenizer, cfg.max_length)

    if cfg.num_workers and cfg.num_workers > 1 and len(rows) > 256:
        with ThreadPoolExecutor(cfg.num_workers) as ex:
            toks = list(ex.map(one, rows, chunksize=64))
    else:
        toks = [one(r) for r in rows]
    toks = [t for t in toks if t is not None]
    if not cfg.disable_cache:
        os.makedirs(cfg.cache_dir, exist_ok=True)
        tmp = path + f".tmp{os.getpid()}"
        with open(tmp, "wb") as f:
            pickle.dump(toks, f)
        os.replace(tmp, path)
    return toks


def load_pretokenized(path: str) -> List[dict]:
    """Rows that already carry ``input_ids`` (+ optional ``loss_mask`` / ``num_actions``)."""
    from .dataset import _read_rows

    out = []
    for r in _read_rows(os.path.expanduser(path)):
        ids = list(r["input_ids"])
        lm = list(r["loss_mask"]) if r.get("loss_mask") is not None else [1] * (len(ids) - 1)
        na = int(r.get("num_actions") or len(lm))
        out.append({"input_ids": ids, "attention_mask": [1] * len(ids), "loss_mask": lm[-na:], "num_actions": na})
    return out


# ----------------------------------------------------------------------------- bin packing
def ffd_pack(lengths: Sequence[int], capacity: int) -> List[List[int]]:
    """First-fit-decreasing: bins of indices whose lengths sum to at most ``capacity`` (C++ when available)."""
    n = len(lengths)
    if n == 0:
        return []
    if max(lengths) > capacity:
        raise ValueError(f"a sequence of {max(lengths)} tokens does not fit the bin capacity {capacity}")
    try:
        from ..ops import _lib

        rt = _lib.runtime()
        arr = np.asarray(lengths, dtype=np.int32)
        out = np.empty(n, dtype=np.int32)
        rt.sbrt_ffd_pack.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        nb = rt.sbrt_ffd_pack(arr.ctypes.data, n, int(capacity), out.ctypes.data)
        bins: List[List[int]] = [[] for _ in range(nb)]
        for i, b in enumerate(out.tolist()):
            bins[b].append(i)
        return [b for b in bins if b]
    except (OSError, AttributeError):
        order = sorted(range(n), key=lambda i: -lengths[i])
        bins, room = [], []
        for i in order:
            for b in range(len(bins)):
                if room[b] >= lengths[i]:
                    bins[b].append(i)
                    room[b] -= lengths[i]
                    break
            else:
                bins.append([i])
                room.append(capacity - lengths[i])
        return bins


def balanced_pack(lengths: Sequence[int], capacity: int, num_bins_multiple: int = 1) -> List[List[int]]:
    """FFD for the bin count, then longest-processing-time assignment so bins carry near-equal token counts; the
    count is rounded up to a multiple of ``num_bins_multiple`` (data-parallel ranks get equal numbers of bins)."""
    base = ffd_pack(lengths, capacity)
    k = len(base)
    if num_bins_multiple > 1:
        k = (k + num_bins_multiple - 1) // num_bins_multiple * num_bins_multiple
    k = min(max(k, 1), len(lengths)) if len(lengths) >= num_bins_multiple else k
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[List[int]] = [[] for _ in range(k)]
    load = [0] * k
    for i in order:
        cands = [b for b in range(k) if load[b] + lengths[i] <= capacity]
        b = min(cands, key=lambda j: load[j]) if cands else None
        if b is None:  # cannot happen when k >= FFD count, kept as a guard
            bins.append([i])
            load.append(lengths[i])
            k += 1
            continue
        bins[b].append(i)
        load[b] += lengths[i]
    return bins


def make_seq_packer(strategy: str = "ffd"):
    if strategy in ("ffd", "first_fit_decreasing"):
        return ffd_pack
    if strategy == "balanced":
        return balanced_pack
    raise ValueError(f"unknown packing strategy '{strategy}'")


# ----------------------------------------------------------------------------- collators
def collate_sft_batch(examples: List[dict], tokenizer) -> TrainingInputBatch:
    max_len = max(len(e["input_ids"]) for e in examples)
    max_act = max(e["num_actions"] for e in examples)
    n = len(examples)
    pad = tokenizer.pad_token_id if getattr(tokenizer, "pad_token_id", None) is not None else 0
    seq = np.full((n, max_len), pad, dtype=np.int64)
    att = np.zeros((n, max_len), dtype=np.int64)
    lmask = np.zeros((n, max_act), dtype=np.float32)
    rmask = np.zeros((n, max_act), dtype=np.int64)
    for i, e in enumerate(examples):
        L, a = len(e["input_ids"]), e["num_actions"]
        seq[i, max_len - L:] = e["input_ids"]
        att[i, max_len - L:] = e["attention_mask"]
        lmask[i, max_act - a:] = e["loss_mask"]
        rmask[i, max_act - a:] = 1
    b = TrainingInputBatch({"sequences": torch.from_numpy(seq), "attention_mask": torch.from_numpy(att),
                            "loss_mask": torch.from_numpy(lmask), "response_mask": torch.from_numpy(rmask)})
    b.metadata = {"response_length": max_act}
    return b


class DefaultCollator:
    """Left-padded rows, one example per row."""

    def __init__(self, tokenizer, micro_train_batch_size_per_gpu: int = 1):
        self.tokenizer, self.micro = tokenizer, micro_train_batch_size_per_gpu

    def __call__(self, examples: List[dict], batch_size: int) -> TrainingInputBatch:
        return collate_sft_batch(examples, self.tokenizer)


class PackedDataCollator:
    """Orders the batch by FFD bins of at most ``max_tokens`` tokens (bin count rounded up to ``dp_size``), and records
    the bins in ``metadata["pack_bins"]``; each data-parallel rank then takes whole bins so its varlen micro-batches
    are full.  (The reference concatenates each bin into one row; with a varlen kernel the row boundary carries no
    information, so the rows stay separate and only the grouping is fixed here.)"""

    def __init__(self, tokenizer, max_tokens: int, dp_size: int = 1, strategy: str = "balanced"):
        self.tokenizer, self.max_tokens, self.dp_size, self.strategy = tokenizer, max_tokens, dp_size, strategy

    def __call__(self, examples: List[dict], batch_size: int) -> TrainingInputBatch:
        lens = [len(e["input_ids"]) for e in examples]
        if self.strategy == "balanced":
            bins = balanced_pack(lens, self.max_tokens, self.dp_size)
        else:
            bins = ffd_pack(lens, self.max_tokens)
        order = [i for b in bins for i in b]
        batch = collate_sft_batch([examples[i] for i in order], self.tokenizer)
        sizes = [len(b) for b in bins]
        batch.metadata["pack_bins"] = sizes
        batch.metadata["pack_bin_tokens"] = [sum(lens[i] for i in b) for b in bins]
        return batch


def collate_sft_examples(examples: List[dict], collator, batch_size: int, pad_to_batch_size: bool = False) -> TrainingInputBatch:
    batch = collator(examples, batch_size=batch_size)
    if pad_to_batch_size and len(examples) < batch_size:
        batch = pad_training_input_batch(batch, batch_size)
    return batch


# ----------------------------------------------------------------------------- samplers
class StatefulSampler:
    """Epoch-seeded permutation with ``state_dict`` / ``load_state_dict`` (position within the epoch survives a
    restart).  ``length_grouped`` shuffles mega-batches and sorts inside them, which makes token-budget micro-batches
    denser."""

    def __init__(self, lengths: Sequence[int], batch_size: int, seed: int = 42, mode: str = "random",
                 weights: Optional[Sequence[float]] = None, drop_last: bool = False, mega: int = 50):
        self.lengths, self.batch_size, self.seed, self.mode = list(lengths), batch_size, seed, mode
        self.weights, self.drop_last, self.mega = weights, drop_last, mega
        self.epoch, self.cursor = 0, 0

    def __len__(self) -> int:
        n = len(self.lengths)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def _order(self) -> List[int]:
        n = len(self.lengths)
        g = np.random.default_rng(self.seed + self.epoch)
        if self.mode == "sequential":
            return list(range(n))
        if self.weights is not None:
            p = np.asarray(self.weights, dtype=np.float64)
            return g.choice(n, size=n, replace=True, p=p / p.sum()).tolist()
        perm = g.permutation(n)
        if self.mode == "length_grouped":
            m = self.batch_size * self.mega
            chunks = [perm[i : i + m] for i in range(0, n, m)]
            perm = np.concatenate([c[np.argsort([-self.lengths[j] for j in c], kind="stable")] for c in chunks])
        return perm.tolist()

    def __iter__(self) -> Iterator[List[int]]:
        order = self._order()
        nb = len(self)
        while self.cursor < nb:
            s = self.cursor * self.batch_size
            self.cursor += 1
            yield order[s : s + self.batch_size]
        self.epoch += 1
        self.cursor = 0

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed}

    def load_state_dict(self, s: Dict[str, int]) -> None:
        self.epoch, self.cursor, self.seed = int(s["epoch"]), int(s["cursor"]), int(s.get("seed", self.seed))
