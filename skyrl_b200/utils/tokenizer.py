"""Tokenizer access: HF tokenizers by path, and a dependency-free ``SyntheticTokenizer`` whose text is
the space-separated token ids -- used by plumbing tests and synthetic benchmarks where prompts are
random ids and no vocabulary file exists (reference helper: skyrl/utils/tok.py)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Union


class SyntheticTokenizer:
    """ids <-> "12 7 993" strings; chat template = [role id] + content ids + [eot id] per message.

    Special ids: 0 pad, 1 eos/eot, 2 user/system role marker, 3 assistant role marker; regular ids start at 4.
    """

    pad_token_id = 0
    eos_token_id = 1
    bos_token_id = None
    padding_side = "left"
    chat_template = "synthetic"

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size
        self.pad_token, self.eos_token = "<pad>", "<eos>"
        self.name_or_path = f"synthetic-{vocab_size}"

    def __len__(self) -> int:
        return self.vocab_size

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        out = []
        for tok in text.split():
            if tok.lstrip("-").isdigit():
                out.append(int(tok) % self.vocab_size)
            else:
                out.append(4 + (sum(tok.encode()) % max(1, self.vocab_size - 4)))
        return out

    def __call__(self, text: Union[str, List[str]], add_special_tokens: bool = False, **kw) -> Dict[str, Any]:
        if isinstance(text, str):
            return {"input_ids": self.encode(text)}
        return {"input_ids": [self.encode(t) for t in text]}

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return " ".join(str(int(i)) for i in ids if not (skip_special_tokens and int(i) < 4))

    def batch_decode(self, batch: Sequence[Sequence[int]], skip_special_tokens: bool = True) -> List[str]:
        return [self.decode(x, skip_special_tokens) for x in batch]

    def apply_chat_template(self, conversation: List[Dict[str, Any]], add_generation_prompt: bool = False,
                            tokenize: bool = True, **kw):
        ids: List[int] = []
        for m in conversation:
            ids.append(3 if m.get("role") == "assistant" else 2)
            content = m.get("content", "")
            ids.extend(content if isinstance(content, list) and all(isinstance(c, int) for c in content)
                       else self.encode(str(content)))
            ids.append(self.eos_token_id)
        if add_generation_prompt:
            ids.append(3)
        if kw.get("return_dict"):
            return {"input_ids": ids}
        return ids if tokenize else self.decode(ids, skip_special_tokens=False)

    def save_pretrained(self, path: str) -> None:
        import json
        import os

        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "synthetic_tokenizer.json"), "w") as f:
            json.dump({"vocab_size": self.vocab_size}, f)


def chat_template_ids(tokenizer, messages, **kw) -> List[int]:
    """Token ids of ``messages`` through the tokenizer's chat template, as a plain list.  Newer ``transformers``
    releases return a ``BatchEncoding`` from ``apply_chat_template(tokenize=True)`` unless told otherwise; every caller
    here wants the ids."""
    kw["tokenize"] = True
    kw["return_dict"] = False
    out = tokenizer.apply_chat_template(messages, **kw)
    if hasattr(out, "keys"):
        out = out["input_ids"]
    return list(out)


def get_tokenizer(name_or_path: Optional[str], vocab_size: Optional[int] = None, **kw):
    """HF tokenizer (left padding, pad = eos if missing) or ``SyntheticTokenizer`` for ``synthetic[-N]`` names."""
    if name_or_path is None or str(name_or_path).startswith("synthetic"):
        if vocab_size is None and name_or_path and "-" in str(name_or_path):
            tail = str(name_or_path).rsplit("-", 1)[1]
            vocab_size = int(tail) if tail.isdigit() else None
        return SyntheticTokenizer(vocab_size or 1024)
    import os

    if vocab_size is not None and not os.path.isdir(str(name_or_path)):
        # an architecture preset (random weights, no checkpoint directory): there is no vocabulary file to load
        return SyntheticTokenizer(vocab_size)
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(name_or_path, padding_side="left", **kw)
    if tok.pad_token_id is None:
        tok.pad_token = tok.eos_token
        tok.pad_token_id = tok.eos_token_id
    return tok
