"""REPL-driven long-context environment ("recursive language model" setting): the prompt's context lives in a
persistent Python namespace as ``context``; the model inspects it by emitting ```` ```repl ```` blocks and finishes
with ``FINAL(text)`` or ``FINAL_VAR(name)``.  Behavioural reference: skyrl-gym/skyrl_gym/envs/rlm/{env,repl}.py.

The namespace persists across turns of one episode.  Code runs in-process with a restricted set of builtins and a
per-block time limit enforced from a helper thread; this is an isolation *convenience* for well-behaved policies, not a
security boundary -- run untrusted policies inside a container.
"""

from __future__ import annotations

import contextlib
import ctypes
import io
import re
import threading
from typing import Any, Dict, List, Optional

from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput
from .tool_envs import normalize_answer

_SAFE_BUILTINS = ["abs", "all", "any", "bool", "dict", "enumerate", "filter", "float", "int", "isinstance", "len", "list",
                  "map", "max", "min", "print", "range", "repr", "reversed", "round", "set", "sorted", "str", "sum",
                  "tuple", "zip", "Exception", "ValueError", "KeyError", "IndexError", "TypeError", "iter", "next",
                  "ord", "chr", "divmod", "pow", "slice", "type", "hasattr", "getattr", "format"]
_ALLOWED_IMPORTS = {"re", "json", "math", "collections", "itertools", "statistics", "string", "datetime", "functools"}


class PersistentREPL:
    def __init__(self, context: Any, timeout_s: float = 10.0, max_output_chars: int = 6000, tools: Optional[dict] = None):
        import builtins

        def _imp(name, *a, **k):
            if name.split(".")[0] not in _ALLOWED_IMPORTS:
                raise ImportError(f"import of '{name}' is not allowed in this REPL")
            return __import__(name, *a, **k)

        safe = {k: getattr(builtins, k) for k in _SAFE_BUILTINS}
        safe["__import__"] = _imp
        self.ns: Dict[str, Any] = {"__builtins__": safe, "context": context}
        self.ns["SHOW_VARS"] = lambda: {k: type(v).__name__ for k, v in self.ns.items()
                                        if not k.startswith("__") and k not in ("SHOW_VARS",) and not callable(v)}
        for name, fn in (tools or {}).items():
            self.ns[name] = fn
        self.timeout_s, self.max_output_chars = timeout_s, max_output_chars

    def run(self, code: str) -> str:
        buf = io.StringIO()
        err: List[str] = []
        done = threading.Event()

        def target():
            try:
                with contextlib.redirect_stdout(buf):
                    exec(compile(code, "<repl>", "exec"), self.ns)  # noqa: S102 - the purpose of this environment
            except BaseException as e:  # noqa: BLE001
                err.append(f"{type(e).__name__}: {e}")
            finally:
                done.set()

        t = threading.Thread(target=target, daemon=True)
        t.start()
        if not done.wait(self.timeout_s):
            # ask the interpreter to raise inside the worker thread; it stops at its next bytecode boundary
            ctypes.pythonapi.PyThreadState_SetAsyncExc(ctypes.c_ulong(t.ident), ctypes.py_object(TimeoutError))
            done.wait(1.0)
            err.append(f"TimeoutError: block exceeded {self.timeout_s} s")
        out = buf.getvalue()
        if err:
            out += ("\n" if out else "") + err[0]
        if len(out) > self.max_output_chars:
            out = out[: self.max_output_chars] + f"\n... [{len(out) - self.max_output_chars} characters truncated]"
        return out or "(no output)"

    def get(self, name: str) -> Any:
        return self.ns.get(name)


_REPL_BLOCK = re.compile(r"```repl\s*\n(.*?)```", re.DOTALL)
_FINAL_VAR = re.compile(r"FINAL_VAR\(\s*([A-Za-z_][A-Za-z_0-9]*)\s*\)")
_FINAL = re.compile(r"FINAL\((.*)\)", re.DOTALL)


class RLMEnv(BaseTextEnv):
    """``extras``: ``context`` (any JSON-able object), ``reward_spec.ground_truth`` (string or list), optional
    ``max_turns`` (default 10), ``root_prompt``.  Reward: 1 for a normalised exact match (or containment when
    ``reward_spec.method == "contains"``), else 0."""

    def __init__(self, env_config: Any = None, extras: Optional[Dict[str, Any]] = None):
        super().__init__()
        extras = extras or {}
        assert "reward_spec" in extras and "ground_truth" in extras["reward_spec"], "reward_spec.ground_truth is required"
        self.ground_truth = extras["reward_spec"]["ground_truth"]
        self.method = extras["reward_spec"].get("method", "exact")
        self.max_turns = int(extras.get("max_turns", 10))
        self.root_prompt = extras.get("root_prompt")
        self.repl = PersistentREPL(extras.get("context", ""), timeout_s=float(extras.get("repl_timeout_s", 10.0)))

    def _score(self, answer: Optional[str]) -> float:
        if answer is None:
            return 0.0
        targets = self.ground_truth if isinstance(self.ground_truth, (list, tuple)) else [self.ground_truth]
        na = normalize_answer(str(answer))
        if self.method == "contains":
            return 1.0 if any(normalize_answer(str(t)) in na for t in targets) else 0.0
        return 1.0 if any(normalize_answer(str(t)) == na for t in targets) else 0.0

    def _next_prompt(self) -> str:
        root = f' to answer the original prompt: "{self.root_prompt}"' if self.root_prompt else ""
        return ("Think step by step about what to do with the REPL (it holds `context`)" + root +
                ". Continue by writing a ```repl``` block, or finish with FINAL(...) / FINAL_VAR(name). Your next action:")

    def step(self, action: str) -> BaseTextEnvStepOutput:
        self.turns += 1
        blocks = _REPL_BLOCK.findall(action)
        outside = _REPL_BLOCK.sub("", action)
        mv = _FINAL_VAR.search(outside)
        mf = _FINAL.search(outside) if mv is None else None
        outputs = [self.repl.run(b) for b in blocks]
        if mv is not None and not blocks:  # the variable must exist from an earlier turn
            val = self.repl.get(mv.group(1))
            if val is None:
                msg = f"Variable '{mv.group(1)}' does not exist. Create it in a ```repl``` block first."
                if self.turns >= self.max_turns:
                    return BaseTextEnvStepOutput(observations=[], reward=0.0, done=True, metadata={"final": None})
                return BaseTextEnvStepOutput(observations=[{"role": "user", "content": msg}], reward=0.0, done=False, metadata={})
            return BaseTextEnvStepOutput(observations=[], reward=self._score(str(val)), done=True, metadata={"final": str(val)})
        if mf is not None and not blocks:
            ans = mf.group(1).strip()
            return BaseTextEnvStepOutput(observations=[], reward=self._score(ans), done=True, metadata={"final": ans})
        if self.turns >= self.max_turns:
            return BaseTextEnvStepOutput(observations=[], reward=0.0, done=True, metadata={"final": None})
        parts = [f"REPL output {i + 1}:\n{o}" for i, o in enumerate(outputs)] or ["No ```repl``` block found."]
        content = "\n\n".join(parts) + "\n\n" + self._next_prompt()
        return BaseTextEnvStepOutput(observations=[{"role": "user", "content": content}], reward=0.0, done=False,
                                     metadata={"n_blocks": len(blocks)})
