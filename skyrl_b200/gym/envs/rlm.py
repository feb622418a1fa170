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
    """``lm_callback(prompts: list[str]) -> list[str]`` makes ``llm_query`` / ``llm_query_batched`` available to the
    code; ``subcall_fn(prompt) -> str`` (a child agent with its own REPL) backs ``rlm_query`` / ``rlm_query_batched``,
    which fall back to the plain calls without it.  Failures come back as ``Error: LM query failed: ...`` strings, so
    a flaky endpoint does not kill the episode; the four names are put back after every block, so the code cannot
    shadow them for good (reference: skyrl-gym/skyrl_gym/envs/rlm/repl.py)."""

    def __init__(self, context: Any = "", timeout_s: float = 10.0, max_output_chars: int = 6000, tools: Optional[dict] = None,
                 lm_callback=None, subcall_fn=None):
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
        self.lm_callback, self.subcall_fn = lm_callback, subcall_fn
        self._scaffold: Dict[str, Any] = {}
        if lm_callback is not None:
            self._scaffold = {"llm_query": self._llm_query, "llm_query_batched": self._llm_query_batched,
                              "rlm_query": self._rlm_query, "rlm_query_batched": self._rlm_query_batched}
            self.ns.update(self._scaffold)

    # the namespace under its reference name
    @property
    def globals(self) -> Dict[str, Any]:
        return self.ns

    def _llm_query_batched(self, prompts, model=None) -> List[str]:
        prompts = [str(p) for p in prompts]
        try:
            out = list(self.lm_callback(prompts))
            if len(out) != len(prompts):
                raise ValueError(f"{len(out)} answers for {len(prompts)} prompts")
            return [str(o) for o in out]
        except Exception as e:  # noqa: BLE001 - reported to the model as text
            return [f"Error: LM query failed: {e}"] * len(prompts)

    def _llm_query(self, prompt, model=None) -> str:
        return self._llm_query_batched([prompt])[0]

    def _rlm_query(self, prompt, context=None) -> str:
        if self.subcall_fn is None:
            return self._llm_query(prompt)
        try:
            return str(self.subcall_fn(str(prompt)))
        except Exception as e:  # noqa: BLE001
            return f"Error: RLM query failed: {e}"

    def _rlm_query_batched(self, prompts, context=None) -> List[str]:
        prompts = [str(p) for p in prompts]
        if self.subcall_fn is None:
            return self._llm_query_batched(prompts)
        if len(prompts) <= 1:
            return [self._rlm_query(p) for p in prompts]
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=min(8, len(prompts))) as ex:  # children run side by side; order is kept
            return list(ex.map(self._rlm_query, prompts))

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
        self.ns.update(self._scaffold)  # whatever the block did to the LM helpers' names is undone
        out = buf.getvalue()
        if err:
            out += ("\n" if out else "") + err[0]
        if len(out) > self.max_output_chars:
            out = out[: self.max_output_chars] + f"\n... [{len(out) - self.max_output_chars} characters truncated]"
        return out or "(no output)"

    def get(self, name: str) -> Any:
        return self.ns.get(name)

    def execute(self, code: str):
        """``run`` under the reference's name: an object with ``.stdout``."""
        from types import SimpleNamespace

        return SimpleNamespace(stdout=self.run(code))


_REPL_BLOCK = re.compile(r"```repl\s*\n(.*?)```", re.DOTALL)
_FINAL_VAR = re.compile(r"FINAL_VAR\(\s*([A-Za-z_][A-Za-z_0-9]*)\s*\)")
_FINAL = re.compile(r"FINAL\((.*)\)", re.DOTALL)


class RLMEnv(BaseTextEnv):
    """``extras``: ``context`` (any JSON-able object), ``reward_spec.ground_truth`` (string or list), optional
    ``max_turns`` (default 10), ``root_prompt``.  Reward: 1 for a normalised exact match (or containment when
    ``reward_spec.method == "contains"``), else 0."""

    LM_TOOLS_NOTE = ("LM query tools available in the REPL:\n"
                     "- `llm_query(prompt)`: one direct call to a language model, returns str\n"
                     "- `llm_query_batched(prompts)`: several calls at once, returns list[str]\n"
                     "- `rlm_query(prompt)`: a child agent with its own REPL works on the prompt, returns str\n"
                     "- `rlm_query_batched(prompts)`: several child agents side by side, returns list[str]")

    def __init__(self, env_config: Any = None, extras: Optional[Dict[str, Any]] = None):
        super().__init__()
        extras = extras or {}
        assert "reward_spec" in extras and "ground_truth" in extras["reward_spec"], "reward_spec.ground_truth is required"
        self.extras = extras
        self.ground_truth = extras["reward_spec"]["ground_truth"]
        self.method = extras["reward_spec"].get("method", "exact")
        self.max_turns = int(extras.get("max_turns", 10))
        self.root_prompt = extras.get("root_prompt")
        # injected by the generator (``RLMGenerator``): callables, not data
        self.lm_callback, self.subcall_fn = extras.get("lm_callback"), extras.get("subcall_fn")
        self.depth = int(extras.get("depth", 0))
        context = extras.get("context")
        if context is None:
            context = (extras.get("extra_info") or {}).get("context_text", "")
        self._context = context
        self._final: Optional[str] = None
        self._reward = 0.0
        self.repl = PersistentREPL(context, timeout_s=float(extras.get("repl_timeout_s", extras.get(
                                       "repl_timeout", 180.0 if self.lm_callback is not None else 10.0))),
                                   tools=self._get_repl_tools(), lm_callback=self.lm_callback, subcall_fn=self.subcall_fn)

    # ------------------------------------------------------------------ hooks for task-specific subclasses
    def _get_repl_tools(self) -> Dict[str, Any]:
        """Extra names for the REPL (``self._context`` is set when this runs, so closures may capture it)."""
        return {}

    def _get_system_prompt(self) -> str:
        return ("You answer a question about a long context that does not fit in your prompt. The context is the Python "
                "variable `context` in a persistent REPL. Inspect it by writing ```repl``` code blocks (their printed "
                "output comes back to you), keep intermediate results in variables, and finish with FINAL(answer) or "
                "FINAL_VAR(variable_name).{custom_tools_section}")

    def _get_reward(self, final_answer: str) -> float:
        return self._score(final_answer)

    def init(self, prompt):
        """System prompt (with the LM helpers' description when a callback is present), a note on the context's type
        and size, then the caller's messages."""
        tools = self._get_repl_tools()
        section = ""
        if self.lm_callback is not None:
            section += "\n\n" + self.LM_TOOLS_NOTE
        if tools:
            section += "\n\nCustom tools and data available in the REPL: " + ", ".join(f"`{k}`" for k in sorted(tools))
        system = self._get_system_prompt().replace("{custom_tools_section}", section)
        c = self._context
        size = len(c) if hasattr(c, "__len__") else 0
        meta = f"`context` is a {type(c).__name__} of length {size}."
        if self.root_prompt is None:
            self.root_prompt = "\n".join(str(m.get("content", "")) for m in prompt if m.get("role") == "user") or None
        msgs = [{"role": "system", "content": system}, {"role": "user", "content": meta}]
        return msgs + [dict(m) for m in prompt if m.get("role") != "system"], {}

    def get_metrics(self) -> Dict[str, Any]:
        return {"turns_used": self.turns, "final_value_set": self._final is not None, "final_answer": self._final,
                "reward": self._reward, "depth": self.depth}

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

    def _finish(self, answer: str) -> BaseTextEnvStepOutput:
        self._final, self._reward = answer, float(self._get_reward(answer))
        return BaseTextEnvStepOutput(observations=[], reward=self._reward, done=True, metadata={"final": answer})

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
            return self._finish(str(val))
        if mf is not None and not blocks:
            return self._finish(mf.group(1).strip())
        if self.turns >= self.max_turns:
            return BaseTextEnvStepOutput(observations=[], reward=0.0, done=True, metadata={"final": None})
        parts = [f"REPL output {i + 1}:\n{o}" for i, o in enumerate(outputs)] or ["No ```repl``` block found."]
        content = "\n\n".join(parts) + "\n\n" + self._next_prompt()
        return BaseTextEnvStepOutput(observations=[{"role": "user", "content": content}], reward=0.0, done=False,
                                     metadata={"n_blocks": len(blocks)})
