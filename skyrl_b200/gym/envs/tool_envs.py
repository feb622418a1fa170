"""Multi-turn tool-use environments: retrieval search (Search-R1 style), text-to-SQL, code search, LiveCodeBench-style
program synthesis.  Behavioural references: skyrl-gym/skyrl_gym/envs/{search,sql,searchcode,lcb}/env.py.

Common protocol: the model either calls a tool by wrapping the input in a tag (``<search>..</search>``,
``<sql>..</sql>``, ``<python>..</python>``) or finishes with ``<answer>`` / ``<solution>``.  The reward is given once, on
the final turn; intermediate turns return the tool output as a user message.
"""

from __future__ import annotations

import json
import os
import re
import sqlite3
import string
from typing import Any, Dict, List, Optional

from ..tools.builtin import PythonCodeExecutorToolGroup, SearchToolGroup, SQLCodeExecutorToolGroup, run_python_tests
from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput


def _cfg(env_config: Any, key: str, default: Any) -> Any:
    if env_config is None:
        return default
    if isinstance(env_config, dict):
        return env_config.get(key, default)
    return getattr(env_config, key, default)


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def extract_tag(text: str, tag: str, last: bool = True, strip: bool = True) -> Optional[str]:
    m = re.findall(rf"<{tag}>(.*?)</{tag}>", text, re.DOTALL)
    if not m:
        return None
    out = m[-1] if last else m[0]
    return out.strip() if strip else out


def em_score(history: str, ground_truth: Any, format_score: float = 0.0) -> float:
    """Exact match of the last ``<answer>`` against any accepted target (after normalisation)."""
    ans = extract_tag(history, "answer")
    if ans is None:
        return 0.0
    targets = ground_truth.get("target", ground_truth) if isinstance(ground_truth, dict) else ground_truth
    if isinstance(targets, str):
        targets = [targets]
    na = normalize_answer(ans)
    return 1.0 if any(normalize_answer(str(t)) == na for t in targets) else format_score


class _ToolLoopEnv(BaseTextEnv):
    """Shared step logic: finish tag -> score; otherwise run the tool and return its output as the observation."""

    tool_tag = "tool"
    done_tag = "answer"
    tool_name = "tool"

    def __init__(self, extras: Dict[str, Any], default_turns: int):
        super().__init__()
        assert "reward_spec" in extras and "ground_truth" in extras["reward_spec"], "reward_spec.ground_truth is required"
        self.ground_truth = extras["reward_spec"]["ground_truth"]
        self.max_turns = int(extras.get("max_turns", default_turns))
        self.chat_history: List[Dict[str, str]] = []

    def _is_done(self, action: str) -> bool:
        return self.turns >= self.max_turns or (f"<{self.done_tag}>" in action and f"</{self.done_tag}>" in action)

    def _final_reward(self) -> float:
        raise NotImplementedError

    def _tool_input(self, action: str) -> Any:
        return (extract_tag(action, self.tool_tag, last=False, strip=False),)  # the tool sees the text as written

    def _wrap(self, out: str) -> str:
        return out

    def step(self, action: str) -> BaseTextEnvStepOutput:
        self.turns += 1
        self.chat_history.append({"role": "assistant", "content": action})
        if self._is_done(action):
            return BaseTextEnvStepOutput(observations=[], reward=float(self._final_reward()), done=True, metadata={})
        group = self.tool_groups[0]
        tool_input = None
        try:
            tool_input = self._tool_input(action)
            obs = self._wrap(self._execute_tool(group.get_name(), self.tool_name, tool_input))
        except Exception as e:  # noqa: BLE001 - the error text is the observation
            obs = str(e)
        msg = {"role": "user", "content": obs}
        self.chat_history.append(msg)
        return BaseTextEnvStepOutput(observations=[msg], reward=0.0, done=False,
                                     metadata={"tool_group": group.get_name(), "tool_name": self.tool_name,
                                               "tool_input": tool_input})


class SearchEnv(_ToolLoopEnv):
    tool_tag, done_tag, tool_name = "search", "answer", "search"

    def __init__(self, env_config: Any = None, extras: Optional[Dict[str, Any]] = None):
        super().__init__(extras or {}, default_turns=2)
        self.init_tool_groups([SearchToolGroup(_cfg(env_config, "search_url", "http://127.0.0.1:8000/retrieve"),
                                               _cfg(env_config, "topk", 3), _cfg(env_config, "timeout", 30),
                                               _cfg(env_config, "log_requests", False),
                                               transport=(extras or {}).get("_transport"))])

    def _wrap(self, out: str) -> str:
        return "\n<information>" + out + "</information>\n"

    def _final_reward(self) -> float:
        return em_score("".join(m["content"] for m in self.chat_history), self.ground_truth)


class SearchCodeEnv(BaseTextEnv):
    """Several tools behind one calling convention: ``<tool><name>input</name></tool>`` with ``name`` one of the
    registered tools (``search``, ``python``).  The episode ends on ``<solution>...</solution>`` or after
    ``max_turns``; the reward is the GSM8K-style exact match of ``#### answer`` over the whole conversation.  A call
    that cannot be parsed comes back as the observation text.  Reference: skyrl-gym/skyrl_gym/envs/searchcode/env.py."""

    def __init__(self, env_config: Any = None, extras: Optional[Dict[str, Any]] = None):
        super().__init__()
        extras = extras or {}
        assert "reward_spec" in extras, "reward_spec field is required"
        assert "ground_truth" in extras["reward_spec"], "ground_truth is required in reward_spec field"
        self.ground_truth = str(extras["reward_spec"]["ground_truth"])
        self.max_turns = int(extras.get("max_turns", 2))
        self.init_tool_groups([SearchToolGroup(_cfg(env_config, "search_url", "http://127.0.0.1:8000/retrieve"),
                                               _cfg(env_config, "topk", 3), _cfg(env_config, "timeout", 30),
                                               _cfg(env_config, "log_requests", False), transport=extras.get("_transport")),
                               PythonCodeExecutorToolGroup(plain_errors=True)])
        self.chat_history: List[Dict[str, str]] = []

    def _parse_action(self, action: str):
        block = re.search(r"<tool>(.*?)</tool>", action, re.DOTALL)
        if not block:
            raise ValueError("No <tool>...</tool> block found in action string.")
        inner = re.search(r"<(\w+)>(.*?)</\1>", block.group(1).strip(), re.DOTALL)
        if not inner:
            raise ValueError("No valid inner tool tag found inside <tool> block.")
        name, arg = inner.group(1), inner.group(2).strip()
        if name not in self.tool_to_toolgroup:
            raise ValueError(f"Tool '{name}' not found in any registered tool group.")
        return self.tool_to_toolgroup[name], name, [arg]

    def _is_done(self, action: str) -> bool:
        return self.turns >= self.max_turns or ("<solution>" in action and "</solution>" in action)

    def step(self, action: str) -> BaseTextEnvStepOutput:
        from .math_utils import extract_gsm8k_answer

        self.turns += 1
        self.chat_history.append({"role": "assistant", "content": action})
        if self._is_done(action):
            found = extract_gsm8k_answer("\n".join(m["content"] for m in self.chat_history), "strict")
            return BaseTextEnvStepOutput(observations=[], reward=1.0 if found == self.ground_truth else 0.0, done=True,
                                         metadata={})
        group = name = None
        arg: Any = ""
        try:
            group, name, arg = self._parse_action(action)
            text = self._execute_tool(group, name, arg)
        except Exception as e:  # noqa: BLE001 - the error text is the observation
            group = name = None
            arg, text = "", str(e)
        obs = [{"role": "user", "content": text}] if text else []
        self.chat_history.extend(obs)
        return BaseTextEnvStepOutput(observations=obs, reward=0.0, done=False,
                                     metadata={"tool_group": group, "tool_name": name, "tool_input": arg,
                                               "tools": [g.get_tool_names() for g in self.tool_groups]})


def _run_sql(db_file: str, sql: str, timeout_s: float = 10.0):
    import threading

    conn = sqlite3.connect(f"file:{db_file}?mode=ro", uri=True, check_same_thread=False)
    t = threading.Timer(timeout_s, conn.interrupt)
    t.start()
    try:
        return frozenset(conn.execute(sql).fetchall())
    finally:
        t.cancel()
        conn.close()


def verify_format_and_extract(output: str):
    """``(valid, thoughts, solution, None)`` for a whole trajectory's text.  Valid means: exactly one ``<solution>`` and
    one ``</solution>`` after it, no think / sql / observation tag inside the solution, at least one complete
    ``<think>`` block somewhere, and every ``</observation>`` before the solution followed (after whitespace) by a
    ``<think>``.  Rules of the reference's scorer (skyrl-gym/skyrl_gym/envs/sql/utils.py:21-45)."""
    if output.count("<solution>") != 1:
        return False, None, None, None
    before, after = output.split("<solution>", 1)
    if after.count("</solution>") != 1:
        return False, None, None, None
    solution = after.split("</solution>", 1)[0]
    if re.search(r"</?(think|sql|observation)\b", solution, re.I):
        return False, None, None, None
    thoughts = re.findall(r"<think>(.*?)</think>", output, re.S)
    if not thoughts:
        return False, None, None, None
    for m in re.finditer(r"</observation>", before, re.I):
        if not before[m.end():].lstrip().lower().startswith("<think>"):
            return False, None, None, None
    return True, thoughts, solution.strip(), None


def sql_score(history: str, gold_sql: str, db_file: str) -> float:
    """-1 when the trajectory breaks the think / sql / solution format, else 1 if the solution query returns the same
    row set as the gold query and 0 if not (a query that fails to run counts as a wrong result)."""
    ok, _, sol, _ = verify_format_and_extract(history)
    if not ok:
        return -1.0
    sol = re.sub(r"^```(?:sql)?|```$", "", sol.strip(), flags=re.MULTILINE).strip()
    try:
        pred = _run_sql(db_file, sol)
    except sqlite3.Error:
        return 0.0
    try:
        return 1.0 if pred == _run_sql(db_file, gold_sql) else 0.0
    except sqlite3.Error:
        return 0.0


class Text2SQLEnv(_ToolLoopEnv):
    tool_tag, done_tag, tool_name = "sql", "solution", "sql"
    _SUBDIR = {"synsql": "SynSQL-2.5M/databases", "spider": "spider/database", "bird": "bird/train/train_databases"}

    def __init__(self, env_config: Any = None, extras: Optional[Dict[str, Any]] = None):
        extras = extras or {}
        assert "db_id" in extras and "data" in extras, "db_id and data fields are required"
        super().__init__(extras, default_turns=5)
        root = _cfg(env_config, "db_path", os.path.expanduser("~/data/sql"))
        if extras["data"] not in self._SUBDIR:
            raise NotImplementedError(f"unknown text2sql task '{extras['data']}'")
        self.db_root = os.path.join(root, self._SUBDIR[extras["data"]])
        self.db_id = extras["db_id"]
        self.db_file = os.path.join(self.db_root, self.db_id, self.db_id + ".sqlite")
        if not os.path.exists(self.db_file):
            raise FileNotFoundError(f"Database file not found at: {self.db_file}")
        self.init_tool_groups([SQLCodeExecutorToolGroup(self.db_root)])

    def _tool_input(self, action: str) -> Any:
        return (self.db_id, extract_tag(action, "sql", last=False), self.max_turns - self.turns)

    def _final_reward(self) -> float:
        return sql_score("".join(m["content"] for m in self.chat_history), self.ground_truth, self.db_file)


class LiveCodeBenchEnv(BaseTextEnv):
    """Single turn: the last fenced code block is run against the stdin/stdout tests in
    ``reward_spec.ground_truth`` (a JSON list of ``{"input", "output"}``); reward 1 only if every test passes."""

    def __init__(self, env_config: Any = None, extras: Optional[Dict[str, Any]] = None):
        super().__init__()
        extras = extras or {}
        assert "reward_spec" in extras and "ground_truth" in extras["reward_spec"], "reward_spec.ground_truth is required"
        gt = extras["reward_spec"]["ground_truth"]
        self.tests = json.loads(gt) if isinstance(gt, str) else list(gt)
        self.timeout_s = float(extras.get("timeout_s", 6.0))

    @staticmethod
    def extract_code(text: str) -> Optional[str]:
        blocks = re.findall(r"```(?:python|py)?\n(.*?)```", text, re.DOTALL)
        return blocks[-1] if blocks else None

    def step(self, action: str) -> BaseTextEnvStepOutput:
        code = self.extract_code(action)
        if code is None:
            return BaseTextEnvStepOutput(observations=[], reward=0.0, done=True, metadata={"error": "no code block"})
        verdicts = run_python_tests(code, self.tests, self.timeout_s)
        return BaseTextEnvStepOutput(observations=[], reward=1.0 if verdicts and all(verdicts) else 0.0, done=True,
                                     metadata={"passed": sum(verdicts), "total": len(verdicts)})
