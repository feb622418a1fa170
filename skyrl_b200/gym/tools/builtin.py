"""Built-in tool groups: SQL execution, HTTP search, sandboxed Python
(reference: skyrl-gym/skyrl_gym/tools/{sql,search,python}.py)."""

from __future__ import annotations

import json
import os
import sqlite3
import subprocess
import sys
import tempfile
import threading
from typing import Any, List, Optional

from .core import ToolGroup, tool


class SQLCodeExecutorToolGroup(ToolGroup):
    """Runs a query against ``<db_root>/<db_id>/<db_id>.sqlite`` with a wall-clock limit; returns a short table."""

    def __init__(self, db_file_path: str, timeout_s: float = 5.0, max_rows: int = 50, max_chars: int = 9000):
        self.db_root, self.timeout_s, self.max_rows, self.max_chars = db_file_path, timeout_s, max_rows, max_chars
        super().__init__("SQLCodeExecutorToolGroup")

    INVALID_ACTION = ("Your previous action is invalid. Follow the format of outputting thinking process and sql tool, "
                      "and try again.")

    @tool
    def sql(self, db_id: str, query: Optional[str], turns_left: int = 0) -> str:
        """The observation the model sees next: the result table (or the error, the timeout notice, or the note that
        no ``<sql>`` block was found) followed by a reminder of the turns left, inside one ``<observation>`` element
        (message layout of the reference's tool, skyrl-gym/skyrl_gym/tools/sql.py:88-97)."""
        return (f"\n\n<observation>{self._run(db_id, query)}\n"
                f"<reminder>You have {turns_left} turns left to complete the task.</reminder></observation>\n\n")

    def _run(self, db_id: str, query: Optional[str]) -> str:
        if query is None:
            return self.INVALID_ACTION
        db = os.path.join(self.db_root, db_id, db_id + ".sqlite")
        if not os.path.exists(db):
            return f"Error executing SQL: database '{db_id}' not found, db file: {db}"
        conn = sqlite3.connect(f"file:{db}?mode=ro", uri=True, check_same_thread=False)
        fired = threading.Event()

        def interrupt():
            fired.set()
            conn.interrupt()

        timer = threading.Timer(self.timeout_s, interrupt)
        timer.start()
        try:
            cur = conn.execute(query)
            cols = [d[0] for d in cur.description] if cur.description else []
            rows = cur.fetchall()
        except sqlite3.Error as e:
            if fired.is_set():
                return f"SQL Timeout:\n{query}"
            return f"Error executing SQL: {e}, db file: {db}"
        finally:
            timer.cancel()
            conn.close()

        def table(rs):
            return "\n".join([" | ".join(cols)] + [" | ".join(str(v) for v in r) for r in rs])

        out = table(rows)
        if len(out) > self.max_chars:
            out = f"Truncated to {self.max_rows} lines since returned response too long: " + table(rows[: self.max_rows])
        return out


class SearchToolGroup(ToolGroup):
    """POSTs ``{"queries": [q], "topk": k, "return_scores": true}`` to a retrieval server and formats the passages."""

    def __init__(self, search_url: str = "http://127.0.0.1:8000/retrieve", topk: int = 3, timeout: int = 30,
                 log_requests: bool = False, transport=None):
        self.search_url, self.topk, self.timeout, self.log_requests = search_url, topk, timeout, log_requests
        self._transport = transport  # injectable for tests: callable(url, payload, timeout) -> dict
        super().__init__("SearchToolGroup")

    def _post(self, payload: dict) -> dict:
        if self._transport is not None:
            return self._transport(self.search_url, payload, self.timeout)
        import requests

        r = requests.post(self.search_url, json=payload, timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    @staticmethod
    def _format(results: List[Any]) -> str:
        out = []
        for i, item in enumerate(results):
            doc = item.get("document", item) if isinstance(item, dict) else {"contents": str(item)}
            content = doc.get("contents", "") if isinstance(doc, dict) else str(doc)
            title, _, text = content.partition("\n")
            out.append(f"Doc {i + 1}(Title: {title.strip()}) {text.strip()}")
        return "\n".join(out)

    @tool
    def search(self, query: Optional[str]) -> str:
        if not query or not query.strip():
            return "No query found: put the search query between <search> and </search>."
        res = self._post({"queries": [query.strip()], "topk": self.topk, "return_scores": True})
        hits = (res.get("result") or [[]])[0]
        return self._format(hits) if hits else "No results."


class PythonCodeExecutorToolGroup(ToolGroup):
    """Runs a snippet in a fresh interpreter process with a time limit; returns stdout (or the error tail)."""

    def __init__(self, timeout_s: float = 10.0, max_chars: int = 4000, plain_errors: bool = False):
        """``plain_errors``: report like the reference's tool does (skyrl-gym/skyrl_gym/tools/python.py) -- stripped
        stdout, or ``Error executing Python code: <stderr>`` whenever anything was written to stderr."""
        self.timeout_s, self.max_chars, self.plain_errors = timeout_s, max_chars, plain_errors
        super().__init__("PythonCodeExecutorToolGroup")

    @tool
    def python(self, code: Optional[str], stdin: str = "") -> str:
        if not code:
            return "No code found."
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "snippet.py")
            with open(path, "w") as f:
                f.write(code)
            try:
                argv = [sys.executable, "-I", "-c", code] if self.plain_errors else [sys.executable, "-I", path]
                p = subprocess.run(argv, input=stdin, capture_output=True, text=True,
                                   timeout=self.timeout_s, cwd=d, env={"PATH": os.environ.get("PATH", "")})
            except subprocess.TimeoutExpired:
                if self.plain_errors:
                    return f"Error executing Python code: Execution timed out after {self.timeout_s} seconds."
                return f"Error: execution exceeded {self.timeout_s} s."
        if self.plain_errors:
            if p.stderr:
                return ("Error executing Python code: " + p.stderr.strip())[: self.max_chars]
            return p.stdout.strip()[: self.max_chars]
        out = p.stdout if p.returncode == 0 else (p.stdout + "\n" + p.stderr[-1500:])
        return out[: self.max_chars]


def run_python_tests(code: str, tests: List[dict], timeout_s: float = 6.0) -> List[bool]:
    """stdin/stdout test cases ``{"input": str, "output": str}`` against a program; one verdict per case."""
    ex = PythonCodeExecutorToolGroup(timeout_s=timeout_s, max_chars=1 << 20)
    verdicts = []
    for t in tests:
        got = ex.python(code, stdin=t.get("input", ""))
        verdicts.append(got.strip().split() == str(t.get("output", "")).strip().split())
    return verdicts
