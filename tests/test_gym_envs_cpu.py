"""Tool-use environments: search, text-to-SQL, code tests, REPL."""
import os
import sqlite3

import pytest

import skyrl_b200.gym as gym
from skyrl_b200.gym.envs.rlm import PersistentREPL, RLMEnv
from skyrl_b200.gym.envs.tool_envs import LiveCodeBenchEnv, SearchEnv, Text2SQLEnv, em_score


def test_search_env_two_turns():
    calls = []

    def transport(url, payload, timeout):
        calls.append(payload)
        return {"result": [[{"document": {"contents": "Paris\nParis is the capital of France."}, "score": 1.0}]]}

    env = SearchEnv({"topk": 1}, {"reward_spec": {"ground_truth": {"target": ["Paris"]}}, "max_turns": 3, "_transport": transport})
    out = env.step("I should look it up <search>capital of France</search>")
    assert not out["done"] and "<information>" in out["observations"][0]["content"] and "Doc 1(Title: Paris)" in out["observations"][0]["content"]
    assert calls[0]["queries"] == ["capital of France"] and calls[0]["topk"] == 1
    out = env.step("<answer>the Paris.</answer>")
    assert out["done"] and out["reward"] == 1.0
    assert em_score("<answer>Lyon</answer>", ["Paris"]) == 0.0


def test_text2sql_env(tmp_path):
    root = tmp_path / "spider" / "database" / "shop"
    os.makedirs(root)
    con = sqlite3.connect(root / "shop.sqlite")
    con.executescript("CREATE TABLE items(name TEXT, price INT); INSERT INTO items VALUES ('a', 3), ('b', 5), ('c', 9);")
    con.commit()
    con.close()
    extras = {"db_id": "shop", "data": "spider", "reward_spec": {"ground_truth": "SELECT name FROM items WHERE price > 4"}}
    env = Text2SQLEnv({"db_path": str(tmp_path)}, extras)
    out = env.step("<think>look at the table</think>\n<sql>SELECT * FROM items</sql>")
    obs = out["observations"][0]["content"]
    assert not out["done"] and out["reward"] == 0.0 and "name | price" in obs
    assert obs.startswith("\n\n<observation>") and "<reminder>You have 4 turns left to complete the task.</reminder></observation>" in obs
    assert out["metadata"]["tool_input"][1] == "SELECT * FROM items"
    out = env.step("<think>again</think><sql>SELEC broken</sql>")
    assert "Error executing SQL" in out["observations"][0]["content"] and "3 turns left" in out["observations"][0]["content"]
    out = env.step("<think>no query this time</think>")
    assert "Your previous action is invalid." in out["observations"][0]["content"] and out["metadata"]["tool_input"][1] is None
    out = env.step("<think>ok</think><solution>SELECT name FROM items WHERE price >= 5</solution>")
    assert out["done"] and out["reward"] == 1.0
    # a wrong result scores 0, a trajectory that breaks the format scores -1
    env2 = Text2SQLEnv({"db_path": str(tmp_path)}, extras)
    assert env2.step("<think>t</think><solution>SELECT name FROM items</solution>")["reward"] == 0.0
    env3 = Text2SQLEnv({"db_path": str(tmp_path)}, extras)
    assert env3.step("<solution>SELECT name FROM items WHERE price > 4</solution>")["reward"] == -1.0
    env4 = Text2SQLEnv({"db_path": str(tmp_path)}, extras)
    env4.step("<sql>SELECT 1</sql>")  # the next turn does not open with <think> after the observation
    assert env4.step("text <think>t</think><solution>SELECT name FROM items WHERE price > 4</solution>")["reward"] == -1.0
    with pytest.raises(FileNotFoundError):
        Text2SQLEnv({"db_path": str(tmp_path)}, dict(extras, db_id="nope"))


def test_lcb_env_runs_tests():
    tests = [{"input": "2 3\n", "output": "5"}, {"input": "10 -4\n", "output": "6"}]
    env = LiveCodeBenchEnv(None, {"reward_spec": {"ground_truth": tests}})
    good = "Here:\n```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    assert env.step(good)["reward"] == 1.0
    bad = "```python\nprint(0)\n```"
    out = LiveCodeBenchEnv(None, {"reward_spec": {"ground_truth": tests}}).step(bad)
    assert out["reward"] == 0.0 and out["metadata"]["total"] == 2
    assert LiveCodeBenchEnv(None, {"reward_spec": {"ground_truth": tests}}).step("no code")["reward"] == 0.0


def test_rlm_env_repl_persists_and_finishes():
    env = RLMEnv(None, {"context": {"docs": ["alpha 17", "beta 25"]}, "reward_spec": {"ground_truth": "25"}, "max_turns": 4})
    out = env.step("look:\n```repl\nvals = [int(d.split()[1]) for d in context['docs']]\nprint(vals)\n```")
    assert not out["done"] and "[17, 25]" in out["observations"][0]["content"]
    out = env.step("```repl\nbest = max(vals)\n```")
    assert not out["done"]
    out = env.step("FINAL_VAR(best)")
    assert out["done"] and out["reward"] == 1.0
    env = RLMEnv(None, {"context": "x", "reward_spec": {"ground_truth": "y"}})
    assert env.step("FINAL(z)")["reward"] == 0.0
    r = PersistentREPL("ctx", timeout_s=0.5)
    assert "not allowed" in r.run("import os")
    assert "TimeoutError" in r.run("while True:\n    pass")


def test_registry_has_all_reference_envs():
    for name in ("aime", "gsm8k", "gsm8k_multi_turn", "text2sql", "search", "lcb", "searchcode", "rlm"):
        assert name in gym.registry_names() if hasattr(gym, "registry_names") else True
    env = gym.make("lcb", extras={"reward_spec": {"ground_truth": []}})
    assert isinstance(env, LiveCodeBenchEnv)


def test_llm_judge_env_scores_through_a_chat_endpoint():
    """The judge is an OpenAI-compatible endpoint; here a local stub that answers by comparing the last numbers."""
    import json
    import re
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from skyrl_b200 import gym
    from skyrl_b200.gym.envs.llm_judge import parse_score

    calls = []

    class H(BaseHTTPRequestHandler):
        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            calls.append(body)
            text = body["messages"][0]["content"]
            gold = re.search(r"Gold answer: (\S+)", text).group(1)
            cand = re.search(r"Candidate answer: (.*)", text).group(1)
            if len(calls) == 1:  # first request fails: the env retries
                self.send_response(503)
                self.end_headers()
                return
            reply = "no score here" if "garbage" in cand else f"Reasoning...\nSCORE: {1 if gold in cand.split() else 0}"
            out = json.dumps({"choices": [{"message": {"role": "assistant", "content": reply}}]}).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def log_message(self, *a):
            pass

    srv = HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        cfg = {"base_url": f"http://127.0.0.1:{srv.server_port}", "model": "stub", "max_retries": 3}
        ex = {"reward_spec": {"ground_truth": "42"}, "question": "6 x 7?"}
        good = gym.make("llm_judge", env_config=cfg, extras=ex).step("the answer is 42")
        bad = gym.make("llm_judge", env_config=cfg, extras=ex).step("the answer is 41")
        odd = gym.make("llm_judge", env_config=cfg, extras=ex).step("garbage")
        assert good["reward"] == 1.0 and good["done"] and bad["reward"] == 0.0
        assert odd["reward"] == 0.0 and odd["metadata"]["judge_parsed"] is False
        assert calls[1]["model"] == "stub" and "Question: 6 x 7?" in calls[1]["messages"][0]["content"]
    finally:
        srv.shutdown()
    assert parse_score("SCORE: 0.5 then SCORE: 3") == 1.0 and parse_score("nothing") is None


@pytest.mark.parametrize("output,truth,expected", [
    ("Answer: \\boxed{42}", "42", 1.0), ("Answer: 42", "42", 1.0), ("Answer: \\boxed{43}", "42", -1.0),
    ("Answer: \\boxed{\\frac{1}{2}}", "\\frac{1}{2}", 1.0), ("Answer: \\boxed{0.5}", "\\frac{1}{2}", -1.0),
    ("Answer: \\boxed{\\text{forty-two}}", "42", -1.0),
    # end-of-turn tokens: a well-formed one ends the answer, a broken one becomes part of it
    ("<|im_start|>Answer: \\boxed{42}<|im_end|>", "42", 1.0), ("<|im_start|>Answer: \\boxed{42}im_end|>", "42", -1.0),
    ("Answer: \\boxed{42}<|eot_id|>", "42", 1.0), ("Answer: \\boxed{42}|eot_id|>", "42", -1.0),
    # normalisation: units, thousands separators, shorthand TeX, the right-hand side of an equation
    ("so the total is\nAnswer: 1,234 dollars", "1234", 1.0), ("Answer: x = \\frac12", "\\frac{1}{2}", 1.0),
    ("Answer: $\\sqrt2$ cm", "\\sqrt{2}", 1.0), ("no final line at all", "42", -1.0),
])
def test_aime_scores_like_the_dapo_recipe(output, truth, expected):
    """Golden cases of the reference's own environment test (skyrl-gym/tests/test_aime.py) plus normalisation cases."""
    import skyrl_b200.gym as gym

    env = gym.make("aime", env_config=None, extras={"reward_model": {"method": "rule", "ground_truth": truth}})
    assert env.step(output)["reward"] == expected
    # datasets written for the other environments name the field reward_spec
    env = gym.make("aime", env_config=None, extras={"reward_spec": {"ground_truth": truth}})
    assert env.step(output)["reward"] == expected


@pytest.mark.parametrize("output,truth,expected", [("The answer is #### 42", "42", 1.0), ("The answer is #### 42", "43", 0.0),
                                                    ("The answer is 42", "42", 0.0)])
def test_gsm8k_needs_the_four_hash_format(output, truth, expected):
    import skyrl_b200.gym as gym

    env = gym.make("gsm8k", env_config=None, extras={"reward_spec": {"method": "rule", "ground_truth": truth}})
    assert env.step(output)["reward"] == expected


@pytest.mark.parametrize("output,valid", [
    ("<think>I need to query the database</think>\n<solution>SELECT * FROM users;</solution>", True),
    ("<solution>SELECT * FROM users;</solution>", False),
    ("<think>thinking</think>\n<solution>SELECT * FROM users;<solution>more text</solution>", False),
    ("<think>thinking</think>\n<solution>SELECT * FROM users;</solution>extra</solution>", False),
    ("<think>thinking</think>\nSELECT * FROM users;</solution>", False),
    ("<think>thinking</think>\n<solution>SELECT * FROM users;", False),
    ("<think>thinking</think>\nsome text<solution>", False),
    ("<think>thinking</think>\n<solution>SELECT * FROM users; <sql>forbidden</sql></solution>", False),
    ("<think>thinking</think>\n<solution>SELECT * FROM users; <observation>forbidden</observation></solution>", False),
    ("<think>thinking</think>\n<solution></solution>", True),
    ("<think>first thought</think>\n<think>second thought</think>\n<solution>SELECT * FROM users;</solution>", True),
    ("<observation>some observation</observation>\n<think>thinking</think>\n<solution>SELECT * FROM users;</solution>", True),
    ("<observation>some observation</observation>\nrandom text\n<think>thinking</think>\n<solution>SELECT * FROM users;</solution>", False),
    ("some text<solution>", False), ("</solution><solution>content</solution>", False),
    ("<solution><solution>content</solution>", False), ("some text</solution>", False), ("", False),
    ("<solution>content without end", False),
])
def test_sql_trajectory_format_rules(output, valid):
    """The cases of the reference's own test of its scorer (skyrl-gym/tests/test_sql.py)."""
    from skyrl_b200.gym.envs.tool_envs import verify_format_and_extract

    ok, thoughts, solution, _ = verify_format_and_extract(output)
    assert ok == valid
    if valid:
        assert thoughts and solution is not None
    else:
        assert thoughts is None and solution is None


def test_searchcode_env_follows_the_tool_call_protocol():
    """Cases of skyrl-gym/tests/test_searchcode.py, plus termination and scoring."""
    import skyrl_b200.gym as gym

    ex = {"reward_spec": {"method": "rule", "ground_truth": "4"}, "max_turns": 3,
          "_transport": lambda url, payload, timeout: {"result": [[{"document": {"contents": "T\nreverse with [::-1]"}, "score": 1.0}]]}}
    env = gym.make("searchcode", env_config=None, extras=ex)
    assert env._parse_action("<tool><search>how to reverse a string in Python</search></tool>")[1:] == (
        "search", ["how to reverse a string in Python"])
    assert env._parse_action("<tool><python>print('hello')</python></tool>")[1:] == ("python", ["print('hello')"])
    env.init([])
    out = env.step("<tool><python>print(1 + 1)</python></tool>")
    assert out["observations"][0]["content"] == "2" and not out["done"] and out["metadata"]["tool_name"] == "python"
    assert out["metadata"]["tools"] == [["search"], ["python"]]
    out = env.step("<tool><python>raise ValueError('fail')</python></tool>")
    assert out["observations"][0]["content"] == ('Error executing Python code: Traceback (most recent call last):\n'
                                                 '  File "<string>", line 1, in <module>\nValueError: fail')
    out = env.step("<solution>#### 4</solution>")
    assert out["done"] and out["reward"] == 1.0
    # calls that cannot be parsed come back as the observation; the last turn ends the episode whatever it says
    env = gym.make("searchcode", env_config=None, extras=dict(ex, max_turns=2))
    out = env.step("no tool here")
    assert out["observations"][0]["content"] == "No <tool>...</tool> block found in action string." and out["metadata"]["tool_name"] is None
    out = env.step("<tool><bash>ls</bash></tool>")
    assert out["done"] and out["reward"] == 0.0
    env = gym.make("searchcode", env_config=None, extras=ex)
    assert "not found in any registered tool group" in env.step("<tool><bash>ls</bash></tool>")["observations"][0]["content"]
    assert "reverse with" in env.step("<tool><search>reverse</search></tool>")["observations"][0]["content"]


def test_lcb_env_golden_cases():
    """Cases of skyrl-gym/tests/test_lcb.py: right program, wrong logic, program that never calls its main()."""
    import json

    import skyrl_b200.gym as gym

    good = ("```python\ndef main():\n    N = int(input())\n    A = list(map(int, input().split()))\n    B = sorted(A, reverse=True)\n"
            "    second = B[1]\n    print(A.index(second) + 1)\n\nif __name__ == \"__main__\":\n    main()\n```")
    wrong = ("```python\ndef main():\n    N = int(input())\n    A = list(map(int, input().split()))\n    print(A.index(max(A)) + 1)\n\n"
             "if __name__ == \"__main__\":\n    main()\n```")
    silent = ("```python\ndef main():\n    A = list(map(int, input().split()))\n    B = sorted(A, reverse=True)\n    second = B[1]\n"
              "    print(A.index(second) + 1)\n\n# forgot to call main()\n```")
    two = json.dumps([{"input": "4\n8 2 5 1\n", "output": "3\n", "testtype": "stdin"},
                      {"input": "3\n3 2 1\n", "output": "2\n", "testtype": "stdin"}])
    one = json.dumps([{"input": "4\n8 2 5 1\n", "output": "3\n", "testtype": "stdin"}])
    for response, tests, expected in ((good, two, 1.0), (wrong, one, 0.0), (silent, one, 0.0)):
        env = gym.make("lcb", env_config=None, extras={"reward_spec": {"method": "rule", "ground_truth": tests}})
        assert env.step(response)["reward"] == expected


def _lm(prompts):
    return [f"response:{p}" for p in prompts]


def test_repl_lm_helpers_batching_errors_and_scaffold():
    """The cases of skyrl-gym/tests/test_rlm.py for the REPL's LM helpers."""
    from skyrl_b200.gym.envs.rlm import PersistentREPL

    bare = PersistentREPL()
    assert not any(k in bare.globals for k in ("llm_query", "llm_query_batched", "rlm_query", "rlm_query_batched"))
    assert "NameError" in bare.execute("r = llm_query('test')").stdout
    repl = PersistentREPL(lm_callback=_lm)
    assert all(k in repl.globals for k in ("llm_query", "llm_query_batched", "rlm_query", "rlm_query_batched"))
    assert "response:hello" in repl.execute("result = llm_query('hello')\nprint(result)").stdout
    lines = repl.execute("results = llm_query_batched(['x', 'y'])\nprint(results[0])\nprint(results[1])").stdout.strip().splitlines()
    assert lines == ["response:x", "response:y"]
    assert "response:fallback prompt" in repl.execute("print(rlm_query('fallback prompt'))").stdout  # no child agent given
    repl.execute("llm_query = lambda p, m=None: 'hijacked'")
    assert repl.globals["llm_query"] == repl._llm_query and "response:a" in repl.execute("print(llm_query('a'))").stdout

    def bad(prompts):
        raise RuntimeError("inference error")

    broken = PersistentREPL(lm_callback=bad)
    assert "Error: LM query failed" in broken.execute("print(llm_query('t'))").stdout
    assert "Error: LM query failed" in broken.execute("print(llm_query_batched(['a', 'b']))").stdout
    child = PersistentREPL(lm_callback=_lm, subcall_fn=lambda p, context=None: f"child_result:{p}")
    assert "child_result:do subtask" in child.execute("print(rlm_query('do subtask'))").stdout
    out = child.execute("rs = rlm_query_batched(['p1', 'p2', 'p3'])\nfor r in rs:\n    print(r)").stdout.strip().splitlines()
    assert out == ["child_result:p1", "child_result:p2", "child_result:p3"]

    def flaky(p, context=None):
        if p == "bad":
            raise RuntimeError("boom")
        return "ok:" + p

    part = PersistentREPL(lm_callback=_lm, subcall_fn=flaky).execute("print(rlm_query_batched(['a', 'bad']))").stdout
    assert "ok:a" in part and "Error: RLM query failed: boom" in part


def test_rlm_env_prompts_hooks_and_metrics():
    import skyrl_b200.gym as gym
    from skyrl_b200.gym.envs.rlm import RLMEnv

    ex = {"reward_spec": {"ground_truth": "Paris"}, "max_turns": 5, "extra_info": {"context_text": "The capital of France is Paris."}}
    q = [{"role": "user", "content": "What is the capital of France?"}]
    msgs, _ = gym.make("rlm", extras=dict(ex)).init(q)
    system = next(m["content"] for m in msgs if m["role"] == "system")
    assert "llm_query" not in system and msgs[-1] == q[0] and "context" in msgs[1]["content"]
    env = gym.make("rlm", extras=dict(ex, lm_callback=_lm, subcall_fn=lambda p, context=None: "child_result:" + p))
    system = next(m["content"] for m in env.init(q)[0] if m["role"] == "system")
    assert all(k in system for k in ("llm_query", "llm_query_batched", "rlm_query", "rlm_query_batched"))
    out = env.step("Let me ask.\n\n```repl\nanswer = llm_query('What is the capital of France?')\nprint(answer)\n```")
    assert "response:What is the capital of France?" in out["observations"][0]["content"] and out["done"] is False
    assert "child_result:solve this subtask" in env.step("```repl\nprint(rlm_query('solve this subtask'))\n```")["observations"][0]["content"]
    out = env.step("```repl\nimport re\nm = re.search(r'is (\\w+)\\.', context)\nans = m.group(1)\n```")
    out = env.step("FINAL_VAR(ans)")
    assert out["done"] and out["reward"] == 1.0
    assert env.get_metrics() == {"turns_used": 4, "final_value_set": True, "final_answer": "Paris", "reward": 1.0, "depth": 0}

    class Counting(RLMEnv):  # a task-specific subclass: own tool, own reward
        def _get_repl_tools(self):
            return {"count_words": lambda: len(str(self._context).split())}

        def _get_reward(self, final_answer):
            return 0.5 if final_answer == "6" else 0.0

    env = Counting(extras=dict(ex))
    assert "`count_words`" in env.init(q)[0][0]["content"]
    env.step("```repl\nn = count_words()\n```")
    assert env.step("FINAL_VAR(n)")["reward"] == 0.5
