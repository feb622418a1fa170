"""ReAct agent runner against a scripted inference client."""
import asyncio

from skyrl_b200.agent import AsyncDispatcher, ReActAgent, Tool
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


class _ScriptedClient:
    def __init__(self, tok, scripts):
        self.tok, self.scripts, self.calls = tok, scripts, {}

    async def generate(self, inp):
        sid = inp["session_ids"][0]
        k = self.calls.get(sid, 0)
        self.calls[sid] = k + 1
        text = self.scripts[min(k, len(self.scripts) - 1)]
        ids = self.tok.encode(text)
        return {"response_ids": [ids], "responses": [text], "response_logprobs": [[-0.1] * len(ids)], "stop_reasons": ["stop"]}


def test_react_loop_masks_observations_and_stops_on_answer():
    tok = SyntheticTokenizer(2048)
    scripts = ['I need to add <tool>{"name": "add", "arguments": {"a": 2, "b": 40}}</tool>', "so <answer>42</answer>"]
    agent = ReActAgent(_ScriptedClient(tok, scripts), tok, [Tool("add", lambda a, b: str(a + b), "adds")], max_turns=4)
    r = asyncio.run(agent.run("what is 2+40?", session_id="s"))
    assert r.answer == "42" and r.stop_reason == "answer" and r.turns == 2
    assert len(r.response_ids) == len(r.loss_mask) == len(r.logprobs)
    assert 0 in r.loss_mask and r.loss_mask[0] == 1 and r.loss_mask[-1] == 1
    assert any(m["role"] == "user" and m["content"] == "42" for m in r.messages)
    bad = ReActAgent(_ScriptedClient(tok, ['<tool>{"name": "nope"}</tool>', "<answer>x</answer>"]), tok, [], max_turns=3)
    r2 = asyncio.run(bad.run("t", session_id="s"))
    assert "Unknown tool" in r2.messages[3]["content"] and r2.answer == "x"
    out = asyncio.run(AsyncDispatcher(agent, 2).run(["a", "b", "c"]))
    assert [o.answer for o in out] == ["42"] * 3
