"""On-policy regeneration against a fake chat endpoint: fan-out per generation,
boundary masks, tool-call splicing rules, resume keys, error rows."""

import asyncio
import json

import pytest

from speculators_b200.data_generation import regeneration as rg
from speculators_b200.data_generation.configs import DATASET_CONFIGS, DatasetConfig


def _reply(content=None, calls=None, prompt=(1, 2, 3), completion=(7, 8)):
    return {"prompt_token_ids": list(prompt), "usage": {"completion_tokens": len(completion)},
            "choices": [{"message": {"content": content, "tool_calls": calls}, "token_ids": list(completion), "finish_reason": "stop"}]}


def _call(name, cid="c1"):
    return [{"id": cid, "function": {"name": name, "arguments": "{}"}}]


class FakeServer:
    def __init__(self, replies):
        self.replies = list(replies)
        self.payloads = []

    async def __call__(self, payload):
        self.payloads.append(json.loads(json.dumps(payload)))
        r = self.replies.pop(0)
        if isinstance(r, Exception):
            raise r
        return r


def test_row_ingestion():
    row = {"conversations": [{"from": "system", "value": "be brief"}, {"from": "human", "value": "hi"}, {"from": "gpt", "value": "old"},
                             {"from": "tool", "value": '<tool_response>{"name": "get_weather", "content": 3}</tool_response>'},
                             {"from": "human", "value": "bye"}], "tools": '[{"type": "function"}]'}
    turns, results = rg.extract_conversation(row, None)
    assert [t["role"] for t in turns] == ["system", "user", "user"] and results[0][1] == ["get_weather"]
    assert rg.extract_tools(row) == [{"type": "function"}] and rg.extract_tools({"tools": ""}) is None
    with pytest.raises(ValueError):
        rg.extract_tools({"tools": "not a list"})
    assert rg.extract_conversation({"instruction": "do it"}, "instruction") == ([{"role": "user", "content": "do it"}], [])
    assert rg.extract_conversation({"conversations": [{"from": "gpt", "value": "x"}]}, None) == ([], [])
    a, b = rg.primary_identifier({"id": 5, "x": 1}), rg.primary_identifier({"x": 1})
    assert a == "5" and b.startswith("hash_") and b == rg.primary_identifier({"x": 1})
    cfg = DatasetConfig(name="t", hf_path="p", split="s", filter_fn=lambda r: r.get("keep", True), prompt_field="q")
    assert rg.prepare_item({"q": "x", "keep": False}, cfg, 0) is None
    item = rg.prepare_item({"q": "x"}, cfg, 3)
    assert item["idx"] == 3 and item["turns"] == [{"role": "user", "content": "x"}] and item["tools"] is None
    assert "sharegpt4v_coco" not in rg.REGEN_DATASETS and "ultrachat" in rg.REGEN_DATASETS and set(rg.REGEN_DATASETS) < set(DATASET_CONFIGS)
    assert rg.sanitize_filename("org/model name:v1.") == "org_model_name_v1"


def test_tool_call_splice_and_truncation():
    item = {"idx": 0, "primary_id": "conv", "tools": [{"type": "function"}],
            "turns": [{"role": "system", "content": "s"}, {"role": "user", "content": "weather?"}, {"role": "user", "content": "thanks"}],
            "tool_results": [("<tool_response>{\"name\": \"get_weather\"}</tool_response>", ["get_weather"])]}
    server = FakeServer([_reply(None, _call("get_weather"), prompt=(1, 2), completion=(5,)), _reply("sunny", prompt=(1, 2, 5, 6), completion=(9, 9, 9)),
                         _reply("welcome")])
    rows: list = []
    cut = asyncio.run(rg.regenerate_conversation(server, item, model="m", max_tokens=16, sampling_params={"temperature": 0.5, "model": "x"}, samples=rows))
    assert cut is False and [r["id"] for r in rows] == ["conv_gen0", "conv_gen1", "conv_gen2"]
    assert rows[0]["input_ids"] == [1, 2, 5] and rows[0]["loss_mask"] == [0, 0, 1] and rows[0]["metadata"]["is_tool_call"]
    assert rows[1]["loss_mask"] == [0, 0, 0, 0, 1, 1, 1] and all(r["primary_id"] == "conv" for r in rows)
    second = server.payloads[1]
    assert [m["role"] for m in second["messages"]] == ["system", "user", "assistant", "tool"] and second["messages"][3]["tool_call_id"] == "c1"
    assert second["model"] == "m" and second["temperature"] == 0.5 and second["return_token_ids"] is True and second["tool_choice"] == "auto"
    assert [m["role"] for m in server.payloads[2]["messages"]][-2:] == ["assistant", "user"]
    # a call for another tool than the cached result answers cuts the conversation after the call row
    rows = []
    cut = asyncio.run(rg.regenerate_conversation(FakeServer([_reply(None, _call("get_time"))]), item, model="m", max_tokens=8, samples=rows))
    assert cut is True and len(rows) == 1
    # two parallel calls, or no cached result left, do the same
    rows = []
    assert asyncio.run(rg.regenerate_conversation(FakeServer([_reply(None, _call("get_weather") * 2)]), item, model="m", max_tokens=8, samples=rows))
    with pytest.raises(ValueError, match="empty assistant generation"):
        asyncio.run(rg.regenerate_conversation(FakeServer([_reply(None, None)]), item, model="m", max_tokens=8, samples=[]))
    with pytest.raises(ValueError, match="return_token_ids"):
        asyncio.run(rg.regenerate_conversation(FakeServer([_reply("x", prompt=())]), item, model="m", max_tokens=8, samples=[]))


def test_driver_writes_partial_rows_and_resume(tmp_path):
    items = [{"idx": i, "primary_id": f"p{i}", "turns": [{"role": "user", "content": "a"}, {"role": "user", "content": "b"}], "tools": None,
              "tool_results": []} for i in range(3)]
    # conversation 1 fails on its second request
    plan = {"p0": [_reply("x"), _reply("y")], "p1": [_reply("x"), RuntimeError("boom")], "p2": [_reply("x"), _reply("y")]}

    async def post(payload):
        # the first user turn identifies nothing; route by history length and a counter per conversation
        key = post.order[post.n // 2] if post.n % 2 == 0 else post.current
        post.current = key
        post.n += 1
        r = plan[key].pop(0)
        if isinstance(r, Exception):
            raise r
        return r

    post.order, post.n, post.current = ["p0", "p1", "p2"], 0, None
    out = tmp_path / "out.jsonl"
    with out.open("w") as fh:
        stats = asyncio.run(rg.run_regeneration(items, post, lambda row: fh.write(json.dumps(row) + "\n"), model="m", max_tokens=4, concurrency=1))
    assert (stats.ok, stats.errors, stats.requests, stats.completion_tokens) == (2, 1, 5, 10)
    lines = [json.loads(x) for x in out.read_text().splitlines()]
    assert [r["id"] for r in lines] == ["p0_gen0", "p0_gen1", "p1_gen0", "p1_error", "p2_gen0", "p2_gen1"]
    assert "boom" in lines[3]["error"] and "conversations" in stats.summary()
    # resume keys: the conversations' primary ids (the error record falls back to its own id)
    assert rg.load_seen(str(out)) == {"p0", "p1", "p2", "p1_error"}
