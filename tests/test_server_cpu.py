"""HTTP server against a toy checkpoint on CPU: routes, SSE framing, auth, 429, metrics."""
import json
import socket
import threading
import time

import pytest
import requests
import uvicorn

from hartsyinference_b200.engine.requests import EngineOptions
from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
from hartsyinference_b200.server import ServerOptions, create_app
from tests.test_llm_loader_cpu import _synthetic


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("srv")
    cfg, t = _synthetic(seed=8)
    save_hf_checkpoint(cfg, t, d / "toy")
    opts = ServerOptions(backend="cpu", models={"toy": str(d / "toy"), "flux-tiny": "synthetic:flux-tiny"},
                         default_text_model="toy", default_image_model="flux-tiny", api_keys=["k1"])
    app = create_app(opts, engine_options=EngineOptions(max_batch=8, max_model_len=256, kv_pool_bytes_budget=8 << 20))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    for _ in range(100):
        try:
            requests.get(f"http://127.0.0.1:{port}/health", timeout=0.5)
            break
        except Exception:
            time.sleep(0.1)
    yield f"http://127.0.0.1:{port}"
    srv.should_exit = True
    th.join(timeout=5)


H = {"x-api-key": "k1"}


def test_health_ready_version_metrics_auth(server):
    assert requests.get(server + "/health").json() == {"status": "ok"}
    assert requests.get(server + "/ready").json()["status"] == "ready"
    assert "version" in requests.get(server + "/version").json()
    assert requests.get(server + "/v1/models").status_code == 401
    assert requests.get(server + "/v1/models", headers={"Authorization": "Bearer k1"}).json()["data"][0]["id"] == "toy"
    m = requests.get(server + "/metrics").text
    assert "hartsyinference_requests_total" in m and "hartsyinference_queue_pending" in m


def test_chat_completion_and_sse_stream(server):
    body = {"model": "toy", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0}
    r = requests.post(server + "/v1/chat/completions", json=body, headers=H).json()
    assert r["object"] == "chat.completion" and r["usage"]["completion_tokens"] >= 1
    assert r["choices"][0]["finish_reason"] in ("stop", "length")
    with requests.post(server + "/v1/chat/completions", json=dict(body, stream=True), headers=H, stream=True) as resp:
        raw = resp.content.decode()
    frames = [f for f in raw.split("\n\n") if f]
    assert all(f.startswith("data: ") for f in frames) and frames[-1] == "data: [DONE]"
    first = json.loads(frames[0][6:])
    assert first["choices"][0]["delta"] == {"role": "assistant"}
    last = json.loads(frames[-2][6:])
    assert last["choices"][0]["finish_reason"] in ("stop", "length") and "usage" in last
    n = requests.post(server + "/v1/native/text/count-tokens", json=body, headers=H).json()["tokens"]
    assert n > 0
    nat = requests.post(server + "/v1/native/text", json={"prompt": "abc", "max_tokens": 4, "greedy": True}, headers=H).json()
    assert nat["completion_tokens"] >= 1 and nat["stop_reason"] in ("stop", "length")
    emb = requests.post(server + "/v1/embeddings", json={"model": "toy", "input": ["a", "b"]}, headers=H).json()
    assert len(emb["data"]) == 2 and len(emb["data"][0]["embedding"]) == 128


def test_image_generation_and_unsupported_routes(server):
    r = requests.post(server + "/v1/images/generations", json={"model": "flux-tiny", "prompt": "x", "size": "64x64", "steps": 2, "seed": 3},
                      headers=H, timeout=120).json()
    import base64
    png = base64.b64decode(r["data"][0]["b64_json"])
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and r["data"][0]["seed"] == 3
    assert requests.post(server + "/v1/audio/speech", json={}, headers=H).status_code == 400
    assert requests.post(server + "/v1/native/music", json={}, headers=H).status_code == 400
    assert requests.post(server + "/v1/chat/completions", json={"model": "/no/such/model", "messages": []}, headers=H).status_code in (400, 500)


def test_tool_call_parsing_and_openai_shape():
    from hartsyinference_b200.assets.tool_calls import ToolCall, forced_prefix, parse_tool_calls, tool_names
    from hartsyinference_b200.engine.requests import StopReason, TextResult
    from hartsyinference_b200.server.app import _finish, _forced_tool, _message
    import json
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {}}}, {"name": "lookup"}]
    known = tool_names(tools)
    assert known == {"get_weather", "lookup"}
    txt = 'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>'
    rest, calls = parse_tool_calls(txt, known)
    assert rest == "Let me check." and len(calls) == 1 and calls[0].name == "get_weather" and json.loads(calls[0].arguments) == {"city": "Oslo"}
    two = '<tool_call>{"name": "lookup", "arguments": {"q": 1}}</tool_call><tool_call>{"name": "lookup", "arguments": {"q": 2}}</tool_call>'
    assert [json.loads(c.arguments)["q"] for c in parse_tool_calls(two, known)[1]] == [1, 2]
    rest, calls = parse_tool_calls('[TOOL_CALLS] [{"name": "lookup", "arguments": {"q": "x"}}]', known)
    assert rest == "" and calls[0].name == "lookup"
    rest, calls = parse_tool_calls('<|python_tag|>{"name": "get_weather", "parameters": {"city": "Rome"}}', known)
    assert rest == "" and json.loads(calls[0].arguments) == {"city": "Rome"}
    # not calls: unknown tool, ordinary JSON, broken JSON, unterminated tag with valid JSON is still a call
    assert parse_tool_calls('<tool_call>{"name": "rm_rf", "arguments": {}}</tool_call>', known)[1] == []
    assert parse_tool_calls('{"name": "Bob", "age": 3}', None)[1] == []
    assert parse_tool_calls('<tool_call>{"name": </tool_call>', known) == ('<tool_call>{"name": </tool_call>', [])
    assert len(parse_tool_calls(forced_prefix("lookup") + '{"q": 5}}', known)[1]) == 1
    r = TextResult(text="", stop_reason=StopReason.TOOL_CALL, tool_calls=[ToolCall("call_1", "lookup", '{"q": 5}')])
    m = _message(r)
    assert _finish(r) == "tool_calls" and m["content"] is None and m["tool_calls"][0]["function"] == {"name": "lookup", "arguments": '{"q": 5}'}
    assert _forced_tool({"type": "function", "function": {"name": "lookup"}}) == "lookup" and _forced_tool("auto") is None
