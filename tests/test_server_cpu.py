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
    assert requests.post(server + "/v1/chat/completions", json={"model": "/no/such/model", "messages": []}, headers=H).status_code in (400, 500)
