"""Router mode: two tiny checkpoints behind one front, one resident at a time."""
import argparse

from fastapi.testclient import TestClient

from mlxcel_b200 import cli
from mlxcel_b200.server.router import create_router_app, discover_models


def _models(tmp_path):
    for name, seed in (("alpha", 1), ("beta", 2)):
        cli.cmd_random_init(argparse.Namespace(preset="tiny-llama", out=str(tmp_path / name), seed=seed, quantize=None,
                                               bits=4, group_size=64))
    (tmp_path / "not-a-model").mkdir()
    return tmp_path


def test_router_loads_on_demand_and_evicts_lru(tmp_path):
    d = _models(tmp_path)
    ini = tmp_path / "presets.ini"
    ini.write_text(f"[gamma]\nmodel = {d / 'alpha'}\nctx_size = 256\nparallel = 2\n")
    assert sorted(discover_models(str(d), str(ini))) == ["alpha", "beta", "gamma"]
    app = create_router_app(str(d), str(ini), max_loaded=1, device="cpu",
                            engine_defaults=dict(ctx_size=256, parallel=2, num_blocks=64))
    with TestClient(app) as c:
        status = {m["id"]: m["status"] for m in c.get("/v1/models").json()["data"]}
        assert status == {"alpha": "unloaded", "beta": "unloaded", "gamma": "unloaded"}
        body = dict(prompt=[1, 2, 3, 4], max_tokens=4, temperature=0)
        ra = c.post("/v1/completions", json=dict(model="alpha", **body))
        assert ra.status_code == 200 and ra.json()["model"] == "alpha"
        status = {m["id"]: m["status"] for m in c.get("/models").json()["data"]}
        assert status["alpha"] == "loaded" and status["beta"] == "unloaded"
        rb = c.post("/v1/completions", json=dict(model="beta", **body))          # evicts alpha
        assert rb.status_code == 200 and rb.json()["model"] == "beta"
        status = {m["id"]: m["status"] for m in c.get("/models").json()["data"]}
        assert status["alpha"] == "unloaded" and status["beta"] == "loaded"
        rg = c.post("/v1/completions", json=dict(model="gamma", **body))         # same weights as alpha
        assert rg.json()["choices"][0]["text"] == ra.json()["choices"][0]["text"]
        assert c.post("/v1/completions", json=dict(model="nope", **body)).status_code == 404
        assert c.post("/models/unload", json=dict(model="gamma")).json()["changed"] is True
        assert c.post("/models/load", json=dict(model="beta")).json()["status"] == "loaded"
        # streaming passes through the front untouched
        with c.stream("POST", "/v1/chat/completions",
                      json=dict(model="beta", messages=[dict(role="user", content="hi")], max_tokens=3, stream=True)) as r:
            text = "".join(r.iter_text())
        assert "data: [DONE]" in text
        ev = [e["event"] for e in c.get("/models/events").json()["events"]]
        assert ev.count("loaded") >= 4 and "unloaded" in ev
        # a request without a model goes to the default (first) one
        assert c.post("/tokenize", json=dict(content="abc")).status_code == 200
