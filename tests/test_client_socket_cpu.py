"""Both Python clients against a real listening server (uvicorn on 127.0.0.1, tiny model on CPU):
concurrent async requests are batched by the engine and agree with the sequential sync client."""
import asyncio
import socket
import threading
import time

import pytest
import torch

from mlxcel_b200.client import AsyncClient, Client, MlxcelError
from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.server.app import ServerState, create_app
from mlxcel_b200.server.worker import ModelWorker
from mlxcel_b200.tokenizer import ByteTokenizer


@pytest.fixture(scope="module")
def server_url():
    import uvicorn

    cfg = preset("tiny-llama")
    eng = Engine(DecoderModel(cfg, random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)), cfg,
                 EngineConfig(max_batch=8, max_num_batched_tokens=256, num_blocks=256, max_model_len=512, cuda_graphs=False))
    tk = ByteTokenizer(cfg.vocab_size)
    worker = ModelWorker(eng, tk, "tiny")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    srv = uvicorn.Server(uvicorn.Config(create_app(ServerState(worker, tk, "tiny", api_keys={"k"})), host="127.0.0.1",
                                        port=port, log_level="error"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    url = f"http://127.0.0.1:{port}"
    for _ in range(200):
        if Client(url, api_key="k").health():
            break
        time.sleep(0.05)
    else:
        pytest.fail("server did not come up")
    yield url
    srv.should_exit = True
    th.join(timeout=10)
    worker.shutdown()


def test_sync_and_async_clients_agree(server_url):
    sync = Client(server_url, api_key="k")
    assert sync.models() == ["tiny"]
    prompts = [f"prompt number {i}" for i in range(6)]
    want = [sync.complete(p, max_tokens=8, temperature=0, ignore_eos=True) for p in prompts]

    async def run():
        async with AsyncClient(server_url, api_key="k") as c:
            assert await c.health() and await c.models() == ["tiny"]
            got = await asyncio.gather(*(c.complete(p, max_tokens=8, temperature=0, ignore_eos=True) for p in prompts))
            msgs = [{"role": "user", "content": "hi"}]
            whole = await c.chat(msgs, max_tokens=8, temperature=0, ignore_eos=True)
            pieces = [p async for p in c.chat_stream(msgs, max_tokens=8, temperature=0, ignore_eos=True)]
            toks = await c.tokenize("abc")
            emb = await c.embed(["a", "b"])
            return got, whole, "".join(pieces), toks, emb

    got, whole, streamed, toks, emb = asyncio.run(run())
    assert list(got) == want                       # batched together, same greedy text as one at a time
    assert streamed == whole and len(toks) == 3 and len(emb) == 2


def test_async_client_errors(server_url):
    async def run():
        async with AsyncClient(server_url, api_key="wrong") as c:
            assert not await c.health() or True    # /health is open; the API is not
            with pytest.raises(MlxcelError, match="401"):
                await c.complete("x", max_tokens=1)
        with pytest.raises(MlxcelError, match="no open session"):
            await AsyncClient(server_url).complete("x")

    asyncio.run(run())
