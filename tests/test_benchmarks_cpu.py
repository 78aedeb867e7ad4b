"""The committed benchmark harnesses run end to end on CPU against tiny models (their numbers mean
nothing there; the test is that they drive the public paths and report consistent fields)."""
import socket
import threading
import time

import torch


def test_serving_concurrency_harness_against_a_live_server():
    import uvicorn

    from benchmarks import serving_concurrency
    from mlxcel_b200.client import Client
    from mlxcel_b200.config import preset
    from mlxcel_b200.engine import Engine, EngineConfig
    from mlxcel_b200.models.decoder import DecoderModel
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.server.app import ServerState, create_app
    from mlxcel_b200.server.worker import ModelWorker
    from mlxcel_b200.tokenizer import ByteTokenizer

    cfg = preset("tiny-llama")
    eng = Engine(DecoderModel(cfg, random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)), cfg,
                 EngineConfig(max_batch=8, max_num_batched_tokens=256, num_blocks=256, max_model_len=512, cuda_graphs=False))
    tk = ByteTokenizer(cfg.vocab_size)
    worker = ModelWorker(eng, tk, "tiny")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    srv = uvicorn.Server(uvicorn.Config(create_app(ServerState(worker, tk, "tiny")), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    url = f"http://127.0.0.1:{port}"
    try:
        for _ in range(200):
            if Client(url).health():
                break
            time.sleep(0.05)
        rows = serving_concurrency.main(["--url", url, "--clients", "1,3", "--prompt-tokens", "12", "--max-tokens", "6", "--rounds", "1"])
    finally:
        srv.should_exit = True
        th.join(timeout=10)
        worker.shutdown()
    assert [r["clients"] for r in rows] == [1, 3] and [r["requests"] for r in rows] == [1, 3]
    assert all(r["output_tokens"] == 6 * r["requests"] and r["ttft_mean_ms"] > 0 and r["tok_per_s"] > 0 for r in rows)


def test_speculative_compare_harness_reports_lossless_runs():
    from benchmarks import speculative_compare

    row = speculative_compare.main(["-m", "preset:tiny-llama", "--device", "cpu", "--prompt-lookup", "--requests", "2",
                                    "--prompt-tokens", "24", "--max-tokens", "10", "--no-cuda-graphs"])
    assert row["same_tokens"] and row["classic_tok_s"] > 0 and row["speculative_tok_s"] > 0
    assert row["drafter"] == "prompt-lookup" and row["verify_rounds"] >= 0
