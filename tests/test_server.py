"""HTTP layer on the CPU engine: schemas, continuous batching across requests, mode switch."""
import pytest
import torch

from fastcache_b200.serving.server import FastCacheServer, create_app
from helpers import tiny_llama_config


@pytest.fixture(scope="module")
def server():
    s = FastCacheServer(tiny_llama_config(), compression_mode="eager", compression_backend="kvpress",
                        kvpress_method="knorm", compression_factor=2, max_model_len=256, device="cpu",
                        kvcache_block_size=16, num_kvcache_blocks=128, enforce_eager=True)
    yield s
    s.shutdown()


def _ids(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(3, 1000, (n,), generator=g).tolist()


def test_generate_and_status(server):
    from fastapi.testclient import TestClient
    c = TestClient(create_app(server))
    r = c.post("/generate", json={"prompt_token_ids": _ids(40, 1), "max_tokens": 5, "temperature": 0.0})
    assert r.status_code == 200, r.text
    body = r.json()
    assert body["tokens_generated"] == 5 and len(body["token_ids"]) == 5 and body["compression_mode"] == "eager"
    r = c.post("/generate_batch", json={"prompt_token_ids": [_ids(30, 2), _ids(50, 3), _ids(20, 4)],
                                        "max_tokens": 4, "temperature": 0.0})
    assert r.status_code == 200 and r.json()["total_tokens"] == 12
    st = c.get("/status").json()
    assert st["completed_requests"] == 4 and st["total_tokens_generated"] == 17
    assert st["compression_stats"]["compression_count"] >= 3
    assert len(c.get("/metrics", params={"last_n": 2}).json()) == 2
    assert c.post("/generate", json={"prompt": "needs a tokenizer"}).status_code == 400


def test_concurrent_requests_share_decode_batches(server):
    before = server.llm.stats.decode_steps
    futs = [server.submit(_ids(24, 10 + i), 8, 0.0) for i in range(6)]
    res = [f.result(60) for f in futs]
    assert all(r["tokens_generated"] == 8 for r in res)
    # six requests of 8 tokens decoded together need far fewer than 6 * 7 decode steps
    assert server.llm.stats.decode_steps - before < 6 * 7


def test_switch_mode(server):
    from fastapi.testclient import TestClient
    c = TestClient(create_app(server))
    assert c.post("/switch_mode", params={"mode": "bogus"}).status_code == 400
    r = c.post("/switch_mode", params={"mode": "lazy", "method": "streaming_llm"})
    assert r.status_code == 200 and r.json()["mode"] == "lazy"
    out = server.generate(_ids(33, 9), 3, 0.0, timeout=60)
    assert out["compression_mode"] == "lazy" and out["tokens_generated"] == 3
