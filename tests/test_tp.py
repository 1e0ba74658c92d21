"""Tensor parallelism: TP ranks must reproduce the single-rank model.

CPU tier: gloo ranks in fp32 (exact up to summation order, so tokens must match).
GPU tier: NCCL ranks with the fused communication kernels (run when >= 2 GPUs are visible)."""
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, device, out, port, extra=()):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_worker.py"),
           "--device", device, "--out", out, *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.load(open(out))


@pytest.mark.parametrize("world,kv_heads", [(2, 2), (4, 2)])
def test_tp_cpu_gloo_matches_single_rank(tmp_path, world, kv_heads):
    one = _run(1, "cpu", str(tmp_path / "a.json"), 29611, ["--kv-heads", str(kv_heads)])
    many = _run(world, "cpu", str(tmp_path / "b.json"), 29612 + world, ["--kv-heads", str(kv_heads)])
    assert one["tokens"] == many["tokens"]


def test_tp_cpu_gloo_split_prompts_match_unsplit(tmp_path):
    """Two gloo ranks with chunked prefill (replicated schedulers must cut the same pieces) against one rank
    without it."""
    one = _run(1, "cpu", str(tmp_path / "a.json"), 29641, ["--kv-heads", "2"])
    two = _run(2, "cpu", str(tmp_path / "b.json"), 29642, ["--kv-heads", "2", "--chunk", "16"])
    assert one["tokens"] == two["tokens"]


def test_tp_cpu_gloo_several_decode_steps_per_call(tmp_path):
    """Two gloo ranks that run three decode steps per engine step (replicated engines must take the same
    decisions about when they may) against one rank stepping one at a time, greedy and sampled."""
    one = _run(1, "cpu", str(tmp_path / "a.json"), 29661, ["--kv-heads", "2"])
    two = _run(2, "cpu", str(tmp_path / "b.json"), 29662, ["--kv-heads", "2", "--decode-steps", "3"])
    assert one["tokens"] == two["tokens"] and one["sampled"] == two["sampled"] and two["ranks_agree"]
    assert one["decode_steps"] + one["prefill_steps"] == one["engine_steps"]
    assert two["decode_steps"] + two["prefill_steps"] > two["engine_steps"]       # some steps made several


def test_tp_cpu_gloo_sharded_embedding_matches_single_rank(tmp_path):
    """The vocabulary-parallel table (masked lookup + all-reduce), which large vocabularies fall back to."""
    one = _run(1, "cpu", str(tmp_path / "a.json"), 29651, ["--kv-heads", "2"])
    two = _run(2, "cpu", str(tmp_path / "b.json"), 29652, ["--kv-heads", "2", "--shard-embedding"])
    assert one["tokens"] == two["tokens"] and two["ranks_agree"]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_gpu_fused_comm(tmp_path, world):
    """NCCL ranks with the fused communication kernels at 2, 4 and 8 GPUs (as many as are visible): the fused
    decode and prefill paths against a library all-reduce, token agreement with one GPU, and the same tokens on
    every rank, greedy and sampled."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29630 + 10 * world
    one = _run(1, "cuda", str(tmp_path / "a.json"), port)
    many = _run(world, "cuda", str(tmp_path / "b.json"), port + 1)
    assert many["status"] == 0 and many["engine_status"] == 0
    # absolute errors of bf16 results: sums over 8 ranks reach magnitudes where one bf16 step is 0.0625
    step = max(1, world // 4)
    assert many["allreduce_max_err"] < 6e-2 * step
    assert many["fused_prefill_max_err"] < 8e-2 * step
    assert many["ranks_agree"] and many["local_logits"] and many["embedding_replicated"]
    # several decode steps per launch (sampled tokens fed back on the device, one candidate exchange per step)
    multi = _run(world, "cuda", str(tmp_path / "d.json"), port + 3, ["--decode-steps", "3"])
    assert multi["status"] == 0 and multi["engine_status"] == 0 and multi["ranks_agree"]
    assert multi["tokens"] == many["tokens"] and multi["sampled"] == many["sampled"]
    assert multi["decode_steps"] + multi["prefill_steps"] > multi["engine_steps"]
    # same engine with the one-shot limit lowered so that prefill takes the GEMM + reduce-scatter path
    big = _run(world, "cuda", str(tmp_path / "c.json"), port + 2, ["--one-shot-tokens", "64"])
    assert big["status"] == 0 and big["engine_status"] == 0 and big["ranks_agree"]
    assert sum(a[0] == b[0] for a, b in zip(one["tokens"], big["tokens"])) >= len(one["tokens"]) - 1, (one, big)
    # bf16 summation order differs between 1 and N ranks: the first tokens (pure prefill) agree
    same = sum(a[0] == b[0] for a, b in zip(one["tokens"], many["tokens"]))
    assert same >= len(one["tokens"]) - 1, (one, many)


def _tp_inference(world, cfg_path, port, extra=()):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=os.path.dirname(HERE))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "fastcache_b200.serving.tp_inference",
           "--model", cfg_path, "--tp-size", str(world), "--backend", "gloo", "--num-prompts", "3",
           "--prompt-len", "40", "--max-tokens", "5", *extra]
    r = subprocess.run(cmd, env=dict(env, CUDA_VISIBLE_DEVICES=""), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout          # rank 0 alone prints the result
    return json.loads(lines[0])


def test_tp_inference_command_line_two_gloo_ranks(tmp_path):
    """`python -m fastcache_b200.serving.tp_inference` (the reference's tp_inference.py:34-123) on a random-init
    model given as an HF config file: two ranks print one result with the tokens of one rank, with and without
    key-norm eviction."""
    cfg = dict(model_type="llama", architectures=["LlamaForCausalLM"], hidden_size=128, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=512,
               rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=512, tie_word_embeddings=False,
               eos_token_id=2, torch_dtype="float32")
    path = str(tmp_path / "config.json")
    json.dump(cfg, open(path, "w"))
    one = _tp_inference(1, path, 29671)
    two = _tp_inference(2, path, 29672)
    assert one["tp"] == 1 and two["tp"] == 2 and one["output_tokens"] == two["output_tokens"] == 15
    assert one["first"] == two["first"]
    pressed = _tp_inference(2, path, 29673, ["--enable-compression", "--kvpress-method", "knorm",
                                             "--compression-factor", "2"])
    assert pressed["output_tokens"] == 15
