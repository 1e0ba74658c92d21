"""End-to-end engine on a CUDA device: eager vs CUDA-graph decode, GPU vs CPU oracle."""
import pytest
import torch

from fastcache_b200 import LLM, SamplingParams
from helpers import tiny_qwen3_config

pytestmark = pytest.mark.gpu


def _cfg():
    return tiny_qwen3_config(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                             intermediate_size=1024, vocab_size=2048)


def _prompts(n=5, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, 2048, (int(torch.randint(20, 200, (1,), generator=g)),), generator=g).tolist()
            for _ in range(n)]


def _run(device, eager, dtype="auto"):
    llm = LLM(_cfg(), device=device, dtype=dtype, kvcache_block_size=32, num_kvcache_blocks=128,
              max_model_len=512, max_num_seqs=8, enforce_eager=eager, init_device="cpu")
    out = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    llm.exit()
    return [o["token_ids"] for o in out]


def test_graph_decode_matches_eager():
    assert _run("cuda", True) == _run("cuda", False)


def test_gpu_first_tokens_match_cpu_oracle():
    """bf16 kernels vs the fp32 CPU path of the same seeded model: the first sampled token
    (a pure prefill result) agrees for most prompts; later tokens may drift in bf16."""
    gpu = _run("cuda", True)
    cpu = _run("cpu", True, "fp32")
    agree = sum(g[0] == c[0] for g, c in zip(gpu, cpu))
    assert agree >= len(gpu) - 1, (gpu, cpu)


def _llava_cfg():
    from fastcache_b200 import ModelConfig
    text = dict(model_type="llama", hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=4, intermediate_size=512, vocab_size=600, rms_norm_eps=1e-5,
                max_position_embeddings=1024, rope_theta=10000.0)
    vis = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
               image_size=56, patch_size=14)
    return ModelConfig(model_type="llava", architectures=["LlavaForConditionalGeneration"], text_config=text,
                       vision_config=vis, image_token_index=500)


def _minicpm_cfg():
    from fastcache_b200 import ModelConfig
    return ModelConfig(model_type="minicpmv", architectures=["MiniCPMV"], hidden_size=256, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, intermediate_size=512, vocab_size=600,
                       rms_norm_eps=1e-6, max_position_embeddings=2048, rope_theta=1e6, query_num=4,
                       max_slice_nums=9, scale_resolution=56, image_token_id=501,
                       vision_config=dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                          num_attention_heads=4, image_size=140, patch_size=14))


@pytest.mark.parametrize("make_cfg,img_tok", [(_llava_cfg, 500), (_minicpm_cfg, 501)])
def test_multimodal_request_on_gpu_matches_cpu_first_token(make_cfg, img_tok):
    """Vision tower (dense attention kernel, GEMMs), projector / resampler and the language model on
    the GPU against the fp32 CPU path of the same seeded model: same image rows, same first token."""
    g = torch.Generator().manual_seed(5)
    img = torch.rand(3, 90, 70, generator=g)
    prompt = [5, 6, img_tok, 7, 8, 9, 10]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs, rows = {}, {}
    for dev, dtype in (("cuda", "auto"), ("cpu", "fp32")):
        llm = LLM(make_cfg(), device=dev, dtype=dtype, kvcache_block_size=16, num_kvcache_blocks=128,
                  max_model_len=512, enforce_eager=True, init_device="cpu")
        seq = llm.add_request(prompt, sp, image=img)
        rows[dev] = seq.prompt_rows
        while not llm.is_finished():
            llm.step()
        outs[dev] = list(seq.completion_token_ids)
        llm.exit()
    assert rows["cuda"] == rows["cpu"] and len(outs["cuda"]) == 6
    assert outs["cuda"][0] == outs["cpu"][0], (outs["cuda"], outs["cpu"])


def test_multi_step_decode_matches_single_steps_on_gpu():
    """Several graph replays per engine step with the sampled tokens fed back on the device: same tokens as one
    step at a time, greedy and sampled (the sampler's step counter advances once per decode step either way)."""
    for temperature in (0.0, 0.7):
        outs = []
        for k in (1, 4):
            llm = LLM(_cfg(), device="cuda", kvcache_block_size=32, num_kvcache_blocks=128, max_model_len=512,
                      max_num_seqs=8, enforce_eager=False, init_device="cpu", prefix_caching=False, seed=5,
                      decode_steps_per_call=k)
            sps = [SamplingParams(temperature=temperature, max_tokens=m, ignore_eos=True) for m in (17, 3, 12, 9, 20)]
            out = llm.generate(_prompts(), sps)
            outs.append([o["token_ids"] for o in out])
            assert llm.model_runner.read_device_status() == 0
            llm.exit()
        assert outs[0] == outs[1]


def test_chunked_prefill_on_gpu_matches_unsplit_prefill():
    """A prompt prefetched in pieces (the prefill kernels' cached-prefix path, queries shorter than the keys) against
    the same prompt in one piece on the GPU and against the fp32 CPU engine: the first sampled token is a pure
    prefill result and agrees for all prompts but at most one (bf16 near-ties)."""
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, 2048, (n,), generator=g).tolist() for n in (300, 40, 150, 90, 260)]
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)

    def run(device, budget, chunk, dtype="auto"):
        llm = LLM(_cfg(), device=device, dtype=dtype, kvcache_block_size=32, num_kvcache_blocks=128,
                  max_model_len=512, max_num_seqs=8, enforce_eager=True, init_device="cpu", prefix_caching=False,
                  max_num_batched_tokens=budget, chunked_prefill_tokens=chunk)
        out = [o["token_ids"] for o in llm.generate(prompts, sp)]
        steps = llm.stats.prefill_steps
        bm = llm.scheduler.block_manager
        assert bm.num_free_blocks == bm.num_blocks
        if device == "cuda":
            assert llm.model_runner.read_device_status() == 0
        llm.exit()
        return out, steps

    pieces, n_pieces = run("cuda", 128, 32)
    whole, n_whole = run("cuda", 4096, 0)
    oracle, _ = run("cpu", 4096, 0, "fp32")
    assert n_whole == 1 and n_pieces > 5
    assert sum(a[0] == b[0] for a, b in zip(pieces, whole)) >= len(prompts) - 1, (pieces, whole)
    assert sum(a[0] == b[0] for a, b in zip(pieces, oracle)) >= len(prompts) - 1, (pieces, oracle)


@pytest.mark.parametrize("mode", ["compressed", "original"])
def test_position_mode_with_graph_decode_on_gpu(mode):
    """Tokens decoded after an eviction take their rotary position from the KV length or from the true index; the
    CUDA-graph decode path feeds the same positions as the eager one and samples the same tokens."""
    outs, fed = [], []
    for eager in (True, False):
        llm = LLM(_cfg(), device="cuda", kvcache_block_size=32, num_kvcache_blocks=128, max_model_len=512,
                  max_num_seqs=8, enforce_eager=eager, init_device="cpu", prefix_caching=False,
                  enable_compression=True, compression_backend="kvpress", kvpress_method="knorm",
                  compression_factor=2, compression_pipeline="prefill", position_mode=mode)
        inner, seen = llm.model_runner.prepare_decode, []

        def spy(seqs, inner=inner, seen=seen):
            out = inner(seqs)
            seen.append([(len(s.prompt_token_ids), int(p), int(n)) for s, p, n in zip(seqs, out[1], out[3])])
            return out

        llm.model_runner.prepare_decode = spy
        out = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
        assert llm.model_runner.read_device_status() == 0 and llm.stats.compressions == len(out)
        outs.append([o["token_ids"] for o in out])
        fed.append(seen)
        llm.exit()
    assert outs[0] == outs[1] and fed[0] == fed[1]
    for step in fed[0]:
        for prompt_len, pos, kv in step:
            if mode == "compressed":
                assert pos == kv - 1
            else:
                assert pos >= prompt_len and pos > kv - 1
