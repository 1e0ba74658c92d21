"""Multimodal models on the CPU path: image rows replace the placeholder, KV accounting, slicing."""
import torch

from fastcache_b200 import LLM, ModelConfig, SamplingParams
from fastcache_b200.models.minicpm import best_grid, slice_image
from fastcache_b200.models.vision import CLIPVisionTower, sincos_2d


def _llava_cfg():
    text = dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=4, intermediate_size=256, vocab_size=600, rms_norm_eps=1e-5,
                max_position_embeddings=1024, rope_theta=10000.0)
    vis = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
               image_size=56, patch_size=14)
    return ModelConfig(model_type="llava", architectures=["LlavaForConditionalGeneration"], text_config=text,
                       vision_config=vis, image_token_index=500)


def _minicpm_cfg():
    return ModelConfig(model_type="minicpmv", architectures=["MiniCPMV"], hidden_size=128, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, intermediate_size=256, vocab_size=600,
                       rms_norm_eps=1e-6, max_position_embeddings=2048, rope_theta=1e6, query_num=4,
                       max_slice_nums=9, scale_resolution=56, image_token_id=501,
                       vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                          num_attention_heads=4, image_size=140, patch_size=14))


def test_llava_image_rows_and_generation():
    llm = LLM(_llava_cfg(), device="cpu", kvcache_block_size=16, num_kvcache_blocks=64, max_model_len=256,
              enforce_eager=True)
    assert llm.model_runner.is_multimodal and llm.image_token_len == 16
    img = torch.rand(3, 80, 60)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    prompt = [5, 6, 500, 7, 8, 9]
    seq = llm.add_request(prompt, sp, image=img)
    assert seq.num_image_tokens == 16 and seq.image_token_pos == 2 and seq.prompt_rows == 6 + 15
    llm.add_request([11, 12, 13], sp)                        # a text request in the same prefill batch
    llm.step()
    assert seq.kv_cache_len == 21 + 1 and len(seq.block_table) == 2
    llm.scheduler.block_manager.check_invariants(list(llm.scheduler.running))
    while not llm.is_finished():
        llm.step()
    # a different image must change the continuation; the same image must not
    out_a = llm.generate([prompt], sp, images=[img])[0]["token_ids"]
    out_b = llm.generate([prompt], sp, images=[img])[0]["token_ids"]
    out_c = llm.generate([prompt], sp, images=[torch.rand(3, 80, 60)])[0]["token_ids"]
    assert out_a == out_b and len(out_c) == 4


def test_clip_tower_feature_layer_selection():
    from fastcache_b200.models.llava import _vision_cfg
    cfg = _vision_cfg(_llava_cfg())
    torch.manual_seed(0)
    t2 = CLIPVisionTower(cfg, feature_layer=-2)
    for p in t2.parameters():
        torch.nn.init.normal_(p, std=0.05)
    assert t2.num_layers_run == 2
    x = torch.rand(2, 3, 56, 56)
    f = t2(x)
    assert f.shape == (2, 16, 64)


def test_minicpm_slicing_and_rows():
    assert best_grid(1344, 896, 9, 448) == (3, 2)
    assert best_grid(400, 400, 9, 448) is None
    slices = slice_image(torch.rand(3, 896, 1344), 9, 448, 14)
    assert len(slices) == 7 and all(s.shape[1] % 14 == 0 and s.shape[2] % 14 == 0 for s in slices)
    llm = LLM(_minicpm_cfg(), device="cpu", kvcache_block_size=16, num_kvcache_blocks=64, max_model_len=512,
              enforce_eager=True)
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    seq = llm.add_request([4, 501, 5, 6], sp, image=torch.rand(3, 112, 168))      # 3 x 2 grid + thumbnail
    assert seq.num_image_tokens == 7 * 4
    out = []
    while not llm.is_finished():
        o, _ = llm.step()
        out += o
    assert len(out[0][1]) == 3
    assert sincos_2d(32, 3, 5).shape == (3, 5, 32)
