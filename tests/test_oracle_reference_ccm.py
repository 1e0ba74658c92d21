"""The merge compressors against the reference's own module as a CPU oracle.

`utils_ccm/module_ccm_v11.py` of the reference is importable CPU code.  These tests build its
`KVCacheLinearDecoupleCompressor` / `KVCacheHybridCompressor`, move state dicts in both directions with
`strict=True`, and compare forward outputs on image / text splits with remainders, short segments and a
text-only request (utils_ccm/module_ccm_v11.py:666-729, :940-953).  The same weights are then packed and run
through the in-pool path, which is what the engine uses.  Skipped when the reference module cannot be imported
(it needs `transformers`; the import takes some seconds).
"""
import importlib.util
import os
import types

import pytest
import torch

from fastcache_b200.compress import ccm as our
from fastcache_b200.compress.inpool import ccm_compress_in_pool

_CANDIDATES = [
    os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "utils_ccm",
                 "module_ccm_v11.py"),
]
if os.environ.get("FASTCACHE_REFERENCE_DIR"):                # a checkout of the reference elsewhere
    _CANDIDATES.append(os.path.join(os.environ["FASTCACHE_REFERENCE_DIR"], "utils_ccm", "module_ccm_v11.py"))


@pytest.fixture(scope="module")
def ref():
    for path in _CANDIDATES:
        if not os.path.isfile(path):
            continue
        try:
            spec = importlib.util.spec_from_file_location("_reference_module_ccm_v11", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod
        except Exception as exc:                             # pragma: no cover - environment dependent
            reason = f"{type(exc).__name__}: {exc}"
            continue
    pytest.skip("the reference's utils_ccm/module_ccm_v11.py is not importable here"
                + (f" ({reason})" if "reason" in locals() else ""))


L, H, D = 3, 2, 16


def _llava_like_config():
    # the reference derives head_dim as hidden_size // num_key_value_heads (module_ccm_v11.py:611-615)
    text = types.SimpleNamespace(num_hidden_layers=L, num_key_value_heads=H, num_attention_heads=H,
                                 hidden_size=H * D, head_dim=D)
    return types.SimpleNamespace(text_config=text, architectures=["LlavaForConditionalGeneration"])


def _kv(B, S, seed):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B, H, S, D, generator=g), torch.randn(B, H, S, D, generator=g)) for _ in range(L)]


def _randomise(module, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.2)
    return module.eval()


@pytest.mark.parametrize("f", [2, 4, 5])
def test_decouple_compressor_state_dict_and_forward_match_reference(ref, f):
    theirs = _randomise(ref.KVCacheLinearDecoupleCompressor(_llava_like_config(), f, 2), 1)
    mine = our.KVCacheLinearDecoupleCompressor(None, f, 2, n_layer=L, nhead=H, head_dim=D)
    mine.load_state_dict(theirs.state_dict(), strict=True)            # their checkpoint loads here ...
    theirs2 = ref.KVCacheLinearDecoupleCompressor(_llava_like_config(), f, 2).eval()
    theirs2.load_state_dict(mine.state_dict(), strict=True)           # ... and ours loads there
    assert set(mine.state_dict()) == set(theirs.state_dict())
    # (image rows, total rows): remainders on both sides, an image part too short to compress, no image at all
    for img, S in [(f * 3 + 1, f * 7 + 2), (f * 2, f * 2 + 1), (f, 4 * f), (0, 3 * f + 1), (2 * f + 1, 2 * f + 1)]:
        kv = _kv(2, S, S)
        with torch.no_grad():
            want = theirs(kv, it_len=[img, S - img])
            got = mine(kv, it_len=[img, S - img])
            back = theirs2(kv, it_len=[img, S - img])
        for (wk, wv), (gk, gv), (bk, bv) in zip(want, got, back):
            assert wk.shape == gk.shape and wv.shape == gv.shape
            torch.testing.assert_close(gk, wk, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(gv, wv, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(bk, wk, rtol=0, atol=0)


@pytest.mark.parametrize("f", [2, 5])
def test_hybrid_compressor_matches_reference_on_text_only_requests(ref, f):
    cfg = types.SimpleNamespace(architectures=["MiniCPMV"], num_hidden_layers=L, num_key_value_heads=H,
                                num_attention_heads=H, hidden_size=H * D)
    theirs = _randomise(ref.KVCacheHybridCompressor(cfg, f, 2), 2)
    mine = our.KVCacheHybridCompressor(None, f, 2, n_layer=L, nhead=H, head_dim=D)
    mine.load_state_dict(theirs.state_dict(), strict=True)
    assert set(mine.state_dict()) == set(theirs.state_dict())
    for S in (f * 6 + 3, 2 * f, f + 1, 3):
        kv = _kv(1, S, 10 + S)
        with torch.no_grad():
            want = theirs(kv, it_len=[0, S])                          # module_ccm_v11.py:940-953
            got = mine(kv, it_len=[0, S])
        for (wk, wv), (gk, gv) in zip(want, got):
            assert wk.shape == gk.shape
            torch.testing.assert_close(gk, wk, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(gv, wv, rtol=1e-5, atol=1e-5)


def test_in_pool_merge_matches_reference_module(ref):
    """Reference module -> state dict -> this package's packed weights -> compression inside a paged pool."""
    f, bs = 4, 8
    theirs = _randomise(ref.KVCacheLinearDecoupleCompressor(_llava_like_config(), f, 2), 3)
    mine = our.KVCacheLinearDecoupleCompressor(None, f, 2, n_layer=L, nhead=H, head_dim=D)
    mine.load_state_dict(theirs.state_dict(), strict=True)
    packed = mine.pack(torch.float32, torch.device("cpu"))
    lens, imgs = [37, 22, 9], [13, 0, 9]
    nblk = sum(-(-n // bs) for n in lens) + 1
    pool = torch.zeros(L, 2, nblk, H, bs, D)
    g = torch.Generator().manual_seed(4)
    perm = torch.randperm(nblk, generator=g).tolist()
    tables, kvs, k0 = [], [], 0
    for n in lens:
        nb = -(-n // bs)
        tables.append(perm[k0:k0 + nb])
        k0 += nb
        kv = _kv(1, n, 100 + n)
        kvs.append(kv)
        for l, (k, v) in enumerate(kv):
            for r in range(n):
                pool[l, 0, tables[-1][r // bs], :, r % bs] = k[0, :, r]
                pool[l, 1, tables[-1][r // bs], :, r % bs] = v[0, :, r]
    new = ccm_compress_in_pool(pool, tables, lens, imgs, packed)
    for table, n, img, kv, n_new in zip(tables, lens, imgs, kvs, new):
        with torch.no_grad():
            want = theirs(kv, it_len=[img, n - img])
        assert n_new == want[0][0].shape[2]
        for l, (wk, wv) in enumerate(want):
            rows = torch.arange(n_new)
            blocks = torch.tensor(table)[rows // bs]
            gk = pool[l, 0, blocks, :, rows % bs].permute(1, 0, 2)
            gv = pool[l, 1, blocks, :, rows % bs].permute(1, 0, 2)
            torch.testing.assert_close(gk, wk[0], rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(gv, wv[0], rtol=1e-4, atol=1e-5)
