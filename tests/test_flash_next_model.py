"""The Flash-Next oracle model: chunk invariance, sparse selection, conditional memory."""
import numpy as np
import pytest
import torch

from orinfer_b200.core.host_rows import (ConditionalMemory, HashLayer, Int8RowStore, NgramHasher,
                                         write_int8_table)
from orinfer_b200.models.flash_next import FlashNextConfig, FlashNextOracle, random_weights

TOKENS = [(7 * i * i + 3 * i + 1) % 200 for i in range(26)]


def memory(tmp_path, seed=0, heads=2, dim=4):
    primes = [11, 13, 17, 19, 23, 29]
    rows = sum(primes)
    table = np.random.default_rng(seed).standard_normal((rows, dim)).astype(np.float32)
    path = tmp_path / f"ple{seed}.bin"
    rb = write_int8_table(path, table)
    hasher = NgramHasher(list(range(256)), 0, [255], heads,
                         [HashLayer(0, rows, [3, 5, 7, 9], primes)])
    return ConditionalMemory(hasher, [[Int8RowStore(path, rb, rows)]])


def test_any_chunking_gives_the_same_logits(tmp_path):
    cfg = FlashNextConfig(top_groups=2)                     # 26 tokens = 6 groups: selection is live
    model = FlashNextOracle(cfg, random_weights(cfg, seed=1), memory(tmp_path))
    whole, st = model.forward(TOKENS)
    assert whole.shape == (26, cfg.vocab) and torch.isfinite(whole).all()
    for cuts in ((9, 17), (1, 2, 3, 25), (13,)):
        parts, state, lo = [], None, 0
        for hi in list(cuts) + [len(TOKENS)]:
            lg, state = model.forward(TOKENS[lo:hi], state)
            parts.append(lg)
            lo = hi
        assert torch.allclose(torch.cat(parts), whole, atol=5e-3, rtol=1e-3), cuts
        assert state.tokens == TOKENS
    # decoding continues the same state: teacher-forced single steps equal the prefill rows
    lg, state = model.forward(TOKENS[:20])
    for i in range(20, 26):
        step, state = model.forward([TOKENS[i]], state)
        assert torch.allclose(step[0], whole[i], atol=5e-3, rtol=1e-3)
    out = model.generate(TOKENS[:10], 5, chunk=4)
    assert out == model.generate(TOKENS[:10], 5, chunk=64) and len(out) == 5


def test_sparse_selection_and_memory_matter(tmp_path):
    dense_cfg, sparse_cfg = FlashNextConfig(), FlashNextConfig(top_groups=1)
    w = random_weights(dense_cfg, seed=2)
    mem = memory(tmp_path)
    dense = FlashNextOracle(dense_cfg, w, mem).forward(TOKENS)[0]
    sparse = FlashNextOracle(sparse_cfg, w, mem).forward(TOKENS)[0]
    # up to 7 tokens (one complete group + tail) nothing can be dropped; later rows differ
    assert torch.allclose(dense[:7], sparse[:7], atol=1e-5)
    assert not torch.allclose(dense[12:], sparse[12:], atol=1e-3)
    other = FlashNextOracle(dense_cfg, w, memory(tmp_path, seed=9)).forward(TOKENS)[0]
    none = FlashNextOracle(dense_cfg, w, None).forward(TOKENS)[0]
    assert not torch.allclose(dense, other, atol=1e-3) and not torch.allclose(dense, none, atol=1e-3)
    with pytest.raises(ValueError, match="feature width"):
        FlashNextOracle(dense_cfg, w, memory(tmp_path, seed=3, dim=5)).forward(TOKENS[:3])


def test_layer_recipe():
    cfg = FlashNextConfig(layers=8)
    assert [cfg.is_attention(i) for i in range(8)] == [False, False, False, True] * 2
    w = random_weights(cfg, seed=0)
    assert "index" in w["layers"][3] and "qkvz" in w["layers"][0] and "ple" in w["layers"][0]
    assert "ple" not in w["layers"][1]
