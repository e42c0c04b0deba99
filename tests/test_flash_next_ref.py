"""Properties of the Flash-Next block oracles (hyper-connections, PLE, QSA)."""
import math

import pytest
import torch

from orinfer_b200.ref import flash_next_ref as FN


def g(seed=0):
    return torch.Generator().manual_seed(seed)


def test_hc_read_write_limits():
    t, s, h, r = 5, 4, 16, 8
    x = torch.randn(t, s, h, generator=g())
    w = {"norm": torch.zeros(s * h), "down": torch.randn(r, s * h, generator=g(1)) * 0.1,
         "up": torch.zeros(s * h, r), "inject": torch.zeros(s, s * h)}
    mixed, gate = FN.hc_read(x, w)
    n = FN.rms(x, torch.zeros(s, h))
    assert torch.allclose(mixed, n.mean(1) * 0.5, atol=1e-6)        # sigmoid(0) gates
    assert torch.equal(gate, torch.ones(t, s))                      # 2 * sigmoid(0)
    block = torch.randn(t, h, generator=g(2))
    y = FN.hc_write(x, block, gate)
    assert torch.allclose(y - x, block[:, None, :].expand(t, s, h))
    w["up"] = torch.randn(s * h, r, generator=g(3))
    w["inject"] = torch.randn(s, s * h, generator=g(4))
    mixed2, gate2 = FN.hc_read(x, w)
    assert not torch.allclose(mixed2, mixed) and ((gate2 > 0) & (gate2 < 2)).all()
    assert FN.hc_read(x, w, inject=False)[1] is None
    # tokens are independent: a row's result does not depend on the other rows
    assert torch.allclose(FN.hc_read(x[2:3], w)[0], mixed2[2:3], atol=1e-6)


def test_causal_conv_chunks_carry_history():
    x = torch.randn(23, 6, generator=g())
    w = torch.randn(6, 4, generator=g(1))
    for dilation in (1, 3):
        whole, hist = FN.causal_conv(x, w, dilation)
        a, h1 = FN.causal_conv(x[:7], w, dilation)
        b, h2 = FN.causal_conv(x[7:8], w, dilation, h1)
        c, h3 = FN.causal_conv(x[8:], w, dilation, h2)
        assert torch.allclose(torch.cat([a, b, c]), whole, atol=1e-6)
        assert torch.equal(h3, hist) and hist.shape == (3 * dilation, 6)
        # causal: changing a later row leaves earlier outputs alone
        y = x.clone()
        y[15] += 1.0
        assert torch.equal(FN.causal_conv(y, w, dilation)[0][:15], whole[:15])
        # the taps are `dilation` apart: row 0 sees only the last tap
        assert torch.allclose(whole[0], torch.nn.functional.silu(x[0] * w[:, -1]), atol=1e-6)
    with pytest.raises(ValueError):
        FN.causal_conv(x, w, 1, torch.zeros(2, 6))


def test_ple_chunked_equals_whole_and_zero_value_is_identity():
    t, s, h, f = 11, 2, 8, 12
    x = torch.randn(t, s, h, generator=g())
    feats = torch.randn(t, f, generator=g(1))
    w = {"key": torch.randn(s * h, f, generator=g(2)) * 0.3,
         "value": torch.randn(h, f, generator=g(3)) * 0.3,
         "norm_key": torch.zeros(s * h), "norm_query": torch.zeros(s * h),
         "norm_conv": torch.zeros(s * h), "conv": torch.randn(s * h, 4, generator=g(4)) * 0.3}
    whole, hist = FN.ple(x, feats, w)
    a, h1 = FN.ple(x[:4], feats[:4], w)
    b, h2 = FN.ple(x[4:], feats[4:], w, history=h1)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-5) and torch.allclose(h2, hist)
    assert not torch.allclose(whole, x)
    w0 = dict(w, value=torch.zeros(h, f))
    assert torch.allclose(FN.ple(x, feats, w0)[0], x, atol=1e-3)    # nothing to inject


def test_qsa_selection_rules():
    top = 8
    cache = torch.randn(40, 128, generator=g())
    q = torch.randn(3, 4, 128, generator=g(1))
    sel = FN.qsa_select(q, cache, [10, 31, 130], top=top)
    assert sel.shape == (3, top * 4 + 3)
    assert sel[0][sel[0] >= 0].tolist() == list(range(11))          # few groups: everything causal
    assert sel[1][sel[1] >= 0].tolist() == list(range(32))          # exactly `top` groups, no tail
    row = sel[2][sel[2] >= 0]
    n = 131 // 4
    score = (q[2] @ cache[:n].t()).relu().sum(0) / math.sqrt(128)
    want = score.argsort(descending=True, stable=True)[:top]
    assert row[:top * 4:4].tolist() == (want * 4).tolist()
    assert row[top * 4:].tolist() == [128, 129, 130]                # the incomplete tail group
    assert row.max() <= 130 and len(set(row.tolist())) == len(row)
    tied = torch.zeros(40, 128)
    sel = FN.qsa_select(q[:1], tied, [130], top=top)                # all scores equal
    assert sel[0][:top * 4:4].tolist() == [4 * i for i in range(top)]


def test_qsa_attention_over_everything_is_dense_causal_attention():
    t, hq, hkv, d = 9, 4, 2, 16
    q = torch.randn(t, hq, d, generator=g())
    k = torch.randn(t, hkv, d, generator=g(1))
    v = torch.randn(t, hkv, d, generator=g(2))
    gate = torch.full((t, hq, d), 30.0)                             # sigmoid -> 1
    sel = torch.stack([torch.nn.functional.pad(torch.arange(i + 1), (0, t - i - 1), value=-1)
                       for i in range(t)]).int()
    got = FN.qsa_attention(q, k, v, gate, sel)
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("thd,shd->hts", q, kk) * d ** -0.5
    s = s.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool), 1), float("-inf"))
    want = torch.einsum("hts,shd->thd", s.softmax(-1), vv)
    assert torch.allclose(got, want, atol=1e-5)
    closed = FN.qsa_attention(q, k, v, torch.full((t, hq, d), -30.0), sel)
    assert closed.abs().max() < 1e-6


def test_qsa_index_groups_and_kv_codec():
    qk = torch.randn(10, 5, 128, generator=g())
    q, k = FN.qsa_index(qk, torch.zeros(128), torch.zeros(128))
    assert q.shape == (10, 4, 128) and k.shape == (2, 128)          # 10 // 4 complete groups
    q8, k8 = FN.qsa_index(qk[:8], torch.zeros(128), torch.zeros(128))
    assert torch.equal(q8, q[:8]) and torch.equal(k8, k)            # tail tokens change nothing
    qb, kb = FN.qsa_index(qk[4:8], torch.zeros(128), torch.zeros(128), first=4)
    assert torch.allclose(qb, q[4:8], atol=1e-6) and torch.allclose(kb[0], k[1], atol=1e-6)
    # rotation keeps norms and leaves channels >= 64 alone
    x = torch.randn(3, 2, 128, generator=g(1))
    y = FN.qsa_rope(x, torch.tensor([0, 5, 900]))
    assert torch.equal(y[..., 64:], x[..., 64:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    kv = torch.randn(6, 2, 256, generator=g(2))
    codes, scale = FN.quantize_kv(kv)
    assert codes.dtype == torch.int8 and scale.shape == (6, 2, 4) and scale.dtype == torch.float16
    assert (FN.dequantize_kv(codes, scale) - kv).abs().max() < kv.abs().max() / 127 * 0.51 + 1e-3
