"""CUDA kernels against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

from orinfer_b200.quant import e8p_torch
from orinfer_b200.ref import ops_ref as R

pytestmark = pytest.mark.gpu


def _signs(k, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (1 - 2 * torch.randint(0, 2, (k,), generator=g)).to(torch.int8).to(dev)


def _codes_close(q, q_ref, frac=0.01):
    d = (q.int() - q_ref.int()).abs()
    assert int(d.max()) <= 1, f"max code diff {int(d.max())}"
    assert float((d > 0).float().mean()) <= frac


def test_basis_matches_python(cuda):
    from orinfer_b200.ops import native
    from orinfer_b200.quant import e8p
    assert torch.equal(native.basis_host(), torch.from_numpy(e8p.basis().copy()))


def test_embed_w8(cuda):
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(0)
    table = torch.randint(-127, 128, (300, 256), generator=g, dtype=torch.int8).to(cuda)
    scale = (torch.rand(300, generator=g) * 0.01 + 1e-3).half().to(cuda)
    ids = torch.randint(0, 300, (37,), generator=g, dtype=torch.int32).to(cuda)
    out = F.embed_w8(ids, table, scale)
    assert torch.equal(out.float(), R.embed_w8(ids, table, scale))


@pytest.mark.parametrize("k,m", [(128, 19), (256, 19), (2560, 19), (2560, 3), (5120, 1),
                                 (1152, 16)])
@pytest.mark.parametrize("mode", ["norm_rot", "rot", "norm", "plain", "zero"])
def test_act_prep(cuda, k, m, mode):
    """m <= 16 with at least 8 blocks of 128 channels runs as a cluster of CTAs per row."""
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(k)
    x = (torch.randn(m, k, generator=g) * 0.5).half().to(cuda)
    if mode == "zero":
        x.zero_()
    resid = torch.randn(m, k, generator=g).to(cuda) if mode in ("norm_rot", "norm") else None
    w = (1 + 0.1 * torch.randn(k, generator=g)).half().to(cuda) if "norm" in mode else None
    sg = _signs(k, cuda) if "rot" in mode else None
    r_in = None if resid is None else resid.clone()
    y_out = torch.empty(m, k, dtype=torch.float16, device=cuda)
    q, s = F.act_prep(x, resid, w, sg, eps=1e-6, y_out=y_out)
    q_ref, s_ref, r_ref, y_ref = R.act_prep(x, r_in, w, sg, 1e-6)
    assert torch.allclose(s, s_ref, rtol=2e-3, atol=0)
    if resid is not None:
        assert torch.allclose(resid, r_ref, atol=1e-6)
    assert float((y_out.float() - y_ref).abs().max()) <= 2e-3 * max(1.0, float(y_ref.abs().max()))
    _codes_close(q, q_ref, 0.02)


@pytest.mark.parametrize("m,f", [(11, 512), (2, 2560), (1, 9728), (40, 1280)])
def test_act_prep_swiglu(cuda, m, f):
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(m, 2 * f, generator=g).half().to(cuda)
    sg = _signs(f, cuda)
    q, s = F.act_prep(gu, None, None, sg, swiglu=True)
    q_ref, s_ref, _, _ = R.act_prep(gu, None, None, sg, swiglu=True)
    assert torch.allclose(s, s_ref, rtol=2e-3)
    _codes_close(q, q_ref, 0.02)


def _rand_weight(fmt, n, k, dev, seed):
    g = torch.Generator().manual_seed(seed)
    ws = (torch.rand(n, generator=g) * 0.01 + 1e-3).half().to(dev)
    if fmt == "w8":
        codes = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(dev)
        return codes, ws, codes
    if fmt == "q4":
        codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 128, n, 16), generator=g,
                              dtype=torch.int64).to(torch.int32).to(dev)
        rows = codes.permute(1, 0, 2).reshape(n, k // 8).to(torch.int64) & 0xFFFFFFFF
        w_int = (4 * e8p_torch.decode_t(rows & 0xFFFF).to(torch.int32)
                 + e8p_torch.decode_t(rows >> 16).to(torch.int32)).reshape(n, k).to(torch.int8)
        return codes, ws, w_int
    codes = torch.randint(-2 ** 15, 2 ** 15 - 1, (k // 128, n, 16), generator=g,
                          dtype=torch.int64).to(torch.int16).to(dev)
    rows = codes.permute(1, 0, 2).reshape(n, k // 8).to(torch.int64) & 0xFFFF
    return codes, ws, e8p_torch.decode_t(rows).reshape(n, k)


@pytest.mark.parametrize("fmt", ["w8", "q4", "q2"])
@pytest.mark.parametrize("m,n,k,path", [
    (1, 256, 256, 1), (3, 136, 128, 1), (8, 2560, 1024, 1), (5, 256, 512, 2),
    (16, 128, 128, 2), (128, 384, 1024, 2), (200, 2560, 2560, 2), (512, 1536, 1280, 0),
    # tile variants: 4 / 2 / 1 accumulators x 128 / 64 / 32 weight rows per CTA, ragged N
    (600, 19456, 256, 0), (1000, 6400, 128, 0), (250, 12800, 128, 0), (100, 12800, 256, 0),
    (700, 8200, 256, 0), (50, 1000, 128, 0), (513, 2560, 1024, 0),
    # split-K (narrow N, long K): INT32 partials + finalize must equal the unsplit result
    (512, 2560, 9728, 0), (100, 2560, 4096, 0), (300, 1024, 2560, 0), (512, 6144, 2560, 0),
    # one M tile, a few weight tiles more than SMs: full wave + split-K tail launch
    (512, 19456, 1024, 0), (100, 19968, 1024, 0),
    # persistent kernel: several tiles per CTA, last M tile with one active sub-tile, 8 k-blocks
    (1100, 19456, 1024, 0), (2100, 9728, 384, 0),
    # K-split GEMV shapes (narrow N) and a wide one
    (1, 2560, 9728, 1), (7, 6144, 2560, 1), (2, 320, 1280, 1), (1, 19456, 2560, 1),
    # rows too long to stage eight of them beside the tables: the rows go in two launches
    (7, 256, 20480, 1),
])
def test_qgemm(cuda, fmt, m, n, k, path):
    from orinfer_b200.ops import functional as F
    from orinfer_b200.ops import native
    native.qgemm_set_impl(1)
    g = torch.Generator().manual_seed(m * 7 + n)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(cuda)
    sa = (torch.rand(m, generator=g) * 0.05 + 1e-3).to(cuda)
    codes, ws, w_int = _rand_weight(fmt, n, k, cuda, seed=k + n)
    for f32 in (False, True):
        out = F.qgemm(a, sa, codes, ws, fmt, n, out_f32=f32, path=path)
        ref = R.qgemm(a, sa, w_int, ws, out_f32=f32)
        torch.cuda.synchronize()
        assert torch.equal(out.float(), ref), \
            f"max diff {float((out.float() - ref).abs().max())}"


@pytest.mark.parametrize("fmt", ["w8", "q4"])
@pytest.mark.parametrize("m,n,k", [(600, 19456, 256), (512, 2560, 9728), (100, 12800, 256),
                                   (513, 2560, 1024), (1100, 19456, 1024), (2100, 9728, 384)])
def test_qgemm_persistent_form(cuda, fmt, m, n, k):
    """The persistent kernel gives the same bits as the one-tile-per-CTA one."""
    from orinfer_b200.ops import functional as F
    from orinfer_b200.ops import native
    g = torch.Generator().manual_seed(m + n)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(cuda)
    sa = (torch.rand(m, generator=g) * 0.05 + 1e-3).to(cuda)
    codes, ws, w_int = _rand_weight(fmt, n, k, cuda, seed=k + n)
    try:
        native.qgemm_set_impl(0)
        out = F.qgemm(a, sa, codes, ws, fmt, n)
        torch.cuda.synchronize()
    finally:
        native.qgemm_set_impl(1)
    assert torch.equal(out.float(), R.qgemm(a, sa, w_int, ws))


@pytest.mark.parametrize("fmt", ["w8", "q4", "q2"])
@pytest.mark.parametrize("m,n,k", [(600, 19456, 256), (512, 2560, 9728), (1100, 9728, 1024),
                                   (300, 2432, 2560), (513, 2560, 1024), (129, 256, 128),
                                   (2100, 1000, 384)])
def test_qgemm_cta_pair_form(cuda, fmt, m, n, k):
    """cta_group::2: two CTAs share a 512 x 256 tile; ragged M, ragged N (a pair whose odd
    CTA has no weight rows), several tiles per pair.  Same bits as the oracle."""
    from orinfer_b200.ops import functional as F
    from orinfer_b200.ops import native
    g = torch.Generator().manual_seed(m + n)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(cuda)
    sa = (torch.rand(m, generator=g) * 0.05 + 1e-3).to(cuda)
    codes, ws, w_int = _rand_weight(fmt, n, k, cuda, seed=k + n)
    try:
        native.qgemm_set_impl(2)
        out = F.qgemm(a, sa, codes, ws, fmt, n)
        out32 = F.qgemm(a, sa, codes, ws, fmt, n, out_f32=True)
        torch.cuda.synchronize()
    finally:
        native.qgemm_set_impl(1)
    assert torch.equal(out.float(), R.qgemm(a, sa, w_int, ws))
    assert torch.equal(out32, R.qgemm(a, sa, w_int, ws, out_f32=True))


@pytest.mark.parametrize("fmt", ["q4", "q2"])
@pytest.mark.parametrize("m,n,k", [(1, 2560, 2560), (1, 19456, 2560), (3, 6144, 2560),
                                   (8, 2560, 1024), (1, 2560, 9728), (5, 320, 1280)])
def test_qgemv_fused_equals_separate_kernels(cuda, fmt, m, n, k):
    """The projection with the row preparation fused in gives the bits of act_prep + qgemm,
    for the norm, plain and SwiGLU prologues and for the residual-accumulating epilogue."""
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(m + n + k)
    codes, ws, _ = _rand_weight(fmt, n, k, cuda, seed=n + k)
    sg = _signs(k, cuda)
    norm_w = (1 + 0.1 * torch.randn(k, generator=g)).half().to(cuda)
    x = (torch.randn(8, k, generator=g) * 0.5).half().to(cuda)
    resid = torch.randn(8, k, generator=g).to(cuda)
    gu = torch.randn(8, 2 * k, generator=g).half().to(cuda)
    for pre in (F.PRE_NORM, F.PRE_PLAIN, F.PRE_SWIGLU):
        if pre == F.PRE_NORM:
            r2 = resid.clone()
            q8, sc = F.act_prep(x, r2, norm_w, sg, eps=1e-6, rows=m)
            args = (x, resid, norm_w)
        elif pre == F.PRE_PLAIN:
            q8, sc = F.act_prep(x, None, None, sg, rows=m)
            args = (x, None, None)
        else:
            q8, sc = F.act_prep(gu, None, None, sg, swiglu=True, rows=m)
            args = (gu, None, None)
        want = F.qgemm(q8, sc, codes, ws, fmt, n, rows=m)
        out = torch.zeros(8, n, dtype=torch.float16, device=cuda)
        acc = torch.ones(8, n, device=cuda)
        qo = torch.zeros(8, k, dtype=torch.int8, device=cuda)
        so = torch.zeros(8, device=cuda)
        assert F.qgemv_fused(pre, args[0], args[1], args[2], sg, codes, ws, fmt, n, k, m,
                             out=out, resid_accum=acc, q_out=qo, scale_out=so)
        torch.cuda.synchronize()
        assert torch.equal(qo[:m], q8[:m]) and torch.equal(so[:m], sc[:m]), pre
        assert torch.equal(out[:m], want[:m]), (pre, float((out[:m].float() - want[:m].float()).abs().max()))
        assert torch.equal(acc[:m], 1 + want[:m].float())


def test_qgemm_graph_replay_changed_inputs(cuda):
    """Capture once, replay with different activation contents."""
    from orinfer_b200.ops import functional as F
    m, n, k = 64, 256, 512
    a = torch.zeros(m, k, dtype=torch.int8, device=cuda)
    sa = torch.ones(m, device=cuda)
    codes, ws, w_int = _rand_weight("q4", n, k, cuda, 5)
    out = torch.empty(m, n, dtype=torch.float16, device=cuda)
    F.qgemm(a, sa, codes, ws, "q4", n, out=out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        F.qgemm(a, sa, codes, ws, "q4", n, out=out)
    for seed in (1, 2):
        g = torch.Generator().manual_seed(seed)
        a.copy_(torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8))
        sa.copy_(torch.rand(m, generator=g) * 0.1 + 0.01)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.float(), R.qgemm(a, sa, w_int, ws))


def _paged_setup(cuda, lens, kvh, d, seed=0):
    """Random INT8 KV for requests of the given lengths, scattered over pages."""
    g = torch.Generator().manual_seed(seed)
    n_req = len(lens)
    pages_per = [(l + 127) // 128 for l in lens]
    total = sum(pages_per) + 1
    perm = (torch.randperm(total - 1, generator=g) + 1).tolist()
    table = torch.zeros(n_req, max(pages_per), dtype=torch.int32)
    it = iter(perm)
    for r, npg in enumerate(pages_per):
        for j in range(npg):
            table[r, j] = next(it)
    kc = torch.randint(-127, 128, (total, 128, kvh, d), generator=g, dtype=torch.int8)
    vc = torch.randint(-127, 128, (total, 128, kvh, d), generator=g, dtype=torch.int8)
    ks = (torch.rand(total, 128, kvh, d // 64, generator=g) * 0.02 + 1e-3).half()
    vs = (torch.rand(total, 128, kvh, d // 64, generator=g) * 0.02 + 1e-3).half()
    return table.to(cuda), kc.to(cuda), vc.to(cuda), ks.to(cuda), vs.to(cuda)


def _gather_kv(table, cache, scale, req, length):
    pos = torch.arange(length, device=cache.device)
    pages = table[req, pos // 128].long()
    return R.kv_dequant(cache[pages, pos % 128], scale[pages, pos % 128])


@pytest.mark.parametrize("qh,kvh,d", [(4, 2, 64), (32, 8, 128), (40, 8, 128), (16, 2, 256)])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_attention_rows(cuda, qh, kvh, d, splits):
    from orinfer_b200.ops import functional as F
    lens = [1, 130, 300]
    table, kc, vc, ks, vs = _paged_setup(cuda, lens, kvh, d)
    g = torch.Generator().manual_seed(1)
    # rows: last row of request 0, last 3 rows of request 1, rows 100..101 of request 2
    row_req = torch.tensor([0, 1, 1, 1, 2, 2], dtype=torch.int32, device=cuda)
    row_pos = torch.tensor([0, 127, 128, 129, 100, 299], dtype=torch.int32, device=cuda)
    q = torch.randn(6, qh, d, generator=g).half().to(cuda)
    gate = torch.randn(6, qh, d, generator=g).half().to(cuda) if d == 256 else None
    out = F.attention(q, gate, row_req, row_pos, table, kc, vc, ks, vs, splits=splits)
    for i in range(6):
        r, pos = int(row_req[i]), int(row_pos[i])
        k = _gather_kv(table, kc, ks, r, pos + 1)
        v = _gather_kv(table, vc, vs, r, pos + 1)
        ref = R.causal_gqa(q[i:i + 1], k, v, pos, None if gate is None else gate[i:i + 1])
        assert torch.allclose(out[i].float(), ref[0], atol=2e-3, rtol=2e-3), \
            f"row {i}: {float((out[i].float() - ref[0]).abs().max())}"


@pytest.mark.parametrize("qh,kvh,d,gated", [(4, 2, 64, False), (32, 8, 128, False),
                                             (16, 2, 256, True)])
def test_qk_rope_kv(cuda, qh, kvh, d, gated):
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(2)
    rows = 9
    width = qh * d * (2 if gated else 1) + 2 * kvh * d
    qkv = torch.randn(rows, width, generator=g).half().to(cuda)
    wq = (1 + 0.1 * torch.randn(d, generator=g)).half().to(cuda)
    wk = (1 + 0.1 * torch.randn(d, generator=g)).half().to(cuda)
    row_req = torch.tensor([0, 0, 0, 1, 1, 1, 1, 1, 1], dtype=torch.int32, device=cuda)
    row_pos = torch.tensor([126, 127, 128, 0, 1, 2, 3, 4, 5], dtype=torch.int32, device=cuda)
    table = torch.tensor([[3, 1], [2, 0]], dtype=torch.int32, device=cuda)
    kc = torch.zeros(4, 128, kvh, d, dtype=torch.int8, device=cuda)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(4, 128, kvh, d // 64, dtype=torch.float16, device=cuda)
    vs = torch.zeros_like(ks)
    cos, sin = F.rope_table(row_pos, d, 1e6)
    cos_r, sin_r = R.rope_tables(row_pos, d, 1e6)
    assert torch.allclose(cos, cos_r, atol=1e-6) and torch.allclose(sin, sin_r, atol=1e-6)
    q_out, gate_out = F.qk_rope_kv(qkv, wq, wk, cos, sin, row_req, row_pos, table, kc, vc, ks, vs,
                                   qh=qh, kvh=kvh, head_dim=d, gated=gated)
    qs = d * (2 if gated else 1)
    qraw = qkv[:, :qh * qs].reshape(rows, qh, qs)
    q_ref = R.qk_norm_rope(qraw[..., :d], wq, cos_r, sin_r, 1e-6, False)
    assert float((q_out.float() - q_ref).abs().max()) <= 4e-3
    if gated:
        assert torch.equal(gate_out, qraw[..., d:].contiguous())
    kraw = qkv[:, qh * qs:qh * qs + kvh * d].reshape(rows, kvh, d)
    vraw = qkv[:, qh * qs + kvh * d:].reshape(rows, kvh, d)
    k_ref = R.qk_norm_rope(kraw, wk, cos_r, sin_r, 1e-6, False)
    kq_ref, ks_ref = R.kv_quant(k_ref)
    vq_ref, vs_ref = R.kv_quant(R.f16(vraw.float()))
    for i in range(rows):
        page = int(table[int(row_req[i]), int(row_pos[i]) // 128])
        slot = int(row_pos[i]) % 128
        assert torch.equal(vc[page, slot], vq_ref[i])
        assert torch.equal(vs[page, slot].float(), vs_ref[i])
        assert torch.allclose(ks[page, slot].float(), ks_ref[i], rtol=2e-3)
        deq = R.kv_dequant(kc[page, slot], ks[page, slot])
        assert float((deq - k_ref[i]).abs().max()) <= 1.5 * float(ks_ref[i].max()) + 4e-3


def test_argmax(cuda):
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(4)
    for vocab in (1024, 5000, 151936):
        lg = torch.randn(5, vocab, generator=g).to(cuda)
        lg[1, 7] = lg[1, 900] = 50.0          # tie -> lowest index
        lg[2, vocab - 1] = 99.0
        tok = F.argmax(lg)
        assert torch.equal(tok, R.argmax_lowest(lg))
        assert int(tok[1]) == 7 and int(tok[2]) == vocab - 1
    lg[3, 5] = float("nan")
    assert int(F.argmax(lg)[3]) == -1


def test_e8p_encode_kernel(cuda):
    from orinfer_b200.ops import native
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(5000, 8, generator=g) * 4).to(cuda)
    codes = native.e8p_encode(x)
    ref = e8p_torch.encode_nearest_t(x)
    d_mine = ((x - e8p_torch.decode_t(codes).float()) ** 2).sum(1)
    d_ref = ((x - e8p_torch.decode_t(ref).float()) ** 2).sum(1)
    assert float((d_mine - d_ref).abs().max()) < 1e-3
    assert float((codes == ref).float().mean()) > 0.995


@pytest.mark.parametrize("qh,kvh,d", [(32, 8, 128), (40, 8, 128), (4, 2, 64), (8, 1, 128),
                                       (16, 2, 256), (2, 2, 256)])
def test_attention_prefill_tensor_core(cuda, qh, kvh, d):
    """Two chunks: a fresh 300-token prompt and a 130-row continuation at position 200."""
    from orinfer_b200.ops import functional as F
    lens = [300, 330]
    table, kc, vc, ks, vs = _paged_setup(cuda, lens, kvh, d, seed=7)
    g = torch.Generator().manual_seed(8)
    rows = 300 + 130
    q = torch.randn(rows, qh, d, generator=g).half().to(cuda)
    chunks = torch.tensor([[0, 300, 0, 0], [300, 130, 200, 1]], dtype=torch.int32, device=cuda)
    out = torch.zeros(rows, qh * d, dtype=torch.float16, device=cuda)
    assert F.attention_prefill(q, None, chunks, 300, table, kc, vc, ks, vs, out=out)
    torch.cuda.synchronize()
    for (r0, n, pos0, req) in chunks.tolist():
        k = _gather_kv(table, kc, ks, req, pos0 + n)
        v = _gather_kv(table, vc, vs, req, pos0 + n)
        ref = R.causal_gqa(q[r0:r0 + n], k, v, pos0)
        err = (out[r0:r0 + n].float() - ref).abs()
        assert float(err.max()) < 2e-2 * max(1.0, float(ref.abs().max())), float(err.max())
        assert float(err.mean()) < 2e-3 * max(1.0, float(ref.abs().mean()) * 10)


def test_attention_prefill_matches_row_kernel(cuda):
    from orinfer_b200.ops import functional as F
    qh, kvh, d = 32, 8, 128
    table, kc, vc, ks, vs = _paged_setup(cuda, [700], kvh, d, seed=9)
    g = torch.Generator().manual_seed(10)
    n, pos0 = 200, 500
    q = torch.randn(n, qh, d, generator=g).half().to(cuda)
    gate = torch.randn(n, qh, d, generator=g).half().to(cuda)
    chunks = torch.tensor([[0, n, pos0, 0]], dtype=torch.int32, device=cuda)
    out = torch.zeros(n, qh * d, dtype=torch.float16, device=cuda)
    assert F.attention_prefill(q, gate, chunks, n, table, kc, vc, ks, vs, out=out)
    req = torch.zeros(n, dtype=torch.int32, device=cuda)
    pos = torch.arange(pos0, pos0 + n, dtype=torch.int32, device=cuda)
    rows = F.attention(q, gate, req, pos, table, kc, vc, ks, vs)
    assert float((out.float() - rows.float()).abs().max()) < 2e-2


@pytest.mark.parametrize("experts,top_k,shared", [(8, 2, False), (128, 8, False), (512, 10, True)])
def test_router_topk(cuda, experts, top_k, shared):
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(experts)
    m, h = 37, 256
    y = torch.randn(m, h, generator=g).half().to(cuda)
    w = (torch.randn(experts + int(shared), h, generator=g) * 0.1).half().to(cuda)
    w[3] = w[1]                                             # exact tie -> lower id first
    ids, probs, gate = F.router_topk(y, w, experts, top_k, renorm=True)
    logits = y.float() @ w.float().t()
    p = torch.softmax(logits[:, :experts], -1)
    order = torch.sort(p, dim=-1, descending=True, stable=True).indices[:, :top_k]
    ref_p = torch.gather(p, 1, order)
    ref_p = ref_p / ref_p.sum(-1, keepdim=True)
    same = (ids.long() == order).float().mean()
    assert same > 0.98, same                                # fp32 sum order can swap near-ties
    assert torch.allclose(probs.sum(-1), torch.ones(m, device=cuda), atol=1e-5)
    agree = ids.long() == order
    assert torch.allclose(probs[agree], ref_p[agree], atol=2e-4)
    if shared:
        assert torch.allclose(gate, torch.sigmoid(logits[:, experts]), atol=2e-4)


@pytest.mark.parametrize("fmt", ["q4", "q2", "w8"])
def test_moe_dispatch_grouped_gemm_combine(cuda, fmt):
    """Dispatch -> grouped GEMM -> combine against per-assignment dense arithmetic."""
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(11)
    m, h, n, experts, top_k = 300, 256, 384, 8, 2
    ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(m)]) \
        .to(torch.int32).to(cuda)
    ids[:40] = torch.tensor([5, 2], dtype=torch.int32)      # one expert with > 128 rows
    probs = torch.rand(m, top_k, generator=g).to(cuda)
    q8 = torch.randint(-127, 128, (m, h), generator=g, dtype=torch.int8).to(cuda)
    sa = (torch.rand(m, generator=g) * 0.05 + 1e-3).to(cuda)
    banks = [_rand_weight(fmt, n, h, cuda, seed=100 + e) for e in range(experts)]
    codes = torch.stack([b[0] for b in banks]).contiguous()
    wscale = torch.stack([b[1] for b in banks]).contiguous()
    sc = F.MoeScratch(m, top_k, experts, h, n // 2, cuda)
    F.moe_dispatch(ids, q8, sa, experts, sc, m)
    out = torch.zeros(m * top_k, n, dtype=torch.float16, device=cuda)
    F.qgemm_grouped(sc.q8, sc.scale, codes, wscale, fmt, n, out, sc, m * top_k)
    torch.cuda.synchronize()
    counts = torch.bincount(ids.flatten().long(), minlength=experts)
    assert torch.equal(sc.counts.long(), counts)
    slots = sc.slots.view(m, top_k).long()
    assert sorted(slots.flatten().tolist()) == list(range(m * top_k))
    for r in (0, 1, 39, 40, 150, 299):
        for j in range(top_k):
            e = int(ids[r, j])
            ref = R.qgemm(q8[r:r + 1], sa[r:r + 1], banks[e][2], banks[e][1])
            assert torch.equal(out[slots[r, j]].float(), ref[0]), (r, j)
    # stable slots: within an expert, slots follow (row, k) order
    for e in range(experts):
        s = slots.flatten()[ids.flatten().long() == e]
        assert torch.equal(s, torch.sort(s).values)
    hidden_out = torch.zeros(m, n, dtype=torch.float16, device=cuda)
    F.moe_combine(out, sc.slots, probs, None, None, hidden_out, m)
    ref = (out[slots].float() * probs[..., None]).sum(1)
    assert torch.allclose(hidden_out.float(), ref, atol=2e-2, rtol=2e-3)


def test_moe_expert_parallel_partials_sum_to_full(cuda):
    """Two expert-parallel halves (experts [0,4) and [4,8)): each dispatches only its own
    rows (other slots -1), and their combined partial sums equal the single-rank result."""
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(12)
    m, h, n, experts, top_k = 200, 256, 256, 8, 2
    ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(m)]) \
        .to(torch.int32).to(cuda)
    probs = torch.rand(m, top_k, generator=g).to(cuda)
    q8 = torch.randint(-127, 128, (m, h), generator=g, dtype=torch.int8).to(cuda)
    sa = (torch.rand(m, generator=g) * 0.05 + 1e-3).to(cuda)
    banks = [_rand_weight("q4", n, h, cuda, seed=200 + e) for e in range(experts)]
    codes = torch.stack([b[0] for b in banks]).contiguous()
    wscale = torch.stack([b[1] for b in banks]).contiguous()

    def run(base, local):
        sc = F.MoeScratch(m, top_k, experts, h, n // 2, cuda)
        F.moe_dispatch(ids, q8, sa, experts, sc, m, base, local)
        out = torch.zeros(m * top_k, n, dtype=torch.float16, device=cuda)
        F.qgemm_grouped(sc.q8, sc.scale, codes[base:base + local].contiguous(),
                        wscale[base:base + local].contiguous(), "q4", n, out, sc, m * top_k)
        res = torch.zeros(m, n, dtype=torch.float16, device=cuda)
        F.moe_combine(out, sc.slots, probs, None, None, res, m)
        torch.cuda.synchronize()
        return res.float(), sc.slots.view(m, top_k).clone()

    full, _ = run(0, experts)
    lo, slots_lo = run(0, 4)
    hi, slots_hi = run(4, 4)
    assert torch.equal(slots_lo < 0, ids >= 4) and torch.equal(slots_hi < 0, ids < 4)
    assert torch.allclose(lo + hi, full, atol=3e-2, rtol=3e-3)


def test_device_topk_sampler_matches_host_law(cuda):
    """Same uniform, same law: the device draw equals the host law's draw row by row,
    including ties at the top-k threshold (lowest ids win) and a nucleus cut."""
    from orinfer_b200.core import sampling as S
    from orinfer_b200.ops import functional as F
    g = torch.Generator().manual_seed(21)
    rows, vocab = 48, 5000
    logits = torch.randn(rows, vocab, generator=g) * 3
    logits[5, 100:140] = logits[5].max() + 1.0          # 40 equal maxima: ties inside the top-k
    logits[6] = torch.round(logits[6])                   # many exact ties everywhere
    ks = [1 + (7 * i) % 64 for i in range(rows)]
    temps = [0.3 + 0.03 * i for i in range(rows)]
    tops = [1.0 if i % 3 else 0.8 for i in range(rows)]
    us = [S.counter_uniform(1234, 0, i) for i in range(rows)]
    dev = lambda v, dt: torch.tensor(v, dtype=dt, device=cuda)
    tok, flag = F.sample_topk(logits.to(cuda), dev(ks, torch.int32), dev(temps, torch.float64),
                              dev(tops, torch.float64), dev(us, torch.float64))
    assert flag.sum().item() == 0
    want = [S.sample(logits[i].numpy(), [], S.SamplingOptions(temperature=temps[i], top_p=tops[i],
                                                              top_k=ks[i]), us[i])
            for i in range(rows)]
    assert tok.cpu().tolist() == want
    # a row of all-equal logits has more ties than the shortlist holds: handed to the host
    flat = torch.zeros(1, vocab)
    _, flag = F.sample_topk(flat.to(cuda), dev([8], torch.int32), dev([1.0], torch.float64),
                            dev([1.0], torch.float64), dev([0.5], torch.float64))
    assert flag.item() == 1
