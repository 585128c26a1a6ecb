"""Each mechanism of the Guduzen decoder alone: the kernel, or the part that strings kernels together, against the
plain function of the same name, on sizes of its own (also sizes the kernels must widen or cut)."""
import math

import pytest
import torch

import plain_guduzen as plain
from gpullama3.java_b200.kernels import ops

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
F = torch.float64


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("streams, width, T", [(1, 48, 5), (2, 64, 33), (3, 100, 7), (8, 30, 3), (4, 2500, 2)])
def test_streams(streams, width, T):
    x = _rand(T, width, seed=1).cuda()
    xs = torch.empty(T, streams, width, device="cuda")
    ops.streams_combine(x.view(T, 1, width), xs, torch.ones(streams, device="cuda"))
    assert torch.equal(xs, x[:, None, :].expand(T, streams, width))
    xs = _rand(T, streams, width, seed=2).cuda()
    W = {"h.in": _rand(streams, seed=3).to(F), "h.mix": _rand(streams, streams, seed=4).to(F), "h.out": _rand(streams, seed=5).to(F)}
    nw = _rand(width, seed=6) * 0.3
    # read + norm
    out = torch.empty(T, width, device="cuda")
    ops.streams_read_norm(xs, W["h.in"].float().cuda(), (1 + nw).cuda(), out, 1e-5)
    lst = [xs[:, a].cpu().to(F) for a in range(streams)]
    u = sum(W["h.in"][a] * lst[a] for a in range(streams))
    torch.testing.assert_close(out.cpu().to(F), plain.offset_norm(u, nw.to(F), 1e-5), rtol=2e-5, atol=2e-5)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    out2 = torch.empty(2, width, device="cuda", dtype=torch.bfloat16)
    ops.streams_read_norm(xs, W["h.in"].float().cuda(), (1 + nw).cuda(), out2, 1e-5, rows)
    torch.testing.assert_close(out2.float().cpu(), out[[T - 1, 0]].cpu(), rtol=1e-2, atol=1e-2)
    # write back, in place
    y = _rand(T, width, seed=7).cuda()
    ref = plain.connect(lst, W, "h.", y.cpu().to(F))
    ops.streams_combine(xs, xs, W["h.mix"].float().cuda(), W["h.out"].float().cuda(), y)
    for j in range(streams):
        torch.testing.assert_close(xs[:, j].cpu().to(F), ref[j], rtol=2e-5, atol=2e-5)
    # the sum that closes the streams
    total = torch.empty(T, 1, width, device="cuda")
    ops.streams_combine(xs, total, torch.ones(streams, device="cuda"))
    torch.testing.assert_close(total[:, 0].cpu().to(F), sum(ref), rtol=2e-5, atol=2e-5)


@DTYPES
def test_head_rows(dtype):
    T, H, G, dk, dv, D = 9, 3, 1, 24, 40, 64
    src = _rand(T, H * dk + G * dk + G * dv, seed=1).to(dtype).cuda()
    bias = _rand(src.shape[1], seed=2).cuda()
    weight = _rand(dk, seed=3).cuda()
    dst = torch.full((T, (H + 2 * G) * D), 7.0, dtype=dtype, device="cuda")
    segs = ops.head_row_segments(ops.head_row_segment(0, H, dk, 0, D, 0, True, -1, 2.5),
                                 ops.head_row_segment(H * dk, G, dk, H * D, D, H * dk, True, 0),
                                 ops.head_row_segment((H + G) * dk, G, dv, (H + G) * D, D, (H + G) * dk))
    ops.head_rows(src, dst, segs, 1e-5, bias, weight)
    z = src.cpu().to(F) + bias.cpu().to(F)
    q = plain.rms_normalise(z[:, :H * dk].view(T, H, dk), 1e-5) * 2.5
    k = plain.rms_normalise(z[:, H * dk:(H + G) * dk].view(T, G, dk), 1e-5) * weight.cpu().to(F)
    v = z[:, (H + G) * dk:].view(T, G, dv)
    got = dst.cpu().to(F).view(T, H + 2 * G, D)
    torch.testing.assert_close(got[:, :H, :dk], q, **_tol(dtype))
    torch.testing.assert_close(got[:, H:H + G, :dk], k, **_tol(dtype))
    torch.testing.assert_close(got[:, H + G:, :dv], v, **_tol(dtype))
    assert float(got[:, :H + G, dk:].abs().max()) == 0.0 and float(got[:, H + G:, dv:].abs().max()) == 0.0


def test_softcap():
    x = _rand(7, 300, seed=1, scale=30.0).cuda()
    ref = plain.softcap(x.cpu().to(F), 12.5)
    ops.softcap_rows(x, 12.5)
    torch.testing.assert_close(x.cpu().to(F), ref, rtol=1e-5, atol=1e-5)


@DTYPES
@pytest.mark.parametrize("M, K, N", [(3, 64, 96), (12, 96, 40), (40, 64, 96), (100, 64, 96), (300, 64, 96), (700, 200, 520),
                                     (2048, 512, 1536), (5, 60, 30)])
def test_gated_gelu_feed_forward_product(dtype, M, K, N):
    """The gate/up product with the GELU in its epilogue: the plain kernel, the decode kernel, the tensor-core kernels
    for prompts (single CTAs and pairs), and sizes none of those takes."""
    from gpullama3.java_b200.parts.linear import Linear

    x = _rand(M, K, seed=1).to(dtype).cuda()
    gate, up = _rand(N, K, seed=2, scale=0.2).to(dtype), _rand(N, K, seed=3, scale=0.2).to(dtype)
    lin = Linear(torch.stack([gate, up], dim=1).reshape(2 * N, K).contiguous().cuda())
    out = lin.gated(x, dtype, None, "gelu_tanh")
    xf = x.cpu().to(F)
    ref = plain.gelu_tanh(xf @ gate.to(F).T) * (xf @ up.to(F).T)
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)   # (sums of up to 512 products)
    torch.testing.assert_close(out.cpu().to(F), ref, **tol)


@DTYPES
@pytest.mark.parametrize("taps, C", [(1, 8), (2, 40), (4, 130)])
def test_short_convolution_with_state(dtype, taps, C):
    """Three sequences of unequal length in slots 5, 0 and 2, fed in two steps (the second continues from the state
    the first left, also for a sequence whose first step was shorter than the taps)."""
    lens = [7, 1, 12]
    second = [3, 2, 1]
    slots = torch.tensor([5, 0, 2], dtype=torch.int32, device="cuda")
    w = _rand(C, taps, seed=1).cuda()
    xs = [_rand(a + b, C + 3, seed=10 + i).to(dtype) for i, (a, b) in enumerate(zip(lens, second))]
    state = torch.zeros(6, 17 + (taps - 1) * C, device="cuda")
    outs = [[] for _ in lens]
    for part in (0, 1):
        pieces = [x[:a] if part == 0 else x[a:] for x, a in zip(xs, lens)]
        n = [p.shape[0] for p in pieces]
        packed = torch.cat(pieces).cuda()
        cu = torch.tensor([0, n[0], n[0] + n[1], sum(n)], dtype=torch.int32, device="cuda")
        seq_ids = torch.repeat_interleave(torch.arange(3, dtype=torch.int32), torch.tensor(n)).cuda()
        out = torch.empty(sum(n), C, dtype=dtype, device="cuda")
        ops.causal_conv_silu(packed, w, state[:, 17:], slots, seq_ids, cu, out, C)
        for i in range(3):
            outs[i].append(out[int(cu[i]):int(cu[i + 1])].cpu())
    assert float(state[:, :17].abs().max()) == 0.0 and float(state[[1, 3, 4]].abs().max()) == 0.0
    for i, x in enumerate(xs):
        ref = plain.short_convolution(x[:, :C].to(F), w.cpu().to(F))
        torch.testing.assert_close(torch.cat(outs[i]).to(F), ref, **_tol(dtype))


@DTYPES
@pytest.mark.parametrize("H, G, dk, dv", [(2, 1, 16, 24), (1, 1, 64, 64), (3, 3, 40, 8), (2, 2, 128, 72), (1, 1, 8, 130)])
def test_delta_rule_scan(dtype, H, G, dk, dv):
    """Two sequences in slots 3 and 1, fed as 37 + 1 + 5 and 2 + 20 + 1 tokens: the state is carried in the slot."""
    cuts = [[37, 1, 5], [2, 20, 1]]
    totals = [sum(c) for c in cuts]
    slots = torch.tensor([3, 1], dtype=torch.int32, device="cuda")
    state = torch.zeros(4, H * dk * dv + 5, device="cuda")
    a_log = _rand(H, seed=1, scale=0.3) - 1.0
    dt_bias = _rand(H * dk, seed=2) - 2.0
    seqs = []
    for i, n in enumerate(totals):
        qkv = _rand(n, 2 * G * dk + H * dv, seed=20 + i).to(dtype)
        beta = _rand(n, H + 2, seed=30 + i).to(dtype)
        decay = _rand(n, H * dk, seed=40 + i).to(dtype)
        seqs.append((qkv, beta, decay))
    got = [[], []]
    for part in range(3):
        pieces = []
        for (qkv, beta, decay), c in zip(seqs, cuts):
            lo = sum(c[:part])
            pieces.append((qkv[lo:lo + c[part]], beta[lo:lo + c[part]], decay[lo:lo + c[part]]))
        n = [p[0].shape[0] for p in pieces]
        cu = torch.tensor([0, n[0], n[0] + n[1]], dtype=torch.int32, device="cuda")
        out = torch.empty(sum(n), H * dv, device="cuda")
        ops.delta_rule_scan(torch.cat([p[0] for p in pieces]).cuda(), torch.cat([p[1] for p in pieces]).cuda(),
                            torch.cat([p[2] for p in pieces]).cuda(), dt_bias.cuda(), a_log.cuda(), state, slots, cu, out,
                            H, G, dk, dv, dk ** -0.5, 1e-6)
        got[0].append(out[:n[0]].cpu())
        got[1].append(out[n[0]:].cpu())
    assert float(state[[0, 2]].abs().max()) == 0.0 and float(state[:, H * dk * dv:].abs().max()) == 0.0
    for i, (qkv, beta, decay) in enumerate(seqs):
        n = totals[i]
        q = qkv[:, :G * dk].to(F).view(n, G, dk)
        k = qkv[:, G * dk:2 * G * dk].to(F).view(n, G, dk)
        v = qkv[:, 2 * G * dk:].to(F).view(n, H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        b = torch.sigmoid(beta[:, :H].to(F))
        g = torch.exp(-torch.exp(a_log.to(F))[None, :, None] *
                      torch.nn.functional.softplus((decay.to(F) + dt_bias.to(F)).view(n, H, dk)))
        ref = torch.stack([plain.delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], b[:, h], g[:, h])
                           for h in range(H)], dim=1).reshape(n, H * dv)
        torch.testing.assert_close(torch.cat(got[i]).to(F), ref, rtol=1e-4, atol=1e-5)


@DTYPES
def test_gated_rmsnorm(dtype):
    T, H, d = 6, 3, 40
    x = _rand(T, H * d, seed=1).cuda()
    w = _rand(d, seed=2).cuda()
    gate = _rand(T, H * d + 8, seed=3).to(dtype).cuda()
    out = torch.empty(T, H * d, dtype=dtype, device="cuda")
    ops.gated_rmsnorm(x, w, gate, out, H, d, 1e-5)
    ref = plain.rms_normalise(x.cpu().to(F).view(T, H, d), 1e-5) * w.cpu().to(F) * torch.sigmoid(gate[:, :H * d].cpu().to(F).view(T, H, d))
    torch.testing.assert_close(out.cpu().to(F).view(T, H, d), ref, **_tol(dtype))


@DTYPES
@pytest.mark.parametrize("T", [1, 9, 70, 300])
def test_products_per_head(dtype, T):
    H, n, k = 3, 40, 24
    a = _rand(T, H * k + 8, seed=1).to(dtype).cuda()[:, :H * k]      # rows wider than the heads: a row stride of its own
    w = _rand(H, n, k, seed=2).to(dtype).cuda()
    c = torch.empty(T, H * n, dtype=dtype, device="cuda")
    ops.gemm_per_head(a, w, c)
    ref = torch.einsum("thk,hnk->thn", a.cpu().to(F).view(T, H, k), w.cpu().to(F)).reshape(T, H * n)
    torch.testing.assert_close(c.cpu().to(F), ref, **_tol(dtype))


@pytest.mark.parametrize("streams, width, T", [(1, 48, 5), (3, 100, 7), (2, 2500, 3)])
def test_streams_step(streams, width, T):
    """Write-back, clearing of the sublayer result and the next read with its norm, in one kernel."""
    xs = _rand(T, streams, width, seed=2).cuda()
    lst = [xs[:, a].cpu().to(F) for a in range(streams)]
    W = {"h.mix": _rand(streams, streams, seed=4).to(F), "h.out": _rand(streams, seed=5).to(F)}
    read, nw = _rand(streams, seed=3), _rand(width, seed=6) * 0.3
    y = _rand(T, width, seed=7).cuda()
    ref = plain.connect(lst, W, "h.", y.cpu().to(F))
    out = torch.empty(T, width, device="cuda")
    ops.streams_step(xs, W["h.mix"].float().cuda(), W["h.out"].float().cuda(), y, read.cuda(), (1 + nw).cuda(), out, 1e-5)
    for j in range(streams):
        torch.testing.assert_close(xs[:, j].cpu().to(F), ref[j], rtol=2e-5, atol=2e-5)
    u = sum(read[a].to(F) * ref[a] for a in range(streams))
    torch.testing.assert_close(out.cpu().to(F), plain.offset_norm(u, nw.to(F), 1e-5), rtol=5e-5, atol=5e-5)
    assert float(y.abs().max()) == 0.0
    y2 = _rand(T, width, seed=8).cuda()
    ref2 = plain.connect(ref, W, "h.", y2.cpu().to(F))
    ops.streams_step(xs, W["h.mix"].float().cuda(), W["h.out"].float().cuda(), y2)       # nothing runs next
    for j in range(streams):
        torch.testing.assert_close(xs[:, j].cpu().to(F), ref2[j], rtol=5e-5, atol=5e-5)
    assert float(y2.abs().max()) == 0.0


@DTYPES
def test_head_rows_into_cache_pages(dtype):
    """Keys as rows and values transposed, each at its token's position in the page its sequence's table names."""
    T, G, dk, dv, D, n_pages = 7, 2, 24, 16, 32, 5
    src = _rand(T, G * dk + G * dv, seed=1).to(dtype).cuda()
    positions = torch.tensor([62, 63, 64, 65, 0, 1, 130], dtype=torch.int32, device="cuda")
    seq_ids = torch.tensor([0, 0, 0, 0, 1, 1, 1], dtype=torch.int32, device="cuda")
    table = torch.tensor([[3, 1, 0], [4, 0, 2]], dtype=torch.int32, device="cuda")
    k_pool = torch.full((n_pages, G, 64, D), 9.0, dtype=dtype, device="cuda")
    v_pool = torch.full((n_pages, G, D, 64), 9.0, dtype=dtype, device="cuda")
    segs = ops.head_row_segments(ops.head_row_segment(0, G, dk, 0, D, -1, True, target=ops.TO_CACHE_KEYS),
                                 ops.head_row_segment(G * dk, G, dv, 0, D, target=ops.TO_CACHE_VALUES))
    ops.head_rows(src, None, segs, 1e-6, cache=(positions, seq_ids, table, k_pool, v_pool))
    k_ref = plain.rms_normalise(src[:, :G * dk].cpu().to(F).view(T, G, dk), 1e-6)
    v_ref = src[:, G * dk:].cpu().to(F).view(T, G, dv)
    written_k = torch.zeros(n_pages, G, 64, dtype=torch.bool)
    for t in range(T):
        pos, page = int(positions[t]), int(table[int(seq_ids[t]), int(positions[t]) // 64])
        torch.testing.assert_close(k_pool[page, :, pos % 64, :dk].cpu().to(F), k_ref[t], **_tol(dtype))
        torch.testing.assert_close(v_pool[page, :, :dv, pos % 64].cpu().to(F), v_ref[t], **_tol(dtype))
        assert float(k_pool[page, :, pos % 64, dk:].abs().max()) == 0.0 and float(v_pool[page, :, dv:, pos % 64].abs().max()) == 0.0
        written_k[page, :, pos % 64] = True
    assert bool((k_pool.cpu()[~written_k] == 9.0).all())      # nothing else was touched
    assert int((v_pool.cpu() != 9.0).sum()) == T * G * D
