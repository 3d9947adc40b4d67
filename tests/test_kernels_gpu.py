"""Each CUDA kernel alone against the plain implementation, at sizes the engine's models do not use."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
F64 = torch.float64
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from llama_rs_metal_b200.kernels import ops
    return ops


def close(got, want, tol, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(want.abs().max().item(), 1e-30)
    err = (got - want).abs().max().item() / scale
    assert err <= tol, f"{what}: off by {err:.3e} of the largest value (allowed {tol:.1e})"


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


TOL = {torch.float32: 1e-5, torch.bfloat16: 1.2e-2}


# --------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(ops, dtype):
    table = rnd(301, 72, dtype=dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = ops.embed_rows(table, ids)
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), P.embedding(table.float().cpu(), ids.tolist()))


# --------------------------------------------------------------------------- norm
@pytest.mark.parametrize("hidden", [24, 100, 1000, 4104])
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                           (torch.float32, torch.bfloat16)])
def test_rms_norm(ops, hidden, wdtype, odtype):
    x = rnd(7, hidden, scale=3.0)
    w = (1 + 0.2 * rnd(hidden)).to(wdtype)
    want = P.rms_norm(x.double().cpu(), w.double().cpu(), 1e-6)
    close(ops.rms_norm(x, w, 1e-6, odtype), want, 1e-5 if odtype == torch.float32 else 5e-3, "norm")
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    close(ops.rms_norm(x, w, 1e-6, odtype, rows=rows), want[[6, 0, 3]],
          1e-5 if odtype == torch.float32 else 5e-3, "norm rows")


def test_rms_norm_folds_partial_sums_into_the_residual(ops):
    x = rnd(5, 136)
    parts = rnd(3, 5, 136, seed=4)
    w = torch.ones(136, device=DEV)
    total = x.double().cpu() + parts.double().cpu().sum(0)
    y = ops.rms_norm(x, w, 1e-5, torch.float32, partials=parts)
    close(x, total, 1e-6, "residual after fold")
    close(y, P.rms_norm(total, torch.ones(136, dtype=F64), 1e-5), 1e-5, "norm of folded")


@pytest.mark.parametrize("ranks,rows,hidden,slices", [(0, 16, 3072, 6), (0, 64, 2048, 9), (2, 3, 1032, 1),
                                                     (4, 5, 2052, 3), (8, 2, 4104, 10), (4, 7, 8192, 2)])
def test_rms_norm_with_a_row_cut_among_the_ctas_of_a_cluster(ops, ranks, rows, hidden, slices):
    """Few rows with slices to fold and a bfloat16 output: the row is cut among the CTAs of a
    cluster, which exchange their shares of the sum of squares (ranks 0: the kernel's own rule
    chooses it at these sizes). The folded residual is bit-equal to the one-CTA kernel's."""
    from llama_rs_metal_b200.kernels import library
    lib = library.load()
    x = rnd(rows, hidden, scale=2.0)
    parts = rnd(slices, rows, hidden, seed=4)
    w = rnd(hidden, dtype=torch.bfloat16, seed=9) + 1.0
    total = x.double().cpu() + parts.double().cpu().sum(0)
    want = P.rms_norm(total, w.double().cpu(), 1e-5)
    lib.lrm_set_norm_ranks(1)
    try:
        x_one = x.clone()
        y_one = ops.rms_norm(x_one, w, 1e-5, torch.bfloat16, partials=parts)
        lib.lrm_set_norm_ranks(ranks)
        x_cut = x.clone()
        y_cut = ops.rms_norm(x_cut, w, 1e-5, torch.bfloat16, partials=parts)
        picked = ops.rms_norm(x_cut, w, 1e-5, torch.bfloat16, rows=i32([rows - 1, 0]))
        # float32 output never takes the cluster: its bits must not depend on the number of rows
        y32_cut = ops.rms_norm(x.clone(), w, 1e-5, torch.float32, partials=parts)
        lib.lrm_set_norm_ranks(1)
        y32_one = ops.rms_norm(x.clone(), w, 1e-5, torch.float32, partials=parts)
    finally:
        lib.lrm_set_norm_ranks(0)
    assert torch.equal(x_cut, x_one)
    close(x_cut, total, 1e-6, "residual after fold")
    close(y_cut, want, TOL[torch.bfloat16] / 2, "norm of folded, cut among a cluster")
    close(y_one, want, TOL[torch.bfloat16] / 2, "norm of folded, one CTA per row")
    close(picked, want[[rows - 1, 0]], TOL[torch.bfloat16] / 2, "listed rows")
    assert torch.equal(y32_cut, y32_one)


# --------------------------------------------------------------------------- matrix products
SHAPES = [(1, 1, 1), (1, 130, 68), (3, 63, 15), (17, 64, 129), (65, 200, 256), (130, 7, 40), (4, 307, 68)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_float32(ops, M, N, K):
    x, w = rnd(M, K), rnd(N, K, seed=1)
    want = P.linear(x.double().cpu(), w.double().cpu())
    close(ops.linear(x, w), want, 1e-5, "gemm f32")
    resid = rnd(M, N, seed=2)
    before = resid.double().cpu()
    ops.linear(x, w, epilogue=ops.ADD, out=resid)
    close(resid, before + want, 1e-5, "gemm f32 add")


def test_linear_float32_row_does_not_depend_on_the_batch(ops):
    x, w = rnd(70, 200), rnd(150, 200, seed=1)
    full = ops.linear(x, w)
    for r in (0, 63, 64, 69):
        assert torch.equal(ops.linear(x[r:r + 1].contiguous(), w)[0], full[r])


@pytest.fixture(params=["fast kernels", "prompt attention in tensor memory", "warp-level attention",
                        "fallback kernels"])
def kernel_choice(request, monkeypatch):
    """Run a test with the kernels the dispatchers pick for short prompts, with the tcgen05 prompt
    attention that long prompts get, with prompts kept off the tcgen05 attention, and with every
    fallback forced."""
    from llama_rs_metal_b200.kernels import attention_dispatch, gemm_dispatch
    if request.param == "fast kernels":
        monkeypatch.setattr(attention_dispatch, "prefill_kernel", "single")
    if request.param == "prompt attention in tensor memory":
        monkeypatch.setattr(attention_dispatch, "prefill_kernel", "pingpong")
    if request.param == "fallback kernels":
        monkeypatch.setattr(gemm_dispatch, "force_tiled", True)
        monkeypatch.setattr(attention_dispatch, "force_rowwise", True)
    if request.param == "warp-level attention":
        monkeypatch.setattr(attention_dispatch, "force_warp_level", True)
    yield request.param
    gemm_dispatch.check_status()


@pytest.mark.parametrize("M,N,K", SHAPES + [(64, 128, 2048), (5, 48, 8), (8, 3072, 2048), (33, 40, 1160)])
def test_linear_bfloat16(ops, kernel_choice, M, N, K):
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    want = P.linear(x.double().cpu(), w.double().cpu())
    close(ops.linear(x, w), want, 6e-3, "gemm bf16 -> bf16")
    close(ops.linear(x, w, out_dtype=torch.float32), want, 2e-5 * math.sqrt(K), "gemm bf16 -> f32")
    resid = rnd(M, N, seed=2)
    before = resid.double().cpu()
    ops.linear(x, w, epilogue=ops.ADD, out=resid)
    close(resid, before + want, 2e-5 * math.sqrt(K), "gemm bf16 add")


@pytest.mark.parametrize("M,I,K", [(1, 8, 16), (5, 24, 68), (70, 136, 64), (64, 512, 256), (9, 40, 1048)])
def test_linear_bfloat16_silu_gate(ops, kernel_choice, M, I, K):
    x = rnd(M, K, dtype=torch.bfloat16)
    gate, up = rnd(I, K, dtype=torch.bfloat16, seed=1), rnd(I, K, dtype=torch.bfloat16, seed=2)
    fused = torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    xd = x.double().cpu()
    want = P.silu(P.linear(xd, gate.double().cpu())) * P.linear(xd, up.double().cpu())
    close(ops.linear(x, fused, epilogue=ops.SILU_GATE), want, 8e-3, "fused gate")
    close(ops.silu_mul(ops.linear(x, fused), 8), want, 1.5e-2, "unfused gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block", [4, 100])
def test_silu_mul_blocks(ops, dtype, block):
    I = 100
    g, u = rnd(6, I, dtype=dtype, scale=2.0), rnd(6, I, dtype=dtype, seed=3)
    gu = torch.stack([g.view(6, I // block, block), u.view(6, I // block, block)], dim=2).reshape(6, 2 * I)
    want = P.silu(g.double().cpu()) * u.double().cpu()
    close(ops.silu_mul(gu.contiguous(), block), want, TOL[dtype] / 2, "silu_mul")


def test_add_and_cast(ops):
    x, d = rnd(9, 77), rnd(9, 77, dtype=torch.bfloat16, seed=5)
    want = x.double().cpu() + d.double().cpu()
    close(ops.add_(x, d), want, 1e-6, "add_")
    y = rnd(1000, 3)
    assert torch.equal(ops.cast(y, torch.bfloat16), y.to(torch.bfloat16))
    assert torch.equal(ops.cast(y.to(torch.bfloat16), torch.float32), y.to(torch.bfloat16).float())


# --------------------------------------------------------------------------- rope + store
class View:
    def __init__(self, pages, kv_heads, page_size, d, dtype, slots=3, per_seq=6, fill=float("nan")):
        self.k = torch.full((pages, kv_heads, page_size, d), fill, dtype=dtype, device=DEV)
        self.v = torch.full((pages, kv_heads, page_size, d), fill, dtype=dtype, device=DEV)
        self.page_table = torch.full((slots, per_seq), -1, dtype=torch.int32, device=DEV)
        self.page_size, self.kv_heads, self.head_dim, self.window = page_size, kv_heads, d, None


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hk,d,R", [(4, 2, 16, 16), (3, 1, 48, 32), (5, 5, 80, 80), (2, 1, 48, 24), (32, 8, 64, 64)])
def test_rope_store(ops, dtype, Hq, Hk, d, R):
    cfg = dict(rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
               high_freq_factor=4.0, original_max_position_embeddings=64))
    inv = P.rope_inverse_frequencies(cfg, R)
    positions = [0, 1, 63, 64, 130, 4999]
    T = len(positions)
    qkv = rnd(T, (Hq + 2 * Hk) * d, dtype=dtype)
    view = View(pages=90, kv_heads=Hk, page_size=64, d=d, dtype=dtype, slots=3, per_seq=80)
    # where each token's key and value go: page * 64 + row in page
    pages = {0: (7, 0), 1: (7, 1), 2: (7, 63), 3: (3, 0), 4: (11, 2), 5: (5, 4999 % 64)}
    dest = i32([pages[t][0] * 64 + pages[t][1] for t in range(T)])
    q, k, v = ops.rope_store(qkv, Hq, Hk, d, torch.from_numpy(inv).to(DEV), R, i32(positions),
                             kv=view, dest_rows=dest)
    x = qkv.double().cpu()
    want_q = P.rope(x[:, :Hq * d].reshape(T, Hq, d), positions, inv, R)
    want_k = P.rope(x[:, Hq * d:(Hq + Hk) * d].reshape(T, Hk, d), positions, inv, R)
    want_v = x[:, (Hq + Hk) * d:].reshape(T, Hk, d)
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    close(q, want_q, tol, "q")
    close(k, want_k, tol, "k")
    assert torch.equal(v.double().cpu(), want_v)
    written = torch.zeros(90, 64, dtype=torch.bool)
    for t, (page, row) in pages.items():
        assert torch.equal(view.k[page, :, row], k[t]) and torch.equal(view.v[page, :, row], v[t])
        written[page, row] = True
    untouched = ~written
    assert torch.isnan(view.k.float().cpu().permute(0, 2, 1, 3)[untouched]).all(), "a row outside the step was written"
    assert torch.isnan(view.v.float().cpu().permute(0, 2, 1, 3)[untouched]).all()


@pytest.mark.parametrize("width", [None, 128, 192, 256, 512, "pair"])
@pytest.mark.parametrize("Hq,Hk,d,T,rotate", [(6, 2, 64, 300, True), (4, 1, 128, 200, True), (5, 5, 64, 129, False),
                                               (32, 8, 64, 700, True)])
def test_projection_with_rotation_and_stores_in_its_epilogue(ops, monkeypatch, width, Hq, Hk, d, T, rotate):
    """A prompt's q|k|v product that rotates and stores in its epilogue leaves the bits that the
    product followed by rope_store leaves: q, k, v packed and the cache rows, nothing else written.
    Every tile shape whose width is a whole number of heads, and the pairs of SMs."""
    from llama_rs_metal_b200.kernels import gemm_dispatch
    if width is not None and {128: 128, 192: 192, 256: 256, 512: 256, "pair": 256}[width] % d:
        pytest.skip("this tile is no whole number of heads")
    h = 264
    x, w = rnd(T, h, dtype=torch.bfloat16), rnd((Hq + 2 * Hk) * d, h, dtype=torch.bfloat16, seed=1, scale=0.2)
    inv = torch.from_numpy(P.rope_inverse_frequencies(dict(rope_theta=10000.0), d)).to(DEV) if rotate else None
    positions = i32([(7 * t) % 3000 for t in range(T)])
    dest = [t + 64 * 3 if t % 5 else -1 for t in range(T)]        # some tokens are not kept (a window dropped them)
    pages = (T + 64 * 3) // 64 + 2
    fused_view, plain_view = (View(pages, Hk, 64, d, torch.bfloat16) for _ in range(2))
    monkeypatch.setattr(gemm_dispatch, "umma_width", width)
    table = ops.rope_table(positions, inv) if rotate else None
    got = ops.linear_rope_store(x, w, Hq, Hk, d, table, fused_view, i32(dest))
    gemm_dispatch.check_status()
    assert got is not None, "the tensor-core product refused a shape it is built for"
    monkeypatch.setattr(gemm_dispatch, "umma_width", None)
    want = ops.rope_store(ops.linear(x, w), Hq, Hk, d, inv, d if rotate else 0, positions, kv=plain_view,
                          dest_rows=i32(dest))
    for name, a, b in zip("qkv", got, want):
        assert torch.equal(a, b), f"{name} differs from the separate kernels'"
    for a, b in ((fused_view.k, plain_view.k), (fused_view.v, plain_view.v)):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), "the cache differs (NaN = never written)"
    if rotate:   # and the table holds the angles of the plain implementation
        angles = positions.double().cpu()[:, None] * inv.double().cpu()[None, :]
        close(table[..., 0], torch.cos(angles), 2e-3, "cosines")   # float32 angle of positions up to 3,000
        close(table[..., 1], torch.sin(angles), 2e-3, "sines")


def test_rope_store_skips_pages_a_window_dropped_and_can_leave_q_unrotated(ops):
    view = View(pages=4, kv_heads=1, page_size=64, d=16, dtype=torch.float32)
    qkv = rnd(2, 3 * 16)
    q, k, v = ops.rope_store(qkv, 1, 1, 16, None, 0, i32([10, 70]), kv=view, dest_rows=i32([-1, -1]))
    assert torch.isnan(view.k).all()                      # neither position is kept: nothing stored
    assert torch.equal(q.view(2, 16), qkv[:, :16]) and torch.equal(k.view(2, 16), qkv[:, 16:32])


# --------------------------------------------------------------------------- attention
def packed_case(lengths, Hq, Hk, d, dtype, seed=0):
    T = sum(lengths)
    q, k, v = rnd(T, Hq, d, dtype=dtype, seed=seed), rnd(T, Hk, d, dtype=dtype, seed=seed + 1), \
        rnd(T, Hk, d, dtype=dtype, seed=seed + 2)
    cu = np.concatenate([[0], np.cumsum(lengths)])
    seq_of = np.repeat(np.arange(len(lengths)), lengths)
    return q, k, v, cu, seq_of


def plain_packed(q, k, v, cu, window=None):
    out = []
    for a, b in zip(cu[:-1], cu[1:]):
        out.append(P.attention(q[a:b].double().cpu(), k[a:b].double().cpu(), v[a:b].double().cpu(), window))
    return torch.cat(out).reshape(q.shape[0], -1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hk,d", [(4, 2, 16), (3, 1, 48), (6, 6, 80), (8, 2, 128), (3, 1, 32), (10, 5, 64)])
@pytest.mark.parametrize("window", [None, 5, 64, 200])
def test_attention_prefill(ops, kernel_choice, dtype, Hq, Hk, d, window):
    lengths = [1, 9, 70, 33, 130, 400, 128, 257]
    q, k, v, cu, seq_of = packed_case(lengths, Hq, Hk, d, dtype)
    got = ops.attention_prefill(q, k, v, i32(cu), i32(seq_of), max(lengths), d ** -0.5, window)
    close(got, plain_packed(q, k, v, cu, window), TOL[dtype], f"prefill window {window}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [32, 64])
def test_attention_prefill_finds_one_far_key_among_hundreds(ops, kernel_choice, dtype, d):
    # One key far back is scaled so that its score stands out: the output must be its value.
    lengths = [300, 257]
    q, k, v, cu, seq_of = packed_case(lengths, 4, 2, d, dtype, seed=9)
    far = {0: 3, 1: 300 + 64}                 # packed index of the far key of each sequence
    for s, idx in far.items():
        k[idx] = 0
        k[idx, :, 0] = 40.0
    q[cu[1] - 1, :, :] = 0
    q[cu[1] - 1, :, 0] = 40.0                 # last query of sequence 0
    q[cu[2] - 1, :, :] = 0
    q[cu[2] - 1, :, 0] = 40.0
    got = ops.attention_prefill(q, k, v, i32(cu), i32(seq_of), 300, d ** -0.5).view(-1, 4, d)
    close(got, plain_packed(q, k, v, cu).view(-1, 4, d), TOL[dtype], "far key")
    for s, idx in far.items():
        last = cu[s + 1] - 1
        for h in range(4):
            close(got[last, h], v[idx, h // 2].double(), 2e-2 if dtype == torch.bfloat16 else 1e-4, "value of the far key")


def paged_case(ops, lengths, Hq, Hk, d, dtype, page_size=64, poison=1e4, seed=0):
    """Sequences in shuffled slots and pages; every row no sequence owns is poisoned."""
    B = len(lengths)
    slots = [5, 0, 3, 1, 4, 2][:B]
    per_seq = max(-(-n // page_size) for n in lengths) + 1
    n_pages = sum(-(-n // page_size) for n in lengths) + 3
    view = View(n_pages, Hk, page_size, d, dtype, slots=6, per_seq=per_seq, fill=poison)
    order = list(np.random.default_rng(seed).permutation(n_pages))
    table = view.page_table.cpu()
    ks, vs = [], []
    for b, n in enumerate(lengths):
        kb, vb = rnd(n, Hk, d, dtype=dtype, seed=seed + 10 + b), rnd(n, Hk, d, dtype=dtype, seed=seed + 20 + b)
        ks.append(kb)
        vs.append(vb)
        for p in range(-(-n // page_size)):
            page = int(order.pop())
            table[slots[b], p] = page
            rows = min(page_size, n - p * page_size)
            view.k[page, :, :rows] = kb[p * page_size:p * page_size + rows].transpose(0, 1)
            view.v[page, :, :rows] = vb[p * page_size:p * page_size + rows].transpose(0, 1)
    view.page_table.copy_(table)
    q = rnd(B, Hq, d, dtype=dtype, seed=seed + 5)
    return q, view, slots, ks, vs


def plain_decode(q, ks, vs, window=None):
    out = []
    for b, (kb, vb) in enumerate(zip(ks, vs)):
        n = kb.shape[0]
        qq = torch.zeros(n, q.shape[1], q.shape[2], dtype=F64)
        qq[-1] = q[b].double().cpu()
        out.append(P.attention(qq, kb.double().cpu(), vb.double().cpu(), window)[-1].reshape(-1))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hk,d", [(4, 2, 16), (3, 1, 48), (8, 2, 128), (32, 8, 64), (3, 1, 32), (40, 2, 64)])
@pytest.mark.parametrize("window", [None, 64, 100])
def test_attention_decode_over_poisoned_pages(ops, kernel_choice, dtype, Hq, Hk, d, window):
    lengths = [1, 64, 65, 300, 129, 1000]
    q, view, slots, ks, vs = paged_case(ops, lengths, Hq, Hk, d, dtype)
    got = ops.attention_decode(q, view, i32(slots), i32(lengths), max(lengths), d ** -0.5, window)
    close(got, plain_decode(q, ks, vs, window), TOL[dtype], f"decode window {window}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_decode_window_edge(ops, kernel_choice, dtype):
    # The key just outside the window would win every score; the key just inside must still count.
    lengths, window = [200, 131], 64
    q, view, slots, ks, vs = paged_case(ops, lengths, 4, 2, 32, dtype, seed=3)
    table = view.page_table.cpu()
    for b, n in enumerate(lengths):
        q[b] = 0
        q[b, :, 1] = 30.0
        for pos, strength in ((n - window - 1, 60.0), (n - window, 30.0)):
            ks[b][pos] = 0
            ks[b][pos, :, 1] = strength
            page = int(table[slots[b], pos // 64])
            view.k[page, :, pos % 64] = ks[b][pos]
    got = ops.attention_decode(q, view, i32(slots), i32(lengths), max(lengths), 32 ** -0.5, window).view(2, 4, 32)
    close(got, plain_decode(q, ks, vs, window).view(2, 4, 32), TOL[dtype], "window edge")
    for b, n in enumerate(lengths):
        close(got[b, 0], vs[b][n - window, 0].double(), 2e-2, "the key at the window's edge")
    # rows before the window may never have been written (a prompt longer than the window stores
    # only its tail): whatever they hold, even NaN, must not reach the result
    for b, n in enumerate(lengths):
        for pos in range(n - window):
            page = int(table[slots[b], pos // 64])
            view.k[page, :, pos % 64] = float("nan")
            view.v[page, :, pos % 64] = float("nan")
    again = ops.attention_decode(q, view, i32(slots), i32(lengths), max(lengths), 32 ** -0.5, window).view(2, 4, 32)
    assert torch.equal(again, got)


def extend_case(ops, lengths, portions, Hq, Hk, d, dtype, seed=0):
    """Sequences in the paged cache, whose last `portions[b]` tokens are the step's packed queries."""
    _, view, slots, ks, vs = paged_case(ops, lengths, Hq, Hk, d, dtype, seed=seed)
    T = sum(portions)
    q = rnd(T, Hq, d, dtype=dtype, seed=seed + 77)
    cu = [0]
    for n in portions:
        cu.append(cu[-1] + n)
    seq_of = [b for b, n in enumerate(portions) for _ in range(n)]
    positions = [lengths[b] - portions[b] + i for b in range(len(lengths)) for i in range(portions[b])]
    return q, view, slots, ks, vs, cu, seq_of, positions


def plain_extend(q, ks, vs, cu, lengths, portions, window=None):
    out = []
    for b, (kb, vb) in enumerate(zip(ks, vs)):
        n, m = lengths[b], portions[b]
        qq = torch.zeros(n, q.shape[1], q.shape[2], dtype=F64)
        qq[n - m:] = q[cu[b]:cu[b + 1]].double().cpu()
        out.append(P.attention(qq, kb.double().cpu(), vb.double().cpu(), window)[n - m:].reshape(m, -1))
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hk,d", [(4, 2, 16), (3, 1, 48), (8, 2, 128), (32, 8, 64), (3, 1, 32)])
@pytest.mark.parametrize("window", [None, 64, 100])
def test_attention_extend_over_poisoned_pages(ops, kernel_choice, dtype, Hq, Hk, d, window):
    """Portions of 1, 2, 63, 64, 65 and 130 tokens onto sequences that cross page edges before,
    inside and after the portion; one sequence is its portion (nothing cached before)."""
    lengths = [64, 66, 300, 129, 65, 1000]
    portions = [1, 2, 63, 64, 65, 130]
    q, view, slots, ks, vs, cu, seq_of, positions = extend_case(ops, lengths, portions, Hq, Hk, d, dtype)
    got = ops.attention_extend(q, view, i32(cu), i32(seq_of), i32(positions), i32(slots), i32(lengths),
                               max(portions), d ** -0.5, window)
    close(got, plain_extend(q, ks, vs, cu, lengths, portions, window), TOL[dtype], f"extend window {window}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_extend_window_edge_inside_a_portion(ops, kernel_choice, dtype):
    """Within one portion the window moves: for the portion's first query the key just outside
    its window would win every score, for a later query another one; the keys just inside must
    still count, and each query must see exactly its own window."""
    lengths, portions, window = [200, 140], [70, 100], 64
    q, view, slots, ks, vs, cu, seq_of, positions = extend_case(ops, lengths, portions, 4, 2, 32, dtype, seed=3)
    table = view.page_table.cpu()
    probes = []
    for b, (n, m) in enumerate(zip(lengths, portions)):
        for row in (0, m // 2, m - 1):                       # three queries of the portion
            pos = n - m + row
            q[cu[b] + row] = 0
            q[cu[b] + row, :, 1 + len(probes) % 3] = 30.0
            for key, strength in ((pos - window, 60.0), (pos - window + 1, 30.0)):
                if key < 0:
                    continue
                ks[b][key] = 0
                ks[b][key, :, 1 + len(probes) % 3] = strength
                view.k[int(table[slots[b], key // 64]), :, key % 64] = ks[b][key]
            probes.append((b, row, pos))
    got = ops.attention_extend(q, view, i32(cu), i32(seq_of), i32(positions), i32(slots), i32(lengths),
                               max(portions), 32 ** -0.5, window)
    close(got, plain_extend(q, ks, vs, cu, lengths, portions, window), TOL[dtype], "window edge inside a portion")
    for b, row, pos in probes:
        if pos - window + 1 >= 0:
            close(got[cu[b] + row].view(4, 32)[0], vs[b][pos - window + 1, 0].double(), 3e-2,
                  "the key at the window's edge")


def test_float32_extend_equals_prefill_bit_for_bit(ops):
    """In float32 a prompt's last tokens, run as a portion over the cache, get the bits the whole
    prompt gets: same keys in the same order, same arithmetic."""
    lengths, portions = [70, 5, 129], [17, 5, 66]
    q, view, slots, ks, vs, cu, seq_of, positions = extend_case(ops, lengths, portions, 4, 2, 16, torch.float32, seed=7)
    ext = ops.attention_extend(q, view, i32(cu), i32(seq_of), i32(positions), i32(slots), i32(lengths),
                               max(portions), 0.25)
    for b, (n, m) in enumerate(zip(lengths, portions)):
        qq = rnd(n, 4, 16, seed=99)
        qq[n - m:] = q[cu[b]:cu[b + 1]]
        pre = ops.attention_prefill(qq, ks[b].contiguous(), vs[b].contiguous(), i32([0, n]), i32([0] * n), n, 0.25)
        assert torch.equal(pre[n - m:], ext[cu[b]:cu[b + 1]])


def test_float32_decode_equals_prefill_bit_for_bit(ops):
    lengths = [70, 5, 129]
    q, view, slots, ks, vs = paged_case(ops, lengths, 4, 2, 16, torch.float32, seed=7)
    dec = ops.attention_decode(q, view, i32(slots), i32(lengths), max(lengths), 0.25)
    for b, n in enumerate(lengths):
        qq = rnd(n, 4, 16, seed=99)
        qq[-1] = q[b]
        pre = ops.attention_prefill(qq, ks[b].contiguous(), vs[b].contiguous(), i32([0, n]),
                                    i32([0] * n), n, 0.25)
        assert torch.equal(pre[-1], dec[b])


@pytest.mark.parametrize("cluster", [None, 1, 2, 7, 8, 16])
@pytest.mark.parametrize("Hq,Hk,d,rotary", [(32, 8, 64, 64), (8, 2, 128, 128), (3, 1, 32, 32), (40, 2, 64, 32),
                                             (6, 3, 128, 64), (6, 3, 128, 96), (4, 4, 64, 0)])
def test_attention_decode_fused_rotates_stores_attends_and_merges(ops, Hq, Hk, d, rotary, cluster):
    """The one-launch decode attention against the plain rotation and attention, and against the
    separate kernels: the new key/value row it leaves in the cache is bit-equal to rope_store's.
    Sequences shorter than the cluster (CTAs without a page), page edges, poisoned free rows."""
    from llama_rs_metal_b200.kernels import attention_dispatch
    dtype = torch.bfloat16
    lengths = [1, 64, 65, 300, 129, 1000]
    B = len(lengths)
    _, view, slots, ks, vs = paged_case(ops, lengths, Hq, Hk, d, dtype, seed=11)
    qkv = rnd(B, (Hq + 2 * Hk) * d, dtype=dtype, seed=77)
    inv = (1.0 / (10000.0 ** (torch.arange(0, rotary, 2, dtype=torch.float64) / max(rotary, 1)))).float() if rotary else None
    positions = [n - 1 for n in lengths]
    table = view.page_table.cpu()
    dest = [int(table[slots[b], (n - 1) // 64]) * 64 + (n - 1) % 64 for b, n in enumerate(lengths)]
    for b, n in enumerate(lengths):                    # the new row is not in the cache yet
        view.k[dest[b] // 64, :, dest[b] % 64] = float("nan")
        view.v[dest[b] // 64, :, dest[b] % 64] = float("nan")
    # what the separate kernels do with the same input, in a copy of the cache
    twin = View(view.k.shape[0], Hk, 64, d, dtype, slots=6, per_seq=view.page_table.shape[1])
    twin.k.copy_(view.k), twin.v.copy_(view.v), twin.page_table.copy_(view.page_table)
    inv_dev = inv.to(DEV) if inv is not None else None
    q_rot, _, _ = ops.rope_store(qkv, Hq, Hk, d, inv_dev, rotary, i32(positions), kv=twin, dest_rows=i32(dest),
                                 keep_packed=False)
    want_unfused = ops.attention_decode(q_rot, twin, i32(slots), i32(lengths), max(lengths), d ** -0.5)
    attention_dispatch.force_cluster_size = cluster
    try:
        got = ops.attention_decode_fused(qkv, Hq, inv_dev, rotary, i32(positions), view, i32(dest), i32(slots),
                                         i32(lengths), max(lengths), d ** -0.5)
    finally:
        attention_dispatch.force_cluster_size = None
    # handing the sequences out longest first changes who starts when, not what anyone computes
    order = i32(sorted(range(B), key=lambda b: (-lengths[b], b)))
    attention_dispatch.force_cluster_size = cluster
    try:
        again = ops.attention_decode_fused(qkv, Hq, inv_dev, rotary, i32(positions), view, i32(dest), i32(slots),
                                           i32(lengths), max(lengths), d ** -0.5, order)
    finally:
        attention_dispatch.force_cluster_size = None
    assert torch.equal(got, again), "the order of the sequences changed a result"
    assert torch.equal(view.k.view(torch.int16), twin.k.view(torch.int16)), "the cache's keys differ from rope_store's"
    assert torch.equal(view.v.view(torch.int16), twin.v.view(torch.int16))
    # against the plain implementation: rotate in float64, round as the cache does
    x = qkv.double().cpu().view(B, Hq + 2 * Hk, d)
    for b, n in enumerate(lengths):
        heads = x[b:b + 1, :Hq + Hk]
        rotated = P.rope(heads, [n - 1], inv.numpy(), rotary) if rotary else heads
        ks[b][n - 1] = rotated[0, Hq:].to(dtype)
        vs[b][n - 1] = x[b, Hq + Hk:].to(dtype)
        x[b, :Hq] = rotated[0, :Hq].to(dtype).double()
    want = plain_decode(x[:, :Hq], ks, vs)
    close(got, want, TOL[dtype], "fused decode attention")
    close(got, want_unfused.double().cpu(), TOL[dtype], "fused against separate kernels")


def test_attention_decode_fused_far_key_and_new_key(ops):
    """One old key far back, or the new key itself, must carry the whole output."""
    dtype, Hq, Hk, d = torch.bfloat16, 8, 2, 64
    lengths = [900, 513]
    _, view, slots, ks, vs = paged_case(ops, lengths, Hq, Hk, d, dtype, seed=5)
    table = view.page_table.cpu()
    dest = [int(table[slots[b], (n - 1) // 64]) * 64 + (n - 1) % 64 for b, n in enumerate(lengths)]
    qkv = torch.zeros(2, (Hq + 2 * Hk) * d, dtype=dtype, device=DEV)
    x = qkv.view(2, Hq + 2 * Hk, d)
    x[:, :Hq, 3] = 40.0                                  # every query looks along dimension 3
    x[:, Hq + Hk:] = rnd(2, Hk, d, dtype=dtype, seed=9)  # the new values
    x[1, Hq:Hq + Hk, 3] = 40.0                           # sequence 1: its new key wins
    far = 70                                             # sequence 0: the key at position 70 wins
    ks[0][far] = 0
    ks[0][far, :, 3] = 40.0
    view.k[int(table[slots[0], far // 64]), :, far % 64] = ks[0][far]
    got = ops.attention_decode_fused(qkv, Hq, None, 0, i32([n - 1 for n in lengths]), view, i32(dest), i32(slots),
                                     i32(lengths), max(lengths), d ** -0.5).view(2, Hq, d)
    for h in range(Hq):
        close(got[0, h], vs[0][far, h // 4].double(), 2e-2, "the far key's value")
        close(got[1, h], x[1, Hq + Hk + h // 4].double().cpu(), 2e-2, "the new key's value")


# --------------------------------------------------------------------------- sampling
def test_argmax_rows_ties_and_non_finite(ops):
    logits = rnd(5, 5003)
    logits[0, 4000] = logits[0, 17] = 50.0        # tie: lowest id wins
    logits[1, 5002] = 60.0
    logits[2, 100] = float("nan")
    logits[3, 7] = float("inf")
    got = ops.argmax_rows(logits).tolist()
    assert got[:2] == [17, 5002] and got[2] == -1 and got[3] == -1
    assert got[4] == P.argmax_lowest(logits[4].cpu())
    small = torch.tensor([[1.0, 3.0, 3.0]], device=DEV)
    assert ops.argmax_rows(small).tolist() == [1]


from helpers import gumbel_twin  # noqa: E402  (the kernel's draw restated on the CPU)


@pytest.mark.parametrize("M", [1, 5, 8, 12])
@pytest.mark.parametrize("N,K", [(5003, 72), (40, 520), (128256, 64)])
def test_head_product_that_chooses_in_its_epilogue(ops, M, N, K):
    """The head product that leaves only the chosen token: equal to the choice over the logits the
    same product writes, for the greedy rule (ties to the lowest id, whether the tied ids share a
    16-row tile or not; -1 for a row with a non-finite logit) and for temperature sampling."""
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    w[N - 1] = w[3]                       # a tie across tiles ...
    w[20] = w[17]                         # ... and one inside a tile
    x[0] = 0
    x[0, :8] = 4.0
    w[3, :8] = w[N - 1, :8] = 8.0         # row 0: ids 3 and N - 1 tie for the largest logit
    if M > 2:
        x[2] = 0
        x[2, 8:16] = 4.0
        w[17, 8:16] = w[20, 8:16] = 8.0   # row 2: ids 17 and 20 tie
    logits = ops.linear(x, w, out_dtype=torch.float32)
    got = ops.linear_pick(x, w)
    assert got is not None and got.dtype == torch.int32
    assert got.tolist() == ops.argmax_rows(logits).tolist()
    assert got[0].item() == 3 and (M <= 2 or got[2].item() == 17)
    for r in range(M):
        assert got[r].item() == P.argmax_lowest(logits[r].cpu())
    keys = torch.tensor([(r << 32) | 5 for r in range(M)], dtype=torch.int64, device=DEV)
    drawn = ops.linear_pick(x, w, temperature=0.8, seed=9, keys=keys)
    assert drawn.tolist() == ops.sample_gumbel_rows(logits, 0.8, 9, keys).tolist()
    if M > 1:
        bad = w.clone()
        bad[N // 2, 0] = float("inf")
        x2 = x.clone()
        x2[1, 0] = 1.0                    # row 1 meets the infinite weight; a row with x = 0 there gives nan
        out = ops.linear_pick(x2, bad).tolist()
        assert out[1] == -1
    assert ops.linear_pick(x.float(), w.float()) is None          # no such kernel in float32: the caller picks from logits
    wide = rnd(13, K, dtype=torch.bfloat16)
    assert ops.linear_pick(wide, w) is None                        # more rows go to the tensor-core product, which writes logits
    assert ops.linear_pick(x, w).tolist() == got.tolist()          # the shared scratch was left clean


def test_gumbel_sampling_matches_its_cpu_twin_and_ignores_batch_company(ops):
    logits = rnd(6, 333, scale=2.0)
    keys = torch.tensor([(r << 32) | 3 for r in range(6)], dtype=torch.int64, device=DEV)
    got = ops.sample_gumbel_rows(logits, 0.8, 9, keys).tolist()
    for r in range(6):
        scores = gumbel_twin(logits[r].cpu().tolist(), 0.8, 9, (r << 32) | 3)
        best = max(scores)
        assert scores[got[r]] >= best - 1e-4       # the same draw, up to float32 rounding of a near tie
    alone = ops.sample_gumbel_rows(logits[4:5].contiguous(), 0.8, 9, keys[4:5].contiguous()).tolist()
    assert alone[0] == got[4]


def test_gumbel_sampling_follows_the_distribution(ops):
    probs = torch.tensor([0.5, 0.25, 0.125, 0.125])
    n = 20000
    logits = (probs.log() * 0.7).repeat(n, 1).contiguous().to(DEV)       # temperature 0.7 undoes the 0.7
    keys = torch.arange(n, dtype=torch.int64, device=DEV)
    counts = torch.bincount(ops.sample_gumbel_rows(logits, 0.7, 1, keys).long().cpu(), minlength=4) / n
    assert torch.allclose(counts, probs, atol=0.015)


def test_decode_attention_never_lets_stale_nan_rows_through(ops):
    # Rows of a page beyond a sequence's length may hold anything, NaN bit patterns included.
    lengths = [70, 3, 129]
    q, view, slots, ks, vs = paged_case(ops, lengths, 8, 2, 64, torch.bfloat16, poison=float("nan"), seed=11)
    got = ops.attention_decode(q, view, i32(slots), i32(lengths), max(lengths), 0.125)
    close(got, plain_decode(q, ks, vs), TOL[torch.bfloat16], "decode over NaN-poisoned pages")


@pytest.mark.parametrize("lengths", [[4096], [1, 2, 3, 4, 5, 6], [700] * 6])
def test_decode_attention_split_counts(ops, lengths):
    q, view, slots, ks, vs = paged_case(ops, lengths, 8, 2, 64, torch.bfloat16, seed=13)
    for bucket in (max(lengths), 8192):     # the launch may be sized for longer sequences than are live
        got = ops.attention_decode(q, view, i32(slots), i32(lengths), bucket, 0.125)
        close(got, plain_decode(q, ks, vs), TOL[torch.bfloat16], f"bucket {bucket}")


# --------------------------------------------------------------------------- TMA + tcgen05 product
UMMA_SHAPES = [(65, 128, 64), (128, 128, 128), (129, 72, 8), (200, 300, 72), (333, 520, 1000),
               (2048, 512, 256), (70, 16, 2048), (256, 1100, 136), (700, 40000, 72)]


@pytest.mark.parametrize("width", [128, 192, 256, 512, "pair"])
@pytest.mark.parametrize("M,N,K", UMMA_SHAPES + [(1000, 1100, 520)])
def test_linear_bfloat16_tensor_core_tiles(ops, monkeypatch, width, M, N, K):
    from llama_rs_metal_b200.kernels import gemm_dispatch
    monkeypatch.setattr(gemm_dispatch, "umma_width", width)
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    want = P.linear(x.double().cpu(), w.double().cpu())
    close(ops.linear(x, w), want, 6e-3, "umma -> bf16")
    close(ops.linear(x, w, out_dtype=torch.float32), want, 2e-5 * math.sqrt(K), "umma -> f32")
    resid = rnd(M, N, seed=2)
    before = resid.double().cpu()
    ops.linear(x, w, epilogue=ops.ADD, out=resid)
    close(resid, before + want, 2e-5 * math.sqrt(K), "umma add")
    gemm_dispatch.check_status()


@pytest.mark.parametrize("width", [128, 192, 256, 512, "pair"])
@pytest.mark.parametrize("M,I,K", [(70, 136, 64), (300, 520, 200), (128, 8, 16), (513, 20000, 64)])
def test_linear_bfloat16_tensor_core_silu_gate(ops, monkeypatch, width, M, I, K):
    from llama_rs_metal_b200.kernels import gemm_dispatch
    monkeypatch.setattr(gemm_dispatch, "umma_width", width)
    x = rnd(M, K, dtype=torch.bfloat16)
    gate, up = rnd(I, K, dtype=torch.bfloat16, seed=1), rnd(I, K, dtype=torch.bfloat16, seed=2)
    fused = torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    xd = x.double().cpu()
    want = P.silu(P.linear(xd, gate.double().cpu())) * P.linear(xd, up.double().cpu())
    close(ops.linear(x, fused, epilogue=ops.SILU_GATE), want, 8e-3, "umma fused gate")
    gemm_dispatch.check_status()


def test_tensor_core_result_does_not_depend_on_the_rows_around_it(ops):
    x, w = rnd(300, 520, dtype=torch.bfloat16), rnd(200, 520, dtype=torch.bfloat16, seed=1)
    full = ops.linear(x, w, out_dtype=torch.float32)
    part = ops.linear(x[100:230].contiguous(), w, out_dtype=torch.float32)
    assert torch.equal(part, full[100:230])


@pytest.mark.parametrize("M", [17, 40, 64])
def test_linear_bfloat16_few_rows_on_the_tensor_cores_and_on_the_streaming_kernel(ops, monkeypatch, M):
    """17 to 64 rows: wide products and split-K adds run on tcgen05, the rest streams; both must agree."""
    from llama_rs_metal_b200.kernels import gemm_dispatch
    x = rnd(M, 520, dtype=torch.bfloat16)
    wide_w, small_w = rnd(128 * 80, 520, dtype=torch.bfloat16, seed=1), rnd(300, 520, dtype=torch.bfloat16, seed=2)
    xd = x.double().cpu()
    for forced in (False, True):
        monkeypatch.setattr(gemm_dispatch, "force_stream", forced)
        close(ops.linear(x, wide_w), P.linear(xd, wide_w.double().cpu()), 6e-3, f"wide, stream={forced}")
        resid = rnd(M, 300, seed=3)
        want = resid.double().cpu() + P.linear(xd, small_w.double().cpu())
        ops.linear(x, small_w, epilogue=ops.ADD, out=resid)
        close(resid, want, 2e-5 * math.sqrt(520), f"add in place, stream={forced}")
    gemm_dispatch.check_status()


@pytest.mark.parametrize("M,N,K", [(1, 300, 8192), (8, 2048, 8192), (8, 2048, 2048), (17, 300, 8192), (40, 2048, 8192),
                                   (64, 520, 4104), (5, 64, 64), (128, 2048, 8192), (200, 520, 2048), (300, 300, 1000),
                                   (512, 2048, 8192), (700, 1000, 4104)])
def test_linear_slices_sum_to_the_product_in_a_fixed_order(ops, M, N, K):
    """A narrow product for the residual stream is cut into K slices stored as planes; whoever
    reads the stream next adds them in plane order (here the standalone kernel and the norm's
    fold). No atomics: two runs give the same bits."""
    from llama_rs_metal_b200.kernels import gemm_dispatch
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    want = P.linear(x.double().cpu(), w.double().cpu())
    planes = ops.linear_slices(x, w)
    if (M, N, K) in ((5, 64, 64), (8, 2048, 2048)):
        assert planes is None                     # too short to be worth cutting: added in place
        return
    assert planes is not None and planes.shape[0] >= 2 and tuple(planes.shape[1:]) == (M, N)
    close(planes.double().sum(0), want, 2e-5 * math.sqrt(K), "sum of the slices")
    again = ops.linear_slices(x, w)
    assert torch.equal(planes, again)
    resid = rnd(M, N, seed=2)
    folded = resid.clone()
    ops.add_planes_(resid, planes)
    close(resid, folded.double().cpu() + want, 2e-5 * math.sqrt(K), "slices added to the stream")
    weight = torch.ones(N, device=DEV)
    y = ops.rms_norm(folded, weight, 1e-5, torch.float32, partials=planes)
    assert torch.equal(folded, resid)             # the norm adds them in the same order
    close(y, P.rms_norm(resid.double().cpu(), torch.ones(N, dtype=F64), 1e-5), 1e-5, "norm of the folded stream")
    gemm_dispatch.check_status()
