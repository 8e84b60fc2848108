"""Each kernel alone against a plain PyTorch 32-bit statement of the same
operation, at sizes other than the engine's (odd widths, head sizes in steps
of 16, vocabularies that are no power of two)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.fixture(params=["copies", "tma"])
def decode_tiles(request):
    """Both ways the tensor-core decode attention brings its key / value tiles (TMA wherever
    the sizes allow it); afterwards no bounded wait of the TMA form may have given up."""
    from agave_b200 import kernels
    before = kernels.attention_decode_tiles(request.param)
    yield request.param
    kernels.attention_decode_tiles(before)
    assert kernels.attention_decode_status() == 0


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


# ------------------------------------------------------------------- products
@pytest.mark.parametrize("T,N,K", [(1, 96, 64), (5, 200, 96), (16, 128, 1152), (33, 384, 224),
                                   (64, 1000, 136), (130, 260, 72), (300, 520, 264)])
def test_linear_tensor_cores_plain(T, N, K):
    from agave_b200 import kernels
    x, w = rnd(T, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    ref = x.float() @ w.float().T
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
        kernels.linear_tc(x, w, out)
        assert kernels.linear_tc_status() == 0
        tol = 1e-5 if out_dtype == torch.float32 else 5e-3
        assert rel_err(out, ref) < tol, (T, N, K, out_dtype)


@pytest.mark.parametrize("T,N,K,splits", [(2048, 1536, 1152, 1), (2048, 1152, 1024, 1),
                                          (2000, 1152, 2304, 2), (1999, 8192, 256, 1),
                                          (700, 200, 320, 1), (3000, 2560, 192, 1)])
def test_linear_tensor_cores_prompts_every_token_tile_choice(T, N, K, splits):
    """The persistent kernel picks token tiles of 256, 192 or 128 from the shape: sizes
    that take each, token counts that end inside a tile, and K in two halves."""
    from agave_b200 import kernels
    x, w = rnd(T, K, dtype=torch.bfloat16, seed=21), rnd(N, K, dtype=torch.bfloat16, seed=22)
    ref = x.float() @ w.float().T
    s_real = kernels.linear_tc_splits(K, splits)
    out = torch.full((s_real, T, N) if s_real > 1 else (T, N), float("nan"), dtype=torch.float32,
                     device=DEV)
    kernels.linear_tc(x, w, out, splits=splits)
    assert kernels.linear_tc_status() == 0
    got = out.sum(0) if s_real > 1 else out
    assert torch.isfinite(got).all()
    assert rel_err(got, ref) < 1e-5
    wu = rnd(N, K, dtype=torch.bfloat16, seed=23, scale=0.3)
    if splits == 1 and N <= 2560:
        ob = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.linear_tc(x, w, ob, w2=wu, activation="gelu_tanh")
        g, u = ref, x.float() @ wu.float().T
        assert rel_err(ob, torch.nn.functional.gelu(g, approximate="tanh") * u) < 6e-3


@pytest.mark.parametrize("tile", [16, 32, 64, 128, 256])
def test_linear_tensor_cores_every_token_tile(tile):
    from agave_b200 import kernels
    T, N, K = 70, 300, 200
    x, w = rnd(T, K, dtype=torch.bfloat16, seed=3), rnd(N, K, dtype=torch.bfloat16, seed=4)
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.linear_tc(x, w, out, token_tile=tile)
    assert kernels.linear_tc_status() == 0
    assert rel_err(out, x.float() @ w.float().T) < 1e-5


def test_linear_tensor_cores_row_strided_input_and_output():
    from agave_b200 import kernels
    T, N, K = 9, 160, 128
    big = rnd(T, K + 64, dtype=torch.bfloat16, seed=5)
    x = big[:, 32:32 + K]            # row stride K + 64, first element 64 bytes in
    w = rnd(N, K, dtype=torch.bfloat16, seed=6)
    outbig = torch.zeros((T, N + 24), dtype=torch.bfloat16, device=DEV)
    kernels.linear_tc(x, w, outbig[:, :N])
    assert kernels.linear_tc_status() == 0
    assert rel_err(outbig[:, :N], x.float() @ w.float().T) < 5e-3
    assert (outbig[:, N:] == 0).all()


@pytest.mark.parametrize("T,N,K,act", [(3, 224, 96, "gelu_tanh"), (40, 130, 320, "silu"),
                                       (150, 256, 64, "gelu_tanh"), (256, 128, 64, "gelu_tanh"),
                                       (600, 390, 448, "silu"), (2049, 1000, 1152, "gelu_tanh"),
                                       (9, 19230, 448, "gelu_tanh")])
def test_linear_tensor_cores_gated(T, N, K, act):
    """From 256 tokens on, the gated product runs on pairs of CTAs (cta_group::2): one
    pair and one k-block, token and feature counts that end inside a tile, many rounds.
    A few tokens over a weight with between two and three tiles per SM run with three
    CTAs to the SM and a ring of three stages (more k-blocks than stages)."""
    from agave_b200 import kernels
    x = rnd(T, K, dtype=torch.bfloat16, seed=7)
    wg, wu = rnd(N, K, dtype=torch.bfloat16, seed=8, scale=0.3), rnd(N, K, dtype=torch.bfloat16, seed=9, scale=0.3)
    g, u = x.float() @ wg.float().T, x.float() @ wu.float().T
    a = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" \
        else torch.nn.functional.silu(g)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.linear_tc(x, wg, out, w2=wu, activation=act)
    assert kernels.linear_tc_status() == 0
    assert rel_err(out, a * u) < 6e-3
    if T <= 64:
        for c in (2, 4):                      # K over a cluster, the activation after the sum
            out2 = torch.full_like(out, float("nan"))
            kernels.linear_tc(x, wg, out2, w2=wu, activation=act, splits=c, cluster=c)
            assert kernels.linear_tc_status() == 0
            assert rel_err(out2, a * u) < 6e-3


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_linear_tensor_cores_partial_sums(splits):
    from agave_b200 import kernels
    T, N, K = 6, 200, 6912 // 4
    x, w = rnd(T, K, dtype=torch.bfloat16, seed=10), rnd(N, K, dtype=torch.bfloat16, seed=11)
    s = kernels.linear_tc_splits(K, splits)
    out = torch.full((s, T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.linear_tc(x, w, out, splits=splits)
    assert kernels.linear_tc_status() == 0
    assert rel_err(out.sum(0), x.float() @ w.float().T) < 1e-5


@pytest.mark.parametrize("splits", [2, 3, 5, 8])
@pytest.mark.parametrize("T,tile", [(6, 0), (40, 0), (100, 128), (300, 256)])
def test_linear_tensor_cores_cluster_reduction(splits, T, tile):
    """Ranges of K added inside the kernel by a thread-block cluster."""
    from agave_b200 import kernels
    N, K = 200, 6912 // 4
    x, w = rnd(T, K, dtype=torch.bfloat16, seed=12), rnd(N, K, dtype=torch.bfloat16, seed=13)
    ref = x.float() @ w.float().T
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
        kernels.linear_tc(x, w, out, splits=splits, cluster=splits, token_tile=tile)
        assert kernels.linear_tc_status() == 0
        assert rel_err(out, ref) < (1e-5 if out_dtype == torch.float32 else 5e-3)
    # several clusters per tile: groups of partial sums, and ranks without a range of K
    for groups, c in ((2, splits), (3, 2)):
        out = torch.full((groups, T, N), float("nan"), dtype=torch.float32, device=DEV)
        kernels.linear_tc(x, w, out, splits=groups * c, cluster=c, token_tile=tile)
        assert kernels.linear_tc_status() == 0
        assert rel_err(out.sum(0), ref) < 1e-5
    small = rnd(T, 128, dtype=torch.bfloat16, seed=14)           # two blocks of K, eight ranks
    wsm = rnd(N, 128, dtype=torch.bfloat16, seed=15)
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.linear_tc(small, wsm, out, splits=8, cluster=8, token_tile=tile)
    assert rel_err(out, small.float() @ wsm.float().T) < 1e-5


@pytest.mark.parametrize("T", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(1152, 1024), (1536, 1152), (200, 6912), (6912, 1152), (50, 72),
                                 (1000, 5376)])
def test_projection_of_a_few_tokens_with_the_join_in_its_prologue(T, N, K):
    """One dot product per warp and row: plain and gated, x given; and x formed in the
    prologue from the stream, a branch and both norms (every combination), with the stream
    written to another buffer."""
    from agave_b200 import kernels
    assert kernels.gemv_few_supported(T, N, K, K) and not kernels.gemv_few_supported(5, N, K, K)
    x = rnd(T + 1, K + 8, dtype=torch.bfloat16, seed=31)[:T, :K]           # a row-strided view
    w = rnd(N, K, dtype=torch.bfloat16, seed=32, scale=0.05)
    w2 = rnd(N, K, dtype=torch.bfloat16, seed=33, scale=0.05)
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemv_few(w, out, x=x)
    assert rel_err(out, x.float() @ w.float().T) < 1e-5
    for act in ("gelu_tanh", "silu"):
        g, u = x.float() @ w.float().T, x.float() @ w2.float().T
        a = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" \
            else torch.nn.functional.silu(g)
        outb = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemv_few(w, outb, x=x, w2=w2, activation=act)
        assert rel_err(outb, a * u) < 6e-3
    if not kernels.gemv_few_supported(T, N, K, join=True):
        assert T * K * 8 + K * 8 > 200 * 1024
        return
    h = rnd(T, K, seed=34)
    y = rnd(T, K, seed=35)
    wp, wn = rnd(K, seed=36) * 0.2 + 1, rnd(K, seed=37) * 0.2 + 1

    def norm(v, wt, eps):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * wt

    for yy, post in ((y, wp), (y, None), (None, None)):
        h_out = torch.full_like(h, float("nan"))
        out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
        kernels.gemv_few(w, out, h_in=h, h_out=h_out if yy is not None else None, y=yy, w_post=post,
                         w_next=wn, eps_post=1e-5, eps_next=1e-6)
        href = h if yy is None else h + (norm(yy, post, 1e-5) if post is not None else yy)
        if yy is not None:
            assert rel_err(h_out, href) < 1e-6
        xr = norm(href, wn, 1e-6).to(torch.bfloat16).float()
        assert rel_err(out, xr @ w.float().T) < 2e-3      # (x is rounded to bfloat16 in both)
    outb = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    h_out = torch.full_like(h, float("nan"))
    kernels.gemv_few(w, outb, w2=w2, h_in=h, h_out=h_out, y=y, w_post=wp, w_next=wn, eps_post=1e-5,
                     eps_next=1e-6)
    href = h + norm(y, wp, 1e-5)
    xr = norm(href, wn, 1e-6).to(torch.bfloat16).float()
    ref = torch.nn.functional.gelu(xr @ w.float().T, approximate="tanh") * (xr @ w2.float().T)
    assert rel_err(outb, ref) < 8e-3 and rel_err(h_out, href) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_simt_plain_and_gated(dtype):
    from agave_b200 import kernels
    T, N, K = 37, 131, 67          # nothing a multiple of anything
    x, w, w2 = rnd(T, K, dtype=dtype, seed=1), rnd(N, K, dtype=dtype, seed=2), rnd(N, K, dtype=dtype, seed=3)
    out = torch.empty((T, N), dtype=dtype, device=DEV)
    kernels.linear_simt(x, w, out)
    tol = 1e-5 if dtype == torch.float32 else 6e-3
    assert rel_err(out, x.float() @ w.float().T) < tol
    kernels.linear_simt(x, w, out, w2=w2, activation="gelu_tanh")
    ref = torch.nn.functional.gelu(x.float() @ w.float().T, approximate="tanh") * (x.float() @ w2.float().T)
    assert rel_err(out, ref) < tol
    if dtype == torch.float32:
        # true 32-bit: no reduced-precision matrix mode hides in the product
        big = rnd(8, 4096, seed=4) + 1.0
        wb = rnd(8, 4096, seed=5) + 1.0
        o = torch.empty((8, 8), dtype=torch.float32, device=DEV)
        kernels.linear_simt(big, wb, o)
        assert rel_err(o, big.double() @ wb.double().T) < 2e-6


# ---------------------------------------------------------------------- norms
@pytest.mark.parametrize("H,R", [(48, 7), (1000, 7), (5376, 7), (1152, 300), (2048, 257), (72, 513),
                                 (2560, 300), (5376, 260), (8192, 257), (2052, 258),
                                 (1152, 64), (2560, 40), (5376, 100), (100, 33), (8192, 32)])
def test_norm_family(H, R):
    from agave_b200 import kernels
    h = rnd(R, H, seed=1)
    y = rnd(R, H, dtype=torch.bfloat16, seed=2)
    wp, wn = rnd(H, seed=3) * 0.2 + 1, rnd(H, seed=4) * 0.2 + 1
    eps_p, eps_n = 1e-5, 1e-6

    def norm(v, w, eps):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w

    # plain norm with a row gather
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    # (with many rows and a 32-bit branch the one-warp-per-row kernel runs below)
    x = torch.empty((3, H), dtype=torch.float32, device=DEV)
    kernels.norm_residual(h, None, None, wn, x, eps_next=eps_n, rows=rows)
    assert rel_err(x, norm(h[rows.long()], wn, eps_n)) < 1e-6
    # h += post(y); x = next(h)
    h2 = h.clone()
    xb = torch.empty((R, H), dtype=torch.bfloat16, device=DEV)
    kernels.norm_residual(h2, y, wp, wn, xb, eps_post=eps_p, eps_next=eps_n)
    href = h + norm(y.float(), wp, eps_p)
    assert rel_err(h2, href) < 1e-6
    assert rel_err(xb, norm(href, wn, eps_n)) < 5e-3
    # partial sums as the branch, no post norm, no next norm
    parts = rnd(3, R, H, seed=5)
    h3 = h.clone()
    kernels.norm_residual(h3, parts, None, None, None)
    assert rel_err(h3, h + parts.sum(0)) < 1e-6
    # 32-bit partial sums with both norms (what follows a tensor-core product)
    h4 = h.clone()
    kernels.norm_residual(h4, parts, wp, wn, xb, eps_post=eps_p, eps_next=eps_n)
    href = h + norm(parts.sum(0), wp, eps_p)
    assert rel_err(h4, href) < 1e-6
    assert rel_err(xb, norm(href, wn, eps_n)) < 5e-3


# ------------------------------------------------------ embedding and rotation
def test_embed_and_rope_table():
    from agave_b200 import kernels
    V, H = 1003, 72
    table = rnd(V, H, dtype=torch.bfloat16, seed=1)
    toks = torch.tensor([0, 1002, 17, 17], dtype=torch.int32, device=DEV)
    out = torch.empty((4, H), dtype=torch.float32, device=DEV)
    kernels.embed(toks, table, math.sqrt(H), out)
    assert torch.equal(out, table[toks.long()].float() * torch.tensor(math.sqrt(H), dtype=torch.float32))
    pos = torch.tensor([0, 1, 4095, 8191], dtype=torch.int32, device=DEV)
    rd = 48
    cos = torch.empty((4, rd // 2), dtype=torch.float32, device=DEV)
    sin = torch.empty_like(cos)
    kernels.rope_table(pos, rd, 5e5, 8.0, cos, sin)
    i = torch.arange(rd // 2, dtype=torch.float64)
    ang = (pos.cpu().double() / 8.0)[:, None] * torch.exp(-math.log(5e5) * 2 * i / rd)[None, :]
    assert (cos.cpu().double() - torch.cos(ang)).abs().max() < 1e-7
    assert (sin.cpu().double() - torch.sin(ang)).abs().max() < 1e-7


# ------------------------------------------- q/k norm, rotation and cache store
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rd", [(3, 1, 16, 16), (6, 2, 48, 32), (4, 4, 80, 80),
                                          (4, 1, 256, 256), (8, 2, 128, 128), (2, 2, 64, 64),
                                          (3, 1, 192, 192), (2, 1, 128, 64)])
def test_qk_norm_rope_store(dtype, nh, nkv, hd, rd):
    from agave_b200 import kernels
    T, PAGE, cap = 11, 4, 8            # a ring of 8 rows in pages of 4
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=1)
    orig = qkv.clone().float()
    wq, wk = rnd(hd, seed=2) * 0.1 + 1, rnd(hd, seed=3) * 0.1 + 1
    # two sequences: tokens 0..6 are positions 0..6 of entry 0, tokens 7..10 positions 0..3 of entry 1
    positions = torch.tensor(list(range(7)) + list(range(4)), dtype=torch.int32, device=DEV)
    seq_index = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    lens = torch.tensor([7, 4], dtype=torch.int32, device=DEV)
    table = torch.tensor([[5, 1], [0, 0], [3, 4]], dtype=torch.int32, device=DEV)
    k_pool = torch.zeros((6, PAGE, nkv, hd), dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    cos = torch.empty((T, rd // 2), dtype=torch.float32, device=DEV)
    sin = torch.empty_like(cos)
    kernels.rope_table(positions, rd, 10000.0, 1.0, cos, sin)
    kernels.qk_norm_rope_store(qkv, nh, nkv, hd, wq, wk, 1e-6, cos, sin, rd, positions, k_pool,
                               v_pool, table, slots, lens, seq_index, PAGE, cap)
    x = orig.reshape(T, nh + 2 * nkv, hd)

    def ref_head(v, w):
        v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + 1e-6) * w
        half = rd // 2
        c, s = cos[:, None, :], sin[:, None, :]
        out = v.clone()
        out[..., :half] = v[..., :half] * c - v[..., half:rd] * s
        out[..., half:rd] = v[..., :half] * s + v[..., half:rd] * c
        return out

    q_ref, k_ref, v_ref = ref_head(x[:, :nh], wq), ref_head(x[:, nh:nh + nkv], wk), x[:, nh + nkv:]
    got = qkv.float().reshape(T, nh + 2 * nkv, hd)
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert rel_err(got[:, :nh], q_ref) < tol and rel_err(got[:, nh:nh + nkv], k_ref) < tol
    for t in range(T):
        b, p = int(seq_index[t]), int(positions[t])
        row = p % cap
        page = int(table[int(slots[b]), row // PAGE])
        assert rel_err(k_pool[page, row % PAGE].float(), k_ref[t]) < tol
        assert rel_err(v_pool[page, row % PAGE].float(), v_ref[t]) < tol
    # pages nobody owns stay untouched
    assert (k_pool[2] == 0).all() and (k_pool[1, 3] == 0).all()
    # the same input given as 32-bit partial sums over three ranges of K
    parts = torch.randn(3, T, (nh + 2 * nkv) * hd, device=DEV)
    parts[2] = orig - parts[0] - parts[1]
    qkv2 = torch.full_like(qkv, float("nan"))
    k2, v2 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    kernels.qk_norm_rope_store(qkv2, nh, nkv, hd, wq, wk, 1e-6, cos, sin, rd, positions, k2, v2,
                               table, slots, lens, seq_index, PAGE, cap, partial=parts)
    assert rel_err(qkv2, qkv) < (2e-5 if dtype == torch.float32 else 8e-3)
    assert rel_err(k2, k_pool) < (2e-5 if dtype == torch.float32 else 8e-3)
    assert rel_err(v2, v_pool) < (2e-5 if dtype == torch.float32 else 8e-3)


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("nh,nkv,hd,norm,rotate", [(4, 1, 256, True, True), (6, 2, 128, True, True),
                                                   (3, 2, 64, False, True), (8, 4, 128, True, False),
                                                   (2, 1, 64, True, True)])
def test_qkv_product_with_norm_rotation_and_stores_in_its_epilogue(nh, nkv, hd, norm, rotate):
    """The prompt step's q/k/v product whose epilogue norms and rotates q and k, writes the
    cache rows and the transposed values, against the plain product followed by the
    separate norm / rotation / store kernel: three sequences of unequal lengths, one
    longer than its ring (its early rows are not stored), a padding slot in between,
    token counts that end inside a tile, a projection whose rows do not fill the last
    chunk of 256."""
    from agave_b200 import kernels
    K, PAGE, cap = 320, 64, 256
    lens = [300, 70, 197]
    T, B = sum(lens), 3
    width = (nh + 2 * nkv) * hd
    x = rnd(T, K, dtype=torch.bfloat16, seed=1, scale=0.5)
    w = rnd(width, K, dtype=torch.bfloat16, seed=2, scale=0.1)
    wq = (1.0 + 0.3 * rnd(hd, seed=5)) if norm else None
    wk = (1.0 + 0.3 * rnd(hd, seed=6)) if norm else None
    positions = torch.cat([torch.arange(n) for n in lens]).int().to(DEV)
    seq_index = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().to(DEV)
    cu = torch.tensor([0, 300, 370, 567], dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
    max_pages = cap // PAGE
    g = torch.Generator().manual_seed(3)
    table = torch.randperm(4 * max_pages, generator=g).int().reshape(4, max_pages).contiguous().to(DEV)
    cos = sin = None
    if rotate:
        cos = torch.empty((T, hd // 2), dtype=torch.float32, device=DEV)
        sin = torch.empty_like(cos)
        kernels.rope_table(positions, hd, 10000.0, 1.0, cos, sin)
    import ctypes
    assert kernels.library().agv_qkv_prefill_tc_supported(
        hd, hd if rotate else 0, K, ctypes.c_longlong(K), ctypes.c_longlong(width))
    # the separate path
    part = torch.empty((1, T, width), dtype=torch.float32, device=DEV)
    kernels.linear_tc(x, w, part[0])
    k_ref = torch.zeros((4 * max_pages, PAGE, nkv, hd), dtype=torch.bfloat16, device=DEV)
    v_ref = torch.zeros_like(k_ref)
    qkv_ref = torch.empty((T, width), dtype=torch.bfloat16, device=DEV)
    vt_ref = kernels.prefill_values_scratch(T, B, nkv, hd, torch.device(DEV))
    vt_ref.fill_(7.0)
    kernels.qk_norm_rope_store(qkv_ref, nh, nkv, hd, wq, wk, 1e-5, cos, sin, hd if rotate else 0,
                               positions, k_ref, v_ref, table, slots, lens_t, seq_index, PAGE, cap,
                               partial=part, vt=vt_ref, cu_seqlens=cu, max_len=max(lens))
    # the product with the epilogue
    k_got, v_got = torch.zeros_like(k_ref), torch.zeros_like(v_ref)
    qkv = torch.full((T, width), float("nan"), dtype=torch.bfloat16, device=DEV)
    vt = torch.full_like(vt_ref, 7.0)
    kernels.qkv_prefill(x, w, qkv, nh, nkv, hd, wq, wk, 1e-5, cos, sin, positions, seq_index,
                        k_pool=k_got, v_pool=v_got, page_table=table, slots=slots, lens=lens_t,
                        page=PAGE, cap=cap, vt=vt, cu_seqlens=cu)
    assert kernels.linear_tc_status() == 0
    assert torch.isfinite(qkv.float()).all()
    assert rel_err(qkv, qkv_ref) < 6e-3
    for lo in range(0, width, hd):                       # head by head
        assert rel_err(qkv[:, lo:lo + hd], qkv_ref[:, lo:lo + hd]) < 8e-3, lo // hd
    assert rel_err(k_got, k_ref) < 8e-3 and rel_err(v_got, v_ref) < 8e-3
    # the same rows and no others were written (sequence 0 is longer than its ring)
    assert torch.equal(k_got.abs().sum(dim=(2, 3)) > 0, k_ref.abs().sum(dim=(2, 3)) > 0)
    assert torch.equal(vt == 7.0, vt_ref == 7.0)         # the same columns, the same zero padding
    assert rel_err(vt, vt_ref) < 8e-3
    # without a cache and without the transposed copy: only qkv
    qkv2 = torch.full_like(qkv, float("nan"))
    kernels.qkv_prefill(x, w, qkv2, nh, nkv, hd, wq, wk, 1e-5, cos, sin, positions, seq_index)
    assert torch.equal(qkv2, qkv)


def ref_attention(q, k, v, scale, window):
    """q [Tq, nh, hd] at positions pos (last Tq of the keys), k/v [Tk, nkv, hd]."""
    Tq, nh, hd = q.shape
    Tk, nkv = k.shape[0], k.shape[1]
    out = torch.zeros(Tq, nh, hd, dtype=torch.float64)
    for i in range(Tq):
        p = Tk - Tq + i
        lo = max(0, p - window + 1) if window else 0
        for h in range(nh):
            g = h // (nh // nkv)
            s = (k[lo:p + 1, g].double() @ q[i, h].double()) * scale
            a = torch.softmax(s, 0)
            out[i, h] = a @ v[lo:p + 1, g].double()
    return out.reshape(Tq, nh * hd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 1, 16, 5), (6, 2, 48, 0), (2, 2, 128, 9)])
def test_attention_prefill_ragged(dtype, nh, nkv, hd, window):
    from agave_b200 import kernels
    lens = [13, 1, 30]
    T = sum(lens)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=1)
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    out = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
    positions = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32, device=DEV)
    seq_index = torch.tensor(sum([[i] * n for i, n in enumerate(lens)], []), dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 13, 14, 44], dtype=torch.int32, device=DEV)
    scale = 0.17
    kernels.attention_prefill_simt(q, k, v, out, positions, seq_index, cu, nh, nkv, hd, scale, window)
    o = 0
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    for n in lens:
        qs = q[o:o + n].float().cpu().reshape(n, nh, hd)
        ks = k[o:o + n].float().cpu().reshape(n, nkv, hd)
        vs = v[o:o + n].float().cpu().reshape(n, nkv, hd)
        assert rel_err(out[o:o + n], ref_attention(qs, ks, vs, scale, window)) < tol
        o += n


def test_attention_finds_a_far_key_and_respects_the_window_edge():
    """One key among hundreds is made to dominate: without a window the query
    must return that key's value; with a window that just excludes it, it must not."""
    from agave_b200 import kernels
    nh = nkv = 1
    hd, n, far = 32, 300, 3
    k = rnd(n, hd, seed=1, scale=0.1)
    v = rnd(n, hd, seed=2)
    q = rnd(n, hd, seed=3, scale=0.1)
    k[far] = 0; k[far, 0] = 40.0
    q[-1] = 0; q[-1, 0] = 40.0
    qkv = torch.cat([q, k, v], dim=1).contiguous()
    positions = torch.arange(n, dtype=torch.int32, device=DEV)
    seq_index = torch.zeros(n, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    out = torch.empty((n, hd), dtype=torch.float32, device=DEV)
    args = (qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], out, positions, seq_index, cu, 1, 1, hd, 1.0)
    kernels.attention_prefill_simt(*args, 0)
    assert rel_err(out[-1], v[far]) < 1e-4
    kernels.attention_prefill_simt(*args, n - far)          # window reaches exactly key `far`
    assert rel_err(out[-1], v[far]) < 1e-4
    kernels.attention_prefill_simt(*args, n - far - 1)      # one shorter: the key is outside
    assert (out[-1] - v[far]).abs().max() > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 1, 16, 0), (6, 2, 48, 7), (8, 2, 64, 0)])
def test_attention_over_the_paged_cache(dtype, nh, nkv, hd, window):
    from agave_b200 import kernels
    PAGE = 4
    lens = [9, 1, 22]                      # lengths after this step; queries are the last tokens
    cap = 24 if not window else 8          # the window ring is shorter than the sequences
    max_pages = cap // PAGE
    n_pages = 40
    k_pool = rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=1)
    v_pool = rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=2)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).int()
    table = perm[:4 * max_pages].reshape(4, max_pages).contiguous().to(DEV)
    slots = torch.tensor([3, -1, 1, 0], dtype=torch.int32, device=DEV)   # entry 1 is padding
    lens_t = [9, 0, 1, 22]
    q = rnd(4, nh * hd, dtype=dtype, seed=4)
    positions = torch.tensor([8, 0, 0, 21], dtype=torch.int32, device=DEV)
    seq_index = torch.arange(4, dtype=torch.int32, device=DEV)
    out = torch.full((4, nh * hd), float("nan"), dtype=dtype, device=DEV)
    kernels.attention_paged_simt(q, out, k_pool, v_pool, table, slots, positions, seq_index, PAGE,
                                 cap, nh, nkv, hd, 0.2, window)
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert (out[1] == 0).all()
    # the split kernel on the same cache: same result, whatever bound on the keys is given
    for max_keys in (22, 200):
        out2 = torch.full_like(out, float("nan"))
        kernels.attention_decode_split(q, out2, k_pool, v_pool, table, slots, positions, PAGE, cap,
                                       nh, nkv, hd, 0.2, window, window or max_keys)
        assert (out2[1] == 0).all()
        assert rel_err(out2, out) < tol
    for b in (0, 2, 3):
        n, slot = lens_t[b], int(slots[b])
        lo = max(0, n - window) if window else 0
        ks, vs = [], []
        for j in range(lo, n):
            row = j % cap
            page = int(table[slot, row // PAGE])
            ks.append(k_pool[page, row % PAGE].float().cpu())
            vs.append(v_pool[page, row % PAGE].float().cpu())
        ks, vs = torch.stack(ks), torch.stack(vs)
        qs = q[b].float().cpu().reshape(1, nh, hd)
        ref = ref_attention(qs, ks, vs, 0.2, 0)
        assert rel_err(out[b:b + 1], ref) < tol, b


@pytest.mark.parametrize("H,R,S", [(1152, 64, 16), (2560, 48, 9), (5376, 33, 6), (1152, 8, 16),
                                   (640, 256, 2), (1152, 300, 5)])
def test_norm_of_many_partial_sums(H, R, S):
    """The branch as S 32-bit partial sums (what a product with K cut into ranges leaves),
    at row counts that take each of the norm kernels; S that is no multiple of the number
    of partial sums a kernel loads together."""
    from agave_b200 import kernels
    h = rnd(R, H, seed=1)
    parts = rnd(S, R, H, seed=2, scale=0.5)
    wp, wn = rnd(H, seed=3) * 0.2 + 1, rnd(H, seed=4) * 0.2 + 1

    def norm(v, w, eps):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w

    h2 = h.clone()
    xb = torch.empty((R, H), dtype=torch.bfloat16, device=DEV)
    kernels.norm_residual(h2, parts, wp, wn, xb, eps_post=1e-5, eps_next=1e-6)
    href = (h.double() + norm(parts.double().sum(0), wp.double(), 1e-5)).float()
    assert rel_err(h2, href) < 2e-6
    assert rel_err(xb, norm(href, wn, 1e-6)) < 5e-3


# ------------------------------------------------------------------- sampling
@pytest.mark.parametrize("V", [257, 5000, 262144 + 64])
def test_argmax_first_index_on_ties(V):
    from agave_b200 import kernels
    logits = rnd(3, V, seed=1)
    logits[0, 100] = 50.0; logits[0, 200] = 50.0
    logits[1, V - 1] = 60.0
    logits[2, 0] = 70.0
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    kernels.argmax(logits, out)
    assert out.tolist() == [100, V - 1, 0]


@pytest.mark.parametrize("V,T", [(262144 + 64, 8), (5003, 33), (130, 1), (1000, 128), (40000, 64)])
def test_arg_max_in_the_head_products_epilogue(V, T):
    """The product whose rows are reduced to the index of their greatest element before
    anything is written: against torch.argmax of the 32-bit product, with ties inside a
    tile of 128 features, across tile borders and in the last, partial tile (equal weight
    rows give equal logits), and twice in a row (the keys go back to zero)."""
    from agave_b200 import kernels
    K = 320
    x = rnd(T, K, dtype=torch.bfloat16, seed=1, scale=0.5)
    w = rnd(V, K, dtype=torch.bfloat16, seed=2, scale=0.1)
    # a row that wins for token 0, stored at several places: the first must be chosen
    big = (x[0].float() * 0.2).to(torch.bfloat16)
    places = sorted({V - 1, V - 2, min(V - 1, 129), min(V - 1, 127), V // 2})
    w[places] = big
    # and a pair of equal rows elsewhere for the last token
    if T > 1:
        w[[3, min(V - 1, 700)]] = (x[T - 1].float() * 0.2).to(torch.bfloat16)
    logits = torch.empty((T, V), dtype=torch.float32, device=DEV)
    kernels.linear_tc(x, w, logits)
    want = torch.argmax(logits, dim=1).int()
    # torch.argmax's tie rule is not promised: the first index of the maximum is
    first = (logits == logits.max(dim=1, keepdim=True).values).int().argmax(dim=1).int()
    for _ in range(2):
        out = torch.full((T,), -7, dtype=torch.int32, device=DEV)
        kernels.linear_argmax(x, w, out)
        assert kernels.linear_tc_status() == 0
        assert torch.equal(out, first), (out[:8], first[:8], want[:8])
    assert int(out[0]) == places[0]
    if T > 1:
        assert int(out[T - 1]) == 3


def test_sampling_matches_the_filtered_distribution():
    import sys, os
    from agave_b200 import kernels
    from plain import gemma3_plain as P
    V, n = 1000, 4000
    base = rnd(V, seed=5) * 2.0
    temperature, top_k, top_p = 0.8, 50, 0.9
    wts = P.filtered_weights(base.cpu(), temperature, top_k, top_p)
    probs = (wts / wts.sum()).double()
    logits = base[None, :].expand(n, V).contiguous()
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    seq = torch.arange(n, dtype=torch.int64, device=DEV)
    steps = torch.zeros(n, dtype=torch.int32, device=DEV)
    kernels.sample(logits, out, temperature, top_k, top_p, 1234, seq, steps)
    counts = torch.bincount(out.cpu().long(), minlength=V).double()
    assert counts[probs == 0].sum() == 0              # nothing outside the kept set
    kept = probs > 0
    assert int(kept.sum()) <= top_k
    # chi-square-like bound on the kept set
    exp = probs[kept] * n
    chi = (((counts[kept] - exp) ** 2) / exp.clamp_min(1e-9)).sum().item()
    assert chi < 3 * int(kept.sum()) + 30, chi
    # same seed, same draw; other seed, other draws; batch position does not matter
    out2 = torch.empty_like(out)
    kernels.sample(logits, out2, temperature, top_k, top_p, 1234, seq, steps)
    assert torch.equal(out, out2)
    kernels.sample(logits, out2, temperature, top_k, top_p, 99, seq, steps)
    assert not torch.equal(out, out2)
    perm = torch.randperm(n, device=DEV)
    kernels.sample(logits, out2, temperature, top_k, top_p, 1234, seq[perm].contiguous(), steps)
    assert torch.equal(out2, out[perm])


def test_repeat_penalty_per_occurrence_and_history():
    from agave_b200 import kernels
    V = 300
    logits = torch.ones((2, V), device=DEV)
    logits[:, 7] = -2.0
    hist = torch.zeros((4, 16), dtype=torch.int32, device=DEV)
    hist_len = torch.zeros(4, dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, -1], dtype=torch.int32, device=DEV)
    for tok in (5, 7, 5):
        kernels.history_append(torch.tensor([tok, 9], dtype=torch.int32, device=DEV), slots, hist, hist_len)
    assert hist_len.tolist() == [0, 0, 3, 0] and hist[2, :3].tolist() == [5, 7, 5]
    kernels.repeat_penalty(logits, slots, hist, hist_len, 2.0)
    assert logits[0, 5].item() == 0.25 and logits[0, 7].item() == -4.0
    assert logits[0, 6].item() == 1.0 and (logits[1] == torch.where(torch.arange(V, device=DEV) == 7, -2.0, 1.0)).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 1, 256), (16, 2, 128), (5, 5, 80), (12, 2, 512),
                                       (3, 1, 208), (2, 2, 48), (34, 2, 112)])
def test_attention_decode_split_long_sequences(dtype, nh, nkv, hd, decode_tiles):
    """Several chunks per sequence, groups wider than the kernel's head tile,
    a far key that must win, and a window edge in the middle of a chunk."""
    from agave_b200 import kernels
    PAGE = 64
    lens = [700, 65, 1]
    max_pages = 12
    n_pages = 3 * max_pages
    k_pool = rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=1, scale=0.3)
    v_pool = rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=2)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).int()
    table = perm.reshape(3, max_pages).contiguous().to(DEV)
    slots = torch.tensor([1, 2, 0], dtype=torch.int32, device=DEV)
    q = rnd(3, nh * hd, dtype=dtype, seed=4, scale=0.3)
    # sequence 0: key 5 dominates head 0
    page5 = int(table[1, 0])
    k_pool[page5, 5, 0] = 0; k_pool[page5, 5, 0, 0] = 30.0
    q[0, :hd] = 0; q[0, 0] = 30.0
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq_index = torch.arange(3, dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    for window in (0, 100, 695):
        cap = max_pages * PAGE
        ref = torch.empty((3, nh * hd), dtype=dtype, device=DEV)
        kernels.attention_paged_simt(q, ref, k_pool, v_pool, table, slots, positions, seq_index,
                                     PAGE, cap, nh, nkv, hd, 1.0, window)
        out = torch.full_like(ref, float("nan"))
        kernels.attention_decode_split(q, out, k_pool, v_pool, table, slots, positions, PAGE, cap,
                                       nh, nkv, hd, 1.0, window, window or 768)
        assert rel_err(out, ref) < tol, window
        if window in (0, 695):
            assert rel_err(out[0, :hd], v_pool[page5, 5, 0]) < 2e-2     # the far key is seen
        else:
            assert (out[0, :hd].float() - v_pool[page5, 5, 0].float()).abs().max() > 0.1


@pytest.mark.parametrize("B,nh,nkv,hd", [(64, 8, 4, 256), (96, 4, 1, 128), (200, 4, 2, 64),
                                        (700, 4, 2, 64), (300, 2, 2, 128)])
def test_attention_decode_many_sequences_walk_several_tiles(B, nh, nkv, hd, decode_tiles):
    """With many sequences a sequence gets few CTAs, each of which walks several key
    tiles with a running softmax (and, with fewer still, a single CTA the whole
    sequence): unequal lengths up to a dozen tiles, padding entries in between, a
    window, against the one-warp kernel.  What the last page of a sequence holds beyond
    its newest position is not a number: a kernel that brings whole pages must not let
    it through."""
    from agave_b200 import kernels
    PAGE, max_pages = 64, 12
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(1, max_pages * PAGE, (B,), generator=g).tolist()
    lens[0], lens[1], lens[2] = max_pages * PAGE, 1, 64
    k_pool = rnd(B * max_pages, PAGE, nkv, hd, dtype=torch.bfloat16, seed=1, scale=0.3)
    v_pool = rnd(B * max_pages, PAGE, nkv, hd, dtype=torch.bfloat16, seed=2)
    table = torch.randperm(B * max_pages, generator=g).int().reshape(B, max_pages).contiguous().to(DEV)
    slots = torch.arange(B, dtype=torch.int32)
    slots[5::17] = -1                                   # padding entries
    slots = slots.to(DEV)
    q = rnd(B, nh * hd, dtype=torch.bfloat16, seed=4, scale=0.3)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq_index = torch.arange(B, dtype=torch.int32, device=DEV)
    cap = max_pages * PAGE
    for b in range(0, B, 3):
        if int(slots[b]) >= 0 and lens[b] % PAGE:
            pg = int(table[int(slots[b]), (lens[b] - 1) // PAGE])
            k_pool[pg, lens[b] % PAGE:] = float("nan")
            v_pool[pg, lens[b] % PAGE:] = float("nan")
    for window in (0, 200):
        ref = torch.empty((B, nh * hd), dtype=torch.bfloat16, device=DEV)
        live = (slots >= 0).nonzero().flatten()
        kernels.attention_paged_simt(q[live].contiguous(), ref[: live.numel()], k_pool, v_pool, table,
                                     slots[live].contiguous(), positions[live].contiguous(),
                                     torch.arange(live.numel(), dtype=torch.int32, device=DEV),
                                     PAGE, cap, nh, nkv, hd, 0.5, window)
        out = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.attention_decode_split(q, out, k_pool, v_pool, table, slots, positions, PAGE, cap,
                                       nh, nkv, hd, 0.5, window, window or cap)
        assert torch.isfinite(out.float()).all()
        assert rel_err(out[live], ref[: live.numel()]) < 8e-3, window
        assert (out[slots < 0] == 0).all()


@pytest.mark.parametrize("nh,nkv,hd,window,G", [(4, 1, 256, 0, 8), (4, 1, 256, 100, 3),
                                                (16, 2, 128, 0, 1), (40, 2, 64, 0, 5),
                                                (8, 8, 64, 70, 9), (6, 3, 128, 64, 16),
                                                (32, 2, 256, 0, 2), (20, 1, 128, 0, 4)])
@pytest.mark.parametrize("norm,rotate", [(True, True), (False, False)])
def test_attention_decode_with_norm_rotation_and_store_inside(nh, nkv, hd, window, G, norm, rotate,
                                                              decode_tiles):
    """The decode attention that forms q, k and v of the new position from the
    projection's partial sums, against the separate norm / rotation / store launch
    followed by the plain decode attention: the outputs, the cache rows it writes, and
    that it writes no other row.  Lengths put the new position at a tile's first and
    last row and in a page's first row; more heads per group than the kernel's head tile
    (two CTAs form the same key, one writes it) and as many as it has warps; a padding
    entry; a layer that only reads the cache (store_kv off)."""
    from types import SimpleNamespace
    from agave_b200 import kernels
    assert kernels.attention_decode_fused_supported(torch.bfloat16, hd, hd if rotate else 0)
    PAGE, max_pages = 64, 12
    lens = [700, 65, 1, 64, 129, 5, 300]
    B = len(lens)
    cap = max_pages * PAGE
    width = (nh + 2 * nkv) * hd
    k0 = rnd(B * max_pages, PAGE, nkv, hd, dtype=torch.bfloat16, seed=1, scale=0.3)
    v0 = rnd(B * max_pages, PAGE, nkv, hd, dtype=torch.bfloat16, seed=2)
    g = torch.Generator().manual_seed(3)
    table = torch.randperm(B * max_pages, generator=g).int().reshape(B, max_pages).contiguous().to(DEV)
    slots = torch.tensor([3, 0, 6, -1, 2, 5, 1], dtype=torch.int32, device=DEV)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    seq_index = torch.arange(B, dtype=torch.int32, device=DEV)
    part = rnd(G, B, width, seed=4, scale=0.5 / G ** 0.5)
    wq = (1.0 + 0.3 * rnd(hd, seed=5)) if norm else None
    wk = (1.0 + 0.3 * rnd(hd, seed=6)) if norm else None
    cos = sin = None
    if rotate:
        cos = torch.empty((B, hd // 2), dtype=torch.float32, device=DEV)
        sin = torch.empty_like(cos)
        kernels.rope_table(positions, hd, 10000.0, 1.0, cos, sin)
    view = SimpleNamespace(page_table=table, page=PAGE, cap=cap)
    ctx = SimpleNamespace(slots=slots, positions=positions, max_len=max(lens))

    k_ref, v_ref = k0.clone(), v0.clone()
    qkv = torch.empty((B, width), dtype=torch.bfloat16, device=DEV)
    kernels.qk_norm_rope_store(qkv, nh, nkv, hd, wq, wk, 1e-5, cos, sin, hd if rotate else 0,
                               positions, k_ref, v_ref, table, slots, lens_t, seq_index, PAGE, cap,
                               partial=part)
    ref = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.attention_decode_split(qkv[:, :nh * hd], ref, k_ref, v_ref, table, slots, positions,
                                   PAGE, cap, nh, nkv, hd, 0.4, window, window or cap)
    k, v = k0.clone(), v0.clone()
    view.k_pool, view.v_pool = k, v
    out = torch.full_like(ref, float("nan"))
    kernels.attention_decode_fused(part, wq, wk, 1e-5, cos, sin, True, out, view, ctx, nh, nkv, hd,
                                   0.4, window)
    live = (slots >= 0).nonzero().flatten().tolist()
    assert torch.isfinite(out.float()).all()
    assert (out[3] == 0).all()
    assert rel_err(out[live], ref[live]) < 8e-3
    touched = torch.zeros(B * max_pages, PAGE, dtype=torch.bool, device=DEV)
    for b in live:
        row = (lens[b] - 1) % cap
        pg = int(table[int(slots[b]), row // PAGE])
        touched[pg, row % PAGE] = True
        assert rel_err(k[pg, row % PAGE], k_ref[pg, row % PAGE]) < 6e-3, b
        assert rel_err(v[pg, row % PAGE], v_ref[pg, row % PAGE]) < 6e-3, b
        assert not torch.equal(k[pg, row % PAGE], k0[pg, row % PAGE])
    assert torch.equal(k[~touched], k0[~touched]) and torch.equal(v[~touched], v0[~touched])
    # a layer that reads another layer's entry: the new row is in the cache already
    view.k_pool, view.v_pool = k_ref.clone(), v_ref.clone()
    out2 = torch.full_like(ref, float("nan"))
    kernels.attention_decode_fused(part, wq, wk, 1e-5, cos, sin, False, out2, view, ctx, nh, nkv,
                                   hd, 0.4, window)
    assert rel_err(out2[live], ref[live]) < 8e-3
    assert torch.equal(view.k_pool, k_ref) and torch.equal(view.v_pool, v_ref)


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 1, 256, 0), (4, 1, 256, 100), (6, 2, 128, 70),
                                              (3, 3, 64, 0), (4, 2, 16, 5), (2, 1, 40, 33),
                                              (2, 1, 200, 64)])
def test_attention_prefill_tensor_cores(nh, nkv, hd, window):
    """The mma kernel against the one-warp kernel and a 64-bit statement, ragged
    batch whose lengths straddle the 64-row tiles."""
    from agave_b200 import kernels
    lens = [1, 63, 64, 65, 200, 130]
    T = sum(lens)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=1, scale=0.5)
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    positions = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32, device=DEV)
    seq_index = torch.tensor(sum([[i] * n for i, n in enumerate(lens)], []), dtype=torch.int32, device=DEV)
    ref = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill_simt(q, k, v, ref, positions, seq_index, cu, nh, nkv, hd, 0.3, window)
    out = torch.full_like(ref, float("nan"))
    kernels.attention_prefill_mma(q, k, v, out, cu, max(lens), nh, nkv, hd, 0.3, window)
    assert torch.isfinite(out.float()).all()
    assert rel_err(out, ref) < 1.2e-2
    o = sum(lens[:4])
    n = lens[4]
    exact = ref_attention(q[o:o + n].float().cpu().reshape(n, nh, hd),
                          k[o:o + n].float().cpu().reshape(n, nkv, hd),
                          v[o:o + n].float().cpu().reshape(n, nkv, hd), 0.3, window)
    assert rel_err(out[o:o + n], exact) < 1.2e-2


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 1, 256, 0), (4, 1, 256, 100), (8, 4, 256, 0),
                                              (6, 2, 128, 70), (3, 3, 64, 0), (4, 2, 16, 5),
                                              (2, 1, 48, 33), (2, 1, 208, 64), (32, 2, 32, 0)])
def test_attention_prefill_tcgen05(nh, nkv, hd, window):
    """The tcgen05 kernel against the one-warp kernel and a 64-bit statement: ragged
    batch whose lengths straddle the tiles, heads packed per CTA (4, 2, 16), not
    packed (3 heads per kv head; 1), head sizes that end inside a 64-wide block."""
    from agave_b200 import kernels
    lens = [1, 63, 64, 65, 200, 130, 31, 450]
    T = sum(lens)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=1, scale=0.5)
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    positions = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32, device=DEV)
    seq_index = torch.tensor(sum([[i] * n for i, n in enumerate(lens)], []), dtype=torch.int32, device=DEV)
    ref = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill_simt(q, k, v, ref, positions, seq_index, cu, nh, nkv, hd, 0.3, window)
    out = torch.full_like(ref, float("nan"))
    kernels.attention_prefill_tc(q, k, v, out, cu, max(lens), nh, nkv, hd, 0.3, window)
    assert kernels.attention_tc_status() == 0
    assert torch.isfinite(out.float()).all()
    assert rel_err(out, ref) < 1.2e-2
    o = sum(lens[:4])
    n = lens[4]
    exact = ref_attention(q[o:o + n].float().cpu().reshape(n, nh, hd),
                          k[o:o + n].float().cpu().reshape(n, nkv, hd),
                          v[o:o + n].float().cpu().reshape(n, nkv, hd), 0.3, window)
    assert rel_err(out[o:o + n], exact) < 1.2e-2


def torch_attention(q, k, v, lens, nh, nkv, hd, scale, window):
    """softmax(q k^T * scale) v on the GPU in 32-bit, sequence by sequence: a plain
    statement of the sum with the causal and window masks written out."""
    out = torch.empty((q.shape[0], nh * hd), dtype=torch.float32, device=q.device)
    o = 0
    for n in lens:
        qs = q[o:o + n].float().reshape(n, nh, hd).transpose(0, 1)             # [nh, n, hd]
        ks = k[o:o + n].float().reshape(n, nkv, hd).transpose(0, 1)
        vs = v[o:o + n].float().reshape(n, nkv, hd).transpose(0, 1)
        ks = ks.repeat_interleave(nh // nkv, dim=0)
        vs = vs.repeat_interleave(nh // nkv, dim=0)
        p = torch.arange(n, device=q.device)[:, None]
        j = torch.arange(n, device=q.device)[None, :]
        mask = j <= p
        if window:
            mask = mask & (j > p - window)
        sc = (qs @ ks.transpose(1, 2)) * scale
        sc = sc.masked_fill(~mask, float("-inf"))
        a = torch.softmax(sc, dim=-1)
        out[o:o + n] = (a @ vs).transpose(0, 1).reshape(n, nh * hd)
        o += n
    return out


@pytest.mark.parametrize("window", [0, 512])
def test_attention_prefill_tcgen05_long_sequences(window):
    """Thousands of positions, two sequences, at the benchmark's sizes (2,048 positions,
    four heads of 256, window 512), against the sum written out in torch."""
    from agave_b200 import kernels
    nh, nkv, hd = 4, 1, 256
    lens = [2048, 1500]
    T = sum(lens)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=5, scale=0.7)
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    cu = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
    ref = torch_attention(q, k, v, lens, nh, nkv, hd, 0.0625, window)
    out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill_tc(q, k, v, out, cu, max(lens), nh, nkv, hd, 0.0625, window)
    assert kernels.attention_tc_status() == 0
    assert torch.isfinite(out.float()).all()
    assert rel_err(out, ref) < 1.2e-2
    for row in (0, 63, 64, 511, 512, 513, 2047, 2048, T - 1):
        assert rel_err(out[row], ref[row]) < 2e-2, row
    # the mma.sync kernel is a second implementation of the same sum
    out2 = torch.full_like(out, float("nan"))
    kernels.attention_prefill_mma(q, k, v, out2, cu, max(lens), nh, nkv, hd, 0.0625, window)
    assert rel_err(out2, ref) < 1.2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,nh,nkv,hd", [(128, 4, 1, 64), (64, 6, 2, 128), (128, 4, 1, 256)])
def test_attention_decode_ring_as_large_as_the_window(dtype, W, nh, nkv, hd, decode_tiles):
    """cap == window: the row that held key p - W holds key p itself, so the oldest key in
    the window sits in the row right after the newest.  Lengths below, at and past the
    first wrap (129, 256, 300 for a ring of 128).  The newest key and the oldest key in
    the window each carry about a third of the weight (their scores stand out by ln(W)),
    so a kernel that looked one row too far, or counted the newest key twice, would be off
    by tens of percent; the reference is the sum over the sequence's own history, written
    out in torch."""
    from types import SimpleNamespace
    from agave_b200 import kernels
    PAGE = 64
    cap = W
    max_pages = cap // PAGE
    lens = [W + 1, 2 * W, 2 * W + 44, W, W - 1, 1, 3 * W + 7]
    B = len(lens)
    g = torch.Generator().manual_seed(11)
    table = torch.randperm(B * max_pages, generator=g).int().reshape(B, max_pages).contiguous().to(DEV)
    slots = torch.tensor([2, 0, 5, 1, 6, 3, 4], dtype=torch.int32, device=DEV)
    k_pool = torch.zeros((B * max_pages, PAGE, nkv, hd), dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    q = rnd(B, nh * hd, dtype=dtype, seed=4, scale=0.1)
    boost = float(torch.log(torch.tensor(float(W))))
    refs = []
    for b, n in enumerate(lens):
        kh = rnd(n, nkv, hd, dtype=dtype, seed=20 + b, scale=0.1)
        vh = rnd(n, nkv, hd, dtype=dtype, seed=40 + b)
        p = n - 1
        lo = max(0, p - W + 1)
        # dimension 0 carries the marks: q has sqrt(boost) there, the two marked keys too
        kh[:, :, 0] = 0
        q.view(B, nh, hd)[b, :, 0] = boost ** 0.5 * 4
        kh[p, :, 0] = boost ** 0.5 / 4
        kh[lo, :, 0] = boost ** 0.5 / 4
        if lo > 0:
            kh[lo - 1, :, 0] = 3.0          # just outside: would swamp everything if it were seen
        for j in range(max(0, n - cap), n):                       # what the ring still holds
            row = j % cap
            pg = int(table[int(slots[b]), row // PAGE])
            k_pool[pg, row % PAGE] = kh[j]
            v_pool[pg, row % PAGE] = vh[j]
        qs = q[b].float().reshape(nh, hd)
        ks = kh[lo:].float().repeat_interleave(nh // nkv, dim=1)  # [n_vis, nh, hd]
        vs = vh[lo:].float().repeat_interleave(nh // nkv, dim=1)
        a = torch.softmax(torch.einsum("hd,jhd->hj", qs, ks) * 1.0, dim=-1)
        refs.append(torch.einsum("hj,jhd->hd", a, vs).reshape(nh * hd))
        if n > 2:
            assert 0.2 < float(a[0, -1]) < 0.5 and 0.2 < float(a[0, 0]) < 0.5
    ref = torch.stack(refs)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    out = torch.full((B, nh * hd), float("nan"), dtype=dtype, device=DEV)
    kernels.attention_decode_split(q, out, k_pool, v_pool, table, slots, positions, PAGE, cap, nh,
                                   nkv, hd, 1.0, W, W)
    assert rel_err(out, ref) < tol
    for b in range(B):
        assert rel_err(out[b], ref[b]) < 2 * tol, (b, lens[b])
    seq_index = torch.arange(B, dtype=torch.int32, device=DEV)
    out1 = torch.full_like(out, float("nan"))
    kernels.attention_paged_simt(q, out1, k_pool, v_pool, table, slots, positions, seq_index, PAGE,
                                 cap, nh, nkv, hd, 1.0, W)
    assert rel_err(out1, ref) < tol
    if dtype == torch.bfloat16 and kernels.attention_decode_fused_supported(dtype, hd, 0):
        # the kernel that forms q, k and v of the new position itself: hand it q | k_p | v_p
        # as one "partial sum" and let it store the row the ring wraps onto
        part = torch.zeros((1, B, (nh + 2 * nkv) * hd), dtype=torch.float32, device=DEV)
        for b, n in enumerate(lens):
            row = (n - 1) % cap
            pg = int(table[int(slots[b]), row // PAGE])
            part[0, b, :nh * hd] = q[b].float()
            part[0, b, nh * hd:(nh + nkv) * hd] = k_pool[pg, row % PAGE].float().reshape(-1)
            part[0, b, (nh + nkv) * hd:] = v_pool[pg, row % PAGE].float().reshape(-1)
            k_pool[pg, row % PAGE] = 7.0            # stale contents the kernel must replace
            v_pool[pg, row % PAGE] = 7.0
        view = SimpleNamespace(page_table=table, page=PAGE, cap=cap, k_pool=k_pool, v_pool=v_pool)
        ctx = SimpleNamespace(slots=slots, positions=positions, max_len=max(lens))
        out2 = torch.full_like(out, float("nan"))
        kernels.attention_decode_fused(part, None, None, 0.0, None, None, True, out2, view, ctx,
                                       nh, nkv, hd, 1.0, W)
        assert rel_err(out2, ref) < tol
        for b in range(B):
            assert rel_err(out2[b], ref[b]) < 2 * tol, (b, lens[b])


def test_attention_prefill_tcgen05_far_key_window_edge_and_growing_scores():
    """One score that stands out among hundreds; the window's edge; and scores that
    grow along the sequence, so that the running maximum moves by more than the
    kernel lets it lag and the accumulator is rescaled."""
    from agave_b200 import kernels
    hd, n, far = 256, 300, 3
    k = rnd(n, hd, dtype=torch.bfloat16, seed=1, scale=0.1)
    v = rnd(n, hd, dtype=torch.bfloat16, seed=2)
    q = rnd(n, hd, dtype=torch.bfloat16, seed=3, scale=0.1)
    k[far] = 0; k[far, 0] = 40.0
    q[-1] = 0; q[-1, 0] = 40.0
    qkv = torch.cat([q, k, v], dim=1).contiguous()
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    out = torch.empty((n, hd), dtype=torch.bfloat16, device=DEV)
    args = (qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], out, cu, n, 1, 1, hd, 1.0)
    kernels.attention_prefill_tc(*args, 0)
    assert rel_err(out[-1], v[far]) < 1e-2
    kernels.attention_prefill_tc(*args, n - far)
    assert rel_err(out[-1], v[far]) < 1e-2
    kernels.attention_prefill_tc(*args, n - far - 1)
    assert (out[-1].float() - v[far].float()).abs().max() > 0.1
    # scores grow by about 0.2 per key: the maximum rises by 60 over the sequence
    k2 = torch.zeros(n, hd, dtype=torch.bfloat16, device=DEV)
    k2[:, 0] = torch.arange(n, device=DEV).to(torch.bfloat16) * 0.2
    q2 = torch.zeros(n, hd, dtype=torch.bfloat16, device=DEV)
    q2[:, 0] = 1.0
    qkv2 = torch.cat([q2, k2, v], dim=1).contiguous()
    kernels.attention_prefill_tc(qkv2[:, :hd], qkv2[:, hd:2 * hd], qkv2[:, 2 * hd:], out, cu, n, 1,
                                 1, hd, 1.0, 0)
    assert kernels.attention_tc_status() == 0
    exact = ref_attention(q2.float().cpu().reshape(n, 1, hd), k2.float().cpu().reshape(n, 1, hd),
                          v.float().cpu().reshape(n, 1, hd), 1.0, 0)
    assert rel_err(out, exact) < 1.2e-2


@pytest.mark.parametrize("nh,nkv,hd,splits", [(4, 1, 256, 1), (4, 2, 128, 2), (2, 2, 64, 0),
                                              (2, 1, 48, 1), (2, 1, 208, 0)])
def test_qk_norm_rope_store_writes_values_transposed(nh, nkv, hd, splits):
    """The transposed copy of the values: every sequence starts at a multiple of 64
    columns and is followed by zeros up to the next one; from partial sums (splits
    > 0) and from the projected rows; head sizes that take the general kernel."""
    from agave_b200 import kernels
    lens = [1, 63, 64, 65, 200, 130]
    T, B = sum(lens), len(lens)
    width = (nh + 2 * nkv) * hd
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    positions = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32, device=DEV)
    seq_index = torch.tensor(sum([[i] * n for i, n in enumerate(lens)], []), dtype=torch.int32, device=DEV)
    if splits:
        part = rnd(splits, T, width, seed=4, scale=0.5)
        qkv = torch.empty(T, width, dtype=torch.bfloat16, device=DEV)
        want_v = part.sum(0)[:, (nh + nkv) * hd:].to(torch.bfloat16)
    else:
        part = None
        qkv = rnd(T, width, dtype=torch.bfloat16, seed=4, scale=0.5)
        want_v = qkv[:, (nh + nkv) * hd:].clone()
    vt = kernels.prefill_values_scratch(T, B, nkv, hd, DEV)
    vt.fill_(float("nan"))
    kernels.qk_norm_rope_store(qkv, nh, nkv, hd, None, None, 0.0, None, None, 0, positions,
                               seq_index=seq_index, partial=part, vt=vt, cu_seqlens=cu,
                               max_len=max(lens))
    start = 0
    for b, n in enumerate(lens):
        o = int(cu[b])
        padded = (n + 63) // 64 * 64
        got = vt[:, start:start + padded].float()
        assert torch.equal(got[:, :n], want_v[o:o + n].float().t()), b
        assert (got[:, n:] == 0).all(), b
        start += padded
    assert torch.equal(qkv[:, (nh + nkv) * hd:].float(), want_v.float())


def test_attention_prefill_tensor_cores_far_key_and_window_edge():
    from agave_b200 import kernels
    hd, n, far = 256, 300, 3
    k = rnd(n, hd, dtype=torch.bfloat16, seed=1, scale=0.1)
    v = rnd(n, hd, dtype=torch.bfloat16, seed=2)
    q = rnd(n, hd, dtype=torch.bfloat16, seed=3, scale=0.1)
    k[far] = 0; k[far, 0] = 40.0
    q[-1] = 0; q[-1, 0] = 40.0
    qkv = torch.cat([q, k, v], dim=1).contiguous()
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    out = torch.empty((n, hd), dtype=torch.bfloat16, device=DEV)
    args = (qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], out, cu, n, 1, 1, hd, 1.0)
    kernels.attention_prefill_mma(*args, 0)
    assert rel_err(out[-1], v[far]) < 1e-2
    kernels.attention_prefill_mma(*args, n - far)
    assert rel_err(out[-1], v[far]) < 1e-2
    kernels.attention_prefill_mma(*args, n - far - 1)
    assert (out[-1].float() - v[far].float()).abs().max() > 0.1
