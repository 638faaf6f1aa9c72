"""Each CUDA kernel alone against a plain 32-bit reference of the same operation, at sizes other
than the engine tests use (widths and vocabularies that are no power of two, head sizes in
steps of 16, several group sizes).  Where random inputs would hide a fault, the inputs are
made so that it shows: one key that dominates the softmax far back in a long context, at a
window's edge or on either side of a page's edge."""
import math

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from llmengine_b200.kernels.ops import CudaOps
    return CudaOps(torch.device(DEV))


@pytest.fixture(params=["two blocks an SM", "three blocks an SM", "as the kernel chooses"])
def skinny(ops, request):
    """The weight-streaming product also for shapes that the executor's own choice would give to the library, in its
    form with two blocks an SM, in its lighter form with three (up to 8 tokens), and as it chooses itself."""
    ops.choose("linear.decode", "skinny")
    ops.gemm_skinny_form({"two blocks an SM": "two", "three blocks an SM": "three", "as the kernel chooses": "auto"}[request.param])
    yield ops
    ops.gemm_skinny_form("auto")
    ops.choose("linear.decode", "auto")


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ----------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,vocab", [(72, 301), (1000, 77), (4096, 513)])
def test_embedding(ops, dtype, hidden, vocab):
    table = _rand(vocab, hidden, dtype=dtype, seed=1)
    ids = torch.randint(0, vocab, (37,), generator=torch.Generator().manual_seed(2)).to(torch.int32).to(DEV)
    out = torch.empty(37, hidden, device=DEV)
    ops.embedding(ids, table, out)
    want = pm.embedding(table.cpu().float(), ids.cpu().tolist())
    assert torch.equal(out.cpu(), want)


# ----------------------------------------------------------------------------- rmsnorm
@pytest.mark.parametrize("hidden", [48, 96, 1000, 4096, 5120])
@pytest.mark.parametrize("gain_dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                                  (torch.float32, torch.bfloat16)])
def test_rmsnorm(ops, hidden, gain_dtype, out_dtype):
    eps = 3e-6
    x = _rand(19, hidden, seed=3, scale=2.0)
    gain = (1 + 0.1 * _rand(hidden, seed=4)).to(gain_dtype)
    out = torch.empty(19, hidden, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, gain, eps, out)
    want = pm.rms_norm(x.cpu(), gain.cpu().float(), eps)
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    assert (out.cpu().float() - want).abs().max() < tol
    if out_dtype == torch.bfloat16:      # rounding is the only difference
        assert (out.cpu().float() - want.to(torch.bfloat16).float()).abs().max() <= 0.016 * want.abs().max()


@pytest.mark.parametrize("delta_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_adds_delta_and_selects_rows(ops, delta_dtype):
    hidden, eps = 200, 1e-5
    x = _rand(23, hidden, seed=5)
    delta = _rand(23, hidden, seed=6).to(delta_dtype)
    gain = 1 + 0.1 * _rand(hidden, seed=7)
    x0 = x.clone()
    out = torch.empty(23, hidden, device=DEV)
    ops.rmsnorm(x, gain, eps, out, delta=delta)
    total = x0.cpu() + delta.cpu().float()
    assert torch.allclose(x.cpu(), total, atol=0, rtol=0), "the sum must be stored back into the residual stream"
    assert (out.cpu() - pm.rms_norm(total, gain.cpu(), eps)).abs().max() < 1e-5
    rows = torch.tensor([22, 0, 7], dtype=torch.int32, device=DEV)
    x2 = x0.clone()
    out2 = torch.empty(3, hidden, device=DEV)
    ops.rmsnorm(x2, gain, eps, out2, delta=delta, rows=rows)
    assert (out2.cpu() - pm.rms_norm(total[[22, 0, 7]], gain.cpu(), eps)).abs().max() < 1e-5


# ----------------------------------------------------------------------------- swiglu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [56, 1000, 12288])
def test_swiglu(ops, dtype, inter):
    gu = _rand(9, 2 * inter, dtype=dtype, seed=8, scale=3.0)
    out = torch.empty(9, inter, dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    f = gu.cpu().float()
    want = pm.swiglu(f[:, :inter], f[:, inter:])
    if dtype == torch.float32:
        assert (out.cpu() - want).abs().max() < 1e-5
    else:                                 # one rounding of the result to bfloat16
        assert ((out.cpu().float() - want).abs() <= want.abs() * 2 ** -8 + 1e-6).all()


# ----------------------------------------------------------------------------- 32-bit matrix product
@pytest.mark.parametrize("M,N,K", [(1, 130, 70), (7, 64, 64), (65, 129, 257), (200, 1000, 96), (33, 48, 4096)])
def test_gemm_f32_is_true_32bit(ops, M, N, K):
    a = _rand(M, K, seed=9)
    w = _rand(N, K, seed=10)
    out = torch.empty(M, N, device=DEV)
    ops.linear(a, w, out)
    want = a.cpu().double() @ w.cpu().double().t()
    err = (out.cpu().double() - want).abs().max().item()
    # a product in a reduced-precision mode would be off by ~1e-3 * sqrt(K); true 32-bit stays near 1e-6 * sqrt(K)
    assert err < 2e-6 * math.sqrt(K) * 4, err


def test_gemm_f32_rows_do_not_depend_on_the_batch(ops):
    a = _rand(100, 300, seed=11)
    w = _rand(77, 300, seed=12)
    full = torch.empty(100, 77, device=DEV)
    ops.linear(a, w, full)
    one = torch.empty(1, 77, device=DEV)
    for r in (0, 63, 64, 99):
        ops.linear(a[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (8, 1000, 96), (130, 520, 264)])
def test_linear_bf16(ops, M, N, K):
    a = _rand(M, K, dtype=torch.bfloat16, seed=13)
    w = _rand(N, K, dtype=torch.bfloat16, seed=14)
    want = a.cpu().float() @ w.cpu().float().t()
    out32 = torch.empty(M, N, device=DEV)
    ops.linear(a, w, out32)
    assert (out32.cpu() - want).abs().max() < 1e-3 * math.sqrt(K)
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, out16)
    assert (out16.cpu().float() - want).abs().max() < 0.02 * want.abs().max()


@pytest.mark.parametrize("M,N,K", [(7, 576, 161), (12, 543, 119), (16, 543, 160), (17, 543, 4096), (64, 543, 4100),
                                   (33, 80, 4100), (5, 1131, 119)])
def test_linear_bf16_sums_in_32bit_whatever_the_shape(ops, M, N, K):
    """Products that go to the library (a width that is no multiple of 8, or 17 to 127 tokens): every output is
    within a few bfloat16 steps of the exact value, also where the library, left to itself, adds partial sums
    in bfloat16 (a few tokens and odd sizes: a thousand steps off)."""
    a = _rand(M, K, dtype=torch.bfloat16, seed=15)
    w = _rand(N, K, dtype=torch.bfloat16, seed=16, scale=0.1)
    want = (a.double() @ w.double().t()).cpu()
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, out16)
    # 32-bit accumulation of K products of size |a||w|, then one rounding to bfloat16
    sums = (a.double().abs() @ w.double().abs().t()).cpu()
    assert ((out16.double().cpu() - want).abs() <= want.abs() * 2 ** -8 + sums * 2e-6).all()
    out32 = torch.empty(M, N, device=DEV)
    ops.linear(a, w, out32)
    assert ((out32.double().cpu() - want).abs() <= sums * 2e-6).all()


@pytest.fixture(params=["single", "pair"])
def pairing(ops, request):
    """The tcgen05 product on single SMs (128-row tiles) and on pairs of SMs (tcgen05 with .cta_group::2, 256-row
    tiles, each block loading half of the tile's rows of W), whatever the size."""
    ops.gemm_tc_pairing(request.param)
    yield request.param
    ops.gemm_tc_pairing("auto")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 72), (129, 257, 264), (300, 1000, 96), (2048, 520, 1024),
                                   (1000, 4096, 4096), (257, 24, 8), (1, 8, 8), (255, 136, 40), (513, 1032, 200)])
def test_tcgen05_gemm(ops, pairing, M, N, K, out_dtype):
    """The prompt-portion product on the tcgen05 tensor cores: tiles that hang over every edge, one and
    many k blocks, more tiles than SMs."""
    a = _rand(M, K, dtype=torch.bfloat16, seed=50)
    w = _rand(N, K, dtype=torch.bfloat16, seed=51, scale=0.05)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear_tc(a, w, out)
    assert ops.linear_tc_status() == 0, "a bounded wait gave up"
    want = (a.double() @ w.double().t()).cpu()
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    tol = 2e-5 * math.sqrt(K) * float(want.abs().max() + 1)
    if out_dtype == torch.bfloat16:
        assert ((got - want).abs() <= want.abs() * 2 ** -8 + tol).all()
    else:
        assert (got - want).abs().max() < tol


def test_tcgen05_gemm_into_a_strided_unaligned_output(ops, pairing):
    """An output whose rows do not start on 16-byte boundaries takes the register-store epilogue."""
    a = _rand(200, 128, dtype=torch.bfloat16, seed=52)
    w = _rand(77, 128, dtype=torch.bfloat16, seed=53)
    buf = torch.zeros(200, 81, device=DEV)
    ops.linear_tc(a, w, buf[:, 1:78])
    assert ops.linear_tc_status() == 0
    want = (a.double() @ w.double().t()).cpu()
    assert (buf[:, 1:78].double().cpu() - want).abs().max() < 1e-3
    assert buf[:, 0].abs().max() == 0 and buf[:, 78:].abs().max() == 0


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (8, 6144, 4096), (3, 100, 72), (16, 1000, 264), (9, 33, 8),
                                   (5, 24576, 512), (2, 151936, 128), (8, 4096, 12288), (8, 7168, 5120), (8, 5120, 17408),
                                   (13, 1000, 2120), (2, 100, 2624), (17, 4096, 4096), (32, 1000, 264)])
def test_skinny_gemm(ops, skinny, M, N, K, out_dtype):
    """The decode-step product (at most 16 tokens run this package's kernel, more the library's): rows and widths that are
    no multiple of the tiles, K with every kind of remainder."""
    a = _rand(M, K, dtype=torch.bfloat16, seed=40)
    w = _rand(N, K, dtype=torch.bfloat16, seed=41, scale=0.05)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear(a, w, out)
    want = (a.double() @ w.double().t()).cpu()
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    tol = 2e-5 * math.sqrt(K) * float(want.abs().max() + 1)
    if out_dtype == torch.bfloat16:
        assert ((got - want).abs() <= want.abs() * 2 ** -8 + tol).all()
    else:
        assert (got - want).abs().max() < tol


def test_skinny_gemm_rows_do_not_depend_on_the_batch(ops, skinny):
    a = _rand(16, 1096, dtype=torch.bfloat16, seed=42)
    w = _rand(300, 1096, dtype=torch.bfloat16, seed=43)
    full = torch.empty(16, 300, device=DEV)
    ops.linear(a, w, full)
    for m in (1, 7, 8, 9):
        part = torch.empty(m, 300, device=DEV)
        ops.linear(a[:m].contiguous(), w, part)
        assert torch.equal(part, full[:m])


@pytest.mark.parametrize("M,inter,K", [(8, 12288, 4096), (1, 3072, 1024), (16, 100, 72), (3, 8, 8), (11, 5000, 264), (7, 20, 520),
                                       (8, 17408, 5120), (5, 100, 2120)])
def test_skinny_gemm_with_swiglu(ops, skinny, M, inter, K):
    """Product and activation in one kernel against the product followed by the activation kernel (the same
    arithmetic, so the same bits) and against 64-bit arithmetic."""
    a = _rand(M, K, dtype=torch.bfloat16, seed=46)
    w = _rand(2 * inter, K, dtype=torch.bfloat16, seed=47, scale=0.08)
    fused = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(a, w, fused)
    gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, gate_up)
    two = torch.empty(M, inter, dtype=torch.bfloat16, device=DEV)
    ops.swiglu(gate_up, two)
    assert torch.equal(fused, two)
    y = a.double() @ w.double().t()
    g, u = y[:, :inter], y[:, inter:]
    want = (g / (1 + torch.exp(-g)) * u).cpu()
    got = fused.double().cpu()
    assert torch.isfinite(got).all()
    # gate and up pass through bfloat16 (a relative 2^-9 each; |d silu / d gate| <= 1.1), and so may the result
    tol = 2e-5 * math.sqrt(K) * float(want.abs().max() + 1)
    bound = (1.1 * (g.abs() * u.abs()).cpu() + 2 * want.abs()) * 2 ** -8 + tol
    assert ((got - want).abs() <= bound).all()


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(2048, 4096, 4096), (2048, 2560, 520), (1500, 3000, 72), (2048, 6144, 264), (130, 40000, 128)])
def test_tcgen05_gemm_more_tiles_than_sms(ops, pairing, M, N, K, out_dtype):
    """More tiles than SMs and not a multiple of them: a block walks over several tiles, the last wave is partly
    empty, both accumulator buffers are in use.  The same bits every time."""
    a = _rand(M, K, dtype=torch.bfloat16, seed=54)
    w = _rand(N, K, dtype=torch.bfloat16, seed=55, scale=0.05)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear_tc(a, w, out)
    assert ops.linear_tc_status() == 0
    want = (a.double() @ w.double().t()).cpu()
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    tol = 2e-5 * math.sqrt(K) * float(want.abs().max() + 1)
    if out_dtype == torch.bfloat16:
        assert ((got - want).abs() <= want.abs() * 2 ** -8 + tol).all()
    else:
        assert (got - want).abs().max() < tol
    for _ in range(2):
        again = torch.full_like(out, float("nan"))
        ops.linear_tc(a, w, again)
        assert torch.equal(again, out)


@pytest.mark.parametrize("M,inter,K", [(2048, 12288, 4096), (128, 128, 64), (300, 1000, 264), (129, 72, 520), (1000, 136, 8)])
def test_tcgen05_gemm_with_swiglu(ops, monkeypatch, pairing, M, inter, K):
    """The tcgen05 product with the activation in its epilogue against the product followed by the activation
    kernel, and against 64-bit arithmetic; widths that end inside a tile."""
    monkeypatch.setattr(ops, "plain_gemm", "tcgen05")     # also at sizes that the product path gives to cuBLAS
    a = _rand(M, K, dtype=torch.bfloat16, seed=48)
    w = _rand(2 * inter, K, dtype=torch.bfloat16, seed=49, scale=0.08)
    fused = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.linear_swiglu_supports(a, w, fused)
    ops.linear_swiglu(a, w, fused)
    assert ops.linear_tc_status() == 0
    gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(a, w, gate_up)
    two = torch.empty(M, inter, dtype=torch.bfloat16, device=DEV)
    ops.swiglu(gate_up, two)
    assert torch.equal(fused, two)
    y = a.double() @ w.double().t()
    g, u = y[:, :inter], y[:, inter:]
    want = (g / (1 + torch.exp(-g)) * u).cpu()
    got = fused.double().cpu()
    assert torch.isfinite(got).all()
    tol = 2e-5 * math.sqrt(K) * float(want.abs().max() + 1)
    bound = (1.1 * (g.abs() * u.abs()).cpu() + 2 * want.abs()) * 2 ** -8 + tol
    assert ((got - want).abs() <= bound).all()


# ----------------------------------------------------------------------------- QK norm + rope + cache write
def _paged_layout(T, page_size, num_pages, seed):
    """Scatter T consecutive positions over pages in a scrambled order."""
    g = torch.Generator().manual_seed(seed)
    blocks = torch.randperm(num_pages, generator=g)[: -(-T // page_size)]
    pos = torch.arange(T)
    slots = blocks[pos // page_size] * page_size + pos % page_size
    return blocks.to(torch.int32), slots.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 8), (6, 3, 48, 16), (8, 1, 80, 4), (32, 8, 128, 16), (2, 2, 256, 32)])
def test_qkv_post(ops, dtype, nh, nkv, hd, page):
    _check_qkv_post(ops, dtype, nh, nkv, hd, page, 29, torch.float32)


@pytest.mark.parametrize("dtype,gain_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                              (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("nh,nkv,hd,page,T", [(32, 8, 128, 64, 1001), (5, 1, 64, 16, 3000), (3, 3, 32, 8, 2500),
                                              (2, 1, 256, 32, 4003), (6, 3, 48, 16, 4500), (7, 7, 128, 128, 700)])
def test_qkv_post_many_tokens(ops, dtype, gain_dtype, nh, nkv, hd, page, T):
    """The kernels that a prompt portion takes (a warp per token and run of heads for bfloat16 with a head size
    of 32, 64, 128 or 256, else a warp per head of four tokens): head counts that end inside a warp's run,
    token counts that end inside a block."""
    _check_qkv_post(ops, dtype, nh, nkv, hd, page, T, gain_dtype)


def _check_qkv_post(ops, dtype, nh, nkv, hd, page, T, gain_dtype):
    from llmengine_b200.parts.position import RotaryEncoding
    eps, theta, maxpos = 2e-6, 12345.0, T + 300
    qs, kvs = nh * hd, nkv * hd
    qkv = _rand(T, qs + 2 * kvs, dtype=dtype, seed=15)
    qg = (1 + 0.1 * _rand(hd, seed=16)).to(gain_dtype)
    kg = (1 + 0.1 * _rand(hd, seed=17)).to(gain_dtype)
    table = RotaryEncoding.build_table(hd, theta, maxpos).to(DEV)
    positions = (torch.arange(T) + 200).to(torch.int32).to(DEV)
    num_pages = -(-T // page) + 11
    blocks, slots = _paged_layout(T, page, num_pages, 18)
    slots[5] = -1                                     # a token that is not stored
    cache = torch.zeros(num_pages, 2, nkv, page, hd, dtype=dtype, device=DEV)
    q_out = torch.empty(T, qs, dtype=dtype, device=DEV)
    ops.qkv_post(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs], v_in=qkv[:, qs + kvs:], num_heads=nh, num_kv_heads=nkv,
                 head_dim=hd, q_gain=qg, k_gain=kg, eps=eps, cos_sin=table, positions=positions, q_out=q_out,
                 cache=cache, slot_mapping=slots.to(DEV), page_size=page)
    f = qkv.cpu().float()
    pos = positions.cpu()
    q_want = pm.rope(pm.qk_norm(f[:, :qs].view(T, nh, hd), qg.cpu().float(), eps), pos, theta).reshape(T, qs)
    k_want = pm.rope(pm.qk_norm(f[:, qs:qs + kvs].view(T, nkv, hd), kg.cpu().float(), eps), pos, theta)
    v_want = f[:, qs + kvs:].view(T, nkv, hd)
    tol = 2e-5 if dtype == torch.float32 else 0.04
    assert (q_out.cpu().float() - q_want).abs().max() < tol
    c = cache.cpu().float().permute(0, 3, 1, 2, 4).reshape(num_pages * page, 2, nkv, hd)     # [slot, k|v, head, hd]
    stored = slots >= 0
    idx = slots[stored].long()
    assert (c[idx, 0] - k_want[stored]).abs().max() < tol
    assert torch.equal(c[idx, 1], v_want[stored])
    untouched = torch.ones(num_pages * page, dtype=torch.bool)
    untouched[idx] = False
    assert c[untouched].abs().max() == 0, "a cache row that no token maps to was written"


# ----------------------------------------------------------------------------- attention
def _attention_case(nh, nkv, hd, page, ctx_lens, q_lens, window, dtype, seed, spike=None):
    """Builds a paged cache holding `ctx_lens[r]` keys per request and queries for the last
    `q_lens[r]` positions of each.  Returns kernel inputs and the plain result.
    `spike = (request, key position)`: that key is aligned with the request's last query and
    scaled so that it takes nearly all of the softmax weight."""
    R = len(ctx_lens)
    g = torch.Generator().manual_seed(seed)
    num_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    max_blocks = max(-(-c // page) for c in ctx_lens) + 1
    tables = torch.full((R + 2, max_blocks), -1, dtype=torch.int32)
    cache = torch.full((num_pages, 2, nkv, page, hd), float("nan"))       # unwritten rows stay NaN
    ks, vs, qs = [], [], []
    for r, c in enumerate(ctx_lens):
        k = torch.randn(c, nkv, hd, generator=g)
        v = torch.randn(c, nkv, hd, generator=g)
        q = torch.randn(c, nh, hd, generator=g)
        if spike is not None and spike[0] == r:
            j = spike[1]
            grp = nh // nkv
            for kvh in range(nkv):          # score of key j becomes ~2*sqrt(hd) for every query head, others ~N(0,1)
                k[j, kvh] = 2.0 * q[c - 1, kvh * grp:(kvh + 1) * grp].sum(0)
        ks.append(k), vs.append(v), qs.append(q)
        row = r + 1                                                        # table rows need not be 0..R-1
        for b in range(-(-c // page)):
            p = perm.pop()
            tables[row, b] = p
            n = min(page, c - b * page)
            cache[p, 0, :, :n] = k[b * page:b * page + n].transpose(0, 1)
            cache[p, 1, :, :n] = v[b * page:b * page + n].transpose(0, 1)
    cache = cache.to(dtype)
    q_rows, positions, token_req, want = [], [], [], []
    for r, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        kf = cache_round(ks[r], dtype)
        vf = cache_round(vs[r], dtype)
        qf = cache_round(qs[r], dtype)
        full = pm.attention(qf, kf, vf, window)
        for p in range(c - n, c):
            q_rows.append(qf[p].reshape(-1))
            positions.append(p)
            token_req.append(r + 1)
            want.append(full[p].reshape(-1))
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    return dict(
        cu_q_lens=torch.tensor(cu, dtype=torch.int32, device=DEV),
        ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
        table_rows=torch.arange(1, R + 1, dtype=torch.int32, device=DEV),
        q=torch.stack(q_rows).to(dtype).to(DEV), cache=cache.to(DEV),
        positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
        token_request=torch.tensor(token_req, dtype=torch.int32, device=DEV),
        block_tables=tables.to(DEV), want=torch.stack(want))


def cache_round(x, dtype):
    return x.to(dtype).float()


ATTN_SHAPES = [(4, 2, 16, 8), (6, 3, 48, 16), (8, 1, 80, 4), (8, 2, 128, 16), (3, 3, 32, 16), (16, 4, 64, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", ATTN_SHAPES)
@pytest.mark.parametrize("window", [0, 13])
def test_attention_plain_mixed_batch(ops, dtype, nh, nkv, hd, page, window):
    case = _attention_case(nh, nkv, hd, page, ctx_lens=[1, 37, 64, 150], q_lens=[1, 37, 1, 9], window=window,
                           dtype=dtype, seed=20)
    out = torch.empty_like(case["q"])
    ops.attention_plain(q=case["q"], cache=case["cache"], out=out, positions=case["positions"],
                        token_request=case["token_request"], block_tables=case["block_tables"], num_heads=nh,
                        num_kv_heads=nkv, head_dim=hd, page_size=page, window=window, scale=1 / math.sqrt(hd))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.isfinite(out).all()
    assert (out.cpu().float() - case["want"]).abs().max() < tol


@pytest.mark.parametrize("where", ["far_back", "page_last", "page_first", "window_inside", "window_outside"])
def test_attention_plain_finds_the_one_key_that_matters(ops, where):
    nh, nkv, hd, page, ctx, window = 8, 2, 64, 16, 700, 0
    key = {"far_back": 3, "page_last": 16 * 20 - 1, "page_first": 16 * 20}.get(where)
    if where.startswith("window"):
        window = 100
        key = ctx - 100 if where == "window_inside" else ctx - 101       # query at ctx-1 sees keys > ctx-1-100
    case = _attention_case(nh, nkv, hd, page, [ctx], [1], window, torch.float32, 21, spike=(0, key))
    out = torch.empty_like(case["q"])
    ops.attention_plain(q=case["q"], cache=case["cache"], out=out, positions=case["positions"],
                        token_request=case["token_request"], block_tables=case["block_tables"], num_heads=nh,
                        num_kv_heads=nkv, head_dim=hd, page_size=page, window=window, scale=1 / math.sqrt(hd))
    assert (out.cpu() - case["want"]).abs().max() < 2e-5


def _run_fast(ops, case, nh, nkv, hd, page, window, q_lens, splits=None):
    out = torch.full_like(case["q"], float("nan"))
    common = dict(q=case["q"], cache=case["cache"], out=out, cu_q_lens=case["cu_q_lens"], ctx_lens=case["ctx_lens"],
                  table_rows=case["table_rows"], block_tables=case["block_tables"], num_heads=nh, num_kv_heads=nkv,
                  head_dim=hd, page_size=page, window=window, scale=1 / math.sqrt(hd))
    dec = [r for r, n in enumerate(q_lens) if n == 1]
    por = [r for r, n in enumerate(q_lens) if n != 1]
    if por:
        ops.attention_portions(rows=torch.tensor(por, dtype=torch.int32, device=DEV), max_q_len=max(q_lens), **common)
    if dec:
        sp = splits or 3
        need = ops.attention_decode_scratch_floats(hd, len(dec), nh, sp)
        scratch = torch.full((max(need, 1),), float("nan"), device=DEV)
        scratch[:65536] = 0                       # the ticket counters start at zero; the rest may hold anything
        ops.attention_decode(rows=torch.tensor(dec, dtype=torch.int32, device=DEV), splits=sp, scratch=scratch, **common)
    return out


FAST_SHAPES = [(4, 2, 16, 8), (6, 3, 48, 16), (8, 1, 80, 4), (8, 2, 128, 16), (3, 3, 32, 16), (16, 4, 64, 32),
               (40, 2, 64, 16), (32, 8, 128, 16)]


@pytest.mark.parametrize("nh,nkv,hd,page", FAST_SHAPES)
@pytest.mark.parametrize("window", [0, 13, 100])
def test_attention_fast_mixed_batch(ops, nh, nkv, hd, page, window):
    """Portions of several lengths (one request whole, one deep into its context, one of two tokens)
    beside single decoded tokens, in one batch; unwritten cache rows hold NaN."""
    ctx_lens = [1, 37, 64, 150, 333, 65, 700]
    q_lens = [1, 37, 1, 9, 200, 2, 1]
    case = _attention_case(nh, nkv, hd, page, ctx_lens, q_lens, window, torch.bfloat16, 30)
    out = _run_fast(ops, case, nh, nkv, hd, page, window, q_lens)
    assert torch.isfinite(out).all()
    assert (out.cpu().float() - case["want"]).abs().max() < 2e-2


TC_SHAPES = [(8, 2, 128, 16), (32, 8, 128, 16), (4, 4, 64, 8), (16, 2, 64, 32), (2, 1, 128, 128), (8, 8, 128, 64)]


@pytest.mark.parametrize("nh,nkv,hd,page", TC_SHAPES)
@pytest.mark.parametrize("window", [0, 100])
def test_attention_tcgen05_portions(ops, nh, nkv, hd, page, window):
    """The tcgen05 portion kernel: portions that start deep inside a context, end on and off page and tile
    edges, a two-token portion, requests of very different length in one launch; unwritten cache rows hold NaN."""
    ctx_lens = [37, 150, 333, 65, 700, 128, 257]
    q_lens = [37, 9, 200, 2, 300, 128, 129]
    assert ops.tc_attention_supports(hd, torch.bfloat16, nh, nkv, page)
    case = _attention_case(nh, nkv, hd, page, ctx_lens, q_lens, window, torch.bfloat16, 33)
    out = torch.full_like(case["q"], float("nan"))
    ops.attention_portions_tc(q=case["q"], cache=case["cache"], out=out, rows=torch.arange(len(q_lens), dtype=torch.int32, device=DEV),
                              cu_q_lens=case["cu_q_lens"], ctx_lens=case["ctx_lens"], table_rows=case["table_rows"],
                              block_tables=case["block_tables"], num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                              page_size=page, window=window, scale=1 / math.sqrt(hd), max_q_len=max(q_lens))
    assert ops.attention_tc_status(hd) == 0, "a bounded wait gave up"
    assert torch.isfinite(out).all()
    assert (out.cpu().float() - case["want"]).abs().max() < 2e-2


@pytest.mark.parametrize("where", ["far_back", "page_last", "page_first", "tile_last", "tile_first", "window_inside",
                                   "window_outside"])
def test_attention_tcgen05_finds_the_one_key_that_matters(ops, where):
    nh, nkv, hd, page, ctx, window = 8, 2, 128, 16, 700, 0
    key = {"far_back": 3, "page_last": 16 * 20 - 1, "page_first": 16 * 20, "tile_last": 128 * 3 - 1,
           "tile_first": 128 * 3}.get(where)
    if where.startswith("window"):
        window = 100
        key = ctx - 100 if where == "window_inside" else ctx - 101
    case = _attention_case(nh, nkv, hd, page, [ctx], [40], window, torch.bfloat16, 34, spike=(0, key))
    out = torch.full_like(case["q"], float("nan"))
    ops.attention_portions_tc(q=case["q"], cache=case["cache"], out=out, rows=torch.zeros(1, dtype=torch.int32, device=DEV),
                              cu_q_lens=case["cu_q_lens"], ctx_lens=case["ctx_lens"], table_rows=case["table_rows"],
                              block_tables=case["block_tables"], num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                              page_size=page, window=window, scale=1 / math.sqrt(hd), max_q_len=40)
    assert ops.attention_tc_status(hd) == 0
    assert (out.cpu().float() - case["want"]).abs().max() < 2e-2


@pytest.mark.parametrize("splits", [1, 2, 7, 64])
def test_attention_decode_any_number_of_splits(ops, splits):
    nh, nkv, hd, page = 8, 2, 128, 16
    ctx_lens, q_lens = [5, 64, 65, 1000], [1, 1, 1, 1]
    case = _attention_case(nh, nkv, hd, page, ctx_lens, q_lens, 0, torch.bfloat16, 31)
    out = _run_fast(ops, case, nh, nkv, hd, page, 0, q_lens, splits=splits)
    assert torch.isfinite(out).all()
    assert (out.cpu().float() - case["want"]).abs().max() < 2e-2


@pytest.mark.parametrize("splits", [1, 3])
def test_attention_decode_long_context_small_pages(ops, splits):
    """More block-table entries in a block's share than it keeps in shared memory (it then reads them from
    global memory), and a far key that matters."""
    nh, nkv, hd, page = 4, 2, 64, 8
    ctx_lens, q_lens = [9000, 4500], [1, 1]
    case = _attention_case(nh, nkv, hd, page, ctx_lens, q_lens, 0, torch.bfloat16, 35, spike=(0, 11))
    out = _run_fast(ops, case, nh, nkv, hd, page, 0, q_lens, splits=splits)
    assert torch.isfinite(out).all()
    assert (out.cpu().float() - case["want"]).abs().max() < 2e-2


@pytest.mark.parametrize("splits", [1, 4, 16])
@pytest.mark.parametrize("hd,page,norm,rope", [(128, 64, "bf16", True), (64, 16, "f32", True), (128, 16, None, True),
                                               (32, 8, "bf16", False), (128, 128, None, False)])
def test_attention_decode_on_raw_projections(ops, hd, page, norm, rope, splits):
    """The decode kernel that norms, rotates and stores the new token's heads itself, against the kernel of
    elementwise.cu followed by the decode kernel: the same cache contents (to the last bfloat16 digit or one
    off, where a fused multiply-add rounds differently) and the same outputs."""
    from llmengine_b200.parts.position import RotaryEncoding
    nh, nkv = 8, 2
    ctx_lens = [1, 17, page, page + 1, 300, 64]
    R = len(ctx_lens)
    g = torch.Generator().manual_seed(77)
    blocks = [-(-c // page) for c in ctx_lens]
    num_pages = sum(blocks) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    tables = torch.zeros(R, max(blocks) + 1, dtype=torch.int32)
    cache = torch.full((num_pages, 2, nkv, page, hd), float("nan"))
    slots = []
    for r, c in enumerate(ctx_lens):
        for b in range(blocks[r]):
            tables[r, b] = perm.pop()
        for j in range(c - 1):                                   # everything but the new token is in the cache
            cache[tables[r, j // page], :, :, j % page] = torch.randn(2, nkv, hd, generator=g)
        slots.append(int(tables[r, (c - 1) // page]) * page + (c - 1) % page)
    cache = cache.to(torch.bfloat16).to(DEV)
    qkv = torch.randn(R, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16).to(DEV)
    gains = None
    if norm:
        dt = torch.bfloat16 if norm == "bf16" else torch.float32
        gains = [(1 + 0.1 * torch.randn(hd, generator=g)).to(dt).to(DEV) for _ in range(2)]
    table = RotaryEncoding.build_table(hd, 10000.0, 512).to(DEV) if rope else None
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, slot_mapping = dev([c - 1 for c in ctx_lens]), dev(slots)
    meta = dict(rows=dev(list(range(R))), cu_q_lens=dev(list(range(R + 1))), ctx_lens=dev(ctx_lens), table_rows=dev(list(range(R))),
                block_tables=tables.to(DEV), num_heads=nh, num_kv_heads=nkv, head_dim=hd, page_size=page, window=0,
                scale=1 / math.sqrt(hd), splits=splits)
    need = ops.attention_decode_scratch_floats(hd, R, nh, splits) if splits > 1 else 1
    qs, kvs = nh * hd, nkv * hd
    # two kernels
    cache_a, q = cache.clone(), torch.empty(R, qs, dtype=torch.bfloat16, device=DEV)
    ops.qkv_post(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs], v_in=qkv[:, qs + kvs:], num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                 q_gain=gains[0] if gains else None, k_gain=gains[1] if gains else None, eps=1e-6 if gains else 0.0,
                 cos_sin=table, positions=positions, q_out=q, cache=cache_a, slot_mapping=slot_mapping, page_size=page)
    out_a = torch.full((R, qs), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(q=q, cache=cache_a, out=out_a, scratch=torch.zeros(need, device=DEV) if splits > 1 else None, **meta)
    # one kernel
    cache_b = cache.clone()
    out_b = torch.full((R, qs), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_decode_fused(qkv=qkv, q_gain=gains[0] if gains else None, k_gain=gains[1] if gains else None,
                               eps=1e-6 if gains else 0.0, cos_sin=table, write_kv=True, cache=cache_b, out=out_b,
                               scratch=torch.zeros(need, device=DEV) if splits > 1 else None, **meta)
    a, b = cache_a.float().cpu(), cache_b.float().cpu()
    assert torch.equal(torch.isnan(a), torch.isnan(b)), "exactly the new tokens' rows are written"
    a, b = torch.nan_to_num(a), torch.nan_to_num(b)
    assert ((a - b).abs() <= a.abs() * 2 ** -7 + 1e-6).all()
    assert torch.isfinite(out_b.float()).all()
    assert (out_a.float() - out_b.float()).abs().max() < 2e-2
    # nothing is stored when the layer reads another layer's cache
    cache_c = cache_a.clone()
    ops.attention_decode_fused(qkv=qkv[:, :qs], q_gain=gains[0] if gains else None, k_gain=gains[1] if gains else None,
                               eps=1e-6 if gains else 0.0, cos_sin=table, write_kv=False, cache=cache_c, out=out_b,
                               scratch=torch.zeros(need, device=DEV) if splits > 1 else None, **meta)
    assert torch.equal(torch.nan_to_num(cache_c.float()), torch.nan_to_num(cache_a.float()))
    assert (out_a.float() - out_b.float()).abs().max() < 2e-2


@pytest.mark.parametrize("q_len", [1, 40])
@pytest.mark.parametrize("where", ["far_back", "page_last", "page_first", "tile_last", "tile_first", "window_inside",
                                   "window_outside"])
def test_attention_fast_finds_the_one_key_that_matters(ops, where, q_len):
    nh, nkv, hd, page, ctx, window = 8, 2, 64, 16, 700, 0
    key = {"far_back": 3, "page_last": 16 * 20 - 1, "page_first": 16 * 20, "tile_last": 64 * 5 - 1,
           "tile_first": 64 * 5}.get(where)
    if where.startswith("window"):
        window = 100
        key = ctx - 100 if where == "window_inside" else ctx - 101
    case = _attention_case(nh, nkv, hd, page, [ctx], [q_len], window, torch.bfloat16, 32, spike=(0, key))
    out = _run_fast(ops, case, nh, nkv, hd, page, window, [q_len], splits=4)
    assert (out.cpu().float() - case["want"]).abs().max() < 2e-2


# ----------------------------------------------------------------------------- sampling
def _sample(ops, logits, **kw):
    R = logits.shape[0]
    dev = lambda v, dt: torch.tensor(v, dtype=dt, device=DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, greedy=dev(kw["greedy"], torch.int32), temperature=dev(kw["temperature"], torch.float32),
               top_k=dev(kw["top_k"], torch.int32), top_p=dev(kw["top_p"], torch.float32),
               u=dev(kw["u"], torch.float32), out=out)
    return out.cpu().tolist()


@pytest.mark.parametrize("vocab", [77, 1000, 151936])
def test_sample_greedy_is_first_argmax(ops, vocab):
    logits = _rand(5, vocab, seed=22)
    logits[1, 10] = logits[1, 40] = 50.0           # a tie: the first one wins
    logits[2] = float("-inf")                      # src/runtime/sampler.cpp:41-47: uniform, token 0
    got = _sample(ops, logits, greedy=[1] * 5, temperature=[1.0, 0.5, 1.0, 0.0, 2.0], top_k=[0] * 5, top_p=[0.0] * 5,
                  u=[0.5] * 5)
    want = [int(torch.argmax(logits[i].cpu())) for i in range(5)]
    want[1], want[2] = 10, 0
    assert got == want


@pytest.mark.parametrize("vocab", [77, 5000])
def test_sample_draw_follows_the_cdf(ops, vocab):
    logits = _rand(1, vocab, seed=23, scale=2.0)
    for temperature, top_k, top_p in [(1.0, 0, 0.0), (0.7, 0, 0.0), (1.3, 12, 0.0), (1.0, 0, 0.8), (0.9, 20, 0.6)]:
        for u in (0.003, 0.21, 0.5, 0.77, 0.999):
            got = _sample(ops, logits, greedy=[0], temperature=[temperature], top_k=[top_k], top_p=[top_p], u=[u])[0]
            want = pm.plain_sample(logits[0].cpu(), greedy=False, temperature=temperature, top_k=top_k, top_p=top_p, u=u)
            if got != want:
                # sums in another order may move a boundary by a rounding step: then u must lie on it
                z = logits[0].cpu().double() / temperature
                p = torch.softmax(z, 0)
                lo, hi = sorted((got, want))
                kept = _kept(p, top_k, top_p)
                cdf = torch.cumsum(torch.where(kept, p, torch.zeros((), dtype=torch.double)), 0) / p[kept].sum()
                assert kept[got], (temperature, top_k, top_p, u)
                assert abs(float(cdf[lo]) - u) < 1e-4 and not kept[lo + 1:hi].any(), (temperature, top_k, top_p, u, got, want)


def _kept(p, top_k, top_p):
    keep = torch.ones_like(p, dtype=torch.bool)
    if 0 < top_k < p.numel():
        keep &= p >= torch.sort(p, descending=True).values[top_k - 1]
    if 0 < top_p < 1:
        sp = torch.sort(torch.where(keep, p, torch.zeros((), dtype=p.dtype)), descending=True).values
        cut = int((torch.cumsum(sp, 0) >= top_p).nonzero()[0])
        keep &= p >= sp[cut]
    return keep


def test_repetition_penalty(ops):
    logits = _rand(3, 50, seed=24)
    ref = logits.cpu().clone()
    rows = torch.tensor([0, 0, 2], dtype=torch.int32, device=DEV)
    toks = torch.tensor([4, 9, 9], dtype=torch.int32, device=DEV)
    counts = torch.tensor([1, 3, 2], dtype=torch.int32, device=DEV)
    pen = torch.tensor([1.1, 1.0, 1.5], device=DEV)
    ops.repetition_penalty(logits, rows, toks, counts, pen)
    for r, t, c in ((0, 4, 1), (0, 9, 3), (2, 9, 2)):
        v = ref[r, t]
        for _ in range(c):
            v = v / pen[r].item() if v > 0 else v * pen[r].item()
        ref[r, t] = v
    assert torch.allclose(logits.cpu(), ref, atol=1e-6)
