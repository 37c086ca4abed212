"""Each kernel alone against a plain PyTorch float32/float64 statement of the same op,
at sizes other than the engine tests' (widths and vocabularies that are no power of
two, head sizes in steps of 16, any number of heads and groups), with pages handed
out in a shuffled order (reference: src/cuda/qwen2/tests.rs:1076-1503,
src/cuda/qwen2/paged_tests.rs:216,609)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
# products and sums of bfloat16 inputs are exact in float32; what differs from the
# float64 statement is the rounding of the *output* (and of float32 accumulation)
OUT_TOL = {torch.float32: 2e-5, torch.bfloat16: 1e-2}


@pytest.fixture(scope="module")
def ops():
    from axon_b200.kernels import ops as o
    return o


def close(got, want, tol, what=""):
    want = want.to(torch.float64)
    scale = max(float(want.abs().max()), 1e-6)
    err = float((got.to(torch.float64) - want).abs().max())
    assert err <= tol * scale, f"{what}: error {err:.3e} = {err / scale:.2e} of scale (limit {tol:.0e})"


def rand(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, dtype):
    table = rand(37, 50, dtype=dtype)
    tokens = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    x = torch.empty(5, 50, dtype=torch.float32, device=DEV)
    ops.embed(tokens, table, x, scale=1.0)
    assert torch.equal(x, table[tokens.long()].float())
    ops.embed(tokens, table, x, scale=3.0)
    assert torch.equal(x, table[tokens.long()].float() * 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
# whole float4s take the one-pass kernel with 1, 2, 4 or 8 of them per thread; the others the scalar one
@pytest.mark.parametrize("dim", [1, 50, 96, 1000, 3584 + 8, 8192, 12288, 16400, 40000])
def test_rmsnorm(ops, dtype, dim):
    x = rand(9, dim, seed=1, std=3.0)
    gain = rand(dim, seed=2) * 0.1 + 1.0
    out = torch.empty(9, dim, dtype=dtype, device=DEV)
    for eps in (1e-6, 0.5):
        ops.rmsnorm(x, gain, out, eps)
        xd = x.double()
        want = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * gain.double()
        close(out, want, OUT_TOL[dtype], f"rmsnorm dim {dim} eps {eps}")
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, dim, dtype=dtype, device=DEV)
    ops.rmsnorm(x, gain, out3, 1e-6, rows=rows)
    assert torch.equal(out3, _norm_rows(ops, x, gain, rows, dtype, dim)), "gathered rows differ from their norms"
    ops.rmsnorm(x, gain - 1.0, out, 1e-6, unit_offset=True)
    xd = x.double()
    close(out, xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-6) * gain.double(), OUT_TOL[dtype], "1 + w gain")


def _norm_rows(ops, x, gain, rows, dtype, dim):
    full = torch.empty(x.shape[0], dim, dtype=dtype, device=DEV)
    ops.rmsnorm(x, gain, full, 1e-6)
    return full[rows.long()]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (1, 33, 5), (7, 200, 64), (65, 129, 97), (130, 64, 256), (3, 1000, 160)])
def test_gemm_plain(ops, dtype, M, N, K):
    a, w = rand(M, K, dtype=dtype, seed=3), rand(N, K, dtype=dtype, seed=4, std=0.2)
    bias = rand(N, seed=5)
    want = a.double() @ w.double().T
    for out_dtype in (torch.float32, dtype):
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        ops.gemm_plain(a, w, out)
        close(out, want, OUT_TOL[out_dtype], f"gemm {M}x{N}x{K}")
        ops.gemm_plain(a, w, out, bias=bias)
        close(out, want + bias.double(), OUT_TOL[out_dtype], "gemm + bias")
    res = rand(M, N, seed=6)
    acc = res.clone()
    ops.gemm_plain(a, w, acc, accumulate=True)
    close(acc, want + res.double(), OUT_TOL[torch.float32], "gemm into the residual")


def test_gemm_plain_mixed_dtypes(ops):
    a, w = rand(5, 40, dtype=torch.bfloat16, seed=7), rand(9, 40, seed=8)
    out = torch.empty(5, 9, dtype=torch.float32, device=DEV)
    ops.gemm_plain(a, w, out)       # a matrix stored in 32-bit under bfloat16 activations
    close(out, a.double() @ w.double().T, 2e-5)


def test_gemm_refuses_bad_shapes(ops):
    a, w = rand(4, 8), rand(5, 9)
    with pytest.raises(ValueError, match="shapes"):
        ops.gemm_plain(a, w, torch.empty(4, 5, device=DEV))
    with pytest.raises(ValueError, match="CUDA"):
        ops.gemm_plain(a.cpu(), w.cpu(), torch.empty(4, 5))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    n, f = 6, 75
    gu = rand(n, 2 * f, seed=9, std=2.0)
    act = torch.empty(n, f, dtype=dtype, device=DEV)
    ops.swiglu(gu, act)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    close(act, g / (1 + torch.exp(-g)) * u, OUT_TOL[dtype], "swiglu")


@pytest.mark.parametrize("half,theta", [(8, 1e4), (64, 1e6), (24, 5e5)])
def test_rope_table(ops, half, theta):
    pos = torch.tensor([0, 1, 17, 4095, 131071], dtype=torch.int32, device=DEV)
    inv = torch.tensor([theta ** (-2.0 * i / (2 * half)) for i in range(half)], dtype=torch.float64, device=DEV)
    table = torch.empty(5, half, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(pos, inv, table)
    ang = pos.double()[:, None] * inv[None, :]
    # the angle is exact in float64 and rounded to float32 once: half an ulp of error
    assert float((table[..., 0].double() - torch.cos(ang)).abs().max()) <= 6e-8
    assert float((table[..., 1].double() - torch.sin(ang)).abs().max()) <= 6e-8


def make_cache(ops, dtype, kv_heads, head_dim, page_size, n_pages, slots, max_pos, entries=2, entry=1, window=0, seed=0):
    """A pool with pages handed out in a shuffled order, and its table."""
    stride = -(-max_pos // page_size)
    pool = torch.zeros(n_pages + 1, entries, 2, kv_heads, page_size, head_dim, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)
    table = torch.full((slots, stride), n_pages, dtype=torch.int32)
    at = 0
    for s in range(slots):
        for lp in range(stride):
            if at < n_pages:
                table[s, lp] = perm[at]
                at += 1
    table = table.to(DEV)
    return ops.KvView(pool, table, entry, page_size, kv_heads, head_dim, window), table


def read_cache(view, table, slot, pos, which):
    ps = view.page_size
    page = int(table[slot, pos // ps])
    return view.pool[page, view.entry, which, :, pos % ps, :]     # [kv_heads, head_dim]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,rot,adjacent", [(4, 2, 16, 16, False), (3, 1, 32, 32, True),
                                                            (6, 3, 48, 16, False), (2, 2, 128, 0, False)])
def test_rope_kv_write(ops, dtype, heads, kv_heads, hd, rot, adjacent):
    n, ps = 11, 4
    view, table = make_cache(ops, dtype, kv_heads, hd, ps, 12, 2, 24, seed=5)
    qkv = rand(n, (heads + 2 * kv_heads) * hd, seed=11)
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 9, 10, 11, 12], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32, device=DEV)
    tab = None
    if rot:
        inv = torch.tensor([1e4 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64, device=DEV)
        tab = torch.empty(n, rot // 2, 2, dtype=torch.float32, device=DEV)
        ops.rope_table(positions, inv, tab)
    q_out = torch.empty(n, heads * hd, dtype=dtype, device=DEV)
    ops.rope_kv_write(qkv, tab, positions, slots, q_out, view, heads, rot, adjacent)

    def rotate(v, t):      # v [..., hd] float64
        if not rot:
            return v
        out = v.clone()
        c, s = tab[t, :, 0].double(), tab[t, :, 1].double()
        if adjacent:
            a, b = v[..., 0:rot:2], v[..., 1:rot:2]
            out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, a * s + b * c
        else:
            a, b = v[..., :rot // 2], v[..., rot // 2:rot]
            out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * s, a * s + b * c
        return out

    q = qkv[:, :heads * hd].double().view(n, heads, hd)
    k = qkv[:, heads * hd:(heads + kv_heads) * hd].double().view(n, kv_heads, hd)
    v = qkv[:, (heads + kv_heads) * hd:].double().view(n, kv_heads, hd)
    for t in range(n):
        close(q_out[t].view(heads, hd), rotate(q[t], t), OUT_TOL[dtype], "q")
        close(read_cache(view, table, int(slots[t]), int(positions[t]), 0), rotate(k[t], t), OUT_TOL[dtype], "k page")
        close(read_cache(view, table, int(slots[t]), int(positions[t]), 1), v[t], OUT_TOL[dtype], "v page")
    # the other plane of the pool (another layer's) was not touched
    assert float(view.pool[:, 0].abs().max()) == 0.0
    # write_kv off leaves the cache alone
    before = view.pool.clone()
    ops.rope_kv_write(qkv * 2, tab, positions, slots, q_out, view, heads, rot, adjacent, write_kv=False)
    assert torch.equal(before, view.pool)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,ps,window", [(4, 2, 16, 4, 0), (3, 1, 32, 16, 0), (7, 7, 48, 8, 0),
                                                         (8, 2, 128, 16, 0), (2, 1, 256, 16, 0), (4, 2, 64, 4, 5)])
def test_attention_plain(ops, dtype, heads, kv_heads, hd, ps, window):
    lens = [37, 70]                  # two requests of different lengths
    n_pages = 2 * -(-80 // ps)      # make_cache fills every table entry of both slots
    view, table = make_cache(ops, dtype, kv_heads, hd, ps, n_pages, 2, 80, window=window, seed=9)
    ks = [rand(l, kv_heads, hd, dtype=dtype, seed=20 + i) for i, l in enumerate(lens)]
    vs = [rand(l, kv_heads, hd, dtype=dtype, seed=30 + i) for i, l in enumerate(lens)]
    for s, l in enumerate(lens):
        for p in range(l):
            page = int(table[s, p // ps])
            view.pool[page, view.entry, 0, :, p % ps, :] = ks[s][p]
            view.pool[page, view.entry, 1, :, p % ps, :] = vs[s][p]
    # queries: the last 5 positions of request 0 and positions 0, 1, 33 and the last of request 1
    qpos = [(0, p) for p in range(32, 37)] + [(1, 0), (1, 1), (1, 33), (1, 69)]
    q = rand(len(qpos), heads * hd, dtype=dtype, seed=40)
    positions = torch.tensor([p for _, p in qpos], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in qpos], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(hd)
    ops.attention_plain(q, view, positions, slots, out, heads, scale)
    group = heads // kv_heads
    for i, (s, p) in enumerate(qpos):
        lo = max(0, p - window + 1) if window else 0
        for h in range(heads):
            qh = q[i].view(heads, hd)[h].double()
            kk, vv = ks[s][lo:p + 1, h // group].double(), vs[s][lo:p + 1, h // group].double()
            w = torch.softmax((kk @ qh) * scale, dim=0)
            close(out[i].view(heads, hd)[h], w @ vv, OUT_TOL[dtype], f"attention query {i} head {h}")


def test_argmax_rule(ops):
    row = torch.zeros(4, 1003, dtype=torch.float32, device=DEV)
    row[0, 17] = 5.0; row[0, 900] = 5.0            # equal maxima: the last index
    row[1, :] = -1.0; row[1, 3] = float("nan")     # NaN is never picked
    row[1, 44] = -0.5
    row[2, :] = float("nan")                        # all NaN: the last index
    row[3, 0] = 0.0; row[3, 5] = -0.0               # -0 ties +0: larger id among them
    row[3, 6:] = -1.0
    best = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.argmax(row, best)
    assert best.tolist() == [900, 44, 1002, 5]
    big = rand(3, 152064, seed=50)
    best = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(big, best)
    assert best.tolist() == big.argmax(dim=1).tolist()


@pytest.mark.parametrize("vocab", [300, 1000, 152064])
def test_topk_and_penalty(ops, vocab):
    logits = rand(3, vocab, seed=51, std=3.0)
    logits[1, 7] = logits[1, 9] = logits[1].max() + 1.0         # a tie at the top: larger id first
    logits[2, 5] = float("nan")
    ks = torch.tensor([40, 256, 3], dtype=torch.int32, device=DEV)
    cl = torch.empty(3, 256, dtype=torch.float32, device=DEV)
    ci = torch.empty(3, 256, dtype=torch.int32, device=DEV)
    ops.topk(logits, ks, cl, ci)
    for r, k in enumerate(ks.tolist()):
        row = logits[r].clone()
        row[row != row] = -float("inf")
        key = row.double().cpu()
        order = sorted(range(vocab), key=lambda i: (key[i].item(), i), reverse=True)[:k]
        assert ci[r, :k].tolist() == order
        assert torch.equal(cl[r, :k].cpu(), logits[r].cpu()[order])
    ids = torch.tensor([[1, 2, -1], [7, -1, -1], [0, 1, 2]], dtype=torch.int32, device=DEV)
    pen = torch.tensor([1.5, 1.0, 2.0], dtype=torch.float32, device=DEV)
    before = logits.clone()
    ops.repeat_penalty(logits, ids, pen)
    for r in range(3):
        for j in ids[r].tolist():
            if j < 0:
                continue
            b = before[r, j]
            want = b if pen[r] == 1.0 else (b / pen[r] if b > 0 else b * pen[r])
            assert logits[r, j] == want
    untouched = torch.ones_like(logits, dtype=torch.bool)
    for r in range(3):
        for j in ids[r].tolist():
            if j >= 0:
                untouched[r, j] = False
    same = (logits == before) | (logits != logits)
    assert bool(same[untouched].all())


def test_topk_when_thousands_of_logits_share_their_top_byte(ops):
    """More values in the deciding top byte than the kernel pools in shared memory (a flat row; a row
    of nearly equal values): the general eight-pass selection takes over.  Same rule: larger id first."""
    vocab = 152064
    logits = torch.zeros(3, vocab, dtype=torch.float32, device=DEV)
    logits[1] = 1.0 + rand(vocab, seed=53, std=1e-3)              # all within one top byte
    logits[2] = rand(vocab, seed=54, std=3.0)
    logits[2, 1000:90000] = 2.5                                   # 89,000 equal values among the largest
    ks = torch.tensor([40, 256, 100], dtype=torch.int32, device=DEV)
    cl = torch.empty(3, 256, dtype=torch.float32, device=DEV)
    ci = torch.empty(3, 256, dtype=torch.int32, device=DEV)
    ops.topk(logits, ks, cl, ci)
    assert ci[0, :40].tolist() == list(range(vocab - 1, vocab - 41, -1))
    for r in (1, 2):
        k = int(ks[r])
        key = logits[r].double().cpu()
        top = torch.topk(key, 2000).indices.tolist()                # a superset of the k best, then the exact rule
        order = sorted(set(top) | set(range(89999, 89999 - 300, -1)), key=lambda i: (key[i].item(), i), reverse=True)[:k]
        assert ci[r, :k].tolist() == order
        assert torch.equal(cl[r, :k].cpu(), logits[r].cpu()[order])


def test_sample_temperature_large_rows(ops):
    """The same inverse CDF over a vocabulary of 152,064 (float4 reads of each thread's stretch)."""
    vocab, rows = 152064, 256
    p = torch.softmax(rand(vocab, seed=55, std=4.0).double(), 0)
    logits = torch.log(p).float().repeat(rows, 1).contiguous()
    temps = torch.full((rows,), 1.0, dtype=torch.float32, device=DEV)
    us = torch.rand(rows, generator=torch.Generator().manual_seed(2), dtype=torch.float64).to(DEV)
    picked = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits, temps, us, picked)
    cdf = torch.cumsum(p, 0)
    want = torch.searchsorted(cdf, us * cdf[-1], right=True).clamp(max=vocab - 1)
    agree = (picked.long() == want).float().mean().item()
    assert agree > 0.98, f"only {agree:.4f} of the picks match the inverse CDF"


def test_sample_temperature(ops):
    vocab = 1000
    p = torch.softmax(rand(vocab, seed=52, std=2.0).double(), 0)
    logits = torch.log(p).float().repeat(4000, 1).contiguous()
    temps = torch.full((4000,), 1.0, dtype=torch.float32, device=DEV)
    g = torch.Generator().manual_seed(1)
    us = torch.rand(4000, generator=g, dtype=torch.float64).to(DEV)
    picked = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits, temps, us, picked)
    # each pick is the inverse CDF at its u, ids ascending
    cdf = torch.cumsum(p, 0)
    want = torch.searchsorted(cdf, us * cdf[-1], right=True).clamp(max=vocab - 1)
    agree = (picked.long() == want).float().mean().item()
    assert agree > 0.995, f"only {agree:.4f} of the picks match the inverse CDF"   # float32 weights vs float64 cdf
    # a low temperature concentrates on the best token
    temps.fill_(0.05)
    ops.sample_temperature(logits, temps, us, picked)
    assert (picked.long() == int(p.argmax())).float().mean().item() > 0.95


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_add_and_convert(ops, dtype):
    x, y = rand(7, 33, seed=60), rand(7, 33, dtype=dtype, seed=61)
    want = x + y.float()
    ops.residual_add(x, y)
    assert torch.equal(x, want)
    out = torch.empty(7, 33, dtype=dtype, device=DEV)
    ops.convert(x, out)
    assert torch.equal(out, x.to(dtype))


# ---------------------------------------------------------------------------
# the tuned bfloat16 kernels, each against float64

@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 23, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(16, 64), (2, 8), (33, 24), (1000, 160), (344, 344), (130, 1096), (4608, 3584),
                                 (3584, 18944), (76032 + 6, 72)])
def test_gemm_small_m(ops, M, N, K):
    from axon_b200.kernels import fast
    a = rand(M, K, dtype=torch.bfloat16, seed=70)
    w = rand(N, K, dtype=torch.bfloat16, seed=71, std=0.1)
    bias = rand(N, seed=72)
    want = a.double() @ w.double().T
    out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    assert fast.gemm(a, w, out, None, False)
    close(out, want, 2e-5, f"small-M product {M}x{N}x{K}")
    assert fast.gemm(a, w, out, bias, False)
    close(out, want + bias.double(), 2e-5, "with bias")
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert fast.gemm(a, w, outb, bias, False)
    close(outb, want + bias.double(), OUT_TOL[torch.bfloat16], "bfloat16 output")
    res = rand(M, N, seed=73)
    acc = res.clone()
    assert fast.gemm(a, w, acc, None, True)
    close(acc, want + res.double(), 2e-5, "into the residual")
    if N % 2 == 0:
        act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        assert fast.gemm_swiglu(a, w, act)
        g, u = want[:, 0::2], want[:, 1::2]
        close(act, g / (1 + torch.exp(-g)) * u, OUT_TOL[torch.bfloat16], "SwiGLU epilogue")
    assert fast.gemm_tc_status() == 0, "a wait inside a tensor-core kernel gave up"


def test_gemm_small_m_refusals(ops):
    from axon_b200.kernels import fast
    a, w = rand(4, 12, dtype=torch.bfloat16), rand(5, 12, dtype=torch.bfloat16)
    out = torch.empty(4, 5, dtype=torch.float32, device=DEV)
    assert not fast.gemm(a, w, out, None, False)            # K % 8 != 0: the caller takes the plain kernel
    assert not fast.gemm(a.float(), w.float(), out, None, False)
    from axon_b200.kernels import linear
    linear.linear(a, w, out)                                 # and gets the right result there
    close(out, a.double() @ w.double().T, 2e-5)


@pytest.fixture(params=["auto", "1x256", "1x224", "1x192", "1x128", "2x256", "2x224", "2x192", "2x128"])
def tile_shape(request):
    """Every tile shape of the prefill product (rows / 128 x columns), and the model's own choice."""
    from axon_b200.kernels import lib
    if request.param == "auto":
        lib.cuda().axon_gemm_tc_force_tile(0, 0)
    else:
        rm, bn = request.param.split("x")
        lib.cuda().axon_gemm_tc_force_tile(int(rm), int(bn))
    yield request.param
    lib.cuda().axon_gemm_tc_force_tile(0, 0)


@pytest.mark.parametrize("M", [65, 129, 300, 1100])
@pytest.mark.parametrize("N,K", [(256, 64), (128, 8), (130, 72), (1000, 160), (344, 344), (2, 1096), (4608, 3584)])
def test_gemm_tensor_core(ops, tile_shape, M, N, K, monkeypatch):
    """The tcgen05 kernel at sizes with tails in M, N and K, every epilogue, every tile shape."""
    from axon_b200.kernels import fast
    monkeypatch.setattr(fast, "SWAP_RULE", "never")         # the tiled kernel, also where the swapped one would run
    a = rand(M, K, dtype=torch.bfloat16, seed=80)
    w = rand(N, K, dtype=torch.bfloat16, seed=81, std=0.1)
    bias = rand(N, seed=82)
    want = a.double() @ w.double().T
    out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    assert fast.gemm(a, w, out, None, False)
    close(out, want, 2e-5, f"tensor-core product {M}x{N}x{K}")
    assert fast.gemm(a, w, out, bias, False)
    close(out, want + bias.double(), 2e-5, "with bias")
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert fast.gemm(a, w, outb, bias, False)
    close(outb, want + bias.double(), OUT_TOL[torch.bfloat16], "bfloat16 output")
    res = rand(M, N, seed=83)
    acc = res.clone()
    assert fast.gemm(a, w, acc, None, True)
    close(acc, want + res.double(), 2e-5, "into the residual")
    if N % 2 == 0:
        act = torch.full((M, N // 2), 3.0, dtype=torch.bfloat16, device=DEV)
        assert fast.gemm_swiglu(a, w, act)
        g, u = want[:, 0::2], want[:, 1::2]
        close(act, g / (1 + torch.exp(-g)) * u, OUT_TOL[torch.bfloat16], "SwiGLU epilogue")
    # a view into a larger buffer (rows of a workspace) is a valid operand too
    big = torch.zeros(M + 3, K, dtype=torch.bfloat16, device=DEV)
    big[3:] = a
    assert fast.gemm(big[3:], w, out, None, False)
    close(out, want, 2e-5, "operand at an offset")
    assert fast.gemm_tc_status() == 0, "a wait inside the kernel gave up"


@pytest.mark.parametrize("M", [65, 128, 129, 256, 300, 700, 1024])
@pytest.mark.parametrize("N,K", [(256, 64), (130, 72), (1000, 160), (3584, 1024), (2, 1096)])
def test_gemm_swapped_in_blocks_of_tokens(ops, M, N, K, monkeypatch):
    """The product with the tokens as the MMA's columns beyond 64 rows: 128 or 256 columns, and
    blocks of 256 tokens beyond that; every epilogue, split over K or not, folded by itself or by the reader."""
    from axon_b200.kernels import fast
    monkeypatch.setattr(fast, "SWAP_RULE", "always")
    a = rand(M, K, dtype=torch.bfloat16, seed=140)
    w = rand(N, K, dtype=torch.bfloat16, seed=141, std=0.1)
    bias = rand(N, seed=142)
    res = rand(M, N, seed=143)
    want = a.double() @ w.double().T
    out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    assert fast.gemm(a, w, out, bias, False) is True
    close(out, want + bias.double(), 2e-5, "float output")
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert fast.gemm(a, w, outb, None, False) is True
    close(outb, want, OUT_TOL[torch.bfloat16], "bfloat16 output")
    acc = res.clone()
    assert fast.gemm(a, w, acc, None, True) is True
    close(acc, want + res.double(), 2e-5, "into the residual")
    acc2 = res.clone()
    owed = fast.gemm(a, w, acc2, None, True, defer=True)
    if isinstance(owed, fast.PendingFold):
        assert owed.ntok >= M and owed.ntok % 16 == 0
        ops.fold_partials(owed)
    assert torch.equal(acc2, acc), "the reader's fold differs from the kernel's"
    if N % 2 == 0:
        act = torch.full((M, N // 2), 3.0, dtype=torch.bfloat16, device=DEV)
        assert fast.gemm_swiglu(a, w, act)
        g, u = want[:, 0::2], want[:, 1::2]
        close(act, g / (1 + torch.exp(-g)) * u, OUT_TOL[torch.bfloat16], "SwiGLU epilogue")
    assert fast.gemm_tc_status() == 0


@pytest.mark.parametrize("M,N,K", [(300, 1024, 160), (1100, 4608, 512)])
def test_gemm_tensor_core_output_paths(ops, M, N, K, monkeypatch):
    """Outputs that TMA can address leave through shared memory and TMA (clipped at the edges, the
    residual by TMA's add); the others are stored from registers.  Both give the same numbers."""
    from axon_b200.kernels import fast, lib
    monkeypatch.setattr(fast, "SWAP_RULE", "never")
    a = rand(M, K, dtype=torch.bfloat16, seed=90)
    w = rand(N, K, dtype=torch.bfloat16, seed=91, std=0.1)
    bias = rand(N, seed=92)
    res = rand(M, N, seed=93)
    got = {}
    try:
        for plain in (0, 1):
            lib.cuda().axon_gemm_tc_force_plain_out(plain)
            f32 = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
            bf = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
            acc = res.clone()
            act = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
            assert fast.gemm(a, w, f32, bias, False) and fast.gemm(a, w, bf, bias, False)
            assert fast.gemm(a, w, acc, None, True) and fast.gemm_swiglu(a, w, act)
            # a window into a wider buffer: rows further apart than they are long, edges must stay untouched
            wide = torch.full((M + 2, N + 8), 5.0, dtype=torch.float32, device=DEV)
            assert fast.gemm(a, w, wide[1:M + 1, 4:N + 4], None, False)
            got[plain] = (f32, bf, acc, act, wide)
    finally:
        lib.cuda().axon_gemm_tc_force_plain_out(0)
    want = a.double() @ w.double().T
    close(got[0][0], want + bias.double(), 2e-5, "float output through TMA")
    close(got[0][2], want + res.double(), 2e-5, "residual through TMA's add")
    g, u = want[:, 0::2], want[:, 1::2]
    close(got[0][3], g / (1 + torch.exp(-g)) * u, OUT_TOL[torch.bfloat16], "SwiGLU through TMA")
    for x, y, name in zip(got[0], got[1], ("float", "bfloat16", "residual", "SwiGLU", "window")):
        close(x, y.double(), 1e-6 if x.dtype == torch.float32 else 8e-3, f"{name}: TMA against registers")
    wide = got[0][4]
    close(wide[1:M + 1, 4:N + 4], want, 2e-5, "window")
    assert (wide[0] == 5).all() and (wide[-1] == 5).all() and (wide[:, :4] == 5).all() and (wide[:, -4:] == 5).all()
    assert fast.gemm_tc_status() == 0


@pytest.mark.parametrize("M,N,K", [(8, 3584, 1024), (1, 1002, 2048), (33, 640, 4096), (64, 256, 8192)])
def test_split_product_leaves_its_fold_to_the_reader(ops, M, N, K):
    """A product for few rows that is split over K may leave its partial sums to whoever reads the
    output next.  Every reader (the norm, the generic fold) gives the numbers of the product that
    folds by itself, bit for bit; a PendingFold that nobody claims is an error at the next product."""
    from axon_b200.kernels import fast
    a = rand(M, K, dtype=torch.bfloat16, seed=110)
    w = rand(N, K, dtype=torch.bfloat16, seed=111, std=0.1)
    bias = rand(N, seed=112)
    res = rand(M, N, seed=113)
    want = res.clone()
    assert fast.gemm(a, w, want, bias, True) is True                 # folds by itself
    # the generic fold
    got = res.clone()
    owed = fast.gemm(a, w, got, bias, True, defer=True)
    assert isinstance(owed, fast.PendingFold) and owed.splits > 1, "this shape is meant to split"
    assert torch.equal(got, res), "a deferred product must not touch its output"
    ops.fold_partials(owed)
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):
        ops.fold_partials(owed)                                       # claimed once
    # stored, not accumulated, into bfloat16-free float output
    plain = torch.empty(M, N, dtype=torch.float32, device=DEV)
    assert fast.gemm(a, w, plain, bias, False) is True
    got = torch.full((M, N), 3.0, dtype=torch.float32, device=DEV)
    owed = fast.gemm(a, w, got, bias, False, defer=True)
    ops.fold_partials(owed)
    assert torch.equal(got, plain)
    # the norm as reader: x brought up to date and normed in one kernel, all rows or gathered ones
    gain = rand(N, seed=114) * 0.1 + 1.0
    h_want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(want, gain, h_want, 1e-6)
    x = res.clone()
    owed = fast.gemm(a, w, x, bias, True, defer=True)
    h = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, gain, h, 1e-6, pending=owed)
    assert torch.equal(x, want) and torch.equal(h, h_want)
    rows = torch.tensor([M - 1, 0], dtype=torch.int32, device=DEV)
    x = res.clone()
    owed = fast.gemm(a, w, x, bias, True, defer=True)
    h2 = torch.empty(2, N, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, gain, h2, 1e-6, rows=rows, pending=owed)
    assert torch.equal(h2, h_want[rows.long()]) and torch.equal(x[rows.long()], want[rows.long()])
    # dropped: the next split product refuses to overwrite the scratch
    owed = fast.gemm(a, w, res.clone(), bias, True, defer=True)
    with pytest.raises(RuntimeError):
        fast.gemm(a, w, res.clone(), bias, True)
    owed.claimed = True
    with pytest.raises(RuntimeError):                                 # folded into the wrong tensor
        o2 = fast.gemm(a, w, res.clone(), bias, True, defer=True)
        ops.rmsnorm(res.clone(), gain, h, 1e-6, pending=o2)
    o2.claimed = True
    assert fast.gemm_tc_status() == 0


def test_rotation_reads_a_split_product(ops):
    """rope_kv_write folding the partial sums of the q/k/v product gives what it gives on the folded product."""
    from axon_b200.kernels import fast
    heads, kv_heads, hd, n, ps = 6, 2, 64, 5, 4
    width = (heads + 2 * kv_heads) * hd
    a = rand(n, 2048, dtype=torch.bfloat16, seed=120)
    w = rand(width, 2048, dtype=torch.bfloat16, seed=121, std=0.1)
    bias = rand(width, seed=122)
    positions = torch.tensor([0, 1, 2, 7, 8], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    table = torch.empty(n, hd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions, inv.to(DEV), table)
    outs = []
    for defer in (False, True):
        view, _ = make_cache(ops, torch.bfloat16, kv_heads, hd, ps, 8, 2, 16, seed=9)
        qkv = torch.full((n, width), 2.0, dtype=torch.float32, device=DEV)
        owed = fast.gemm(a, w, qkv, bias, False, defer=defer)
        assert isinstance(owed, fast.PendingFold) == defer
        q = torch.zeros(n, heads * hd, dtype=torch.bfloat16, device=DEV)
        ops.rope_kv_write(qkv, table, positions, slots, q, view, heads, hd, pending=owed if defer else None)
        outs.append((q, view.pool.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert outs[0][1].abs().sum() > 0


def _ctx_for(segs):
    """A StepContext for segments [(slot, q_len, kv_len)] with tokens flattened in order."""
    from axon_b200.parts import Runtime, StepContext
    rt = Runtime(torch.bfloat16, DEV)
    pos, slot_of, rows, at = [], [], [[], [], [], []], 0
    for slot, n, kv_len in segs:
        pos += list(range(kv_len - n, kv_len))
        slot_of += [slot] * n
        for lst, v in zip(rows, (slot, at, n, kv_len)):
            lst.append(v)
        at += n
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(rt=rt, n_tokens=at, tokens=i32([0] * at), positions=i32(pos), token_slot=i32(slot_of),
                       seg_slot=rows[0], seg_q_start=rows[1], seg_q_len=rows[2], seg_kv_len=rows[3],
                       segments=i32(rows), host_positions=pos)


@pytest.mark.parametrize("heads,kv_heads,hd,ps,window", [
    (4, 2, 16, 4, 0), (3, 1, 32, 16, 0), (6, 2, 64, 8, 0), (28, 4, 128, 16, 0), (8, 8, 128, 16, 0),
    (40, 2, 64, 16, 0), (7, 1, 128, 1, 0), (6, 2, 64, 16, 70), (4, 2, 128, 16, 9)])
@pytest.mark.parametrize("fold,tcgen05", [("second_kernel", True), ("last_cta", True), ("second_kernel", False)])
def test_attention_tensor_core(ops, heads, kv_heads, hd, ps, window, fold, tcgen05, monkeypatch):
    """The tensor-core kernel on a mixed batch: decoded tokens at short and long contexts
    (one key; several splits), two-token portions, a whole prompt, a portion in the middle
    of a long request.  One key far back gets a large score so that a wrong page or a
    dropped tile shows."""
    from axon_b200.kernels import fast
    # the two ways of folding the key splits of a decoded token
    monkeypatch.setattr(fast, "FA_FOLD_IN_KERNEL", fold == "last_cta")
    # prompt portions at head size 128: the tcgen05 kernel, or the mma.sync one as for other head sizes
    monkeypatch.setitem(fast.ENABLED, "attention_tc", tcgen05)
    # (q_len, kv_len) per request
    shapes = [(1, 1), (1, 700), (2, 131), (100, 100), (37, 300), (1, 64), (1, 65), (3, 3)]
    max_pos = 704
    slots = len(shapes)
    view, table = make_cache(ops, torch.bfloat16, kv_heads, hd, ps, slots * -(-max_pos // ps), slots, max_pos,
                             window=window, seed=13)
    group = heads // kv_heads
    ks, vs = [], []
    for s, (n, kv_len) in enumerate(shapes):
        k = rand(kv_len, kv_heads, hd, dtype=torch.bfloat16, seed=200 + s)
        v = rand(kv_len, kv_heads, hd, dtype=torch.bfloat16, seed=300 + s)
        ks.append(k); vs.append(v)
        for pos in range(kv_len):
            page = int(table[s, pos // ps])
            view.pool[page, view.entry, 0, :, pos % ps, :] = k[pos]
            view.pool[page, view.entry, 1, :, pos % ps, :] = v[pos]
    ctx = _ctx_for([(s, n, kv_len) for s, (n, kv_len) in enumerate(shapes)])
    q = rand(ctx.n_tokens, heads * hd, dtype=torch.bfloat16, seed=400)
    # the last query of request 1 lines up with its key 17 (far back) on every head
    qv = q.view(ctx.n_tokens, heads, hd)
    for h in range(heads):
        qv[1, h] = (ks[1][17, h // group].float() * 1.5).to(torch.bfloat16)
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(hd)
    assert fast.attention(q, view, ctx, out, heads, scale)
    plain_out = torch.zeros_like(q)
    ops.attention_plain(q, view, ctx.positions, ctx.token_slot, plain_out, heads, scale)
    at = 0
    for s, (n, kv_len) in enumerate(shapes):
        for i in range(n):
            pos = kv_len - n + i
            lo = max(0, pos - window + 1) if window else 0
            for h in range(heads):
                qh = q[at + i].view(heads, hd)[h].double()
                kk, vv = ks[s][lo:pos + 1, h // group].double(), vs[s][lo:pos + 1, h // group].double()
                w = torch.softmax((kk @ qh) * scale, dim=0)
                want = w @ vv
                close(out[at + i].view(heads, hd)[h], want, 1.5e-2, f"request {s} token {i} head {h}")
                close(plain_out[at + i].view(heads, hd)[h], want, 1e-2, f"plain kernel, request {s} token {i} head {h}")
        at += n


@pytest.mark.parametrize("heads,kv_heads,ps,window,shapes", [
    (28, 4, 16, 0, [(600, 600), (300, 900), (129, 129)]),        # 126-row tiles, many key tiles
    (12, 2, 8, 200, [(700, 700), (90, 1000)]),                   # a window: tiles wholly inside it, at its edges, before it
    (3, 3, 32, 0, [(260, 260), (5, 400)]),                       # one head per kv head: 128 tokens a tile
    (64, 1, 16, 0, [(70, 200)]),                                 # 64 heads to a kv head: two tokens a tile
    (8, 2, 16, 0, [(6000, 6000), (200, 9000)]),                  # more CTAs than SMs, 140 key tiles: every ring and barrier wraps many times
])
def test_attention_tcgen05_prompts(ops, heads, kv_heads, ps, window, shapes):
    """The tcgen05 kernel for prompt portions (head size 128) over several key tiles, against
    float64.  One key far back gets a large score in one query of every request."""
    from axon_b200.kernels import fast
    hd = 128
    max_pos = max(kv for _, kv in shapes)
    slots = len(shapes)
    view, table = make_cache(ops, torch.bfloat16, kv_heads, hd, ps, slots * -(-max_pos // ps), slots, max_pos,
                             window=window, seed=21)
    group = heads // kv_heads
    ks, vs = [], []
    for s, (n, kv_len) in enumerate(shapes):
        k = rand(kv_len, kv_heads, hd, dtype=torch.bfloat16, seed=500 + s)
        v = rand(kv_len, kv_heads, hd, dtype=torch.bfloat16, seed=600 + s)
        ks.append(k); vs.append(v)
        pages = table[s, : -(-kv_len // ps)].long()
        pad = len(pages) * ps - kv_len
        for which, t in ((0, k), (1, v)):
            t = torch.cat([t, torch.zeros(pad, kv_heads, hd, dtype=t.dtype, device=DEV)])
            view.pool[pages, view.entry, which] = t.view(len(pages), ps, kv_heads, hd).permute(0, 2, 1, 3)
    ctx = _ctx_for([(s, n, kv_len) for s, (n, kv_len) in enumerate(shapes)])
    q = rand(ctx.n_tokens, heads * hd, dtype=torch.bfloat16, seed=700)
    qv = q.view(ctx.n_tokens, heads, hd)
    at = 0
    for s, (n, kv_len) in enumerate(shapes):
        # the request's last query lines up with the oldest key it may still see
        far = max(0, kv_len - window) if window else 3
        for h in range(heads):
            qv[at + n - 1, h] = (ks[s][far, h // group].float() * 1.5).to(torch.bfloat16)
        at += n
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(hd)
    assert fast.ENABLED["attention_tc"]
    assert fast.attention(q, view, ctx, out, heads, scale)
    assert fast.attention_tc_status() == 0, "a wait inside the kernel gave up"
    at = 0
    for s, (n, kv_len) in enumerate(shapes):
        qpos = torch.arange(kv_len - n, kv_len, device=DEV)[:, None]
        kpos = torch.arange(kv_len, device=DEV)[None, :]
        mask = kpos <= qpos
        if window:
            mask &= kpos > qpos - window
        for h in range(heads):
            sc = (qv[at:at + n, h].double() @ ks[s][:, h // group].double().T) * scale
            w = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1)
            if h == 0:
                assert w[-1].max() > 0.5, "the planted key does not stand out"
            close(out.view(-1, heads, hd)[at:at + n, h], w @ vs[s][:, h // group].double(), 1.5e-2,
                  f"request {s} head {h}")
        at += n


@pytest.mark.parametrize("heads,kv_heads,hd,window", [(28, 4, 128, 0), (6, 2, 64, 0), (8, 8, 128, 5000)])
def test_decode_attention_at_long_contexts(ops, heads, kv_heads, hd, window):
    """Decoded tokens at contexts of thousands of positions (many key splits, hundreds of tiles a
    share, block-table rows of two thousand entries), against float64; one key far back gets a
    large score."""
    from axon_b200.kernels import fast
    ps = 16
    shapes = [(1, 20000), (1, 33000), (2, 8191), (1, 4097)]
    max_pos = max(kv for _, kv in shapes)
    slots = len(shapes)
    view, table = make_cache(ops, torch.bfloat16, kv_heads, hd, ps, slots * -(-max_pos // ps), slots, max_pos,
                             window=window, seed=29)
    group = heads // kv_heads
    ks, vs = [], []
    for s, (n, kv_len) in enumerate(shapes):
        k = rand(kv_len, kv_heads, hd, dtype=torch.bfloat16, seed=800 + s)
        v = rand(kv_len, kv_heads, hd, dtype=torch.bfloat16, seed=900 + s)
        ks.append(k); vs.append(v)
        pages = table[s, : -(-kv_len // ps)].long()
        pad = len(pages) * ps - kv_len
        for which, t in ((0, k), (1, v)):
            t = torch.cat([t, torch.zeros(pad, kv_heads, hd, dtype=t.dtype, device=DEV)])
            view.pool[pages, view.entry, which] = t.view(len(pages), ps, kv_heads, hd).permute(0, 2, 1, 3)
    ctx = _ctx_for([(s, n, kv_len) for s, (n, kv_len) in enumerate(shapes)])
    q = rand(ctx.n_tokens, heads * hd, dtype=torch.bfloat16, seed=77)
    qv = q.view(ctx.n_tokens, heads, hd)
    at = 0
    for s, (n, kv_len) in enumerate(shapes):
        far = max(0, kv_len - window) if window else 7
        for h in range(heads):
            qv[at + n - 1, h] = (ks[s][far, h // group].float() * (8.0 / math.sqrt(hd) if hd < 128 else 1.5)).to(torch.bfloat16)
        at += n
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(hd)
    assert fast.attention(q, view, ctx, out, heads, scale)
    at = 0
    for s, (n, kv_len) in enumerate(shapes):
        qpos = torch.arange(kv_len - n, kv_len, device=DEV)[:, None]
        kpos = torch.arange(kv_len, device=DEV)[None, :]
        mask = kpos <= qpos
        if window:
            mask &= kpos > qpos - window
        for h in range(heads):
            sc = (qv[at:at + n, h].double() @ ks[s][:, h // group].double().T) * scale
            w = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1)
            close(out.view(-1, heads, hd)[at:at + n, h], w @ vs[s][:, h // group].double(), 1.5e-2, f"request {s} head {h}")
        at += n


@pytest.mark.parametrize("heads,kv_heads,hd,ps,window,split_product", [
    (28, 4, 128, 16, 0, True), (6, 2, 64, 8, 0, False), (8, 8, 128, 16, 40, True), (4, 1, 32, 4, 0, True),
    (16, 1, 16, 16, 0, False)])
def test_decode_attention_rotates_and_writes_by_itself(ops, heads, kv_heads, hd, ps, window, split_product):
    """A step of single tokens: the kernel that rotates the queries, writes the new keys and values
    and attends, against the rotation kernel followed by the attention kernel.  Same bits out, same
    cache; also when the q/k/v product is still owed its partial sums, and when the cache is only read."""
    from axon_b200.kernels import fast
    from axon_b200.parts import Runtime, StepContext
    kv_lens = [1, 64, 65, 700, 129, 2]
    n, width = len(kv_lens), (heads + 2 * kv_heads) * hd
    K = 2048 if split_product else 64
    a = rand(n, K, dtype=torch.bfloat16, seed=130)
    w = rand(width, K, dtype=torch.bfloat16, seed=131, std=0.05 if split_product else 0.3)
    bias = rand(width, seed=132)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    positions, slots = i32([k - 1 for k in kv_lens]), i32(list(range(n)))
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    table = torch.empty(n, hd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions, inv.to(DEV), table)
    rows = [list(range(n)), list(range(n)), [1] * n, kv_lens]
    results = []
    for fused in (False, True):
        for write_kv in (True, False):
            view, tbl = make_cache(ops, torch.bfloat16, kv_heads, hd, ps, n * -(-704 // ps), n, 704, window=window, seed=17)
            view.pool.copy_(rand(*view.pool.shape, dtype=torch.bfloat16, seed=133))     # older keys and values
            ctx = StepContext(rt=Runtime(torch.bfloat16, DEV), n_tokens=n, tokens=i32([0] * n), positions=positions,
                              token_slot=slots, seg_slot=rows[0], seg_q_start=rows[1], seg_q_len=rows[2],
                              seg_kv_len=rows[3], segments=i32(rows), unit_items=i32([[s, 0] for s in range(n)]).flatten(),
                              host_positions=[k - 1 for k in kv_lens])
            qkv = torch.zeros(n, width, dtype=torch.float32, device=DEV)
            owed = fast.gemm(a, w, qkv, bias, False, defer=True)
            assert isinstance(owed, fast.PendingFold) == split_product
            owed = owed if split_product else None
            out = torch.zeros(n, heads * hd, dtype=torch.bfloat16, device=DEV)
            scale = 1.0 / math.sqrt(hd)
            if fused:
                assert fast.attention_decode_fused(qkv, owed, table, hd, False, view, ctx, out, heads, scale, write_kv)
            else:
                q = torch.zeros(n, heads * hd, dtype=torch.bfloat16, device=DEV)
                ops.rope_kv_write(qkv, table, positions, slots, q, view, heads, hd, write_kv=write_kv, pending=owed)
                assert fast.attention(q, view, ctx, out, heads, scale)
            results.append((out, view.pool.clone()))
    for (o_two, c_two), (o_one, c_one) in zip(results[:2], results[2:]):
        assert torch.equal(c_two, c_one), "the caches differ"
        assert torch.equal(o_two, o_one), "the outputs differ"
    assert not torch.equal(results[0][1], results[1][1]), "writing the cache changed nothing"
    assert results[0][0].float().abs().sum() > 0


def test_attention_tensor_core_refusals(ops):
    from axon_b200.kernels import fast
    view, _ = make_cache(ops, torch.bfloat16, 1, 48, 16, 4, 1, 64)
    ctx = _ctx_for([(0, 1, 5)])
    q = rand(1, 2 * 48, dtype=torch.bfloat16)
    assert not fast.attention(q, view, ctx, torch.empty_like(q), 2, 0.1)       # head size 48: the plain kernel runs


# ---------------------------------------------------------------------------
# Caches whose key and value rows differ in width, and caches with one plane.

def _odd_cache(ops, dtype, kv_heads, hd, v_dim, planes, ps, n_pages, slots, max_pos, entries=2, entry=1, seed=0):
    from axon_b200.parts.spec import KvNeed
    need = KvNeed(kv_heads, hd, None, v_dim if planes == 2 else None, planes)
    stride = -(-max_pos // ps)
    pool = torch.zeros(n_pages + 1, entries, ps * need.elements_per_token, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(seed)
    table = torch.randperm(n_pages, generator=g)[: slots * stride].to(torch.int32).view(slots, stride).to(DEV)
    return ops.KvView(pool, table, entry, ps, kv_heads, hd, 0, v_dim=need.value_dim, planes=planes), table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,v_dim,planes", [(4, 2, 16, 40, 2), (3, 1, 24, 8, 2), (4, 1, 32, 32, 1)])
def test_plain_kernels_with_other_planes(ops, dtype, heads, kv_heads, hd, v_dim, planes):
    """The rotate-and-write kernel and the plain attention on a cache whose value rows are wider or
    narrower than its key rows, and on a cache with one plane (values read from the key rows)."""
    n, ps = 9, 4
    view, table = _odd_cache(ops, dtype, kv_heads, hd, v_dim, planes, ps, 6, 1, 12, seed=3)
    vd = view.v_dim
    width = (heads + kv_heads) * hd + (kv_heads * vd if planes == 2 else 0)
    qkv = rand(n, width, seed=21)
    positions = torch.arange(n, dtype=torch.int32, device=DEV)
    slots = torch.zeros(n, dtype=torch.int32, device=DEV)
    q_out = torch.empty(n, heads * hd, dtype=dtype, device=DEV)
    ops.rope_kv_write(qkv, None, positions, slots, q_out, view, heads, 0, False)
    q = qkv[:, :heads * hd].view(n, heads, hd)
    k = qkv[:, heads * hd:(heads + kv_heads) * hd].view(n, kv_heads, hd)
    v = qkv[:, (heads + kv_heads) * hd:].view(n, kv_heads, vd) if planes == 2 else k
    keys, values = view.keys(), view.values()
    for t in range(n):
        page = int(table[0, t // ps])
        close(keys[page, :, t % ps], k[t], OUT_TOL[dtype], "key rows")
        close(values[page, :, t % ps], v[t], OUT_TOL[dtype], "value rows")
    assert float(view.pool[:, 0].abs().max()) == 0.0, "the other entry's planes were touched"
    out = torch.empty(n, heads * vd, dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.attention_plain(q_out, view, positions, slots, out, heads, scale)
    group = heads // kv_heads
    kd, vdd = k.to(dtype).double(), v.to(dtype).double()
    for t in range(n):
        for h in range(heads):
            w = torch.softmax((kd[: t + 1, h // group] @ q_out[t].view(heads, hd)[h].double()) * scale, 0)
            close(out[t].view(heads, vd)[h], w @ vdd[: t + 1, h // group], OUT_TOL[dtype], f"token {t} head {h}")
    # the tuned kernels refuse such a cache instead of misreading it
    from axon_b200.kernels import fast
    if dtype == torch.bfloat16:
        assert not fast.attention(q_out, view, _ctx_for([(0, n, n)]), torch.empty_like(q_out), heads, scale)


def test_checked_tables_catch_an_entry_outside_the_pool(ops):
    """With checked tables a block-table entry beyond the pool is not followed: the kernel uses the
    sink page and records the entry.  The "bad" entry here still lies inside the tensor (the
    view is told that the pool is smaller than it is), so nothing could go astray either way."""
    heads, kv_heads, hd, ps = 4, 2, 64, 16
    real_pages, said_pages = 12, 6
    pool = (torch.randn(real_pages + 1, 1, 2, kv_heads, ps, hd) * 0.5).to(torch.bfloat16).to(DEV)
    table = torch.tensor([[0, 1, 2, 3], [4, 9, 5, said_pages]], dtype=torch.int32, device=DEV)    # 9 > 6: outside
    fault = torch.zeros(2, dtype=torch.int32, device=DEV)
    view = ops.KvView(pool[: said_pages + 1], table, 0, ps, kv_heads, hd, 0, fault=fault)
    assert view.n_pages == said_pages
    from axon_b200.kernels import fast
    ctx = _ctx_for([(0, 1, 60), (1, 1, 40)])
    q = rand(2, heads * hd, dtype=torch.bfloat16, seed=5)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(hd)
    # the request whose table is fine: nothing recorded
    ok = ops.KvView(pool[: said_pages + 1], table[:1].contiguous(), 0, ps, kv_heads, hd, 0, fault=fault)
    assert fast.attention(q[:1].contiguous(), ok, _ctx_for([(0, 1, 60)]), out[:1], heads, scale)
    assert fault.tolist() == [0, 0]
    for run in ("tuned", "plain", "write"):
        fault.zero_()
        if run == "tuned":
            assert fast.attention(q, view, ctx, out, heads, scale)
        elif run == "plain":
            ops.attention_plain(q, view, ctx.positions, ctx.token_slot, out, heads, scale)
        else:
            qkv = rand(1, (heads + 2 * kv_heads) * hd, seed=6)
            ops.rope_kv_write(qkv, None, torch.tensor([20], dtype=torch.int32, device=DEV),
                              torch.tensor([1], dtype=torch.int32, device=DEV), torch.empty_like(q[:1]), view, heads, 0)
        assert fault.tolist() == [1, 9], f"{run}: the entry outside the pool was not recorded"
    assert float(pool[9].float().abs().sum()) > 0 and torch.isfinite(out.float()).all()


def test_a_wait_that_gives_up_sets_the_status_and_the_next_launch_works(ops):
    """The failure path of the tensor-core product: its epilogue's wait for the accumulator is
    never answered (a test mode of the launcher) and gives up after a few thousand polls.  The
    kernel still ends in order, the status word says which role gave up, and once the word is
    cleared the next launch gives the right product."""
    from axon_b200.kernels import fast, lib
    cu = lib.cuda()
    M, N, K = 300, 512, 256
    a = rand(M, K, dtype=torch.bfloat16, seed=80)
    w = rand(N, K, dtype=torch.bfloat16, seed=81, std=0.1)
    out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    old = fast.ENABLED["gemm_tc_small"]
    fast.ENABLED["gemm_tc_small"] = False                 # the tiled kernel, whatever the row count
    try:
        assert fast.gemm_tc_status() == 0
        cu.axon_gemm_tc_test_stuck_wait(4096)
        try:
            assert fast.gemm(a, w, out, None, False)
            torch.cuda.synchronize()                      # the kernel returned by itself
        finally:
            cu.axon_gemm_tc_test_stuck_wait(0)
        assert fast.gemm_tc_status() == 3, "1 + role 2: the epilogue's wait gave up"
        assert cu.axon_gemm_tc_clear_status() == 0 and fast.gemm_tc_status() == 0
        assert fast.gemm(a, w, out, None, False)
        close(out, a.double() @ w.double().T, 2e-5, "the launch after the failure")
        assert fast.gemm_tc_status() == 0
    finally:
        fast.ENABLED["gemm_tc_small"] = old


def test_pickers_read_rows_by_index(ops):
    """argmax, top-k and the temperature draw on some rows of a batch, named by an index, give what
    they give on a copy of those rows."""
    vocab = 1000
    logits = rand(7, vocab, seed=3)
    idx = torch.tensor([5, 0, 6], dtype=torch.int32, device=DEV)
    sub = logits[idx.long()].contiguous()
    a, b = torch.empty(3, dtype=torch.int32, device=DEV), torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(logits, a, rows=idx)
    ops.argmax(sub, b)
    assert torch.equal(a, b) and a.tolist() == sub.argmax(1).tolist()
    ks = torch.tensor([5, 40, 1], dtype=torch.int32, device=DEV)
    kmax = ops.topk_max()
    c1, i1 = torch.zeros(3, kmax, device=DEV), torch.zeros(3, kmax, dtype=torch.int32, device=DEV)
    c2, i2 = torch.zeros(3, kmax, device=DEV), torch.zeros(3, kmax, dtype=torch.int32, device=DEV)
    ops.topk(logits, ks, c1, i1, rows=idx)
    ops.topk(sub, ks, c2, i2)
    for r, k in enumerate(ks.tolist()):
        assert torch.equal(c1[r, :k], c2[r, :k]) and torch.equal(i1[r, :k], i2[r, :k])
    temps = torch.tensor([0.7, 1.0, 1.5], device=DEV)
    us = torch.tensor([0.1, 0.5, 0.93], dtype=torch.float64, device=DEV)
    ops.sample_temperature(logits, temps, us, a, rows=idx)
    ops.sample_temperature(sub, temps, us, b)
    assert torch.equal(a, b)
    got = torch.empty(3, vocab, device=DEV)
    ops.gather_rows(logits, idx, got)
    assert torch.equal(got, sub)


def test_tensor_pipe_probe_times_the_attention_products(ops):
    """The measuring kernel of ``microbench mma_probe``: both issuing threads finish, no wait gives
    up, and a step of score products takes at least its 512 cycles of arithmetic and not ten
    times as long."""
    import ctypes
    from axon_b200.kernels import fast, lib
    scratch = torch.zeros(2, dtype=torch.int64, device=DEV)
    cycles = (ctypes.c_ulonglong * 2)()
    steps = 200
    fast.check(lib.cuda().axon_mma_probe(1, steps, scratch.data_ptr(), cycles, fast._stream()))
    assert 512 <= cycles[0] / steps <= 5120 and cycles[1] == 0
    fast.check(lib.cuda().axon_mma_probe(5, steps, scratch.data_ptr(), cycles, fast._stream()))
    assert cycles[0] / steps >= 1024 and cycles[1] / steps >= 1024
    assert lib.cuda().axon_mma_probe(1, 0, scratch.data_ptr(), cycles, fast._stream()) != 0      # refused: no steps
