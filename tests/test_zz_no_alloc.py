"""The decode-attention entry point that allocates nothing
(``axon_attention_fa_decode_noalloc``, declared in
``axon_b200/csrc/cuda/attention_fa_noalloc.h``).

It is for callers that may not call cudaMalloc: a host program with a fixed memory plan
that hands out its own buffers and forbids later allocations, or a plug-in that must not
go around its host's allocator.  The split partials go to a 16 MiB array inside the
library instead of caller-provided scratch.  The test calls it through its exported C
symbol, twice in a row with different inputs (the array keeps the first call's
contents, which must not leak into the second: before each of them a call with NaN
queries of another shape fills the array with NaN partials), and compares each result
bit for bit with the regular entry point given scratch and counters from PyTorch (the
same fold, so any difference is a fault of the plumbing) and, within the tolerance of
the kernel tests, with a float64 softmax written out in the test.  It also checks that
a launch too large for the array is refused with a message.  This file is collected last so that a run
stopping at the first failure has run every other test before.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(seed, shapes, heads, kv_heads, hd, ps):
    from axon_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    max_pos = max(kv for _, kv in shapes)
    stride = -(-max_pos // ps)
    slots = len(shapes)
    n_pages = slots * stride
    pool = (torch.randn(n_pages + 1, 1, 2, kv_heads, ps, hd, generator=g) * 0.7).to(torch.bfloat16).to(DEV)
    table = torch.randperm(n_pages, generator=g).to(torch.int32).view(slots, stride).to(DEV)
    view = ops.KvView(pool, table, 0, ps, kv_heads, hd, 0)
    n_tok = sum(n for n, _ in shapes)
    q = torch.randn(n_tok, heads * hd, generator=g).to(torch.bfloat16).to(DEV)
    seg = [[], [], [], []]
    at = 0
    for s, (n, kv) in enumerate(shapes):
        for lst, v in zip(seg, (s, at, n, kv)):
            lst.append(v)
        at += n
    segments = torch.tensor(seg, dtype=torch.int32, device=DEV)
    items = torch.tensor([[s, 0] for s in range(slots)], dtype=torch.int32, device=DEV).flatten()
    return view, q, segments, items


def _oracle(view, q, shapes, heads, hd):
    """softmax(q k / sqrt(hd)) v in float64, gathered through the block table."""
    kvh, ps = view.kv_heads, view.page_size
    group = heads // kvh
    pool, table = view.pool.double().cpu(), view.block_table.cpu()
    qd = q.double().cpu().view(-1, heads, hd)
    out = torch.zeros_like(qd)
    at = 0
    for s, (n, kv) in enumerate(shapes):
        pages = table[s, : -(-kv // ps)].long()
        k = pool[pages, 0, 0].permute(1, 0, 2, 3).reshape(kvh, -1, hd)[:, :kv]
        v = pool[pages, 0, 1].permute(1, 0, 2, 3).reshape(kvh, -1, hd)[:, :kv]
        for j in range(n):
            pos = kv - n + j
            for h in range(heads):
                sc = (k[h // group, : pos + 1] @ qd[at + j, h]) / math.sqrt(hd)
                out[at + j, h] = torch.softmax(sc, 0) @ v[h // group, : pos + 1]
        at += n
    return out.view(-1, heads * hd)


def _call(fn, view, q, segments, items, heads, hd, splits, scratch, out=None, counters=None):
    out = torch.zeros_like(q) if out is None else out
    n_seg = segments.shape[1]
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(hd)
    group = heads // view.kv_heads
    if scratch is None:
        rc = fn(q.data_ptr(), view.pool.data_ptr(), out.data_ptr(), segments.data_ptr(), n_seg, items.data_ptr(),
                items.numel() // 2, view._ref, heads, scale, 0, 16 // group, splits, stream)
    else:
        rc = fn(q.data_ptr(), view.pool.data_ptr(), out.data_ptr(), segments.data_ptr(), n_seg, items.data_ptr(),
                items.numel() // 2, view._ref, heads, scale, 0, 1, 16 // group, splits, scratch.data_ptr(),
                None if counters is None else counters.data_ptr(), stream)
    torch.cuda.synchronize()
    return rc, out


def test_no_alloc_entry_point_matches_the_regular_one():
    from axon_b200.kernels import lib
    cu = lib.cuda()
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    noalloc = cu.axon_attention_fa_decode_noalloc          # the exported C symbol
    noalloc.restype = I
    noalloc.argtypes = [P, P, P, P, I, P, I, ctypes.POINTER(lib.KvLayout), I, F, I, I, I, P]
    regular = cu.axon_attention_fa
    heads, kv_heads, hd, ps = 14, 2, 128, 16
    for call, (seed, shapes, splits) in enumerate([(1, [(1, 700), (1, 90), (2, 333)], 5),
                                                   (2, [(1, 64), (1, 1), (1, 1000), (2, 129)], 7)]):
        # first a call of another shape whose queries are NaN: every partial it leaves in the
        # built-in array is NaN, so a slot that the next call read without writing it would show
        nview, nq, nseg, nitems = _setup(90 + call, [(1, 500)] * 6, heads, kv_heads, hd, ps)
        rc, poisoned = _call(noalloc, nview, torch.full_like(nq, float("nan")), nseg, nitems, heads, hd, 8, None)
        assert rc == 0 and bool(poisoned.float().isnan().all())
        view, q, segments, items = _setup(seed, shapes, heads, kv_heads, hd, ps)
        n_items = items.numel() // 2
        scratch = torch.empty(n_items * kv_heads * splits * 16 * (hd + 2), dtype=torch.float32, device=DEV)
        counters = torch.zeros(n_items * kv_heads, dtype=torch.int32, device=DEV)
        rc_ref, want = _call(regular, view, q, segments, items, heads, hd, splits, scratch, counters=counters)
        got = torch.zeros_like(q)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc, got = _call(noalloc, view, q, segments, items, heads, hd, splits, None, out=got)
        assert rc_ref == 0 and rc == 0, cu.axon_last_error().decode()
        assert torch.cuda.mem_get_info()[0] >= free_before, "the call took device memory"
        assert torch.equal(got, want), f"call {call}: differs from the regular entry point given the same fold"
        oracle = _oracle(view, q, shapes, heads, hd)
        scale = float(oracle.abs().max())
        err = float((got.double().cpu() - oracle).abs().max())
        assert err <= 1.5e-2 * scale, f"call {call}: error {err:.3e} = {err / scale:.2e} of the float64 softmax's scale"
    # a launch whose partials do not fit the built-in array is refused, with a reason
    view, q, segments, items = _setup(3, [(1, 40)] * 8, heads, kv_heads, hd, ps)
    big_items = items.repeat(600)                      # 4800 items x 2 heads x 4 splits x 16 x 130 floats
    rc, _ = _call(noalloc, view, q, segments, big_items, heads, hd, 4, None)
    assert rc == 1
    msg = cu.axon_last_error().decode()
    assert "floats of scratch" in msg and "holds" in msg
