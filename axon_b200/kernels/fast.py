"""The tuned sm_100a kernels of the bfloat16 path.

Each function returns True when it ran and False when it refuses the sizes or
dtypes, in which case the caller takes the plain kernel.  What each kernel needs is
checked here, before the launch, so a refusal never costs a failed launch.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import lib
from .lib import check

EPI_STORE_F32, EPI_STORE_BF16, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
#: Which of the two tcgen05 kernels a product takes.  The swapped one has the tokens as the MMA's
#: columns and streams each weight row once: always up to 32 rows, never beyond 1,024, and between
#: those whichever the launchers' two time models call faster (``axon_gemm_prefers_swapped``:
#: products that may leave their partial sums to the reader, q/k/v, o and down in the standard
#: block, stay swapped up to a few hundred rows; wide products that may not, gate/up and the head,
#: leave it from 33 or 64 rows on).  SWAP_RULE: "model", or for tests and measurements
#: "always" (wherever the swapped kernel takes the size) and "never".
SWAP_RULE = "model"
SWAP_MAX_ROWS = 1024


def _takes_swapped_kernel(M: int, N: int, K: int, deferred: bool = False) -> bool:
    """``deferred``: the caller takes a PendingFold (a split product may skip its own fold)."""
    if SWAP_RULE == "never":
        return False
    if SWAP_RULE == "always":
        return M <= SWAP_MAX_ROWS
    return bool(lib.cuda().axon_gemm_prefers_swapped(M, N, K, SPLIT_TARGET_CTAS, int(deferred and DEFER_FOLD)))

#: switches for tests that compare a tuned kernel with the plain one
ENABLED = {"gemm_tc_small": True, "gemm_tc": True, "attention_prefill": True,
           "attention_decode": True, "attention_tc": True, "attention_fused": True}


_stream = lib.current_stream


_SPLIT_SCRATCH = {}
#: how many CTAs a product for few rows aims at (K is cut into slabs until there are about
#: this many): one per SM measured best, because the CTAs of the next kernel then fit beside them and preload their weights
SPLIT_TARGET_CTAS = 148


def _split_scratch(device: torch.device):
    """Scratch of the split-K products of one device: partial tiles (about two CTAs per SM
    times 64 tokens times 128 rows) and zeroed tile counters that the kernel leaves zeroed."""
    got = _SPLIT_SCRATCH.get(device)
    if got is None:
        got = (torch.empty(8 * SM_COUNT * 64 * 128, dtype=torch.float32, device=device),
               torch.zeros(1024, dtype=torch.int32, device=device),      # tile counters of the products
               torch.zeros(4096, dtype=torch.int32, device=device))      # split counters of attention
        _SPLIT_SCRATCH[device] = got
    return got


class PendingFold:
    """The partial sums a split-K product left in scratch instead of its output: whoever reads
    ``out`` next adds them (``ops.rmsnorm(..., pending=)``, ``ops.rope_kv_write(..., pending=)``)
    or calls ``ops.fold_partials``.  One may be outstanding per device (the scratch is shared);
    starting another split product before it is claimed is an error, not a wrong result."""

    def __init__(self, partial, splits, ntok, bias, out, accumulate):
        self.partial, self.splits, self.ntok, self.bias = partial, splits, ntok, bias
        self.out, self.accumulate = out, accumulate
        self.claimed = False

    def claim(self, tensor: torch.Tensor, accumulate: bool) -> None:
        if self.claimed:
            raise RuntimeError("these partial sums were folded already")
        if tensor.data_ptr() != self.out.data_ptr() or accumulate != self.accumulate:
            raise RuntimeError("partial sums folded into a tensor (or in a way) they were not made for")
        self.claimed = True
        if _OUTSTANDING.get(self.out.device) is self:
            _OUTSTANDING[self.out.device] = None


_OUTSTANDING = {}


def forget_owed(device: torch.device) -> None:
    """Drop the record of partial sums nobody claimed (a step that failed half way leaves one)."""
    device = torch.device(device)
    for k in list(_OUTSTANDING):
        if k.type == device.type and (device.index is None or k.index == device.index):
            _OUTSTANDING[k] = None

#: whether products for few rows may leave their partial sums to the reader of the output
#: (tests switch it off to compare the two ways of folding)
DEFER_FOLD = True


def _gemm_small(a, w, bias, out, epi, M, N, K, defer: bool = False):
    """Few rows (``_takes_swapped_kernel``): the swapped tcgen05 kernel.  With ``defer`` a
    split product returns a PendingFold instead of folding its partial sums itself."""
    if ENABLED["gemm_tc_small"]:
        partial, counters, _ = _split_scratch(a.device)
        owed = _OUTSTANDING.get(a.device)
        if owed is not None and not owed.claimed:
            raise RuntimeError("a product's partial sums were never folded into its output "
                               "(PendingFold dropped): the scratch they lie in is about to be overwritten")
        plan = (ctypes.c_int * 3)()
        check(lib.cuda().axon_gemm_tc_small(a.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(),
                                            out.data_ptr(), epi, M, N, K, out.stride(0), partial.data_ptr(),
                                            partial.numel(), counters.data_ptr(), counters.numel(),
                                            SPLIT_TARGET_CTAS, int(defer and DEFER_FOLD), plan, _stream()))
        if plan[2]:
            owed = PendingFold(partial, plan[0], plan[1], bias, out, epi == EPI_RESIDUAL)
            _OUTSTANDING[a.device] = owed
            return owed
        return True
    return False


def _bf16_operands(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
            and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor],
         accumulate: bool, defer: bool = False):
    """True when it ran, False when it refuses; with ``defer`` possibly a PendingFold (the
    output is still owed the partial sums of a split product)."""
    if not _bf16_operands(a, w):
        return False
    M, K = a.shape
    N = w.shape[0]
    if accumulate:
        if out.dtype != torch.float32:
            return False
        epi = EPI_RESIDUAL
    elif out.dtype == torch.float32:
        epi = EPI_STORE_F32
    elif out.dtype == torch.bfloat16:
        epi = EPI_STORE_BF16
    else:
        return False
    defer = defer and out.is_contiguous() and epi in (EPI_STORE_F32, EPI_RESIDUAL)
    if _takes_swapped_kernel(M, N, K, defer):
        ran = _gemm_small(a, w, bias, out, epi, M, N, K, defer)
        if ran:
            return ran
    if ENABLED["gemm_tc"]:
        check(lib.cuda().axon_gemm_tc(a.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(),
                                      out.data_ptr(), epi, M, N, K, out.stride(0), _stream()))
        return True
    return False


def gemm_tc_status() -> int:
    """0 when no tensor-core product ever gave up on a wait (synchronises the device)."""
    return lib.cuda().axon_gemm_tc_status()


def attention_tc_status() -> int:
    """0 when no tensor-core attention ever gave up on a wait (synchronises the device)."""
    return lib.cuda().axon_attention_tc_status()


def gemm_swiglu(h: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor) -> bool:
    if not _bf16_operands(h, w_gate_up) or act.dtype != torch.bfloat16:
        return False
    M, K = h.shape
    N = w_gate_up.shape[0]
    if _takes_swapped_kernel(M, N, K) and _gemm_small(h, w_gate_up, None, act, EPI_SWIGLU, M, N, K):
        return True
    if ENABLED["gemm_tc"]:
        check(lib.cuda().axon_gemm_tc(h.data_ptr(), w_gate_up.data_ptr(), None, act.data_ptr(), EPI_SWIGLU,
                                      M, N, K, act.stride(0), _stream()))
        return True
    return False


FA_HEAD_DIMS = (16, 32, 64, 128)
FA_MAX_SPLITS = 64
#: CTAs the decode attention never exceeds when it splits the keys of each request: two CTAs fit
#: an SM, and a launch that spills into a second wave pays for it (measured at 7B sizes: 320 CTAs
#: at batch 16 cost 10 % of the step against 256)
FA_TARGET_CTAS = 2 * 148
#: the split rule's model, in units of one key tile's time in a CTA: what each further share adds to
#: the fold, and what the fold's kernel costs when there is one
FA_SPLIT_COST = 0.15
FA_FOLD_COST = 2.0
#: launches of more CTAs than this pay a further tile's time in the model
FA_ROOMY_CTAS, FA_CROWD_COST = 256, 1.0
#: whether the last split folds the partials itself (else a second kernel does; measured at 7B
#: sizes the second kernel is a little faster up to batch 8 and equal at 64, because it overlaps
#: with the kernels around it while the in-kernel fold lengthens the slowest CTA)
#: (the entry point that allocates nothing folds this way; tests switch it on to cover it)
FA_FOLD_IN_KERNEL = False
SM_COUNT = 148


def _attention_items(ctx, group: int, pre_rows: int = 64):
    """Work lists for the step's segments, cached per step and group size: segments that
    fit a 16-row tile (one or two decoded tokens) go to the decode shape, the others are
    cut into tiles of up to `pre_rows` rows."""
    key = ("fa_items", group, pre_rows)
    got = ctx.scratch.get(key)
    if got is not None:
        return got
    tpt_dec, tpt_pre = (16 // group if group <= 16 else 0), pre_rows // group
    if ctx.unit_items is not None:
        # single tokens only: the step brought its work list (segment, 0) along
        n = len(ctx.seg_q_len)
        # (the decode shape takes "no list" to mean item i = segment i, which saves it a load)
        got = {"dec": None, "n_dec": n if tpt_dec else 0, "dec_kv": ctx.max_kv_len,
               "pre": None if tpt_dec else ctx.unit_items, "n_pre": 0 if tpt_dec else n,
               "tpt_dec": tpt_dec, "tpt_pre": tpt_pre}
        ctx.scratch[key] = got
        return got
    dec, pre, pre_work = [], [], []
    dec_kv = 0
    for s, (n, kv_len) in enumerate(zip(ctx.seg_q_len, ctx.seg_kv_len)):
        if tpt_dec and n <= tpt_dec:
            dec += [s, 0]
            dec_kv = max(dec_kv, kv_len)
        else:
            for t0 in range(0, n, tpt_pre):
                pre_work.append((kv_len - n + min(t0 + tpt_pre, n), s, t0))
    # tiles with the most keys first: a causal tile's work grows with its position, and the
    # long ones must not be the last to start
    for _, s, t0 in sorted(pre_work, reverse=True):
        pre += [s, t0]
    both = ctx.rt.upload_i32(f"fa_items_{group}_{pre_rows}", dec + pre) if dec or pre else None
    got = {"dec": both[:len(dec)] if dec else None, "n_dec": len(dec) // 2, "dec_kv": dec_kv,
           "pre": both[len(dec):] if pre else None, "n_pre": len(pre) // 2,
           "tpt_dec": tpt_dec, "tpt_pre": tpt_pre}
    ctx.scratch[key] = got
    return got


def _key_splits(pairs: int, tiles: int) -> int:
    """Into how many shares to cut the keys of each of ``pairs`` (request, kv head) whose longest
    context has ``tiles`` key tiles.  All CTAs must fit at once (``FA_TARGET_CTAS``); among the
    counts that do, the cheapest by a small model: the key tiles of the longest share, plus what
    every further share costs the fold, plus the fold's own kernel when there is more than one, plus
    a little when the launch takes nearly every place on the GPU.  Measured at 7B sizes and 2,048 keys:
    against "as many shares as fit in 256 CTAs" the step is 2 % faster at batch 24 (3 shares instead
    of 2) and 7 % at batch 36 (2 instead of 1), and the same at batches 1 to 16; 288 CTAs instead of
    256 at batch 8 (9 shares of 4 tiles instead of 8 of 5) was 1.3 % slower, hence the last term."""
    most = max(1, min(tiles, FA_MAX_SPLITS, FA_TARGET_CTAS // max(pairs, 1)))
    best, best_cost = 1, float(tiles)
    for s in range(2, most + 1):
        cost = -(-tiles // s) + FA_SPLIT_COST * s + FA_FOLD_COST + (FA_CROWD_COST if pairs * s > FA_ROOMY_CTAS else 0.0)
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def decode_split_count(n_dec: int, kv_heads: int, max_kv_len: int) -> int:
    """Into how many shares the decode attention cuts each request's keys: the one launch
    parameter of a step of single tokens that depends on the contexts' lengths."""
    return _key_splits(n_dec * kv_heads, -(-max_kv_len // 64))


def _decode_splits(n_dec: int, kv, tiles: int, rt):
    """Key splits for the decode shape and the scratch their partials go to (None: one split)."""
    splits = _key_splits(n_dec * kv.kv_heads, tiles)
    scratch = None
    if splits > 1:
        # sized for the most splits this batch can get, so that the buffer never moves
        # while the contexts grow (captured graphs hold its address)
        most = max(1, min(FA_MAX_SPLITS, FA_TARGET_CTAS // (n_dec * kv.kv_heads)))
        scratch = rt.buffer("fa_scratch", (n_dec * kv.kv_heads * most * 16 * (kv.head_dim + 2),), torch.float32)
    return splits, scratch


def attention_decode_fused(qkv, pending, table, rot: int, adjacent: bool, kv, ctx, out, heads: int, scale: float,
                           write_kv: bool) -> bool:
    """Rotation, cache write and attention of a step of single tokens in one kernel: reads
    the q/k/v product (or the partial sums it is still owed) instead of rotated queries.
    Refuses what ``attention`` refuses, steps with prompt portions, partial or adjacent-pair
    rotation, and head sizes that are no multiple of 8; the caller then takes the two kernels."""
    if not (ENABLED["attention_decode"] and ENABLED["attention_fused"]) or ctx.unit_items is None:
        return False
    if out.dtype != torch.bfloat16 or kv.pool.dtype != torch.bfloat16 or kv.head_dim not in FA_HEAD_DIMS:
        return False
    if kv.planes != 2 or kv.v_dim != kv.head_dim:
        return False
    if heads % kv.kv_heads or heads // kv.kv_heads > 16 or ctx.segments is None or qkv.dtype != torch.float32:
        return False
    if table is not None and (adjacent or rot != kv.head_dim):
        return False
    if not qkv.is_contiguous() or (table is not None and not table.is_contiguous()):
        return False
    n = len(ctx.seg_slot)
    tiles = -(-ctx.max_kv_len // 64)
    splits, scratch = _decode_splits(n, kv, tiles, ctx.rt)
    # every CTA rotates its own queries: worth it while all CTAs run at once (three per SM);
    # beyond that the separate rotation kernel is cheaper (measured at batch 64: 15 % of the step)
    if n * kv.kv_heads * splits > 3 * SM_COUNT:
        return False
    counters = _split_scratch(qkv.device)[2]
    if pending is not None:
        pending.claim(qkv, accumulate=False)
    check(lib.cuda().axon_attention_fa_decode_fused(
        qkv.data_ptr(), None if pending is None else pending.partial.data_ptr(),
        0 if pending is None else pending.splits, 0 if pending is None else pending.ntok,
        None if pending is None or pending.bias is None else pending.bias.data_ptr(),
        None if table is None else table.data_ptr(), int(write_kv), kv.pool.data_ptr(), out.data_ptr(),
        ctx.segments.data_ptr(), n, kv._ref, heads, float(scale), int(kv.window), 16 // (heads // kv.kv_heads),
        ctx.max_q_len, splits,
        None if scratch is None else scratch.data_ptr(),
        counters.data_ptr() if FA_FOLD_IN_KERNEL and n * kv.kv_heads <= counters.numel() else None, _stream()))
    return True


def attention(q, kv, ctx, out, heads: int, scale: float) -> bool:
    """Tensor-core attention over the paged cache; refuses head sizes other than
    16/32/64/128, groups of more than 64 heads, and dtypes other than bfloat16."""
    if not (ENABLED["attention_prefill"] and ENABLED["attention_decode"]):
        return False
    if q.dtype != torch.bfloat16 or kv.pool.dtype != torch.bfloat16 or kv.head_dim not in FA_HEAD_DIMS:
        return False
    if kv.planes != 2 or kv.v_dim != kv.head_dim:
        return False
    if heads % kv.kv_heads or heads // kv.kv_heads > 64 or ctx.segments is None:
        return False
    group = heads // kv.kv_heads
    # prompt portions at head size 128 take the tcgen05 kernel with tiles of 256 rows (two sub-tiles of 128)
    use_tc = ENABLED["attention_tc"] and kv.head_dim == 128 and ctx.unit_items is None
    it = _attention_items(ctx, group, 256 if use_tc else 64)
    cu = lib.cuda()
    n_seg = len(ctx.seg_slot)
    if it["n_dec"]:
        tiles = -(-it["dec_kv"] // 64)
        splits, scratch = _decode_splits(it["n_dec"], kv, tiles, ctx.rt)
        counters = _split_scratch(q.device)[2]
        check(cu.axon_attention_fa(q.data_ptr(), kv.pool.data_ptr(), out.data_ptr(), ctx.segments.data_ptr(), n_seg,
                                   None if it["dec"] is None else it["dec"].data_ptr(), it["n_dec"], kv._ref, heads,
                                   float(scale), int(kv.window),
                                   1, it["tpt_dec"], splits, None if scratch is None else scratch.data_ptr(),
                                   counters.data_ptr() if FA_FOLD_IN_KERNEL and it["n_dec"] * kv.kv_heads <= counters.numel() else None,
                                   _stream()))
    if it["n_pre"] and use_tc:
        check(cu.axon_attention_tc(q.data_ptr(), kv.pool.data_ptr(), out.data_ptr(), ctx.segments.data_ptr(), n_seg,
                                   it["pre"].data_ptr(), it["n_pre"], kv._ref, heads, float(scale), int(kv.window),
                                   it["tpt_pre"], _stream()))
    elif it["n_pre"]:
        check(cu.axon_attention_fa(q.data_ptr(), kv.pool.data_ptr(), out.data_ptr(), ctx.segments.data_ptr(), n_seg,
                                   it["pre"].data_ptr(), it["n_pre"], kv._ref, heads, float(scale), int(kv.window),
                                   0, it["tpt_pre"], 1, None, None, _stream()))
    return True
