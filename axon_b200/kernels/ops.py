"""The engine's operations on device tensors, each a hand-written CUDA kernel.

Every function launches on the current CUDA stream and returns nothing: outputs
are tensors the caller passes in.  Tensors must live on the GPU; there is no CPU
path.  ``precise=True`` (the 32-bit model) always takes the plain FFMA kernels; the
bfloat16 model takes the tuned sm_100a kernels where the sizes allow and the plain
ones otherwise.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib
from .lib import KvLayout, check

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"dtype {t.dtype} is not one the kernels take (float32, bfloat16)") from None


def _dev(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("kernels take contiguous CUDA tensors; there is no CPU path")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_stream = lib.current_stream


@dataclass
class KvView:
    """One schedule entry's keys and values inside its group's page pool.

    ``pool`` is ``[pages + 1][entries][2][kv_heads][page_size][head_dim]`` (the last
    page is the sink) when keys and values are alike, else ``[pages + 1][entries][elements]``
    with an entry's key plane ``[kv_heads][page_size][head_dim]`` followed, when ``planes``
    is 2, by its value plane ``[kv_heads][page_size][v_dim]``.  With one plane the kernels
    read values from the key plane.  ``block_table`` is the group's device table
    ``[slots][stride]`` of int32.  ``fault`` (two uint32 on the device) switches checked
    tables on: see ``kv_layout.h``.
    """

    pool: torch.Tensor
    block_table: torch.Tensor
    entry: int
    page_size: int
    kv_heads: int
    head_dim: int
    window: int = 0
    v_dim: int = 0
    planes: int = 2
    fault: Optional[torch.Tensor] = None

    def __post_init__(self) -> None:
        if self.planes not in (1, 2):
            raise ValueError(f"a cache entry has one or two planes, not {self.planes}")
        self.v_dim = self.head_dim if self.planes == 1 or not self.v_dim else self.v_dim
        entries = self.pool.shape[1]
        self.k_plane = self.kv_heads * self.page_size * self.head_dim
        self.v_plane = self.kv_heads * self.page_size * self.v_dim if self.planes == 2 else 0
        per_entry = self.k_plane + self.v_plane
        if self.pool[0].numel() != entries * per_entry:
            raise ValueError(f"a page of {self.pool[0].numel()} elements does not hold {entries} entries of {per_entry}")
        self.n_pages = self.pool.shape[0] - 1
        self.layout = KvLayout(
            block_table=self.block_table.data_ptr(), table_stride=self.block_table.shape[1],
            page_size=self.page_size, kv_heads=self.kv_heads, head_dim=self.head_dim,
            page_stride=entries * per_entry, entry_offset=self.entry * per_entry,
            v_offset=self.k_plane if self.planes == 2 else 0, v_dim=self.v_dim, planes=self.planes,
            n_pages=self.n_pages, reserved=0, fault=None if self.fault is None else self.fault.data_ptr())
        self._ref = ctypes.byref(self.layout)

    def _plane(self, offset: int, dim: int) -> torch.Tensor:
        flat = self.pool.view(self.pool.shape[0], -1)
        start = self.layout.entry_offset + offset
        return flat[:, start:start + self.kv_heads * self.page_size * dim].view(-1, self.kv_heads, self.page_size, dim)

    def keys(self) -> torch.Tensor:
        """This entry's key rows as a view ``[pages + 1][kv_heads][page_size][head_dim]``."""
        return self._plane(0, self.head_dim)

    def values(self) -> torch.Tensor:
        """Its value rows ``[pages + 1][kv_heads][page_size][v_dim]`` (the key rows with one plane)."""
        return self._plane(self.layout.v_offset, self.v_dim)


def embed(tokens: torch.Tensor, table: torch.Tensor, x: torch.Tensor, scale: float = 1.0) -> None:
    _dev(tokens, table, x)
    n, dim = x.shape
    check(lib.cuda().axon_embed(_ptr(tokens), _ptr(table), dtype_code(table), _ptr(x), n, dim, scale, _stream()))


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None, unit_offset: bool = False, pending=None) -> None:
    """out[r] = norm(x[rows[r]] if rows is given else x[r]); x and gain are float32.

    ``pending`` (a ``fast.PendingFold`` whose output is ``x``): the partial sums that a
    split-K product still owes ``x`` are added to the rows read (and written back) first."""
    _dev(x, gain, out, rows)
    if x.dtype != torch.float32 or gain.dtype != torch.float32:
        raise TypeError("rmsnorm reads a float32 residual and a float32 gain")
    n, dim = out.shape
    if pending is not None:
        pending.claim(x, accumulate=True)
        check(lib.cuda().axon_rmsnorm_fold(_ptr(x), _ptr(gain), _ptr(rows), _ptr(out), dtype_code(out), n, dim,
                                           float(eps), int(unit_offset), _ptr(pending.partial), pending.splits,
                                           pending.ntok, _ptr(pending.bias), _stream()))
        return
    check(lib.cuda().axon_rmsnorm(_ptr(x), _ptr(gain), _ptr(rows), _ptr(out), dtype_code(out), n, dim,
                                  float(eps), int(unit_offset), _stream()))


def fold_partials(pending) -> None:
    """Bring the output of a deferred split-K product up to date (for readers that cannot
    fold the partial sums themselves)."""
    out = pending.out
    accumulate = pending.accumulate
    pending.claim(out, accumulate=accumulate)
    check(lib.cuda().axon_fold_partials(_ptr(pending.partial), pending.splits, pending.ntok, _ptr(pending.bias),
                                        _ptr(out), dtype_code(out), out.shape[0], out.shape[1], out.stride(0),
                                        int(accumulate), _stream()))


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
               accumulate: bool = False) -> None:
    """out = a @ w.T (+ bias), or out += ... when ``accumulate``; FFMA, any sizes."""
    _dev(a, w, out, bias)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise ValueError(f"gemm shapes do not fit: a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise ValueError("a bias is float32 with one value per output column")
    check(lib.cuda().axon_gemm_plain(_ptr(a), dtype_code(a), _ptr(w), dtype_code(w), _ptr(bias), _ptr(out),
                                     dtype_code(out), M, N, K, K, N, int(accumulate), _stream()))


def swiglu(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act[t][j] = silu(gate_up[t][2j]) * gate_up[t][2j+1]; gate_up is float32."""
    _dev(gate_up, act)
    n, ffn = act.shape
    if gate_up.dtype != torch.float32 or gate_up.shape != (n, 2 * ffn):
        raise ValueError("swiglu reads float32 [n][2 * ffn] with gate and up interleaved")
    check(lib.cuda().axon_swiglu(_ptr(gate_up), _ptr(act), dtype_code(act), n, ffn, _stream()))


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor, magnitude: float = 1.0) -> None:
    """table[t][i] = (cos, sin)(positions[t] * inv_freq[i]); inv_freq is float64."""
    _dev(positions, inv_freq, table)
    n, half = table.shape[0], table.shape[1]
    if inv_freq.dtype != torch.float64 or inv_freq.numel() != half or table.dtype != torch.float32:
        raise ValueError("rope_table takes float64 frequencies and writes float32 [n][half][2]")
    check(lib.cuda().axon_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), n, half, float(magnitude), _stream()))


def rope_kv_write(qkv: torch.Tensor, table: Optional[torch.Tensor], positions: torch.Tensor,
                  token_slot: torch.Tensor, q_out: torch.Tensor, kv: KvView, heads: int, rot: int,
                  adjacent: bool = False, write_kv: bool = True, pending=None) -> None:
    """``pending`` (a ``fast.PendingFold`` whose output is ``qkv``): the product is still in
    partial sums; they are folded here (with the bias) and ``qkv`` itself is not read."""
    _dev(qkv, table, positions, token_slot, q_out, kv.pool)
    n = q_out.shape[0]
    width = (heads + kv.kv_heads) * kv.head_dim + (kv.kv_heads * kv.v_dim if kv.planes == 2 else 0)
    if qkv.dtype != torch.float32 or qkv.shape[1] != width:
        raise ValueError("rope_kv_write reads float32 [n][(heads + kv_heads) * head_dim + kv_heads * v_dim]")
    if q_out.dtype != kv.pool.dtype:
        raise TypeError("queries and the cache have one dtype")
    if pending is not None:
        pending.claim(qkv, accumulate=False)
    check(lib.cuda().axon_rope_kv_write(_ptr(qkv), _ptr(table), _ptr(positions), _ptr(token_slot), _ptr(q_out),
                                        _ptr(kv.pool), dtype_code(q_out), kv._ref, n, heads, rot, int(adjacent),
                                        int(write_kv), None if pending is None else _ptr(pending.partial),
                                        0 if pending is None else pending.splits,
                                        0 if pending is None else pending.ntok,
                                        None if pending is None else _ptr(pending.bias), _stream()))


def attention_plain(q: torch.Tensor, kv: KvView, positions: torch.Tensor, token_slot: torch.Tensor,
                    out: torch.Tensor, heads: int, scale: float) -> None:
    _dev(q, positions, token_slot, out, kv.pool)
    n = q.shape[0]
    if q.dtype != kv.pool.dtype or out.dtype != q.dtype:
        raise TypeError("queries, cache and output have one dtype")
    check(lib.cuda().axon_attention_plain(_ptr(q), _ptr(kv.pool), dtype_code(q), _ptr(positions), _ptr(token_slot),
                                          _ptr(out), kv._ref, n, heads, float(scale), int(kv.window), _stream()))


def residual_add(x: torch.Tensor, y: torch.Tensor) -> None:
    _dev(x, y)
    if x.dtype != torch.float32 or x.numel() != y.numel():
        raise ValueError("the residual is float32 and as large as what is added")
    check(lib.cuda().axon_residual_add(_ptr(x), _ptr(y), dtype_code(y), x.numel(), _stream()))


def convert(src: torch.Tensor, dst: torch.Tensor) -> None:
    _dev(src, dst)
    if src.numel() != dst.numel():
        raise ValueError("convert needs equally large tensors")
    check(lib.cuda().axon_convert(_ptr(src), dtype_code(src), _ptr(dst), dtype_code(dst), src.numel(), _stream()))


def argmax(logits: torch.Tensor, best: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """best[r] = the id of the largest logit of row r, or of row ``rows[r]`` when given."""
    _dev(logits, best, rows)
    n, vocab = best.shape[0], logits.shape[1]
    if rows is None:
        check(lib.cuda().axon_argmax(_ptr(logits), _ptr(best), n, vocab, logits.stride(0), _stream()))
    else:
        check(lib.cuda().axon_argmax_rows(_ptr(logits), _ptr(rows), _ptr(best), n, vocab, logits.stride(0), _stream()))


def gather_rows(src: torch.Tensor, rows: Optional[torch.Tensor], dst: torch.Tensor) -> None:
    """dst[r] = src[rows[r]] (float32 rows; ``rows`` None copies them in order)."""
    _dev(src, rows, dst)
    if src.dtype != torch.float32 or dst.dtype != torch.float32 or dst.shape[1] != src.shape[1]:
        raise ValueError("gather_rows copies float32 rows of one width")
    check(lib.cuda().axon_gather_rows(_ptr(src), _ptr(rows), _ptr(dst), dst.shape[0], dst.shape[1], src.stride(0), _stream()))


def repeat_penalty(logits: torch.Tensor, ids: torch.Tensor, penalty: torch.Tensor) -> None:
    _dev(logits, ids, penalty)
    rows, vocab = logits.shape
    check(lib.cuda().axon_repeat_penalty(_ptr(logits), _ptr(ids), _ptr(penalty), rows, vocab, logits.stride(0),
                                         ids.shape[1], _stream()))


def topk_max() -> int:
    return lib.cuda().axon_topk_max()


def topk(logits: torch.Tensor, ks: torch.Tensor, cand_logit: torch.Tensor, cand_id: torch.Tensor,
         rows: Optional[torch.Tensor] = None) -> None:
    _dev(logits, ks, cand_logit, cand_id, rows)
    n, vocab = ks.shape[0], logits.shape[1]
    check(lib.cuda().axon_topk(_ptr(logits), _ptr(rows), _ptr(ks), _ptr(cand_logit), _ptr(cand_id), n, vocab,
                               logits.stride(0), _stream()))


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                       picked: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    _dev(logits, temperature, uniform, picked, rows)
    n, vocab = picked.shape[0], logits.shape[1]
    if uniform.dtype != torch.float64 or temperature.dtype != torch.float32:
        raise TypeError("temperatures are float32, uniform numbers float64")
    check(lib.cuda().axon_sample_temperature(_ptr(logits), _ptr(rows), _ptr(temperature), _ptr(uniform), _ptr(picked), n,
                                             vocab, logits.stride(0), _stream()))
