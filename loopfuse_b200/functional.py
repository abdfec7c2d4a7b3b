"""Tensor-level entry points: torch CUDA tensors in, kernels of liblf_sm100.so out.

These are what the compiled callable produced by ``loopfuse_backend`` calls; they can also be
used directly. PyTorch only supplies device memory and the current stream here - all arithmetic
happens in the library. Nothing in this module computes attention on the CPU or with torch ops.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _native
from .spec import MASK_NONE, MAX_MODS, ScoreMod, TILE_Q

_DEV_TIMEOUT = 1
_DEV_BAD_PAGE = 2


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(
                "loopfuse_b200 kernels need CUDA tensors on an sm_100 GPU; there is no CPU path")
        if t.device != dev:
            raise ValueError("all tensors must live on the same device")
    return dev


def _check_bf16_lastdim(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must have a contiguous last dim")


def _fill_mods(args, scale: float, mods: Sequence[ScoreMod]) -> None:
    if len(mods) > MAX_MODS:
        raise ValueError(f"at most {MAX_MODS} score-mod ops")
    args.scale = float(scale)
    args.n_mod = len(mods)
    for i, m in enumerate(mods):
        args.mod_op[i] = int(m.op)
        args.mod_arg[i] = float(m.arg)


def _stream_ptr(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def new_status(device) -> torch.Tensor:
    """A zeroed device word the kernels report device-side problems into."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor, what: str = "kernel") -> None:
    """Synchronising read of a status word; raises if a kernel recorded a problem."""
    code = int(status.item())
    if code == 0:
        return
    if (code & 0xFF) == _DEV_TIMEOUT:
        raise RuntimeError(f"{what}: a bounded device-side wait ran out (site {code >> 8})")
    if (code & 0xFF) == _DEV_BAD_PAGE:
        raise RuntimeError(f"{what}: block_table holds a page id outside the pool")
    raise RuntimeError(f"{what}: device status {code}")


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0,
                      mods: Sequence[ScoreMod] = (), mask_kind: int = MASK_NONE,
                      window: int = 0, causal_offset: int = 0,
                      out: Optional[torch.Tensor] = None,
                      status: Optional[torch.Tensor] = None,
                      dbg_ranges: Optional[torch.Tensor] = None,
                      kv_tile: int = 0, sm_margin: int = 0,
                      k_block_table: Optional[torch.Tensor] = None,
                      v_block_table: Optional[torch.Tensor] = None,
                      seq_len: Optional[int] = None,
                      score_bias: Optional[torch.Tensor] = None,
                      bias_pos: Optional[int] = None,
                      q_pe: Optional[torch.Tensor] = None,
                      k_pe: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(mask(mods(scale * q k^T))) v for q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] (bf16).

    ``score_bias`` (bf16 ``[B, Hq, Sq, Skv]``) is added to the scores after the first
    ``bias_pos`` ops of ``mods`` (default: after all of them) and before the mask; the kernel
    reads it tile by tile (dense k / v only).

    ``q_pe`` ``[B, Hq, Sq, D_pe]`` and ``k_pe`` ``[B, Hkv, Skv, D_pe]`` (bf16, D_pe a multiple of
    8 up to 64) add a second product to the scores: ``scale * (q k^T + q_pe k_pe^T)``, the
    two-matmul (MLA-style) form; ``mods`` may then hold constant multipliers only.

    With ``k_block_table`` (``v_block_table``), ``k`` (``v``) is a paged pool
    ``[pages, page_size, Hkv, D]`` (or ``[pages, Hkv, D]``, one token per page) read through that
    int32 table ``[B, blocks]``; the gather is fused into the kernel's tile loads. ``seq_len``
    bounds the keys when the table covers more.

    ``kv_tile`` pins the KV tile of the kernel (64 or 128 keys; 0 lets the library choose);
    ``sm_margin`` leaves that many SMs free of the persistent kernels' CTAs (for a collective
    that runs at the same time on another stream)."""
    a, out, dev = _prefill_args(q, k, v, scale, mods, mask_kind, window, causal_offset, out,
                                status, dbg_ranges, kv_tile, sm_margin, k_block_table,
                                v_block_table, seq_len)
    if score_bias is not None:
        _require_cuda(score_bias)
        _check_bf16_lastdim(score_bias, "score_bias")
        if tuple(score_bias.shape) != (a.B, a.Hq, a.Sq, a.Skv):
            raise ValueError(f"score_bias must be [B, Hq, Sq, Skv] = "
                             f"{(a.B, a.Hq, a.Sq, a.Skv)}, got {tuple(score_bias.shape)}")
        a.score_bias = score_bias.data_ptr()
        for i in range(3):
            a.bias_stride[i] = score_bias.stride(i)
        a.bias_pos = a.n_mod if bias_pos is None else int(bias_pos)
    if (q_pe is None) != (k_pe is None):
        raise ValueError("q_pe and k_pe go together")
    if q_pe is not None:
        _require_cuda(q_pe, k_pe)
        _check_bf16_lastdim(q_pe, "q_pe")
        _check_bf16_lastdim(k_pe, "k_pe")
        if (q_pe.dim() != 4 or k_pe.dim() != 4 or q_pe.shape[:3] != q.shape[:3]
                or tuple(k_pe.shape[:3]) != (a.B, a.Hkv, a.Skv) or q_pe.shape[3] != k_pe.shape[3]):
            raise ValueError(f"q_pe {tuple(q_pe.shape)} / k_pe {tuple(k_pe.shape)} do not fit "
                             f"q {tuple(q.shape)} and the keys")
        a.q_pe, a.k_pe, a.D_pe = q_pe.data_ptr(), k_pe.data_ptr(), q_pe.shape[3]
        for i in range(3):
            a.qpe_stride[i] = q_pe.stride(i)
            a.kpe_stride[i] = k_pe.stride(i)
    with torch.cuda.device(dev):
        rc = _native.load().lf_prefill_bf16(C.byref(a), _stream_ptr(dev))
    _native.check(rc, "lf_prefill_bf16")
    return out


def add_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = a + b for bf16 [B, H, S, D] tensors of one shape (any strides with innermost 1);
    ``out`` may be ``a`` or ``b``. The query-bias and output-bias steps of a biased attention."""
    dev = _require_cuda(a, b)
    for t, n in ((a, "a"), (b, "b")):
        _check_bf16_lastdim(t, n)
    if a.dim() != 4 or a.shape != b.shape:
        raise ValueError(f"add_bf16 takes two 4-D tensors of one shape, got {tuple(a.shape)} "
                         f"and {tuple(b.shape)}")
    if out is None:
        out = torch.empty(a.shape, dtype=torch.bfloat16, device=dev)
    else:
        _require_cuda(out)
        _check_bf16_lastdim(out, "out")
        if out.shape != a.shape:
            raise ValueError("out must have the operands' shape")
    B, H, S, D = a.shape
    strides = [(C.c_int64 * 3)(*[t.stride(i) for i in range(3)]) for t in (a, b, out)]
    with torch.cuda.device(dev):
        rc = _native.load().lf_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), B, H, S, D,
                                        strides[0], strides[1], strides[2], _stream_ptr(dev))
    _native.check(rc, "lf_add_bf16")
    return out


class PreparedPrefill:
    """A prefill call bound once to its tensors and parameters, for loops that launch the same
    problem again and again (a serving step, a benchmark): the argument record of the C ABI is
    filled and validated a single time, ``run()`` only launches. This is the per-call host work
    the reference's generated launcher repeats on every call (loopfuse/codegen.py:215-298:
    output allocation, stride extraction, grid computation). The tensors are kept alive by the
    object; new data written into the same buffers is picked up by the next ``run()``."""

    def __init__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0,
                 mods: Sequence[ScoreMod] = (), mask_kind: int = MASK_NONE, window: int = 0,
                 causal_offset: int = 0, out: Optional[torch.Tensor] = None,
                 status: Optional[torch.Tensor] = None, kv_tile: int = 0,
                 sm_margin: int = 0) -> None:
        self._args, self.out, self._dev = _prefill_args(
            q, k, v, scale, mods, mask_kind, window, causal_offset, out, status, None, kv_tile,
            sm_margin)
        self._keep = (q, k, v, status)
        self._fn = _native.load().lf_prefill_bf16
        self._ref = C.byref(self._args)
        self._dev_index = self._dev.index if self._dev.index is not None else \
            torch.cuda.current_device()

    def run(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Launch on the current stream of the tensors' device (which must be the current
        device); ``out`` replaces the output buffer (same shape and strides) for this and later
        runs."""
        if out is not None:
            if out.shape != self.out.shape or out.stride() != self.out.stride():
                raise ValueError("out must match the prepared output's shape and strides")
            self.out = out
            self._args.out = out.data_ptr()
        rc = self._fn(self._ref, torch.cuda.current_stream(self._dev_index).cuda_stream)
        if rc:
            _native.check(rc, "lf_prefill_bf16")
        return self.out


def prefill_kv_tile(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0,
                    mods: Sequence[ScoreMod] = (), mask_kind: int = MASK_NONE, window: int = 0,
                    causal_offset: int = 0, kv_tile: int = 0) -> int:
    """KV tile size (64 or 128 keys) of the kernel ``prefill_attention`` runs for these
    arguments; skip ranges and ``dbg_ranges`` are in units of it."""
    a, _, _ = _prefill_args(q, k, v, scale, mods, mask_kind, window, causal_offset, q,
                            None, None, kv_tile, 0)
    rc = _native.load().lf_prefill_kv_tile(C.byref(a))
    if rc < 0:
        _native.check(rc, "lf_prefill_kv_tile")
    return rc


def prefill_q_tile(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0,
                   mods: Sequence[ScoreMod] = (), mask_kind: int = MASK_NONE, window: int = 0,
                   causal_offset: int = 0, kv_tile: int = 0) -> int:
    """Query rows per head that one tile of the kernel ``prefill_attention`` runs for these
    arguments covers (128, or 32 in the packed grouped-query layout); ``dbg_ranges`` holds one
    (lo, hi) per (batch, head, tile of that many rows)."""
    a, _, _ = _prefill_args(q, k, v, scale, mods, mask_kind, window, causal_offset, q,
                            None, None, kv_tile, 0)
    rc = _native.load().lf_prefill_q_tile(C.byref(a))
    if rc < 0:
        _native.check(rc, "lf_prefill_q_tile")
    return rc


def _prefill_args(q, k, v, scale, mods, mask_kind, window, causal_offset, out, status,
                  dbg_ranges, kv_tile, sm_margin=0, k_block_table=None, v_block_table=None,
                  seq_len=None):
    dev = _require_cuda(q, k, v)
    _check_bf16_lastdim(q, "q")
    if q.dim() != 4:
        raise ValueError("q must be 4-D")
    B, Hq, Sq, D = q.shape
    tables = {}
    Skv = None
    keep = []
    # A paged operand is a pool [pages, page_size, Hkv, D] (or [pages, Hkv, D]) plus its block
    # table; a dense one is [B, Hkv, Skv, D].
    for name, ten, table in (("k", k, k_block_table), ("v", v, v_block_table)):
        if table is None:
            _check_bf16_lastdim(ten, name)
            if ten.dim() != 4 or ten.shape[0] != B or ten.shape[3] != D:
                raise ValueError(f"shape mismatch: q {tuple(q.shape)} {name} {tuple(ten.shape)}")
            tables[name] = (ten, None, ten.shape[1], ten.shape[2])
        else:
            pool = _pool_view(ten, name + " pool")
            bt = _table_i32(table)
            if not bt.is_cuda or bt.shape[0] != B or pool.shape[3] != D:
                raise ValueError(f"{name}: pool {tuple(pool.shape)} / block table {tuple(bt.shape)} "
                                 f"do not fit q {tuple(q.shape)}")
            tables[name] = (pool, bt, pool.shape[2], bt.shape[1] * pool.shape[1])
            keep.append(bt)
    (kt, kbt, Hkv, Skv_k), (vt, vbt, Hkv_v, Skv_v) = tables["k"], tables["v"]
    if Hkv != Hkv_v:
        raise ValueError("k and v must have the same number of kv heads")
    if kbt is None and vbt is None and Skv_k != Skv_v:
        raise ValueError("k and v must have the same length")
    Skv = seq_len if seq_len is not None else min(Skv_k, Skv_v)
    if Skv > min(Skv_k, Skv_v) or Skv <= 0:
        raise ValueError("seq_len exceeds what k / v hold")
    if Hq % Hkv:
        raise ValueError("Hq must be a multiple of Hkv")
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=torch.bfloat16, device=dev)
    else:
        _require_cuda(out)
        _check_bf16_lastdim(out, "out")
    a = _native.LfPrefillArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), kt.data_ptr(), vt.data_ptr(), out.data_ptr()
    a.B, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = B, Hq, Hkv, Sq, Skv, D
    for i in range(3):
        a.q_stride[i] = q.stride(i)
        a.k_stride[i] = kt.stride(i)
        a.v_stride[i] = vt.stride(i)
        a.o_stride[i] = out.stride(i)
    if kbt is not None or vbt is not None:
        pools = [x for x, bt in ((kt, kbt), (vt, vbt)) if bt is not None]
        bts = [bt for bt in (kbt, vbt) if bt is not None]
        if len(pools) == 2 and pools[0].shape[:2] != pools[1].shape[:2]:
            raise ValueError("paged k and v must share the page geometry")
        if len(bts) == 2 and bts[0].stride(0) != bts[1].stride(0):
            bts = [x.contiguous() for x in bts]
            kbt, vbt = bts
            keep += bts
        a.k_block_table = kbt.data_ptr() if kbt is not None else None
        a.v_block_table = vbt.data_ptr() if vbt is not None else None
        a.bt_stride = bts[0].stride(0)
        a.page_size, a.n_pages = pools[0].shape[1], pools[0].shape[0]
    _fill_mods(a, scale, mods)
    a.mask_kind, a.window, a.causal_offset = int(mask_kind), int(window), int(causal_offset)
    a.status = status.data_ptr() if status is not None else None
    a.kv_tile = int(kv_tile)
    if dbg_ranges is not None:
        q_tile = _native.load().lf_prefill_q_tile(C.byref(a))
        if q_tile < 0:
            _native.check(q_tile, "lf_prefill_q_tile")
        need = B * Hq * (-(-Sq // q_tile)) * 2
        if dbg_ranges.dtype != torch.int32 or dbg_ranges.numel() < need or not dbg_ranges.is_cuda:
            raise ValueError(f"dbg_ranges must be a CUDA int32 tensor with >= {need} elements")
        a.dbg_ranges = dbg_ranges.data_ptr()
    a.kv_tile = int(kv_tile)
    a.sm_margin = int(sm_margin)
    a._keep = keep   # (tables converted on the fly must outlive the launch)
    return a, out, dev


class DecodeWorkspace:
    """Caller-owned scratch for split-KV partials, grown on demand and reused across calls."""

    def __init__(self) -> None:
        self._buf: Optional[torch.Tensor] = None

    def get(self, nbytes: int, device) -> Optional[torch.Tensor]:
        if nbytes == 0:
            return None
        if self._buf is None or self._buf.numel() < nbytes or self._buf.device != device:
            self._buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return self._buf


_default_ws = DecodeWorkspace()


def _decode_common(q, out, B, Hkv, G, Skv, D, scale, mods, splits, workspace, status, dev,
                   page_size=0):
    a = _native.LfDecodeArgs()
    a.q, a.out = q.data_ptr(), out.data_ptr()
    a.B, a.Hkv, a.G, a.Skv, a.D = B, Hkv, G, Skv, D
    for i in range(3):
        a.q_stride[i] = q.stride(i)
        a.o_stride[i] = out.stride(i)
    _fill_mods(a, scale, mods)
    lib = _native.load()
    with torch.cuda.device(dev):
        n_splits = splits if splits else lib.lf_decode_auto_splits(B, Hkv, G, Skv, D, page_size)
    a.splits = n_splits
    nbytes = lib.lf_decode_workspace_bytes(B, Hkv, G, D, n_splits)
    ws = (workspace or _default_ws).get(nbytes, dev)
    a.workspace = ws.data_ptr() if ws is not None else None
    a.workspace_bytes = nbytes
    a.status = status.data_ptr() if status is not None else None
    return a, ws


def decode_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0,
                     mods: Sequence[ScoreMod] = (), splits: int = 0,
                     out: Optional[torch.Tensor] = None,
                     workspace: Optional[DecodeWorkspace] = None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Unmasked attention of G query rows per kv head: q [B,Hkv,G,D], k/v [B,Hkv,Skv,D]."""
    dev = _require_cuda(q, k, v)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_bf16_lastdim(t, n)
        if t.dim() != 4:
            raise ValueError(f"{n} must be 4-D")
    B, Hkv, G, D = q.shape
    if k.shape[0] != B or k.shape[1] != Hkv or k.shape[3] != D or v.shape != k.shape:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)}")
    Skv = k.shape[2]
    if out is None:
        out = torch.empty((B, Hkv, G, D), dtype=torch.bfloat16, device=dev)
    a, ws = _decode_common(q, out, B, Hkv, G, Skv, D, scale, mods, splits, workspace, status, dev)
    a.k, a.v = k.data_ptr(), v.data_ptr()
    for i in range(3):
        a.k_stride[i] = k.stride(i)
        a.v_stride[i] = v.stride(i)
    with torch.cuda.device(dev):
        rc = _native.load().lf_decode_bf16(C.byref(a), _stream_ptr(dev))
    _native.check(rc, "lf_decode_bf16")
    return out


def _pool_view(pool: torch.Tensor, name: str) -> torch.Tensor:
    _check_bf16_lastdim(pool, name)
    if pool.dim() == 3:  # [pages, Hkv, D]: one token per page
        pool = pool.unsqueeze(1)
    if pool.dim() != 4:
        raise ValueError(f"{name} must be [pages, page_size, Hkv, D] or [pages, Hkv, D]")
    return pool


def _table_i32(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("block_table must be [batch, blocks]")
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    if t.stride(1) != 1:
        t = t.contiguous()
    return t


def paged_decode_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                           block_table: torch.Tensor, *, seq_len: Optional[int] = None,
                           block_table_v: Optional[torch.Tensor] = None, scale: float = 1.0,
                           mods: Sequence[ScoreMod] = (), splits: int = 0,
                           out: Optional[torch.Tensor] = None,
                           workspace: Optional[DecodeWorkspace] = None,
                           status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode attention over a paged KV cache: q [B,Hkv,G,D]; pools [pages, page_size, Hkv, D]
    (or [pages, Hkv, D] for one-token pages); block_table int32 [B, blocks]. Token t of sequence
    b lives at pool[block_table[b, t // page_size], t % page_size]."""
    dev = _require_cuda(q, k_pool, v_pool, block_table)
    _check_bf16_lastdim(q, "q")
    k_pool = _pool_view(k_pool, "k_pool")
    v_pool = _pool_view(v_pool, "v_pool")
    B, Hkv, G, D = q.shape
    n_pages, page_size = k_pool.shape[0], k_pool.shape[1]
    if k_pool.shape[2] != Hkv or k_pool.shape[3] != D or v_pool.shape != k_pool.shape:
        raise ValueError(f"pool shape mismatch: q {tuple(q.shape)} pool {tuple(k_pool.shape)}")
    bt = _table_i32(block_table)
    btv = _table_i32(block_table_v) if block_table_v is not None else None
    if bt.shape[0] != B:
        raise ValueError("block_table batch mismatch")
    Skv = seq_len if seq_len is not None else bt.shape[1] * page_size
    if Skv > bt.shape[1] * page_size:
        raise ValueError("seq_len exceeds the block table")
    if btv is not None and (btv.shape != bt.shape or btv.stride(0) != bt.stride(0)):
        btv = btv.contiguous()
        bt = bt.contiguous()
    if out is None:
        out = torch.empty((B, Hkv, G, D), dtype=torch.bfloat16, device=dev)
    a, ws = _decode_common(q, out, B, Hkv, G, Skv, D, scale, mods, splits, workspace, status, dev,
                           page_size=page_size)
    a.k, a.v = k_pool.data_ptr(), v_pool.data_ptr()
    for i in range(3):
        a.k_stride[i] = k_pool.stride(i)
        a.v_stride[i] = v_pool.stride(i)
    a.block_table = bt.data_ptr()
    a.block_table_v = btv.data_ptr() if btv is not None else None
    a.bt_stride = bt.stride(0)
    a.page_size, a.n_pages = page_size, n_pages
    with torch.cuda.device(dev):
        rc = _native.load().lf_decode_paged_bf16(C.byref(a), _stream_ptr(dev))
    _native.check(rc, "lf_decode_paged_bf16")
    return out


def paged_gather(pool: torch.Tensor, block_table: torch.Tensor, *, seq_len: Optional[int] = None,
                 status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Materialise [B, Hkv, S, D] from a paged pool (page-index check and paged prefill input)."""
    dev = _require_cuda(pool, block_table)
    pool = _pool_view(pool, "pool")
    bt = _table_i32(block_table)
    n_pages, page_size, Hkv, D = pool.shape
    B = bt.shape[0]
    S = seq_len if seq_len is not None else bt.shape[1] * page_size
    out = torch.empty((B, Hkv, S, D), dtype=torch.bfloat16, device=dev)
    strides = (C.c_int64 * 3)(pool.stride(0), pool.stride(1), pool.stride(2))
    with torch.cuda.device(dev):
        rc = _native.load().lf_paged_gather_bf16(
            pool.data_ptr(), bt.data_ptr(), out.data_ptr(), B, Hkv, S, D, page_size, n_pages,
            strides, bt.stride(0), status.data_ptr() if status is not None else None,
            _stream_ptr(dev))
    _native.check(rc, "lf_paged_gather_bf16")
    return out


def kv_append(k_new: torch.Tensor, v_new: torch.Tensor, k_pool: torch.Tensor,
              v_pool: torch.Tensor, block_table: torch.Tensor, *,
              seq_pos: Optional[torch.Tensor] = None, start_pos: int = 0,
              block_table_v: Optional[torch.Tensor] = None,
              status: Optional[torch.Tensor] = None) -> None:
    """Write new K/V rows ``[B, Hkv, T, D]`` into the pages of a paged cache, in place: token i
    of sequence b goes to ``pool[block_table[b, pos // page_size], pos % page_size]`` with
    ``pos = seq_pos[b] + i`` (or ``start_pos + i``). The device-side producer of the cache that
    ``paged_decode_attention`` reads."""
    dev = _require_cuda(k_new, v_new, k_pool, v_pool, block_table)
    for t_, n_ in ((k_new, "k_new"), (v_new, "v_new")):
        _check_bf16_lastdim(t_, n_)
        if t_.dim() != 4:
            raise ValueError(f"{n_} must be [B, Hkv, T, D]")
    kp = _pool_view(k_pool, "k_pool")
    vp = _pool_view(v_pool, "v_pool")
    B, Hkv, T, D = k_new.shape
    if v_new.shape != k_new.shape:
        raise ValueError("k_new and v_new must have the same shape")
    if kp.shape[2] != Hkv or kp.shape[3] != D or vp.shape != kp.shape:
        raise ValueError(f"pool shape mismatch: new {tuple(k_new.shape)} pool {tuple(kp.shape)}")
    bt = _table_i32(block_table)
    btv = _table_i32(block_table_v) if block_table_v is not None else None
    if bt.shape[0] != B:
        raise ValueError("block_table batch mismatch")
    if btv is not None and (btv.shape != bt.shape or btv.stride(0) != bt.stride(0)):
        btv, bt = btv.contiguous(), bt.contiguous()
    if seq_pos is not None:
        if seq_pos.dtype != torch.int32 or seq_pos.shape != (B,) or not seq_pos.is_cuda:
            raise ValueError("seq_pos must be a CUDA int32 tensor of shape [B]")
        seq_pos = seq_pos.contiguous()
    a = _native.LfKvAppendArgs()
    a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
    a.k_pool, a.v_pool = kp.data_ptr(), vp.data_ptr()
    a.block_table = bt.data_ptr()
    a.block_table_v = btv.data_ptr() if btv is not None else None
    a.seq_pos = seq_pos.data_ptr() if seq_pos is not None else None
    a.start_pos = int(start_pos)
    a.B, a.Hkv, a.T, a.D = B, Hkv, T, D
    for i in range(3):
        a.kn_stride[i] = k_new.stride(i)
        a.vn_stride[i] = v_new.stride(i)
        a.kp_stride[i] = kp.stride(i)
        a.vp_stride[i] = vp.stride(i)
    a.bt_stride, a.bt_blocks = bt.stride(0), bt.shape[1]
    a.page_size, a.n_pages = kp.shape[1], kp.shape[0]
    a.status = status.data_ptr() if status is not None else None
    with torch.cuda.device(dev):
        rc = _native.load().lf_kv_append_bf16(C.byref(a), _stream_ptr(dev))
    _native.check(rc, "lf_kv_append_bf16")
