"""CPU oracle for the fused-attention hot path. TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 PyTorch on the CPU, what the reference computes when one of
its attention functions runs eagerly - which is the parity target for the CUDA kernels. Only
tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import it; the product
package never does.

Parity pins: tests/golden/ holds outputs of the reference's own eager ops and of its compiler's
generated loop bounds (made by tests/golden/make_golden.py, which imports the reference);
tests/test_oracle.py checks this module against all of them.

What each function follows (paths inside tomatillos/loopfuse):
  causal_mask_ref     loopfuse/torch_backend/__init__.py:4-8 (eager op)
  sliding_mask_eager_ref   loopfuse/torch_backend/__init__.py:16-23 (eager op: keeps j > i - W)
  sliding_mask_ref    loopfuse/torch_backend/ops.py:733-741 (compiled mask: 0 <= i - j <= W-1)
  paged_load_ref      loopfuse/torch_backend/__init__.py:46-56
  attention_ref       the user-level functions of tests/benchmark.py:79-83, 142-147, 221-230,
                      328-334, 481-484 and tests/test_accuracy.py:131-135
  modified_attention_ref   the function of tests/test_accuracy.py:176-181 (query, score and output
                      bias), with the two bf16 roundings its eager graph has around the matmuls
  mla_attention_ref   the two-matmul scores of tests/test_attention.py:126-134
  kv_append_ref       the inverse of paged_load_ref: the cache / table convention of
                      tests/benchmark.py:308-319 read by loopfuse/torch_backend/__init__.py:46-56,
                      used as an indexed store (pool[block_table[b, t // P], t % P] = new row)
  reference_skip_range     closed forms of the range rewrite in
                      loopfuse/compiler/passes/skip_loop_iterations.py:343-376
  brute_force_skip_range   definition of a live tile ("holds >= 1 unmasked in-bounds element")

The arithmetic itself (matmul, tanh, softmax, gather) is PyTorch's (third-party, unpinned in the
reference's pyproject.toml:7-13; 2.11.0 here), exactly as in the reference's eager path.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

NEG_INF = float("-inf")


# ---------------------------------------------------------------------------------------------
# eager ops
# ---------------------------------------------------------------------------------------------
def causal_mask_ref(a: torch.Tensor) -> torch.Tensor:
    """Reference eager causal mask. Square scores only (it builds an [S_kv, S_kv] mask)."""
    s = a.shape[-1]
    keep = torch.tril(torch.ones(s, s, dtype=torch.bool))
    return a.masked_fill(~keep, NEG_INF)


def sliding_mask_eager_ref(a: torch.Tensor, window: int) -> torch.Tensor:
    """Reference *eager* sliding mask: keeps every column j > i - window, future ones included."""
    s = a.shape[-1]
    rows = torch.arange(s)[:, None]
    cols = torch.arange(s)[None, :]
    return a.masked_fill(~(cols > rows - window), NEG_INF)


def sliding_mask_ref(a: torch.Tensor, window: int, offset: int = 0) -> torch.Tensor:
    """Mask of the reference's *compiled* kernel: keeps 0 <= (i + offset) - j <= window - 1."""
    s_q, s_kv = a.shape[-2], a.shape[-1]
    rows = torch.arange(s_q)[:, None] + offset
    cols = torch.arange(s_kv)[None, :]
    d = rows - cols
    return a.masked_fill(~((d >= 0) & (d <= window - 1)), NEG_INF)


def causal_mask_general(a: torch.Tensor, offset: int = 0) -> torch.Tensor:
    """Causal mask for any score shape: keeps j <= i + offset (equals causal_mask_ref when
    the scores are square and offset is 0)."""
    s_q, s_kv = a.shape[-2], a.shape[-1]
    rows = torch.arange(s_q)[:, None] + offset
    cols = torch.arange(s_kv)[None, :]
    return a.masked_fill(cols > rows, NEG_INF)


def paged_load_ref(buffer: torch.Tensor, block_table: torch.Tensor) -> torch.Tensor:
    """out[*s, *t] = buffer[block_table[*s], *t]."""
    return buffer[block_table.long()]


def physical_rows(block_table: torch.Tensor, page_size: int, seq_len: int) -> torch.Tensor:
    """Row of the flattened pool [(page, slot), ...] that token t of sequence b lives in:
    block_table[b, t // P] * P + t % P, as an int64 [B, seq_len] tensor."""
    t = torch.arange(seq_len)
    return block_table.long()[:, t // page_size] * page_size + (t % page_size)[None, :]


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
def kv_append_ref(k_pool: torch.Tensor, new: torch.Tensor, block_table: torch.Tensor,
                  seq_pos) -> torch.Tensor:
    """Append ``new`` [B, Hkv, T, D] to a paged pool [n_pages, P, Hkv, D] (or [n_pages, Hkv, D],
    P = 1): returns a copy of the pool with pool[table[b, t // P], t % P, h] = new[b, h, t - pos_b]
    for t in [pos_b, pos_b + T). ``seq_pos`` is an int (all sequences) or a per-sequence list.
    A plain Python loop over (sequence, token): the definition, not a fast path."""
    pool = k_pool.clone()
    squeeze = pool.dim() == 3
    if squeeze:
        pool = pool.unsqueeze(1)
    P = pool.shape[1]
    B, Hkv, T, D = new.shape
    for b in range(B):
        pos0 = int(seq_pos if isinstance(seq_pos, int) else seq_pos[b])
        for i in range(T):
            t = pos0 + i
            page = int(block_table[b, t // P])
            pool[page, t % P] = new[b, :, i]
    return pool.squeeze(1) if squeeze else pool


def apply_mods(s: torch.Tensor, mods: Sequence[tuple]) -> torch.Tensor:
    """Score-mod chain as (name, arg) pairs, e.g. [("div", 50.0), ("tanh", None), ("mul", 50.0)]."""
    for name, arg in mods:
        if name == "mul":
            s = s * arg
        elif name == "div":
            s = s / arg
        elif name == "add":
            s = s + arg
        elif name == "tanh":
            s = torch.tanh(s)
        elif name == "exp":
            s = torch.exp(s)
        elif name == "exp2":
            s = torch.exp2(s)
        elif name == "sin":
            s = torch.sin(s)
        elif name == "cos":
            s = torch.cos(s)
        elif name == "relu":
            s = torch.relu(s)
        elif name == "square":
            s = s * s
        else:
            raise ValueError(name)
    return s


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
                  mods: Sequence[tuple] = (), mask: str = "none", window: int = 0,
                  offset: int = 0, batch_chunk: int = 1) -> torch.Tensor:
    """softmax(mask(mods(q k^T * scale))) v in fp32 on the CPU, exactly as the eager functions
    do it (scores materialised), one batch chunk at a time to bound memory.

    q [B, Hq, Sq, D]; k, v [B, Hkv, Skv, D] with Hq % Hkv == 0 (kv heads are repeat_interleave'd
    as in tests/benchmark.py:226-227). mask: "none" | "causal" | "window" (= causal and window).
    Inputs of any float dtype are upcast to fp32 first.
    """
    q, k, v = q.float().cpu(), k.float().cpu(), v.float().cpu()
    B, Hq, Sq, D = q.shape
    Hkv = k.shape[1]
    if scale is None:
        scale = D ** -0.5
    g = Hq // Hkv
    outs = []
    for b0 in range(0, B, batch_chunk):
        qb, kb, vb = q[b0:b0 + batch_chunk], k[b0:b0 + batch_chunk], v[b0:b0 + batch_chunk]
        if g > 1:
            kb = kb.repeat_interleave(g, dim=1)
            vb = vb.repeat_interleave(g, dim=1)
        s = qb @ kb.transpose(-2, -1) * scale
        s = apply_mods(s, mods)
        if mask == "causal":
            s = causal_mask_general(s, offset)
        elif mask == "window":
            s = causal_mask_general(sliding_mask_ref(s, window, offset), offset)
        elif mask != "none":
            raise ValueError(mask)
        outs.append(torch.softmax(s, dim=-1) @ vb)
    return torch.cat(outs)


def modified_attention_ref(q, k, v, q_bias, scores_bias, out_bias, *, mult: float = 3.5,
                           batch_chunk: int = 1) -> torch.Tensor:
    """softmax(causal((Q + q_bias) K^T * D^-0.5 * mult + scores_bias)) V + out_bias.

    The eager bf16 graph rounds `Q + q_bias` to bf16 before the matmul and adds `out_bias` to the
    bf16 attention output; both roundings are kept here (they are part of what the function
    computes on bf16 tensors), everything between them is fp32."""
    qb = (q.float().cpu() + q_bias.float().cpu()).to(torch.bfloat16).float()
    k, v = k.float().cpu(), v.float().cpu()
    sb = scores_bias.float().cpu()
    scale = q.shape[-1] ** -0.5
    outs = []
    for b0 in range(0, q.shape[0], batch_chunk):
        s = qb[b0:b0 + batch_chunk] @ k[b0:b0 + batch_chunk].transpose(-2, -1) * scale
        s = causal_mask_general(s * mult + sb[b0:b0 + batch_chunk])
        outs.append(torch.softmax(s, dim=-1) @ v[b0:b0 + batch_chunk])
    att = torch.cat(outs).to(torch.bfloat16).float()
    return att + out_bias.float().cpu()


def mla_attention_ref(q, q_pe, k, k_pe, v, *, mask: str = "causal",
                      batch_chunk: int = 1) -> torch.Tensor:
    """softmax(mask((Q K^T + Q_pe K_pe^T) * (D + D_pe)^-0.5)) V in fp32 on the CPU."""
    q, q_pe, k, k_pe, v = (t.float().cpu() for t in (q, q_pe, k, k_pe, v))
    scale = (q.shape[-1] + q_pe.shape[-1]) ** -0.5
    outs = []
    for b0 in range(0, q.shape[0], batch_chunk):
        sl = slice(b0, b0 + batch_chunk)
        s = (q[sl] @ k[sl].transpose(-2, -1) + q_pe[sl] @ k_pe[sl].transpose(-2, -1)) * scale
        if mask == "causal":
            s = causal_mask_general(s)
        outs.append(torch.softmax(s, dim=-1) @ v[sl])
    return torch.cat(outs)


def softcap_mods(c: float) -> list:
    return [("div", c), ("tanh", None), ("mul", c)]


def paged_kv_ref(pool: torch.Tensor, block_table: torch.Tensor) -> torch.Tensor:
    """Logical [B, Hkv, S, D] K or V of a paged cache [pages, P, Hkv, D] (or [pages, Hkv, D])."""
    g = paged_load_ref(pool.float().cpu(), block_table.cpu())
    if pool.dim() == 4:  # [B, blocks, P, Hkv, D] -> [B, S, Hkv, D]
        g = g.reshape(g.shape[0], -1, g.shape[-2], g.shape[-1])
    return g.transpose(1, 2)


def workload_ref(w, inputs: tuple, batch_chunk: int = 1) -> torch.Tensor:
    """Oracle output for a loopfuse_b200.variants.Workload and the inputs make_inputs() gave.

    Output layout equals the compiled function's: [B, Hq, S, D] for prefill, [B, Hq, 1, D] for
    decode, [B, Hkv, g, D] for paged GQA decode (the reference's query convention).
    """
    if w.kind == "prefill":
        q, k, v = inputs
        mods = softcap_mods(w.softcap) if w.softcap else []
        mask = "window" if w.window else "causal"
        return attention_ref(q, k, v, mods=mods, mask=mask, window=w.window,
                             batch_chunk=batch_chunk)
    if w.kind == "decode":
        q, k, v = inputs
        return attention_ref(q, k, v, batch_chunk=max(batch_chunk, 8))
    q, k_pool, v_pool, table = inputs
    k = paged_kv_ref(k_pool, table)
    v = paged_kv_ref(v_pool, table)
    # q [B, Hkv, g, D]: the g grouped heads are the rows of one kv head's attention
    return attention_ref(q, k, v, batch_chunk=max(batch_chunk, 8))


# ---------------------------------------------------------------------------------------------
# block-skip ranges
# ---------------------------------------------------------------------------------------------
def keep_matrix(mask: str, window: int, s_q: int, s_kv: int, offset: int = 0) -> torch.Tensor:
    rows = torch.arange(s_q)[:, None] + offset
    cols = torch.arange(s_kv)[None, :]
    keep = torch.ones(s_q, s_kv, dtype=torch.bool)
    if mask in ("causal", "window"):
        keep &= cols <= rows
    if mask == "window":
        keep &= cols >= rows - (window - 1)
    return keep


def brute_force_skip_range(mask: str, window: int, s_q: int, s_kv: int, tile_q: int, tile_k: int,
                           iq: int, offset: int = 0, keep: Optional[torch.Tensor] = None):
    """[lo, hi): smallest range of KV tiles covering every tile with a live element."""
    if keep is None:
        keep = keep_matrix(mask, window, s_q, s_kv, offset)
    rows = keep[iq * tile_q:(iq + 1) * tile_q]
    live_cols = rows.any(dim=0).nonzero().flatten()
    if live_cols.numel() == 0:
        return 0, 0
    return int(live_cols[0]) // tile_k, int(live_cols[-1]) // tile_k + 1


def reference_skip_range(mask: str, window: int, s_kv: int, tile_q: int, tile_k: int, iq: int):
    """Closed forms the reference's sparsity pass emits, evaluated like the generated kernel
    does: in floating point, then truncated toward zero (skip_loop_iterations.py:357-373).

        range_end   = min(cdiv(S_kv, tK), trunc(-(1/tK) * ((1 - tQ) - iq*tQ) + 1))      causal/window
        range_start = max(0, trunc(-(1/tK) * ((W - 2 + tK) - iq*tQ) + 1))               window
    """
    n_kt = -(-s_kv // tile_k)
    lo, hi = 0, n_kt
    inv = 1.0 / tile_k
    if mask in ("causal", "window"):
        hi = min(hi, math.trunc((-1 * inv) * ((1 - tile_q) + (-1 * iq) * tile_q) + 1))
    if mask == "window":
        lo = max(0, math.trunc((-1 * inv) * ((window - 2 + tile_k) + (-1 * iq) * tile_q) + 1))
    return lo, hi
