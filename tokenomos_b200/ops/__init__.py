"""The kernels as functions over torch tensors on a CUDA device.

torch is the allocator and the stream owner here, nothing more: every function checks its
tensors, picks the entry point for the storage type (float32 or bfloat16) and launches on the
current stream. Tensors on the CPU are refused: there is no CPU implementation on the product
path (the plain implementation under ``tests/`` is the oracle, not a fallback).
"""

from __future__ import annotations

import torch

from tokenomos_b200.ops import _lib
from tokenomos_b200.ops._lib import BF16, F32, KernelError

__all__ = [
    "KernelError", "available", "checks_enabled", "set_check_bounds", "checks_status", "gather_rows", "add_rmsnorm", "swiglu", "head_gate",
    "qk_norm_rope_write", "attention", "attention_rows", "attention_mma_supported",
    "attention_prefill_mma", "attention_prefill_mma_tokens", "attention_decode_mma",
    "attention_prefill_tc", "attention_prefill_tc_supported", "attention_prefill_tc_tokens",
    "attention_prefill_tc_status",
    "conv_gated", "conv_min_tile",
    "gemm", "gemm_skinny", "gemm_skinny_conv", "gemm_skinny_ok", "gemm_tc", "gemm_tc_ok", "gemm_tc_status", "sample", "sample_status", "gather_rows_select",
]


# What the kernels take, so that a model that asks for more is refused when it is built and not
# at its first step (the entry points check the same limits: conv.cu and gemm_skinny.cu, the row
# that add_rmsnorm keeps in shared memory, attention_generic.cu's MAX_D, qk_rope.cu)
CONV_WIDTHS = (2, 8)
NORM_MAX_WIDTH = 51200
ATTENTION_MAX_HEAD_DIM = 256


def available() -> None:
    """Raise unless the library loads and the current device can run it."""
    _lib.call("tk_check_device")


def checks_enabled() -> bool:
    """Whether the loaded library is the debug build whose kernels check the indices they follow
    (``TOKENOMOS_B200_CHECKS=1`` at first use; csrc/checks.cuh)."""
    return bool(_lib.call("tk_checks_enabled"))


def set_check_bounds(pages: int, slots: int) -> None:
    """What the index checks compare against: pages per paged pool, rows per state tensor."""
    _lib.call("tk_checks_set_bounds", int(pages), int(slots))


CHECKED_KERNELS = {1: "row gather", 2: "q/k norm + rope + cache write", 3: "attention (generic)",
                   4: "attention (tensor cores)", 5: "gated short conv", 6: "projection with the conv inside"}
CHECKED_INDICES = {1: "page", 2: "state row", 3: "table row"}


def checks_status() -> str | None:
    """None, or what the first index was that a kernel found outside its pool since the last call
    (the kernel went on with the null page or row instead of following it)."""
    import ctypes

    word = (ctypes.c_int * 2)()
    _lib.call("tk_checks_status", ctypes.cast(word, ctypes.c_void_p))
    if word[0] == 0:
        return None
    kernel, what = divmod(word[0], 8)
    return (f"{CHECKED_KERNELS.get(kernel, f'kernel {kernel}')}: {CHECKED_INDICES.get(what, 'index')} "
            f"{word[1]} is outside its pool")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"storage type {t.dtype} is not built (float32 and bfloat16 are)")


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("tokenomos_b200 kernels run on CUDA tensors only; got a "
                              f"{t.device} tensor (there is no CPU path)")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream():
    # the raw handle of torch's current stream (a capture's side stream included); the private
    # getters skip torch.cuda's Python wrappers, which cost more than a kernel launch
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


def _f32vec(t: torch.Tensor | None, name: str, n: int) -> torch.Tensor | None:
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
        raise KernelError(f"{name} must be a contiguous float32 vector of {n} elements, got "
                          f"{t.dtype} {tuple(t.shape)}")
    return t


def gather_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None):
    """``out[r] = table[ids[r]]``: the embedding lookup and the row selection before the head."""
    _cuda(table, ids, out)
    rows, width = ids.numel(), table.shape[1]
    if not table.is_contiguous():
        raise KernelError("gather_rows: the table must be contiguous")
    if out is None:
        out = torch.empty(rows, width, dtype=table.dtype, device=table.device)
    _lib.call("tk_gather_rows", _ptr(table), _ptr(_i32(ids, "ids")), _ptr(out), rows, width,
              table.shape[0], _dtype_code(table), _stream())
    return out


def gather_rows_select(table: torch.Tensor, ids_host: torch.Tensor, use_prev: torch.Tensor,
                       last_token: torch.Tensor, slot: torch.Tensor) -> torch.Tensor:
    """``out[r] = table[last_token[slot[r]] if use_prev[r] else ids_host[r]]`` (ids int32): the
    decode step's embedding lookup, fed on the device by the step before."""
    _cuda(table, ids_host, use_prev, last_token, slot)
    rows, width = ids_host.numel(), table.shape[1]
    if not table.is_contiguous():
        raise KernelError("gather_rows_select: the table must be contiguous")
    for name, t in (("use_prev", use_prev), ("slot", slot)):
        if _i32(t, name).numel() < rows:
            raise KernelError(f"gather_rows_select: {name} is shorter than ids_host")
    out = torch.empty(rows, width, dtype=table.dtype, device=table.device)
    _lib.call("tk_gather_rows_select", _ptr(table), _ptr(_i32(ids_host, "ids_host")), _ptr(use_prev),
              _ptr(_i32(last_token, "last_token")), _ptr(slot), _ptr(out), rows, width, table.shape[0],
              _dtype_code(table), _stream())
    return out


def scale_rows(x: torch.Tensor, scale: float) -> torch.Tensor:
    """In place ``x = round(x * round(scale))`` (both to ``x``'s type): an embedding scale."""
    _cuda(x)
    if not x.is_contiguous():
        raise KernelError("scale_rows: x must be contiguous")
    _lib.call("tk_scale_rows", _ptr(x), x.numel(), float(scale), _dtype_code(x), _stream())
    return x


def logit_options(logits: torch.Tensor, softcap: float | None, suppress: torch.Tensor | None) -> torch.Tensor:
    """In place on float32 ``logits`` [rows, vocab]: ``softcap * tanh(logits / softcap)`` if a cap
    is given, then ``-inf`` at the token ids of ``suppress`` (int32, each inside the vocabulary)."""
    _cuda(logits, suppress)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logit_options: logits must be float32 [rows, vocab] with contiguous rows")
    n = 0 if suppress is None else _i32(suppress, "suppress").numel()
    _lib.call("tk_logit_options", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1],
              float(softcap or 0.0), _ptr(suppress), n, _stream())
    return logits


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor | None,
                eps: float, pre: tuple[torch.Tensor, float] | None = None):
    """``stream = residual + [pre-norm](x)``; ``y = rmsnorm(stream) * weight``.

    Returns ``(y, stream)``; ``stream`` is ``x`` itself when nothing was added, ``y`` is None
    without ``weight``. ``x`` may be a row-strided view; the other tensors are contiguous."""
    _cuda(x, residual, weight)
    rows, width = x.shape
    if x.stride(1) != 1:
        raise KernelError("add_rmsnorm: rows of x must be contiguous")
    w = _f32vec(weight, "norm weight", width)
    pre_w = _f32vec(pre[0], "pre-norm weight", width) if pre is not None else None
    y = torch.empty(rows, width, dtype=x.dtype, device=x.device) if w is not None else None
    writes = residual is not None or pre is not None
    stream = torch.empty(rows, width, dtype=x.dtype, device=x.device) if writes else None
    if residual is not None and (not residual.is_contiguous() or residual.shape != x.shape
                                 or residual.dtype != x.dtype):
        raise KernelError("add_rmsnorm: residual must match x and be contiguous")
    _lib.call("tk_add_rmsnorm", _ptr(x), x.stride(0), _ptr(residual), _ptr(pre_w),
              float(pre[1]) if pre is not None else 0.0, _ptr(w), float(eps), _ptr(y),
              _ptr(stream), rows, width, _dtype_code(x), _stream())
    if stream is None:
        stream = x if x.is_contiguous() else x.contiguous()
    return y, stream


def swiglu(gu: torch.Tensor, block: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` for ``gu`` of width ``2 I``: ``gu = [gate | up]`` (``block`` 0), or gate
    and up alternating in runs of ``block`` channels."""
    _cuda(gu)
    if not gu.is_contiguous() or gu.shape[1] % 2:
        raise KernelError("swiglu: input must be contiguous with an even width")
    rows, inter = gu.shape[0], gu.shape[1] // 2
    out = torch.empty(rows, inter, dtype=gu.dtype, device=gu.device)
    _lib.call("tk_swiglu", _ptr(gu), _ptr(out), rows, inter, int(block), _dtype_code(gu), _stream())
    return out


def head_gate(x: torch.Tensor, g: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    """In place: ``x[t, h, :] *= sigmoid(g[t, h])``; ``g`` [T, heads] may be a column block of a
    wider tensor (rows any distance apart)."""
    _cuda(x, g)
    if not (x.is_contiguous() and g.dim() == 2 and g.stride(1) == 1 and g.dtype == x.dtype):
        raise KernelError("head_gate: contiguous x, g with contiguous rows, one storage type")
    rows = x.numel() // (heads * head_dim)
    if tuple(g.shape) != (rows, heads):
        raise KernelError("head_gate: one gate per (token, head)")
    _lib.call("tk_head_gate", _ptr(x), _ptr(g), g.stride(0), rows, heads, head_dim, _dtype_code(x),
              _stream())
    return x


def qk_norm_rope_write(qkv: torch.Tensor, kv_pool: torch.Tensor | None,
                       wq: torch.Tensor | None, wk: torch.Tensor | None, eps: float,
                       inv_freq: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor,
                       block_table: torch.Tensor | None, heads: int, kv_heads: int,
                       head_dim: int, page: int) -> torch.Tensor:
    """Norm + rotate the q and k heads of ``qkv`` [T, (H + 2 Hkv) D]; returns q [T, H, D] and
    writes k, v into ``kv_pool`` [pages, 2, Hkv, P, D] at each token's position. ``kv_heads`` 0:
    queries only (the layer reads another layer's cache)."""
    _cuda(qkv, kv_pool, wq, wk, inv_freq, positions, tok_seq, block_table)
    T = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope_write: qkv of width {qkv.shape[1]} for {heads}+2*{kv_heads} "
                          f"heads of {head_dim}")
    rot = 2 * inv_freq.numel()
    _f32vec(inv_freq, "inv_freq", rot // 2)
    q = torch.empty(T, heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    if kv_heads:
        if kv_pool is None or block_table is None:
            raise KernelError("qk_norm_rope_write: keys need a cache and a block table")
        if kv_pool.dtype != qkv.dtype or not kv_pool.is_contiguous() or tuple(kv_pool.shape[1:]) != (
                2, kv_heads, page, head_dim):
            raise KernelError(f"qk_norm_rope_write: cache {tuple(kv_pool.shape)} {kv_pool.dtype} does "
                              f"not match [pages, 2, {kv_heads}, {page}, {head_dim}] {qkv.dtype}")
        _i32(block_table, "block_table")
    _lib.call("tk_qk_norm_rope_write", _ptr(qkv), qkv.stride(0), _ptr(q), _ptr(kv_pool),
              _ptr(_f32vec(wq, "q_norm weight", head_dim)), _ptr(_f32vec(wk, "k_norm weight", head_dim)),
              float(eps), _ptr(inv_freq), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(block_table),
              block_table.stride(0) if block_table is not None else 0, T, heads, kv_heads,
              head_dim, rot, page, _dtype_code(qkv), _stream())
    return q


def attention_rows() -> int:
    """Rows (token x query head of one group) a tile of the generic attention kernel holds."""
    return _lib.call("tk_attn_generic_rows")


def attention(q: torch.Tensor, kv_pool: torch.Tensor, positions: torch.Tensor,
              tok_seq: torch.Tensor, block_table: torch.Tensor, tile_tok0: torch.Tensor,
              tile_ntok: torch.Tensor, tokens_per_tile: int, window: int | None,
              scale: float) -> torch.Tensor:
    """Causal (optionally windowed) attention of ``q`` [T, H, D] over the paged cache
    ``kv_pool`` [pages, 2, Hkv, P, D], which already holds this step's keys. Tiles name runs of
    at most ``tokens_per_tile`` tokens of one sequence."""
    _cuda(q, kv_pool, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    T, H, D = q.shape
    _, two, Hkv, P, D2 = kv_pool.shape
    if two != 2 or D2 != D or kv_pool.dtype != q.dtype or not (q.is_contiguous() and kv_pool.is_contiguous()):
        raise KernelError("attention: q / cache layouts do not match")
    out = torch.empty_like(q)
    _lib.call("tk_attn_generic", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tile_tok0, "tile_tok0")),
              _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(), tokens_per_tile, H, Hkv, D, P,
              int(window or 0), float(scale), _dtype_code(q), _stream())
    return out


def attention_mma_supported(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernels take this shape (else: ``attention``)."""
    return dtype == torch.bfloat16 and bool(_lib.call("tk_attn_mma_supported", heads, kv_heads, head_dim))


def attention_prefill_mma_tokens(heads: int, kv_heads: int) -> int:
    """Tokens per tile the tensor-core prefill kernel expects."""
    return _lib.call("tk_attn_prefill_mma_tokens", heads, kv_heads)


def _check_attention(q, kv_pool, name):
    T, H, D = q.shape
    _, two, Hkv, P, D2 = kv_pool.shape
    if (two != 2 or D2 != D or kv_pool.dtype != q.dtype or q.dtype != torch.bfloat16
            or not (q.is_contiguous() and kv_pool.is_contiguous())):
        raise KernelError(f"{name}: bfloat16 q [T, H, D] and cache [pages, 2, Hkv, P, D] expected")
    return T, H, D, Hkv, P


def _gate_view(gate: torch.Tensor | None, T: int, H: int, name: str):
    """(pointer, row stride) of a per-head output gate [T, H] (a bfloat16 view with unit column
    stride), or (None, 0)."""
    if gate is None:
        return None, 0
    if not gate.is_cuda or gate.dtype != torch.bfloat16 or tuple(gate.shape) != (T, H) or gate.stride(1) != 1:
        raise KernelError(f"{name}: gate must be a bfloat16 [T, H] CUDA view with unit column stride")
    return gate.data_ptr(), gate.stride(0)


def attention_prefill_mma(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor,
                          positions: torch.Tensor, tok_seq: torch.Tensor,
                          block_table: torch.Tensor, tile_tok0: torch.Tensor,
                          tile_ntok: torch.Tensor, window: int | None, scale: float,
                          gate: torch.Tensor | None = None) -> None:
    """Tensor-core attention for tiles of ``attention_prefill_mma_tokens`` tokens of one
    sequence; writes the tiles' rows of ``out`` [T, H, D], times the per-head output gate
    ``round(sigmoid(gate))`` [T, H] if one is given."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_prefill_mma")
    g_ptr, ldg = _gate_view(gate, T, H, "attention_prefill_mma")
    _lib.call("tk_attn_prefill_mma", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tile_tok0, "tile_tok0")),
              _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(), H, Hkv, D, P, int(window or 0),
              float(scale), g_ptr, ldg, _stream())


def attention_prefill_tc_supported(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (bfloat16, head size 64, a group that
    divides 128)."""
    return dtype == torch.bfloat16 and bool(_lib.call("tk_attn_prefill_tc_supported", heads, kv_heads, head_dim))


def attention_prefill_tc_tokens(heads: int, kv_heads: int) -> int:
    """Tokens of one sequence per tile of ``attention_prefill_tc``."""
    return _lib.call("tk_attn_prefill_tc_tokens", heads, kv_heads)


def attention_prefill_tc(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor,
                         positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                         tile_tok0: torch.Tensor, tile_ntok: torch.Tensor, window: int | None,
                         scale: float, gate: torch.Tensor | None = None, nsplit: int = 1) -> None:
    """``attention_prefill_mma`` on tcgen05.mma with the accumulators in tensor memory, for tiles
    of ``attention_prefill_tc_tokens`` tokens of one sequence; writes the tiles' rows of ``out``
    (gated like ``attention_prefill_mma``'s). ``nsplit`` > 1: that many CTAs share each tile's
    keys and the last one to finish merges their shares (through scratch memory that this
    function allocates): for steps with few tiles behind long contexts."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_prefill_tc")
    g_ptr, ldg = _gate_view(gate, T, H, "attention_prefill_tc")
    n_tiles = tile_tok0.numel()
    nsplit = max(1, int(nsplit))
    scratch = tickets = None
    if nsplit > 1 and n_tiles:
        scratch = torch.empty(n_tiles * Hkv * nsplit * (128 * D + 256), dtype=torch.float32, device=q.device)
        tickets = _decode_tickets(n_tiles * Hkv, q.device)
    _lib.call("tk_attn_prefill_tc", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tile_tok0, "tile_tok0")),
              _ptr(_i32(tile_ntok, "tile_ntok")), n_tiles, H, Hkv, D, P, int(window or 0),
              float(scale), g_ptr, ldg, nsplit, _ptr(scratch), _ptr(tickets), _stream())


def attention_prefill_tc_status() -> int:
    """0, or where a CTA of the tcgen05 prefill kernel gave up waiting since the last call."""
    return _lib.call("tk_attn_prefill_tc_status")


def attention_decode_mma(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor,
                         positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                         tok_index: torch.Tensor | None, window: int | None, scale: float,
                         nsplit: int, gate: torch.Tensor | None = None) -> None:
    """Tensor-core attention for sequences that bring one token (``tok_index``: their rows in
    the packed batch; None: every row of ``q`` is one, in order, which spares the kernel a
    lookup), each split ``nsplit`` ways over its keys; partial results go through scratch memory
    that this function allocates and a merge kernel. Writes those rows of ``out`` [T, H, D]
    (gated like ``attention_prefill_mma``'s)."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tok_index)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_decode_mma")
    g_ptr, ldg = _gate_view(gate, T, H, "attention_decode_mma")
    n = tok_index.numel() if tok_index is not None else T
    scratch = None
    if nsplit > 1:
        scratch = torch.empty(n * H * nsplit * (D + 2), dtype=torch.float32, device=q.device)
    _lib.call("tk_attn_decode_mma", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tok_index, "tok_index") if tok_index is not None else None),
              n, H, Hkv, D, P, int(window or 0), float(scale), int(nsplit), _ptr(scratch), g_ptr, ldg,
              _stream())


def attention_decode_fused_supported(heads: int, kv_heads: int, head_dim: int, rotary: int,
                                     dtype: torch.dtype) -> bool:
    """Whether ``attention_decode_fused`` takes this shape and rotary width."""
    return dtype == torch.bfloat16 and bool(
        _lib.call("tk_attn_decode_fused_supported", heads, kv_heads, head_dim, rotary))


# per device: [n * kv_heads] zeros the fused decode kernel counts finished splits in and zeroes
# again; a buffer that a captured step may point at is never freed, only outgrown
_tickets: dict = {}
_tickets_outgrown: list = []


def _decode_tickets(n: int, device: torch.device) -> torch.Tensor:
    have = _tickets.get(device)
    if have is None or have.numel() < n:
        if have is not None:
            _tickets_outgrown.append(have)
        have = _tickets[device] = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
    return have


def clear_tickets() -> None:
    """Put the ticket counters back to zero. The kernels that use them leave them at zero; one
    that gave up on a barrier half way may not have, and the next launch must not inherit that."""
    for t in list(_tickets.values()) + _tickets_outgrown:
        t.zero_()


def attention_decode_fused(qkv: torch.Tensor, kv_pool: torch.Tensor, q_norm: torch.Tensor | None,
                           k_norm: torch.Tensor | None, eps: float, inv_freq: torch.Tensor,
                           gate: torch.Tensor | None, positions: torch.Tensor, tok_seq: torch.Tensor,
                           block_table: torch.Tensor, heads: int, kv_heads: int, window: int | None,
                           scale: float, nsplit: int, write_kv: bool = True,
                           carveout: int = -1) -> torch.Tensor:
    """A decode step's attention in one kernel, for sequences that bring one token each (row i of
    ``qkv`` is sequence i's): from the raw projection rows ``qkv`` [T, >= (H + 2 Hkv) D] (q heads,
    k heads, v heads; rows may be strided) through q/k norm, the rotate-half rotation by
    ``position * inv_freq`` [R / 2], the write of the new keys and values into ``kv_pool``
    [pages, 2, Hkv, P, D], attention over the cache split ``nsplit`` ways, the merge of the splits
    and the per-head gate ``gate`` [T, H] (a strided view; None: no gate) to the heads' outputs
    [T, H, D]. ``write_kv`` False: the layer reads a cache that another layer wrote this step and
    ``qkv`` holds queries only. ``carveout``: the share of an SM's memory, in percent of the most,
    that the launch prefers as shared memory (-1: the driver's choice). ``nsplit`` is cut to what
    the kernel's merge can hold."""
    _cuda(qkv, kv_pool, q_norm, k_norm, inv_freq, gate, positions, tok_seq, block_table)
    T = qkv.shape[0]
    _, two, Hkv, P, D = kv_pool.shape
    need = (heads + (2 * Hkv if write_kv else 0)) * D
    if (two != 2 or Hkv != kv_heads or qkv.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16
            or qkv.stride(1) != 1 or qkv.shape[1] < need or not kv_pool.is_contiguous()):
        raise KernelError("attention_decode_fused: qkv [T, >= (H + 2 Hkv) D] with contiguous rows and "
                          "kv_pool [pages, 2, Hkv, P, D], both bfloat16")
    if gate is not None and (gate.dtype != torch.bfloat16 or gate.shape != (T, heads) or gate.stride(1) != 1):
        raise KernelError("attention_decode_fused: gate must be a bfloat16 [T, H] view with unit column stride")
    R = 2 * inv_freq.numel()
    out = torch.empty(T, heads, D, dtype=torch.bfloat16, device=qkv.device)
    nsplit = max(1, min(int(nsplit), _lib.call("tk_attn_decode_fused_max_splits", heads, Hkv, D)))
    scratch = tickets = None
    if nsplit > 1:
        scratch = torch.empty(T * heads * nsplit * (D + 2), dtype=torch.float32, device=qkv.device)
        tickets = _decode_tickets(T * Hkv, qkv.device)
    _lib.call("tk_attn_decode_fused", _ptr(qkv), qkv.stride(0), _ptr(kv_pool), _ptr(out),
              _ptr(_f32vec(q_norm, "q_norm", D)), _ptr(_f32vec(k_norm, "k_norm", D)), float(eps),
              _ptr(_f32vec(inv_freq, "inv_freq", R // 2)), R, _ptr(gate),
              gate.stride(0) if gate is not None else 0, _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
              T, heads, Hkv, D, P, int(window or 0), float(scale), int(nsplit), _ptr(scratch), _ptr(tickets),
              1 if write_kv else 0, int(carveout), _stream())
    return out


def conv_min_tile(width: int) -> int:
    return _lib.call("tk_conv_min_tile", width)


def conv_gated(bcx: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
               state: torch.Tensor, cu: torch.Tensor, seq_ctx: torch.Tensor,
               seq_slot: torch.Tensor, tile_seq: torch.Tensor, tile_off: torch.Tensor,
               tile_n: torch.Tensor, block: int = 0, tile_cap: int = 0,
               tile_tok0: torch.Tensor | None = None) -> torch.Tensor:
    """Gated short conv of ``bcx`` [T, 3d] = (B | C | X): returns ``C * conv(B * X)`` [T, d] and
    replaces each sequence's row of ``state`` [slots, W-1, d]. ``weight`` [d, W] float32.
    ``block`` b > 0: a row of ``bcx`` holds runs of b channels of B, of C and of X in turn.
    ``tile_cap``: the most tokens a tile has, if the caller knows (up to 16 a faster kernel takes
    the call); every tile but a portion's last has at least W - 1 tokens. ``tile_tok0``: each
    tile's first token in the batch, if the caller has it (it spares that kernel a lookup)."""
    _cuda(bcx, weight, bias, state, cu, seq_ctx, seq_slot, tile_seq, tile_off, tile_n)
    T, three_d = bcx.shape
    d = three_d // 3
    W = weight.shape[1]
    if bcx.stride(1) != 1 or three_d != 3 * d:
        raise KernelError("conv_gated: bcx must be [T, 3d] with contiguous rows")
    if weight.dtype != torch.float32 or not weight.is_contiguous() or weight.shape[0] != d:
        raise KernelError("conv_gated: weight must be contiguous float32 [d, W]")
    if state.dtype != bcx.dtype or not state.is_contiguous() or tuple(state.shape[1:]) != (W - 1, d):
        raise KernelError(f"conv_gated: state {tuple(state.shape)} does not match [slots, {W - 1}, {d}]")
    out = torch.empty(T, d, dtype=bcx.dtype, device=bcx.device)
    _lib.call("tk_conv_gated", _ptr(bcx), bcx.stride(0), d, _ptr(weight), _ptr(_f32vec(bias, "conv bias", d)),
              _ptr(state), _ptr(out), _ptr(_i32(cu, "cu")), _ptr(_i32(seq_ctx, "seq_ctx")),
              _ptr(_i32(seq_slot, "seq_slot")), _ptr(_i32(tile_seq, "tile_seq")),
              _ptr(_i32(tile_off, "tile_off")), _ptr(_i32(tile_n, "tile_n")),
              _ptr(_i32(tile_tok0, "tile_tok0")) if tile_tok0 is not None else None, tile_seq.numel(), W,
              int(block), int(tile_cap), _dtype_code(bcx), _stream())
    return out


def gemm_skinny_conv(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, taps: torch.Tensor,
                     conv_bias: torch.Tensor | None, state: torch.Tensor, seq_ctx: torch.Tensor,
                     seq_slot: torch.Tensor, norm_eps: float = 0.0) -> torch.Tensor:
    """A gated short conv's in-projection with the conv in its epilogue, for a step whose tokens
    are one new token of a sequence each (decoding): ``x`` [M <= 16, K] bfloat16, ``w`` [3d, K]
    with rows in blocks of 24 (8 rows of B, of C and of X of the same 8 channels), ``bias`` in the
    same order; returns ``C * conv(B * X)`` [M, d] and moves each request's row of ``state``
    [slots, W-1, d] on by its token. ``seq_ctx``, ``seq_slot``: [M]. ``norm_eps`` > 0 (at most 8
    rows): ``x`` is an un-normed stream; see ``gemm_skinny``."""
    _cuda(x, w, bias, taps, conv_bias, state, seq_ctx, seq_slot)
    M, K = x.shape
    d, W = taps.shape
    if tuple(w.shape) != (3 * d, K) or not gemm_skinny_ok(x, w):
        raise KernelError(f"gemm_skinny_conv: x {tuple(x.shape)} against w {tuple(w.shape)} for {d} channels")
    if taps.dtype != torch.float32 or not taps.is_contiguous():
        raise KernelError("gemm_skinny_conv: taps must be contiguous float32 [d, W]")
    if state.dtype != torch.bfloat16 or not state.is_contiguous() or tuple(state.shape[1:]) != (W - 1, d):
        raise KernelError(f"gemm_skinny_conv: state {tuple(state.shape)} for width {W}, {d} channels")
    if seq_ctx.numel() < M or seq_slot.numel() < M:
        raise KernelError("gemm_skinny_conv: one sequence per token")
    out = torch.empty(M, d, dtype=x.dtype, device=x.device)
    _lib.call("tk_gemm_skinny_conv", _ptr(x), x.stride(0), _ptr(w), w.stride(0),
              _ptr(_f32vec(bias, "bias", 3 * d)), _ptr(out), d, M, d, K, _ptr(taps),
              _ptr(_f32vec(conv_bias, "conv bias", d)), _ptr(state), _ptr(_i32(seq_ctx, "seq_ctx")),
              _ptr(_i32(seq_slot, "seq_slot")), W, float(norm_eps), _stream())
    return out


def gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` on the CUDA cores with 32-bit accumulation, any shape.
    ``x`` [M, K] (row stride free), ``w`` [N, K]; ``bias`` float32 [N]."""
    _cuda(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or x.dtype != w.dtype or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype} against w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or x.dtype
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    _lib.call("tk_gemm_simt", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), N, M, N, K, _dtype_code(x), _dtype_code(out), _stream())
    return out


SKINNY_MAX_ROWS = 16


def gemm_skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_skinny`` takes this product: bfloat16, at most 16 rows of ``x``, K and the
    row strides multiples of 8 elements, 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


SKINNY_FUSED_ROWS = 8


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None, swiglu: bool = False, norm_eps: float = 0.0,
                residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for at most 16 rows of ``x`` (decode): a weight-streaming kernel.
    ``swiglu``: the rows of ``w`` alternate in runs of 8 (8 gate rows, the 8 up rows of the same
    channels) and the result is ``silu(gate) * up`` of width ``N / 2``.
    The two halves of a residual add + RMSNorm, for at most 8 rows: ``norm_eps`` > 0: ``x`` is the
    un-normed stream and row r of the product is scaled by ``1 / sqrt(mean(x[r]^2) + norm_eps)``
    (the norm's weight is expected in ``w``'s columns); ``residual`` [M, N]: the result is
    ``residual + product`` (the product rounded to 16 bits first, the sum once)."""
    _cuda(x, w, bias, residual)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)} against w {tuple(w.shape)}")
    width = N // 2 if swiglu else N
    if residual is not None and (tuple(residual.shape) != (M, N) or residual.dtype != torch.bfloat16
                                 or residual.stride(1) != 1):
        raise KernelError(f"gemm_skinny: residual {tuple(residual.shape)} {residual.dtype} for a "
                          f"[{M}, {N}] bfloat16 result")
    out = torch.empty(M, width, dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("tk_gemm_skinny", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), width, M, N, K, _dtype_code(out), int(swiglu), float(norm_eps), _ptr(residual),
              residual.stride(0) if residual is not None else 0, _stream())
    return out


TC_MAX_TOKENS = 256


def gemm_tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_tc`` takes this product: bfloat16, at most 256 rows of ``x``, K and the row
    strides multiples of 8 elements, 16-byte aligned bases."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= TC_MAX_TOKENS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
            out_dtype: torch.dtype | None = None, swiglu: bool = False,
            split_k: bool = True) -> torch.Tensor:
    """``x @ w.T (+ bias)`` through TMA, tcgen05.mma and tensor memory, the weight rows on the
    MMA's M axis (decode: up to 256 rows of ``x``). ``swiglu`` as in ``gemm_skinny``. ``split_k``:
    matrices with few rows may be split along K over a thread-block cluster."""
    _cuda(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: x {tuple(x.shape)} against w {tuple(w.shape)}")
    width = N // 2 if swiglu else N
    out = torch.empty(M, width, dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("tk_gemm_tc_decode", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), width, M, N, K, _dtype_code(out), int(swiglu), int(split_k), _stream())
    return out


def gemm_tc_status() -> int:
    """0, or where a tensor-core GEMM gave up waiting on a barrier since the last call (the
    kernels bound every wait instead of hanging)."""
    return _lib.call("tk_gemm_tc_status")


def sample_status() -> int:
    """0, or 1 + the first row since the last call whose logits held no finite value (the sampler
    answered token 0 for it)."""
    return _lib.call("tk_sample_status")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor,
           top_k: torch.Tensor, min_p: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
           out: torch.Tensor | None = None, scatter: tuple[torch.Tensor, torch.Tensor] | None = None
           ) -> torch.Tensor:
    """One token per row of ``logits`` [rows, V] float32; the parameters are per-row arrays.
    ``scatter`` = (index [rows] int32, target int32): also ``target[index[r]] = token``."""
    _cuda(logits, temperature, top_p, top_k, min_p, seed, step, out)
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with contiguous rows")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("min_p", min_p, torch.float32), ("top_k", top_k, torch.int32),
                        ("seed", seed, torch.int32), ("step", step, torch.int32)):
        if t.dtype != dt or t.numel() < rows or not t.is_contiguous():
            raise KernelError(f"sample: {name} must be a contiguous {dt} array of {rows}")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    idx, target = scatter if scatter is not None else (None, None)
    if scatter is not None:
        _cuda(idx, target)
        _i32(idx, "scatter index"), _i32(target, "scatter target")
    _lib.call("tk_sample", _ptr(logits), logits.stride(0), rows, V, _ptr(temperature), _ptr(top_p),
              _ptr(top_k), _ptr(min_p), _ptr(seed), _ptr(step), _ptr(out), _ptr(idx), _ptr(target),
              _stream())
    return out
