"""Grouped-query attention mixer over the paged cache.

``qkv = x @ [Wq; Wk; Wv].T``; per head of q and k an RMSNorm over the head (optional) and the
rotary encoding; the new keys and values go into the cache; every query attends over the cache
(its own step's keys included) causally, within ``window`` positions when the layer has one;
optional per-head sigmoid gate from the same input; output projection
(Tokenomos models/blocks/attention.py:225-259). ``kv_source``: the layer has queries only and
reads the cache of another call of the layer list.
"""

from __future__ import annotations

import os

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import HeadLayout, PagedKV, SharedState, StepContext, WindowKV
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import DEFAULT_TUNING, Runtime, Tuning, builder_of, register


class Attention:
    def __init__(self, qkv: Linear, o: Linear, heads: int, kv_heads: int, head_dim: int, rope,
                 eps: float, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                 window: int | None = None, scale: float | None = None,
                 gate: Linear | None = None, kv_source: int | None = None,
                 gate_fused: bool = False, tuning: Tuning = DEFAULT_TUNING):
        """``gate``: the per-head gate's projection as a part of its own; ``gate_fused``: its rows
        are the last of ``qkv``'s instead (after q, k, v, then zero rows up to a multiple of 8), so
        that one product yields both."""
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads over {kv_heads} KV heads")
        if head_dim > ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"attention: a head size of {head_dim} is above the "
                             f"{ops.ATTENTION_MAX_HEAD_DIM} the attention kernels take")
        self.qkv, self.o, self.gate = qkv, o, gate
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, head_dim
        self.rope = rope
        self.tuning = tuning
        # this part reads the batch from device tensors only; its position part must as well
        self.capture_safe = bool(getattr(rope, "capture_safe", False))
        self.eps = float(eps)
        self.q_norm = q_norm.float().contiguous() if q_norm is not None else None
        self.k_norm = k_norm.float().contiguous() if k_norm is not None else None
        self.window = window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.kv_source = kv_source
        own_kv = 0 if kv_source is not None else kv_heads
        self.qkv_width = (heads + 2 * own_kv) * head_dim
        self.gate_fused = gate_fused
        if gate_fused and gate is not None:
            raise ValueError("attention: the gate is either fused into qkv or a projection of its own")
        if qkv.out_features != self.qkv_width + (-(-heads // 8) * 8 if gate_fused else 0):
            raise ValueError("attention: the fused projection does not match the head counts")
        self.norm_folded = False
        self._fused_freqs = None        # the rotation's frequencies once asked for; False: not fusable
        self.head_layout = HeadLayout(heads, own_kv, head_dim, self.q_norm,
                                      self.k_norm if own_kv else None, self.eps)

    def state_specs(self) -> dict:
        if self.kv_source is not None:
            return {"kv": SharedState(self.kv_source, "kv")}
        if self.window is None:
            return {"kv": PagedKV(self.kv_heads, self.head_dim)}
        return {"kv": WindowKV(self.kv_heads, self.head_dim, self.window)}

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        T = x.shape[0]
        out = self._heads(self.qkv(x), x, ctx, call)
        return self.o(out.view(T, self.heads * self.head_dim))

    def _heads(self, proj: torch.Tensor, x: torch.Tensor | None, ctx: StepContext, call: int) -> torch.Tensor:
        """From the fused projection's rows to the gated heads' outputs [T, H, D]."""
        if self._fused_decode(ctx):
            return self._decode_fused(proj, ctx, call)
        n = self.qkv_width
        if self.gate_fused:
            return self._core(proj[:, :n], ctx, call, proj[:, n:n + self.heads])
        return self._core(proj, ctx, call, self.gate(x) if self.gate is not None else None)

    # ---- the block's norm and residual add taken into the two products (parts.contract) ----

    def fold_norm(self, weight: torch.Tensor) -> bool:
        if self.qkv.weight.dtype != torch.bfloat16 or not self.tuning.fuse_norms or self.gate is not None:
            return False
        self.qkv.fold_columns(weight)
        self.norm_folded = True
        return True

    def can_stream(self, rows: int, ctx: StepContext) -> bool:
        return (self.norm_folded and rows <= ops.SKINNY_FUSED_ROWS and self.qkv.in_features % 8 == 0
                and self.qkv.out_features % 8 == 0 and self.o.in_features % 8 == 0)

    def forward_stream(self, stream: torch.Tensor, eps: float, ctx: StepContext, call: int) -> torch.Tensor:
        self.qkv.note("skinny+norm")
        self.o.note("skinny+add")
        T = stream.shape[0]
        proj = ops.gemm_skinny(stream, self.qkv.weight, self.qkv.bias, norm_eps=eps)
        out = self._heads(proj, None, ctx, call)
        return ops.gemm_skinny(out.view(T, self.heads * self.head_dim), self.o.weight, self.o.bias,
                               residual=stream)

    # whether decode steps may take the one-kernel form (TOKENOMOS_B200_ATTN_FUSED=0: never)
    decode_fused = os.environ.get("TOKENOMOS_B200_ATTN_FUSED", "1") != "0"

    def _fused_decode(self, ctx: StepContext) -> bool:
        """Whether this step's attention runs as one kernel: every sequence brings one token, the
        position encoding is a plain rotation that says so, and the kernel takes the shape."""
        if not (self.decode_fused and ctx.host.decode_only and self.gate is None
                and ctx.n_tokens <= self.tuning.decode_fused_rows):
            return False
        if self._fused_freqs is None:
            offer = getattr(self.rope, "rotate_half_frequencies", None)
            freqs = offer() if offer is not None else None
            self._fused_freqs = freqs if freqs is not None and ops.attention_decode_fused_supported(
                self.heads, self.kv_heads, self.head_dim, 2 * freqs.numel(), self.qkv.weight.dtype) else False
        return self._fused_freqs is not False

    def _decode_fused(self, proj: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        """From the fused projection's rows (q, k, v and the gate's columns) to the gated heads'
        outputs [T, H, D] in one kernel."""
        pool = ctx.states[(call, "kv")]
        table = ctx.block_tables[ctx.state_groups[(call, "kv")]]
        layout = self.head_layout
        longest = ctx.host.longest
        if self.window is not None:
            longest = min(longest, self.window)
        nsplit = self.fused_splits(ctx.n_tokens, self.kv_heads, longest, self.tuning)
        n = self.qkv_width
        gate = proj[:, n:n + self.heads] if self.gate_fused else None
        return ops.attention_decode_fused(
            proj, pool, layout.q_norm, layout.k_norm if layout.kv_heads else None, layout.eps,
            self._fused_freqs, gate, ctx.positions, ctx.tok_seq, table, self.heads, self.kv_heads,
            self.window, self.scale, nsplit, write_kv=bool(layout.kv_heads),
            carveout=self.tuning.decode_fused_carveout if ctx.n_tokens <= self.tuning.skinny_rows else -1)

    def _core(self, qkv: torch.Tensor, ctx: StepContext, call: int,
              gate: torch.Tensor | None = None) -> torch.Tensor:
        """From q, k, v to the heads' outputs [T, H, D]: q/k norm, rotation, cache write, attention
        over the cache, the per-head output gate ``gate`` [T, H] if the layer has one (the
        tensor-core kernels apply it as they write, the generic one is followed by a kernel)."""
        pool = ctx.states[(call, "kv")]
        table = ctx.block_tables[ctx.state_groups[(call, "kv")]]
        own_kv = self.head_layout.kv_heads
        q = self.rope.encode_qk(qkv, ctx, self.head_layout, pool if own_kv else None,
                                table if own_kv else None)
        if ops.attention_mma_supported(self.heads, self.kv_heads, self.head_dim, q.dtype):
            return self._attend_mma(q, pool, table, ctx, gate)
        rows = ops.attention_rows()
        group = self.heads // self.kv_heads
        per_tile = max(1, rows // group)
        _, tok0, _, ntok = ctx.tiles(per_tile)
        out = ops.attention(q, pool, ctx.positions, ctx.tok_seq, table, tok0, ntok, per_tile,
                            self.window, self.scale)
        if gate is not None:
            ops.head_gate(out, gate, self.heads, self.head_dim)
        return out

    # whether prompt portions may take the tcgen05 kernel (TOKENOMOS_B200_ATTN_TC=0: never)
    prefill_tc = os.environ.get("TOKENOMOS_B200_ATTN_TC", "1") != "0"

    @staticmethod
    def decode_splits(rows: int, kv_heads: int, longest: int, tuning: Tuning = DEFAULT_TUNING) -> int:
        """Ways to split each decoded token's keys over CTAs, for ``rows`` tokens whose sequences
        hold at most ``longest`` positions, which is all a captured step knows (in practice a CTA
        then reads about half as many keys as the rule aims at). The thresholds are ``Tuning``'s,
        measured at batch 1 to 64 and 512 to 32,768 cached positions."""
        per_split = max(1, rows * kv_heads)                 # CTAs one split puts on the GPU
        by_keys = -(-longest // tuning.decode_keys)
        to_fill = min(-(-tuning.decode_fill // per_split), -(-longest // tuning.decode_min_keys))
        most = tuning.decode_ctas_per_sm * tuning.sm_count
        return max(1, min(-(-most // per_split), max(by_keys, to_fill)))

    @staticmethod
    def fused_splits(rows: int, kv_heads: int, longest: int, tuning: Tuning = DEFAULT_TUNING) -> int:
        """The same for the one-kernel form: as many splits as keep every CTA resident at once
        (``decode_fused_ctas_per_sm`` fit an SM by shared memory; one CTA more than that and the
        kernel runs in two waves: 0.82 ms a step against 0.76 at 8 rows and 4,000 positions),
        never fewer than ``decode_min_keys`` keys each. The CTA that merges the splits does so
        alone, so fewer and longer splits beat the other kernel's rule at every length measured
        (2,048 to 32,000 positions)."""
        per_split = max(1, rows * kv_heads)
        resident = tuning.decode_fused_ctas_per_sm * tuning.sm_count // per_split
        return max(1, min(resident, -(-longest // tuning.decode_min_keys)))

    @staticmethod
    def prefill_splits(tokens: int, entries: int, per_tile: int, kv_heads: int,
                       tuning: Tuning = DEFAULT_TUNING) -> int:
        """The most CTAs that may share one tile's keys in the tcgen05 prefill kernel, for a step
        of ``tokens`` tokens whose tile list has ``entries`` entries (a captured step's list is
        longer than what it uses). A tile is walked by one CTA, key tile after key tile; a step
        with few tiles behind a long context would leave the GPU idle for hundreds of
        microseconds (128 tokens behind 32,000 positions: 474 us a layer, 98 us shared 8 ways).
        So: as many as fill the GPU once (``prefill_split_ctas_per_sm`` CTAs an SM), no more than
        the scratch memory for the shares allows; the kernel gives each tile as many of them as
        leave a CTA 8 key tiles, so a short context uses one whatever this says."""
        tiles = max(1, -(-tokens // per_tile))
        by_ctas = tuning.prefill_split_ctas_per_sm * tuning.sm_count // (tiles * max(1, kv_heads))
        by_memory = (tuning.prefill_split_scratch_mb << 20) // (max(1, entries) * max(1, kv_heads) * 128 * 66 * 4)
        return max(1, min(16, by_ctas, by_memory))

    def _attend_mma(self, q, pool, table, ctx: StepContext, gate=None) -> torch.Tensor:
        """The tensor-core kernels: prompt portions in tiles of 64 rows, decoded tokens split
        over their keys so that a small batch still fills the GPU."""
        out = torch.empty_like(q)
        # prompt portions: the tcgen05 kernel (tiles of 128 rows) where it takes the shape, else
        # the mma.sync one (tiles of 64 rows)
        tc = self.prefill_tc and ops.attention_prefill_tc_supported(self.heads, self.kv_heads, self.head_dim,
                                                                     q.dtype)
        per_tile = (ops.attention_prefill_tc_tokens if tc else ops.attention_prefill_mma_tokens)(
            self.heads, self.kv_heads)
        _, tok0, _, ntok = ctx.tiles(per_tile, "multi")
        if tok0.numel() and tc:
            nsplit = self.prefill_splits(ctx.n_tokens, tok0.numel(), per_tile, self.kv_heads, self.tuning)
            ops.attention_prefill_tc(q, pool, out, ctx.positions, ctx.tok_seq, table, tok0, ntok, self.window,
                                     self.scale, gate, nsplit)
        elif tok0.numel():
            ops.attention_prefill_mma(q, pool, out, ctx.positions, ctx.tok_seq, table, tok0, ntok, self.window,
                                      self.scale, gate)
        # every sequence brings one token: row i is sequence i's, no list of rows needed
        decode_only = ctx.host.decode_only
        singles = None if decode_only else ctx.singles()
        if decode_only or singles.numel():
            longest = ctx.host.longest
            if self.window is not None:
                longest = min(longest, self.window)
            rows = ctx.n_tokens if decode_only else singles.numel()
            nsplit = self.decode_splits(rows, self.kv_heads, longest, self.tuning)
            ops.attention_decode_mma(q, pool, out, ctx.positions, ctx.tok_seq, table, singles,
                                     self.window, self.scale, nsplit, gate)
        return out


@register("mixer", "attention")
def build_attention(params: dict, tensors: dict, rt: Runtime) -> Attention:
    rope_spec = params["position"]
    # tensors whose role name starts with "position." belong to the position encoding
    own = {k[len("position."):]: v for k, v in tensors.items() if k.startswith("position.")}
    rope = builder_of("position", rope_spec["kind"])(rope_spec["params"], own, rt)
    source = params.get("kv_source")
    mats = [tensors["q"]] if source is not None else [tensors["q"], tensors["k"], tensors["v"]]
    gated = "gate" in tensors
    if gated:
        # the gate reads the same input as q, k, v: its rows join theirs (padded to whole
        # 16-byte chunks of the output row), one product instead of two
        g = tensors["gate"]
        pad = -g.shape[0] % 8
        mats.append(torch.cat((g, g.new_zeros(pad, g.shape[1]))) if pad else g)
    return Attention(
        Linear.fused(mats, tuning=rt.tuning), Linear(tensors["o"], tuning=rt.tuning), params["heads"],
        params["kv_heads"], params["head_dim"], rope, params["eps"], tensors.get("q_norm"),
        tensors.get("k_norm"), params.get("window"), params.get("scale"), None, source,
        gate_fused=gated, tuning=rt.tuning)
