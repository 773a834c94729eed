"""A plain, slow implementation of the LFM3 hybrid conv decoder: whole sequences, no cache, one
function per part, plain torch on the CPU. It shares no code with ``tokenomos_b200``: it reads
the safetensors file and config.json itself and restates the reference's formulas, each cited
by file:line of KohakuBlueleaf/Tokenomos. It is the oracle of the tests, never a fallback.

``tests/golden/`` holds logits that Tokenomos's own model code produced on the CPU for a tiny
random model (see ``tests/golden/make_golden.py``); ``tests/test_plain.py`` holds this file to
them, so the oracle rests on the reference's code and not only on a reading of it.

Everything is computed in ``dtype`` (float64 by default) except the rotary angle, which the
reference forms as a float32 product ``float(pos) * inv_freq`` (models/blocks/rope.py:33-35,
51-54): that rounding is part of the model's definition and is kept.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open


# ---- reading a model folder -------------------------------------------------------------------

def read_folder(path) -> tuple[dict, dict[str, torch.Tensor]]:
    path = Path(path)
    config = json.loads((path / "config.json").read_text("utf-8"))
    tensors = {}
    with safe_open(path / "model.safetensors", "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return config, tensors


def settings(config: dict) -> dict:
    """The constants the formulas need, with the defaults the reference's declaration applies
    (models/lfm3/arch.py:57-67,78,95,106; models/load/checkpoint.py:160-165)."""
    c = config.get("text_config", config)
    heads = c["num_attention_heads"]
    head_dim = c.get("head_dim", c["hidden_size"] // heads)
    ropes = {}
    params = c.get("rope_parameters")
    kinds = sorted({k for k in c["layer_types"] if k != "conv"})
    for kind in kinds:
        if params is not None:
            p = params if "rope_theta" in params else params[kind]
            theta, factor = p["rope_theta"], p.get("partial_rotary_factor", 1.0)
        else:
            theta, factor = c["rope_theta"], c.get("partial_rotary_factor", 1.0)
        ropes[kind] = (float(theta), int(factor * head_dim) // 2)
    if "tie_word_embeddings" in config:
        tied = config["tie_word_embeddings"]
    elif "tie_embedding" in config:
        tied = config["tie_embedding"]
    else:
        tied = c.get("tie_word_embeddings", c.get("tie_embedding", True))
    return dict(
        layer_types=list(c["layer_types"]), heads=heads, kv_heads=c["num_key_value_heads"],
        head_dim=head_dim, eps=c["norm_eps"], ropes=ropes, tied=bool(tied),
        window=c.get("sliding_window"), sandwich=c.get("use_sandwich_norm", False),
        conv_bias=c.get("conv_bias", False), width=c["conv_L_cache"])


# ---- parts ------------------------------------------------------------------------------------

def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w``, eps inside the root, mean over the full last dim
    (models/blocks/norm.py:41-45; kernels/norm/fused.py:22-28)."""
    rstd = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * rstd * weight.to(x.dtype)


def rope_tables(positions: torch.Tensor, head_dim: int, angles: int, theta: float, dtype):
    """cos / sin [T, head_dim]: ``inv_i = theta ** (-2 i / head_dim)`` for ``i < angles``, zero
    for the rest of ``head_dim / 2``; the angle is a float32 product; the table is
    ``cat(f, f)`` (models/blocks/rope.py:33-35,51-59)."""
    idx = torch.arange(0, 2 * angles, 2, dtype=torch.float32)
    inv = 1.0 / (theta ** (idx / head_dim))
    inv = torch.cat((inv, torch.zeros(head_dim // 2 - angles, dtype=torch.float32)))
    freqs = positions.to(torch.float32)[:, None] * inv[None, :]   # float32, as the reference
    emb = torch.cat((freqs, freqs), dim=-1).to(torch.float64)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half: ``x * cos + cat(-x[half:], x[:half]) * sin`` on [T, heads, D]
    (models/blocks/rope.py:66-73; kernels/attention/qk.py:72-94)."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos[:, None, :] + rot * sin[:, None, :]


def attention(x, w, prefix: str, s: dict, kind: str, dtype) -> torch.Tensor:
    """GQA attention of one whole sequence ``x`` [T, d] (models/blocks/attention.py:197-259):
    q/k/v projections, per-head RMSNorm of q and k, RoPE on q and k, scores ``q.k * D^-0.5``,
    key j visible to query i iff ``j <= i`` and, on a sliding layer, ``i - j < window``
    (models/blocks/attention.py:31-40), softmax, optional per-head sigmoid gate from the same
    input, output projection. Query head h reads KV head ``h // (H / Hkv)``
    (kernels/attention/paged.py:200)."""
    T = x.shape[0]
    H, Hkv, D = s["heads"], s["kv_heads"], s["head_dim"]
    q = (x @ w[f"{prefix}q_proj.weight"].to(dtype).T).view(T, H, D)
    k = (x @ w[f"{prefix}k_proj.weight"].to(dtype).T).view(T, Hkv, D)
    v = (x @ w[f"{prefix}v_proj.weight"].to(dtype).T).view(T, Hkv, D)
    q = rmsnorm(q, w[f"{prefix}q_norm.weight"], s["eps"])
    k = rmsnorm(k, w[f"{prefix}k_norm.weight"], s["eps"])
    theta, angles = s["ropes"][kind]
    cos, sin = rope_tables(torch.arange(T), D, angles, theta, dtype)
    q, k = rotate(q, cos, sin), rotate(k, cos, sin)
    group = H // Hkv
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * (D ** -0.5)
    i = torch.arange(T)
    visible = i[None, :] <= i[:, None]
    if kind == "sliding_attention":
        visible &= (i[:, None] - i[None, :]) < s["window"]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", p, v)
    gate = f"{prefix}gate_proj.weight"
    if gate in w:
        g = x @ w[gate].to(dtype).T                      # [T, H]
        out = out * torch.sigmoid(g)[:, :, None]
    return out.reshape(T, H * D) @ w[f"{prefix}o_proj.weight"].to(dtype).T


def short_conv(x, w, prefix: str, s: dict, dtype) -> torch.Tensor:
    """Gated short convolution of one whole sequence (models/blocks/shortconv.py:39-59):
    ``B, C, X = in_proj(x)`` in that order along the output axis; ``u = B * X``;
    ``y[t] = sum_j w[:, j] * u[t - (W - 1 - j)]`` (+ bias), zeros before the sequence, tap
    ``W - 1`` on the current token, no activation (kernels/conv/varlen.py:73-93,
    models/lfm3/arch.py:76-85); ``out_proj(C * y)``."""
    T, d = x.shape
    bcx = x @ w[f"{prefix}in_proj.weight"].to(dtype).T
    if f"{prefix}in_proj.bias" in w:
        bcx = bcx + w[f"{prefix}in_proj.bias"].to(dtype)
    B, C, X = bcx[:, :d], bcx[:, d:2 * d], bcx[:, 2 * d:]
    u = B * X
    taps = w[f"{prefix}conv.weight"].to(dtype)
    taps = taps.view(taps.shape[0], taps.shape[-1])      # [d, W]
    W = taps.shape[1]
    padded = torch.cat((torch.zeros(W - 1, d, dtype=dtype), u), dim=0)
    y = torch.zeros(T, d, dtype=dtype)
    for j in range(W):
        y = y + padded[j:j + T] * taps[:, j][None, :]
    if f"{prefix}conv.bias" in w:
        y = y + w[f"{prefix}conv.bias"].to(dtype)
    out = (C * y) @ w[f"{prefix}out_proj.weight"].to(dtype).T
    if f"{prefix}out_proj.bias" in w:
        out = out + w[f"{prefix}out_proj.bias"].to(dtype)
    return out


def swiglu(x, w, prefix: str, dtype) -> torch.Tensor:
    """``w2(silu(w1 x) * w3 x)`` (models/blocks/ffn.py:25-32; models/lfm3/arch.py:102-105)."""
    g = x @ w[f"{prefix}w1.weight"].to(dtype).T
    u = x @ w[f"{prefix}w3.weight"].to(dtype).T
    return (torch.nn.functional.silu(g) * u) @ w[f"{prefix}w2.weight"].to(dtype).T


# ---- the model --------------------------------------------------------------------------------

def forward_logits(config: dict, w: dict, ids: list[int], dtype=torch.float64) -> torch.Tensor:
    """Teacher-forced logits [len(ids), vocab] of one sequence. Residual wiring: pre-norm,
    ``r += mixer(N_op(r))``, ``r += ffn(N_ffn(r))``, with sandwich norms the block outputs pass
    ``post_operator_norm`` / ``post_ffn_norm`` before the add; final ``embedding_norm``; head is
    the embedding when tied (models/blocks/decoder.py:104-125,173-195; models/lfm3/arch.py:
    106-126)."""
    s = settings(config)
    root = "model.language_model." if "model.language_model.embed_tokens.weight" in w else "model."
    emb = w[f"{root}embed_tokens.weight"].to(dtype)
    r = emb[torch.tensor(ids, dtype=torch.long)]
    for i, kind in enumerate(s["layer_types"]):
        p = f"{root}layers.{i}."
        x = rmsnorm(r, w[f"{p}operator_norm.weight"], s["eps"])
        if kind == "conv":
            m = short_conv(x, w, f"{p}conv.", s, dtype)
        else:
            m = attention(x, w, f"{p}self_attn.", s, kind, dtype)
        if s["sandwich"]:
            m = rmsnorm(m, w[f"{p}post_operator_norm.weight"], s["eps"])
        r = r + m
        x = rmsnorm(r, w[f"{p}ffn_norm.weight"], s["eps"])
        f = swiglu(x, w, f"{p}feed_forward.", dtype)
        if s["sandwich"]:
            f = rmsnorm(f, w[f"{p}post_ffn_norm.weight"], s["eps"])
        r = r + f
    out = rmsnorm(r, w[f"{root}embedding_norm.weight"], s["eps"])
    head = emb if s["tied"] else w["lm_head.weight"].to(dtype)
    return out @ head.T


def sample_greedy(logits_row: torch.Tensor) -> int:
    """The first maximum (kernels/sampling/sample.py:60-66)."""
    return int(torch.argmax(logits_row))


def generate_greedy(config: dict, w: dict, prompt: list[int], steps: int, dtype=torch.float64):
    """Greedy continuation by re-running the whole sequence each step (no cache)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        tok = sample_greedy(forward_logits(config, w, ids, dtype)[-1])
        out.append(tok)
        ids.append(tok)
    return out
