"""Host side of the sampler: per-row parameter arrays for the sampling kernel.

A row's random stream is keyed by (seed, step) with ``step`` the number of tokens the request
has generated so far, and the vocabulary index as the counter, so a request draws the same
tokens alone, in any batch, and after being recomputed (Tokenomos kernels/sampling/sample.py:
1-11 has the same contract; the generator's bits differ)."""

from __future__ import annotations

import struct

import torch

from tokenomos_b200 import ops


def pack_rows(rows: list[tuple[float, float, int, float, int, int]]) -> list[int]:
    """(temperature, top_p, top_k, min_p, seed, step) per row -> int32 words, column-major
    (all temperatures, all top_p, ...), floats by their bit pattern, ready for one upload."""
    def bits(x: float) -> int:
        return struct.unpack("<i", struct.pack("<f", x))[0]

    n = len(rows)
    out = [0] * (6 * n)
    for i, (t, p, k, m, seed, step) in enumerate(rows):
        out[i] = bits(float(t))
        out[n + i] = bits(float(p))
        out[2 * n + i] = int(k)
        out[3 * n + i] = bits(float(m))
        out[4 * n + i] = int(seed) & 0x7FFFFFFF
        out[5 * n + i] = int(step)
    return out


def pack_rows_into(dst, rows: list[tuple[float, float, int, float, int, int]], n: int) -> None:
    """``pack_rows`` straight into ``dst``, a numpy int32 view of ``6 * n`` words; rows beyond
    ``len(rows)`` are greedy padding."""
    import numpy as np

    k = len(rows)
    f = dst.view(np.float32)
    dst[:] = 0
    f[n:2 * n] = 1.0
    if k:
        cols = list(zip(*rows))
        f[0:k] = cols[0]
        f[n:n + k] = cols[1]
        dst[2 * n:2 * n + k] = cols[2]
        f[3 * n:3 * n + k] = cols[3]
        dst[4 * n:4 * n + k] = [int(v) & 0x7FFFFFFF for v in cols[4]]
        dst[5 * n:5 * n + k] = cols[5]


def sample_packed(logits: torch.Tensor, packed: torch.Tensor, out: torch.Tensor | None = None,
                  scatter=None):
    """``packed``: device int32 [6 * rows] from ``pack_rows``."""
    n = logits.shape[0]
    f = packed.view(torch.float32)
    return ops.sample(logits, f[:n], f[n:2 * n], packed[2 * n:3 * n], f[3 * n:4 * n],
                      packed[4 * n:5 * n], packed[5 * n:6 * n], out, scatter)
