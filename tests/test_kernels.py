"""Each CUDA kernel alone against a plain float64 reference of the same op, at sizes other than
the engine's tiny models: widths and vocabularies that are no power of two, head sizes in steps
of 16 (and 24), any number of heads and groups, several page sizes. Where random inputs would
hide a fault the inputs are made so that it shows: a far key whose score dominates, keys at the
window's edge, unread cache rows poisoned with NaN."""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, what="", scale=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all(), what
    s = scale if scale is not None else max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    assert err <= tol(dtype) * s, f"{what}: error {err:.3e} allowed {tol(dtype) * s:.3e}"


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ---- gather / norm / swiglu / gate -------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [100, 128, 2050])
def test_gather_rows(dtype, width):
    from tokenomos_b200 import ops
    table = torch.randn(37, width).to(dtype)
    ids = [36, 0, 5, 5, 17]
    out = ops.gather_rows(dev(table), i32(ids))
    assert torch.equal(out.cpu(), table[ids])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [100, 2048])
def test_gather_rows_select(dtype, width):
    """Row r reads the id the host gave, or the one an earlier step left for its slot."""
    from tokenomos_b200 import ops
    table = torch.randn(41, width).to(dtype)
    ids_host = [3, 40, 7, 0, 9]
    use_prev = [0, 1, 1, 0, 1]
    slot = [2, 5, 1, 4, 3]
    last = [11, 12, 13, 14, 15, 16, 17]
    out = ops.gather_rows_select(dev(table), i32(ids_host), i32(use_prev), i32(last), i32(slot))
    want = [last[slot[r]] if use_prev[r] else ids_host[r] for r in range(5)]
    assert torch.equal(out.cpu(), table[want])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [100, 2048, 5000])
@pytest.mark.parametrize("residual, pre", [(False, False), (True, False), (True, True)])
def test_add_rmsnorm(dtype, width, residual, pre):
    from tokenomos_b200 import ops
    rows, eps = 7, 3e-6
    x = (torch.randn(rows, width) * 3).to(dtype)
    r = torch.randn(rows, width).to(dtype) if residual else None
    w = 1 + 0.2 * torch.randn(width)
    wp = 1 + 0.2 * torch.randn(width)

    def rms(v, weight, e):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + e) * weight.double()

    xd = x.double()
    if pre:
        xd = rms(xd, wp, 1e-5)
    stream = xd + r.double() if residual else xd
    want = rms(stream, w, eps)
    y, s = ops.add_rmsnorm(dev(x), dev(r) if residual else None, dev(w), eps,
                           (dev(wp), 1e-5) if pre else None)
    close(y, want, dtype, "normed")
    close(s, stream, dtype, "stream")


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_rmsnorm_strided_input(dtype):
    from tokenomos_b200 import ops
    big = torch.randn(5, 300).to(dtype)
    x = big[:, 100:200]
    w = torch.ones(100)
    y, _ = ops.add_rmsnorm(dev(big)[:, 100:200], None, dev(w), 1e-5)
    xd = x.double()
    close(y, xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + 1e-5), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_head_gate(dtype):
    from tokenomos_b200 import ops
    gu = (torch.randn(9, 2 * 77) * 2).to(dtype)
    out = ops.swiglu(dev(gu))
    g, u = gu.double()[:, :77], gu.double()[:, 77:]
    close(out, torch.nn.functional.silu(g) * u, dtype, "swiglu")
    x = torch.randn(6, 5, 24).to(dtype)
    gate = torch.randn(6, 5).to(dtype)
    got = ops.head_gate(dev(x).clone(), dev(gate), 5, 24)
    close(got, x.double() * torch.sigmoid(gate.double())[:, :, None], dtype, "head gate")
    # head sizes in whole 16-byte chunks (the vector form in bfloat16), the gate a column block
    # of a wider tensor, enough rows for several trips of the grid-stride loop
    for T, H, D in ((3, 4, 16), (700, 32, 64), (41, 6, 40)):
        x = torch.randn(T, H, D).to(dtype)
        wide = torch.randn(T, H + 11).to(dtype)
        got = ops.head_gate(dev(x).clone(), dev(wide)[:, 3:3 + H], H, D)
        want = x.double() * torch.sigmoid(wide[:, 3:3 + H].double())[:, :, None]
        close(got, want, dtype, f"head gate {T}x{H}x{D}")
        if dtype == torch.bfloat16:      # bit for bit what the scalar form gives (head size 24 above)
            s = torch.sigmoid(wide[:, 3:3 + H].float()).to(dtype).float()
            assert torch.equal(got.cpu(), (x.float() * s[:, :, None]).to(dtype))


# ---- matrix product ----------------------------------------------------------------------------

@pytest.mark.parametrize("m, n, k", [(1, 33, 17), (5, 1000, 96), (70, 130, 2048), (64, 64, 16), (129, 65, 200)])
@pytest.mark.parametrize("in_dtype, out_dtype", [(torch.float32, torch.float32),
                                                 (torch.bfloat16, torch.bfloat16),
                                                 (torch.bfloat16, torch.float32)])
def test_gemm_simt(m, n, k, in_dtype, out_dtype):
    from tokenomos_b200 import ops
    x = torch.randn(m, k).to(in_dtype)
    w = torch.randn(n, k).to(in_dtype)
    b = torch.randn(n)
    want = x.double() @ w.double().T + b.double()
    got = ops.gemm(dev(x), dev(w), dev(b), out_dtype)
    assert got.dtype == out_dtype
    close(got, want, out_dtype, f"gemm {m}x{n}x{k}")
    # a row-strided input (a slice of a wider activation)
    wide = torch.randn(m, k + 40).to(in_dtype)
    got = ops.gemm(dev(wide)[:, 8:8 + k], dev(w), None, out_dtype)
    close(got, wide[:, 8:8 + k].double() @ w.double().T, out_dtype, "strided gemm")


def test_gemm_float32_is_not_tf32():
    """A product whose exact value needs more than TF32's 10 mantissa bits."""
    from tokenomos_b200 import ops
    x = torch.full((4, 64), 1.0 + 2.0 ** -12)
    w = torch.full((8, 64), 1.0 + 2.0 ** -12)
    got = ops.gemm(dev(x), dev(w)).double().cpu()
    want = x.double() @ w.double().T
    assert (got - want).abs().max().item() < 1e-5
    assert (want - 64.0).abs().min().item() > 1e-2   # TF32 inputs would give exactly 64


@pytest.mark.parametrize("dtype", DTYPES)
def test_scale_rows_and_logit_options(dtype):
    from tokenomos_b200 import ops
    x = torch.randn(7, 301).to(dtype)
    got = ops.scale_rows(dev(x.clone()), 3.3)
    s = torch.tensor(3.3).to(dtype).double()                  # the scale is rounded to the storage type first
    assert torch.equal(got.cpu(), (x.double() * s).to(dtype))
    logits = torch.randn(5, 1003) * 30
    strided = dev(torch.cat((logits, torch.zeros(5, 13)), 1))[:, :1003]       # rows 1016 apart
    ids = [0, 17, 1002]
    ops.logit_options(strided, 12.5, i32(ids))
    want = 12.5 * torch.tanh(logits.double() / 12.5)
    keep = [c for c in range(1003) if c not in ids]
    assert torch.isneginf(strided[:, ids]).all()
    assert (strided.double().cpu()[:, keep] - want[:, keep]).abs().max().item() < 1e-5
    only_suppress = dev(logits.clone())
    ops.logit_options(only_suppress, None, i32([5]))
    assert torch.isneginf(only_suppress[:, 5]).all() and torch.equal(only_suppress[:, 6:].cpu(), logits[:, 6:])
    untouched = dev(logits.clone())
    ops.logit_options(untouched, None, None)
    assert torch.equal(untouched.cpu(), logits)


# ---- q/k norm + rotary + cache write -----------------------------------------------------------

def rope_ref(x, pos, inv_freq, rot):
    """x [T, H, D] float64; rotate-half on the first ``rot`` dims with float32 angles."""
    f = pos.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((f, f), -1).double()
    cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
    xr, rest = x[..., :rot], x[..., rot:]
    half = rot // 2
    rotated = torch.cat((-xr[..., half:], xr[..., :half]), -1)
    return torch.cat((xr * cos + rotated * sin, rest), -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, Hkv, D, angles, P", [(4, 2, 16, 8, 16), (3, 1, 24, 12, 8), (8, 8, 64, 16, 4),
                                                  (6, 2, 128, 64, 32), (2, 1, 48, 24, 5)])
def test_qk_norm_rope_write(dtype, H, Hkv, D, angles, P):
    from tokenomos_b200 import ops
    T, eps, theta = 11, 1e-6, 10000.0
    pos = torch.tensor([0, 1, 2, 3, 4000, 4001, 7, 8, 9, 10, 11])
    seq = torch.tensor([0, 0, 0, 0, 1, 1, 2, 2, 2, 2, 2])
    blocks = 4002 // P + 1
    table = torch.randperm(3 * blocks)[: 3 * blocks].view(3, blocks).to(torch.int32) + 1
    pages = 3 * blocks + 1
    qkv = torch.randn(T, (H + 2 * Hkv) * D).to(dtype)
    wq, wk = 1 + 0.3 * torch.randn(D), 1 + 0.3 * torch.randn(D)
    inv = 1.0 / (theta ** (torch.arange(0, 2 * angles, 2, dtype=torch.float32) / D))
    inv = torch.cat((inv, torch.zeros(D // 2 - angles)))
    pool = torch.full((pages, 2, Hkv, P, D), float("nan"), dtype=dtype, device="cuda")
    q = ops.qk_norm_rope_write(dev(qkv), pool, dev(wq), dev(wk), eps, dev(inv), i32(pos.tolist()),
                               i32(seq.tolist()), dev(table), H, Hkv, D, P)
    x = qkv.double().view(T, H + 2 * Hkv, D)

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.double()

    want_q = rope_ref(norm(x[:, :H], wq), pos, inv, D)
    want_k = rope_ref(norm(x[:, H:H + Hkv], wk), pos, inv, D)
    want_v = x[:, H + Hkv:]
    close(q, want_q, dtype, "q")
    pool = pool.cpu()
    written = torch.zeros(pages, P, dtype=torch.bool)
    for t in range(T):
        page, row = int(table[seq[t], pos[t] // P]), int(pos[t] % P)
        close(pool[page, 0, :, row], want_k[t], dtype, f"k of token {t}", scale=want_k.abs().max().item())
        assert torch.equal(pool[page, 1, :, row].double(), want_v[t]), f"v of token {t}"
        written[page, row] = True
    # nothing else was touched
    assert torch.isnan(pool[:, :, :, :, 0].double()[~written[:, None, None, :].expand(-1, 2, Hkv, -1)]).all()


# ---- paged attention ---------------------------------------------------------------------------

def attention_case(dtype, H, Hkv, D, P, seqs, window=None, poison=True, boost=None):
    """``seqs``: list of (ctx, n). Builds a shuffled paged cache holding every sequence's keys
    for positions [0, ctx + n), runs the kernel for the last n of each, returns (got, want)."""
    from tokenomos_b200 import ops
    G = H // Hkv
    total = [c + n for c, n in seqs]
    blocks = [-(-t // P) for t in total]
    width = max(blocks)
    pages = sum(blocks) + 1
    perm = (torch.randperm(pages - 1) + 1).tolist()
    fill = float("nan") if poison else 0.0
    pool = torch.full((pages, 2, Hkv, P, D), fill, dtype=torch.float64)
    table = torch.zeros(len(seqs), width, dtype=torch.int32)
    ks, vs, qs = [], [], []
    for s, (c, n) in enumerate(seqs):
        k = torch.randn(total[s], Hkv, D).to(dtype).double()
        v = torch.randn(total[s], Hkv, D).to(dtype).double()
        q = torch.randn(n, H, D).to(dtype).double()
        if boost is not None:
            boost(s, q, k, v)
        for b in range(blocks[s]):
            page = perm.pop()
            table[s, b] = page
            rows = min(P, total[s] - b * P)
            pool[page, 0, :, :rows] = k[b * P:b * P + rows].transpose(0, 1)
            pool[page, 1, :, :rows] = v[b * P:b * P + rows].transpose(0, 1)
        ks.append(k), vs.append(v), qs.append(q)
    positions = [p for (c, n) in seqs for p in range(c, c + n)]
    tok_seq = [s for s, (c, n) in enumerate(seqs) for _ in range(n)]
    per_tile = max(1, ops.attention_rows() // G)
    tok0, ntok, start = [], [], 0
    for c, n in seqs:
        for o in range(0, n, per_tile):
            tok0.append(start + o)
            ntok.append(min(per_tile, n - o))
        start += n
    got = ops.attention(dev(torch.cat(qs), dtype), dev(pool, dtype), i32(positions), i32(tok_seq),
                        dev(table), i32(tok0), i32(ntok), per_tile, window, D ** -0.5)
    want = []
    for s, (c, n) in enumerate(seqs):
        k = ks[s].repeat_interleave(G, 1)
        v = vs[s].repeat_interleave(G, 1)
        sc = torch.einsum("ihd,jhd->hij", qs[s], k) * D ** -0.5
        i = torch.arange(c, c + n)[:, None]
        j = torch.arange(total[s])[None, :]
        vis = j <= i
        if window:
            vis &= (i - j) < window
        sc = sc.masked_fill(~vis[None], float("-inf"))
        want.append(torch.einsum("hij,jhd->ihd", sc.softmax(-1), v))
    return got, torch.cat(want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, Hkv, D, P", [(4, 2, 16, 16), (4, 1, 24, 8), (6, 2, 32, 4), (8, 2, 64, 64),
                                          (5, 5, 48, 16), (32, 1, 16, 16), (2, 1, 128, 32),
                                          (3, 1, 80, 7), (1, 1, 256, 16)])
def test_attention_mixed_batches(dtype, H, Hkv, D, P):
    seqs = [(0, 1), (17, 3), (0, 40), (40, 100), (333, 1), (5, 2)]
    got, want = attention_case(dtype, H, Hkv, D, P, seqs)
    close(got, want, dtype, f"attention H{H} Hkv{Hkv} D{D} P{P}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 33])
def test_attention_window(dtype, window):
    got, want = attention_case(dtype, 6, 2, 32, 8, [(0, 50), (70, 1), (20, 30), (3, 2)], window=window)
    close(got, want, dtype, f"window {window}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_far_key_and_window_edge(dtype):
    """One key's score dominates: far back among hundreds (it must be found on its page), just
    inside the window (it must be seen) and just outside (it must not)."""
    D, ctx = 32, 700

    def far(s, q, k, v):
        q[:] = 0.0
        k[:] = 0.0
        q[:, :, 0] = 8.0
        k[13, :, 0] = 8.0          # position 13 of 701: score 64 * D^-0.5 above all others

    got, want = attention_case(dtype, 4, 2, D, 16, [(ctx, 1)], boost=far)
    close(got, want, dtype, "far key")
    assert (got.double().cpu() - want).abs().max().item() < 0.05

    for offset, seen in ((9, True), (10, False)):
        def edge(s, q, k, v, offset=offset):
            q[:] = 0.0
            k[:] = 0.0
            q[:, :, 0] = 8.0
            k[ctx - offset, :, 0] = 8.0
            v[ctx - offset] = 5.0

        got, want = attention_case(dtype, 4, 2, D, 16, [(ctx, 1)], window=10, boost=edge)
        close(got, want, dtype, f"window edge {offset}")
        assert (got.double().cpu().mean().item() > 2.0) == seen


def test_attention_poison_is_a_real_control():
    """If the kernel read a row it must not, the NaN would surface: reading one position too
    many (a table that claims one more token) does surface it."""
    from tokenomos_b200 import ops
    D, P = 16, 8
    pool = torch.full((3, 2, 1, P, D), float("nan"), device="cuda")
    pool[1, :, :, :5] = 1.0
    q = torch.ones(1, 1, D, device="cuda")
    table = i32([[1]])
    ok = ops.attention(q, pool, i32([4]), i32([0]), table, i32([0]), i32([1]), 16, None, 1.0)
    assert torch.isfinite(ok).all()
    bad = ops.attention(q, pool, i32([5]), i32([0]), table, i32([0]), i32([1]), 16, None, 1.0)
    assert torch.isnan(bad).any()


# ---- gated short conv --------------------------------------------------------------------------

def conv_ref(bcx, taps, bias, prev):
    """One whole sequence: bcx [T, 3d] float64, prev [W-1, d] the inputs before it."""
    T, d = bcx.shape[0], bcx.shape[1] // 3
    W = taps.shape[1]
    u = bcx[:, :d] * bcx[:, 2 * d:]
    padded = torch.cat((prev, u))
    y = sum(padded[j:j + T] * taps[:, j][None] for j in range(W))
    if bias is not None:
        y = y + bias
    return bcx[:, d:2 * d] * y, padded[-(W - 1):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tile", [32, 16, 7])
@pytest.mark.parametrize("W, d, with_bias", [(2, 100, True), (3, 64, False), (4, 96, True), (7, 300, False),
                                             (8, 2048, True), (3, 136, False)])
def test_conv_gated_mixed_batch_and_state(dtype, W, d, with_bias, tile):
    """Tiles of 32 tokens take the kernel that walks a tile's tokens in order; tiles of at most 16
    (given as ``tile_cap``) the tiled kernel: one thread per token and 16 bytes of channels, inputs
    through shared memory. Channel counts that are and are not whole 16-byte chunks."""
    from tokenomos_b200 import ops
    slots = 6
    taps = torch.randn(d, W)
    bias = torch.randn(d) if with_bias else None
    # (slot, ctx, n): fresh sequences, continued ones, single tokens, one shorter than W - 1
    seqs = [(3, 0, 1), (1, 12, 70), (5, 0, 33), (2, 4, 1), (4, 9, 2)]
    state0 = torch.randn(slots, W - 1, d).to(dtype)
    state = dev(state0).clone()
    T = sum(n for _, _, n in seqs)
    bcx = torch.randn(T, 3 * d).to(dtype)
    cu = [0]
    for _, _, n in seqs:
        cu.append(cu[-1] + n)
    tseq, toff, tn, ttok0 = [], [], [], []
    for s, (_, _, n) in enumerate(seqs):
        for o in range(0, n, tile):
            tseq.append(s), toff.append(o), tn.append(min(tile, n - o)), ttok0.append(cu[s] + o)
    # (each tile's first token in the batch is optional: given for the tile of 16, left out for 7)
    out = ops.conv_gated(dev(bcx), dev(taps), dev(bias) if with_bias else None, state, i32(cu),
                         i32([c for _, c, _ in seqs]), i32([s for s, _, _ in seqs]),
                         i32(tseq), i32(toff), i32(tn), 0, tile if tile <= 16 else 0,
                         i32(ttok0) if tile == 16 else None)
    new_state = state.cpu()
    touched = set()
    for s, (slot, ctx, n) in enumerate(seqs):
        prev = state0[slot].double().clone()
        for k in range(W - 1):                      # inputs before position 0 are zero
            if ctx - (W - 1) + k < 0:
                prev[k] = 0.0
        want, want_state = conv_ref(bcx[cu[s]:cu[s + 1]].double(), taps.double(),
                                    bias.double() if with_bias else None, prev)
        close(out[cu[s]:cu[s + 1]], want, dtype, f"conv out of sequence {s}")
        close(new_state[slot], want_state, dtype, f"conv state of sequence {s}",
              scale=max(want_state.abs().max().item(), 1.0))
        touched.add(slot)
    for slot in range(slots):
        if slot not in touched:
            assert torch.equal(new_state[slot], state0[slot])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tile", [32, 16, 5])
def test_conv_gated_cut_anywhere_equals_whole(dtype, tile):
    """A sequence fed in portions (down to one token) through its state row gives what the whole
    sequence gives: bit for bit, since every output sums the same values in the same order; in
    both forms of the kernel (tiles of 32: the walking one; up to 16: the tiled one)."""
    from tokenomos_b200 import ops
    W, d, T = 4, 72, 57
    taps, bcx = torch.randn(d, W), torch.randn(T, 3 * d).to(dtype)

    def run(cuts):
        state = torch.full((2, W - 1, d), float("nan"), dtype=dtype, device="cuda")
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            n = b - a
            tiles = [(0, o, min(tile, n - o)) for o in range(0, n, tile)]
            outs.append(ops.conv_gated(dev(bcx[a:b]), dev(taps), None, state, i32([0, n]), i32([a]),
                                       i32([1]), i32([t[0] for t in tiles]), i32([t[1] for t in tiles]),
                                       i32([t[2] for t in tiles]), 0, tile if tile <= 16 else 0))
        return torch.cat(outs)

    whole = run([0, T])
    assert torch.isfinite(whole).all()
    for cuts in ([0, 1, 2, 3, 4, 5, T], [0, 2, 33, 34, 36, T], list(range(T + 1))):
        assert torch.equal(run(cuts), whole), cuts


def test_conv_gated_blocked_columns_equal_plain_columns():
    """Rows of bcx in runs of 8 channels of B, of C and of X in turn (what the in-projection with
    interleaved rows produces) give what the plain [B | C | X] rows give, bit for bit, state too."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.shortconv import interleave_bcx
    for dtype in DTYPES:
        W, d, slots = 3, 40, 4
        taps, bias = torch.randn(d, W), torch.randn(d)
        seqs = [(2, 0, 19), (1, 7, 1), (3, 3, 33)]
        T = sum(n for _, _, n in seqs)
        bcx = torch.randn(T, 3 * d).to(dtype)
        blocked = interleave_bcx(bcx.t().contiguous(), 8).t().contiguous()
        cu = [0]
        for _, _, n in seqs:
            cu.append(cu[-1] + n)
        tiles = [(s, o, min(8, n - o)) for s, (_, _, n) in enumerate(seqs) for o in range(0, n, 8)]
        state0 = torch.randn(slots, W - 1, d).to(dtype)
        outs, states = [], []
        for rows, block, cap in ((bcx, 0, 0), (blocked, 8, 0), (bcx, 0, 8), (blocked, 8, 8)):
            state = dev(state0).clone()
            outs.append(ops.conv_gated(dev(rows), dev(taps), dev(bias), state, i32(cu),
                                       i32([c for _, c, _ in seqs]), i32([s for s, _, _ in seqs]),
                                       i32([t[0] for t in tiles]), i32([t[1] for t in tiles]),
                                       i32([t[2] for t in tiles]), block, cap))
            states.append(state)
        assert all(torch.equal(o, outs[0]) for o in outs) and all(torch.equal(st, states[0]) for st in states)


@pytest.mark.parametrize("W, tile", [(3, 16), (4, 16), (8, 16), (3, 8), (2, 4)])
def test_conv_gated_many_tiles_per_block_equal_the_walking_kernel(W, tile):
    """Enough tiles that a block of the tiled kernel takes several in a row through its staging
    pipeline (more than it has stages), in both row layouts, with portions that start at a cached
    position, at position 0 and one shorter than the state: outputs and states are the walking
    kernel's, bit for bit."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.shortconv import interleave_bcx
    dtype, d, slots = torch.bfloat16, 1000, 6
    taps, bias = torch.randn(d, W), torch.randn(d)
    seqs = [(2, 0, 1500), (1, 7, 1), (3, 3, 2500), (4, 5, 37), (5, 0, max(1, W - 2))]
    T = sum(n for _, _, n in seqs)
    bcx = torch.randn(T, 3 * d).to(dtype)
    blocked = interleave_bcx(bcx.t().contiguous(), 8).t().contiguous()
    cu = [0]
    for _, _, n in seqs:
        cu.append(cu[-1] + n)
    tiles = [(s_, o, min(tile, n - o)) for s_, (_, _, n) in enumerate(seqs) for o in range(0, n, tile)]
    tok0 = [cu[s_] + o for s_, o, _ in tiles]
    state0 = torch.randn(slots, W - 1, d).to(dtype)
    outs, states = [], []
    for rows, block, cap, first in ((bcx, 0, 0, None), (bcx, 0, tile, None), (blocked, 8, tile, None),
                                    (blocked, 8, tile, i32(tok0))):
        state = dev(state0).clone()
        outs.append(ops.conv_gated(dev(rows), dev(taps), dev(bias), state, i32(cu),
                                   i32([c for _, c, _ in seqs]), i32([s_ for s_, _, _ in seqs]),
                                   i32([t[0] for t in tiles]), i32([t[1] for t in tiles]),
                                   i32([t[2] for t in tiles]), block, cap, first))
        states.append(state)
    assert all(torch.equal(o, outs[0]) for o in outs[1:])
    assert all(torch.equal(st, states[0]) for st in states[1:])


@pytest.mark.parametrize("W, d, K, M, with_bias", [(3, 64, 128, 8, False), (2, 40, 72, 5, True),
                                                  (4, 96, 520, 13, True), (8, 24, 64, 1, False),
                                                  (3, 2048, 2048, 8, False)])
def test_gemm_skinny_conv_equals_projection_then_conv(W, d, K, M, with_bias):
    """The decode kernel that runs the gated short conv in the epilogue of its in-projection
    (rows of the weight in blocks of 24) against the two kernels it replaces: the projection with
    plain rows, then the conv with one token per sequence. Requests at positions 0, 1 and beyond
    (the state row reads as zeros before position 0); state rows of other slots stay."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.shortconv import interleave_bcx
    dtype = torch.bfloat16
    slots = M + 3
    w = (torch.randn(3 * d, K) * K ** -0.5).to(dtype)
    b_in = torch.randn(3 * d) if with_bias else None
    taps = torch.randn(d, W)
    conv_bias = torch.randn(d) if with_bias else None
    x = torch.randn(M, K).to(dtype)
    ctx = [(0, 1, 2, 5, 40, 3, 0, 9, 1, 2, 100, 7, 6)[i % 13] for i in range(M)]
    slot = torch.randperm(slots)[:M].tolist()
    state0 = torch.randn(slots, W - 1, d).to(dtype)
    # the unfused path
    s1 = dev(state0).clone()
    bcx = ops.gemm_skinny(dev(x), dev(w), dev(b_in) if with_bias else None)
    want = ops.conv_gated(bcx, dev(taps), dev(conv_bias) if with_bias else None, s1, i32(list(range(M + 1))),
                          i32(ctx), i32(slot), i32(list(range(M))), i32([0] * M), i32([1] * M))
    # the fused kernel
    s2 = dev(state0).clone()
    got = ops.gemm_skinny_conv(dev(x), dev(interleave_bcx(w, 8)),
                               dev(interleave_bcx(b_in, 8)) if with_bias else None, dev(taps),
                               dev(conv_bias) if with_bias else None, s2, i32(ctx), i32(slot))
    assert torch.equal(got, want), (got.float() - want.float()).abs().max().item()
    assert torch.equal(s1, s2)
    untouched = [i for i in range(slots) if i not in slot]
    assert torch.equal(s2[untouched].cpu(), state0[untouched])
    # and against 64-bit arithmetic
    bcx64 = x.double() @ w.double().t() + (b_in.double() if with_bias else 0.0)
    for i in range(M):
        prev = state0[slot[i]].double().clone()
        for k in range(W - 1):
            if ctx[i] - (W - 1) + k < 0:
                prev[k] = 0.0
        ref, _ = conv_ref(bcx64[i:i + 1], taps.double(), conv_bias.double() if with_bias else None, prev)
        close(got[i:i + 1], ref, dtype, f"fused conv token {i}", scale=max(ref.abs().max().item(), 1.0))


# ---- sampling ----------------------------------------------------------------------------------

def sample_rows(logits, rows):
    from tokenomos_b200 import ops
    n = len(rows)
    f = lambda i: torch.tensor([r[i] for r in rows], dtype=torch.float32, device="cuda")  # noqa: E731
    k = lambda i: torch.tensor([r[i] for r in rows], dtype=torch.int32, device="cuda")    # noqa: E731
    assert logits.shape[0] == n
    return ops.sample(logits, f(0), f(1), k(2), f(3), k(4), k(5)).cpu()


def test_sample_greedy_is_the_first_maximum():
    V = 1000
    logits = torch.randn(5, V)
    logits[0, [400, 17, 900]] = 9.0
    logits[1, V - 1] = 9.0
    logits[2, 0] = 9.0
    got = sample_rows(logits.cuda(), [(0.0, 1.0, 0, 0.0, 0, 0)] * 5)
    assert got.tolist() == [17, V - 1, 0, int(logits[3].argmax()), int(logits[4].argmax())]


def test_sample_row_without_a_finite_logit_gives_a_valid_token_and_is_reported():
    """A row of NaN (or of -inf) has no best token. The sampler must not hand out the sentinel it
    starts from (2**31 - 1, which the next step's embedding lookup would clamp silently): it
    answers token 0, greedy or sampled, and leaves 1 + the row in a word the host reads."""
    from tokenomos_b200 import ops
    V = 300
    ops.sample_status()
    logits = torch.randn(4, V)
    logits[1] = float("nan")
    logits[3] = float("-inf")
    got = sample_rows(logits.cuda(), [(0.0, 1.0, 0, 0.0, 0, 0), (0.0, 1.0, 0, 0.0, 0, 0),
                                      (0.9, 0.8, 5, 0.0, 3, 1), (0.9, 0.8, 5, 0.0, 3, 1)])
    assert got[0] == int(logits[0].argmax()) and got[1] == 0 and got[3] == 0 and 0 <= got[2] < V
    assert ops.sample_status() in (2, 4)       # 1 + one of the two bad rows (the first to report)
    assert ops.sample_status() == 0            # reading resets it
    sample_rows(torch.randn(2, V).cuda(), [(0.0, 1.0, 0, 0.0, 0, 0)] * 2)
    assert ops.sample_status() == 0


@pytest.mark.parametrize("params", [(0.8, 1.0, 0, 0.0), (1.3, 1.0, 7, 0.0), (1.0, 0.6, 0, 0.0),
                                    (1.0, 1.0, 0, 0.15), (0.7, 0.8, 12, 0.02)])
def test_sample_distribution(params):
    """Empirical distribution over many seeds against the float64 restricted softmax."""
    temp, top_p, top_k, min_p = params
    V, N = 50, 40000
    g = torch.Generator().manual_seed(3)
    row = torch.randn(V, generator=g) * 2
    x = row.double() / temp
    keep = torch.ones(V, dtype=torch.bool)
    if min_p > 0:
        keep &= x >= x.max() + math.log(min_p)
    if top_k:
        kth = torch.sort(x[keep], descending=True).values[min(top_k, int(keep.sum())) - 1]
        keep &= x >= kth
    if top_p < 1:
        p = torch.where(keep, (x - x.max()).exp(), torch.zeros_like(x))
        order = torch.argsort(p, descending=True)
        csum = torch.cumsum(p[order], 0) / p.sum()
        cut = int((csum < top_p).sum()) + 1
        mask = torch.zeros(V, dtype=torch.bool)
        mask[order[:cut]] = True
        keep &= mask
    want = torch.where(keep, (x - x.max()).exp(), torch.zeros_like(x))
    want /= want.sum()
    logits = row[None].repeat(N, 1).cuda()
    got = sample_rows(logits, [(temp, top_p, top_k, min_p, seed, 0) for seed in range(N)])
    freq = torch.bincount(got, minlength=V).double() / N
    assert freq[~keep].sum().item() == 0.0, "a token outside the allowed set was drawn"
    assert 0.5 * (freq - want).abs().sum().item() < 0.02


def test_sample_is_batch_invariant_and_step_dependent():
    V = 777
    logits = torch.randn(6, V).cuda()
    rows = [(0.9, 0.95, 40, 0.0, 11 * i, 3) for i in range(6)]
    together = sample_rows(logits, rows)
    alone = [sample_rows(logits[i:i + 1], rows[i:i + 1])[0] for i in range(6)]
    assert together.tolist() == [int(a) for a in alone]
    shuffled = sample_rows(logits.flip(0), rows[::-1])
    assert shuffled.tolist() == together.flip(0).tolist()
    steps = [sample_rows(logits[:1].repeat(64, 1), [(1.5, 1.0, 0, 0.0, 5, s) for s in range(64)])]
    assert len(set(steps[0].tolist())) > 8


# ---- tensor-core attention (bfloat16, head sizes 64 and 128) -------------------------------------

def attention_mma_case(H, Hkv, D, P, seqs, window=None, boost=None, nsplit=None, tc=False, gate=None,
                       tc_split=1):
    """Like ``attention_case`` but through the tensor-core kernels: multi-token sequences go to
    the prefill kernel (``tc``: the tcgen05 one), single-token ones to the decode kernel (split
    ``nsplit`` ways). ``gate`` [T, H] (on the device): the kernels apply the per-head output gate
    as they write (the reference returned stays ungated). ``tc_split``: CTAs that share a tile's
    keys in the tcgen05 prefill kernel."""
    from tokenomos_b200 import ops
    dtype = torch.bfloat16
    assert ops.attention_mma_supported(H, Hkv, D, dtype)
    G = H // Hkv
    total = [c + n for c, n in seqs]
    blocks = [-(-t // P) for t in total]
    width = max(blocks)
    pages = sum(blocks) + 1
    perm = (torch.randperm(pages - 1) + 1).tolist()
    pool = torch.full((pages, 2, Hkv, P, D), float("nan"), dtype=torch.float64)
    table = torch.zeros(len(seqs), width, dtype=torch.int32)
    ks, vs, qs = [], [], []
    for s, (c, n) in enumerate(seqs):
        k = torch.randn(total[s], Hkv, D).to(dtype).double()
        v = torch.randn(total[s], Hkv, D).to(dtype).double()
        q = torch.randn(n, H, D).to(dtype).double()
        if boost is not None:
            boost(s, q, k, v)
        for b in range(blocks[s]):
            page = perm.pop()
            table[s, b] = page
            rows = min(P, total[s] - b * P)
            pool[page, 0, :, :rows] = k[b * P:b * P + rows].transpose(0, 1)
            pool[page, 1, :, :rows] = v[b * P:b * P + rows].transpose(0, 1)
        ks.append(k), vs.append(v), qs.append(q)
    positions = [p for (c, n) in seqs for p in range(c, c + n)]
    tok_seq = [s for s, (c, n) in enumerate(seqs) for _ in range(n)]
    per_tile = ops.attention_prefill_tc_tokens(H, Hkv) if tc else ops.attention_prefill_mma_tokens(H, Hkv)
    tok0, ntok, singles, start = [], [], [], 0
    for c, n in seqs:
        if n == 1:
            singles.append(start)
        else:
            for o in range(0, n, per_tile):
                tok0.append(start + o)
                ntok.append(min(per_tile, n - o))
        start += n
    q_dev, pool_dev = dev(torch.cat(qs), dtype), dev(pool, dtype)
    out = torch.full_like(q_dev, float("nan"))
    if tok0:
        prefill = ops.attention_prefill_tc if tc else ops.attention_prefill_mma
        prefill(q_dev, pool_dev, out, i32(positions), i32(tok_seq), dev(table), i32(tok0), i32(ntok),
                window, D ** -0.5, gate, **({"nsplit": tc_split} if tc else {}))
        if tc:
            assert ops.attention_prefill_tc_status() == 0
    if singles:
        ops.attention_decode_mma(q_dev, pool_dev, out, i32(positions), i32(tok_seq), dev(table),
                                 i32(singles), window, D ** -0.5, nsplit or 1, gate)
    want = []
    for s, (c, n) in enumerate(seqs):
        k = ks[s].repeat_interleave(G, 1)
        v = vs[s].repeat_interleave(G, 1)
        sc = torch.einsum("ihd,jhd->hij", qs[s], k) * D ** -0.5
        i = torch.arange(c, c + n)[:, None]
        j = torch.arange(total[s])[None, :]
        vis = j <= i
        if window:
            vis &= (i - j) < window
        sc = sc.masked_fill(~vis[None], float("-inf"))
        want.append(torch.einsum("hij,jhd->ihd", sc.softmax(-1), v))
    return out, torch.cat(want)


@pytest.mark.parametrize("H, Hkv, D, P", [(32, 8, 64, 16), (8, 8, 64, 64), (4, 2, 128, 32), (16, 1, 64, 8),
                                          (6, 3, 64, 7), (8, 1, 128, 16)])
@pytest.mark.parametrize("nsplit", [1, 3, 16])
def test_attention_mma_mixed_batches(H, Hkv, D, P, nsplit):
    seqs = [(0, 1), (17, 3), (0, 40), (40, 100), (333, 1), (5, 2), (64, 64), (1000, 1), (0, 130)]
    got, want = attention_mma_case(H, Hkv, D, P, seqs, nsplit=nsplit)
    close(got, want, torch.bfloat16, f"mma attention H{H} Hkv{Hkv} D{D} P{P} split {nsplit}")


def decode_fused_case(H, Hkv, D, P, angles, window, nsplit, gated, normed, ctxs, write_kv=True):
    """One decode step's attention for sequences holding ``ctxs`` positions, through the one-kernel
    form and through the chain it replaces (norm + rotation + cache write, split attention + merge,
    gate), on two copies of the same NaN-poisoned cache, and in float64 from the same inputs."""
    from tokenomos_b200 import ops
    dtype, eps = torch.bfloat16, 1e-5
    G, n = H // Hkv, len(ctxs)
    own = Hkv if write_kv else 0
    blocks = [-(-(c + 1) // P) for c in ctxs]
    pages = sum(blocks) + 1
    perm = (torch.randperm(pages - 1) + 1).tolist()
    pool = torch.full((pages, 2, Hkv, P, D), float("nan"), dtype=torch.float64)
    table = torch.zeros(n, max(blocks), dtype=torch.int32)
    ks, vs = [], []
    for s_, c in enumerate(ctxs):
        held = c + (0 if write_kv else 1)           # without keys of its own the cache holds this step's already
        k = torch.randn(held, Hkv, D).to(dtype).double()
        v = torch.randn(held, Hkv, D).to(dtype).double()
        for b in range(blocks[s_]):
            page = perm.pop()
            table[s_, b] = page
            rows = max(0, min(P, held - b * P))
            pool[page, 0, :, :rows] = k[b * P:b * P + rows].transpose(0, 1)
            pool[page, 1, :, :rows] = v[b * P:b * P + rows].transpose(0, 1)
        ks.append(k), vs.append(v)
    width = (H + 2 * own) * D
    pad = -(-H // 8) * 8 if gated else 0
    proj = (torch.randn(n, width + pad) * 1.5).to(dtype)
    wq = (1 + 0.3 * torch.randn(D)) if normed else None
    wk = (1 + 0.3 * torch.randn(D)) if normed else None
    inv = 1.0 / (10000.0 ** (torch.arange(0, 2 * angles, 2, dtype=torch.float32) / (2 * angles)))
    rot = 2 * angles
    positions, tok_seq = i32(ctxs), i32(list(range(n)))
    proj_d, table_d, inv_d = dev(proj), dev(table), dev(inv)
    wq_d, wk_d = (dev(wq), dev(wk)) if normed else (None, None)
    gate = proj_d[:, width:width + H] if gated else None
    scale = D ** -0.5

    pool_a = dev(pool, dtype)
    got = ops.attention_decode_fused(proj_d, pool_a, wq_d, wk_d if own else None, eps, inv_d, gate, positions,
                                     tok_seq, table_d, H, Hkv, window, scale, nsplit, write_kv=write_kv)
    pool_b = dev(pool, dtype)
    q = ops.qk_norm_rope_write(proj_d[:, :width], pool_b if own else None, wq_d, wk_d if own else None, eps,
                               inv_d, positions, tok_seq, table_d if own else None, H, own, D, P)
    chain = torch.empty_like(q)
    ops.attention_decode_mma(q, pool_b, chain, positions, tok_seq, table_d, None, window, scale, nsplit)
    if gated:
        ops.head_gate(chain, gate, H, D)

    x = proj.double()[:, :width].view(n, H + 2 * own, D)

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.double() if w is not None else v

    pos = torch.tensor(ctxs)
    inv_full = torch.cat((inv, torch.zeros(0)))
    want_q = rope_ref(norm(x[:, :H], wq), pos, inv_full, rot)
    want = []
    for s_, c in enumerate(ctxs):
        k, v = ks[s_], vs[s_]
        if write_kv:
            k = torch.cat((k, rope_ref(norm(x[s_:s_ + 1, H:H + Hkv], wk), pos[s_:s_ + 1], inv_full, rot)
                           .to(dtype).double()))
            v = torch.cat((v, x[s_:s_ + 1, H + Hkv:]))
        k, v = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
        sc = torch.einsum("hd,jhd->hj", want_q[s_].to(dtype).double(), k) * scale
        j = torch.arange(c + 1)
        vis = j <= c
        if window:
            vis &= (c - j) < window
        sc = sc.masked_fill(~vis[None], float("-inf"))
        o = torch.einsum("hj,jhd->hd", sc.softmax(-1), v)
        if gated:
            o = o * torch.sigmoid(proj.double()[s_, width:width + H])[:, None]
        want.append(o)
    tickets = ops._tickets.get(got.device)
    return got, chain, torch.stack(want), pool_a, pool_b, tickets


@pytest.mark.parametrize("H, Hkv, D, P, angles", [(32, 8, 64, 16, 32), (8, 8, 64, 64, 16), (4, 2, 128, 32, 64),
                                                  (16, 1, 64, 8, 32), (6, 3, 64, 7, 8), (8, 1, 128, 16, 24),
                                                  (2, 2, 64, 16, 0)])
@pytest.mark.parametrize("nsplit, window, gated, normed", [(1, None, True, True), (3, None, True, True),
                                                           (16, None, False, True), (5, 40, True, False),
                                                           (2, 1, False, False)])
def test_attention_decode_fused_equals_the_chain_it_replaces(H, Hkv, D, P, angles, nsplit, window, gated, normed):
    ctxs = [0, 1, 31, 32, 33, 100, 1000, 333, 64, 95]
    got, chain, want, pool_a, pool_b, tickets = decode_fused_case(H, Hkv, D, P, angles, window, nsplit, gated,
                                                                   normed, ctxs)
    what = f"fused decode attention H{H} Hkv{Hkv} D{D} P{P} R{2 * angles} split {nsplit} window {window}"
    close(got, want, torch.bfloat16, what)
    # the same bits as norm + rotation + write, split attention + merge, gate: outputs and cache
    assert torch.equal(got.view(torch.int16), chain.view(torch.int16)), what
    assert torch.equal(pool_a.view(torch.int16), pool_b.view(torch.int16)), what + ": cache"
    assert tickets is None or int(tickets.abs().sum()) == 0, "tickets are zero again"


def test_attention_decode_fused_without_keys_of_its_own_and_twice_in_a_row():
    """A layer that reads another layer's cache (queries only, nothing written), and the same
    launch repeated: the tickets of the first leave the second alone."""
    ctxs = [5, 700, 31, 32]
    for _ in range(2):
        got, chain, want, pool_a, pool_b, tickets = decode_fused_case(8, 2, 64, 16, 32, None, 4, False, True, ctxs,
                                                                       write_kv=False)
        close(got, want, torch.bfloat16, "fused decode attention over a shared cache")
        assert torch.equal(got.view(torch.int16), chain.view(torch.int16))
        assert torch.equal(pool_a.view(torch.int16), pool_b.view(torch.int16))
        assert int(tickets.abs().sum()) == 0


def test_attention_decode_fused_refuses_what_it_cannot_take():
    from tokenomos_b200 import ops
    assert not ops.attention_decode_fused_supported(8, 2, 48, 32, torch.bfloat16)      # head size
    assert not ops.attention_decode_fused_supported(8, 2, 64, 24, torch.bfloat16)      # rotary halves of 12
    assert not ops.attention_decode_fused_supported(8, 2, 64, 64, torch.float32)
    assert ops.attention_decode_fused_supported(8, 2, 64, 0, torch.bfloat16)
    pool = torch.zeros(4, 2, 2, 16, 48, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="not taken"):
        ops.attention_decode_fused(torch.zeros(1, 12 * 48, dtype=torch.bfloat16, device="cuda"), pool, None, None,
                                   1e-5, torch.ones(16, device="cuda"), None, i32([0]), i32([0]),
                                   torch.ones(1, 1, dtype=torch.int32, device="cuda"), 8, 2, None, 0.1, 1)


@pytest.mark.parametrize("tc, H, Hkv, D, nsplit", [(True, 32, 8, 64, 1), (False, 32, 8, 64, 5), (False, 4, 2, 128, 2),
                                                   (True, 6, 3, 64, 3)])
def test_attention_gate_in_the_epilogue_equals_the_gate_kernel(tc, H, Hkv, D, nsplit):
    """The per-head output gate applied by the attention kernels as they write gives the bits that
    the same kernels followed by the gate kernel give (one seed, two runs)."""
    from tokenomos_b200 import ops
    seqs = [(0, 1), (17, 3), (0, 40), (40, 100), (333, 1), (5, 2), (64, 64), (1000, 1), (0, 130)]
    T = sum(n for _, n in seqs)
    wide = torch.randn(T, H + 11, device="cuda").to(torch.bfloat16)
    gate = wide[:, 3:3 + H]                                  # a strided view, as the fused projection gives
    torch.manual_seed(7)
    plain, want = attention_mma_case(H, Hkv, D, 16, seqs, nsplit=nsplit, tc=tc)
    torch.manual_seed(7)
    gated, _ = attention_mma_case(H, Hkv, D, 16, seqs, nsplit=nsplit, tc=tc, gate=gate)
    ops.head_gate(plain, gate, H, D)
    assert torch.equal(plain.view(torch.int16), gated.view(torch.int16))
    close(gated, want * torch.sigmoid(gate.double().cpu())[:, :, None], torch.bfloat16, "gated attention")


@pytest.mark.parametrize("H, Hkv, P", [(32, 8, 16), (8, 8, 64), (16, 1, 8), (6, 3, 7), (4, 4, 32)])
def test_attention_tc_prefill(H, Hkv, P):
    """The tcgen05 prefill kernel (head size 64): portions of every length beside cached
    positions, tiles that are not full, groups of 1, 2, 4 and 16, a page size that is no power of
    two."""
    from tokenomos_b200 import ops
    assert ops.attention_prefill_tc_supported(H, Hkv, 64, torch.bfloat16)
    assert not ops.attention_prefill_tc_supported(H, Hkv, 128, torch.bfloat16)
    seqs = [(17, 3), (0, 40), (40, 100), (5, 2), (64, 64), (0, 130), (300, 257), (1, 63), (0, 2)]
    got, want = attention_mma_case(H, Hkv, 64, P, seqs, tc=True)
    close(got, want, torch.bfloat16, f"tc attention H{H} Hkv{Hkv} P{P}")


@pytest.mark.parametrize("H, Hkv, P", [(32, 8, 16), (6, 3, 7), (4, 4, 32)])
@pytest.mark.parametrize("split, window", [(2, None), (3, None), (8, None), (4, 70), (5, 1)])
def test_attention_tc_prefill_with_a_tiles_keys_shared_by_several_ctas(H, Hkv, P, split, window):
    """Portions behind long and short contexts with each tile's keys split over CTAs: sequences with
    fewer key tiles than splits (some CTAs have nothing), a window, a gate; twice in a row (the
    tickets of the first launch leave the second alone)."""
    from tokenomos_b200 import ops
    seqs = [(0, 40), (1900, 130), (17, 3), (333, 64), (0, 2), (700, 33), (64, 64), (5000, 70), (2600, 40)]
    T = sum(n for _, n in seqs)
    gate = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        got, want = attention_mma_case(H, Hkv, 64, P, seqs, window=window, tc=True, gate=gate, tc_split=split)
        close(got, want * torch.sigmoid(gate.double().cpu())[:, :, None], torch.bfloat16,
              f"tcgen05 prefill H{H} Hkv{Hkv} P{P} split {split} window {window}")
        assert ops.attention_prefill_tc_status() == 0
        assert int(ops._tickets[got.device].abs().sum()) == 0


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_tc_prefill_window_and_far_key(window):
    seqs = [(0, 150), (20, 30), (3, 2), (200, 70)]
    got, want = attention_mma_case(8, 2, 64, 16, seqs, window=window, tc=True)
    close(got, want, torch.bfloat16, f"tc window {window}")

    def far(s, q, k, v):
        q[:] = 0.0
        k[:] = 0.0
        q[:, :, 0] = 8.0
        k[13, :, 0] = 8.0

    got, want = attention_mma_case(8, 2, 64, 16, [(670, 31), (0, 700)], boost=far, tc=True)
    close(got, want, torch.bfloat16, "tc far key")
    assert (got.double().cpu() - want).abs().max().item() < 0.05


@pytest.mark.parametrize("shape", ["rising", "falling", "leap"])
def test_attention_tc_prefill_moving_maxima(shape):
    """The tcgen05 kernel rescales its accumulated output only when a score exceeds its reference
    maximum by 2^8. Scores that climb a few units per key tile (probabilities above 1 for a while,
    then a rescale every other tile), scores that fall from the first key on, and one late score
    far above all before it go through both branches."""
    def boost(s, q, k, v):
        n = k.shape[0]
        ramp = torch.arange(n, dtype=torch.float64)
        q[:, :, 0] = 8.0
        if shape == "rising":
            k[:, :, 0] = (ramp * 0.05)[:, None]
        elif shape == "falling":
            k[:, :, 0] = ((n - ramp) * 0.05)[:, None]
        else:
            k[:, :, 0] = 0.0
            k[n // 2 + 37, :, 0] = 60.0
        k[:] = k.to(torch.bfloat16).double()

    seqs = [(0, 700), (300, 257), (650, 31)]
    got, want = attention_mma_case(8, 2, 64, 16, seqs, boost=boost, tc=True)
    close(got, want, torch.bfloat16, f"tc moving maxima {shape}")


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_mma_window(window):
    seqs = [(0, 150), (70, 1), (20, 30), (3, 2), (500, 1), (63, 1)]
    got, want = attention_mma_case(8, 2, 64, 16, seqs, window=window, nsplit=2)
    close(got, want, torch.bfloat16, f"mma window {window}")


def test_attention_mma_far_key_and_window_edge():
    D, ctx = 64, 700

    def far(s, q, k, v):
        q[:] = 0.0
        k[:] = 0.0
        q[:, :, 0] = 8.0
        k[13, :, 0] = 8.0

    for seqs, nsplit in (([(ctx, 1)], 1), ([(ctx, 1)], 5), ([(ctx - 30, 31)], 1)):
        got, want = attention_mma_case(8, 2, D, 16, seqs, boost=far, nsplit=nsplit)
        close(got, want, torch.bfloat16, "far key")
        assert (got.double().cpu() - want).abs().max().item() < 0.05
    for offset, seen in ((9, True), (10, False)):
        def edge(s, q, k, v, offset=offset):
            q[:] = 0.0
            k[:] = 0.0
            q[:, :, 0] = 8.0
            k[ctx - offset, :, 0] = 8.0
            v[ctx - offset] = 5.0

        for nsplit in (1, 4):
            got, want = attention_mma_case(8, 2, D, 16, [(ctx, 1)], window=10, boost=edge, nsplit=nsplit)
            close(got, want, torch.bfloat16, f"window edge {offset}")
            assert (got.double().cpu().mean().item() > 2.0) == seen


def test_attention_mma_refuses_other_shapes():
    from tokenomos_b200 import ops
    assert not ops.attention_mma_supported(4, 1, 24, torch.bfloat16)
    assert not ops.attention_mma_supported(6, 2, 64, torch.bfloat16)      # group of 3
    assert not ops.attention_mma_supported(32, 8, 64, torch.float32)
    q = torch.zeros(1, 4, 24, dtype=torch.bfloat16, device="cuda")
    pool = torch.zeros(2, 2, 1, 8, 24, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="is not taken"):
        ops.attention_decode_mma(q, pool, q.clone(), i32([0]), i32([0]), i32([[1]]), i32([0]), None, 1.0, 1)


# ---- skinny matrix product (decode) ---------------------------------------------------------------

@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n, k", [(16, 64), (100, 200), (2056, 2048), (300, 8192), (1000, 96), (6144, 2048), (20000, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_skinny(m, n, k, out_dtype):
    from tokenomos_b200 import ops
    x = torch.randn(m, k).to(torch.bfloat16)
    w = torch.randn(n, k).to(torch.bfloat16)
    b = torch.randn(n)
    assert ops.gemm_skinny_ok(dev(x), dev(w))
    got = ops.gemm_skinny(dev(x), dev(w), dev(b), out_dtype)
    close(got, x.double() @ w.double().T + b.double(), out_dtype, f"skinny {m}x{n}x{k}")
    # a row-strided view of a wider activation, no bias
    wide = torch.randn(m, k + 24).to(torch.bfloat16)
    view = dev(wide)[:, 8:8 + k]
    assert ops.gemm_skinny_ok(view, dev(w))
    got = ops.gemm_skinny(view, dev(w), None, out_dtype)
    close(got, wide[:, 8:8 + k].double() @ w.double().T, out_dtype, "skinny strided")


def test_gemm_skinny_refuses_what_it_cannot_take():
    from tokenomos_b200 import ops
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_skinny_ok(x, w)
    assert not ops.gemm_skinny_ok(x[:4, :60], w[:, :60])
    with pytest.raises(ops.KernelError, match="at most 16"):
        ops.gemm_skinny(x, w)


@pytest.mark.parametrize("m", [1, 8, 13])
@pytest.mark.parametrize("inter, k", [(64, 128), (8192, 2048), (104, 72)])
def test_gemm_skinny_fused_swiglu_and_interleaved_layout(m, inter, k):
    """Gate and up rows alternating in runs of 8: the decode kernel's fused epilogue and the
    stand-alone activation kernel on the same layout agree with the plain formula."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.ffn import interleave_rows
    x = torch.randn(m, k).to(torch.bfloat16)
    gate = (torch.randn(inter, k) * 0.1).to(torch.bfloat16)
    up = (torch.randn(inter, k) * 0.1).to(torch.bfloat16)
    w = interleave_rows(gate, up, 8)
    assert torch.equal(w[:8], gate[:8]) and torch.equal(w[8:16], up[:8]) and torch.equal(w[16:24], gate[8:16])
    want = torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    fused = ops.gemm_skinny(dev(x), dev(w), swiglu=True)
    assert tuple(fused.shape) == (m, inter)
    close(fused, want, torch.bfloat16, "fused swiglu")
    unfused = ops.swiglu(ops.gemm_skinny(dev(x), dev(w)), 8)
    close(unfused, want, torch.bfloat16, "interleaved swiglu kernel")
    assert (fused.float() - unfused.float()).abs().max().item() <= 0.02 * want.abs().max().item()


@pytest.mark.parametrize("m", [1, 5, 8])
@pytest.mark.parametrize("n, k", [(2048, 2048), (3104, 2048), (1024, 1024), (72, 200), (2048, 8192), (48, 64)])
def test_gemm_skinny_with_the_norm_and_the_residual_add_inside(m, n, k):
    """The two halves of a residual add + RMSNorm taken into the products on either side of it.
    NORM: x is the un-normed stream; the kernel sums its squares while it streams and scales the
    product by each row's 1 / rms, against (x * rstd) @ W.T in 64-bit. ADD: the product, rounded to
    16 bits, joins the residual and the sum is rounded once, bit for bit what the product kernel
    followed by the add + norm kernel's stream gives. Shapes: every CTA form the launch rule picks
    (16-row and 8-row CTAs, two and four slices in flight), sizes that are no power of two."""
    from tokenomos_b200 import ops
    eps = 1e-5
    x = (torch.randn(m, k) * 3.0).to(torch.bfloat16)           # far from unit rms
    w = (torch.randn(n, k) * k ** -0.5).to(torch.bfloat16)
    b = torch.randn(n)
    rstd = (x.double().pow(2).mean(dim=1, keepdim=True) + eps).rsqrt()
    for bias in (None, b):
        got = ops.gemm_skinny(dev(x), dev(w), dev(bias) if bias is not None else None, norm_eps=eps)
        want = (x.double() * rstd) @ w.double().T + (bias.double() if bias is not None else 0.0)
        close(got, want, torch.bfloat16, f"skinny with norm {m}x{n}x{k}")
    residual = (torch.randn(m, n) * 2.0).to(torch.bfloat16)
    got = ops.gemm_skinny(dev(x), dev(w), dev(b), residual=dev(residual))
    product = ops.gemm_skinny(dev(x), dev(w), dev(b))
    _, stream = ops.add_rmsnorm(product, dev(residual), None, 0.0)
    assert torch.equal(got, stream), (got.float() - stream.float()).abs().max().item()
    # a row-strided residual
    wide = (torch.randn(m, n + 16) * 2.0).to(torch.bfloat16)
    got = ops.gemm_skinny(dev(x), dev(w), None, residual=dev(wide)[:, 8:8 + n])
    _, stream = ops.add_rmsnorm(ops.gemm_skinny(dev(x), dev(w)), dev(wide)[:, 8:8 + n].contiguous(), None, 0.0)
    assert torch.equal(got, stream)
    with pytest.raises(ops.KernelError, match="at most 8 rows"):
        ops.gemm_skinny(dev(torch.zeros(9, k, dtype=torch.bfloat16)), dev(w), norm_eps=eps)


@pytest.mark.parametrize("m, inter, k", [(1, 64, 128), (8, 8192, 2048), (3, 104, 72)])
def test_gemm_skinny_fused_swiglu_with_the_norm_inside(m, inter, k):
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.ffn import interleave_rows
    eps = 1e-6
    x = (torch.randn(m, k) * 2.5).to(torch.bfloat16)
    gate = (torch.randn(inter, k) * 0.1).to(torch.bfloat16)
    up = (torch.randn(inter, k) * 0.1).to(torch.bfloat16)
    normed = x.double() * (x.double().pow(2).mean(dim=1, keepdim=True) + eps).rsqrt()
    want = torch.nn.functional.silu(normed @ gate.double().T) * (normed @ up.double().T)
    got = ops.gemm_skinny(dev(x), dev(interleave_rows(gate, up, 8)), swiglu=True, norm_eps=eps)
    close(got, want, torch.bfloat16, "fused swiglu with norm")


@pytest.mark.parametrize("W, d, K, M", [(3, 2048, 2048, 8), (4, 96, 96, 3), (2, 80, 80, 1)])
def test_gemm_skinny_conv_with_the_norm_inside(W, d, K, M):
    """The conv epilogue on a stream that is normed inside the kernel, against the same kernel on
    the stream normed beforehand (weight one) in 64-bit and rounded: B, C, X differ by the
    rounding of the normed input only."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.shortconv import interleave_bcx
    eps = 1e-5
    w = interleave_bcx((torch.randn(3 * d, K) * K ** -0.5).to(torch.bfloat16), 8)
    taps = torch.randn(d, W)
    x = (torch.randn(M, K) * 2.0).to(torch.bfloat16)
    normed = (x.double() * (x.double().pow(2).mean(dim=1, keepdim=True) + eps).rsqrt()).to(torch.bfloat16)
    ctx = [(0, 1, 5, 40, 3, 0, 9, 2)[i % 8] for i in range(M)]
    slot = list(range(1, M + 1))
    state0 = torch.randn(M + 2, W - 1, d).to(torch.bfloat16)
    s1, s2 = dev(state0).clone(), dev(state0).clone()
    want = ops.gemm_skinny_conv(dev(normed), dev(w), None, dev(taps), None, s1, i32(ctx), i32(slot))
    got = ops.gemm_skinny_conv(dev(x), dev(w), None, dev(taps), None, s2, i32(ctx), i32(slot), norm_eps=eps)
    scale = want.float().abs().max().item()
    assert (got.float() - want.float()).abs().max().item() <= 3e-2 * scale
    assert (s1.float() - s2.float()).abs().max().item() <= 3e-2 * s1.float().abs().max().item()
    assert torch.equal(s2[[0, M + 1]].cpu(), state0[[0, M + 1]])


# ---- TMA + tcgen05 matrix product -----------------------------------------------------------------

@pytest.mark.parametrize("m, n, k, split", [(8, 128, 64, False), (1, 256, 512, False), (16, 2048, 2048, True),
                                            (3, 6144, 2048, True), (8, 2048, 8192, True), (8, 200, 72, False),
                                            (40, 1000, 200, True), (64, 3072, 2048, True), (130, 512, 512, True),
                                            (256, 384, 1024, True), (5, 70000, 256, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tc(m, n, k, split, out_dtype):
    from tokenomos_b200 import ops
    x = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) * 0.1).to(torch.bfloat16)
    b = torch.randn(n)
    assert ops.gemm_tc_ok(dev(x), dev(w))
    want = x.double() @ w.double().T + b.double()
    for _ in range(2):         # twice: the split-K scratch must be clean again after a call
        got = ops.gemm_tc(dev(x), dev(w), dev(b), out_dtype, split_k=split)
        close(got, want, out_dtype, f"tc {m}x{n}x{k}")
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("m, inter, k", [(13, 128, 128), (8, 8192, 2048), (64, 1024, 512)])
def test_gemm_tc_fused_swiglu(m, inter, k):
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.ffn import interleave_rows
    x = torch.randn(m, k).to(torch.bfloat16)
    gate = (torch.randn(inter, k) * 0.1).to(torch.bfloat16)
    up = (torch.randn(inter, k) * 0.1).to(torch.bfloat16)
    want = torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    got = ops.gemm_tc(dev(x), dev(interleave_rows(gate, up, 8)), swiglu=True)
    close(got, want, torch.bfloat16, "tc fused swiglu")
    assert ops.gemm_tc_status() == 0


def test_swiglu_vectorised_path_matches_the_scalar_one():
    from tokenomos_b200 import ops
    gu = (torch.randn(33, 2 * 256) * 2).to(torch.bfloat16)
    for block in (0, 8):
        fast = ops.swiglu(dev(gu), block)                      # 16-byte path
        slow = ops.swiglu(dev(gu.float()), block)              # float32 goes through the scalar kernel
        assert (fast.float() - slow).abs().max().item() <= 0.02 * slow.abs().max().item()
