"""The entry point that allocates nothing (``tk_attn_decode_mma_static``, csrc/no_alloc.h),
called the way its users call it: through the exported C symbol, with raw pointers. It exists
for callers that cannot ask for device memory (someone else's stream capture, a serving loop
with a spoken-for pool, a bare C binding); its scratch is an array inside the library. The test
holds its output to the ordinary entry point's, on calls in a row (the array keeps the earlier
call's contents when the next one starts): both head sizes the kernel takes, a window, a single
split (no scratch at all) and a list of rows with a skipped entry; and it checks that an
oversized request is refused."""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n_seqs: int, ctx: int, H: int, Hkv: int, D: int, P: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    blocks = -(-(ctx + 1) // P)
    pages = n_seqs * blocks + 1
    pool = torch.randn(pages, 2, Hkv, P, D, generator=g).to(torch.bfloat16).cuda()
    table = (torch.randperm(pages - 1, generator=g) + 1).to(torch.int32).view(n_seqs, blocks).cuda()
    q = torch.randn(n_seqs, H, D, generator=g).to(torch.bfloat16).cuda()
    positions = torch.full((n_seqs,), ctx, dtype=torch.int32).cuda()
    seq = torch.arange(n_seqs, dtype=torch.int32).cuda()
    return q, pool, table, positions, seq


def _call_static(lib, q, pool, table, positions, seq, nsplit, window=0, index=None):
    n, H, D = q.shape
    _, _, Hkv, P, _ = pool.shape
    out = torch.full_like(q, float("nan"))
    index = seq if index is None else index
    fn = lib.tk_attn_decode_mma_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_void_p] + [ctypes.c_int] * 6 + [
        ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    rc = fn(q.data_ptr(), pool.data_ptr(), out.data_ptr(), positions.data_ptr(), seq.data_ptr(),
            table.data_ptr(), table.stride(0), index.data_ptr(), index.numel(), H, Hkv, D, P, window,
            D ** -0.5, nsplit, torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_static_scratch_entry_point_matches_the_allocating_one():
    from tokenomos_b200 import ops
    from tokenomos_b200.ops import _lib

    lib = _lib.lib()
    for seed, (n_seqs, ctx, nsplit) in enumerate([(5, 700, 4), (3, 1500, 7)]):   # two calls in a row
        q, pool, table, positions, seq = _case(n_seqs, ctx, 8, 2, 64, 16, seed)
        rc, got = _call_static(lib, q, pool, table, positions, seq, nsplit)
        assert rc == 0, lib.tk_last_error().decode()
        want = torch.full_like(q, float("nan"))
        ops.attention_decode_mma(q, pool, want, positions, seq, table, seq, None, 64 ** -0.5, nsplit)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= 2e-2 * scale
        assert torch.equal(got, want)      # same kernel, same order of sums: bit for bit


@pytest.mark.parametrize("what, n_seqs, ctx, H, Hkv, D, nsplit, window, skip", [
    ("head size 128", 4, 900, 8, 2, 128, 5, 0, None),
    ("a window", 5, 1200, 8, 2, 64, 3, 300, None),
    ("one split, no scratch", 6, 200, 8, 4, 64, 1, 0, None),
    ("a skipped entry in the list of rows", 5, 700, 8, 2, 64, 4, 0, 2),
])
def test_static_scratch_entry_point_in_its_other_forms(what, n_seqs, ctx, H, Hkv, D, nsplit, window, skip):
    """Each form twice in a row, against the ordinary entry point given the same arguments. An
    entry of -1 in the list of rows is a padded slot of a captured step: its row of ``out`` stays
    untouched."""
    from tokenomos_b200 import ops
    from tokenomos_b200.ops import _lib

    lib = _lib.lib()
    for seed in (20, 21):
        q, pool, table, positions, seq = _case(n_seqs, ctx, H, Hkv, D, 16, seed)
        index = seq.clone()
        if skip is not None:
            index[skip] = -1
        rc, got = _call_static(lib, q, pool, table, positions, seq, nsplit, window, index)
        assert rc == 0, (what, lib.tk_last_error().decode())
        want = torch.full_like(q, float("nan"))
        ops.attention_decode_mma(q, pool, want, positions, seq, table, index, window or None, D ** -0.5, nsplit)
        torch.cuda.synchronize()
        rows = [i for i in range(n_seqs) if i != skip]
        assert torch.isfinite(got[rows].float()).all(), what
        assert torch.equal(got[rows], want[rows]), what
        if skip is not None:
            assert torch.isnan(got[skip].float()).all() and torch.isnan(want[skip].float()).all()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from tokenomos_b200.ops import _lib

    lib = _lib.lib()
    lib.tk_attn_decode_mma_static_capacity.restype = ctypes.c_longlong
    capacity = lib.tk_attn_decode_mma_static_capacity()
    assert capacity == 2 << 20
    q, pool, table, positions, seq = _case(64, 100, 32, 8, 64, 16, 9)
    nsplit = capacity // (64 * 32 * 66) + 1
    rc, out = _call_static(lib, q, pool, table, positions, seq, int(nsplit))
    assert rc < 0 and "built-in array holds" in lib.tk_last_error().decode()
    assert torch.isnan(out.float()).all()      # nothing was launched
