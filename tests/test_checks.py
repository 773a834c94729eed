"""The debug build of the kernel library (``TOKENOMOS_B200_CHECKS=1``, csrc/checks.cuh): every
kernel that follows a page number, a state row or a table row compares it with the pool's size,
records the first one outside and carries on with the null page or row. No memory checker can
be run on the test machines; this build is the stand-in, and the replay runs once under it.

It is a different library, chosen when the library is first loaded, so each test runs in a
process of its own."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def run_checked(code: str, *args: str) -> str:
    env = dict(os.environ, TOKENOMOS_B200_CHECKS="1")
    proc = subprocess.run([sys.executable, "-c", code, *args], capture_output=True, text=True, env=env,
                          cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    return proc.stdout


REPLAY = """
import sys
sys.path.insert(0, "tests")
import torch
import trace_util, test_replay
from tokenomos_b200 import ops
folder, name, dtype, page = sys.argv[1], sys.argv[2], sys.argv[3], int(sys.argv[4])
assert ops.checks_enabled()
reqs = test_replay.requests_for(name)
steps = trace_util.mixed(reqs, live=4, seed=ord(name))
per_step = trace_util.run_in_process(folder, dtype, steps, trace_util.max_live_tokens(steps, page), page)
got = trace_util.collect(steps, per_step)
assert all(torch.isfinite(v).all() for v in got.values())
assert ops.checks_status() is None, ops.checks_status()
tail = trace_util.tail_decoded(reqs, 32)
trace_util.run_in_process(folder, dtype, tail, trace_util.max_live_tokens(tail, page), page)
assert ops.checks_status() is None, ops.checks_status()
print("clean", len(steps) + len(tail))
"""


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("D", "bfloat16"), ("C", "bfloat16")])
def test_replay_under_the_index_checks_finds_nothing(name, dtype, model_folders):
    """The mixed trace (pages and state rows used again, a pool with not a page to spare) and the
    tail-decoded one, in the generic kernels (A in 32-bit, C with its windows) and the tensor-core
    ones (D): no kernel follows an index outside its pool."""
    out = run_checked(REPLAY, str(model_folders[name][torch.bfloat16]), name, dtype, str(TINY[name]["page"]))
    assert out.startswith("clean")


CONTROL = """
import sys
sys.path.insert(0, "tests")
import torch
from tokenomos_b200 import models, ops
from tokenomos_b200.cache.manager import CacheManager
from tokenomos_b200.engine.step import StepEntry, StepFunction
folder, dtype = sys.argv[1], sys.argv[2]
conf = models.configure(folder, work=dtype)
model = models.load(folder, "cuda", conf)
cache = CacheManager(model.state_specs(), 16, 12, 6, conf.work, "cuda", max_len=64)
step = StepFunction(model, cache)
for r in range(5):                       # requests 0..4 take slots 1..5 and pages 1..10
    cache.admit(r)
    step.run([StepEntry(r, list(range(3, 23)), [])])
assert ops.checks_status() is None
# the kernels are told of smaller pools than the real ones: request 4's pages (9, 10) and its
# state row (5) are inside the memory that exists, and outside what the checks allow
ops.set_check_bounds(9, 5)
logits = step.run([StepEntry(4, [7], [0]), StepEntry(0, [8], [0])])
torch.cuda.synchronize()
found = ops.checks_status()
print(found)
assert found is not None and "outside its pool" in found
assert ops.checks_status() is None       # reading resets the word
assert torch.isfinite(logits[1]).all()   # the request inside the bounds is not disturbed
"""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_index_outside_the_pool_is_reported_and_not_followed(dtype, model_folders):
    """Negative control. The pools are real and larger than the bounds the kernels are given, so
    the reported index never leaves allocated memory even if a check were missing; with the check
    the kernel goes to the null page or row, the word names the index, and the context lives."""
    out = run_checked(CONTROL, str(model_folders["D"][torch.bfloat16]), dtype)
    assert "outside its pool" in out
