"""The dense backward runs a batch in slices of whole sequences when the partial gradient rows of
the whole batch would not fit their budget; the slices share one workspace.

The budget is read once per process, so the sliced run happens in a child process with a budget
small enough that a five-sequence batch needs two slices (3 + 2 sequences).  The child
compares the sliced call with five single-sequence calls at the matching dropout batch
coordinates -- bit for bit, outputs and gradients -- with and without dropout and window, and
checks that the workspace the sliced call asks for is that of its largest slice."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

_CHILD = r"""
import sys
import torch
import rosa_soft_b200 as rs
from rosa_soft_b200 import cabi, sharding
from tests.helpers import nonzero_randn

dev = torch.device("cuda", 0)
B, T, H, D, Hv, Dv = 5, 512, 4, 8, 2, 8
lib = cabi.load()
whole = lib.rosa_b200_surrogate_vjp_workspace_bytes(B * T, H, D, Hv, Dv, B, T, 16, 7)
three = lib.rosa_b200_surrogate_vjp_workspace_bytes(3 * T, H, D, Hv, Dv, 3, T, 16, 7)
four = lib.rosa_b200_surrogate_vjp_workspace_bytes(4 * T, H, D, Hv, Dv, 4, T, 16, 7)
# two slices, the larger of three sequences (which on its own runs unsliced)
assert whole == three and four < three, (whole, three, four)
for W, p in ((16, 0.0), (16, 0.25), (T, 0.25)):
    kw = dict(max_suffix_length=W, scale=1.0, dropout_p=p, mismatch_scale=3.0)
    q = nonzero_randn((B, T, H, D), 11).to(dev)
    k = nonzero_randn((B, T, H, D), 12).to(dev)
    v = nonzero_randn((B, T, Hv, Dv), 13).to(dev)
    go = nonzero_randn((B, T, H, Dv), 14).to(dev)

    def run(q, k, v, go, first):
        q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
        torch.cuda.manual_seed(5)
        with sharding.dropout_coordinates(first, 0):
            out = rs.rosa_soft(q, k, v, **kw)
            out.backward(go)
        return out.detach(), q.grad, k.grad, v.grad

    sliced = run(q, k, v, go, 0)
    for b in range(B):
        one = run(q[b:b + 1], k[b:b + 1], v[b:b + 1], go[b:b + 1], b)
        for name, got, want in zip(("out", "dq", "dk", "dv"), sliced, one):
            if not torch.equal(got[b:b + 1], want):
                sys.exit(f"W={W} p={p} batch {b}: {name} differs, max "
                         f"{float((got[b:b + 1] - want).abs().max()):.3e}")
print("slices ok")
"""


def test_sliced_dense_backward_equals_single_sequences():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ROSA_B200_PARTIAL_BUDGET_MB="2", PYTHONPATH=root)
    done = subprocess.run([sys.executable, "-c", _CHILD], cwd=root, env=env, capture_output=True,
                          text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    assert "slices ok" in done.stdout
