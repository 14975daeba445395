"""The two halves of the forward for a caller that fuses its neighbours: symbols packed by the
caller's projection epilogue go straight into matching, the routed signs come out as int8.
Checked against pack-then-forward (the operator's own path) and against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import rosa_oracle as orc
from tests.helpers import nonzero_randn, repeated_stream_logits

DEV = "cuda"


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D,Dv", [(2, 16), (8, 8), (13, 5), (32, 32)])
def test_packed_symbol_forward_equals_the_operator(dt, D, Dv):
    from rosa_soft_b200 import cabi
    cabi.load()
    B, T, H, Hv, W = 2, 300, 4, 2, 24
    if D <= 2:
        q = repeated_stream_logits(B * T, H, D, seed=3).to(dt).to(DEV)
        k = q.clone()
    else:
        q = nonzero_randn((B * T, H, D), 1, dt).to(DEV)
        k = nonzero_randn((B * T, H, D), 2, dt).to(DEV)
    v = nonzero_randn((B * T, Hv, Dv), 3, dt).to(DEV)
    for desc in ((B, T), torch.tensor([0, 7, 7, 350, B * T], dtype=torch.int32, device=DEV)):
        out, pq, pk, routes, _ = cabi.hard_forward(q, k, v, desc, W)
        # the epilogue contract: words equal to the operator's packed symbols, layout included
        mine_q, mine_k = cabi.pack_symbols(q, desc), cabi.pack_symbols(k, desc)
        assert torch.equal(mine_q, pq) and torch.equal(mine_k, pk)
        out8, routes8, ws = cabi.hard_forward_packed(mine_q, mine_k, v, D, desc, W)
        assert out8.dtype == torch.int8 and cabi.read_status(ws) == 0
        assert torch.equal(out8.float(), out.float()) and torch.equal(routes8, routes)
    cu = np.array([0, 7, 7, 350, B * T], dtype=np.int64)
    f = lambda t: t.float().cpu().numpy()
    ref_out, _ = orc.hard_forward(f(q), f(k), f(v), cu, W)
    assert np.array_equal(out8.cpu().numpy().astype(np.float32), ref_out)


def test_vectorised_and_scalar_paths_of_pack_and_gather_agree():
    """Rows that are whole 16-byte words take 128-bit loads and stores; a misaligned view of the
    same values must give the same words and outputs."""
    from rosa_soft_b200 import cabi
    cabi.load()
    N, H, D, Hv, Dv, W = 500, 4, 8, 2, 16, 16
    base_q = torch.empty(N * H * D + 1, dtype=torch.bfloat16, device=DEV)
    base_v = torch.empty(N * Hv * Dv + 1, dtype=torch.bfloat16, device=DEV)
    q = nonzero_randn((N, H, D), 5, torch.bfloat16).to(DEV)
    v = nonzero_randn((N, Hv, Dv), 6, torch.bfloat16).to(DEV)
    q_off = base_q[1:].view(N, H, D)          # 2 bytes past a 16-byte boundary
    v_off = base_v[1:].view(N, Hv, Dv)
    q_off.copy_(q)
    v_off.copy_(v)
    a = cabi.hard_forward(q, q, v, (1, N), W)
    b = cabi.hard_forward(q_off, q_off, v_off, (1, N), W)
    for x, y in zip(a[:4], b[:4]):
        assert torch.equal(x, y)
