"""CUDA-graph capture of the operators: the library only enqueues work on the caller's stream
(no allocation, no synchronisation, device-side sequence plan, device-resident dropout seed), so a
forward+backward step can be captured once and replayed on new data."""
import pytest
import torch

from tests.helpers import nonzero_randn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _static_inputs(B, T, H, D, Hv, Dv, dtype):
    q = nonzero_randn((B, T, H, D), 1, dtype).to(DEV).requires_grad_(True)
    k = nonzero_randn((B, T, H, D), 2, dtype).to(DEV).requires_grad_(True)
    v = nonzero_randn((B, T, Hv, Dv), 3, dtype).to(DEV).requires_grad_(True)
    go = nonzero_randn((B, T, H, Dv), 4, dtype).to(DEV)
    return q, k, v, go


@pytest.mark.parametrize("dropout_p", [0.0, 0.25])
def test_forward_backward_replays_from_a_cuda_graph(dropout_p):
    import rosa_soft_b200 as rs
    B, T, H, D, Hv, Dv, W = 2, 300, 4, 4, 2, 8, 16
    q, k, v, go = _static_inputs(B, T, H, D, Hv, Dv, torch.float32)
    kw = dict(max_suffix_length=W, scale=1.0, dropout_p=dropout_p, mismatch_scale=3.0)

    def step():
        out = rs.rosa_soft(q, k, v, **kw)
        return (out, *torch.autograd.grad(out, (q, k, v), go))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    # new data in the captured buffers, then replay
    with torch.no_grad():
        q.copy_(nonzero_randn(q.shape, 11, torch.float32))
        k.copy_(nonzero_randn(k.shape, 12, torch.float32))
        v.copy_(nonzero_randn(v.shape, 13, torch.float32))
        go.copy_(nonzero_randn(go.shape, 14, torch.float32))
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in captured]
    assert all(torch.isfinite(t).all() for t in replayed)
    eager = step()
    assert torch.equal(replayed[0], eager[0])           # the hard forward does not depend on dropout
    if dropout_p == 0.0:
        for a, b in zip(replayed[1:], eager[1:]):
            assert torch.equal(a, b)                     # fixed reduction order: bitwise equal
    else:
        graph.replay()                                   # every replay draws a new seed
        torch.cuda.synchronize()
        assert not torch.equal(captured[1], replayed[1])


def test_streaming_runtime_update_replays_from_a_cuda_graph():
    """One decode step (one token per slot) captured and replayed: the state tensors and the
    device-side lengths advance inside the graph."""
    import numpy as np
    from rosa_soft_b200 import cabi
    from oracle import rosa_oracle as orc
    S, H, Hp, bits, W, cap, steps = 3, 4, 2, 2, 8, 256, 40
    rng = np.random.default_rng(5)
    q = rng.integers(0, 1 << bits, size=(S, steps, H), dtype=np.uint8)
    k = np.where(rng.random((S, steps, H)) < 0.7, q, rng.integers(0, 1 << bits, size=(S, steps, H))).astype(np.uint8)
    p = rng.integers(0, 256, size=(S, steps, Hp), dtype=np.uint8)
    kh = torch.zeros((S, H, 1 << bits, cap // 32), dtype=torch.int32, device=DEV)
    run = torch.zeros((S, H, cap), dtype=torch.uint8, device=DEV)
    ph = torch.zeros((S, Hp, cap), dtype=torch.uint8, device=DEV)
    lengths = torch.zeros(S, dtype=torch.int32, device=DEV)
    off = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    sq, sk = (torch.zeros((S, H), dtype=torch.uint8, device=DEV) for _ in range(2))
    sp = torch.zeros((S, Hp), dtype=torch.uint8, device=DEV)
    tq, tk, tp = (torch.from_numpy(x).to(DEV) for x in (q, k, p))
    outs, ends = [], []
    graph, captured = None, None
    for t in range(steps):
        sq.copy_(tq[:, t]); sk.copy_(tk[:, t]); sp.copy_(tp[:, t])
        if t < 3:        # eager steps first (they also serve as warm-up)
            out, end, _ = cabi.stream_update(sq, sk, sp, off, bits, 8, W, kh, run, ph, lengths, steps)
        else:
            if graph is None:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    captured = cabi.stream_update(sq, sk, sp, off, bits, 8, W, kh, run, ph, lengths, steps)
            # capture does not execute: every step from here on is one replay
            graph.replay()
            out, end = captured[0], captured[1]
        outs.append(out.clone().cpu().numpy())
        ends.append(end.clone().cpu().numpy())
    got_out = np.stack(outs, axis=1).reshape(S * steps, H)
    got_end = np.stack(ends, axis=1).reshape(S * steps, H)
    cu = np.arange(S + 1) * steps
    want_out, want_end = orc.hard_inference(q.reshape(-1, H).astype(np.uint32), k.reshape(-1, H).astype(np.uint32),
                                            p.reshape(-1, Hp).astype(np.float32)[:, :, None], cu, W)
    assert np.array_equal(got_end, want_end)
    assert np.array_equal(got_out, want_out[:, :, 0].astype(np.uint8))
