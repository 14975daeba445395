"""Benchmark of the rosa_soft training step (hard forward + dense surrogate VJP).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line.  A step is one forward + backward of the operator over one batch of
seeded synthetic inputs of the named workload.  `value` is whole-job throughput in
M token-heads/s (B*T*H token-heads per step and rank, summed over ranks, divided by the
slowest rank's device time) with inputs resident in HBM; `e2e` is the same metric measured
through the public operator with pinned HOST buffers copied in and results copied out inside
the timed region.  Multi-GPU runs are weak scaling: every rank holds one (batch x head)
shard of identical size, there is no collective inside the operator, and the only
communication is the barrier / max-reduce of the timings.

--impl reference times the CPU restatement of the reference's algorithm (the oracle, all host
threads) on a bounded sample of the same workload; the Python reference itself cannot travel
to the benchmark box.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> per-rank shape; "metric" is the shape the headline metric is quoted on
# (T=8192, H=64, D=8 with the value-head grouping and controls of the README training shape).
WORKLOADS = {
    "metric": dict(B=2, T=8192, H=64, D=8, Hv=16, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                   dtype="bfloat16", gen="randn"),
    "c2": dict(B=2, T=1024, H=64, D=8, Hv=16, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
               dtype="bfloat16", gen="randn"),
    "c3": dict(B=1, T=8192, H=64, D=2, Hv=64, Dv=16, W=256, scale=1.0, p=0.0, m=3.0,
               dtype="bfloat16", gen="repeat"),
    # a case small enough for a full-metric profiler capture whose scratch still exceeds L2
    "profile": dict(B=1, T=4096, H=32, D=8, Hv=8, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                    dtype="bfloat16", gen="randn"),
    # packed variable-length case: 32768 tokens in sequences of 64..4096 tokens
    "c4": dict(kind="varlen", N=32768, Lmin=64, Lmax=4096, B=1, T=32768, H=32, D=16, Hv=8, Dv=32,
               W=64, scale=1.0, p=0.05, m=9.0, dtype="float16", gen="randn"),
    # batched hard inference: 64 streams x 16384 tokens x 64 heads of 32-bit symbols, forward only
    "c5": dict(kind="inference", B=64, T=16384, H=64, D=32, Hv=64, Dv=8, W=32, scale=1.0, p=0.0,
               m=3.0, dtype="float32", gen="symbols"),
    # streaming runtime: 64 slots x 16384 tokens x 64 heads of 8-bit symbols fed in chunks of 2048
    # tokens per slot to a runtime whose state stays on the GPU (the reference's RosaRuntime use)
    "stream": dict(kind="stream", B=64, T=16384, H=64, D=8, Hv=64, Dv=8, W=32, chunk=2048, scale=1.0,
                   p=0.0, m=3.0, dtype="uint8", gen="symbols"),
    # 8 of the inference workload's streams: small enough for a multi-pass profiler capture
    "c5_profile": dict(kind="inference", B=8, T=16384, H=64, D=32, Hv=64, Dv=8, W=32, scale=1.0,
                       p=0.0, m=3.0, dtype="float32", gen="symbols"),
    # 8 of the stream workload's slots: small enough for a multi-pass profiler capture
    "stream_profile": dict(kind="stream", B=8, T=16384, H=64, D=8, Hv=64, Dv=8, W=32, chunk=2048,
                           scale=1.0, p=0.0, m=3.0, dtype="uint8", gen="symbols"),
    "small": dict(B=1, T=1024, H=8, D=8, Hv=2, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                  dtype="bfloat16", gen="randn"),
}
# bounded CPU sample of a workload: same D/Dv/W/controls, fewer heads and a shorter sequence
CPU_SAMPLE = dict(B=1, T=2048, H=64)


def varlen_lengths(cfg, seed):
    """Sequence lengths uniform in [Lmin, Lmax] until the token budget is used (last one cut)."""
    import numpy as np

    rng = np.random.default_rng(seed)
    lengths, total = [], 0
    while total < cfg["N"]:
        n = min(int(rng.integers(cfg["Lmin"], cfg["Lmax"] + 1)), cfg["N"] - total)
        lengths.append(n)
        total += n
    return lengths


def make_inference_inputs(cfg, seed, device):
    """i.i.d. 32-bit symbols; 10 % of the positions start a copy of an earlier window of 8..512
    symbols into both streams, so that long matches exist."""
    import numpy as np
    import torch

    rng = np.random.default_rng(seed)
    B, T, H = cfg["B"], cfg["T"], cfg["H"]
    k = rng.integers(0, 1 << 32, size=(B, T, H), dtype=np.uint64).astype(np.uint32)
    q = rng.integers(0, 1 << 32, size=(B, T, H), dtype=np.uint64).astype(np.uint32)
    for b in range(B):
        t = 600
        while t < T - 520:
            if rng.random() < 0.1:
                n = int(rng.integers(8, 513))
                src = int(rng.integers(0, t - n))
                k[b, t:t + n] = k[b, src:src + n]
                q[b, t + 1:t + 1 + n] = k[b, src + 1:src + 1 + n]
                t += n
            t += int(rng.integers(1, 20))
    payload = rng.standard_normal((B, T, cfg["Hv"], cfg["Dv"])).astype(np.float32)
    to = lambda a: torch.from_numpy(a).to(device)
    return to(q.view(np.int32)), to(k.view(np.int32)), to(payload)


def make_inputs(cfg, seed, device, dtype):
    import torch

    g = torch.Generator().manual_seed(seed)
    B, T, H, D, Hv, Dv = (cfg[k] for k in ("B", "T", "H", "D", "Hv", "Dv"))
    if cfg["gen"] == "repeat":
        import numpy as np

        rng = np.random.default_rng(seed)
        toks = np.empty((B, H, T), np.int64)
        for b in range(B):
            for h in range(H):
                out = []
                while len(out) < T:
                    n = int(rng.integers(16, 257))
                    if out and rng.random() < 0.3 and len(out) > n:
                        s = int(rng.integers(0, len(out) - n + 1))
                        out.extend(out[s:s + n])
                    else:
                        out.extend(rng.integers(0, 1 << D, size=n).tolist())
                toks[b, h] = out[:T]
        bits = (toks[..., None] >> np.arange(D)) & 1            # [B,H,T,D]
        q = torch.from_numpy(np.where(bits, 1.0, -1.0).astype("float32")).permute(0, 2, 1, 3)
        q = q.contiguous()
        k = q.clone()
    else:
        q = torch.randn(B, T, H, D, generator=g)
        k = torch.randn(B, T, H, D, generator=g)
    v = torch.randn(B, T, Hv, Dv, generator=g)
    go = torch.randn(B, T, H, Dv, generator=g)
    return [t.to(dtype).to(device) if device is not None else t.to(dtype) for t in (q, k, v, go)]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.time() + 3.0   # let the first sample arrive before timing starts
            while not self.samples and time.time() < deadline:
                time.sleep(0.02)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def make_stream_inputs(cfg, seed, device):
    """i.i.d. 8-bit symbols per (slot, head); 10 % of the positions start a copy of an earlier
    window of 8..512 tokens into both streams, so that matches reach the horizon."""
    import numpy as np
    import torch

    rng = np.random.default_rng(seed)
    B, T, H = cfg["B"], cfg["T"], cfg["H"]
    hi = 1 << cfg["D"]
    k = rng.integers(0, hi, size=(B, T, H), dtype=np.uint8)
    q = rng.integers(0, hi, size=(B, T, H), dtype=np.uint8)
    for b in range(B):
        t = 600
        while t < T - 520:
            if rng.random() < 0.1:
                n = int(rng.integers(8, 513))
                src = int(rng.integers(0, t - n))
                k[b, t:t + n] = k[b, src:src + n]
                q[b, t + 1:t + 1 + n] = k[b, src + 1:src + 1 + n]
                t += n
            t += int(rng.integers(1, 20))
    payload = rng.integers(0, 1 << cfg["Dv"], size=(B, T, cfg["Hv"]), dtype=np.uint8)
    to = lambda a: torch.from_numpy(a).to(device)
    return to(q), to(k), to(payload)


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_stream_run(cfg, steps, warmup):
    """The reference's own RosaRuntime (suffix automata on the host cores, compiled from its
    source into oracle/_ref/) fed the same chunks; the oracle's one-shot matcher when that
    library is absent."""
    import numpy as np
    import torch

    sample = dict(cfg, B=min(cfg["B"], 16))
    q, k, pay = make_stream_inputs(sample, 7, "cpu")
    B, T, H, chunk = sample["B"], sample["T"], sample["H"], sample["chunk"]
    lib = os.path.join(ROOT, "oracle", "_ref", "librosa_runtime_ref.so")
    times = []
    if os.path.exists(lib):
        torch.set_num_threads(host_cores())   # torchrun exports OMP_NUM_THREADS=1
        torch.classes.load_library(lib)
        runtime = torch.classes.rosa_soft.RosaRuntime(H, sample["Hv"], sample["D"], sample["Dv"],
                                                      sample["W"])
        for it in range(warmup + steps):
            runtime.reset()
            t0 = time.perf_counter()
            for a in range(0, T, chunk):
                n = min(chunk, T - a)
                cu = torch.arange(B + 1, dtype=torch.int64) * n
                flat = lambda x: x[:, a:a + n].reshape(B * n, -1).contiguous()
                runtime.update_packed(cu, flat(q), flat(k), flat(pay))
            if it >= warmup:
                times.append(time.perf_counter() - t0)
        kind, cores = "reference", torch.get_num_threads()
        what = "the reference's RosaRuntime (suffix automata, OpenMP over slot x head)"
    else:
        from oracle import rosa_oracle as orc
        orc.set_num_threads(host_cores())
        cu = np.arange(B + 1, dtype=np.int64) * T
        flat = lambda x: x.numpy().reshape((B * T,) + tuple(x.shape[2:]))
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            orc.hard_inference(flat(q).astype(np.uint32), flat(k).astype(np.uint32),
                               flat(pay).astype(np.float32)[:, :, None], cu, sample["W"])
            if it >= warmup:
                times.append(time.perf_counter() - t0)
        kind, cores = "port", orc.num_threads()
        what = "the oracle's one-shot matcher (reference runtime library not built)"
    sec = sum(times) / len(times)
    desc = f"{B} of the {cfg['B']} slots x T={T} x H={H} in chunks of {chunk}: {what}"
    return B * T * H / sec / 1e6, sec, cores, desc, kind


def cpu_reference_run(cfg, steps, warmup):
    """Times the oracle (CPU restatement of the reference algorithm) on a bounded sample."""
    import numpy as np
    import torch

    from oracle import rosa_oracle as orc

    orc.set_num_threads(host_cores())   # torchrun exports OMP_NUM_THREADS=1
    if cfg.get("kind") == "inference":
        sample = dict(cfg, B=4, T=4096, H=8, Hv=8)
        qs, ks, pay = (t.numpy() for t in make_inference_inputs(sample, 7, "cpu"))
        B, T, H = sample["B"], sample["T"], sample["H"]
        cu = np.arange(B + 1, dtype=np.int64) * T
        flat = lambda a: a.reshape((B * T,) + a.shape[2:])
        times = []
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            orc.hard_inference(flat(qs).view(np.uint32), flat(ks).view(np.uint32), flat(pay), cu,
                               sample["W"])
            if it >= warmup:
                times.append(time.perf_counter() - t0)
        sec = sum(times) / len(times)
        desc = (f"{B} streams x T={T} x H={H} of the workload (quadratic run-length matcher; cost per "
                f"token-head grows with T)")
        return B * T * H / sec / 1e6, sec, orc.num_threads(), desc

    sample = dict(cfg, **{k: min(cfg[k], v) for k, v in CPU_SAMPLE.items()})
    sample["Hv"] = max(1, sample["H"] // (cfg["H"] // cfg["Hv"]))
    q, k, v, go = (t.float().numpy() for t in make_inputs(sample, 7, None, torch.float32))
    B, T, H = sample["B"], sample["T"], sample["H"]
    flat = lambda a: a.reshape((B * T,) + a.shape[2:])
    cu = np.arange(B + 1, dtype=np.int64) * T
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        orc.hard_forward(flat(q), flat(k), flat(v), cu, sample["W"])
        orc.surrogate_vjp(flat(q), flat(k), flat(v), flat(go), cu, sample["W"], sample["scale"],
                          sample["p"], sample["m"], 12345)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    desc = (f"B={B} T={T} H={H} of the workload (same D, Dv, W, controls); cost per token-head "
            f"grows with T*W, so the full T={cfg['T']} costs about {cfg['T'] // T}x more per token-head")
    return B * T * H / sec / 1e6, sec, orc.num_threads(), desc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="metric", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    what = {"inference": "batched hard inference, forward only",
            "stream": f"RosaRuntime chunked updates ({cfg.get('chunk')} tokens per slot and call), "
                      "forward only",
            "varlen": "rosa_soft_varlen fwd+bwd"}.get(cfg.get("kind"), "rosa_soft fwd+bwd")
    config = {"workload": f"{args.workload}: {what}, per rank B={cfg['B']} T={cfg['T']} "
                          f"H={cfg['H']} D={cfg['D']} Hv={cfg['Hv']} Dv={cfg['Dv']} W={cfg['W']} "
                          f"p={cfg['p']} m={cfg['m']} scale={cfg['scale']} {cfg['dtype']}",
              "global_batch": cfg["B"] * world, "seq_len": cfg["T"],
              "parallelism": f"{world} independent (batch x head) shards, no collective in the operator",
              "l2": "flushed between timed steps by writing a 512 MiB buffer; the step's own "
                    "checkpoint/partial scratch is larger than L2"}

    if args.impl == "reference":
        if rank != 0:
            return
        base_kind = "port"
        if cfg.get("kind") == "stream":
            value, sec, cores, desc, base_kind = cpu_stream_run(cfg, max(1, args.steps),
                                                                max(0, min(args.warmup, 1)))
        else:
            value, sec, cores, desc = cpu_reference_run(cfg, max(1, args.steps),
                                                        max(0, min(args.warmup, 1)))
        forward_only = cfg.get("kind") in ("inference", "stream")
        print(json.dumps({
            "impl": "reference",
            "metric": "forward M token-heads/s" if forward_only else "fwd+bwd M token-heads/s",
            "value": value,
            "unit": "M token-heads/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "u8 symbols" if cfg.get("kind") == "stream" else "f64", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": value, "unit": "M token-heads/s", "cores": cores,
                             "kind": base_kind, "sample": desc},
            "e2e": {"value": value, "unit": "M token-heads/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
        }))
        return

    import torch

    import rosa_soft_b200 as rs
    from rosa_soft_b200 import cabi

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (the package has no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    dtype = getattr(torch, cfg["dtype"])
    kind = cfg.get("kind", "dense")
    forward_only = kind in ("inference", "stream")
    kw = dict(max_suffix_length=cfg["W"], scale=cfg["scale"], dropout_p=cfg["p"], mismatch_scale=cfg["m"])
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    if kind == "inference":
        inputs = list(make_inference_inputs(cfg, 1000 + rank, dev))
        pairs = cfg["B"] * cfg["H"] * cfg["T"] * (cfg["T"] - 1) // 2

        def step(qs, ks, pay):
            return list(rs.rosa_hard_inference(qs, ks, pay, max_suffix_length=cfg["W"]))
    elif kind == "stream":
        inputs = list(make_stream_inputs(cfg, 1000 + rank, dev))
        pairs = cfg["B"] * cfg["H"] * cfg["T"] * (cfg["T"] - 1) // 2
        runtime = rs.RosaRuntime(cfg["H"], cfg["Hv"], cfg["D"], cfg["Dv"], cfg["W"])

        def step(qs, ks, pay):
            runtime.reset()
            outs, ends = [], []
            for a in range(0, cfg["T"], cfg["chunk"]):
                b = min(cfg["T"], a + cfg["chunk"])
                out, end = runtime.update_packed(qs[:, a:b], ks[:, a:b], pay[:, a:b])
                outs.append(out)
                ends.append(end)
            return [torch.cat(outs, dim=1), torch.cat(ends, dim=1)]
    elif kind == "varlen":
        lengths = varlen_lengths(cfg, 1004)
        cu = torch.tensor([0] + list(__import__("itertools").accumulate(lengths)), dtype=torch.int32,
                          device=dev)
        inputs = [t.squeeze(0).contiguous() for t in make_inputs(cfg, 1000 + rank, dev, dtype)]
        pairs = cfg["H"] * sum(n * (n - 1) // 2 for n in lengths)
        config["sequence_lengths"] = lengths

        def step(qq, kk, vv, gg):
            for t in (qq, kk, vv):
                t.grad = None
                t.requires_grad_(True)
            out = rs.rosa_soft_varlen(qq, kk, vv, cu, **kw)
            out.backward(gg)
            return [out.detach(), qq.grad, kk.grad, vv.grad]
    else:
        inputs = make_inputs(cfg, 1000 + rank, dev, dtype)
        pairs = cfg["B"] * cfg["H"] * cfg["T"] * (cfg["T"] - 1) // 2

        def step(qq, kk, vv, gg):
            for t in (qq, kk, vv):
                t.grad = None
                t.requires_grad_(True)
            out = rs.rosa_soft(qq, kk, vv, **kw)
            out.backward(gg)
            return [out.detach(), qq.grad, kk.grad, vv.grad]

    for _ in range(max(3, args.warmup)):
        step(*inputs)
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing, per-kernel events enabled for the same steps
    cabi.profile_enable(True)
    cabi.profile_collect()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    with ClockSampler(local_rank) as clocks:
        for i in range(args.steps):
            flush.fill_(i)
            starts[i].record()
            step(*inputs)
            stops[i].record()
        barrier()
    kernels = cabi.profile_collect()
    cabi.profile_enable(False)
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = sum(step_ms)

    # ---- end to end: pinned host buffers in, results out, inside the timed region
    host = [t.detach().cpu().pin_memory() for t in inputs]
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in step(*inputs)]
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_stop = torch.cuda.Event(enable_timing=True)

    def e2e_step():
        device_inputs = [h.to(dev, non_blocking=True) for h in host]
        for dst, src in zip(host_out, step(*device_inputs)):
            dst.copy_(src, non_blocking=True)

    e2e_step()
    barrier()
    e2e_start.record()
    for _ in range(args.steps):
        e2e_step()
    e2e_stop.record()
    barrier()
    e2e_ms = e2e_start.elapsed_time(e2e_stop)

    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = times.tolist()
    units = cfg["B"] * cfg["T"] * cfg["H"] * world
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (the backward's second sweep)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    flop = (6 * cfg["D"] + 4 * cfg["Dv"]) * pairs           # algorithmic contraction FLOP per launch
    if forward_only:
        flop = 0
    k_ms, k_n = kernels.get("vjp_sweep2", (0.0, 0))
    k_avg_s = (k_ms / k_n / 1e3) if k_n else None
    tensor_peak = peaks.get("bf16_tflops_sustained")
    peak_note = "measured (sustained bf16 cuBLAS)"
    if tensor_peak is None:
        tensor_peak, peak_note = 1400.0, "fallback"
    achieved = flop / k_avg_s / 1e12 if k_avg_s else None
    s = 2 if cfg["dtype"] != "float32" else 4
    per_unit = (80 if kind == "inference" else 12 if kind == "stream" else
                2 * cfg["D"] * s + cfg["Dv"] * s * cfg["Hv"] / cfg["H"] + cfg["Dv"] * s + 8)
    fwd_bytes = per_unit * cfg["B"] * cfg["T"] * cfg["H"]
    fwd_ms = sum(kernels.get(n, (0.0, 0))[0] for n in ("pack_symbols", "transpose_symbols", "build_match_masks", "hard_match", "hard_match_hashed",
                                                       "gather_output", "inference_finish",
                                                       "stream_prepare", "stream_append", "stream_match",
                                                       "stream_finish"))
    fwd_n = 1 if kind == "stream" else (kernels.get("hard_match", (0.0, 1))[1] or 1)
    if kind == "stream":
        fwd_ms /= args.steps
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    fwd_gbs = fwd_bytes / (fwd_ms / fwd_n / 1e3) / 1e9 if fwd_ms else None
    result = {
        "metric": ("forward M token-heads/s" if forward_only else "fwd+bwd M token-heads/s"),
        "value": units * args.steps / (total_ms / 1e3) / 1e6,
        "unit": "M token-heads/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": ("u8 symbols" if kind == "stream" else
                  "f32 accumulate on " + cfg["dtype"] + " inputs; integer symbols"),
        "data": "synthetic", "config": config,
        "clocks": clocks.summary(),
        "e2e": {"value": units * args.steps / (e2e_ms / 1e3) / 1e6, "unit": "M token-heads/s",
                "h2d_bytes_per_step": sum(h.numel() * h.element_size() for h in host),
                "d2h_bytes_per_step": sum(h.numel() * h.element_size() for h in host_out)},
        "gpu_launches": sum(n for _, n in kernels.values()),
        "roofline": {"bound": "tensor", "kernel": "vjp_sweep2", "achieved": achieved,
                     "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": (achieved / tensor_peak) if achieved else None,
                     # dram__bytes_read + dram__bytes_write of one launch: 0.986 B per causal pair,
                     # captured with ncu on the `profile` workload (268.4 M pairs) and scaled by
                     # pairs -- checkpoints, keep ballots and partials all grow with the pairs
                     "traffic": (0.986 * pairs) if flop else None,
                     "peak_source": peak_note,
                     "note": "algorithmic contraction work (6D+4Dv FLOP per causal pair) over the "
                             "kernel's mean launch time; the kernel is bound by CUDA-core issue, "
                             "not by the tensor pipe"},
        "roofline_forward": {"bound": "hbm",
                             "kernels": ("stream_append+stream_match+stream_finish" if kind == "stream"
                                         else "pack_symbols+build_match_masks+hard_match(+hashed)+gather_output"),
                             "achieved": fwd_gbs, "peak": hbm_peak, "unit": "GB/s",
                             "frac": (fwd_gbs / hbm_peak) if fwd_gbs else None},
        "kernel_ms_per_step": {n: ms / args.steps for n, (ms, _) in sorted(kernels.items())},
    }
    if not args.no_cpu_baseline and world == 1:   # the CPU baseline is reported at N=1 only
        base_kind = "port"
        if kind == "stream":
            value, sec, cores, desc, base_kind = cpu_stream_run(cfg, 1, 1)
        else:
            value, sec, cores, desc = cpu_reference_run(cfg, 1, 0)
        result["cpu_baseline"] = {"value": value, "unit": "M token-heads/s", "cores": cores,
                                  "kind": base_kind, "sample": desc, "seconds": sec}
    print(json.dumps(result))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
