"""Benchmark of the rosa_soft operator family on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]
                    [--only-headline] [--no-cpu-baseline]

Prints ONE JSON line.  A step is one pass of the hot path (forward + backward of the operator,
or a forward-only hard-inference pass) over one batch of seeded synthetic inputs.

Every workload is ONE FIXED global problem.  With N ranks it is split into independent units --
(batch x value-head group) for dense batches, whole packed sequences balanced by their
quadratic cost, (stream) for hard inference -- with `rosa_soft_b200.sharding`; a rank runs the
unmodified operator on its share and passes the share's global coordinates to the dropout
counter, so the N-rank result is bit-equal to the 1-rank result.  There is no collective inside
the operator; NCCL is used for the barrier / max-reduce of the timings and, as a second timed
variant, for an all-gather of outputs and gradients (`gather`).  `scaling` is "strong".

`value` is whole-job throughput in M token-heads/s (global token-heads per step divided by the
slowest rank's device time) with inputs resident in HBM; `e2e` is the same metric through the
public operator with pinned HOST buffers copied in and results copied out inside the timed
region.  `workloads` carries the other benchmark configurations, measured the same way with
fewer steps.

--impl reference times the CPU restatement of the reference's algorithm (the oracle, all host
threads; for the streaming workload the reference's own RosaRuntime compiled into oracle/_ref)
on a bounded sample; its line names the sample it really ran.
"""
from __future__ import annotations

import argparse
import itertools
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> GLOBAL problem.  "metric" is the shape the headline metric is quoted on (T=8192, H=64,
# D=8 with the value-head grouping and controls of the README training shape); its batch of 16
# gives each of 8 ranks the two batch elements of the README shape.
WORKLOADS = {
    "metric": dict(B=16, T=8192, H=64, D=8, Hv=16, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                   dtype="bfloat16", gen="randn"),
    "c2_f32": dict(B=2, T=1024, H=64, D=8, Hv=16, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                   dtype="float32", gen="randn"),
    "c2_bf16": dict(B=2, T=1024, H=64, D=8, Hv=16, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                    dtype="bfloat16", gen="randn"),
    "c3": dict(B=4, T=8192, H=64, D=2, Hv=64, Dv=16, W=256, scale=1.0, p=0.0, m=3.0,
               dtype="bfloat16", gen="repeat"),
    # packed variable-length case: 32768 tokens in sequences of 64..4096 tokens
    "c4": dict(kind="varlen", N=32768, Lmin=64, Lmax=4096, B=1, T=32768, H=32, D=16, Hv=8, Dv=32,
               W=64, scale=1.0, p=0.05, m=9.0, dtype="float16", gen="randn"),
    # batched hard inference: 64 streams x 16384 tokens x 64 heads of 32-bit symbols, forward only
    "c5": dict(kind="inference", B=64, T=16384, H=64, D=32, Hv=64, Dv=8, W=32, scale=1.0, p=0.0,
               m=3.0, dtype="float32", gen="symbols"),
    # streaming runtime: 64 slots x 16384 tokens x 64 heads of 8-bit symbols fed in chunks of 2048
    # tokens per slot to a runtime whose state stays on the GPU (the reference's RosaRuntime use)
    "stream": dict(kind="stream", B=64, T=16384, H=64, D=8, Hv=64, Dv=8, W=32, chunk=2048,
                   scale=1.0, p=0.0, m=3.0, dtype="uint8", gen="symbols"),
    # small cases for multi-pass profiler captures (scratch still larger than L2)
    "profile": dict(B=1, T=4096, H=32, D=8, Hv=8, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                    dtype="bfloat16", gen="randn"),
    "profile8k": dict(B=1, T=8192, H=32, D=8, Hv=8, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                      dtype="bfloat16", gen="randn"),
    "c3_profile": dict(B=1, T=4096, H=32, D=2, Hv=32, Dv=16, W=256, scale=1.0, p=0.0, m=3.0,
                       dtype="bfloat16", gen="repeat"),
    "c4_profile": dict(B=1, T=4096, H=32, D=16, Hv=8, Dv=32, W=64, scale=1.0, p=0.05, m=9.0,
                       dtype="float16", gen="randn"),
    # a shape outside the register-tiled kernels (symbols wider than 16 bits)
    "d24_profile": dict(B=1, T=4096, H=32, D=24, Hv=8, Dv=32, W=64, scale=1.0, p=0.05, m=9.0,
                        dtype="float16", gen="randn"),
    "c5_profile": dict(kind="inference", B=8, T=16384, H=64, D=32, Hv=64, Dv=8, W=32, scale=1.0,
                       p=0.0, m=3.0, dtype="float32", gen="symbols"),
    "stream_profile": dict(kind="stream", B=8, T=16384, H=64, D=8, Hv=64, Dv=8, W=32, chunk=2048,
                           scale=1.0, p=0.0, m=3.0, dtype="uint8", gen="symbols"),
    "small": dict(B=2, T=1024, H=8, D=8, Hv=2, Dv=8, W=128, scale=1.0, p=0.1, m=3.0,
                  dtype="bfloat16", gen="randn"),
}
SIDE_WORKLOADS = ("c2_f32", "c2_bf16", "c3", "c4", "c5", "stream")

# DRAM bytes (read + write) of one launch of the backward's second sweep per causal pair, from
# one ncu capture per kernel variant (profiles/); None where no capture backs a figure.
SWEEP2_DRAM_BYTES_PER_PAIR = {
    # vjp_sweep2_tiled_kernel<16,2,true,2> on `profile8k`: 1096.3 MB for 1073.6 M pairs
    # (profiles/vjp_sweep2_tiled__profile8k_T8192_H32.md); same kernel and controls
    "metric": 1.021, "profile8k": 1.021, "profile": 1.021, "small": 1.021, "c2_bf16": 1.021,
    # vjp_sweep2_tiled_kernel<16,4,false,2> on `c3_profile`: 215.4 MB for 268.4 M pairs (same file)
    "c3": 0.803, "c3_profile": 0.803,
    # vjp_sweep2_tiled_pair_kernel<32,8,true,1> on `c4_profile`: 437.2 MB for 268.4 M pairs (same
    # file); `c4` runs the same kernel variant on packed sequences
    "c4": 1.629, "c4_profile": 1.629,
    # no capture of the float32 variant: no figure
    "c2_f32": None,
}


def describe(name, cfg):
    what = {"inference": "batched hard inference, forward only",
            "stream": f"RosaRuntime chunked updates ({cfg.get('chunk')} tokens per slot and call), "
                      "forward only",
            "varlen": "rosa_soft_varlen fwd+bwd"}.get(cfg.get("kind"), "rosa_soft fwd+bwd")
    return (f"{name}: {what}, global B={cfg['B']} T={cfg['T']} H={cfg['H']} D={cfg['D']} "
            f"Hv={cfg['Hv']} Dv={cfg['Dv']} W={cfg['W']} p={cfg['p']} m={cfg['m']} "
            f"scale={cfg['scale']} {cfg['dtype']}")


# ---------------------------------------------------------------------------- inputs
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


def _copy_streams(rng, B, T, draw):
    """i.i.d. symbols; 10 % of the positions start a copy of an earlier window of 8..512 symbols
    into both streams, so that long matches exist."""
    k, q = draw(), draw()
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
    return q, k


def make_inference_inputs(cfg, seed, device, streams=None):
    """32-bit symbols and float32 payload of the streams `streams` (default: all)."""
    import numpy as np
    import torch

    ids = list(range(cfg["B"])) if streams is None else list(streams)
    T, H = cfg["T"], cfg["H"]
    qs, ks, ps = [], [], []
    for s in ids:          # one generator per stream: a shard draws exactly the global problem
        rng = np.random.default_rng(seed + 7919 * s)
        q, k = _copy_streams(rng, 1, T, lambda: rng.integers(0, 1 << 32, size=(1, T, H),
                                                             dtype=np.uint64).astype(np.uint32))
        qs.append(q)
        ks.append(k)
        ps.append(rng.standard_normal((1, T, cfg["Hv"], cfg["Dv"])).astype(np.float32))
    to = lambda parts: torch.from_numpy(np.concatenate(parts, 0))
    q, k, p = to(qs).view(torch.int32), to(ks).view(torch.int32), to(ps)
    return [t.to(device) if device is not None else t for t in (q, k, p)]


def make_stream_inputs(cfg, seed, device, streams=None):
    """8-bit symbols and payload symbols of the slots `streams` (default: all)."""
    import numpy as np
    import torch

    ids = list(range(cfg["B"])) if streams is None else list(streams)
    T, H = cfg["T"], cfg["H"]
    hi = 1 << cfg["D"]
    qs, ks, ps = [], [], []
    for s in ids:
        rng = np.random.default_rng(seed + 7919 * s)
        q, k = _copy_streams(rng, 1, T, lambda: rng.integers(0, hi, size=(1, T, H), dtype=np.uint8))
        qs.append(q)
        ks.append(k)
        ps.append(rng.integers(0, 1 << cfg["Dv"], size=(1, T, cfg["Hv"]), dtype=np.uint8))
    to = lambda parts: torch.from_numpy(np.concatenate(parts, 0))
    return [t.to(device) if device is not None else t for t in (to(qs), to(ks), to(ps))]


def make_dense_inputs(cfg, seed, device, dtype, batches=None, heads=None):
    """Q, K, V, grad_output of the batch elements `batches` (default: all) of the global problem,
    drawn one batch element at a time so that a shard sees exactly the values of the full run;
    `heads` = (first query head, stop) keeps only those query heads and their value heads."""
    import numpy as np
    import torch

    T, H, D, Hv, Dv = (cfg[k] for k in ("T", "H", "D", "Hv", "Dv"))
    group = H // Hv
    ids = list(range(cfg["B"])) if batches is None else list(batches)
    parts = []
    for b in ids:
        g = torch.Generator().manual_seed(seed + 104729 * b)
        if cfg["gen"] == "repeat":
            rng = np.random.default_rng(seed + 104729 * b)
            toks = np.empty((H, T), np.int64)
            for h in range(H):
                out = []
                while len(out) < T:
                    n = int(rng.integers(16, 257))
                    if out and rng.random() < 0.3 and len(out) > n:
                        s = int(rng.integers(0, len(out) - n + 1))
                        out.extend(out[s:s + n])
                    else:
                        out.extend(rng.integers(0, 1 << D, size=n).tolist())
                toks[h] = out[:T]
            bits = (toks[..., None] >> np.arange(D)) & 1            # [H,T,D]
            q = torch.from_numpy(np.where(bits, 1.0, -1.0).astype("float32")).permute(1, 0, 2)
            q = q.contiguous()
            k = q.clone()
        else:
            q = torch.randn(T, H, D, generator=g)
            k = torch.randn(T, H, D, generator=g)
        v = torch.randn(T, Hv, Dv, generator=g)
        go = torch.randn(T, H, Dv, generator=g)
        if heads is not None:
            h0, h1 = heads
            q, k, go = q[:, h0:h1], k[:, h0:h1], go[:, h0:h1]
            v = v[:, h0 // group:h1 // group]
        parts.append([t.to(dtype).contiguous() for t in (q, k, v, go)])
    out = [torch.stack([p[i] for p in parts], 0) for i in range(4)]
    return [t.to(device) if device is not None else t for t in out]


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


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ---------------------------------------------------------------------- CPU baselines
def cpu_stream_run(cfg, steps, warmup):
    """The reference's own RosaRuntime (suffix automata on the host cores, compiled from its
    source into oracle/_ref/) fed the same chunks; the oracle's one-shot matcher when that
    library is absent.  Must run in a process that has not loaded this package's extension
    (both register the class name torch.classes.rosa_soft.RosaRuntime)."""
    import numpy as np
    import torch

    sample = dict(cfg, B=min(cfg["B"], 16))
    q, k, pay = make_stream_inputs(sample, 7, None)
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
    desc = (f"{B} of the {cfg['B']} slots x T={T} x H={H} D={cfg['D']} W={cfg['W']} in chunks of "
            f"{chunk}: {what}")
    return {"value": B * T * H / sec / 1e6, "unit": "M token-heads/s", "cores": cores, "kind": kind,
            "sample": desc, "seconds": sec}


def cpu_port_run(cfg, steps, warmup):
    """Times the oracle (CPU restatement of the reference algorithm, all host threads) on a
    bounded sample of the workload.  Dense and packed workloads are timed at two sequence
    lengths so that the growth of the cost per token-head is measured, not assumed; the value
    extrapolated to the full length is reported beside the measured one."""
    import numpy as np
    import torch

    from oracle import rosa_oracle as orc

    orc.set_num_threads(host_cores())   # torchrun exports OMP_NUM_THREADS=1
    if cfg.get("kind") == "inference":
        sample = dict(cfg, B=4, T=4096, H=8, Hv=8)
        qs, ks, pay = (t.numpy() for t in make_inference_inputs(sample, 7, None))
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
        desc = (f"B={B} streams x T={T} x H={H} 32-bit symbols W={sample['W']}: quadratic "
                f"run-length matcher of the oracle (cost per token-head grows with T)")
        return {"value": B * T * H / sec / 1e6, "unit": "M token-heads/s",
                "cores": orc.num_threads(), "kind": "port", "sample": desc, "seconds": sec}

    full_T = cfg["Lmax"] if cfg.get("kind") == "varlen" else cfg["T"]
    t_hi = min(2048, full_T)
    lengths = sorted({max(64, t_hi // 2), t_hi})
    measured = []
    for T in lengths:
        sample = dict(cfg, B=1, T=T, kind="dense")
        q, k, v, go = (t.float().numpy()[0] for t in make_dense_inputs(sample, 7, None,
                                                                       torch.float32))
        cu = np.array([0, T], dtype=np.int64)
        times = []
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            orc.hard_forward(q, k, v, cu, sample["W"])
            orc.surrogate_vjp(q, k, v, go, cu, sample["W"], sample["scale"], sample["p"],
                              sample["m"], 12345)
            if it >= warmup:
                times.append(time.perf_counter() - t0)
        measured.append((T, sum(times) / len(times)))
    T, sec = measured[-1]
    H = cfg["H"]
    out = {"value": T * H / sec / 1e6, "unit": "M token-heads/s", "cores": orc.num_threads(),
           "kind": "port", "seconds": sec,
           "sample": (f"B=1 T={T} H={H} D={cfg['D']} Hv={cfg['Hv']} Dv={cfg['Dv']} W={cfg['W']} "
                      f"p={cfg['p']} m={cfg['m']} float32 values of the workload's distribution: "
                      f"oracle hard forward + surrogate VJP")}
    if len(measured) == 2:
        (t1, s1), (t2, s2) = measured
        # seconds per token-head ~ T^alpha
        alpha = math.log((s2 / t2) / (s1 / t1)) / math.log(t2 / t1)
        out["length_exponent"] = alpha
        out["measured_lengths"] = {str(t): s for t, s in measured}
        out["extrapolated_full_length_value"] = out["value"] / (full_T / T) ** alpha
        out["extrapolation"] = (f"cost per token-head ~ T^{alpha:.2f} fitted on T={t1} and T={t2}; "
                                f"value scaled to T={full_T}")
    return out


def cpu_baseline_for(name, cfg, steps=1, warmup=0):
    if cfg.get("kind") == "stream":
        # the reference runtime registers the same class name as this package's extension:
        # run it in a process of its own
        cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", name,
               "--steps", str(max(1, steps)), "--warmup", "1"]
        env = dict(os.environ)
        for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS"):
            env.pop(key, None)
        try:
            out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env).stdout
            return json.loads(out.strip().splitlines()[-1])["cpu_baseline"]
        except Exception as error:  # a missing baseline must not lose the GPU numbers
            return {"unavailable": f"{type(error).__name__}: {error}"}
    return cpu_port_run(cfg, steps, warmup)


# ------------------------------------------------------------------------ GPU cases
class Case:
    """One workload on one rank: device-resident inputs of the rank's share, the step, and the
    bookkeeping the report needs."""

    def __init__(self, name, cfg, world, rank, dev):
        import torch

        import rosa_soft_b200 as rs
        from rosa_soft_b200 import sharding

        self.name, self.cfg, self.world, self.rank, self.dev = name, cfg, world, rank, dev
        kind = cfg.get("kind", "dense")
        self.kind = kind
        self.forward_only = kind in ("inference", "stream")
        self.extra = {}
        B, T, H = cfg["B"], cfg["T"], cfg["H"]
        self.units = B * T * H                      # global token-heads per step
        kw = dict(max_suffix_length=cfg["W"], scale=cfg["scale"], dropout_p=cfg["p"],
                  mismatch_scale=cfg["m"])
        if kind in ("inference", "stream"):
            if B % world:
                raise SystemExit(f"{name}: {B} streams do not split over {world} ranks")
            per = B // world
            mine = range(rank * per, (rank + 1) * per)
            self.pairs = per * H * T * (T - 1) // 2
            self.gather_dim = 0
            self.shard_note = f"streams {mine.start}..{mine.stop - 1} of {B}"
            if kind == "inference":
                self.inputs = make_inference_inputs(cfg, 1005, dev, mine)

                def step(qs, ks, pay):
                    return list(rs.rosa_hard_inference(qs, ks, pay, max_suffix_length=cfg["W"]))
            else:
                self.inputs = make_stream_inputs(cfg, 1005, dev, mine)
                runtime = rs.RosaRuntime(H, cfg["Hv"], cfg["D"], cfg["Dv"], cfg["W"])

                def step(qs, ks, pay):
                    runtime.reset()
                    outs, ends = [], []
                    for a in range(0, T, cfg["chunk"]):
                        b = min(T, a + cfg["chunk"])
                        out, end = runtime.update_packed(qs[:, a:b], ks[:, a:b], pay[:, a:b])
                        outs.append(out)
                        ends.append(end)
                    return [torch.cat(outs, dim=1), torch.cat(ends, dim=1)]
            self.local_units = per * T * H
        elif kind == "varlen":
            dtype = getattr(torch, cfg["dtype"])
            lengths = varlen_lengths(cfg, 1004)
            owned = sharding.balance_sequences(lengths, world)
            loads = [sum(lengths[s] ** 2 for s in o) for o in owned]
            cu_list, ranges = sharding.packed_shard_offsets(lengths, owned[rank])
            full = make_dense_inputs(dict(cfg, B=1), 1004, None, dtype)
            take = lambda t: torch.cat([t[0, a:b] for a, b in ranges], 0).contiguous().to(dev) \
                if ranges else t[0, :0].contiguous().to(dev)
            self.inputs = [take(t) for t in full]
            cu = torch.tensor(cu_list, dtype=torch.int32, device=dev)
            self.pairs = H * sum(lengths[s] * (lengths[s] - 1) // 2 for s in owned[rank])
            self.local_units = sum(lengths[s] for s in owned[rank]) * H
            self.gather_dim = None                  # ragged shares: gather is not timed here
            self.extra = {"sequence_lengths": lengths,
                          "lpt_imbalance": max(loads) / (sum(loads) / world),
                          "sequences_per_rank": [len(o) for o in owned]}
            self.shard_note = (f"{len(owned[rank])} of {len(lengths)} sequences (longest-processing-"
                               f"time assignment by squared length; every ordinal kept, foreign "
                               f"sequences empty)")
            have_tokens = bool(ranges)

            def step(qq, kk, vv, gg):
                if not have_tokens:
                    return [qq, qq, kk, vv]
                for t in (qq, kk, vv):
                    t.grad = None
                    t.requires_grad_(True)
                out = rs.rosa_soft_varlen(qq, kk, vv, cu, **kw)
                out.backward(gg)
                return [out.detach(), qq.grad, kk.grad, vv.grad]
        else:
            dtype = getattr(torch, cfg["dtype"])
            shard = sharding.shard_dense(B, cfg["Hv"], world, rank)
            group = H // cfg["Hv"]
            hs = shard.head_slice(group)
            self.inputs = make_dense_inputs(cfg, 1000, dev, dtype,
                                            range(shard.batch_start, shard.batch_stop),
                                            (hs.start, hs.stop))
            nb, nh = shard.batch_stop - shard.batch_start, hs.stop - hs.start
            self.pairs = nb * nh * T * (T - 1) // 2
            self.local_units = nb * T * nh
            self.gather_dim = 0 if world <= B else None
            self.gather_heads = world > B
            self.shard_note = (f"batch elements {shard.batch_start}..{shard.batch_stop - 1}, query "
                               f"heads {hs.start}..{hs.stop - 1}")
            b_off, h_off = shard.dropout_batch_offset, shard.dropout_head_offset(group)

            def step(qq, kk, vv, gg, first_batch=0):
                # `first_batch`: position of qq[0] inside this rank's share, for callers that
                # feed the share in slices (the end-to-end pipeline below)
                for t in (qq, kk, vv):
                    t.grad = None
                    t.requires_grad_(True)
                torch.cuda.manual_seed(20240229)    # every rank draws the same dropout seed
                with sharding.dropout_coordinates(b_off + first_batch, h_off):
                    out = rs.rosa_soft(qq, kk, vv, **kw)
                    out.backward(gg)
                return [out.detach(), qq.grad, kk.grad, vv.grad]
            self.batch_elements = nb
        self.step = step

    def gather(self, results):
        """All-gather of the step's results (outputs and gradients) over the ranks: plain NCCL on
        tensors this rank owns, only when a caller wants the full tensors back."""
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return results
        out = []
        for t in results:
            parts = [torch.empty_like(t) for _ in range(self.world)]
            dist.all_gather(parts, t.contiguous())
            out.append(parts)
        return out


def time_case(case, steps, warmup, flush, dist, clocks_index=None):
    """Device time of `steps` steps (max over ranks), per-kernel times of this rank."""
    import torch

    from rosa_soft_b200 import cabi

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, warmup)):
        case.step(*case.inputs)
    barrier()
    cabi.profile_enable(True)
    cabi.profile_collect()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    sampler = ClockSampler(clocks_index) if clocks_index is not None else None
    if sampler:
        sampler.__enter__()
    barrier()
    for i in range(steps):
        flush.fill_(i)
        starts[i].record()
        case.step(*case.inputs)
        stops[i].record()
    barrier()
    if sampler:
        sampler.__exit__()
    kernels = cabi.profile_collect()
    cabi.profile_enable(False)
    total_ms = sum(s.elapsed_time(e) for s, e in zip(starts, stops))
    peak_bytes = torch.cuda.max_memory_allocated()
    t = torch.tensor([total_ms, float(peak_bytes)], dtype=torch.float64, device=case.dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"total_ms": float(t[0]), "kernels": kernels, "steps": steps,
            "clocks": sampler.summary() if sampler else None, "peak_bytes": float(t[1])}


def rooflines(case, timing, peaks, name):
    """Tensor roofline of the backward's second sweep and HBM roofline of the forward kernels,
    from this rank's per-kernel CUDA events and this rank's share of the algorithmic work."""
    cfg, kernels, steps = case.cfg, timing["kernels"], timing["steps"]
    out = {}
    if not case.forward_only and case.pairs:
        flop = (6 * cfg["D"] + 4 * cfg["Dv"]) * case.pairs
        k_ms, k_n = kernels.get("vjp_sweep2", (0.0, 0))
        tensor_peak = peaks.get("bf16_tflops_sustained")
        source = "measured (sustained bf16 cuBLAS, MEASURED_PEAKS.json)"
        if tensor_peak is None:
            tensor_peak, source = 1400.0, "fallback"
        # work of one launch over the mean launch time: a step may run the sweep once per slice
        # of the batch, so both are taken per launch (flop * steps / k_n over k_ms / k_n)
        achieved = flop * steps / (k_ms / 1e3) / 1e12 if k_n else None
        per_pair = SWEEP2_DRAM_BYTES_PER_PAIR.get(name)
        bwd_ms = sum(kernels.get(n, (0.0, 0))[0] for n in ("pack_value_bits", "vjp_sweep1",
                                                             "vjp_rowstats", "vjp_sweep2",
                                                             "vjp_finalize")) / steps
        out["roofline"] = {
            "bound": "tensor", "kernel": "vjp_sweep2", "achieved": achieved, "peak": tensor_peak,
            "unit": "TFLOP/s", "frac": (achieved / tensor_peak) if achieved else None,
            "traffic": per_pair * case.pairs * steps / k_n if per_pair and k_n else None,
            "peak_source": source,
            "kernel_ms": (k_ms / k_n) if k_n else None,
            "launches_per_step": (k_n / steps) if steps else None,
            "whole_backward_tflops": flop / (bwd_ms / 1e3) / 1e12 if bwd_ms else None,
            "note": "algorithmic contraction work (6D+4Dv FLOP per causal pair of this rank) over "
                    "the kernel's mean launch time; the kernel is bound by CUDA-core issue (ALU "
                    "pipe), not by the tensor pipe"}
    s = 2 if cfg["dtype"] not in ("float32",) else 4
    per_unit = (80 if case.kind == "inference" else 12 if case.kind == "stream" else
                2 * cfg["D"] * s + cfg["Dv"] * s * cfg["Hv"] / cfg["H"] + cfg["Dv"] * s + 8)
    names = ("pack_symbols", "transpose_symbols", "build_match_masks", "hard_match",
             "hard_match_hashed", "gather_output", "inference_finish", "stream_prepare",
             "stream_append", "stream_match", "stream_finish")
    fwd_ms = sum(kernels.get(n, (0.0, 0))[0] for n in names) / steps
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    gbs = per_unit * case.local_units / (fwd_ms / 1e3) / 1e9 if fwd_ms else None
    out["roofline_forward"] = {
        "bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
        "frac": (gbs / hbm_peak) if gbs else None, "forward_ms": fwd_ms,
        "bytes_per_token_head": per_unit,
        "kernels": ("stream_prepare+append+match+finish" if case.kind == "stream" else
                    "pack_symbols+build_match_masks+hard_match(+hashed)+gather_output")}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="metric", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only-headline", action="store_true",
                    help="skip the `workloads` map (other benchmark configurations)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    forward_only = cfg.get("kind") in ("inference", "stream")
    metric = "forward M token-heads/s" if forward_only else "fwd+bwd M token-heads/s"

    if args.impl == "reference":
        if rank != 0:
            return
        if cfg.get("kind") == "stream":
            base = cpu_stream_run(cfg, max(1, args.steps), max(0, min(args.warmup, 1)))
        else:
            base = cpu_port_run(cfg, max(1, args.steps), max(0, min(args.warmup, 1)))
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": base["value"],
            "unit": "M token-heads/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": base["seconds"] * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "u8 symbols" if cfg.get("kind") == "stream" else "f64", "data": "synthetic",
            # the configuration this arm REALLY ran: a bounded sample of the GPU arm's workload
            "config": {"workload": f"CPU sample of {args.workload}: " + base["sample"],
                       "full_workload": describe(args.workload, cfg),
                       "parallelism": f"{base['cores']} host threads, no GPU"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "M token-heads/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
        }))
        return

    import torch

    import rosa_soft_b200  # noqa: F401  (fails loudly without the CUDA extension)

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (the package has no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- headline workload: device-resident timing
    case = Case(args.workload, cfg, world, rank, dev)
    torch.cuda.reset_peak_memory_stats()
    timing = time_case(case, args.steps, args.warmup, flush, dist, clocks_index=local_rank)
    total_ms = timing["total_ms"]

    # ---- the same steps followed by an all-gather of outputs and gradients (on request only)
    gather_ms = None
    if world > 1 and (case.gather_dim is not None or getattr(case, "gather_heads", False)):
        case.gather(case.step(*case.inputs))
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            case.gather(case.step(*case.inputs))
        g1.record()
        barrier()
        t = torch.tensor([g0.elapsed_time(g1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_ms = float(t[0]) / args.steps

    # ---- end to end: pinned host buffers in, results out, inside the timed region
    host = [t.detach().cpu().pin_memory() for t in case.inputs]
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in case.step(*case.inputs)]
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_stop = torch.cuda.Event(enable_timing=True)

    def e2e_serial():
        device_inputs = [h.to(dev, non_blocking=True) for h in host]
        for dst, src in zip(host_out, case.step(*device_inputs)):
            dst.copy_(src, non_blocking=True)

    # Dense workloads: batch elements are independent, so the caller's copies overlap the
    # operator: the share goes through the public operator in slices of `per` batch elements, the
    # host-to-device copy of slice c + 1 and the device-to-host copy of slice c - 1 on streams of
    # their own while slice c computes (dropout coordinates carry the slice's batch position, so
    # the results are those of the unsliced call).
    nb = getattr(case, "batch_elements", 0)
    per = 2 if nb >= 4 else 1
    slices = [(a, min(nb, a + per)) for a in range(0, nb, per)]
    pipelined = len(slices) >= 2
    if pipelined:
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        staging = [[torch.empty((per,) + tuple(h.shape[1:]), dtype=h.dtype, device=dev)
                    for h in host] for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in slices]
        ev_free = [None, None]                       # compute that last read a staging set

    def e2e_pipelined():
        def copy_in(c):
            a, b = slices[c]
            with torch.cuda.stream(s_in):
                if ev_free[c % 2] is not None:
                    s_in.wait_event(ev_free[c % 2])
                for dst, h in zip(staging[c % 2], host):
                    dst[:b - a].copy_(h[a:b], non_blocking=True)
                ev_in[c].record(s_in)

        s_in.wait_stream(main)
        copy_in(0)
        for c, (a, b) in enumerate(slices):
            if c + 1 < len(slices):
                copy_in(c + 1)
            main.wait_event(ev_in[c])
            results = case.step(*[t[:b - a] for t in staging[c % 2]], first_batch=a)
            done = torch.cuda.Event()
            done.record(main)
            ev_free[c % 2] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(host_out, results):
                    src.record_stream(s_out)
                    dst[a:b].copy_(src, non_blocking=True)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    e2e_step = e2e_pipelined if pipelined else e2e_serial
    e2e_how = (f"public operator on {len(slices)} slices of {per} batch element(s) per rank, "
               f"host copies of neighbouring slices overlapped on two copy streams; output checked "
               f"bit-equal and gradients to two ulps of their dtype against the unsliced call" if pipelined else
               "one public-operator call per step, copies and compute on one stream")
    e2e_step()
    if pipelined:
        # The sliced pipeline must reproduce the unsliced call: the output bit for bit; the
        # gradients up to the grouping of their fixed-order partial sums, which follows the
        # number of work items and so the batch size of a call (a few float32 ulps before the cast).
        torch.cuda.synchronize(dev)
        for idx, (got, want) in enumerate(zip(host_out, case.step(*case.inputs))):
            want = want.cpu()
            if idx == 0:
                same = torch.equal(got, want)
            else:
                # gradients come back in the input dtype: allow two of its ulps
                rtol = {torch.bfloat16: 2e-2, torch.float16: 2e-3}.get(got.dtype, 1e-4)
                same = torch.allclose(got.float(), want.float(), rtol=rtol,
                                      atol=1e-5 * float(want.float().abs().max()))
            if not same:
                err = float((got.float() - want.float()).abs().max())
                raise SystemExit(f"end-to-end pipeline: result {idx} differs from the unsliced call "
                                 f"(max abs difference {err:.3e})")
    barrier()
    e2e_start.record()
    for _ in range(args.steps):
        e2e_step()
    e2e_stop.record()
    barrier()
    t = torch.tensor([e2e_start.elapsed_time(e2e_stop)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0])
    h2d = sum(h.numel() * h.element_size() for h in host)
    d2h = sum(h.numel() * h.element_size() for h in host_out)
    io = torch.tensor([h2d, d2h], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(io, op=dist.ReduceOp.SUM)
    h2d, d2h = (int(x) for x in io.tolist())
    head_roof = rooflines(case, timing, peaks, args.workload)
    head_extra, head_note, head_units = case.extra, case.shard_note, case.units
    del host, host_out, case
    torch.cuda.empty_cache()

    # ---- the other benchmark configurations, same method, fewer steps
    side = {}
    if args.workload == "metric" and not args.only_headline:
        for name in SIDE_WORKLOADS:
            scfg = WORKLOADS[name]
            try:
                c = Case(name, scfg, world, rank, dev)
                tm = time_case(c, 3, 3, flush, dist)
                entry = {"config": describe(name, scfg), "ms_per_step": tm["total_ms"] / tm["steps"],
                         "value": c.units * tm["steps"] / (tm["total_ms"] / 1e3) / 1e6,
                         "unit": "M token-heads/s", "steps": tm["steps"], "warmup": 3,
                         "rank0_share": c.shard_note,
                         "kernel_ms_per_step": {n: ms / tm["steps"]
                                                for n, (ms, _) in sorted(tm["kernels"].items())}}
                entry.update(rooflines(c, tm, peaks, name))
                entry.update(c.extra)
                side[name] = entry
                del c
            except Exception as error:   # one workload must not lose the headline line
                side[name] = {"error": f"{type(error).__name__}: {error}"}
            torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    kernels = timing["kernels"]
    result = {
        "metric": metric,
        "value": head_units * args.steps / (total_ms / 1e3) / 1e6,
        "unit": "M token-heads/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("u8 symbols" if cfg.get("kind") == "stream" else
                  "f32 accumulate on " + cfg["dtype"] + " inputs; integer symbols"),
        "data": "synthetic",
        "config": {"workload": describe(args.workload, cfg),
                   "global_batch": cfg["B"], "seq_len": cfg["T"],
                   "parallelism": (f"one fixed global problem split over {world} rank(s) into "
                                   f"independent units, no collective in the operator; rank 0: "
                                   f"{head_note}"),
                   "l2": "flushed between timed steps by writing a 512 MiB buffer; the step's own "
                         "checkpoint/partial scratch is larger than L2",
                   **head_extra},
        "clocks": timing["clocks"],
        "e2e": {"value": head_units * args.steps / (e2e_ms / 1e3) / 1e6, "unit": "M token-heads/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": e2e_how},
        "gpu_launches": sum(n for _, n in kernels.values()) * world,
        "peak_device_bytes": timing["peak_bytes"],
        "kernel_ms_per_step": {n: ms / args.steps for n, (ms, _) in sorted(kernels.items())},
    }
    result.update(head_roof)
    if gather_ms is not None:
        result["gather"] = {"ms_per_step_with_gather": gather_ms,
                            "ms_per_step_without": total_ms / args.steps,
                            "what": "NCCL all_gather of the step's output and three gradients "
                                    "over the ranks, after the operator; not part of `value`"}
    if side:
        result["workloads"] = side
    if not args.no_cpu_baseline and world == 1:   # the CPU baselines are reported at N=1 only
        result["cpu_baseline"] = cpu_baseline_for(args.workload, cfg)
        if side and "stream" in side and "error" not in side["stream"]:
            side["stream"]["cpu_baseline"] = cpu_baseline_for("stream", WORKLOADS["stream"])
    print(json.dumps(result))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
