"""Benchmark of the TPA forward hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c0..c4]

N = 1 runs the headline configuration (c2: bf16 causal B=1 T=32768 h=32 d=128 R 12/4/4)
through tpa_fwd on one GPU.  N > 1 (under torchrun, one rank per GPU) runs the ring
configuration (c3: bf16 causal B=1 T=131072 h=32 d=128 R 6/2/2) over contiguous length
shards.  One step = one forward pass over the whole batch.  Rank 0 prints one JSON line.

`value` is algorithmic attention TFLOP/s (4*B*h*d*pairs / time; pairs = T(T+1)/2 causal),
tokens/s is reported beside it.  `e2e` is the same quantity through the public
tpa_b200.tpa.tpa() call on pinned host arrays (host<->device copies inside the timing).
`--impl reference` times the CPU oracle (a restatement of the reference's math; the
reference itself needs jax, which is not installed) on the host cores instead.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tensor-product-attention-jax_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

# name: (dtype, B, T, h, d, Rq, Rk, causal)
WORKLOADS = {
    "c0": ("f32", 1, 512, 8, 64, 6, 2, True),
    "c1": ("bf16", 4, 4096, 32, 128, 6, 2, True),
    "c2": ("bf16", 1, 32768, 32, 128, 12, 4, True),
    "c3": ("bf16", 1, 131072, 32, 128, 6, 2, True),
    "c4": ("bf16", 8, 2048, 16, 64, 8, 8, False),
}
METRIC = "TPA forward throughput (algorithmic attention FLOPs 4*B*h*d*pairs per second; tokens/s beside it)"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture
# summarised in profiles/tpa_fwd_sm100_staged_c2_T8192.md: taken on the T = 8192 case of the c2 shape
# (305.8 MB read + 62.9 MB written) and scaled by the sequence length, with which every byte the
# attention kernel moves grows in proportion (see profiles/c2_launch_list.md).
NCU_T8192_BYTES = 305767424 + 62907648


def ncu_traffic(name, t):
    """Scaled DRAM traffic per attention launch, for the shape the capture was taken on only."""
    return NCU_T8192_BYTES * t // 8192 if name.split("@")[0] == "c2" else None


def flops(b, t, h, d, causal):
    pairs = t * (t + 1) // 2 if causal else t * t
    return 4.0 * b * h * d * pairs


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        return m["bf16_tflops"], m.get("bf16_tflops_sustained"), m["hbm_gbs"], "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 1400.0, 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def wait_first(self, timeout=5.0):
        """Block until nvidia-smi has delivered its first sample (it takes a moment to start)."""
        t0 = time.perf_counter()
        while not self.rows and time.perf_counter() - t0 < timeout and self.proc is not None:
            time.sleep(0.02)

    def mark(self):
        return len(self.rows)

    def summary(self, start=0, end=None):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows[start:end]:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(name, device, shard=None, seed=0):
    """Seeded synthetic factors with the configuration's shapes and distributions
    (A ~ N(0,1), B ~ N(0,1)/sqrt(d)), in the reference's concatenated layout."""
    dt, b, t, h, d, rq, rk, causal = WORKLOADS[name]
    dtype = torch.float32 if dt == "f32" else torch.bfloat16
    g = torch.Generator(device=device).manual_seed(1000 + seed)
    def fac(r):
        x = torch.randn((b, t, r, h + d), generator=g, device=device, dtype=torch.float32)
        x[..., h:] *= d**-0.5
        return x.to(dtype)
    q, k, v = fac(rq), fac(rk), fac(rk)
    if shard is not None:
        rank, n = shard
        per = t // n
        q, k, v = (x[:, rank * per:(rank + 1) * per].contiguous() for x in (q, k, v))
    return q, k, v


def host_threads(share=1):
    """Use every host core this process may run on (torchrun exports OMP_NUM_THREADS=1); with
    `share` > 1 the cores are divided among that many ranks working at the same time -- eight
    processes each spinning a full team of OpenMP threads on the same cores take minutes for
    what is seconds of work."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n // max(1, share)))
    return torch.get_num_threads()


_T0 = time.perf_counter()


def progress(msg):
    """Rank 0's progress on stderr (where a run that does not finish stopped)."""
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"[bench {time.perf_counter() - _T0:7.1f}s] {msg}", file=sys.stderr, flush=True)


def config_for(name, world, mask_mode, lq=None):
    """The workload description; identical for the b200 and the reference arm."""
    dtn, b, t, h, d, rq, rk, causal = WORKLOADS[name]
    ring = world > 1
    return {"workload": name + (f"@lq{lq}" if lq is not None else ""),
            "shape": f"B{b} T{t} h{h} d{d} R{rq}/{rk}/{rk} causal={causal}"
                     + (f", last {lq} query rows" if lq is not None else ""),
            "parallelism": f"ring sp{world} ({mask_mode} causal mask)" if ring else "single GPU",
            "l2": "inputs + outputs larger than L2 (no flush needed)" if name.split("@")[0] in ("c1", "c2", "c3")
                  else "smaller than L2, not flushed"}


def cpu_sample(name, n_rows):
    """Bounded CPU sample of a workload: `n_rows` evenly spaced query rows against all keys,
    which for a causal workload has the whole job's mean cost per token.  Blocks of >= 1024 rows
    keep the per-head matrix products large enough for the host BLAS to thread."""
    import numpy as np
    from oracle import tpa_oracle as orc

    dt, b, t, h, d, rq, rk, causal = WORKLOADS[name]
    q, k, v = orc.make_factors(2, b, t, t, rq, rk, h, d, d)
    n = min(n_rows, t)
    rows = torch.from_numpy(np.linspace(0, t - 1, n).round().astype(np.int64))
    tq, tk, tv = (torch.from_numpy(x) for x in (q, k, v))
    if dt == "bf16":
        tq, tk, tv = (x.bfloat16().float() for x in (tq, tk, tv))
    fl = 4.0 * b * h * d * float(((rows + 1) if causal else torch.full_like(rows, t)).sum())
    run = lambda: orc.tpa_reference_torch(tq, tk, tv, h, sm_scale=d**-0.5, causal=causal, rows=rows)  # noqa: E731
    return run, fl, b * n, f"{n} evenly spaced query rows of {name} against all {t} keys, torch fp32, {torch.get_num_threads()} threads"


def calibrate_rows(name, seconds_per_step):
    """Number of sample rows whose oracle run takes about `seconds_per_step` on this host
    (one untimed probe of 256 rows; at least 256, at most 4096 rows)."""
    run, _, _, _ = cpu_sample(name, 256)
    t0 = time.perf_counter()
    run()
    probe = time.perf_counter() - t0
    n = int(256 * seconds_per_step / max(probe, 1e-3))
    return max(256, min(4096, n // 256 * 256))


def time_cpu(name, steps, warmup, n_rows):
    run, fl, toks, sample = cpu_sample(name, n_rows)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    return fl / dt / 1e12, toks / dt, dt, sample


def reference_arm(args, name, world):
    """The CPU arm: the oracle port on all host threads, exactly --steps timed and --warmup untimed
    steps, each step a sample of the workload sized so that the whole run takes about two minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    steps, warmup = args.steps, args.warmup
    n_rows = calibrate_rows(name, 120.0 / max(1, steps + warmup))
    tf, toks, dt, sample = time_cpu(name, steps, warmup, n_rows)
    dtn = WORKLOADS[name][0]
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "tokens_per_s": toks,
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": config_for(name, world, args.mask_mode),
        "note": "CPU oracle (restatement of the reference math); the reference itself needs jax, which is not "
                f"installed: reference on the JAX CPU backend unavailable on this box.  Workload dtype {dtn}, oracle in fp32.",
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------- parity of the timed output


def _sample_rows(t, n_random, seed):
    fixed = [0, 1, 2, 3, t - 4, t - 3, t - 2, t - 1]
    rnd = torch.randperm(t, generator=torch.Generator().manual_seed(seed))[:n_random].tolist()
    return torch.tensor(sorted(set(r for r in fixed + rnd if 0 <= r < t)))


def _bounds(dtn):
    # the tolerances of the benchmark: fp32 max-abs 1e-5; bf16 max-abs 2e-2 and mean-abs 5e-3
    return (1e-5, 1e-5) if dtn == "f32" else (2e-2, 5e-3)


def parity_single(o, q, k, v, h, d, causal, q_off, dtn, n_rows=64):
    """Sampled rows of the output the timed loop just produced against the CPU oracle."""
    from oracle import tpa_oracle as orc

    lq = q.shape[1]
    rows = _sample_rows(lq, n_rows, 7)
    f = lambda x: x.float().cpu()  # noqa: E731
    ref = orc.tpa_reference_torch(f(q), f(k), f(v), h, sm_scale=d**-0.5, causal=causal, rows=rows, q_offset=q_off)
    diff = (f(o)[:, rows] - ref).abs()
    mx, mean = float(diff.max()), float(diff.mean())
    bmax, bmean = _bounds(dtn)
    return {"max_abs": mx, "mean_abs": mean, "rows": int(len(rows)), "bound_max_abs": bmax, "bound_mean_abs": bmean,
            "against": "CPU oracle, sampled query rows of the last timed step, all heads",
            "ok": bool(mx <= bmax and mean <= bmean and not torch.isnan(f(o)[:, rows]).any())}


def parity_ring(o, q, k_full, v_full, h, d, causal, mask_mode, rank, world, dtn, n_rows=32):
    """This rank's sampled output rows against the ring definition computed directly on the CPU:
    every key shard contributes a block result under its own mask (shard-local triangle for
    "reference_local", tpa/ring_tpa.py:73-79; global positions for "global"), merged with the
    LSE weights of tpa/ring_tpa.py:82-91."""
    from oracle import tpa_oracle as orc

    lq = q.shape[1]
    rows = _sample_rows(lq, n_rows, 11 + rank)
    f = lambda x: x.float().cpu()  # noqa: E731
    fq, fk, fv = f(q), f(k_full), f(v_full)
    per = fk.shape[1] // world
    parts = []
    for s in range(world):
        sl = slice(s * per, (s + 1) * per)
        offs = (rank * lq, s * per) if mask_mode == "global" else (0, 0)
        if causal and mask_mode == "global" and s > rank:
            continue
        parts.append(orc.tpa_reference_torch(fq, fk[:, sl], fv[:, sl], h, sm_scale=d**-0.5, causal=causal, rows=rows,
                                             q_offset=offs[0], k_offset=offs[1], return_lse=True))
    lse = torch.stack([p[1] for p in parts])            # [steps, b, rows, h]
    tot = torch.logsumexp(lse, dim=0)
    w = torch.exp(lse - tot).unsqueeze(-1)
    ref = (torch.nan_to_num(torch.stack([p[0] for p in parts])) * w).sum(0)
    diff = (f(o)[:, rows] - ref).abs()
    return float(diff.max()), float(diff.mean()), int(len(rows))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--mask-mode", default="reference_local", choices=["reference_local", "global"])
    ap.add_argument("--kernel", default="auto", choices=["auto", "simt", "sm100", "sm100_fused", "sm100_staged"])
    ap.add_argument("--seq-len", type=int, default=None,
                    help="override T of the workload (profiling on a small case; not a headline number)")
    ap.add_argument("--pass", dest="which", default="fwd", choices=["fwd", "bwd"],
                    help="bwd: time tpa_bwd on the forward's results instead (single GPU; 2.5x the forward's "
                         "algorithmic FLOPs: five tile GEMMs instead of two); not the headline metric")
    ap.add_argument("--lq", type=int, default=None,
                    help="keep only the last LQ query rows of the workload (decode shapes against the whole "
                         "key/value factor cache; single GPU, forward; reports the factor stream against the "
                         "HBM roof; not the headline metric)")
    ap.add_argument("--graph", action="store_true",
                    help="capture one step in a CUDA graph and time its replays (single GPU): what a serving "
                         "loop does for launch-bound shapes such as --lq 1")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed output")
    ap.add_argument("--no-n1", action="store_true",
                    help="N > 1: skip timing the unsharded workload on rank 0's GPU (ring_efficiency)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    name = args.workload or ("c2" if world == 1 else "c3")
    if args.seq_len is not None:
        w = list(WORKLOADS[name])
        w[2] = args.seq_len
        name = f"{name}@T{args.seq_len}"
        WORKLOADS[name] = tuple(w)
    if args.impl == "reference":
        return reference_arm(args, name, world)

    import torch.distributed as dist
    import tpa_b200
    from tpa_b200 import _capi

    assert torch.cuda.is_available(), "bench.py needs a GPU (no CPU path exists)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    dtn, b, t, h, d, rq, rk, causal = WORKLOADS[name]
    sm_scale = d**-0.5
    ring = world > 1
    q, k, v = make_inputs(name, device, shard=(rank, world) if ring else None)
    ids = torch.zeros((b, q.shape[1]), dtype=torch.int32, device=device) if ring else None
    bwd = args.which == "bwd"
    q_off = 0
    if args.lq is not None:
        assert not ring and not bwd and 0 < args.lq <= t, "--lq is a single-GPU forward measurement"
        q_off = t - args.lq
        q = q[:, q_off:].contiguous()
    if bwd:
        assert not ring, "--pass bwd is a single-GPU measurement"
        o_fwd, lse_fwd = tpa_b200.tpa.fwd_device(q, k, v, h, None, None, sm_scale, causal)
        gen = torch.Generator(device=device).manual_seed(1234)
        d_o = torch.randn(o_fwd.shape, generator=gen, device=device, dtype=torch.float32).to(q.dtype)
        grads = tuple(torch.empty_like(x) for x in (q, k, v))

    def step():
        if bwd:  # the backward knows "auto", "simt" and "sm100"
            return tpa_b200.tpa.bwd_device(q, k, v, h, None, None, sm_scale, causal, o_fwd, lse_fwd, d_o,
                                           out=grads, kernel=args.kernel.split("_")[0])
        if ring:
            return tpa_b200.ring_tpa.ring_tpa(q, k, v, ids, ids, None, h, sm_scale=sm_scale, causal=causal,
                                              mask_mode=args.mask_mode)
        buf = outs[calls[0] % 2]
        calls[0] += 1
        return tpa_b200.tpa.fwd_device(q, k, v, h, None, None, sm_scale, causal, q_offset=q_off, kernel=args.kernel,
                                       out=buf[0], lse=buf[1])[0]

    calls = [0]
    if not ring and not bwd:  # two result buffers used in turn: no allocator work inside the timed region
        outs = [(torch.empty((b, q.shape[1], h, d), dtype=q.dtype, device=device),
                 torch.empty((b, q.shape[1], h), dtype=torch.float32, device=device)) for _ in range(2)]

    if args.graph:
        assert not ring, "--graph is a single-GPU measurement"
        eager_step = step
        side = torch.cuda.Stream(device)
        with torch.cuda.stream(side):  # warm up on the capture stream: scratch buffers get allocated here
            for _ in range(3):
                eager_step()
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        n_cap = _capi.lib.tpa_launch_count()
        with torch.cuda.graph(graph, stream=side):
            graph_out = eager_step()
        launches_per_replay = _capi.lib.tpa_launch_count() - n_cap  # kernels recorded in the graph

        def step():
            graph.replay()
            return graph_out

    def sync():
        torch.cuda.synchronize(device)
        if ring:
            dist.barrier()
            torch.cuda.synchronize(device)

    progress(f"inputs ready ({name}, {world} GPU(s)); warm-up and timed steps")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local_rank) as clocks:
        clocks.wait_first()
        # the sampler ticks every 100 ms: keep the GPU under this load for at least 0.5 s before
        # the timed steps so that the clocks reported are the ones the kernel runs at
        c_start = clocks.mark()
        sync()
        t0 = time.perf_counter()
        step()
        sync()
        t1 = torch.tensor([time.perf_counter() - t0], device=device)
        if ring:
            dist.all_reduce(t1, op=dist.ReduceOp.MAX)  # every rank must run the same number of steps
        n_warm = max(args.warmup - 1, min(200, int(0.5 / max(float(t1.item()), 1e-4)) + 1))
        for i in range(n_warm):
            step()
            if i % 4 == 3:
                torch.cuda.synchronize(device)
        sync()
        n0 = _capi.lib.tpa_launch_count()
        gc.collect()
        gc.disable()  # no collector pause between the launches of the timed region
        ev[0].record()
        last = None
        for i in range(args.steps):
            last = step()
            ev[i + 1].record()
        sync()
        gc.enable()
        launches = _capi.lib.tpa_launch_count() - n0
        if args.graph:
            launches = launches_per_replay * args.steps
        time.sleep(0.12)  # let the sample that covers the end of the timed region arrive
        clock_summary = clocks.summary(c_start)
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    if ring:
        tt = torch.tensor([total_ms], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    ms = total_ms / args.steps
    fl = flops(b, t, h, d, causal) * (2.5 if bwd else 1.0)
    if args.lq is not None:  # the last lq rows: each sees its own prefix (causal) or every key
        lq = args.lq
        fl = 4.0 * b * h * d * (lq * (t - lq) + lq * (lq + 1) // 2 if causal else lq * t)
    value = fl / (ms * 1e-3) / 1e12
    toks = b * t / (ms * 1e-3)

    # ------------------------------------------------------------- configuration 4's dense-attention arm
    dense_arm = None
    if name.split("@")[0] == "c4" and not ring and not bwd and args.lq is None:
        # the same Q, K, V materialised (fp32 rank mean of the bf16 factors, one bf16 rounding -- what the
        # staging kernel produces) and run as dense attention through the library's mha(), timed the same way
        def dense(x, r_):
            xf = x.float()
            return (torch.einsum("blrh,blrd->blhd", xf[..., :h], xf[..., h:]) / r_).to(q.dtype)

        mq, mk, mv = dense(q, rq), dense(k, rk), dense(v, rk)
        run_dense = lambda: tpa_b200.mha.mha(mq, mk, mv, sm_scale=sm_scale, causal=causal)  # noqa: E731
        od = run_dense()
        for _ in range(max(args.warmup, 3)):
            run_dense()
        torch.cuda.synchronize(device)
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(args.steps):
            run_dense()
        d1.record()
        torch.cuda.synchronize(device)
        d_ms = d0.elapsed_time(d1) / args.steps
        fo = last if not isinstance(last, tuple) else last[0]
        dense_arm = {"ms_per_step": d_ms, "value": fl / (d_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "max_abs_vs_factored": float((od.float() - fo.float()).abs().max()),
                     "what": "mha() of tpa/mha.py:10-37 on the materialised Q, K, V: the same kernels with "
                             "one-hot head factors of rank h; the difference to the factored call is the staging pass"}
        del mq, mk, mv, od

    # ------------------------------------------------------------- end to end on pinned host arrays
    e2e = None
    if not args.no_e2e and not bwd and args.lq is None:
        progress(f"timed steps done ({ms:.3f} ms/step); end to end on pinned host arrays")
        hq, hk, hv = (x.cpu().pin_memory() for x in (q, k, v))
        hid = ids.cpu().pin_memory() if ring else None
        out_host = torch.empty((b, q.shape[1], h, d), dtype=q.dtype).pin_memory()

        def e2e_step():
            if not ring:
                # the public call on host arrays: it moves the factors up and the result down itself,
                # overlapped with its kernels; returns when the result is in out_host
                tpa_b200.tpa.tpa(hq, hk, hv, num_heads=h, sm_scale=sm_scale, causal=causal, out=out_host)
                return
            dq, dk, dv_ = (x.to(device, non_blocking=True) for x in (hq, hk, hv))
            did = hid.to(device, non_blocking=True)
            o = tpa_b200.ring_tpa.ring_tpa(dq, dk, dv_, did, did, None, h, sm_scale=sm_scale, causal=causal,
                                           mask_mode=args.mask_mode)
            out_host.copy_(o, non_blocking=True)

        n_e2e = max(2, min(args.steps, 5))
        e2e_step()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        sync()
        e_ms = e0.elapsed_time(e1) / n_e2e
        e2e_diff = None
        if not ring:  # the host-array call against the device call timed above (same rows, same tiles)
            dev_o = (last if not isinstance(last, tuple) else last[0]).float().cpu()
            e2e_diff = float(torch.nan_to_num(out_host.float() - dev_o).abs().max())
        if ring:
            tt = torch.tensor([e_ms], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e_ms = float(tt.item())
        h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv)) + (hid.numel() * 4 if ring else 0)
        e2e = {"value": fl / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "tokens_per_s": b * t / (e_ms * 1e-3),
               "ms_per_step": e_ms, "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": out_host.numel() * out_host.element_size() * world,
               "max_abs_vs_device_call": e2e_diff,
               "call": "ring_tpa on device tensors between explicit copies" if ring else
                       "tpa() on pinned host arrays (copies inside the call, overlapped with its kernels)"}

    # ------------------------------------------------------------- parity of what was just timed
    parity = None
    if not args.no_parity and not bwd:
        progress("parity check of the timed output")
        host_threads(share=world)
        if ring:
            kf = [torch.empty_like(k) for _ in range(world)]
            vf = [torch.empty_like(v) for _ in range(world)]
            dist.all_gather(kf, k)
            dist.all_gather(vf, v)
            mx, mean, nrows = parity_ring(last, q, torch.cat(kf, 1), torch.cat(vf, 1), h, d, causal, args.mask_mode,
                                          rank, world, dtn, n_rows=max(8, 64 // world))
            del kf, vf
            agg = torch.tensor([mx, mean], device=device)
            dist.all_reduce(agg, op=dist.ReduceOp.MAX)
            bmax, bmean = _bounds(dtn)
            mx, mean = float(agg[0]), float(agg[1])
            parity = {"max_abs": mx, "mean_abs": mean, "rows": nrows * world, "bound_max_abs": bmax,
                      "bound_mean_abs": bmean,
                      "against": f"CPU ring oracle ({args.mask_mode} mask over all {world} key shards), {nrows} sampled rows "
                                 "of every rank's last timed output, all heads; max over ranks",
                      "ok": bool(mx <= bmax and mean <= bmean)}
        else:
            parity = parity_single(last if not isinstance(last, tuple) else last[0], q, k, v, h, d, causal, q_off, dtn)

    # ------------------------------------------------------------- same-box single-GPU time of the ring workload
    n1_ms = None
    if ring and not args.no_n1:
        progress("the unsharded workload on rank 0's GPU")
        if rank == 0:
            fq, fk, fv = make_inputs(name, device)
            fid = torch.zeros((b, t), dtype=torch.int32, device=device)
            # one shard = the whole sequence: the ring's only step is the plain causal forward
            run1 = lambda: tpa_b200.tpa.fwd_device(fq, fk, fv, h, fid, fid, sm_scale, causal, want_lse=False)  # noqa: E731
            run1()
            torch.cuda.synchronize(device)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(3):
                run1()
            a1.record()
            torch.cuda.synchronize(device)
            n1_ms = a0.elapsed_time(a1) / 3
            del fq, fk, fv
        dist.barrier()

    # ------------------------------------------------------------- where a ring step's time goes (rank 0's view)
    breakdown = None
    if ring and args.mask_mode == "reference_local":
        progress("breakdown of a ring step")
        from tpa_b200 import ring_tpa as _ring
        _ring._timing = []
        for _ in range(3):
            step()
        sync()
        recs, _ring._timing = _ring._timing, None
        if recs:
            med = lambda i: statistics.median(r["events"][i].elapsed_time(r["events"][i + 1]) for r in recs)  # noqa: E731
            own, hops, rest = med(0), med(1), med(2)
            rq, kbuf, vbuf, rqs, sbuf, state = recs[-1]["operands"]
            n_rest = world - 1
            kk, vv, ss = (kbuf, vbuf, sbuf) if n_rest > 1 else (kbuf[0], vbuf[0], sbuf[0])
            # the second call again on the tiles the last step staged: what remains is its staging pass
            only = lambda: tpa_b200.tpa.fwd_device(rq, kk, vv, h, rqs, ss, sm_scale, causal, want_lse=False,  # noqa: E731
                                                   kv_parts=n_rest, per_part=causal and n_rest > 1, state=state,
                                                   load_state=True, reuse_staged_q=True, reuse_staged_kv=True)
            only()
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            for _ in range(3):
                only()
            b1.record()
            torch.cuda.synchronize(device)
            attn = b0.elapsed_time(b1) / 3
            breakdown = {"own_shard_call_ms": own, "exposed_wait_for_hops_ms": hops, "visiting_shards_call_ms": rest,
                         "of_which_staging_ms": max(rest - attn, 0.0), "of_which_attention_ms": attn,
                         "note": "rank 0, medians of 3 steps.  All N-1 hops are queued at entry on a side stream and "
                                 "travel while the first call (Q tiles, own K/V shard, its attention) runs; the "
                                 "second call rebuilds the N-1 visiting shards as tiles and attends to them, "
                                 "starting from the first call's partial (o, lse)"}
            del recs
        dist.barrier()

    if rank != 0:
        if ring:
            dist.destroy_process_group()
        return

    burst, sustained, hbm, src = peaks()
    info = tpa_b200.tpa.query_kernel(q, k, v, h, kernel=args.kernel, causal=causal, segments=ring)
    # the dominant (only) kernel of a step; at N > 1 every rank runs `world` launches per step
    kernel_ms = statistics.median(per_step) / (world if ring else 1)
    fl_launch = fl / (world * world) if ring else fl
    achieved = fl_launch / (kernel_ms * 1e-3) / 1e12
    if bwd:
        info = dict(info, kernel="bwd:" + ("simt" if args.kernel == "simt" or info["kernel"] == "simt" else "sm100"))
    roofline = {"bound": "tensor", "achieved": achieved, "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst,
                "frac_of_sustained": achieved / sustained if sustained else None, "peak_source": src,
                "traffic": None if bwd else ncu_traffic(name, t), "kernel": info["kernel"],
                "hbm_algorithmic_bytes": sum(x.numel() * x.element_size() for x in (q, k, v))
                + b * q.shape[1] * h * d * q.element_size() + b * q.shape[1] * h * 4,
                "hbm_peak_gbs": hbm}
    if args.lq is not None:
        # few rows against a long cache: the roof is the K/V factor stream, not the tensor pipe
        stream = sum(x.numel() * x.element_size() for x in (q, k, v)) + b * args.lq * h * d * q.element_size()
        gbs = stream / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "peak_source": src,
                    "traffic": None, "kernel": info["kernel"], "hbm_algorithmic_bytes": stream}
    cpu = None
    if not args.no_cpu_baseline and world == 1 and not bwd and args.lq is None:
        progress("CPU baseline sample")
        cores = host_threads()
        tf, ctoks, cdt, sample = time_cpu(name, 1, 0, 2048)
        cpu = {"value": tf, "unit": "TFLOP/s", "tokens_per_s": ctoks, "cores": cores, "kind": "port",
               "sample": sample}
    line = {
        "metric": METRIC if not bwd else "TPA bwd algorithmic TFLOP/s per B200 (2.5x the forward's FLOPs)", "value": value, "unit": "TFLOP/s", "tokens_per_s": toks, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "ms_per_step_median": statistics.median(per_step),
        "ms_per_step_max": max(per_step), "slowest_step": per_step.index(max(per_step)), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": dtn, "data": "synthetic",
        "config": config_for(name, world, args.mask_mode, args.lq), "kernel": info, "cuda_graph": bool(args.graph),
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clock_summary,
        "parity": parity,
    }
    if dense_arm is not None:
        line["dense_cross_check"] = dense_arm
    if n1_ms is not None:
        # strong scaling on one box: the unsharded workload on one GPU against N GPUs
        line["ring"] = {"n1_ms": n1_ms, "ring_efficiency": n1_ms / (world * ms), "mask_mode": args.mask_mode,
                        "breakdown": breakdown}
    print(json.dumps(line), flush=True)
    if ring:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        sys.exit(3)


if __name__ == "__main__":
    main()
