#!/usr/bin/env python
"""Benchmark of the Lightning Attention-2 forward+backward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): lightning_attn2 forward + backward on b=4, h=32, n=32768, d=e=128, bf16,
q/k/v/do ~ N(0,1) from seed 2024, ALiBi-style slopes -- the largest point of the reference's
benchmark sweep (benchmarks/benchmark_lightning2.py:56-118). Metric: tokens/s (tokens = b*n per step).
With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same workload on its own
(batch, head) units with no communication (weak scaling); the value is the sum over ranks divided by
the slowest rank's time.

Rank 0 prints ONE JSON line. `--impl reference` times the CPU restatement of the reference's
recurrences (oracle/) on the host cores instead, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, N_TOK, D = 4, 32, 32768, 128
SEED = 2024
# Algorithmic work per (token, head) at d = e = 128, bf16, forward + backward: bytes that must cross HBM
# (read q,k,v / write o; read q,k,v,do / write dq,dk,dv) and flops with the reference's 64-token blocks.
ALG_BYTES_PER_UNIT = 2816
ALG_FLOP_PER_UNIT = 344064
LA_LAUNCHES_PER_STEP = 4  # generic-product equivalents per step: o, dq, dk, dv (dk and dv share one fused launch)
# DRAM bytes (read + write) per launch of la_chunk_kernel measured with ncu; see profiles/. None = not captured yet.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 4 * 1048.7e6  # n=8192 capture (1048.7 MB) scaled x4: traffic is linear in n
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML (read-only queries) in a background thread
    while the timed region runs; falls back to one nvidia-smi query if NVML bindings are missing."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index):
        self.index = index
        self.sm, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self.thread = None
        self.nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        nv = self.nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        if self.nvml is None:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=20).stdout
                a, b_ = (float(x) for x in out.strip().split(","))
                return {"sm_mhz": a, "sm_max_mhz": b_, "samples": 1, "reasons": [], "note": "single nvidia-smi query after the region"}
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock query unavailable"]}
        self._stop.set()
        self.thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.sm), "reasons": sorted(self.reasons)}


def cpu_sample(pairs):
    """fwd+bwd of `pairs` (batch, head) units at full sequence length with the numpy oracle (fp32), one unit per
    host thread (BLAS pinned to one thread per worker); returns (seconds, tokens/s scaled to the full b*h workload)."""
    from concurrent.futures import ThreadPoolExecutor

    import numpy as np
    from oracle import lightning_oracle as O

    rng = np.random.default_rng(SEED)
    q, k, v, do = (rng.standard_normal((pairs, 1, N_TOK, D)).astype(np.float32) for _ in range(4))
    slopes = O.build_slopes(H)

    def one(i):
        s = slopes[i % H:i % H + 1]
        O.la2_fwd_blockwise(q[i:i + 1], k[i:i + 1], v[i:i + 1], s, dtype=np.float32)
        O.la2_bwd_blockwise(q[i:i + 1], k[i:i + 1], v[i:i + 1], s, do[i:i + 1], dtype=np.float32)

    try:
        from threadpoolctl import threadpool_limits
        limiter = threadpool_limits(limits=1)
    except Exception:
        limiter = None
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=min(pairs, host_threads())) as pool:
        list(pool.map(one, range(pairs)))
    dt = time.perf_counter() - t0
    if limiter is not None:
        limiter.restore_original_limits()
    tokens = B * N_TOK * (pairs / float(B * H))  # share of the step's tokens this sample stands for
    return dt, tokens / dt


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, rank, emit):
    if rank != 0:
        return
    pairs = host_threads()
    for _ in range(args.warmup):
        cpu_sample(pairs)
    times = [cpu_sample(pairs)[0] for _ in range(args.steps)]
    dt = sum(times) / len(times)
    value = B * N_TOK * (pairs / float(B * H)) / dt
    sample = (f"{pairs} of {B * H} (batch, head) pairs at n={N_TOK}, d=e={D}, fp32 numpy block recurrences, fwd+bwd, "
              "one pair per host thread, scaled to the full step")
    emit(json.dumps({
        "impl": "reference", "metric": "lightning2_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"lightning2 fwd+bwd b{B} h{H} n{N_TOK} d{D} e{D} per GPU, decay slopes", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": host_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# The reference's published tables (ms; hardware not stated): README.md:58-76 and benchmarks/README.md:6-24,52-69.
REF_LIGHTNING2_FWD = {512: 0.351540, 1024: 0.585876, 2048: 1.134238, 4096: 2.240815, 8192: 4.414397, 16384: 8.832678, 32768: 17.661427}
REF_LIGHTNING2_BWD = {512: 1.169621, 1024: 2.334296, 2048: 4.657026, 4096: 9.307817, 8192: 18.617611, 16384: 37.212578, 32768: 74.594788}
REF_NODECAY_FWD = {512: 0.416118, 1024: 0.758793, 2048: 1.477481, 4096: 2.949107, 8192: 6.018426, 16384: 11.795692, 32768: 23.883759}
REF_NODECAY_BWD = {512: 1.378255, 1024: 2.653988, 2048: 5.504418, 4096: 11.009040, 8192: 21.968288, 16384: 36.816639, 32768: 73.657219}
REF_SRMS_FWD = {512: 0.040659, 1024: 0.068261, 2048: 0.124653, 4096: 0.236823, 8192: 0.460920, 16384: 0.912446, 32768: 1.818576}
REF_SRMS_BWD = {512: 0.102669, 1024: 0.186009, 2048: 0.354364, 4096: 0.690570, 8192: 1.363543, 16384: 2.711788, 32768: 5.410873}


def run_sweep(emit):
    """The reference's two benchmark tables on one GPU, same shapes and timing style (warm-up, median of repeated
    CUDA-event timings, L2 flushed between repetitions): benchmarks/benchmark_lightning2.py:56-118 (b4 h32 d=e=128 bf16,
    fwd and bwd separately, with and without decay) and benchmarks/benchmark_srmsnorm.py (b12, dim 2048 bf16)."""
    import torch

    import lightning_attention_b200 as la

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flush_box = [flush]

    def timed(fn, reps=15, warm=5):
        if flush_box[0] is None:
            flush_box[0] = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(reps):
            flush_box[0].zero_()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b_.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b_))
        return statistics.median(ts)

    def peak_mb(fn):
        """Peak allocated memory of one call, inputs included, as the reference's memory table measures it
        (benchmarks/benchmark_lightning2.py:160-190: reset the peak, run, read torch.cuda.max_memory_allocated)."""
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(dev)
        fn()
        torch.cuda.synchronize()
        return torch.cuda.max_memory_allocated(dev) / 1024 / 1024

    def drop_flush():  # the memory columns should not carry the flush buffer
        flush_box[0] = None

    del flush
    torch.manual_seed(SEED)
    s = la._build_slope_tensor(H).to(dev)
    for n in (512, 1024, 2048, 4096, 8192, 16384, 32768):
        q, k, v = (torch.randn((B, H, n, D), device=dev, dtype=torch.bfloat16).requires_grad_() for _ in range(3))
        do = torch.randn((B, H, n, D), device=dev, dtype=torch.bfloat16)
        for name, fn, ref_f, ref_b in (("lightning2", lambda: la.lightning_attn2(q, k, v, s), REF_LIGHTNING2_FWD, REF_LIGHTNING2_BWD),
                                       ("lightning2_no_decay", lambda: la.lightning_attn2_no_decay(q, k, v), REF_NODECAY_FWD, REF_NODECAY_BWD)):
            fwd = timed(fn)
            o = fn()

            def bwd_fn():
                q.grad = k.grad = v.grad = None
                o.backward(do, retain_graph=True)

            bwd = timed(bwd_fn)
            drop_flush()
            del o
            q.grad = k.grad = v.grad = None
            fwd_mb = peak_mb(lambda: fn())

            def fwd_bwd():
                fn().backward(do)

            bwd_mb = peak_mb(fwd_bwd)
            q.grad = k.grad = v.grad = None
            units = B * H * n
            emit(json.dumps({"table": name, "n": n, "fwd_ms": fwd, "bwd_ms": bwd, "ref_fwd_ms": ref_f[n], "ref_bwd_ms": ref_b[n],
                              "fwd_peak_mb": fwd_mb, "fwd_bwd_peak_mb": bwd_mb,
                              "ref_fwd_peak_mb": 64.0 * n / 512, "ref_bwd_peak_mb": 173.6 * n / 512,
                              "tokens_per_s_fwd_bwd": B * n / ((fwd + bwd) * 1e-3),
                              "hbm_frac_of_measured": ALG_BYTES_PER_UNIT * units / ((fwd + bwd) * 1e-3) / 1e9 / load_peaks()[0]}))
        del q, k, v, do
    for n in (512, 1024, 2048, 4096, 8192, 16384, 32768):
        x = torch.randn((12, n, 2048), device=dev, dtype=torch.bfloat16).requires_grad_()
        dy = torch.randn((12, n, 2048), device=dev, dtype=torch.bfloat16)
        norm = la.SimpleRMSNorm(2048)
        fwd = timed(lambda: norm(x))
        y = norm(x)

        def bwd_fn():
            x.grad = None
            y.backward(dy, retain_graph=True)

        bwd = timed(bwd_fn)
        elems = 12 * n * 2048
        emit(json.dumps({"table": "srmsnorm", "n": n, "fwd_ms": fwd, "bwd_ms": bwd, "ref_fwd_ms": REF_SRMS_FWD[n], "ref_bwd_ms": REF_SRMS_BWD[n],
                          "fwd_gbs": 4.0 * elems / fwd / 1e6, "bwd_gbs": 6.0 * elems / bwd / 1e6}))


TRACE_SLOTS = ["mma: block start", "mma: X issued", "mma: P and C ready", "mma: D issued", "mask: S ready", "mask: P written",
               "state: Bm scaled", "state: PC+D done seen", "state: D drained", "state: next state ready", "state: accumulators free",
               "state: output tile staged"]


def run_trace(emit):
    """In-kernel clock trace of the attention block kernel (lab200_la_debug_trace): one forward-time and one reverse-time
    launch at b4 h32 d=e=128, n = --n; CTA (0,0,0) stamps clock64() at twelve hand-over points of every 128-token block.
    Prints one JSON line per direction: the block period and each point's mean offset from the MMA warp's block start,
    in SM cycles, over the steady-state blocks."""
    import torch

    import lightning_attention_b200 as la
    from lightning_attention_b200 import _lib
    from lightning_attention_b200.ops.cuda.lightning_attn2 import la_generic

    if not torch.cuda.is_available():
        raise SystemExit("--trace needs a CUDA GPU")
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    g = torch.Generator(device=dev)
    g.manual_seed(SEED)
    a, bm, c = (torch.randn((B, H, N_TOK, D), device=dev, generator=g).to(torch.bfloat16) for _ in range(3))
    s = la._build_slope_tensor(H).to(dev)
    nb = N_TOK // 128
    for reverse in (False, True):
        for _ in range(3):
            la_generic(a, bm, c, s, reverse=reverse, chunks=1)
        torch.cuda.synchronize()
        tr = torch.zeros(nb * 16, dtype=torch.int64, device=dev)
        L.lab200_la_debug_trace(tr.data_ptr(), nb)
        la_generic(a, bm, c, s, reverse=reverse, chunks=1)
        torch.cuda.synchronize()
        L.lab200_la_debug_trace(None, 0)
        t = tr.view(nb, 16).cpu()
        lo, hi = min(8, nb // 2), max(nb - 2, nb // 2 + 1)
        rel = (t - t[:, 0:1])[lo:hi].double().mean(0).tolist()
        period = (t[1:, 0] - t[:-1, 0])[lo:hi].double().mean().item()
        emit(json.dumps({"trace": "la_pipe_kernel", "direction": "reverse-time" if reverse else "forward-time",
                         "shape": [B, H, N_TOK, D], "blocks_averaged": hi - lo, "block_period_cycles": round(period),
                         "offsets_cycles": {name: round(x) for name, x in zip(TRACE_SLOTS, rel)}}))


def main():
    global N_TOK
    # Libraries (NCCL's version banner, for one) print to file descriptor 1; the contract is ONE JSON line on stdout.
    # Everything that is not that line is sent to stderr by pointing fd 1 at fd 2 and keeping the real stdout aside.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        os.write(real_stdout, (line + "\n").encode())

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--n", type=int, default=N_TOK, help="sequence length (default: the benchmark's largest point)")
    ap.add_argument("--trace", action="store_true",
                    help="print the in-kernel clock trace of the attention block kernel (one JSON line per direction) and exit")
    ap.add_argument("--sweep", action="store_true",
                    help="instead of the single bench line, print one JSON line per point of the reference's benchmark "
                         "tables (Lightning2 / NoDecay fwd and bwd over n; SRMSNorm fwd and bwd over n) and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    N_TOK = args.n

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, emit)
        return
    if args.sweep:
        run_sweep(emit)
        return
    if args.trace:
        run_trace(emit)
        return

    import torch
    import torch.distributed as dist

    import lightning_attention_b200 as la
    from lightning_attention_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (the product has no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- synthetic inputs, resident in HBM (4 x 1.07 GB, far larger than the 126 MB L2) ----------------
    g = torch.Generator(device=dev)
    g.manual_seed(SEED + rank)
    mk = lambda: torch.randn((B, H, N_TOK, D), device=dev, dtype=torch.float32, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(), mk(), mk(), mk()
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    s = la._build_slope_tensor(H).to(dev)

    def step():
        q.grad = k.grad = v.grad = None
        o = la.lightning_attn2(q, k, v, s)
        o.backward(do)
        return o

    for _ in range(args.warmup):
        step()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = L.lab200_launch_count()
    barrier()
    for i in range(args.steps):
        q.grad = k.grad = v.grad = None
        ev[i][0].record()
        o = la.lightning_attn2(q, k, v, s)
        ev[i][1].record()
        o.backward(do)
        ev[i][2].record()
    end = torch.cuda.Event(enable_timing=True)
    end.record()
    barrier()
    launches = L.lab200_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    total_ms = ev[0][0].elapsed_time(end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    t = torch.tensor([total_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms = (float(x) for x in t)
    ms_per_step = total_ms / args.steps
    tokens_per_step = B * N_TOK * world
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- SRMSNorm fwd+bwd GB/s on (32768, 4096) bf16 (rank 0) -------------------------------------------
    srms = None
    if rank == 0:
        M, Nf = 4 * 8192, 4096
        x = torch.randn((M, Nf), device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
        dy = torch.randn((M, Nf), device=dev, dtype=torch.bfloat16, generator=g)
        norm = la.SimpleRMSNorm(Nf)
        # 1 GiB: flushes L2 and keeps the GPU busy long enough for the host to enqueue forward and backward behind it,
        # so the events bracket device time, not the autograd engine's launch latency
        flush = torch.empty(1024 * 1024 * 1024, dtype=torch.uint8, device=dev)
        tf, tb = [], []
        for i in range(8):
            x.grad = None
            flush.zero_()
            a, b_, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record(); y = norm(x); b_.record(); y.backward(dy); c.record()
            torch.cuda.synchronize()
            if i >= 3:
                tf.append(a.elapsed_time(b_)); tb.append(b_.elapsed_time(c))
        fms, bms = statistics.median(tf), statistics.median(tb)
        srms = {"shape": [M, Nf], "fwd_ms": fms, "bwd_ms": bms, "fwd_gbs": 4.0 * M * Nf / fms / 1e6,
                "bwd_gbs": 6.0 * M * Nf / bms / 1e6, "note": "public API (autograd Function); L2 flushed between reps by a 1 GiB memset the launches queue behind"}
        # the same rows through the fused norm + sigmoid gate (6 and 10 bytes per element)
        try:
            gate = torch.randn((M, Nf), device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
            tf, tb = [], []
            for i in range(8):
                x.grad = gate.grad = None
                flush.zero_()
                a, b_, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                a.record(); y = la.srmsnorm_sigmoid_gate(x, gate); b_.record(); y.backward(dy); c.record()
                torch.cuda.synchronize()
                if i >= 3:
                    tf.append(a.elapsed_time(b_)); tb.append(b_.elapsed_time(c))
            gf, gb = statistics.median(tf), statistics.median(tb)
            srms.update({"gate_fwd_ms": gf, "gate_bwd_ms": gb, "gate_fwd_gbs": 6.0 * M * Nf / gf / 1e6,
                         "gate_bwd_gbs": 10.0 * M * Nf / gb / 1e6})
            del gate
        except Exception as ex:
            srms["gate_error"] = repr(ex)[:200]
        del x, dy, flush

    # ---- projection layout: q, k, v, do as (b, h, n, d) views of (b, n, h, d) tensors, as a caller's projections give them.
    # "in_place": the op reads and writes that layout directly. "with_copies": what the reference's wrapper does with such
    # views - .contiguous() on q, k, v and do, and a rearranging copy of o and of the three gradients on the way back.
    proj = None
    if rank == 0:
        try:
            xq, xk, xv = (t.detach().transpose(1, 2).contiguous().requires_grad_() for t in (q, k, v))
            xdo = do.transpose(1, 2).contiguous()

            def in_place():
                xq.grad = xk.grad = xv.grad = None
                o_ = la.lightning_attn2(xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2), s)
                o_.backward(xdo.transpose(1, 2))

            def with_copies():
                xq.grad = xk.grad = xv.grad = None
                o_ = la.lightning_attn2(xq.transpose(1, 2).contiguous(), xk.transpose(1, 2).contiguous(),
                                        xv.transpose(1, 2).contiguous(), s)
                o_.transpose(1, 2).contiguous().backward(xdo)

            res = {}
            for name, fn in (("in_place", in_place), ("with_copies", with_copies)):
                for _ in range(2):
                    fn()
                p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                p0.record()
                for _ in range(5):
                    fn()
                p1.record()
                torch.cuda.synchronize()
                res[name + "_ms"] = p0.elapsed_time(p1) / 5
            proj = {"shape_b_n_h_d": [B, N_TOK, H, D], **res,
                    "note": "fwd+bwd with q, k, v, do given as (b, n, h, d) tensors; tnl_attn.py:56-64 style caller"}
            del xq, xk, xv, xdo
        except Exception as ex:
            proj = {"error": repr(ex)[:200]}

    # ---- decode step (inference API): 256 sequences x 32 heads, d=e=128; the fp32 states (537 MB) exceed L2 -----
    decode = None
    if rank == 0:
        try:
            bd = 256
            st = torch.zeros((bd, H, D, D), device=dev, dtype=torch.float32)
            qd, kd, vd = (torch.randn((bd, H, D), device=dev, generator=g).to(torch.bfloat16) for _ in range(3))
            for _ in range(3):
                la.lightning_attn_decode(qd, kd, vd, s, st)
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            d0.record()
            for _ in range(20):
                la.lightning_attn_decode(qd, kd, vd, s, st)
            d1.record()
            torch.cuda.synchronize()
            dms = d0.elapsed_time(d1) / 20
            decode = {"shape": [bd, H, D, D], "ms_per_step": dms, "gbs": 8.0 * st.numel() / dms / 1e6,
                      "tokens_per_s": bd / (dms * 1e-3), "note": "one token per sequence; bytes = fp32 state read + written"}
            del st, qd, kd, vd
        except Exception as ex:
            decode = {"error": repr(ex)[:200]}

    # ---- long-context leg: b=1, h=32, d=e=128, 131072 tokens per GPU (the sequence-parallel shard size) ----
    # N = 1: plain single-GPU op at n = 131072. N > 1: sequence-parallel over N*131072 tokens (two NCCL
    # all-gathers of 2 MiB states per step). Same per-GPU work in both, so the ratio of the two times is the
    # sequence-parallel overhead.
    sp = None
    if args.n == 32768:
        try:
            from lightning_attention_b200 import distributed as la_dist

            Ls = 131072
            mk2 = lambda: (0.5 * torch.randn((1, H, Ls, D), device=dev, dtype=torch.float32, generator=g)).to(torch.bfloat16)
            q2, k2, v2, do2 = mk2(), mk2(), mk2(), mk2()
            q2.requires_grad_(); k2.requires_grad_(); v2.requires_grad_()

            def sp_step():
                q2.grad = k2.grad = v2.grad = None
                o2 = la_dist.lightning_attn_sp(q2, k2, v2, s) if world > 1 else la.lightning_attn2(q2, k2, v2, s)
                o2.backward(do2)

            for _ in range(3):
                sp_step()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(5):
                sp_step()
            a1.record()
            barrier()
            tt = torch.tensor([a0.elapsed_time(a1) / 5], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            sp = {"mode": "sequence-parallel" if world > 1 else "single-gpu", "tokens_total": Ls * world,
                  "ms_per_step": float(tt[0]), "tokens_per_s": Ls * world / (float(tt[0]) * 1e-3),
                  "shape_per_gpu": [1, H, Ls, D]}
            del q2, k2, v2, do2
        except Exception as ex:
            sp = {"error": repr(ex)[:200]}

    # ---- end to end through the public API with pinned host buffers ---------------------------------------
    e2e = None
    nbytes = q.numel() * 2
    try:
        if args.no_e2e:
            raise RuntimeError("skipped by --no-e2e")
        hq, hk, hv, hdo = (torch.empty((B, H, N_TOK, D), dtype=torch.bfloat16, pin_memory=True) for _ in range(4))
        ho, hdq, hdk, hdv = (torch.empty((B, H, N_TOK, D), dtype=torch.bfloat16, pin_memory=True) for _ in range(4))
        for hsrc, dsrc in ((hq, q), (hk, k), (hv, v), (hdo, do)):
            hsrc.copy_(dsrc.detach())
        dq_, dk_, dv_, ddo_ = (torch.empty_like(do) for _ in range(4))

        # The step is cut into 32 groups of 4 (batch, head) pairs that flow through three streams: host->device copy of
        # group g+1, forward+backward of group g and device->host copy of group g-1 overlap (PCIe is full duplex). A step
        # ends with all results on the host, so only the first copy-in and the last copy-out (1/32 each) run alone.
        gh = 4
        groups = [(ib, h0, h0 + gh) for ib in range(B) for h0 in range(0, H, gh)]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)

        def e2e_step():
            ev_in = [torch.cuda.Event() for _ in groups]
            ev_done = [torch.cuda.Event() for _ in groups]
            s_in.wait_stream(main)
            with torch.cuda.stream(s_in):
                for gi, (ib, h0, h1) in enumerate(groups):
                    for dst, src in ((dq_, hq), (dk_, hk), (dv_, hv), (ddo_, hdo)):
                        dst[ib, h0:h1].copy_(src[ib, h0:h1], non_blocking=True)
                    ev_in[gi].record(s_in)
            outs = []
            for gi, (ib, h0, h1) in enumerate(groups):
                main.wait_event(ev_in[gi])
                qq, kk, vv = (t[ib:ib + 1, h0:h1].detach().requires_grad_() for t in (dq_, dk_, dv_))
                oo = la.lightning_attn2(qq, kk, vv, s[h0:h1])
                oo.backward(ddo_[ib:ib + 1, h0:h1])
                outs.append((oo.detach(), qq.grad, kk.grad, vv.grad))
                ev_done[gi].record(main)
            with torch.cuda.stream(s_out):
                for gi, (ib, h0, h1) in enumerate(groups):
                    s_out.wait_event(ev_done[gi])
                    for dst, src in zip((ho, hdq, hdk, hdv), outs[gi]):
                        dst[ib, h0:h1].copy_(src[0], non_blocking=True)
                        src.record_stream(s_out)
            main.wait_stream(s_out)

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0]) / args.e2e_steps
        e2e = {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes,
               "note": "q,k,v,do copied from pinned host memory and o,dq,dk,dv copied back every step, per rank; 32 groups of 4 (batch, head) pairs pipelined over copy-in / compute / copy-out streams"}
    except Exception as ex:  # pinned allocation can fail on a small host
        e2e = {"value": None, "unit": "tokens/s", "error": repr(ex)[:200]}

    if rank == 0:
        hbm_peak, tf_peak, peak_kind = load_peaks()
        units = B * H * N_TOK
        launch_ms = (fwd_ms + bwd_ms) / LA_LAUNCHES_PER_STEP
        achieved = ALG_BYTES_PER_UNIT * units / LA_LAUNCHES_PER_STEP / (launch_ms * 1e-3) / 1e9
        roofline = {
            "bound": "hbm", "kernel": "la_pipe_kernel", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
            "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}", "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
            "launch_ms": launch_ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "alg_tflops": ALG_FLOP_PER_UNIT * units / ((fwd_ms + bwd_ms) * 1e-3) / 1e12,
            "frac_tensor": ALG_FLOP_PER_UNIT * units / ((fwd_ms + bwd_ms) * 1e-3) / 1e12 / tf_peak,
        }
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            pairs = 2 * host_threads()
            dt, tps = cpu_sample(pairs)
            cpu = {"value": tps, "unit": "tokens/s", "cores": host_threads(), "kind": "port", "seconds": dt,
                   "sample": f"{pairs} of {B * H} (batch, head) pairs at n={N_TOK}, fp32 numpy block recurrences, fwd+bwd, one pair per host thread, scaled to the full step"}
        out = {
            "metric": "lightning2_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"lightning2 fwd+bwd b{B} h{H} n{N_TOK} d{D} e{D} per GPU, decay slopes",
                       "l2": "inputs (4 x 1.07 GB) exceed L2; no flush needed", "parallelism": f"bh-shard x{world}, no collective"},
            # the reference publishes forward and backward milliseconds for this shape (hardware not stated), not tokens/s,
            # so vs_baseline stays null and the ratio of step times is given separately
            "reference_published": ({"fwd_plus_bwd_ms": REF_LIGHTNING2_FWD[N_TOK] + REF_LIGHTNING2_BWD[N_TOK],
                                     "step_time_ratio": (REF_LIGHTNING2_FWD[N_TOK] + REF_LIGHTNING2_BWD[N_TOK]) / ms_per_step}
                                    if N_TOK in REF_LIGHTNING2_FWD else None),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "srmsnorm": srms, "long_context": sp, "decode": decode, "projection_layout": proj,
        }
        emit(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
