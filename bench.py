#!/usr/bin/env python
"""Benchmark of the quantized-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling strong|weak]
    python bench.py --profile-case quant|fwd|fwd_causal|bwd|shortq|q32|midq     (small fixed case for a profiler capture)

Workload: INT8 attention forward at B=4 H=32 S=4096 D=128, bf16 inputs ~N(0,1) with 1 % of the channels scaled
x20, seeded per (batch, head), non-causal.  One step = quantize Q, K, V per token (the batched quantizer, V also
written dequantized) + the int8 attention forward, through the package's `quant_attention_forward`, which cuts
the heads into four slices so that the quantizer of a slice overlaps the attention of the previous one.  `value` = attention ops 4*B*H*D*S^2 of
the WHOLE workload per step / step time, in TOPS, inputs resident in HBM.

With N > 1 the 128 (batch, head) units of that fixed workload are cut into N contiguous slices, one per rank
(128 / 64 / 32 / 16 heads per GPU at 1 / 2 / 4 / 8 GPUs), no collective on the data path: strong scaling.
`--scaling weak` instead gives every rank the full per-GPU workload (global batch 4*N); the default run reports
that figure too, under `extra`.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B, H, S, D = 4, 32, 4096, 128
WORKLOAD = "int8_attn_fwd B4 H32 S4096 D128 non-causal bf16 outlier-channels (quantize q,k,v + forward)"
METRIC = "int8_attention_forward_throughput"
DTYPE = "int8 codes; exact integer logits (fp16*fp16->fp32 over centered codes) + bf16 P.V"


def fwd_ops(b, h, sq, skv, d, causal=False):
    pairs = sq * skv if not causal else sq * (sq + 1) // 2
    return 4 * b * h * d * pairs


def host_threads() -> int:
    """CPU threads this process may use (the affinity mask, not the machine's core count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def make_heads(h0, h1, s, d, device, seed_base, kind="outlier", dtype=torch.bfloat16, tensors=3):
    """Heads [h0, h1) of the flattened (batch x head) axis as `tensors` tensors of shape (1, h1-h0, s, d).
    Generation is seeded per head, so any partition of the heads over ranks sees the same data."""
    out = []
    for t in range(tensors):
        x = torch.empty(h1 - h0, s, d, dtype=dtype, device=device)
        for i in range(h0, h1):
            g = torch.Generator(device=device).manual_seed(seed_base + 1000 * t + i)
            r = torch.randn(s, d, generator=g, device=device, dtype=torch.float32)
            if kind == "loguniform":
                mag = torch.empty(s, 1, device=device).uniform_(math.log(0.1), math.log(10.0), generator=g)
                r = r * torch.exp(mag)
            x[i - h0] = r.to(dtype)
        if kind == "outlier":
            g = torch.Generator().manual_seed(seed_base + 7 + t)
            idx = torch.randperm(d, generator=g)[: max(1, math.ceil(0.01 * d))]
            x[..., idx.to(device)] *= 20.0
        out.append(x.view(1, h1 - h0, s, d))
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read-only queries from a thread
    (a few milliseconds apart, so that even a short timed region gets samples), or an `nvidia-smi -lms` child
    process if the NVML binding is missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None
        self.samples, self._stop, self._thread, self._nvml = [], False, None, None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        self._nvml = pynvml
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            return pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll(self, handle):
        n = self._nvml
        # NVML clocks-event-reason bits
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        try:
            mx = n.nvmlDeviceGetMaxClockInfo(handle, n.NVML_CLOCK_SM)
        except Exception:
            mx = None
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop:
            try:
                sm = n.nvmlDeviceGetClockInfo(handle, n.NVML_CLOCK_SM)
                r = get_reasons(handle)
                self.samples.append((time.time(), float(sm), mx, [k for k, b in bits.items() if r & b]))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            handle = self._nvml_handle()
            self._thread = threading.Thread(target=self._poll, args=(handle,), daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0, t1):
        """Keep only the samples taken inside [t0, t1] (the timed region)."""
        inside = [x for x in self.samples if t0 <= x[0] <= t1]
        self.samples = inside if inside else self.samples[-3:]
        inside = [x for x in self.lines if t0 <= x[0] <= t1]
        self.lines = inside if inside else self.lines[-3:]

    def stop(self):
        if self._thread is not None:
            self._stop = True
            self._thread.join(timeout=1.0)
            sm = sorted(x[1] for x in self.samples)
            mx = [x[2] for x in self.samples if x[2]]
            reasons = sorted({r for x in self.samples for r in x[3]})
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(max(mx)) if mx else None,
                    "reasons": reasons, "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for _ts, ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------- CPU arm

def cpu_reference_sample(heads: int, s: int, d: int, repeats: int, causal=False):
    """Times the CPU restatement of the reference math (per-token quantize -> dequantized softmax attention) on
    `heads` heads of the workload with every host thread this process may use; returns (ops per second, seconds,
    threads).  The thread count is set explicitly: a launcher may have exported OMP_NUM_THREADS=1."""
    import oracle
    threads = host_threads()
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, heads, s, d).bfloat16() for _ in range(3))
    sm = 1.0 / math.sqrt(d)
    oracle.int8_mode_forward(q[:, :1, :256], k[:, :1, :256], v[:, :1, :256], causal, sm)   # warm-up
    t0 = time.perf_counter()
    for _ in range(repeats):
        oracle.int8_mode_forward(q, k, v, causal, sm)
    dt = time.perf_counter() - t0
    return fwd_ops(1, heads, s, s, d, causal) * repeats / dt, dt, torch.get_num_threads()


def run_reference_arm(args):
    """The reference's math on the host cores (the oracle port; the reference itself is a set of Triton GPU
    kernels with no CPU implementation).  Under a multi-rank launcher rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    heads = 2
    for _ in range(min(args.warmup, 1)):
        cpu_reference_sample(1, 1024, D, 1)
    t0 = time.perf_counter()
    ops = 0.0
    threads = host_threads()
    for _ in range(args.steps):
        rate, dt, threads = cpu_reference_sample(heads, S, D, 1)
        ops += rate * dt
    el = time.perf_counter() - t0
    value = ops / el / 1e12
    sample = f"{heads} of {B * H} heads of the workload per step (S={S}, D={D}), oracle port in PyTorch CPU fp32"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": DTYPE,
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- GPU arm helpers

def time_ms(fn, stream, reps=10, warm=3):
    for _ in range(warm):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record(stream)
    for _ in range(reps):
        fn()
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def measure_tensor_peaks(stream):
    """tcgen05.mma issue-rate probe of the library on every SM (operands resident in shared memory, no loads, no
    epilogue): the int8 and bf16 tensor-pipe peaks of THIS GPU, best of 5 launches each."""
    from quant_flash_attn_b200 import _lib
    lib = _lib.load()
    out = {}
    for form, n, name in ((0, 128, "int8_ss_n128"), (0, 256, "int8_ss_n256"), (1, 128, "bf16_ss_n128"),
                          (2, 128, "bf16_ts_n128")):
        ops = ctypes.c_double()
        best = None
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            rc = lib.qfa_probe_mma_rate(form, n, 4000, ctypes.byref(ops), None, stream.cuda_stream)
            b.record(stream)
            torch.cuda.synchronize()
            if rc != 0:
                return {"error": f"qfa_probe_mma_rate returned {rc}"}
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
        out[name] = ops.value / best / 1e9
    out["how"] = ("one CTA per SM issues 16 000 tcgen05.mma (M128, K32 int8 / K16 bf16) on zeroed operand tiles "
                  "resident in shared memory; TOPS = ops / CUDA-event time, best of 5")
    return out


class StepGraphs:
    """One step -- quantize q, k, v and run the attention forward through the package's pipelined operator front
    half (head slices on side streams: the quantizer of a slice overlaps the attention of the previous one) --
    captured once into a CUDA graph and replayed, so that a step costs one graph launch on the host instead of
    dozens of allocations and ctypes calls (at 16 heads per GPU a step is 0.2 ms of GPU time).  A second graph
    holds the attention forward alone (one launch over all local heads) for the per-kernel timing.  Falls back
    to eager calls if capture is refused."""

    eager_only = False      # --eager: no graph capture (for a profiler's launch list)

    def __init__(self, qfa, q, k, v, causal, sm, stream):
        self.qfa, self.q, self.k, self.v, self.causal, self.sm, self.stream = qfa, q, k, v, causal, sm, stream
        self.mode = "eager"
        n0 = qfa.launch_count()
        self._step()
        torch.cuda.synchronize()
        self.launches_per_step = qfa.launch_count() - n0
        self._attn()
        torch.cuda.synchronize()
        if StepGraphs.eager_only:
            return
        try:
            self.g_step, self.g_attn = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g_step):
                self._step()
            with torch.cuda.graph(self.g_attn):
                self._attn()
            torch.cuda.synchronize()
            self.mode = "cuda-graph"
        except Exception as e:        # noqa: BLE001 -- any capture problem: measure with eager launches instead
            self.capture_error = repr(e)[:200]
            torch.cuda.synchronize()

    def _step(self):
        self.o, self.lse, self.qq, self.kq, self.vq = self.qfa.quant_attention_forward(self.q, self.k, self.v,
                                                                                      self.causal, self.sm)

    def _attn(self):
        self.qfa.int8_attention_forward(self.qq, self.kq, self.vq, self.causal, self.sm, self.q.dtype, o=self.o, lse=self.lse)

    def step(self):
        if self.mode == "cuda-graph":
            self.g_step.replay()
        else:
            self._step()

    def attn_only(self):
        if self.mode == "cuda-graph":
            self.g_attn.replay()
        else:
            self._attn()


class RotatingRunner:
    """Round-robin over several StepGraphs whose inputs are copies of the same data at different addresses, so
    that the bytes touched between two uses of one copy exceed the L2 capacity and every step reads its inputs
    from HBM even when one rank's slice of the workload would fit in L2."""

    def __init__(self, runners):
        self.runners, self.i = runners, 0
        r0 = runners[0]
        self.mode, self.launches_per_step = r0.mode, r0.launches_per_step
        self.q, self.k, self.v, self.o, self.lse = r0.q, r0.k, r0.v, r0.o, r0.lse
        self.qq, self.kq, self.vq = r0.qq, r0.kq, r0.vq
        self.capture_error = getattr(r0, "capture_error", None)

    def step(self):
        self.runners[self.i % len(self.runners)].step()
        self.i += 1

    def attn_only(self):
        self.runners[self.i % len(self.runners)].attn_only()
        self.i += 1


L2_BYTES = 126e6


def rotation_count(bytes_per_step: float) -> int:
    """Copies needed so that a round over all of them touches at least twice the L2 capacity."""
    return max(1, int(math.ceil(2 * L2_BYTES / max(bytes_per_step, 1.0))))


def timed_steps(runner, steps, stream, barrier, attn_only=False):
    """`steps` steps (or launches of the attention forward alone) bracketed by a barrier + synchronize on both
    sides, timed with CUDA events on the launching stream; returns (total ms, wall-clock window)."""
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn = runner.attn_only if attn_only else runner.step
    barrier()
    w0 = time.time()
    t0.record(stream)
    for _ in range(steps):
        fn()
    t1.record(stream)
    barrier()
    w1 = time.time()
    return t0.elapsed_time(t1), (w0, w1)


def single_gpu_extras(qfa, extra, runner, dev, stream, sm):
    """Secondary figures measured on one GPU only (untimed region of the bench): tensor-pipe peaks, a sustained
    run, the quantizer sweep, the sequence-length sweep, the reference's own benchmark shapes, the front end."""
    peaks = load_peaks()
    extra["tensor_pipe_peaks_TOPS"] = measure_tensor_peaks(stream)

    # sustained: the same step back to back for >= 2 s, with the SM clock sampled meanwhile
    sampler = ClockSampler(dev.index)
    sampler.start()
    n_done, t0 = 0, time.time()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    w0 = time.time()
    a.record(stream)
    while time.time() - t0 < 2.2:
        for _ in range(50):
            runner.step()
        n_done += 50
        torch.cuda.synchronize()
    b.record(stream)
    torch.cuda.synchronize()
    w1 = time.time()
    sampler.window(w0, w1)
    ck = sampler.stop()
    s_ms = a.elapsed_time(b) / n_done
    tops = fwd_ops(1, runner.q.shape[1], S, S, D) / s_ms / 1e9
    extra["sustained"] = {"seconds": w1 - w0, "steps": n_done, "ms_per_step": s_ms, "TOPS": tops,
                          "sm_mhz_median": ck.get("sm_mhz"), "sm_max_mhz": ck.get("sm_max_mhz"),
                          "reasons": ck.get("reasons"),
                          "TOPS_at_max_clock": (tops * ck["sm_max_mhz"] / ck["sm_mhz"]) if ck.get("sm_mhz") and ck.get("sm_max_mhz") else None,
                          "frac_of_bf16_sustained_" + peaks["source"]: tops / peaks["bf16_tflops_sustained"]}

    # the two routes to the integer logits at the bench shape (same bits): 16-bit MMA over centered codes (what the
    # steps run) against the int8 MMA plus zero-point terms
    routes = {}
    kq_i8 = tuple(runner.kq[:5])
    for causal in (False, True):
        fo = fwd_ops(1, runner.q.shape[1], S, S, D, causal)
        for name, kq_ in (("centered_16bit_mma", runner.kq), ("int8_mma", kq_i8)):
            ms = time_ms(lambda: qfa.int8_attention_forward(runner.qq, kq_, runner.vq, causal, sm, torch.bfloat16,
                                                            o=runner.o, lse=runner.lse), stream, reps=5)
            routes[("causal_" if causal else "noncausal_") + name] = {"ms": ms, "TOPS": fo / ms / 1e9}
    extra["logit_routes_fwd"] = routes

    # quantizer: [N tokens x D] bf16, N from 64 Ki to 16 Mi, D = 64 / 128; rotating buffers so that every launch
    # reads from HBM even where one tensor would fit the 126 MB L2
    sweep = []
    for d in (64, 128):
        for n_tok in (1 << 16, 1 << 18, 1 << 20, 1 << 22, 1 << 24):
            bytes_in = n_tok * d * 2
            n_buf = max(1, min(8, int(math.ceil(512e6 / bytes_in))))
            xs = [torch.randn(1, 1, n_tok, d, device=dev, dtype=torch.bfloat16) for _ in range(n_buf)]
            it = [0]

            def qstep():
                qfa.asymmetric_quant_per_token_ex(xs[it[0] % n_buf])
                it[0] += 1
            ms = time_ms(qstep, stream, reps=max(5, 2 * n_buf), warm=n_buf)
            byt = n_tok * (2 * d + d + 2 + 1 + 4)
            sweep.append({"tokens": n_tok, "D": d, "ms": ms, "GBps": byt / ms / 1e6,
                          "frac_of_hbm_" + peaks["source"]: byt / ms / 1e6 / peaks["hbm_gbs"], "buffers": n_buf})
            del xs
    extra["quantizer_sweep"] = sweep
    big = max((r for r in sweep if r["D"] == 128 and r["tokens"] == 1 << 20), key=lambda r: r["GBps"])
    extra["quantizer"] = {"tokens": big["tokens"], "D": 128, "ms": big["ms"], "GBps": big["GBps"],
                          "bytes_per_token": 2 * D + D + 7,
                          "frac_of_hbm_" + peaks["source"]: big["GBps"] / peaks["hbm_gbs"]}

    # sequence-length sweep: B*S = 32768, H = 16, D = 128, causal, forward + backward (3.5 x forward ops)
    seq = []
    for s_len in (512, 1024, 2048, 4096, 8192, 16384):
        b_ = 32768 // s_len
        tq, tk, tv, tdo = (t.view(b_, 16, s_len, D) for t in make_heads(0, b_ * 16, s_len, D, dev, 500 + s_len, "normal", tensors=4))
        qq, kq, vq = qfa.quantize_qkv(tq, tk, tv)
        o_, lse_ = qfa.int8_attention_forward(qq, kq, vq, True, sm, torch.bfloat16)
        f_ms = time_ms(lambda: qfa.int8_attention_forward(qq, kq, vq, True, sm, torch.bfloat16), stream, reps=5)
        b_ms = time_ms(lambda: qfa.int8_attention_backward(qq, kq, vq, True, sm, o_, lse_, tdo), stream, reps=5)
        fo = fwd_ops(b_, 16, s_len, s_len, D, True)
        seq.append({"S": s_len, "B": b_, "fwd_ms": f_ms, "bwd_ms": b_ms, "fwd_TOPS": fo / f_ms / 1e9,
                    "fwd_bwd_TOPS": 3.5 * fo / (f_ms + b_ms) / 1e9})
        del tq, tk, tv, tdo, qq, kq, vq, o_, lse_
    extra["seq_sweep_BS32768_H16_D128_causal"] = seq

    # training shape: B8 H16 S2048 D64 causal through the autograd operator (quantization included)
    tb, th, ts, td = 8, 16, 2048, 64
    tq, tk, tv, tdo = (t.view(tb, th, ts, td) for t in make_heads(0, tb * th, ts, td, dev, 99, "normal", tensors=4))
    tsm = 1.0 / math.sqrt(td)

    def train_step():
        a_, b2, c = (t.detach().requires_grad_() for t in (tq, tk, tv))
        qfa.quant_attention(a_, b2, c, True, tsm).backward(tdo)
    t_ms = time_ms(train_step, stream, reps=5)
    c3 = {"ms": t_ms, "TOPS": 3.5 * fwd_ops(tb, th, ts, ts, td, True) / t_ms / 1e9,
          "note": "autograd operator, eager: quantize + forward + backward, a dozen launches per step"}
    # the same step captured in a CUDA graph (a step is well under a millisecond of GPU time, so the eager figure
    # is bound by the host's launches and allocations, not by the kernels)
    try:
        a_, b2, c = (t.detach().clone().requires_grad_() for t in (tq, tk, tv))
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            for _ in range(2):
                qfa.quant_attention(a_, b2, c, True, tsm).backward(tdo)
                a_.grad = b2.grad = c.grad = None
        stream.wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            qfa.quant_attention(a_, b2, c, True, tsm).backward(tdo)
        g_ms = time_ms(g.replay, stream, reps=10)
        c3["graph_ms"] = g_ms
        c3["graph_TOPS"] = 3.5 * fwd_ops(tb, th, ts, ts, td, True) / g_ms / 1e9
        del g, a_, b2, c
    except Exception as e:        # noqa: BLE001
        c3["graph_error"] = repr(e)[:200]
        torch.cuda.synchronize()
    # and the two attention kernels on their own (no quantizer, no dequantization, no delta pre-pass in the forward)
    qq, kq, vq = qfa.quantize_qkv(tq, tk, tv)
    o_, lse_ = qfa.int8_attention_forward(qq, kq, vq, True, tsm, torch.bfloat16)
    c3["fwd_kernel_ms"] = time_ms(lambda: qfa.int8_attention_forward(qq, kq, vq, True, tsm, torch.bfloat16), stream, reps=10)
    c3["bwd_ms"] = time_ms(lambda: qfa.int8_attention_backward(qq, kq, vq, True, tsm, o_, lse_, tdo), stream, reps=10)
    extra["fwd_bwd_B8H16S2048D64_causal"] = c3
    del tq, tk, tv, tdo, qq, kq, vq, o_, lse_

    # flash_attn_func-style front end: the headline workload handed over in (B,S,H,D) memory
    fq, fk, fv = (t.view(B, H, S, D).transpose(1, 2).contiguous() for t in (runner.q, runner.k, runner.v))
    fe_ms = time_ms(lambda: qfa.quant_flash_attn_func(fq, fk, fv, causal=False, softmax_scale=sm), stream, reps=5)
    extra["frontend_bshd_B4S4096H32D128"] = {"ms": fe_ms, "TOPS": fwd_ops(B, H, S, S, D) / fe_ms / 1e9}
    del fq, fk, fv

    # the reference's own benchmark regime (test_speed.py:45,56-59; compute_flops.py:94-96): fp16 queries of 16 rows
    # against a long per-token-quantized K=V, ref mode, forward and backward.  HBM-bound on the int8 codes:
    # algorithmic bytes = NKV * (D + 3) per head read once (+ Q, O), reported against the measured copy bandwidth
    sq = []
    # (the shapes with 17 to 128 query rows run on the one-tile tcgen05 forward, which dequantizes K/V in the kernel)
    for (z, hh, nq, nkv, dd) in ((256, 16, 16, 1024, 128), (256, 16, 16, 4096, 128), (64, 16, 16, 4096, 64),
                                 (256, 16, 32, 2048, 128), (64, 16, 64, 2048, 128), (99, 53, 97, 689, 128), (64, 16, 128, 2048, 128),
                                 (64, 16, 128, 4096, 64)):
        rq = torch.randn(z, hh, nq, dd, device=dev, dtype=torch.float16, requires_grad=True)
        rkv = torch.randn(z, hh, nkv, dd, device=dev, dtype=torch.float16, requires_grad=True)
        go = torch.randn_like(rq)
        kvq = qfa.asymmetric_quant_per_token(rkv.detach())
        rsm = 1.0 / math.sqrt(dd)
        with torch.no_grad():
            f_ms = time_ms(lambda: qfa.quant_flash_attn(rq, rkv, kvq, rsm), stream, reps=10)

        def fb():
            rq.grad = None
            rkv.grad = None
            qfa.quant_flash_attn(rq, rkv, kvq, rsm).backward(go)
        fb_ms = time_ms(fb, stream, reps=5)
        byt = z * hh * (nkv * (dd + 3) + 2 * nq * dd * 2)
        sq.append({"Z": z, "H": hh, "NQ": nq, "NKV": nkv, "D": dd, "fwd_ms": f_ms, "fwd_bwd_ms": fb_ms,
                   "fwd_TFLOPs": 4.0 * z * hh * nq * nkv * dd / f_ms / 1e9, "fwd_GBps": byt / f_ms / 1e6,
                   "fwd_frac_of_hbm_" + peaks["source"]: byt / f_ms / 1e6 / peaks["hbm_gbs"]})
        del rq, rkv, go, kvq
    extra["short_query_ref_mode"] = sq


def run_ours(args):
    import torch.distributed as dist
    import quant_flash_attn_b200 as qfa
    from quant_flash_attn_b200 import shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    sm = 1.0 / math.sqrt(D)
    stream = torch.cuda.current_stream()
    n_units = B * H
    weak = args.scaling == "weak"
    if weak:                       # every rank owns B*H heads of a global batch of B*world
        h0, h1, total_units = rank * n_units, (rank + 1) * n_units, n_units * world
    else:                          # the fixed B*H heads are cut into contiguous slices
        (h0, h1), total_units = shard_bounds(n_units, world, rank), n_units
    q, k, v = make_heads(h0, h1, S, D, dev, seed_base=1234)
    ops_total = fwd_ops(1, total_units, S, S, D, False)
    ops_local = fwd_ops(1, h1 - h0, S, S, D, False)

    in_bytes = 3 * q.numel() * q.element_size()
    n_rot = rotation_count(in_bytes)
    runner = RotatingRunner([StepGraphs(qfa, q, k, v, False, sm, stream)] +
                            [StepGraphs(qfa, q.clone(), k.clone(), v.clone(), False, sm, stream) for _ in range(n_rot - 1)])
    for _ in range(max(args.warmup, 3)):
        runner.step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # keep every GPU busy for a few hundred milliseconds before the timed region: the clock sampler comes up and
    # the clocks settle where a long run holds them
    t_spin = time.time()
    while time.time() - t_spin < 0.4:
        for _ in range(20):
            runner.step()
        torch.cuda.synchronize()
    ms_total, (wall0, wall1) = timed_steps(runner, args.steps, stream, barrier)
    # the attention forward alone (one launch over the rank's heads, same rotating buffers), timed the same way
    # right after the step loop: inside a step its launches overlap the next slice's quantizer, so its own
    # duration cannot be read from events placed between them
    attn_total, (_, wall1) = timed_steps(runner, args.steps, stream, barrier, attn_only=True)
    attn_ms = attn_total / args.steps
    qfa.check_kernel_status()
    if rank == 0:
        sampler.window(wall0, wall1)
    ms_total, attn_ms_max = max_over_ranks(ms_total, attn_ms)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms_total / args.steps
    value = ops_total / (ms_step * 1e-3) / 1e12
    launches = runner.launches_per_step * args.steps

    extra = {"launch_mode": runner.mode, "heads_per_gpu": h1 - h0, "rotating_input_copies": n_rot, "attn_ms_rank0": attn_ms,
             "attn_ms_max_over_ranks": attn_ms_max}
    if runner.mode != "cuda-graph":
        extra["graph_capture_error"] = getattr(runner, "capture_error", None)

    # ---- the other figures the metric names, on the same partition, max over ranks: causal forward, fwd+bwd
    def partition_extras():
        out = {}
        qq, kq, vq = runner.qq, runner.kq, runner.vq
        do = make_heads(h0, h1, S, D, dev, seed_base=4321, kind="normal", tensors=1)[0]
        for causal in (False, True):
            tag = "causal" if causal else "noncausal"
            o_, lse_ = qfa.int8_attention_forward(qq, kq, vq, causal, sm, torch.bfloat16)
            f_ms = time_ms(lambda: qfa.int8_attention_forward(qq, kq, vq, causal, sm, torch.bfloat16, o=runner.o,
                                                              lse=runner.lse), stream, reps=5)
            b_ms = time_ms(lambda: qfa.int8_attention_backward(qq, kq, vq, causal, sm, o_, lse_, do), stream, reps=5)
            barrier()
            f_ms, b_ms = max_over_ranks(f_ms, b_ms)
            fo = fwd_ops(1, total_units, S, S, D, causal)
            out["fwd_" + tag] = {"ms": f_ms, "TOPS": fo / f_ms / 1e9}
            out["fwd_bwd_" + tag] = {"fwd_ms": f_ms, "bwd_ms": b_ms, "bwd_TOPS": 2.5 * fo / b_ms / 1e9,
                                     "TOPS": 3.5 * fo / (f_ms + b_ms) / 1e9}
            del o_, lse_
        return out

    if not args.skip_extras:
        extra["B4H32S4096D128_partitioned"] = partition_extras()

    # ---- long context: B1 H32 S32768 D128 causal, log-uniform token magnitudes, its 32 heads partitioned
    def long_context():
        c_h0, c_h1 = (rank * 32, rank * 32 + 32) if weak else shard_bounds(32, world, rank)
        if c_h1 <= c_h0:
            ms = 0.0
        else:
            cq, ck, cv = make_heads(c_h0, c_h1, 32768, D, dev, seed_base=77, kind="loguniform")
            cqq, ckq, cvq = qfa.quantize_qkv(cq, ck, cv)
            del cq, ck, cv
            ms = time_ms(lambda: qfa.int8_attention_forward(cqq, ckq, cvq, True, sm, torch.bfloat16), stream, reps=3, warm=1)
        barrier()
        (ms,) = max_over_ranks(ms)
        heads = 32 * world if weak else 32
        return {"ms": ms, "TOPS": fwd_ops(1, heads, 32768, 32768, D, True) / ms / 1e9, "heads_total": heads}

    if not args.skip_extras:
        extra["long_context_B1H32S32768D128_causal_fwd"] = long_context()

    # ---- with N > 1 also the other scaling mode: every rank runs the full per-GPU workload (replicas)
    if world > 1 and not weak and not args.skip_extras:
        fq, fk, fv = make_heads(rank * n_units, (rank + 1) * n_units, S, D, dev, seed_base=1234)
        rep = StepGraphs(qfa, fq, fk, fv, False, sm, stream)        # 403 MB of inputs per step: larger than L2
        for _ in range(3):
            rep.step()
        r_total, _ = timed_steps(rep, max(5, min(args.steps, 20)), stream, barrier)
        (r_total,) = max_over_ranks(r_total)
        r_step = r_total / max(5, min(args.steps, 20))
        extra["weak_scaling_replicas"] = {"ms_per_step": r_step, "global_batch": B * world,
                                          "TOPS": fwd_ops(B * world, H, S, S, D) / r_step / 1e9}
        del rep, fq, fk, fv

    # ---- the same steps issued alternately on two streams: consecutive steps are independent (they use different
    # copies of the inputs and their own outputs), so the head of step i+1 fills the SMs that the last, partial wave
    # of step i leaves idle.  A throughput figure for a consumer that keeps two batches in flight; NOT the headline,
    # whose steps run strictly one after the other.
    if n_rot >= 2 and not args.skip_extras:
        two = [torch.cuda.Stream(), torch.cuda.Stream()]
        n2 = max(args.steps, 20)
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for s_ in two:
            s_.wait_stream(stream)
        for i in range(n2):
            with torch.cuda.stream(two[i & 1]):
                runner.step()
        for s_ in two:
            stream.wait_stream(s_)
        t1.record(stream)
        barrier()
        (t2,) = max_over_ranks(t0.elapsed_time(t1) / n2)
        extra["steps_on_two_streams"] = {"ms_per_step": t2, "TOPS": ops_total / t2 / 1e9, "steps": n2}

    if rank == 0 and world == 1 and not args.skip_extras:
        single_gpu_extras(qfa, extra, runner, dev, stream, sm)

    # ---- end to end through the public host-tensor operator: pinned host q, k, v in, pinned host o out, every
    # step; the operator cuts the heads into slices and overlaps their copies with the kernels.  Each rank moves
    # only its own heads.
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(q.shape, dtype=q.dtype).pin_memory()

    def e2e_step():
        qfa.quant_attention_host(hq, hk, hv, False, sm, out=ho, device=dev, slices=min(16, h1 - h0))

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    b_.record(stream)
    barrier()
    (e2e_ms,) = max_over_ranks(a.elapsed_time(b_) / e2e_steps)
    qfa.check_kernel_status()
    # bytes of the WHOLE job per step (all ranks), counted from the tensors that are copied
    frac = total_units / (h1 - h0)
    e2e = {"value": ops_total / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
           "h2d_bytes_per_step": int(3 * q.numel() * q.element_size() * frac),
           "d2h_bytes_per_step": int(q.numel() * q.element_size() * frac),
           "ms_per_step": e2e_ms, "steps": e2e_steps,
           "per_rank_h2d_GBps": 3 * q.numel() * q.element_size() / e2e_ms / 1e6}

    if rank == 0:
        print(json.dumps(result_line(args, world, value, ms_step, ms_total, attn_ms, ops_local, launches, clocks, e2e,
                                     extra, weak, h1 - h0)), flush=True)
    if world > 1:
        dist.destroy_process_group()


def result_line(args, world, value, ms_step, ms_total, attn_ms, ops_local, launches, clocks, e2e, extra, weak, n_local):
    peaks = load_peaks()
    long_run = ms_total > 2000.0
    peak = peaks["bf16_tflops_sustained"] if long_run else peaks["bf16_tflops"]
    achieved = ops_local / (attn_ms * 1e-3) / 1e12
    tp = extra.get("tensor_pipe_peaks_TOPS", {})
    roofline = {
        "bound": "tensor", "kernel": "attn_fwd_tc_kernel, centered route (int8 attention forward, rank 0's launch)",
        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "peak_kind": ("sustained" if long_run else "burst") + " bf16 dense (library GEMM), of " + peaks["source"],
        "frac_of_int8_nominal_4500": achieved / 4500.0,
        # DRAM bytes per launch: one profiler capture of the same kernel at B1 H16 (the full workload is too large
        # to capture) read 42.35 MB + wrote 0.84 MB for 16 heads; the centered K (1 MB per head), V^ (1 MB) and the
        # codes of Q (0.5 MB) are read once per head and O (written once) was still in L2 when that small kernel
        # ended, so the figure is per-head reads scaled by the heads of a launch plus the output bytes
        "traffic": n_local * (42.35e6 / 16) + n_local * S * D * 2,
        "traffic_note": "scaled from a 16-head capture: 2.65 MB read per head + output bytes",
        "ms_per_launch": attn_ms,
        "timing": "CUDA events around `steps` launches of the forward alone, right after the step loop",
    }
    if "int8_ss_n128" in tp:
        # both products of the kernel run as 16-bit MMAs (Q'.K'^T over the centered codes, P.V): the probe's measured
        # issue rate of that form is the tensor-pipe floor.  The int8 figures are kept for context: with the int8
        # MMA route half of the operations would run at the int8 rate (mixed floor).
        i8, bf = tp["int8_ss_n128"], tp["bf16_ts_n128"]
        roofline["peak_int8_measured"] = i8
        roofline["peak_bf16_mma_measured"] = bf
        roofline["frac_of_bf16_mma_measured"] = achieved / bf
        roofline["frac_of_int8_measured"] = achieved / i8
        roofline["frac_of_mixed_int8_bf16_measured"] = achieved * (0.5 / i8 + 0.5 / bf)
    else:
        roofline["frac_of_mixed_int8_bf16"] = achieved / (1.0 / (0.5 / (2 * peak) + 0.5 / peak))
    cpu_baseline = None
    if world == 1:
        cpu_rate, cpu_dt, threads = cpu_reference_sample(2, S, D, 2)
        cpu_baseline = {"value": cpu_rate / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
                        "sample": f"2 of {B * H} heads (S={S}, D={D}) x2 repeats, {cpu_dt:.1f} s, PyTorch CPU fp32 oracle"}
    line = {
        "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak" if weak else "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B * world if weak else B, "heads": H, "seq_len": S,
                   "head_dim": D,
                   "partition": (f"replicas: B4 H32 on each of {world} GPUs" if weak else
                                 f"{B * H} (batch x head) units cut into {world} contiguous slices, {n_local} per GPU"),
                   "l2": f"inputs larger than L2: a step reads {3 * n_local * S * D * 2 / 1e6:.0f} MB of q, k, v per GPU and "
                         f"the steps rotate over {extra.get('rotating_input_copies')} copies of them at different "
                         "addresses (>= 252 MB touched between two uses of a copy; L2 is 126 MB)",
                   "launch": extra.get("launch_mode")},
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "extra": extra,
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    return line


def run_profile_case(case: str):
    """A small case of one kernel, launched twice, for a profiler capture: large enough that the operands
    exceed L2 only for the quantizer (1 Mi tokens); the attention cases are B1 H16 S4096 D128 (a few hundred
    microseconds per launch, 1.7 waves of CTAs)."""
    import quant_flash_attn_b200 as qfa
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    if case == "quant":
        x = torch.randn(8, 32, 4096, 128, device=dev, dtype=torch.bfloat16)
        for _ in range(2):
            out = qfa.asymmetric_quant_per_token_ex(x)      # codes, scale, zero point and code sums, as in the bench step
        torch.cuda.synchronize()
        print("ok", int(out[3].sum()))
        return
    if case in ("shortq", "q32", "midq"):
        # the reference's own regime (test_speed.py:69-77) at a quarter of its batch: Z64 H16 NQ16 NKV2048 D128 fp16;
        # "midq" / "q32": 128 / 32 query rows, the one-tile tcgen05 forwards that dequantize K/V inside the kernel
        z, hh, nq, nkv, dd = 64, 16, {"shortq": 16, "q32": 32, "midq": 128}[case], 2048, 128
        q = torch.randn(z, hh, nq, dd, device=dev, dtype=torch.float16, requires_grad=True)
        kv = torch.randn(z, hh, nkv, dd, device=dev, dtype=torch.float16, requires_grad=True)
        go = torch.randn_like(q)
        kvq = qfa.asymmetric_quant_per_token(kv.detach())
        for _ in range(2):
            o = qfa.quant_flash_attn(q, kv, kvq, 1.0 / math.sqrt(dd))
            o.backward(go)
        torch.cuda.synchronize()
        print("ok", float(kv.grad.float().abs().mean()))
        return
    b, h, s, d = 1, 16, 4096, 128
    causal = case == "fwd_causal"
    sm = 1.0 / math.sqrt(d)
    q, k, v, do = (torch.randn(b, h, s, d, device=dev, dtype=torch.bfloat16) for _ in range(4))
    qq, kq, vq = qfa.quantize_qkv(q, k, v)
    reps = 1 if case == "bwd" else 2
    for _ in range(reps):
        o, lse = qfa.int8_attention_forward(qq, kq, vq, causal, sm, torch.bfloat16)
    if case == "bwd":
        for _ in range(2):
            dq, dk, dv = qfa.int8_attention_backward(qq, kq, vq, False, sm, o, lse, do)
        o = dq
    torch.cuda.synchronize()
    print("ok", float(o.float().abs().mean()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="with --gpus N > 1: partition the fixed workload (strong) or replicate it per GPU (weak)")
    ap.add_argument("--skip-extras", action="store_true", help="only the timed step loop and the end-to-end leg")
    ap.add_argument("--eager", action="store_true", help="launch every step eagerly instead of replaying CUDA graphs")
    ap.add_argument("--profile-case", default=None, choices=["quant", "fwd", "fwd_causal", "bwd", "shortq", "q32", "midq"])
    args = ap.parse_args()
    StepGraphs.eager_only = args.eager
    if args.profile_case:
        run_profile_case(args.profile_case)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
