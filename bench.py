#!/usr/bin/env python
"""Benchmark of the streaming-attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg2|cfg5] [--impl reference]

One step = one forward + backward of the operator over one batch of synthetic input.
Prints ONE JSON line on rank 0:

* ``value``     useful (unmasked) TFLOP/s of the whole job, inputs resident in HBM, timed with
                CUDA events on the launching stream, max over ranks;
* ``e2e``       the same metric through the public Python API with HOST (pinned) buffers:
                host->device copies of q, k, v, dO and device->host copies of O, dQ, dK, dV
                are inside the timed region;
* ``roofline``  the dominant kernel (the backward kernel that forms dK and dV) against the measured bf16
                tensor peak;
* ``cpu_baseline`` the CPU oracle (a port of the reference's torch masked-attention path)
                timed on this machine's host cores on a bounded sample of the same workload.

``--impl reference`` times that CPU path alone (rank 0 only) and prints the same line shape.
``--impl context`` (one GPU) times other implementations on the same GPU and inputs for context: the
reference's own Triton kernel (from ``oracle/_ref``, in a child process), compiled ``flex_attention`` with
the streaming block mask and torch SDPA with the dense mask.
``--workload step`` times the streaming inference step, ``--workload cfg4`` dense self-attention and softmax,
``--workload proj`` the fused QKV + RoPE and output projections, ``--workload fp8`` the e4m3 forward.

Multi-GPU: launched by ``torch.distributed.run`` with one rank per GPU.  The batch x heads
slices are sharded over ranks (weak scaling for cfg3/cfg2: every rank gets a full copy of the
single-GPU workload's size; strong scaling for cfg5); there is no collective on the data path,
NCCL carries only the timing barrier and the max-reduction of the elapsed time.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # the long-sequence configuration the >= 60 %-of-peak target is quoted on
    "cfg3": dict(dtype="bf16", B=4, H=32, T=16384, D=128, c=256, back=2, lens=None, qk_scale=1.0, scaling="weak",
                 desc="bf16 B=4 H=32 T=16384 D=128 context=256 back=2 lens=T (per GPU)"),
    # the fp16 head-dim-64 configuration with random lengths
    "cfg2": dict(dtype="f16", B=8, H=16, T=4096, D=64, c=128, back=4, lens=(2048, 4096), qk_scale=64 ** -0.25,
                 scaling="weak", desc="fp16 B=8 H=16 T=4096 D=64 context=128 back=4 lens~U[2048,4096] (per GPU)"),
    # the multi-GPU configuration: fixed total problem, batch x heads split over the GPUs
    "cfg5": dict(dtype="bf16", B=64, H=32, T=8192, D=128, c=64, back=8, lens=(4096, 8192), qk_scale=1.0,
                 scaling="strong", desc="bf16 B=64 H=32 T=8192 D=128 context=64 back=8 lens~U[4096,8192] (total)"),
    # small stand-in for cfg5 (same tiles, schedule and length distribution, 1/16 of the batch) for ncu captures
    "prof5": dict(dtype="bf16", B=4, H=32, T=8192, D=128, c=64, back=8, lens=(4096, 8192), qk_scale=1.0, scaling="weak",
                  desc="bf16 B=4 H=32 T=8192 D=128 context=64 back=8 lens~U[4096,8192] (profiling case)"),
    # small stand-in for cfg3 (same tiles and schedule, 1/4 of the slices) for ncu captures
    "prof": dict(dtype="bf16", B=2, H=16, T=16384, D=128, c=256, back=2, lens=None, qk_scale=1.0, scaling="weak",
                 desc="bf16 B=2 H=16 T=16384 D=128 context=256 back=2 lens=T (profiling case)"),
}
TORCH_DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant backward kernel, per (batch, head)
# slice of T=16384, D=128, c=256, back=2, lens=T, from ncu captures of workload `prof` (32 slices; see profiles/).
# Traffic is proportional to the number of slices: every slice reads Q, K, V, dO once and writes dK, dV once
# (two-pass dK/dV pass: 782 MB), plus, in the single-evaluation main kernel, its 16-bit dS tiles (1 624 MB).
NCU_TRAFFIC_PER_SLICE = {"bwd_dkdv_pass": {"cfg3": 782e6 / 32, "prof": 782e6 / 32},
                         "bwd_main": {"cfg3": 1556e6 / 32, "prof": 1556e6 / 32}}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(tflops=p["bf16_tflops"], tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    hbm_gbs=p["hbm_gbs"], source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period, self.samples, self._stop, self._thr = index, period_s, [], threading.Event(), None

    def _run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            # NVML indexes physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if vis and all(x.strip().isdigit() for x in vis.split(",")):
                idx = int(vis.split(",")[self.index])
            hnd = nv.nvmlDeviceGetHandleByIndex(idx)
            mx = nv.nvmlDeviceGetMaxClockInfo(hnd, nv.NVML_CLOCK_SM)
            bits = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                    "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                    "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
            while not self._stop.is_set():
                sm = nv.nvmlDeviceGetClockInfo(hnd, nv.NVML_CLOCK_SM)
                rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(hnd)
                self.samples.append((float(sm), float(mx), [n for n, b in bits.items() if rs & b]))
                self._stop.wait(self.period)
        except Exception as e:  # no NVML: report that no clock record exists
            self.samples.append((None, None, [f"nvml unavailable: {type(e).__name__}"]))

    def __enter__(self):
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        time.sleep(0.05)
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thr.join(timeout=6)

    def summary(self):
        sm = [s[0] for s in self.samples if s[0] is not None]
        mx = [s[1] for s in self.samples if s[1] is not None]
        reasons = sorted({r for s in self.samples for r in s[2]})
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_min_mhz=min(sm) if sm else None,
                    sm_max_mhz=max(mx) if mx else None, reasons=reasons, samples=len(sm))


# ------------------------------------------------------------------------------------------
# workload construction
# ------------------------------------------------------------------------------------------
def _global_problem(w, n_gpus):
    """Global batch and lens for N GPUs (weak: batch grows with N; strong: fixed)."""
    from kernels_b200 import synthetic as SO

    B = w["B"] * n_gpus if w["scaling"] == "weak" else w["B"]
    lens = None
    if w["lens"] is not None:
        lens = SO.make_lens(B, w["lens"][0], w["lens"][1], seed=0)
    return B, lens


def _useful_pairs_total(w, B, lens, heads):
    from kernels_b200.sharding import useful_pairs

    T = w["T"]
    ls = [T] * B if lens is None else [min(int(x), T) for x in lens.tolist()]
    return heads * sum(useful_pairs(L, w["c"], w["back"]) for L in ls), heads * sum(ls)


def _make_local_inputs(w, B, heads, H, dtype, pin):
    """Host tensors [B, len(heads), T, D] for this rank, one seeded generator per (b, h) slice."""
    from kernels_b200 import synthetic as SO

    T, D = w["T"], w["D"]
    shape = (B, len(heads), T, D)
    host = [torch.empty(shape, dtype=dtype, pin_memory=pin) for _ in range(4)]
    for b in range(B):
        for j, h in enumerate(heads):
            sl = SO.make_slice(b, h, H, T, D, seed=0, qk_scale=w["qk_scale"])
            for dst, src in zip(host, sl):
                dst[b, j].copy_(src)
    return host  # q, k, v, do


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle port on the host cores
# ------------------------------------------------------------------------------------------
def _cpu_step(w, b, h, H, lens):
    """One CPU step = dense masked SDPA forward + backward of ONE (batch, head) slice."""
    from kernels_b200 import synthetic
    from oracle import streaming_attention_oracle as SO  # the CPU leg is the one place the oracle is timed

    q, k, v, do = synthetic.make_slice(b, h, H, w["T"], w["D"], seed=0, qk_scale=w["qk_scale"])
    lens_t = None if lens is None else lens[b:b + 1]
    t0 = time.perf_counter()
    SO.oracle_fwd_bwd(q[None, None], k[None, None], v[None, None], do[None, None], w["c"], w["back"], lens_t)
    return time.perf_counter() - t0


def _cpu_baseline(w, steps, warmup, budget_s=25.0):
    from kernels_b200.sharding import useful_pairs

    torch.set_num_threads(os.cpu_count() or 1)
    B, lens = _global_problem(w, 1)
    H, T = w["H"], w["T"]
    times, flops = [], []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        b, h = (i // H) % B, i % H
        dt = _cpu_step(w, b, h, H, lens)
        if i >= warmup:
            L = T if lens is None else min(int(lens[b]), T)
            times.append(dt)
            flops.append(14.0 * w["D"] * useful_pairs(L, w["c"], w["back"]))
        if budget_s is not None and time.perf_counter() - t_start > budget_s and len(times) >= 1:
            break
    tflops = sum(flops) / sum(times) / 1e12
    return dict(value=tflops, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{len(times)} (batch, head) slices of the workload, dense masked SDPA fwd+bwd in fp32, "
                       f"{statistics.mean(times) * 1e3:.0f} ms per slice"), statistics.mean(times) * 1e3


def _config_block(w, name, world):
    """The ``config`` of a bench line: the same for the own arm and the reference arm of one launch."""
    B, lens = _global_problem(w, world)
    H, T, D = w["H"], w["T"], w["D"]
    pairs_total, _ = _useful_pairs_total(w, B, lens, H)
    tensor_bytes = B * (H // world) * T * D * torch.empty(0, dtype=TORCH_DTYPES[w["dtype"]]).element_size()
    return {"workload": w["desc"], "name": name, "global_batch": B, "heads_per_gpu": H // world,
            "sharding": f"batch x heads, heads round-robin over {world} GPU(s), no collective",
            "l2": "inputs larger than L2 (no flush needed)" if 4 * tensor_bytes > 4 * 126e6 else "L2 not flushed",
            "useful_flops_per_step": 14.0 * D * pairs_total}


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, ms = _cpu_baseline(w, args.steps, args.warmup, budget_s=None)
    base["sample"] += "; one (batch, head) slice per step on the host cores"
    line = {
        "impl": "reference", "metric": "streaming-attn fwd+bwd useful TFLOP/s", "value": base["value"],
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config_block(w, args.workload, args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# own arm
# ------------------------------------------------------------------------------------------
def _bwd_params(lib_mod, q, k, v, o, do, lse, dq, dk, dv, delta, lens, w, flags, ds_ws=None):
    p = lib_mod.SaBwdParams()
    if ds_ws is not None:
        p.ds_ws, p.ds_ws_bytes = ds_ws.data_ptr(), ds_ws.numel()
    p.q, p.k, p.v, p.o, p.d_o = (lib_mod.tensor4(t) for t in (q, k, v, o, do))
    p.lse, p.dq, p.dk, p.dv, p.delta_ws = lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr()
    p.lens = lens.data_ptr() if lens is not None else None
    p.lens_stride = lens.stride(0) if lens is not None else 0
    p.B, p.H, p.T, p.D = q.shape
    p.dtype = lib_mod.dtype_code(q.dtype)
    p.context_size, p.back_contexts, p.sm_scale = w["c"], w["back"], float(w["D"] ** -0.5)
    p.flags = flags
    p.status = lib_mod.status_words().data_ptr()
    return p


def run_own(args, w):
    import torch.distributed as dist

    from kernels_b200 import _lib
    from kernels_b200.sharding import partition
    from kernels_b200.streaming_attention import streaming_attention

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    dtype = TORCH_DTYPES[w["dtype"]]
    H, T, D = w["H"], w["T"], w["D"]

    B, lens = _global_problem(w, world)
    shard = partition(B, H, world, None if lens is None else lens.tolist(), T=T, context_size=w["c"],
                      back_contexts=w["back"])[rank]
    assert shard.mode == "heads", "bench workloads have H divisible by the GPU count"
    heads = list(shard.heads)
    hq, hk, hv, hdo = _make_local_inputs(w, B, heads, H, dtype, pin=True)
    q, k, v, do = (t.to(dev) for t in (hq, hk, hv, hdo))
    lens_d = lens.to(dev) if lens is not None else None
    pairs_local, rows_local = _useful_pairs_total(w, B, lens, len(heads))
    pairs_total, _ = _useful_pairs_total(w, B, lens, H)
    flops_total = 14.0 * D * pairs_total
    scale = float(D ** -0.5)

    # ---- device-resident path through the C ABI, one call per kernel so each can be timed ----
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
    fp = _lib.SaFwdParams()
    fp.q, fp.k, fp.v = _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v)
    fp.o, fp.lse = o.data_ptr(), lse.data_ptr()
    fp.lens = lens_d.data_ptr() if lens_d is not None else None
    fp.lens_stride = lens_d.stride(0) if lens_d is not None else 0
    fp.B, fp.H, fp.T, fp.D = q.shape
    fp.dtype = _lib.dtype_code(dtype)
    fp.context_size, fp.back_contexts, fp.sm_scale, fp.flags = w["c"], w["back"], scale, 0
    fp.status = _lib.status_words().data_ptr()
    # backward: the single-evaluation kernels (delta, main = dK/dV/dS, dQ from the saved dS tiles), one
    # C-ABI call per kernel so that each can be timed; --two-pass times the dQ pass + dK/dV pass instead
    SKIP_DELTA, SKIP_MAIN, SKIP_DQ = _lib.KB_FLAG_BWD_SKIP_DELTA, _lib.KB_FLAG_BWD_SKIP_DKDV, _lib.KB_FLAG_BWD_SKIP_DQ
    if args.two_pass:
        kernel_names = ("fwd", "bwd_dq_pass", "bwd_dkdv_pass")
        bwd_calls = [_bwd_params(_lib, q, k, v, o, do, lse, dq, dk, dv, delta, lens_d, w, f | _lib.KB_FLAG_BWD_TWO_PASS)
                     for f in (SKIP_MAIN, SKIP_DQ)]
    else:
        ws_bytes = int(lib.kb_sa_bwd_workspace_bytes(*q.shape, _lib.dtype_code(dtype), w["c"], w["back"]))
        ds_ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        kernel_names = ("fwd", "bwd_delta", "bwd_main", "bwd_dq")
        bwd_calls = [_bwd_params(_lib, q, k, v, o, do, lse, dq, dk, dv, delta, lens_d, w, f, ds_ws)
                     for f in (SKIP_MAIN | SKIP_DQ, SKIP_DELTA | SKIP_DQ, SKIP_DELTA | SKIP_MAIN)]
    stream = torch.cuda.current_stream(dev)

    def step(events=None):
        marks = []
        for fn, prm in [(lib.kb_sa_fwd, fp)] + [(lib.kb_sa_bwd, b_) for b_ in bwd_calls]:
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            _lib.check(fn(ctypes.byref(prm), stream.cuda_stream), "bench step")
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record(stream)
                marks.append((e0, e1))
        if events is not None:
            events.append(marks)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.check_device_status()

    launches0 = _lib.launch_count()
    per_kernel = []
    with ClockSampler(local_rank) as clk:
        barrier()
        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_begin.record(stream)
        for _ in range(args.steps):
            step(per_kernel)
        t_end.record(stream)
        barrier()
    launches = _lib.launch_count() - launches0
    _lib.check_device_status()
    elapsed_ms = t_begin.elapsed_time(t_end)
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12
    k_ms = {name: statistics.mean(m[i][0].elapsed_time(m[i][1]) for m in per_kernel)
            for i, name in enumerate(kernel_names)}

    # ---- end to end through the public API with host buffers ----
    # The batch is cut into chunks of at least ~128 MB of input; chunk i's host->device copies, chunk
    # i-1's forward + backward and chunk i-2's device->host copies run on three streams, so the two PCIe
    # directions and the GPU work overlap.  Every chunk goes through the public streaming_attention().
    in_bytes = 4 * q.numel() * q.element_size()
    n_chunks = max(1, min(B, in_bytes // (128 << 20)))
    while B % n_chunks:
        n_chunks -= 1
    cb = B // n_chunks  # batch elements per chunk
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    host_in = [[t[i * cb:(i + 1) * cb] for t in (hq, hk, hv, hdo)] for i in range(n_chunks)]
    host_out = [[torch.empty((cb,) + tuple(q.shape[1:]), dtype=dtype, pin_memory=True) for _ in range(4)]
                for _ in range(n_chunks)]
    dev_in = [[torch.empty((cb,) + tuple(q.shape[1:]), dtype=dtype, device=dev) for _ in range(4)] for _ in range(n_chunks)]
    for bufs in dev_in:
        for t_ in bufs[:3]:
            t_.requires_grad_()
    lens_chunks = [None if lens_d is None else lens_d[i * cb:(i + 1) * cb] for i in range(n_chunks)]
    computed = [None] * n_chunks  # per chunk: event after its last forward + backward (readers of dev_in[i])

    def e2e_step():
        done = []
        for i in range(n_chunks):
            qd, kd, vd, dod = dev_in[i]
            ev_in = torch.cuda.Event()
            with torch.cuda.stream(s_in), torch.no_grad():
                if computed[i] is not None:
                    s_in.wait_event(computed[i])  # last step's kernels have read the chunk's buffers
                for dst, src in zip((qd, kd, vd, dod), host_in[i]):
                    dst.copy_(src, non_blocking=True)
                ev_in.record(s_in)
            stream.wait_event(ev_in)
            for t_ in (qd, kd, vd):
                t_.grad = None
            out = streaming_attention(qd, kd, vd, lens_chunks[i], w["c"], w["back"])
            out.backward(dod)
            ev_c = torch.cuda.Event()
            ev_c.record(stream)
            computed[i] = ev_c
            results = (out.detach(), qd.grad, kd.grad, vd.grad)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                for dst, src in zip(host_out[i], results):
                    dst.copy_(src, non_blocking=True)
            done.append(results)  # keeps the device results allocated until the copies are ordered below
        # the launching stream joins the copy streams: work queued after this step (which may reuse the
        # results' memory once `done` is dropped) runs after this step's device->host copies
        stream.wait_stream(s_out)
        stream.wait_stream(s_in)

    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 10))
    for _ in range(3 if e2e_steps else 0):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / max(e2e_steps, 1)
    # the link the end-to-end leg is bound by: plain pinned copies of one chunk's tensors, each direction
    # alone and both at once (outside the timed region; boxes of one pool differ in what they reach)
    pcie = None
    if e2e_steps:
        def copy_rate(h2d, d2h):
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            c0.record(stream)
            s_in.wait_stream(stream)
            s_out.wait_stream(stream)
            with torch.no_grad():
                if h2d:
                    with torch.cuda.stream(s_in):
                        for dst, src in zip(dev_in[0], host_in[0]):
                            dst.copy_(src, non_blocking=True)
                if d2h:
                    with torch.cuda.stream(s_out):
                        for dst, src in zip(host_out[0], dev_in[-1]):
                            dst.copy_(src, non_blocking=True)
            stream.wait_stream(s_in)
            stream.wait_stream(s_out)
            c1.record(stream)
            torch.cuda.synchronize(dev)
            one_way = 4 * dev_in[0][0].numel() * dev_in[0][0].element_size()
            return one_way / (c0.elapsed_time(c1) * 1e-3) / 1e9
        copy_rate(True, True)
        pcie = {"h2d_gbs": copy_rate(True, False), "d2h_gbs": copy_rate(False, True),
                "both_gbs_per_direction": copy_rate(True, True)}
    tensor_bytes = q.numel() * q.element_size()
    _lib.check_device_status()
    config5 = None
    if args.workload == "cfg3" and not args.no_config5:
        config5 = _config5_block(lib, dev, rank, world)

    if rank == 0:
        peaks = _peaks()
        peak = peaks["tflops_sustained"] if ms_per_step * args.steps > 500 else peaks["tflops"]
        # dominant kernel: the one that forms dK and dV (and, in the single-evaluation family, saves
        # dS); its algorithmic work is the 4 matmuls S, dP, dV, dK
        dom = "bwd_dkdv_pass" if args.two_pass else "bwd_main"
        dkdv_flops = 8.0 * D * pairs_local
        achieved = dkdv_flops / (k_ms[dom] * 1e-3) / 1e12
        k_flops = {"fwd": 4.0, "bwd_dq_pass": 2.0, "bwd_dkdv_pass": 8.0, "bwd_main": 8.0, "bwd_dq": 2.0}
        el = q.element_size()
        line = {
            "metric": "streaming-attn fwd+bwd useful TFLOP/s", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "impl": "kernels_b200",
            "config": _config_block(w, args.workload, world),
            "per_gpu_tflops": value / world,
            "frac_of_bf16_peak": {"measured_burst": value / world / peaks["tflops"],
                                  "measured_sustained": value / world / peaks["tflops_sustained"],
                                  "spec_2250": value / world / 2250.0},
            "kernel_ms": k_ms,
            "kernel_tflops": {n_: k_flops[n_] * D * pairs_local / ms_ / 1e9 for n_, ms_ in k_ms.items() if n_ in k_flops},
            "roofline": {"kernel": "backward dK/dV pass" if args.two_pass else "backward main kernel (dK, dV, dS)",
                         "bound": "tensor", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peaks["source"],
                         "traffic": (NCU_TRAFFIC_PER_SLICE[dom][args.workload] * B * len(heads)
                                     if args.workload in NCU_TRAFFIC_PER_SLICE.get(dom, {}) else None),
                         "algorithmic_flops_per_launch": dkdv_flops,
                         "hbm_min_bytes_fwd_bwd": 12 * rows_local * D * el + 8 * rows_local,
                         "hbm_frac_if_min_traffic": (12 * rows_local * D * el + 8 * rows_local) / (ms_per_step * 1e-3) / 1e9
                         / peaks["hbm_gbs"]},
            "e2e": None if not e2e_steps else {"value": flops_total / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 4 * tensor_bytes * world, "d2h_bytes_per_step": 4 * tensor_bytes * world,
                    "steps": e2e_steps, "pcie_copy_rates": pcie},
            "gpu_launches": launches,
            "clocks": clk.summary(),
        }
        if config5 is not None:
            line["config5"] = config5
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = _cpu_baseline(w, steps=6, warmup=1, budget_s=25.0)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _config5_block(lib, dev, rank, world, steps=5, warmup=3):
    """The multi-GPU configuration as a STRONG-scaling record beside the headline: bf16 B=64 H=32 T=8192 D=128
    context=64 back=8 lens~U[4096,8192], one fixed problem whose batch x heads slices ``sharding.partition``
    spreads over the ranks (no collective).  Forward + backward through the C ABI (``kb_sa_fwd``, one
    ``kb_sa_bwd``), device-resident, CUDA events, max over ranks.  With more than one rank, rank 0 then runs
    the WHOLE problem alone (the other GPUs idle) so that the record carries its own t_1 and the efficiency
    t_1 / (N t_N).  Inputs are seeded per (batch, head) slice on the device (the same slice gets the same
    values whatever the GPU count)."""
    import torch.distributed as dist

    from kernels_b200 import _lib
    from kernels_b200.sharding import partition, useful_pairs

    w = WORKLOADS["cfg5"]
    B, H, T, D, c, back = w["B"], w["H"], w["T"], w["D"], w["c"], w["back"]
    dtype = TORCH_DTYPES[w["dtype"]]
    _, lens = _global_problem(w, 1)
    lens_list = [min(int(x), T) for x in lens.tolist()]
    lens_d = lens.to(dev)
    shards = partition(B, H, world, lens_list, T=T, context_size=c, back_contexts=back)
    pairs_per_head = sum(useful_pairs(L, c, back) for L in lens_list)
    stream = torch.cuda.current_stream(dev)

    def timed(heads):
        nh = len(heads)
        gen = torch.Generator(device=dev)
        q, k, v, do = (torch.empty((B, nh, T, D), dtype=dtype, device=dev) for _ in range(4))
        rows = torch.arange(T, device=dev)[:, None]
        for b in range(B):
            for j, h in enumerate(heads):
                gen.manual_seed(1_000_003 * 5 + b * H + h)
                for dst in (q, k, v):
                    dst[b, j].copy_(torch.randn(T, D, device=dev, generator=gen))
                do[b, j].copy_(torch.randn(T, D, device=dev, generator=gen) * (rows < lens_list[b]))
        o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        lse = torch.empty((B, nh, T), dtype=torch.float32, device=dev)
        delta = torch.empty_like(lse)
        ws = int(lib.kb_sa_bwd_workspace_bytes(B, nh, T, D, _lib.dtype_code(dtype), c, back))
        ds_ws = torch.empty(ws, dtype=torch.uint8, device=dev)
        fp = _lib.SaFwdParams()
        fp.q, fp.k, fp.v = _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v)
        fp.o, fp.lse = o.data_ptr(), lse.data_ptr()
        fp.lens, fp.lens_stride = lens_d.data_ptr(), lens_d.stride(0)
        fp.B, fp.H, fp.T, fp.D = q.shape
        fp.dtype = _lib.dtype_code(dtype)
        fp.context_size, fp.back_contexts, fp.sm_scale, fp.flags = c, back, float(D ** -0.5), 0
        fp.status = _lib.status_words().data_ptr()
        bp = _bwd_params(_lib, q, k, v, o, do, lse, dq, dk, dv, delta, lens_d, w, 0, ds_ws)

        def step():
            _lib.check(lib.kb_sa_fwd(ctypes.byref(fp), stream.cuda_stream), "config5 forward")
            _lib.check(lib.kb_sa_bwd(ctypes.byref(bp), stream.cuda_stream), "config5 backward")

        for _ in range(warmup):
            step()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize(dev)
        _lib.check_device_status()
        return e0.elapsed_time(e1) / steps

    shard = shards[rank]
    assert shard.mode == "heads", "H = 32 is divisible by 1, 2, 4 and 8 GPUs"
    if world > 1:
        dist.barrier()
    ms = timed(list(shard.heads))
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_n = float(t.item())
    flops = 14.0 * D * H * pairs_per_head
    block = {"workload": w["desc"], "scaling": "strong", "n_gpus": world, "ms_per_step": ms_n,
             "tflops": flops / ms_n / 1e9, "useful_flops_per_step": flops, "steps": steps, "warmup": warmup,
             "heads_per_gpu": len(shard.heads),
             "work_spread_max_over_mean": 1.0,  # heads round-robin: every rank holds every batch entry's lens
             "sharding": f"heads round-robin over {world} GPU(s), every rank sees all {B} lengths"}
    if world > 1:
        torch.cuda.empty_cache()
        ms_1 = timed(list(range(H))) if rank == 0 else 0.0
        dist.barrier()
        block["ms_per_step_one_gpu_same_run"] = ms_1
        block["strong_scaling_efficiency"] = ms_1 / (world * ms_n) if rank == 0 else None
    torch.cuda.empty_cache()
    return block


def run_dense(args):
    """The dense configuration: self-attention forward (fp16 B=16 H=16 T=2048 D=64, key padding
    lens ~ U[1024, 2048]) and row softmax (fp32 [65536, 4096] ~ N(0, 4)), one GPU.  Each iteration is
    timed with its own event pair; a 512 MB buffer is rewritten between iterations to flush L2."""
    from kernels_b200 import _lib, synthetic
    from kernels_b200.self_attention import self_attention
    from kernels_b200.softmax import softmax

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def timed(fn, steps, warmup):
        for _ in range(max(warmup, 3)):
            fn()
        ts = []
        for _ in range(steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    B, H, T, D = 16, 16, 2048, 64
    g = torch.Generator(device=dev).manual_seed(0)
    q, k, v = (torch.randn(B, H, T, D, device=dev, generator=g).half() for _ in range(3))
    lens = synthetic.make_lens(B, 1024, 2048, seed=0).to(dev)
    launches0 = _lib.launch_count()
    with ClockSampler(0) as clk:
        fa_ms = timed(lambda: self_attention(q, k, v, lens), args.steps, args.warmup)
        x = torch.randn(65536, 4096, device=dev, generator=g) * 2.0
        sm_ms = timed(lambda: softmax(x), args.steps, args.warmup)
    fa_flops = 4.0 * D * H * float((lens.double() ** 2).sum())
    sm_bytes = 2.0 * x.numel() * 4
    line = {
        "metric": "dense self-attention fwd useful TFLOP/s; row softmax GB/s", "value": fa_flops / fa_ms / 1e9,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": fa_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "impl": "kernels_b200",
        "config": {"workload": "fp16 B=16 H=16 T=2048 D=64 non-causal lens~U[1024,2048]; softmax fp32 [65536,4096]",
                   "name": "cfg4", "l2": "flushed between iterations (512 MB write)"},
        "softmax": {"ms": sm_ms, "gbs": sm_bytes / sm_ms / 1e6, "algorithmic_bytes": sm_bytes},
        "roofline": {"kernel": "softmax_rows_kernel", "bound": "hbm", "achieved": sm_bytes / sm_ms / 1e6,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": sm_bytes / sm_ms / 1e6 / peaks["hbm_gbs"],
                     "peak_source": peaks["source"], "traffic": None},
        "gpu_launches": _lib.launch_count() - launches0, "clocks": clk.summary(),
    }
    print(json.dumps(line))


def run_step(args):
    """The streaming inference step (no counterpart in the reference's benchmarks): 64 streams x 32 heads,
    bf16 D=128 c=256 back=2, the 256 queries of the newest chunk against a cache of back + 1 = 3 chunks.
    K + V of the cache are 805 MB and q + o 268 MB: more than L2, no flush.  Useful FLOPs 4*D*pairs with
    pairs = c * 3c per (stream, head); algorithmic bytes: q, k, v read and o written once."""
    from kernels_b200 import _lib
    from kernels_b200.streaming_attention import streaming_attention_step

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    B, H, D, c, back = 64, 32, 128, 256, 2
    T = (back + 1) * c
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, H, c, D, device=dev, generator=g).bfloat16()
    k, v = (torch.randn(B, H, T, D, device=dev, generator=g).bfloat16() for _ in range(2))
    launches0 = _lib.launch_count()
    for _ in range(max(args.warmup, 3)):
        streaming_attention_step(q, k, v, None, c, back)
    torch.cuda.synchronize()
    with ClockSampler(0) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            streaming_attention_step(q, k, v, None, c, back)
        e1.record()
        torch.cuda.synchronize()
    _lib.check_device_status()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * D * B * H * c * T
    nbytes = 2.0 * (2 * q.numel() + 2 * k.numel())
    line = {
        "metric": "streaming step useful TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "kernels_b200",
        "config": {"workload": "bf16 64 streams H=32 D=128 context=256 back=2: newest chunk against a 3-chunk cache",
                   "name": "step", "l2": "inputs larger than L2 (no flush needed)"},
        "roofline": {"kernel": "sa_fwd_sm100_kernel (q_start = 512)", "bound": "hbm", "achieved": nbytes / ms / 1e6,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                     "peak_source": peaks["source"], "traffic": None, "algorithmic_bytes_per_launch": nbytes},
        "tensor_frac_of_measured": flops / ms / 1e9 / peaks["tflops"],
        "gpu_launches": _lib.launch_count() - launches0, "clocks": clk.summary(),
    }
    print(json.dumps(line))


REF_SRC = os.path.join(ROOT, "oracle", "_ref", "src")


def run_reference_triton_child(args, w):
    """Child process of ``--impl context``: the reference's own ``streaming_attention`` (its Triton kernels,
    ``autotune=False``: tiles of at most 64 x 64, src/streaming_attention/kernel.py:1143-1153, 1195-1211)
    on this GPU and the own arm's seeded inputs, forward + backward.  Runs in a process of its own because
    the reference registers operators under the names this package uses; it imports nothing of
    ``kernels_b200`` but the input recipe and the FLOP count."""
    sys.path.insert(0, REF_SRC)
    from streaming_attention import streaming_attention as ref_streaming_attention  # the reference's package

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = TORCH_DTYPES[w["dtype"]]
    H, T, D, c, back = w["H"], w["T"], w["D"], w["c"], w["back"]
    B, lens = _global_problem(w, 1)
    hq, hk, hv, hdo = _make_local_inputs(w, B, list(range(H)), H, dtype, pin=False)
    q, k, v, do = (t.to(dev) for t in (hq, hk, hv, hdo))
    lens_d = None if lens is None else lens.to(dev)
    pairs_total, _ = _useful_pairs_total(w, B, lens, H)
    flops = 14.0 * D * pairs_total
    steps, warm = max(1, min(args.steps, 10)), 3

    def fwd_bwd():
        qg, kg, vg = (t.detach().requires_grad_() for t in (q, k, v))
        ref_streaming_attention(qg, kg, vg, lens_d, c, back, autotune=False).backward(do)

    for _ in range(warm):
        fwd_bwd()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fwd_bwd()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    import triton

    print(json.dumps({"ms_per_step": ms, "tflops": flops / ms / 1e9, "autotune": False, "steps": steps,
                      "triton": triton.__version__, "tile": f"{min(64, max(32, 1 << (c - 1).bit_length()))} x same"}))


def _reference_triton(args):
    """Run the child above; returns its record or why there is none."""
    import subprocess

    if not os.path.isfile(os.path.join(REF_SRC, "streaming_attention", "kernel.py")):
        return {"unavailable": "oracle/_ref is not staged (python oracle/make_ref.py <reference checkout>)"}
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-triton", "--workload", args.workload,
           "--steps", str(args.steps)]
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's Triton kernels did not finish within 900 s"}
    lines = [ln for ln in res.stdout.strip().splitlines() if ln.startswith("{")]
    if res.returncode != 0 or not lines:
        tail = (res.stderr.strip().splitlines() or ["no output"])[-1]
        return {"unavailable": f"child exited {res.returncode}: {tail[:300]}"}
    return json.loads(lines[-1])


def run_proj(args):
    """The fused projections around the operator (no counterpart in the reference's benchmarks), at the long-sequence
    configuration's size with a model width of 4096: x [4, 16384, 4096] -> q [4, 32, 16384, 128], k, v [4, 8, 16384, 128]
    with rotary embedding (3.3 TFLOP), and o [4, 32, 16384, 128] -> y [4, 16384, 4096] (2.2 TFLOP), bf16.  The
    activations (537 MB) exceed L2; the weights (50 / 34 MB) stay in it.  torch.nn.functional.linear (cuBLAS) on
    the same shapes is timed beside them as context."""
    from kernels_b200 import _lib
    from kernels_b200.streaming_attention import output_projection, qkv_rope_projection, rope_tables

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    B, T, E, H, Hk, D = 4, 16384, 4096, 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(B, T, E, device=dev, generator=g).bfloat16()
    wqkv = (torch.randn((H + 2 * Hk) * D, E, device=dev, generator=g) * E ** -0.5).bfloat16()
    wo = (torch.randn(E, H * D, device=dev, generator=g) * (H * D) ** -0.5).bfloat16()
    o = torch.randn(B, H, T, D, device=dev, generator=g).bfloat16()
    cos, sin = rope_tables(T, D, device=dev)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    launches0 = _lib.launch_count()
    with ClockSampler(0) as clk:
        qkv_ms = timed(lambda: qkv_rope_projection(x, wqkv, H, Hk, D, cos, sin))
        out_ms = timed(lambda: output_projection(o, wo))
    launches = _lib.launch_count() - launches0
    _lib.check_device_status()
    lin_qkv_ms = timed(lambda: torch.nn.functional.linear(x, wqkv))
    lin_out_ms = timed(lambda: torch.nn.functional.linear(o.transpose(1, 2).reshape(B, T, H * D), wo))
    f_qkv, f_out = 2.0 * B * T * E * (H + 2 * Hk) * D, 2.0 * B * T * H * D * E
    ms = qkv_ms + out_ms
    peak = peaks["tflops_sustained"] if ms * args.steps > 500 else peaks["tflops"]
    line = {
        "metric": "fused QKV+RoPE and output projection TFLOP/s", "value": (f_qkv + f_out) / ms / 1e9, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "kernels_b200",
        "config": {"workload": "bf16 x [4,16384,4096] -> q [4,32,16384,128], k, v [4,8,16384,128] with RoPE; o -> y [4,16384,4096]",
                   "name": "proj", "l2": "activations larger than L2 (no flush needed)"},
        "kernel_ms": {"qkv_rope_proj": qkv_ms, "out_proj": out_ms},
        "kernel_tflops": {"qkv_rope_proj": f_qkv / qkv_ms / 1e9, "out_proj": f_out / out_ms / 1e9},
        "context_cublas_linear_ms": {"qkv (no RoPE, no head layout)": lin_qkv_ms, "out (incl. the transpose copy of o)": lin_out_ms},
        "roofline": {"kernel": "proj_sm100_kernel (QKV + RoPE)", "bound": "tensor", "achieved": f_qkv / qkv_ms / 1e9,
                     "peak": peak, "unit": "TFLOP/s", "frac": f_qkv / qkv_ms / 1e9 / peak, "peak_source": peaks["source"],
                     "traffic": None, "algorithmic_flops_per_launch": f_qkv},
        "gpu_launches": launches, "clocks": clk.summary(),
    }
    print(json.dumps(line))


def run_fp8(args):
    """The e4m3 forward (no counterpart in the reference's benchmarks) at the long-sequence configuration's shape: B=4
    H=32 T=16384 D=128 context=256 back=2, lens = T; q, k, v ~ N(0, 1) quantised per tile of 128 rows.  Useful FLOPs
    4*D*pairs; the 16-bit forward on the dequantised inputs is timed beside it.  q, k, v are 268 MB each (8-bit) plus
    537 MB of output: more than L2, no flush."""
    from kernels_b200 import _lib
    from kernels_b200.sharding import useful_pairs
    from kernels_b200.streaming_attention import (dequantize_fp8_tiles, quantize_fp8_tiles, streaming_attention,
                                                  streaming_attention_fp8)

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    B, H, T, D, c, back = 4, 32, 16384, 128, 256, 2
    g = torch.Generator(device=dev).manual_seed(0)
    q8, qs = quantize_fp8_tiles(torch.randn(B, H, T, D, device=dev, generator=g))
    k8, ks = quantize_fp8_tiles(torch.randn(B, H, T, D, device=dev, generator=g))
    v8, vs = quantize_fp8_tiles(torch.randn(B, H, T, D, device=dev, generator=g))
    q16, k16, v16 = (dequantize_fp8_tiles(a, b).bfloat16() for a, b in ((q8, qs), (k8, ks), (v8, vs)))

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    launches0 = _lib.launch_count()
    with ClockSampler(0) as clk:
        ms8 = timed(lambda: streaming_attention_fp8(q8, k8, v8, qs, ks, vs, None, c, back))
    launches = _lib.launch_count() - launches0
    with torch.no_grad():
        ms16 = timed(lambda: streaming_attention(q16, k16, v16, None, c, back))
        o8 = streaming_attention_fp8(q8, k8, v8, qs, ks, vs, None, c, back).float()
        o16 = streaming_attention(q16, k16, v16, None, c, back).float()
    _lib.check_device_status()
    rel = float((o8 - o16).norm() / o16.norm())
    flops = 4.0 * D * B * H * useful_pairs(T, c, back)
    line = {
        "metric": "streaming-attn forward useful TFLOP/s, e4m3 inputs", "value": flops / ms8 / 1e9, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms8, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e4m3", "data": "synthetic", "impl": "kernels_b200",
        "config": {"workload": "e4m3 q, k, v with per-128-row scales, B=4 H=32 T=16384 D=128 context=256 back=2 lens=T, forward",
                   "name": "fp8", "l2": "inputs larger than L2 (no flush needed)"},
        "bf16_forward_same_inputs": {"ms_per_step": ms16, "tflops": flops / ms16 / 1e9},
        "rel_l2_vs_bf16_forward": rel,
        "roofline": {"kernel": "sa_fwd_sm100_kernel (e4m3)", "bound": "tensor", "achieved": flops / ms8 / 1e9,
                     "peak": 2 * peaks["tflops"], "unit": "TFLOP/s", "frac": flops / ms8 / 1e9 / (2 * peaks["tflops"]),
                     "peak_source": peaks["source"] + " bf16 peak x 2 (8-bit instructions cover twice the reduction length)",
                     "traffic": None, "algorithmic_flops_per_launch": flops},
        "gpu_launches": launches, "clocks": clk.summary(),
    }
    print(json.dumps(line))


def run_context(args, w):
    """Context, not an arm of the comparison: library kernels on the SAME GPU and the SAME inputs as the
    own arm (the reference's benchmark times these beside its kernel,
    benchmark/benchmark_streaming_attention.py:173-243): ``flex_attention`` compiled with the streaming mask
    as a block mask, and torch SDPA with the dense boolean mask where T x T fits.  Forward + backward,
    useful TFLOP/s by the own arm's formula.  The reference's own Triton kernel is timed first, in a
    child process (``run_reference_triton_child``)."""
    ref_triton = _reference_triton(args)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = TORCH_DTYPES[w["dtype"]]
    H, T, D, c, back = w["H"], w["T"], w["D"], w["c"], w["back"]
    B, lens = _global_problem(w, 1)
    hq, hk, hv, hdo = _make_local_inputs(w, B, list(range(H)), H, dtype, pin=False)
    q, k, v, do = (t.to(dev) for t in (hq, hk, hv, hdo))
    lens_d = torch.full((B,), T, dtype=torch.int32, device=dev) if lens is None else lens.to(dev)
    pairs_total, _ = _useful_pairs_total(w, B, lens, H)
    flops = 14.0 * D * pairs_total
    scale = float(D ** -0.5)
    steps, warm = max(1, min(args.steps, 10)), 3

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def fwd_bwd(attn):
        qg, kg, vg = (t.detach().requires_grad_() for t in (q, k, v))
        attn(qg, kg, vg).backward(do)

    out = {"reference_triton": ref_triton}
    try:
        from torch.nn.attention.flex_attention import create_block_mask, flex_attention

        def mask_mod(b, h, qi, ki):
            d = qi // c - ki // c
            return (d >= 0) & (d <= back) & (qi < lens_d[b]) & (ki < lens_d[b])

        bm = create_block_mask(mask_mod, B, None, T, T, device=dev, BLOCK_SIZE=128)
        flex = torch.compile(flex_attention, dynamic=False)
        ms = timed(lambda: fwd_bwd(lambda a, b_, c_: flex(a, b_, c_, block_mask=bm, scale=scale)))
        out["flex_attention"] = {"ms_per_step": ms, "tflops": flops / ms / 1e9, "block_size": 128}
    except Exception as e:  # context only: say why it is missing
        out["flex_attention"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    torch.cuda.synchronize()
    try:
        if B * T * T > 6e9:
            raise RuntimeError("dense mask too large")
        pos = torch.arange(T, device=dev)
        d = pos[:, None] // c - pos[None, :] // c
        band = (d >= 0) & (d <= back)
        valid = pos[None, :] < lens_d[:, None]
        mask = (band[None] & valid[:, :, None] & valid[:, None, :])[:, None]
        mask = mask | ~valid[:, None, :, None]  # padded rows see everything: no NaN (their dO is zero)
        ms = timed(lambda: fwd_bwd(lambda a, b_, c_: torch.nn.functional.scaled_dot_product_attention(
            a, b_, c_, attn_mask=mask, scale=scale)))
        out["sdpa_dense_mask"] = {"ms_per_step": ms, "tflops": flops / ms / 1e9}
    except Exception as e:
        out["sdpa_dense_mask"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    print(json.dumps({"impl": "context", "metric": "streaming-attn fwd+bwd useful TFLOP/s", "unit": "TFLOP/s",
                      "n_gpus": 1, "steps": steps, "warmup": warm, "dtype": w["dtype"], "data": "synthetic",
                      "config": {"workload": w["desc"], "name": args.workload}, "library_kernels": out}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS) + ["cfg4", "step", "proj", "fp8"])
    ap.add_argument("--impl", default="own", choices=["own", "reference", "context", "reference-triton"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-config5", action="store_true",
                    help="skip the strong-scaling record of the multi-GPU configuration (profiling runs)")
    ap.add_argument("--two-pass", action="store_true",
                    help="time the two-pass backward (dQ pass + dK/dV pass) instead of the single-evaluation kernels")
    args = ap.parse_args()
    if args.workload == "cfg4":
        return run_dense(args)
    if args.workload == "step":
        return run_step(args)
    if args.workload == "proj":
        return run_proj(args)
    if args.workload == "fp8":
        return run_fp8(args)
    w = WORKLOADS[args.workload]
    if args.impl == "context":
        return run_context(args, w)
    if args.impl == "reference-triton":
        return run_reference_triton_child(args, w)
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_own(args, w)


if __name__ == "__main__":
    main()
