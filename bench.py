#!/usr/bin/env python
"""Benchmark of the LSTM hot path (one JSON line on stdout, printed by rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1..c5] [--impl ours|reference|cudnn]

A step is one forward+backward pass (forward only for c2) of the stacked LSTM
over one batch of seeded synthetic input.  Workloads c1..c5 are the five shapes listed in WORKLOADS;
the default (c5: 2-layer bf16, global B=4096 split over the ranks, T=256,
I=H=512, fwd+bwd, weight-gradient allreduce) is the one whose metric is quoted
at 1/2/4/8 GPUs, so the same workload runs at every N (strong scaling).

  value     whole-job layer-tokens/s (L*B*T per step / time), inputs resident in HBM
  e2e       same metric through FastLSTM with pinned-host inputs copied in and the
            step's result (the final hidden state; with --e2e-copy-out also the whole
            output sequence) copied back to pinned host memory inside the timed region;
            the line says what stays on the device
  roofline  both persistent recurrence kernels timed alone with CUDA events; the
            slower one is reported as the dominant kernel
  cudnn     torch.nn.LSTM (cuDNN) on the same GPU, same dtype, same inputs and step
            definition, weights flattened once; timed after the headline region
            (1 GPU only).  `--impl cudnn` prints that arm as a line of its own.
  cpu_baseline / --impl reference
            torch.nn.LSTM fp32 on the host cores (the reference project's own CPU
            oracle), on a bounded batch sample of the same workload
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: dtype, L, B(global), T, I=H, backward, batch_first, h0_std, terminal grads
    "c1": dict(dtype="fp32", L=1, B=16, T=64, H=128, bwd=True, batch_first=True, h0=0.1, term=True),
    "c2": dict(dtype="fp16", L=1, B=64, T=1024, H=256, bwd=False, batch_first=False, h0=0.0, term=False),
    "c3": dict(dtype="fp16", L=1, B=256, T=512, H=1024, bwd=True, batch_first=False, h0=0.01, term=False),
    "c4": dict(dtype="bf16", L=1, B=32, T=1024, H=2048, bwd=True, batch_first=False, h0=0.0, term=False),
    "c5": dict(dtype="bf16", L=2, B=4096, T=256, H=512, bwd=True, batch_first=False, h0=0.0, term=False),
}
ESIZE = {"fp32": 4, "fp16": 2, "bf16": 2}
CPU_SAMPLE_BATCH = {"c1": 16, "c2": 64, "c3": 128, "c4": 32, "c5": 1024}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) every 100 ms."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.mhz, self.reasons, self.max_mhz = index, False, [], set(), None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            }
            while not self.stop_flag:
                self.mhz.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(0.1)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def result(self):
        return {"sm_mhz": statistics.median(self.mhz) if self.mhz else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def workload_config(wl, cfg, world, seq_override=False, batch_override=False):
    """The keys that describe the workload; identical for every arm (ours, reference, cuDNN)."""
    es = ESIZE[cfg["dtype"]]
    B = cfg["B"]
    name = wl
    if seq_override:
        name += f" with T overridden to {cfg['T']} (profiling run, not the benchmark)"
    if batch_override:
        name += f" with B overridden to {cfg['B']} (not the benchmark)"
    return {"workload": name,
            "L": cfg["L"], "B": B, "B_per_gpu": B // world, "T": cfg["T"], "I": cfg["H"], "H": cfg["H"],
            "pass": "fwd+bwd" if cfg["bwd"] else "fwd", "sharding": f"batch/{world}",
            "l2": "inputs larger than L2 (no flush needed)" if (B // world) * cfg["T"] * cfg["H"] * es > 126e6
                  else "inputs smaller than L2: L2 flushed (256 MB rewritten) before every timed step"}


def cpu_baseline(wl, cfg, steps=1, warmup=1):
    """nn.LSTM fp32 on the host cores over a batch sample of the workload."""
    from oracle.torch_cpu import time_nn_lstm
    bs = min(CPU_SAMPLE_BATCH[wl], cfg["B"])
    times = []
    threads = os.cpu_count() or 1
    for i in range(warmup + steps):
        t, threads = time_nn_lstm(cfg["H"], cfg["H"], cfg["L"], cfg["T"], bs, cfg["bwd"], reps=0,
                                  seed=1000 + i, threads=threads)
        if i >= warmup:
            times.append(t)
    sec = sum(times) / len(times)
    return {"value": cfg["L"] * bs * cfg["T"] / sec, "unit": "tokens/s", "cores": threads,
            "kind": "port",
            "sample": f"torch.nn.LSTM fp32 CPU, batch sample {bs} of {cfg['B']}, full T={cfg['T']}, "
                      f"L={cfg['L']}, {'fwd+bwd' if cfg['bwd'] else 'fwd'}; {sec:.3f} s per pass"}, sec


def run_reference(args, wl, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    base, sec = cpu_baseline(wl, cfg, steps=max(1, args.steps), warmup=max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": "fwd+bwd tokens/s per LSTM layer" if cfg["bwd"] else "fwd tokens/s per LSTM layer",
        "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(wl, cfg, max(1, args.gpus), args.seq_len > 0, args.batch > 0),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def time_cudnn(cfg, dev, x_dev, dout, state, steps, warmup, autocast=False):
    """ms per step of torch.nn.LSTM (cuDNN) on the same inputs.  Method of the reference's own
    comparison (scripts/benchmark.py:43-68,118-133): same dtype, fwd or fwd+bwd, CUDA events after
    warm-up; the weights are flattened once so no call compacts them.  autocast=True: fp32
    parameters under torch.autocast (the variant the reference's README singles out for bf16)."""
    import torch
    dt = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[cfg["dtype"]]
    torch.manual_seed(77)
    m = torch.nn.LSTM(cfg["H"], cfg["H"], num_layers=cfg["L"], batch_first=cfg["batch_first"]).to(dev)
    if not autocast:
        m = m.to(dt)
    m.flatten_parameters()
    x = x_dev.detach().to(torch.float32 if autocast else dt).requires_grad_(cfg["bwd"])
    st = None if state is None else tuple(t.to(x.dtype) for t in state)

    def step():
        if cfg["bwd"]:
            for p in m.parameters():
                p.grad = None
            x.grad = None
            with torch.autocast("cuda", dtype=dt, enabled=autocast):
                out, _ = m(x, st)
            out.backward(dout.to(out.dtype))
        else:
            with torch.no_grad(), torch.autocast("cuda", dtype=dt, enabled=autocast):
                m(x, st)

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "cudnn"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cudnn", action="store_true", help="skip the same-GPU torch.nn.LSTM (cuDNN) timing")
    ap.add_argument("--e2e-copy-out", action="store_true",
                    help="end-to-end arm: also copy the whole output sequence back to pinned host memory every step "
                         "(default: only the final hidden state; the sequence and the gradients stay on the device)")
    ap.add_argument("--seq-len", type=int, default=0,
                    help="override T (profiling aid: shorter captures; the line then names the override)")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the global batch (e.g. 512 = one rank's share of c5 at 8 GPUs; the line names the override)")
    args = ap.parse_args()
    wl, cfg = args.workload, dict(WORKLOADS[args.workload])
    if args.seq_len > 0:
        cfg["T"] = args.seq_len
    if args.batch > 0:
        cfg["B"] = args.batch
    if args.impl == "reference":
        return run_reference(args, wl, cfg)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    import fastlstm_b200 as F
    from fastlstm_b200 import _lib
    from fastlstm_b200.sharded import GradBucket, shard_bounds

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    _lib.check(lib.blstm_device_check(local), "device check")

    dt = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[cfg["dtype"]]
    L, T, H, Bg = cfg["L"], cfg["T"], cfg["H"], cfg["B"]
    lo, hi = shard_bounds(Bg, rank, world)
    B = hi - lo
    gen = torch.Generator().manual_seed(1000 + int(wl[1]))
    torch.manual_seed(1000 + int(wl[1]))           # identical weights on every rank
    model = F.FastLSTM(H, H, num_layers=L, batch_first=cfg["batch_first"], device=dev, dtype=dt)
    # seeded synthetic inputs; each rank generates only its own rows (seed offset by rank)
    gen.manual_seed(2000 + 16 * int(wl[1]) + rank)
    shape = (B, T, H) if cfg["batch_first"] else (T, B, H)
    x_host = torch.randn(shape, generator=gen).to(dt).pin_memory()
    dout = torch.randn(shape, generator=gen).to(dt).to(dev)
    state = None
    if cfg["h0"] > 0:
        state = tuple((torch.randn(L, B, H, generator=gen) * cfg["h0"]).to(dt).to(dev) for _ in range(2))
    x_dev = x_host.to(dev).requires_grad_(cfg["bwd"])
    hn_host = torch.empty((L, B, H), dtype=dt, pin_memory=True)
    out_host = torch.empty(shape, dtype=dt, pin_memory=True) if args.e2e_copy_out else None
    # data-parallel runs: every layer's backward writes its fp32 weight gradients straight into its
    # segment of the bucket and starts that segment's allreduce; allreduce() waits and fills p.grad
    bucket = GradBucket(model) if (cfg["bwd"] and world > 1) else None
    if bucket is not None:
        bucket.attach()

    if args.impl == "cudnn":
        if world > 1:
            if rank == 0:
                print(json.dumps({"impl": "cudnn", "unavailable": "the cuDNN arm is a 1-GPU comparison"}), flush=True)
            dist.barrier()
            dist.destroy_process_group()
            return
        sampler = ClockSampler(local)
        sampler.start()
        ms = time_cudnn(cfg, dev, x_dev, dout, state, args.steps, args.warmup)
        ms_ac = time_cudnn(cfg, dev, x_dev, dout, state, args.steps, args.warmup, autocast=True) if cfg["dtype"] != "fp32" else None
        sampler.stop_flag = True
        sampler.join(2)
        print(json.dumps({
            "impl": "cudnn", "metric": "fwd+bwd tokens/s per LSTM layer" if cfg["bwd"] else "fwd tokens/s per LSTM layer",
            "value": L * Bg * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "ms_per_step_autocast": ms_ac, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
            "config": workload_config(wl, cfg, 1, args.seq_len > 0, args.batch > 0),
            "what": "torch.nn.LSTM (cuDNN), weights flattened",
            "clocks": sampler.result()}), flush=True)
        return

    def step(x, after_forward=None):
        if cfg["bwd"]:
            for p in model.parameters():
                p.grad = None
            if x.grad is not None:
                x.grad = None
            out, (hn, cn) = model(x, state)
            if after_forward is not None:
                after_forward(out, hn)
            out.backward(dout)
            if bucket is not None:
                bucket.allreduce()
        else:
            with torch.no_grad():
                out, (hn, cn) = model(x, state)
            if after_forward is not None:
                after_forward(out, hn)
        return out, hn

    # End-to-end input pipeline: every step's input is uploaded from pinned host memory into one of
    # two device buffers on a copy stream; the upload of step i+1 is issued before step i computes,
    # so it overlaps the kernels (one upload per step, all inside the timed region in steady state).
    copy_stream = torch.cuda.Stream(device=dev)
    down_stream = torch.cuda.Stream(device=dev)           # results travel back beside the next step
    x_bufs = [torch.empty(shape, dtype=dt, device=dev) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]     # buffer k holds a fresh input
    consumed = [torch.cuda.Event() for _ in range(2)]     # the step that read buffer k has finished
    pipe = {"i": 0}

    def upload(k):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[k])
            x_bufs[k].copy_(x_host, non_blocking=True)
            uploaded[k].record(copy_stream)

    def e2e_step():
        k = pipe["i"] & 1
        if pipe["i"] == 0:
            upload(k)
        upload(k ^ 1)                                    # next step's input
        torch.cuda.current_stream().wait_event(uploaded[k])
        x = x_bufs[k].detach().requires_grad_(cfg["bwd"])

        def results_home(out, hn):
            # The step's result goes back to pinned host memory as soon as the forward pass has produced
            # it: the final hidden state, on the compute stream.  The output sequence [T,B,H] and the
            # gradients stay on the device (their consumers - the next layer, the loss, the optimizer -
            # live there); --e2e-copy-out also sends the sequence home on a second copy stream, beside
            # the backward pass.
            if out_host is not None:
                down_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(down_stream):
                    out_host.copy_(out.detach(), non_blocking=True)
                    out.record_stream(down_stream)
            hn_host.copy_(hn.detach(), non_blocking=True)

        step(x, results_home)
        consumed[k].record()
        pipe["i"] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Workloads whose tensors fit the 126 MB L2 get the L2 flushed (a 256 MB buffer rewritten) before
    # every timed step; each step then has its own event pair and the flush lies outside of it.
    small = "smaller" in workload_config(wl, cfg, world)["l2"]
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

    def timed(fn, n):
        barrier()
        if flush_buf is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            barrier()
            total = e0.elapsed_time(e1)
        else:
            pairs = []
            for _ in range(n):
                flush_buf.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                pairs.append((e0, e1))
            barrier()
            total = sum(a.elapsed_time(b) for a, b in pairs)
        ms = torch.tensor([total], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step(x_dev)
    F.check_status()
    sampler = ClockSampler(local)
    sampler.start()
    n0 = lib.blstm_launch_count()
    ms_total = timed(lambda: step(x_dev), args.steps)
    launches = int(lib.blstm_launch_count() - n0)
    for _ in range(max(args.warmup, 3)):             # allocator growth for the second input buffer's graph
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    sampler.stop_flag = True
    sampler.join(2)
    F.check_status()
    cudnn = None
    if world == 1 and not args.no_cudnn:
        n_c = max(2, min(args.steps, 5))
        c_ms = time_cudnn(cfg, dev, x_dev, dout, state, n_c, 3)
        cudnn = {"ms_per_step": c_ms, "speedup": c_ms / (ms_total / args.steps),
                 "what": "torch.nn.LSTM (cuDNN) same GPU, dtype, inputs and step; weights flattened; %d steps" % n_c}
        if cfg["dtype"] != "fp32":
            cudnn["ms_per_step_autocast"] = time_cudnn(cfg, dev, x_dev, dout, state, n_c, 3, autocast=True)

    tokens = L * Bg * T                      # layer-tokens per step, whole job
    ms_step = ms_total / args.steps
    value = tokens / (ms_step * 1e-3)
    e2e_value = tokens / (ms_e2e / args.steps * 1e-3)

    # ---- roofline: both persistent recurrence kernels timed by themselves (rank-local, CUDA events on the
    # launching stream); the slower one is the dominant kernel of the step and goes in "roofline"
    hbm_gbs, tflops, which = peaks()
    es = ESIZE[cfg["dtype"]]
    # small shards of a stack run as a layer wavefront (two layers side by side, each recurrence planned
    # for half of the SMs): the kernels are then timed, and their plans reported, as the step runs them
    wave = model._wavefront_chunks(x_dev, None, None) if hasattr(model, "_wavefront_chunks") else 0
    kflags = (0 if cfg["bwd"] else _lib.FLAG_INFERENCE) | (_lib.FLAG_HALF_DEVICE if wave else 0)
    d = _lib.Desc(_lib.DTYPE_CODE[cfg["dtype"]], T, B, H, H, kflags, 0, 0)
    st = torch.cuda.current_stream().cuda_stream
    Wh = model.weight_hh_l0.detach()
    pre = (torch.randn(T, B, 4 * H, device=dev) * 0.5).to(dt)
    ifgo = torch.empty_like(pre)
    states = torch.zeros(2, T + 1, B, H, device=dev, dtype=dt)
    nws = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
    ws = torch.empty(nws, dtype=torch.uint8, device=dev)

    # Each timed launch runs directly behind a full step of the benchmark (no host synchronisation in
    # between), so it sees the clocks of the timed region: under the power cap of a long step the SMs
    # run ~10 % slower than for a kernel launched on an idle GPU, and these kernels are latency bound.
    # The launch gets the arguments the step gives it (the bias gradient included).
    def time_launch(fn, prep=None, n=5, w=2):
        pairs = []
        for i in range(w + n):
            step(x_dev)
            if prep:
                prep()
            if flush_buf is not None:
                flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            if i >= w:
                pairs.append((e0, e1))
        torch.cuda.synchronize()
        F.check_status()
        return sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)

    fwd_ms = time_launch(
        lambda: _lib.check(lib.blstm_fwd_recurrence(d, ifgo.data_ptr(), Wh.data_ptr(), states[0].data_ptr(),
                                                    states[1].data_ptr(), ws.data_ptr(), nws, st), "fwd_recurrence"),
        prep=lambda: ifgo.copy_(pre))
    kernels = {"forward recurrence": fwd_ms}
    if cfg["bwd"]:
        nwb = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
        wsb = torch.empty(nwb, dtype=torch.uint8, device=dev)
        dg = torch.empty_like(pre)
        carries = torch.empty(2, B, H, device=dev, dtype=dt)
        db = torch.empty(4 * H, device=dev, dtype=torch.float32)
        kernels["backward recurrence"] = time_launch(
            lambda: _lib.check(lib.blstm_bwd_recurrence(d, dout.data_ptr() if not cfg["batch_first"] else pre.data_ptr(),
                                                        None, None, ifgo.data_ptr(), states[1].data_ptr(), Wh.data_ptr(),
                                                        dg.data_ptr(), carries[0].data_ptr(), carries[1].data_ptr(),
                                                        db.data_ptr(), wsb.data_ptr(), nwb, st), "bwd_recurrence"))
        del dg, wsb
    per_step = 10.0 if cfg["bwd"] else 5.0                    # forward-only runs save nothing for backward
    alg_bytes = per_step * B * H * es * T + 4.0 * H * H * es   # per_step*B*H*e per step + Wh once
    alg_flops = 8.0 * B * H * H * T
    hbm_time = alg_bytes / (hbm_gbs * 1e9)
    tensor_time = alg_flops / (tflops * 1e12)

    def plan_text(phase):
        import ctypes
        buf = ctypes.create_string_buffer(512)
        lib.blstm_plan_detail(d, phase, buf, 512)
        return buf.value.decode()

    def roof_of(name, ms):
        if hbm_time >= tensor_time:
            r = {"bound": "hbm", "achieved": alg_bytes / (ms * 1e-3) / 1e9, "peak": hbm_gbs, "unit": "GB/s"}
        else:
            r = {"bound": "tensor", "achieved": alg_flops / (ms * 1e-3) / 1e12, "peak": tflops, "unit": "TFLOP/s"}
        r["frac"] = r["achieved"] / r["peak"]
        phase = 1 if name.startswith("backward") else 0
        r.update({"kernel": "%s (%s)" % (name, lib.blstm_plan_name(d, phase).decode()),
                  "peak_source": f"of {which}", "ms_per_launch": ms, "us_per_timestep": ms * 1e3 / T,
                  "algorithmic_bytes_per_launch": alg_bytes, "algorithmic_flops_per_launch": alg_flops,
                  "traffic": None})
        try:
            with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
                tr = json.load(f).get(f"{wl}:{name}")
            if tr:   # DRAM bytes of one ncu capture at T = tr["T"], scaled by the timesteps of this launch
                r["traffic"] = tr["dram_bytes"] * (T / tr["T"]) * (B / tr["B"])
        except Exception:
            pass
        return r

    dominant = max(kernels, key=kernels.get)
    roof = roof_of(dominant, kernels[dominant])
    roof_other = {k: roof_of(k, v) for k, v in kernels.items() if k != dominant}
    del pre, ifgo, states, ws

    line = {
        "metric": "fwd+bwd tokens/s per LSTM layer" if cfg["bwd"] else "fwd tokens/s per LSTM layer",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": cfg["dtype"], "data": "synthetic",
        "config": workload_config(wl, cfg, world, args.seq_len > 0, args.batch > 0),
        "collective": "fp32 sum-allreduce of dWx,dWh,db, one per layer, started from that layer's backward (NCCL)" if bucket is not None else "none",
        "plans": {"fwd": plan_text(0), "bwd": plan_text(1)},
        "layer_wavefront": ("%d time chunks, two layers side by side on two streams, each recurrence on half of the SMs" % wave)
                           if wave else "off (layers run one after the other)",
        "us_per_timestep": ms_step * 1e3 / (T * L),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": x_host.numel() * es * world,
                "d2h_bytes_per_step": (hn_host.numel() + (out_host.numel() if out_host is not None else 0)) * es * world,
                "input_pipeline": "double-buffered upload on a copy stream, one upload per step; h_n"
                                  + (" and the output sequence are" if out_host is not None else " is")
                                  + " copied back to pinned memory every step"
                                  + ("" if out_host is not None else "; the output sequence [T,B,H] and the gradients stay on the device")},
        "gpu_launches": launches,
        "clocks": sampler.result(),
        "roofline": roof,
        "roofline_other_kernels": roof_other,
    }
    if cudnn is not None:
        line["cudnn"] = cudnn
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(wl, cfg)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
