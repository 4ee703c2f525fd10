"""Benchmark of the Mamba2-mixer prefill path (tokens/s) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      # the reference's CPU operators on the host cores

A step is one forward pass of one mixer layer over one synthetic batch. Workload `cfg2` (default) is the
Zamba2-1.2B-shaped layer (batch 4 x 2048 tokens, f16, fp32 scan state) per GPU; with N GPUs each rank runs its own
batch shard (weak scaling, no data-path collective). `cfg4` is the Zamba2-7B-shaped layer with 4 sequences per GPU.
One JSON line is printed by rank 0.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from anygpu_b200 import synth  # noqa: E402

METRIC = "mamba2_mixer_prefill_tokens_per_s"
UNIT = "tokens/s"
STAGES = ["in_proj", "conv1d", "ssd", "gated_rmsnorm", "out_proj"]


def workload(name):
    cfg = dict(synth.CONFIGS[name])
    if name == "cfg4":
        cfg["batch"] = 4  # per GPU: 32 sequences over 8 GPUs
        cfg["norm_group_size"] = cfg["d_inner"]  # the reference normalises the whole row
    return cfg


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class NvmlSampler:
    """Reads SM clock, power and clock-event reasons of one GPU through NVML (read-only queries, the data `nvidia-smi` prints)
    from a thread every millisecond while the timed region runs: the region of the default run lasts ~10 ms, too short for the
    100 ms period of `nvidia-smi -lms`."""

    def __init__(self, cuda_index):
        self.rows, self.stop_flag, self.thread, self.handle, self.nv = [], False, None, None, None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = getattr(torch.cuda.get_device_properties(cuda_index), "uuid", None)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode()) if uuid is not None else None
            except Exception:
                self.handle = None
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self.nv = pynvml
        except Exception:
            self.handle = None

    def available(self):
        return self.handle is not None

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv, h = self.nv, self.handle
        reasons_of = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag:
            try:
                self.rows.append((time.time(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), reasons_of(h),
                                  nv.nvmlDeviceGetPowerUsage(h) / 1000.0))
            except Exception:
                break
            time.sleep(0.001)

    def stop(self, t0, t1):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=1.0)
        rows = [r for r in self.rows if t0 <= r[0] <= t1] or self.rows
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        seen = sorted(n for n, bit in names.items() if any(r[2] & bit for r in rows))
        try:
            sm_max = float(nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM))
        except Exception:
            sm_max = None
        return {"sm_mhz": statistics.median(float(r[1]) for r in rows), "sm_max_mhz": sm_max, "reasons": seen, "samples": len(rows),
                "power_w_max": max(r[3] for r in rows), "source": "nvml, 1 ms period, samples inside the timed region"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.rows, self.proc, self.thread = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.1 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        reasons = set()
        for r in rows:
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons), "samples": len(rows),
                "power_w_max": max(float(r[3]) for r in rows)}


# ---------------------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU operators on the host cores
# ---------------------------------------------------------------------------------------------------------------

def _ref_mixer_tokens(u, w, cfg):
    """One mixer forward over u [1, l, d_model] with the reference's own CPU operators where it has them (linear,
    causal conv1d, gated RMSNorm: compiled from its sources) and the oracle's restatement of its Python SSD script."""
    from oracle import oracle as orc
    use_ref = orc.ref_lib() is not None
    lin = orc.ref_linear if use_ref else (lambda a, b: orc.linear(a, b, fast=False))
    conv = orc.ref_causal_conv1d if use_ref else orc.causal_conv1d
    norm = (lambda x, z, nw, eps: orc.ref_gated_rmsnorm(x, z, nw, eps)) if use_ref else orc.gated_rmsnorm
    b, l, _ = u.shape
    d_inner, H, P, G, N = cfg["d_inner"], cfg["nheads"], cfg["headdim"], cfg["ngroups"], cfg["d_state"]
    conv_dim, d_in_proj = synth.dims(cfg)
    zx = lin(u.reshape(b * l, -1), w["in_proj_weight"]).reshape(b, l, d_in_proj)
    xbc = conv(np.ascontiguousarray(zx[..., d_inner:d_inner + conv_dim].transpose(0, 2, 1)), w["conv1d_weight"], w["conv1d_bias"])
    xbc = np.ascontiguousarray(xbc.transpose(0, 2, 1))
    y, _ = orc.ssd_chunk_scan(xbc[..., :d_inner].reshape(b, l, H, P), np.ascontiguousarray(zx[..., d_inner + conv_dim:]),
                              -np.exp(w["A_log"]), xbc[..., d_inner:d_inner + G * N].reshape(b, l, G, N),
                              xbc[..., d_inner + G * N:].reshape(b, l, G, N), cfg["chunk"], D=w["D"], dt_bias=w["dt_bias"])
    g = norm(y.reshape(b * l, d_inner), np.ascontiguousarray(zx[..., :d_inner]).reshape(b * l, d_inner), w["norm_weight"], cfg["eps"])
    return lin(g, w["out_proj_weight"]).reshape(b, l, -1), ("reference" if use_ref else "port")


_W = {}


def _worker_step(args):
    name, tokens, seed = args
    cfg = workload(name)
    if name not in _W:
        _W[name] = synth.make_weights(cfg, 0)
    u = synth.make_input(cfg, seed, batch=1, seqlen=tokens)
    t0 = time.perf_counter()
    _, kind = _ref_mixer_tokens(u, _W[name], cfg)
    return time.perf_counter() - t0, kind


def cpu_reference_throughput(name, tokens_per_worker, workers, steps, warmup):
    """tokens/s of the reference CPU path: `workers` processes (the reference is single-threaded) each push
    `tokens_per_worker` tokens of one sequence through the mixer per step."""
    import multiprocessing as mp
    ctx = mp.get_context("fork")
    kind = "port"
    with ctx.Pool(workers) as pool:
        for i in range(warmup):
            pool.map(_worker_step, [(name, tokens_per_worker, 100 + i * workers + k) for k in range(workers)])
        t0 = time.perf_counter()
        for i in range(steps):
            res = pool.map(_worker_step, [(name, tokens_per_worker, 1000 + i * workers + k) for k in range(workers)])
            kind = res[0][1]
        dt = time.perf_counter() - t0
    return workers * tokens_per_worker * steps / dt, dt / steps, kind


def reference_cuda_kernels():
    """The reference's own CUDA kernels recompiled for sm_100a (oracle/_ref/ref_cuda_bench, built by `make -C oracle ref_cuda`
    where the reference checkout is present), timed on this GPU at the cfg2 projection shapes and the conv configuration: a second
    baseline beside the CPU one. Runs as a child process (the reference's launchers exit on any CUDA error). None when not built."""
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "ref_cuda_bench")
    if not os.path.exists(exe):
        return None
    out = {}
    for what in ("mm", "conv"):
        try:
            r = subprocess.run([exe, what, "3"], capture_output=True, text=True, timeout=180)
            out[what] = json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 and r.stdout.strip() else {"failed": r.returncode}
        except Exception as ex:  # noqa: BLE001 - a baseline that cannot run is reported, not fatal
            out[what] = {"failed": str(ex)[:100]}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = workload(args.workload)
    workers = os.cpu_count() or 1
    tokens = 16
    value, sec_per_step, kind = cpu_reference_throughput(args.workload, tokens, workers, args.steps, args.warmup)
    sample = (f"{workers} single-threaded processes x {tokens} tokens of one sequence per step (reference CPU linear / conv1d / "
              f"gated RMSNorm compiled from its sources + CPU restatement of its Python SSD script)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": _config_dict(args.workload, cfg, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": workers, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def _config_dict(name, cfg, n):
    return {"workload": f"{name}: Mamba2 mixer prefill, batch {cfg['batch']} x seqlen {cfg['seqlen']} per GPU, d_model {cfg['d_model']}, "
                        f"d_inner {cfg['d_inner']}, {cfg['nheads']} heads x {cfg['headdim']}, d_state {cfg['d_state']}, ngroups {cfg['ngroups']}, "
                        f"chunk {cfg['chunk']}, f16 weights/activations, fp32 scan state",
            "global_batch": cfg["batch"] * n, "seq_len": cfg["seqlen"], "parallelism": f"batch-sharded x{n} (replicated weights, no collective)",
            "l2": "inputs rotate over 4 buffers; per-step working set (~0.45 GB at cfg2) exceeds the 126 MB L2"}



# ---------------------------------------------------------------------------------------------------------------
# records that ride in the default line beside the prefill numbers
# ---------------------------------------------------------------------------------------------------------------

def _sampler(local_rank):
    s = NvmlSampler(local_rank)
    return s if s.available() else ClockSampler(local_rank)


def _timed(fn, n, torch):
    """n calls of fn(i) between two CUDA events on the current stream; returns milliseconds."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def decode_record(torch, ops, local_rank, peaks, steps=128, reps=5):
    """The decode configuration (Zamba2-2.7B-shaped layer, batch 64, `steps` consecutive single-token steps from given states):
    microseconds per step with the step's kernels launched one call per token, with a one-step CUDA graph replayed per token,
    with 16 steps per graph and with the whole run in one graph. Every figure is the best of `reps` runs of all `steps` steps
    (CUDA events around the run); the states keep advancing from run to run."""
    c3 = workload("cfg3")
    wts = ops.ZambaMamba2weights.from_numpy(synth.make_weights(c3, 0), torch.float16)
    mixer = ops.Mamba2Mixer(c3, wts)
    cs, ss = synth.make_decode_state(c3, 0)
    cache = ops.ZambaMambaCache(torch.from_numpy(cs).cuda().half(), torch.from_numpy(ss).cuda())
    g = torch.Generator(device="cuda").manual_seed(3)
    us = torch.randn(steps, c3["batch"], c3["d_model"], device="cuda", generator=g).half()
    outs = torch.empty_like(us)
    cd3, dip3 = synth.dims(c3)
    bytes_alg = (c3["d_model"] * dip3 + c3["d_inner"] * c3["d_model"]) * 2 + 2 * ss.size * 4 + 2 * cs.size * 2
    u1, o1 = us[0].clone(), torch.empty_like(us[0])  # the one-step graph replays this input every time
    g1 = mixer.capture_decode(u1, cache, o1)
    gsteps = 16 if steps % 16 == 0 else 1
    g16 = mixer.capture_decode_steps(us[:gsteps], cache, outs[:gsteps])
    gall = mixer.capture_decode_steps(us, cache, outs)
    lib = __import__("anygpu_b200.capi", fromlist=["capi"]).load()
    modes = {
        "plain_launches": lambda: _timed(lambda t: mixer.decode(us[t], cache, out=outs[t]), steps, torch),
        "graph_1_step_replayed_per_token": lambda: _timed(lambda t: g1.replay(), steps, torch),
        f"graph_{gsteps}_steps": lambda: _timed(lambda t: g16.replay(), steps // gsteps, torch),
        f"graph_{steps}_steps": lambda: _timed(lambda t: gall.replay(), 1, torch),
    }
    for fn in modes.values():  # warm-up of every mode
        fn()
    sampler = _sampler(local_rank)
    sampler.start()
    time.sleep(0.05)
    t0 = time.time()
    res = {}
    for name, fn in modes.items():
        us_per_step = min(fn() for _ in range(reps)) * 1e3 / steps
        res[name] = {"us_per_step": us_per_step, "gbs": bytes_alg / (us_per_step * 1e-6) / 1e9,
                     "frac_of_hbm": bytes_alg / (us_per_step * 1e-6) / 1e9 / peaks["hbm_gbs"]}
        err = lib.b200_last_device_error(None, None)
        if err != 0 or not bool(torch.isfinite(outs).all()) or not bool(torch.isfinite(cache.ssm_state).all()):
            raise SystemExit(f"decode record, mode {name}: device error {err}, outputs finite {bool(torch.isfinite(outs).all())}, "
                             f"state finite {bool(torch.isfinite(cache.ssm_state).all())}")
    lib.b200_launch_count(1)
    mixer.decode(us[0], cache, out=outs[0])
    launches_per_step = int(lib.b200_launch_count(1))
    torch.cuda.synchronize()
    clocks = sampler.stop(t0, time.time())
    if not bool(torch.isfinite(outs).all()):
        raise SystemExit("decode outputs are not finite")
    return {"workload": f"cfg3: Zamba2-2.7B-shaped decode step, batch {c3['batch']}, d_model {c3['d_model']}, d_inner {c3['d_inner']}, "
                        f"{c3['nheads']} heads x {c3['headdim']}, d_state {c3['d_state']}, {steps} consecutive steps, f16 weights, fp32 state",
            "steps": steps, "reps": reps, "statistic": "best of reps, each rep = all steps between two CUDA events",
            "algorithmic_bytes_per_step": bytes_alg, "hbm_peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
            "target_us_per_step_at_70pct": bytes_alg / (0.7 * peaks["hbm_gbs"] * 1e9) * 1e6,
            "kernel_launches_per_step": launches_per_step, "modes": res, "clocks": clocks}


def conv_cfg1_record(torch, ops, peaks, ref_cuda):
    """The standalone conv configuration: causal conv1d + SiLU over (8, 4224, 4096) f16, and its rolling-state decode update
    advanced 256 single-token steps (one CUDA graph of the 256 steps)."""
    B_, C_, L_, W_ = 8, 4224, 4096, 4
    g = torch.Generator(device="cuda").manual_seed(1)
    rn = lambda *shape, std=1.0: (torch.randn(*shape, device="cuda", generator=g) * std).half()
    xs = [rn(B_, C_, L_) for _ in range(3)]  # 277 MB each: every call reads a tensor that is not in L2
    w, bs = rn(C_, W_, std=0.5), rn(C_, std=0.1)
    fn = lambda i: ops.tensor_causal_conv1d(xs[i % 3], w, bs)
    for i in range(3):
        fn(i)
    ms = sorted(_timed(lambda i, k=k: fn(k), 1, torch) for k in range(15))
    med = ms[len(ms) // 2]
    bytes_alg = 2 * B_ * C_ * L_ * 2
    rec = {"prefill": {"shape": [B_, C_, L_], "width": W_, "dtype": "f16", "median_us": med * 1e3, "min_us": ms[0] * 1e3,
                       "algorithmic_bytes": bytes_alg, "gbs": bytes_alg / (med * 1e-3) / 1e9,
                       "frac_of_hbm": bytes_alg / (med * 1e-3) / 1e9 / peaks["hbm_gbs"], "hbm_peak_gbs": peaks["hbm_gbs"]}}
    if ref_cuda and isinstance(ref_cuda.get("conv"), dict):
        rec["prefill"]["reference_cuda_kernel_f32"] = ref_cuda["conv"]
    steps = 256
    state, xts = rn(B_, C_, W_ - 1), rn(steps, B_, C_)
    ops.tensor_causal_conv1d_update(xts[0], state, w, bs)
    torch.cuda.synchronize()
    gobj = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gobj):
        for t in range(steps):
            ops.tensor_causal_conv1d_update(xts[t], state, w, bs)
    gobj.replay()
    ms = sorted(_timed(lambda i: gobj.replay(), 1, torch) for _ in range(9))
    plain = min(_timed(lambda t: ops.tensor_causal_conv1d_update(xts[t], state, w, bs), steps, torch) for _ in range(3))
    step_bytes = B_ * C_ * 2 * (2 * (W_ - 1) + 2) + C_ * (W_ + 1) * 2
    rec["decode"] = {"steps": steps, "us_per_step_in_one_graph": ms[len(ms) // 2] * 1e3 / steps,
                     "us_per_step_plain_launches": plain * 1e3 / steps, "bytes_per_step": step_bytes,
                     "note": "0.6 MB per step: bound by launch latency, no roofline claim"}
    return rec


def sustained_record(torch, lib, mixer, us, out, tokens, flops_total, flops_in, local_rank, peaks, ms_hint, seconds=2.2):
    """The same prefill step looped for `seconds` (power-capped clocks), then 200 more steps with the per-stage events on:
    ms per step, the clock record of the loop, and fractions of the SUSTAINED measured tensor peak."""
    n = max(int(seconds / (ms_hint * 1e-3)), 50)
    sampler = _sampler(local_rank)
    sampler.start()
    time.sleep(0.05)
    t0 = time.time()
    ms = _timed(lambda i: mixer.prefill(us[i % len(us)], out=out), n, torch)
    t1 = time.time()
    lib.b200_stage_timing_enable(1)
    ms_tail = _timed(lambda i: mixer.prefill(us[i % len(us)], out=out), 200, torch)
    stage_ms = (ctypes.c_float * 5)()
    calls = ctypes.c_int(0)
    lib.b200_stage_timing_collect(stage_ms, ctypes.byref(calls))
    lib.b200_stage_timing_enable(0)
    clocks = sampler.stop(t0, t1)
    per = ms / n
    st = {k: stage_ms[j] / max(calls.value, 1) for j, k in enumerate(STAGES)}
    return {"steps": n, "seconds": ms * 1e-3, "ms_per_step": per, "tokens_per_s": tokens / (per * 1e-3), "clocks": clocks,
            "achieved_tflops": flops_total / (per * 1e-3) / 1e12, "peak_tflops_sustained": peaks["tflops_sustained"],
            "frac_of_sustained_peak": flops_total / (per * 1e-3) / 1e12 / peaks["tflops_sustained"],
            "stage_ms_after_the_loop": st, "ms_per_step_after_the_loop": ms_tail / 200,
            "in_proj_frac_of_sustained_peak": (flops_in / (st["in_proj"] * 1e-3) / 1e12 / peaks["tflops_sustained"]) if st["in_proj"] > 0 else None}


def cfg4_dp_record(torch, dist, ops, bdist, rank, world, steps, total_sequences=32):
    """Zamba2-7B-shaped layer, 32 sequences of 4096 tokens in all, split evenly over the ranks (strong scaling, replicated
    weights, no data-path collective): device time per step as the max over ranks."""
    cfg = dict(synth.CONFIGS["cfg4"], norm_group_size=synth.CONFIGS["cfg4"]["d_inner"])
    if total_sequences % world != 0:
        return {"skipped": f"{total_sequences} sequences do not split over {world} ranks"}
    bl = total_sequences // world
    cfg["batch"] = bl
    l = cfg["seqlen"]
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(synth.make_weights(cfg, 0), torch.float16))
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    # at most 8 sequences per call: bounds the workspace (the calls of a step follow each other on the stream)
    per_call = min(bl, 8)
    u = torch.randn(bl, l, cfg["d_model"], device="cuda", generator=g).half()
    out = torch.empty_like(u)

    def step(i):
        for c0 in range(0, bl, per_call):
            mixer.prefill(u[c0:c0 + per_call], out=out[c0:c0 + per_call])

    for i in range(2):
        step(i)
    if world > 1:
        dist.barrier()
    ms = bdist.max_over_ranks(_timed(step, steps, torch), device="cuda") / steps
    ok = bool(torch.isfinite(out[0, :64]).all())
    del mixer, u, out
    return {"workload": f"cfg4: Zamba2-7B-shaped mixer prefill, {total_sequences} sequences x {l} tokens in all, {bl} per rank "
                        f"({per_call} per call)", "scaling": "strong", "ms_per_step": ms, "tokens_per_s": total_sequences * l / (ms * 1e-3),
            "steps": steps, "finite": ok}


def tp_chunk_schedule(batch, world, chunk):
    """Sequences per compute / all-reduce pipeline step of a head-sharded run. chunk > 0: that many in every step. chunk == 0: `world`
    sequences per step, at least 2: the message an all-reduce needs to run at NVLink speed grows with the ranks. Measured at 8 ranks,
    1 / 2 / 4 / 8 / 16 sequences per step: 7.64 / 6.36 / 5.44 / 5.23 / 5.68 ms; a schedule that tapers at the end (8, 8, 8, 4, 2, 2,
    to shorten the last all-reduce, which nothing overlaps) measured 5.37 against 5.29 ms at 8 ranks and 14.4 against 14.1 ms at 2."""
    c = max(1, min(chunk if chunk > 0 else max(2, world), batch))
    return [min(c, batch - c0) for c0 in range(0, batch, c)]


def cfg4_tp_record(torch, dist, ops, bdist, rank, world, steps, chunk, total_sequences=32):
    """Zamba2-7B-shaped layer, head-sharded over the ranks (TP = number of ranks): every rank holds all 32 sequences and
    nheads/TP heads, and the out_proj addends are summed by NCCL all-reduces (f16) together with the per-token sums of squares.
    Reports, as the max over ranks of device times: the compute alone, the all-reduces alone (same buffers), the pipelined step
    (the all-reduce of chunk i on NCCL's stream while chunk i+1 computes), and on rank 0 the parity of the TP result against the
    unsharded mixer for the first sequence."""
    cfg = dict(synth.CONFIGS["cfg4"], batch=total_sequences)
    H = cfg["nheads"]
    if H % world != 0 or (H // world) % 2 != 0 and world > 1:
        return {"skipped": f"{H} heads do not split into even head counts over {world} ranks"}
    b, l = cfg["batch"], cfg["seqlen"]
    w_np = synth.make_weights(cfg, 0)
    loc = synth.tp_local_config(cfg, world)
    wl = ops.ZambaMamba2weights.from_numpy(synth.shard_weights_tp(w_np, cfg, world, rank), torch.float16)
    mixer = ops.Mamba2MixerTP(loc, wl, cfg["d_inner"])
    g = torch.Generator(device="cuda").manual_seed(0)  # the same input on every rank
    u = torch.randn(b, l, cfg["d_model"], device="cuda", generator=g).half()
    out = torch.empty_like(u)
    ss = torch.empty(b * l, device="cuda")
    sched = tp_chunk_schedule(b, world, chunk)
    starts = [sum(sched[:i]) for i in range(len(sched))]
    slices = [(slice(c0, c0 + n), slice(c0 * l, (c0 + n) * l)) for c0, n in zip(starts, sched)]

    def reduce_async(sl, rows):
        if world == 1:
            return []
        return [dist.all_reduce(out[sl], async_op=True), dist.all_reduce(ss[rows], async_op=True)]

    def step_pipelined(i):
        pending = None
        for sl, rows in slices:
            mixer.partial(u[sl], partial_out=out[sl], sumsq=ss[rows])
            works = reduce_async(sl, rows)
            if pending is not None:
                for wk in pending[2]:
                    wk.wait()
                mixer.finish(out[pending[0]], ss[pending[1]])
            pending = (sl, rows, works)
        for wk in pending[2]:
            wk.wait()
        mixer.finish(out[pending[0]], ss[pending[1]])

    def step_compute(i):
        for sl, rows in slices:
            mixer.partial(u[sl], partial_out=out[sl], sumsq=ss[rows])
            mixer.finish(out[sl], ss[rows])

    def step_reduce(i):
        works = []
        for sl, rows in slices:
            works += reduce_async(sl, rows)
        for wk in works:
            wk.wait()

    def timed(fn):
        for i in range(2):
            fn(i)
        if world > 1:
            dist.barrier()
        return bdist.max_over_ranks(_timed(fn, steps, torch), device="cuda") / steps

    t_pipe = timed(step_pipelined)
    result = out[:1].clone()
    t_comp = timed(step_compute)
    t_red = timed(step_reduce) if world > 1 else 0.0
    parity = None
    if rank == 0:
        from_tp = result.float().cpu().numpy()
        del mixer, wl
        torch.cuda.empty_cache()
        whole_cfg = dict(cfg, batch=1, norm_group_size=cfg["d_inner"])  # the TP path normalises the whole row, as the reference does
        whole = ops.Mamba2Mixer(whole_cfg, ops.ZambaMamba2weights.from_numpy(w_np, torch.float16))
        want = whole.prefill(u[:1].contiguous()).float().cpu().numpy()
        err = np.abs(from_tp - want)
        bad = (err > 2e-3) & (err > 2e-2 * np.abs(want))
        parity = {"against": "unsharded mixer on rank 0, first sequence", "fail_fraction": float(bad.mean()), "max_abs_err": float(err.max()),
                  "rel_l2": float(np.sqrt((err.astype(np.float64) ** 2).sum() / ((want.astype(np.float64) ** 2).sum() + 1e-8))),
                  "rule": "rel 2e-2 OR abs 2e-3 per element"}
        del whole
    nbytes = b * l * cfg["d_model"] * 2
    rec = {"workload": f"cfg4: Zamba2-7B-shaped mixer prefill, {b} sequences x {l} tokens on every rank, {H} heads sharded {world}-way, "
                       f"pipeline steps of {'/'.join(str(v) for v in sched)} sequences", "scaling": "strong", "tp": world, "steps": steps,
           "ms_per_step_pipelined": t_pipe, "tokens_per_s": b * l / (t_pipe * 1e-3), "ms_compute_only": t_comp,
           "ms_all_reduce_only": t_red, "exposed_ms": t_pipe - t_comp, "all_reduce_bytes_per_step_f16": nbytes,
           "all_reduce_algbw_gbs": (nbytes / (t_red * 1e-3) / 1e9) if t_red > 0 else None, "parity": parity}
    del u, out, ss
    return rec

# ---------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------

def run_gpu(args):
    import torch
    import torch.distributed as dist
    from anygpu_b200 import capi, ops
    from anygpu_b200 import dist as bdist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = capi.load()

    cfg = workload(args.workload)
    b, l = cfg["batch"], cfg["seqlen"]
    tokens = b * l
    w_np = synth.make_weights(cfg, 0)
    weights = ops.ZambaMamba2weights.from_numpy(w_np, torch.float16)
    mixer = ops.Mamba2Mixer(cfg, weights)
    nbuf = 4
    us = [torch.from_numpy(synth.make_input(cfg, 10 * rank + i)).to("cuda", torch.float16) for i in range(nbuf)]
    out = torch.empty_like(us[0])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        return bdist.max_over_ranks(v, device="cuda")

    # ---- device-resident timing (the headline `value`) -------------------------------------------------------
    for i in range(max(args.warmup, 1)):  # at least one call outside the capture below: workspace and kernel attributes set up
        mixer.prefill(us[i % nbuf], out=out)
    barrier()
    sampler = NvmlSampler(local_rank) if rank == 0 else None
    if rank == 0:
        if not sampler.available():
            sampler = ClockSampler(local_rank)  # nvidia-smi at its 100 ms period: few samples fall into a short region
        sampler.start()
        time.sleep(0.25)
    # The K timed steps are one CUDA graph: the same calls of the public prefill entry point, captured once and replayed, so that
    # the GPU runs the 5 x K kernels back to back (launched one by one from the host they leave ~2 us between kernels, 10 us per
    # step). Inside the timed region only the dominant kernel (in_proj, the first of the step) is bracketed by events, in every
    # fourth step: an event between two kernels costs ~2.5 us, six of them 3% of the step; the table of all five stages comes
    # from a pass of its own below. `--no-graph` times the same steps launched from the host.
    lib.b200_stage_timing_enable(2)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph = None
    lib.b200_launch_count(1)
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.steps):
                mixer.prefill(us[i % nbuf], out=out)
        gpu_launches = int(lib.b200_launch_count(1))  # kernel nodes of the graph: counted by the library at its launch sites during capture
        graph.replay()  # one untimed replay: the first launch of a graph also uploads it
        torch.cuda.synchronize()
    barrier()
    t_wall0 = time.time()
    ev0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(args.steps):
            mixer.prefill(us[i % nbuf], out=out)
    ev1.record()
    barrier()
    t_wall1 = time.time()
    if graph is None:
        gpu_launches = int(lib.b200_launch_count(1))  # kernels this library launched between the two events
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    stage_ms = (ctypes.c_float * 5)()
    calls = ctypes.c_int(0)
    capi.check("b200_stage_timing_collect", lib.b200_stage_timing_collect(stage_ms, ctypes.byref(calls)))
    in_proj_ms_live = stage_ms[0] / max(calls.value, 1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    # the same steps again with an event at every stage boundary (not part of `value`)
    lib.b200_stage_timing_enable(1)
    ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev2.record()
    for i in range(args.steps):
        mixer.prefill(us[i % nbuf], out=out)
    ev3.record()
    torch.cuda.synchronize()
    ms_per_step_with_stage_events = ev2.elapsed_time(ev3) / args.steps
    capi.check("b200_stage_timing_collect", lib.b200_stage_timing_collect(stage_ms, ctypes.byref(calls)))
    lib.b200_stage_timing_enable(0)
    dev_err = lib.b200_last_device_error(None, None)
    if dev_err != 0:
        raise SystemExit(f"device-side wait timed out during the benchmark (status {dev_err})")
    ms_per_step = ms_total / args.steps
    value = world * tokens * args.steps / (ms_total * 1e-3)

    # ---- end to end through the host-buffer entry point --------------------------------------------------------
    u_pin = [torch.from_numpy(synth.make_input(cfg, 10 * rank + i)).half().pin_memory() for i in range(2)]
    out_pin = torch.empty_like(u_pin[0]).pin_memory()
    for i in range(max(1, min(args.warmup, 3))):
        mixer.prefill_host(u_pin[i % 2], out_pin, overlap=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_enq0 = time.perf_counter()
    for i in range(args.steps):
        mixer.prefill_host(u_pin[i % 2], out_pin, overlap=True)
    e2e_enqueue_ms = (time.perf_counter() - t_enq0) * 1e3 / args.steps
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    # one call alone (nothing before it to overlap with): its latency, copy-in of the first sequence and copy-out of the last exposed
    mixer.prefill_host(u_pin[0], out_pin)  # untimed: the first call of the plain form creates its per-sequence events
    torch.cuda.synchronize()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    mixer.prefill_host(u_pin[0], out_pin)
    e3.record()
    torch.cuda.synchronize()
    e2e_single_ms = e2.elapsed_time(e3)
    io_bytes = u_pin[0].numel() * 2
    e2e_value = world * tokens * args.steps / (e2e_ms * 1e-3)
    checksum = float(out_pin.float().abs().mean())
    if not np.isfinite(checksum) or checksum == 0.0:
        raise SystemExit("mixer output is not finite / all zero")

    # ---- the same pinned buffers with no kernels: what the copies alone cost at this number of ranks ----------------
    copy_only = None
    if not args.no_extras:
        dev_in, dev_out = torch.empty_like(us[0]), torch.empty_like(us[0])
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        def copy_step(i):
            with torch.cuda.stream(s_in):
                dev_in.copy_(u_pin[i % 2], non_blocking=True)
            with torch.cuda.stream(s_out):
                out_pin.copy_(dev_out, non_blocking=True)
        for i in range(3):
            copy_step(i)
        barrier()
        t0c = time.perf_counter()
        for i in range(args.steps):
            copy_step(i)
        host_enqueue_ms = (time.perf_counter() - t0c) * 1e3 / args.steps
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(args.steps):
            copy_step(i)
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)
        c1.record()
        barrier()
        copy_ms = max_over_ranks(c0.elapsed_time(c1)) / args.steps
        copy_only = {"ms_per_step": copy_ms, "gbs_per_rank_each_direction": io_bytes / (copy_ms * 1e-3) / 1e9,
                     "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes, "host_enqueue_ms_per_step": host_enqueue_ms,
                     "note": "H2D and D2H of one step's pinned buffers on two streams, no kernels, max over ranks: the floor the "
                             "copies set for e2e at this number of ranks"}
        del dev_in, dev_out

    # ---- cfg4 (Zamba2-7B-shaped layer, 32 sequences): batch-sharded and head-sharded -------------------------------
    cfg4_dp = cfg4_tp = None
    if not args.no_extras and not args.no_cfg4:
        del us, out, u_pin, out_pin, mixer, weights
        torch.cuda.empty_cache()
        cfg4_dp = cfg4_dp_record(torch, dist, ops, bdist, rank, world, steps=max(2, min(args.steps, 4)))
        cfg4_tp = cfg4_tp_record(torch, dist, ops, bdist, rank, world, steps=max(2, min(args.steps, 3)), chunk=args.tp_chunk)
        torch.cuda.empty_cache()
        weights = ops.ZambaMamba2weights.from_numpy(w_np, torch.float16)
        mixer = ops.Mamba2Mixer(cfg, weights)
        us = [torch.from_numpy(synth.make_input(cfg, 10 * rank + i)).to("cuda", torch.float16) for i in range(nbuf)]
        out = torch.empty_like(us[0])

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (in_proj GEMM), live stage times from the timed region --------------------
    peaks = measured_peaks()
    conv_dim, d_in_proj = synth.dims(cfg)
    per_stage = [stage_ms[j] / max(calls.value, 1) for j in range(5)]
    flops_in = 2.0 * tokens * cfg["d_model"] * d_in_proj
    G, N, H, P, Q = cfg["ngroups"], cfg["d_state"], cfg["nheads"], cfg["headdim"], cfg["chunk"]
    nchunks = -(-l // Q)
    flops_out = 2.0 * tokens * cfg["d_inner"] * cfg["d_model"]
    flops_ssd = float(b * nchunks * (H * (2 * Q * Q * P + 4 * Q * N * P) + G * 2 * Q * Q * N))
    flops_total = flops_in + flops_out + flops_ssd
    dom = int(np.argmax(per_stage))
    # Which measured cuBLAS figure a fraction is taken against follows from the conditions of the timed region: a region far
    # shorter than a second at full SM clock with no power cap is a burst, so the burst figure applies; the seconds-long loop in
    # `sustained` is compared with the sustained figure.
    region_s = ms_total * 1e-3
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    burst = region_s < 1.0 and not capped
    peak = peaks["tflops_burst"] if burst else peaks["tflops_sustained"]
    kname = lib.b200_linear_kernel_name(capi.F16, tokens, cfg["d_model"], d_in_proj).decode()
    achieved = flops_in / (in_proj_ms_live * 1e-3) / 1e12 if in_proj_ms_live > 0 else None
    roofline = {"kernel": f"{kname} (in_proj: the stage with the largest share of the step)", "bound": "tensor", "achieved": achieved,
                "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if achieved else None,
                "peak_kind": ("burst" if burst else "sustained") + f" cuBLAS bf16, {peaks['source']}; timed region {region_s * 1e3:.1f} ms, "
                             f"median SM clock {clocks.get('sm_mhz') if clocks else None} MHz, power cap {'active' if capped else 'not active'}",
                # DRAM bytes per launch: measured by ncu on this very launch (M = 8192: 79.9 MB read + 107.4 MB written before the kernel
                # ends; the rest of the output still sits in L2); other shapes: operands read once and output written once, as the capture
                # of the M = 2048 case showed
                "traffic": (187.4e6 if (tokens, cfg["d_model"], d_in_proj) == (8192, 2048, 8384)
                            else float(tokens * cfg["d_model"] * 2 + cfg["d_model"] * d_in_proj * 2 + tokens * d_in_proj * 2)),
                "traffic_note": ("dram__bytes_read.sum + dram__bytes_write.sum of the full-size launch, one ncu pass (profiles/gemm_f16_tcgen05_in_proj_small.md, "
                                 "last section); algorithmic bytes X + W + Y = 205.3 MB"
                                 if (tokens, cfg["d_model"], d_in_proj) == (8192, 2048, 8384)
                                 else "scaled from the ncu capture of the M=2048 case (profiles/gemm_f16_tcgen05_in_proj_small.md): operands read once from DRAM, output written once"),
                "peak_burst": peaks["tflops_burst"], "peak_sustained": peaks["tflops_sustained"],
                "frac_of_burst_peak": achieved / peaks["tflops_burst"] if achieved else None,
                "frac_of_sustained_peak": achieved / peaks["tflops_sustained"] if achieved else None,
                "algorithmic_flops_per_launch": flops_in, "avg_launch_ms": in_proj_ms_live,
                "avg_launch_ms_note": "CUDA events around the in_proj launch of every fourth step of the timed region, on the launching stream",
                "stage_ms": dict(zip(STAGES, per_stage)), "dominant_stage": STAGES[dom],
                "stage_ms_note": f"from a second pass of the same {args.steps} steps with an event at every stage boundary "
                                 f"({ms_per_step_with_stage_events:.4f} ms per step there: the events cost the difference)",
                "stage_achieved": {
                    "in_proj_tflops": flops_in / (per_stage[0] * 1e-3) / 1e12 if per_stage[0] > 0 else None,
                    "out_proj_tflops": flops_out / (per_stage[4] * 1e-3) / 1e12 if per_stage[4] > 0 else None,
                    "ssd_tflops": flops_ssd / (per_stage[2] * 1e-3) / 1e12 if per_stage[2] > 0 else None,
                    "conv1d_gbs": 2.0 * tokens * conv_dim * 2 / (per_stage[1] * 1e-3) / 1e9 if per_stage[1] > 0 else None,
                    "gated_rmsnorm_gbs": 3.0 * tokens * cfg["d_inner"] * 2 / (per_stage[3] * 1e-3) / 1e9 if per_stage[3] > 0 else None,
                    "hbm_peak_gbs": peaks["hbm_gbs"]}}
    whole = {"algorithmic_flops_per_step": flops_total, "achieved_tflops": flops_total / (ms_per_step * 1e-3) / 1e12,
             "frac_of_burst_peak": flops_total / (ms_per_step * 1e-3) / 1e12 / peaks["tflops_burst"],
             "frac_of_sustained_peak": flops_total / (ms_per_step * 1e-3) / 1e12 / peaks["tflops_sustained"],
             "frac": flops_total / (ms_per_step * 1e-3) / 1e12 / peak, "peak": peak}

    # ---- CPU baseline: bounded sample on the host cores ----------------------------------------------------------
    cpu = None
    ref_cuda = None
    if world == 1 and not args.no_cpu_baseline:
        t0 = time.perf_counter()
        cpu_tokens = 32
        _, kind = _ref_mixer_tokens(synth.make_input(cfg, 99, batch=1, seqlen=cpu_tokens), w_np, cfg)
        dt = time.perf_counter() - t0
        cpu = {"value": cpu_tokens / dt, "unit": UNIT, "cores": 1, "kind": kind,
               "sample": f"{cpu_tokens} tokens of one sequence through the whole mixer, single thread (the reference is single-threaded), {dt:.1f} s"}
        ref_cuda = reference_cuda_kernels()
        if ref_cuda:
            cpu["reference_cuda_kernels"] = ref_cuda

    sustained = decode = conv1 = None
    if not args.no_extras:
        sustained = sustained_record(torch, lib, mixer, us, out, tokens, flops_total, flops_in, local_rank, peaks, ms_per_step)
        decode = decode_record(torch, ops, local_rank, peaks)
        conv1 = conv_cfg1_record(torch, ops, peaks, ref_cuda)

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": _config_dict(args.workload, cfg, world), "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                    "ms_per_step": e2e_ms / args.steps, "ms_one_call_alone": e2e_single_ms,
                    "host_enqueue_ms_per_step": e2e_enqueue_ms,
                    "call": "b200_mamba2_mixer_prefill_host_ex with B200_HOST_OVERLAP (the inputs sit complete in pinned host memory before "
                            "each call, the weights do not change), the steps queued back to back: the copy-in of step k+1 runs under the compute and copy-out of step k; "
                            "every step copies its own input in and its own output out"},
            "gpu_launches": gpu_launches,
            "gpu_launches_note": ("kernel nodes of the CUDA graph that is the timed region, counted by the library at its launch sites while the graph was captured (rank 0)"
                                  if not args.no_graph else "counted by the library at its launch sites between the two events of the timed region (rank 0)"),
            "timed_region": ("one CUDA graph of the K steps (captured calls of b200_mamba2_mixer_prefill), replayed once" if not args.no_graph
                             else "K calls of b200_mamba2_mixer_prefill launched from the host"),
            "roofline": roofline, "whole_step": whole, "sustained": sustained, "decode": decode, "conv_cfg1": conv1,
            "copy_only": copy_only, "cfg4_dp": cfg4_dp, "cfg4_tp": cfg4_tp, "cpu_baseline": cpu}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# head-sharded tensor parallelism (cfg4): every rank holds the whole batch and 1/N of the heads
# ---------------------------------------------------------------------------------------------------------------

def run_sp(args):
    """`--mode sp` under torchrun with N ranks: ONE long sequence per batch entry (cfg2 layer sizes, `--sp-seqlen` tokens) split
    into N consecutive segments. Per step: local in_proj / conv1d / chunk states -> all-gather of the zero-state segment states
    [b,H,P,N] and log-decays [b,H] (NCCL) -> incoming state -> state passing, chunk scan, gated norm, out_proj. Strong scaling:
    the sequence is fixed."""
    import torch
    import torch.distributed as dist
    from anygpu_b200 import capi, ops
    from anygpu_b200 import dist as bdist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = capi.load()
    cfg = dict(synth.CONFIGS["cfg2"], batch=args.sp_batch, seqlen=args.sp_seqlen)
    b, l = cfg["batch"], cfg["seqlen"]
    wts = ops.ZambaMamba2weights.from_numpy(synth.make_weights(cfg, 0), torch.float16)
    lo, hi = bdist.sp_segments(l, world, align=cfg["chunk"])[rank]
    g = torch.Generator(device="cuda").manual_seed(0)  # same sequence on every rank; each uses its segment (+ 3 halo tokens)
    u = torch.randn(b, l, cfg["d_model"], device="cuda", generator=g).half()
    u_seg = u[:, lo:hi].contiguous()
    halo = u[:, lo - 3:lo].contiguous() if rank > 0 else None
    del u
    mixer = ops.Mamba2MixerSP(cfg, wts)
    out = torch.empty_like(u_seg)
    H, P, N = cfg["nheads"], cfg["headdim"], cfg["d_state"]
    states = torch.empty((world, b, H, P, N), dtype=torch.float32, device="cuda")
    decays = torch.empty((world, b, H), dtype=torch.float32, device="cuda")

    def step():
        s_, d_ = mixer.begin(u_seg, halo)
        if world > 1:
            dist.all_gather_into_tensor(states, s_)
            dist.all_gather_into_tensor(decays, d_)
        else:
            states[0].copy_(s_)
            decays[0].copy_(d_)
        mixer.finish(mixer.prefix(states, decays, rank), out=out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = bdist.max_over_ranks(e0.elapsed_time(e1), device="cuda")
    capi.check("b200_last_device_error", lib.b200_last_device_error(None, None))
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": b * l * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                          "config": {"workload": f"cfg2 layer sizes, batch {b} x ONE sequence of {l} tokens split into {world} segments",
                                     "global_batch": b, "seq_len": l,
                                     "parallelism": f"sp{world}: sequence-parallel, NCCL all-gather of segment states "
                                                    f"({b * H * P * N * 4 / 1e6:.1f} MB per rank) and log-decays"}}))
    if world > 1:
        dist.destroy_process_group()


def run_tp(args):
    """`--mode tp` under torchrun with N ranks: the Zamba2-7B-shaped layer with nheads/N heads per rank. Per chunk of sequences:
    local mixer up to the out_proj addend -> NCCL all-reduce (sum) of the addends and of the per-token sums of squares ->
    row scaling. The all-reduce of chunk i runs on NCCL's stream while chunk i+1 computes. Strong scaling: the batch is fixed."""
    import torch
    import torch.distributed as dist
    from anygpu_b200 import capi, ops
    from anygpu_b200 import dist as bdist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = capi.load()
    cfg = dict(synth.CONFIGS["cfg4"], batch=args.tp_batch)
    b, l = cfg["batch"], cfg["seqlen"]
    w_np = synth.make_weights(cfg, 0)
    loc = synth.tp_local_config(cfg, world)
    wl = ops.ZambaMamba2weights.from_numpy(synth.shard_weights_tp(w_np, cfg, world, rank), torch.float16)
    del w_np
    mixer = ops.Mamba2MixerTP(loc, wl, cfg["d_inner"])
    g = torch.Generator(device="cuda").manual_seed(0)  # same input on every rank
    u = torch.randn(b, l, cfg["d_model"], device="cuda", generator=g).half()
    out = torch.empty_like(u)
    ss = torch.empty(b * l, device="cuda")
    sched = tp_chunk_schedule(b, world, args.tp_chunk)
    starts = [sum(sched[:i]) for i in range(len(sched))]
    chunk = "/".join(str(v) for v in sched)

    def step():
        pending = None
        for c0, n in zip(starts, sched):
            sl = slice(c0, c0 + n)
            rows = slice(sl.start * l, sl.stop * l)
            mixer.partial(u[sl], partial_out=out[sl], sumsq=ss[rows])
            works = []
            if world > 1:
                works = [dist.all_reduce(out[sl], async_op=True), dist.all_reduce(ss[rows], async_op=True)]
            if pending is not None:
                psl, prows, pw = pending
                for wk in pw:
                    wk.wait()
                mixer.finish(out[psl], ss[prows])
            pending = (sl, rows, works)
        psl, prows, pw = pending
        for wk in pw:
            wk.wait()
        mixer.finish(out[psl], ss[prows])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = bdist.max_over_ranks(e0.elapsed_time(e1), device="cuda")
    capi.check("b200_last_device_error", lib.b200_last_device_error(None, None))
    chk = float(out.float().abs().mean())
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": b * l * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "f16", "data": "synthetic", "checksum_mean_abs": chk,
                          "config": {"workload": f"cfg4: Zamba2-7B-shaped mixer prefill, batch {b} x seqlen {l} on every rank, "
                                                 f"{cfg['nheads']} heads sharded {world}-way, ngroups {cfg['ngroups']}",
                                     "global_batch": b, "seq_len": l,
                                     "parallelism": f"tp{world}: head-sharded, NCCL all-reduce of out_proj addends (f16) and of the "
                                                    f"per-token sum of squares, chunks of {chunk} sequences overlapped with compute"}}))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# single-operator mode (micro-benchmarks of the other configurations; small cases for profiler captures)
# ---------------------------------------------------------------------------------------------------------------

def run_kernel(args):
    """Times one operator alone with CUDA events: `--kernel NAME [--small] --steps K --warmup W`.
    conv1d_prefill / conv1d_decode: the standalone conv configuration (batch 8, 4224 channels, 4096 tokens; 256 decode steps).
    decode: the Zamba2-2.7B-shaped decode step (batch 64); ssm_update: its state recurrence alone. in_proj / out_proj / conv1d_tokens / ssd / gated_rmsnorm: the stages
    of the cfg2 mixer on their in-mixer shapes. --small shrinks the token count (profiler-sized case, still larger than L2
    where the operator is bandwidth-bound)."""
    import torch
    from anygpu_b200 import capi, ops
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    k = args.kernel
    h = torch.float16
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *shape, std=1.0: (torch.randn(*shape, device="cuda", generator=g) * std).to(h)
    cfg = workload("cfg2")
    conv_dim, d_in_proj = synth.dims(cfg)
    T = cfg["batch"] * cfg["seqlen"] // (4 if args.small else 1)
    b, l = (1 if args.small else cfg["batch"]), cfg["seqlen"]
    H, P, N, G, Q = cfg["nheads"], cfg["headdim"], cfg["d_state"], cfg["ngroups"], (args.chunk or cfg["chunk"])
    bytes_alg = flops_alg = None
    nbuf = 3
    if k == "conv1d_prefill":
        B_, C_, L_ = (2 if args.small else 8), 4224, 4096
        xs = [rn(B_, C_, L_) for _ in range(nbuf)]
        w, bs = rn(C_, 4, std=0.5), rn(C_, std=0.1)
        fn = lambda i: ops.tensor_causal_conv1d(xs[i % nbuf], w, bs)
        bytes_alg = 2 * B_ * C_ * L_ * 2
    elif k == "conv1d_decode":
        B_, C_ = 8, 4224
        w, bs = rn(C_, 4, std=0.5), rn(C_, std=0.1)
        state, xt = rn(B_, C_, 3), rn(B_, C_)
        fn = lambda i: ops.tensor_causal_conv1d_update(xt, state, w, bs)
        if args.graph:
            # the configuration's 256 consecutive single-token steps as one CUDA graph: per-step device time without the host's
            # launch path (ctypes + launch, ~20 us per call) in between
            per_call = 256
            xts = rn(per_call, B_, C_)
            fn(0)
            torch.cuda.synchronize()
            gobj = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gobj):
                for t in range(per_call):
                    ops.tensor_causal_conv1d_update(xts[t], state, w, bs)
            fn = lambda i: gobj.replay()
        bytes_alg = B_ * C_ * 2 * (3 + 3 + 1 + 1) + C_ * 5 * 2
    elif k == "conv1d_tokens":
        zx = [rn(b, l, d_in_proj) for _ in range(nbuf)]
        w, bs = rn(conv_dim, 4, std=0.5), rn(conv_dim, std=0.1)
        fn = lambda i: ops.tensor_causal_conv1d_tokens(zx[i % nbuf][:, :, cfg["d_inner"]:cfg["d_inner"] + conv_dim], w, bs)
        bytes_alg = 2 * b * l * conv_dim * 2
    elif k == "gated_rmsnorm":
        xs = [rn(T, cfg["d_inner"]) for _ in range(nbuf)]
        zs = [rn(T, cfg["d_inner"]) for _ in range(nbuf)]
        w = rn(cfg["d_inner"])
        fn = lambda i: ops.tensor_zamba_gated_rmsnorm(xs[i % nbuf], zs[i % nbuf], w, cfg["d_inner"], 1e-5)
        bytes_alg = 3 * T * cfg["d_inner"] * 2
    elif k in ("in_proj", "out_proj"):
        K_, N_ = (cfg["d_model"], d_in_proj) if k == "in_proj" else (cfg["d_inner"], cfg["d_model"])
        xs = [rn(T, K_) for _ in range(nbuf)]
        w = rn(K_, N_, std=0.02)
        outs = torch.empty(T, N_, device="cuda", dtype=h)
        fn = lambda i: ops.tensor_linear(xs[i % nbuf], w, out=outs)
        flops_alg = 2.0 * T * K_ * N_
    elif k == "ssd":
        xbc = [rn(b, l, conv_dim, std=0.5) for _ in range(nbuf)]
        dts = rn(b, l, H)
        A = -(torch.rand(H, device="cuda", generator=g) * 15 + 1)
        D, dtb = torch.ones(H, device="cuda"), torch.full((H,), -3.0, device="cuda")
        def fn(i):
            t = xbc[i % nbuf]
            return ops.tensor_mamba_chunk_scan_combined(t[:, :, :H * P].unflatten(2, (H, P)), dts, A,
                                                        t[:, :, H * P:H * P + G * N].unflatten(2, (G, N)),
                                                        t[:, :, H * P + G * N:].unflatten(2, (G, N)), Q, D=D, dt_bias=dtb)
        nchunks = -(-l // Q)
        flops_alg = float(b * nchunks * (H * (2 * Q * Q * P + 4 * Q * N * P) + G * 2 * Q * Q * N))
    elif k == "varlen":
        # 256 sequences of about 32 tokens in one packed call against the same sequences prefilled one by one (cfg2 layer sizes)
        r = np.random.default_rng(0)
        lens = [int(v) for v in r.integers(20, 45, 256)]
        total = sum(lens)
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        vcfg = dict(cfg, batch=1, seqlen=64, chunk=128)
        wts = ops.ZambaMamba2weights.from_numpy(synth.make_weights(vcfg, 0), h)
        mixer = ops.Mamba2Mixer(vcfg, wts)
        ud = rn(total, vcfg["d_model"])
        od = torch.empty_like(ud)
        seqs = [ud[cu[s]:cu[s + 1]].unsqueeze(0).contiguous() for s in range(len(lens))]
        if args.varlen_loop:
            def fn(i):
                for sq in seqs:
                    mixer.prefill(sq)
        else:
            fn = lambda i: mixer.prefill_varlen(ud, cu, out=od)
        extra = {"sequences": len(lens), "total_tokens": total, "mode": "one prefill per sequence" if args.varlen_loop else "one packed call"}
    elif k == "ssm_update":
        c3 = workload("cfg3")
        B_, H_, P_, N_, G_ = c3["batch"], c3["nheads"], c3["headdim"], c3["d_state"], c3["ngroups"]
        state = torch.randn(B_, H_, P_, N_, device="cuda", generator=g) * 0.1
        xs_, dts_ = rn(B_, H_, P_, std=0.5), rn(B_, H_)
        Bs_, Cs_ = rn(B_, G_, N_, std=0.5), rn(B_, G_, N_, std=0.5)
        A_ = -(torch.rand(H_, device="cuda", generator=g) * 15 + 1)
        D_, dtb_ = torch.ones(H_, device="cuda"), torch.full((H_,), -3.0, device="cuda")
        fn = lambda i: ops.tensor_mamba_selective_state_update(state, xs_, dts_, A_, Bs_, Cs_, D=D_, dt_bias=dtb_)
        bytes_alg = 2 * state.numel() * 4
    elif k == "decode":
        c3 = workload("cfg3")
        wts = ops.ZambaMamba2weights.from_numpy(synth.make_weights(c3, 0), h, layout=ops.W_NK if args.layout == "NK" else ops.W_KN)
        mixer = ops.Mamba2Mixer(c3, wts)
        cs, ss = synth.make_decode_state(c3, 0)
        cache = ops.ZambaMambaCache(torch.from_numpy(cs).cuda().half(), torch.from_numpy(ss).cuda())
        u = rn(c3["batch"], c3["d_model"])
        o = torch.empty_like(u)
        per_call = 1
        if args.graph and args.graph_steps > 1:
            per_call = args.graph_steps
            us_, os_ = rn(per_call, c3["batch"], c3["d_model"]), torch.empty(per_call, c3["batch"], c3["d_model"], device="cuda", dtype=h)
            graph = mixer.capture_decode_steps(us_, cache, os_)
            fn = lambda i: graph.replay()
        elif args.graph:
            graph = mixer.capture_decode(u, cache, o)
            fn = lambda i: graph.replay()
        else:
            fn = lambda i: mixer.decode(u, cache, out=o)
        cd3, dip3 = synth.dims(c3)
        bytes_alg = (c3["d_model"] * dip3 + c3["d_inner"] * c3["d_model"]) * 2 + 2 * ss.size * 4 + 2 * cs.size * 2
    else:
        raise SystemExit(f"unknown kernel {k}")
    for i in range(args.warmup):
        fn(i)
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for i, (e0, e1) in enumerate(evs):
        e0.record()
        fn(i)
        e1.record()
    torch.cuda.synchronize()
    per_call = locals().get("per_call", 1)
    ms = sorted(e0.elapsed_time(e1) / per_call for e0, e1 in evs)
    med, mn = ms[len(ms) // 2], ms[0]
    capi.check("b200_last_device_error", capi.load().b200_last_device_error(None, None))
    out = {"kernel": k, "small": bool(args.small), "graph": bool(args.graph), "graph_steps": (per_call if k == "conv1d_decode" else args.graph_steps) if args.graph else 0, "steps": args.steps, "median_us": med * 1e3, "min_us": mn * 1e3}
    out.update(locals().get("extra", {}))
    if bytes_alg:
        out.update(algorithmic_bytes=bytes_alg, gbs_median=bytes_alg / (med * 1e-3) / 1e9, hbm_peak_gbs=peaks["hbm_gbs"],
                   frac_of_hbm_peak=bytes_alg / (med * 1e-3) / 1e9 / peaks["hbm_gbs"], peak_source=peaks["source"])
    if flops_alg:
        out.update(algorithmic_flops=flops_alg, tflops_median=flops_alg / (med * 1e-3) / 1e12, tensor_peak_tflops=peaks["tflops_burst"],
                   frac_of_tensor_peak=flops_alg / (med * 1e-3) / 1e12 / peaks["tflops_burst"], peak_source=peaks["source"])
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="only the prefill line: no sustained / decode / conv / copy-only / cfg4 records")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps from the host instead of replaying them as one CUDA graph")
    ap.add_argument("--no-cfg4", action="store_true", help="skip the two Zamba2-7B-shaped records (batch-sharded, head-sharded)")
    ap.add_argument("--mode", default="dp", choices=["dp", "tp", "sp"],
                    help="dp: batch-sharded (default); tp: head-sharded cfg4 layer; sp: one long sequence split over the ranks")
    ap.add_argument("--sp-seqlen", type=int, default=32768)
    ap.add_argument("--sp-batch", type=int, default=1)
    ap.add_argument("--tp-batch", type=int, default=32)
    ap.add_argument("--tp-chunk", type=int, default=0,
                    help="sequences per compute / all-reduce pipeline step of the head-sharded runs (0: see tp_chunk_schedule)")
    ap.add_argument("--kernel", default=None, help="time one operator alone (see run_kernel)")
    ap.add_argument("--small", action="store_true", help="with --kernel: profiler-sized case")
    ap.add_argument("--varlen-loop", action="store_true", help="with --kernel varlen: the per-sequence loop instead of the packed call")
    ap.add_argument("--chunk", type=int, default=0, help="with --kernel ssd: chunk length of the scan (default: the configuration's 256)")
    ap.add_argument("--layout", default="KN", choices=["KN", "NK"], help="with --kernel decode: projection weight layout")
    ap.add_argument("--graph-steps", type=int, default=1, help="with --kernel decode --graph: consecutive steps recorded into one graph")
    ap.add_argument("--graph", action="store_true", help="with --kernel decode / conv1d_decode: replay the step(s) from a CUDA graph")
    args = ap.parse_args()
    if args.kernel:
        return run_kernel(args)
    if args.mode == "tp" and args.impl == "b200":
        return run_tp(args)
    if args.mode == "sp" and args.impl == "b200":
        return run_sp(args)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
