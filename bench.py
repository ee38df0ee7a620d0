#!/usr/bin/env python
"""Benchmark of the convolution hot path (forward + backward-data + weight gradient) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--batch B] [--skip-cpu]

Workload: the data-parallel convolution sweep -- batch 1024 of 256x32x32 N(0,1) images, 256 filters
3x3, stride 1, padding 1, He-normal weights, N(0,1) upstream delta; one step = the convolution layer's Forward (ForwardConvolution) and
TrainingBackward (BackwardConvolution + batch-summed CreateDeltaWeightAndBias) over the whole batch (and, for N > 1, the
NCCL all-reduce of the dW/dB arena).  The batch is split over the N ranks (strong scaling).
Metric: algorithmic convolution TFLOP/s, 3 passes x 2*N*K*C*kh*kw*OH*OW flops per step; the extra MMAs
of the 3xTF32 mode and packing passes are not counted as work.

The headline line is measured in plain-TF32 mode (the mode the 60 %-of-TF32-peak target refers to,
parity tolerance 2e-3); the "tf32x3" object of the same line is the same step in 3xTF32 mode
(tolerance 1e-4).  `e2e` times the same step through the C-ABI with HOST buffers: pinned-host -> device
copies of the step's image and delta tensors and the device -> host read of dW/dB are inside the
timed region.  `--impl reference` times the reference's own CPU backend (oracle/_ref/libref.so, one
sample per host thread per step) on the same layer.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(C=256, H=32, W=32, K=256, k=3, s=1, p=1, batch=1024)
METRIC = "conv_fwd_bwd_wgrad_tflops"


_RESULT_FD = None


def keep_stdout_clean():
    """The one JSON line must be all that reaches stdout: libraries (NCCL's version banner) write there too, so the
    process's stdout is pointed at stderr and the result goes to a private copy of the original descriptor."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(text):
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, (text + "\n").encode())


def flops_per_sample(c):
    oh = (c["H"] - c["k"] + 2 * c["p"]) // c["s"] + 1
    ow = (c["W"] - c["k"] + 2 * c["p"]) // c["s"] + 1
    return 3 * 2.0 * c["K"] * c["C"] * c["k"] * c["k"] * oh * ow


def profiled_traffic():
    """dram bytes (read + written) per image and tensor-core launch, from the committed ncu summary of the kernel
    (profiles/tc_kernel_dp_conv_sweep_batch128.md carries one machine-readable line for it); (bytes, source) or (None, why)."""
    path = os.path.join(ROOT, "profiles", "tc_kernel_dp_conv_sweep_batch128.md")
    try:
        for line in open(path):
            if line.startswith("traffic_bytes_per_image_and_launch:"):
                fields = line.split()
                return float(fields[1]), "profiles/tc_kernel_dp_conv_sweep_batch128.md (%s), scaled by the images of a launch" % " ".join(fields[2:])
    except OSError:
        pass
    return None, "no ncu summary with a traffic line under profiles/"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16_sustained=p.get("bf16_tflops_sustained"), bf16_burst=p.get("bf16_tflops"), hbm=p.get("hbm_gbs"),
                    sm_mhz=(p.get("clocks_under_load") or {}).get("sm_mhz_median"), source="MEASURED_PEAKS.json")
    return dict(bf16_sustained=1400.0, bf16_burst=1590.0, hbm=6650.0, sm_mhz=1300.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons of one GPU through NVML from a
    thread while the timed region runs (read-only queries, every ~5 ms); falls back to one
    nvidia-smi query if the NVML binding is missing."""
    REASONS = (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40), ("sw_power_cap", 0x4))

    def __init__(self, index):
        self.samples, self.bits, self.max_mhz, self.stop_flag, self.thread = [], 0, None, False, None
        self.index = index
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:
            self.nv = None

    @staticmethod
    def _physical_index(index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v for v in vis.split(",") if v.strip() != ""]
            if index < len(ids) and ids[index].strip().isdigit():
                return int(ids[index])
        return index

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self, t0, t1):
        if self.nv is None:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
                f = [float(v) for v in out.strip().split(",")]
                return dict(sm_mhz=f[0], sm_max_mhz=f[1], reasons=["sampled once after the timed region (no NVML binding)"], samples=1)
            except Exception:
                return dict(sm_mhz=None, sm_max_mhz=None, reasons=["clock sampling unavailable"], samples=0)
        self.stop_flag = True
        self.thread.join(timeout=2)
        sm = sorted(self.samples)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=self.max_mhz,
                    reasons=[name for name, bit in self.REASONS if self.bits & bit], samples=len(sm))


def reference_arm(args, rank, world):
    """The reference's own CPU backend on the host cores: each step runs one sample of the layer
    (forward, backward, weight gradient) on each of T threads."""
    if rank != 0:
        return
    import numpy as np
    from oracle import Oracle
    try:
        ref = Oracle("reference")
        kind = "reference"
    except FileNotFoundError:
        ref = Oracle("port")
        kind = "port"
    c = CFG
    T = max(1, min(os.cpu_count() or 1, args.cpu_threads))
    r = np.random.default_rng(5)
    xs = [r.normal(0, 1, (1, c["C"], c["H"], c["W"])).astype(np.float32) for _ in range(T)]
    ds = [r.normal(0, 1, (1, c["K"], c["H"], c["W"])).astype(np.float32) for _ in range(T)]
    wt = r.normal(0, (2.0 / (c["C"] * 9)) ** 0.5, (1, c["K"], c["C"] * 9)).astype(np.float32)
    zb = np.zeros((1, c["K"]), np.float32)

    def one(i):
        ref.conv_forward(xs[i], wt, zb, 3, 3, 1, 1, 1, 1)
        ref.conv_backward(ds[i], wt, zb, (c["C"], c["H"], c["W"]), 3, 3, 1, 1, 1, 1)
        ref.conv_wgrad(np.zeros((1, c["K"], c["C"] * 9), np.float32), zb, xs[i], ds[i], 3, 3, 1, 1, 1, 1)

    def step():
        th = [threading.Thread(target=one, args=(i,)) for i in range(T)]
        [t.start() for t in th]
        [t.join() for t in th]

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = flops_per_sample(c) * T * args.steps / dt / 1e12
    sample = f"{T} samples (1 per host thread) of the 256x32x32 -> 256 3x3 layer per step, fwd+bwd+wgrad"
    line = dict(impl="reference", metric=METRIC, value=val, unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=dt / args.steps * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32",
                data="synthetic", config=dict(workload="dp_conv_sweep_256x32x32_k256_3x3 (CPU sample)", sample=sample),
                cpu_baseline=dict(value=val, unit="TFLOP/s", cores=T, kind=kind, sample=sample, host_cores=os.cpu_count()),
                e2e=dict(value=val, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    # the one configuration the CPU backend runs WHOLE (BASELINE configs[0]): same step as the `cfg1` object of the GPU arm
    line["cfg1"] = dict(single_thread=cfg1_cpu(steps=max(2, min(args.steps, 5)), threads=1),
                        all_threads=cfg1_cpu(steps=max(2, min(args.steps, 5)), threads=T))
    emit(json.dumps(line))


def _dot_rel_err(got, want, absdot):
    """max |got - want| / sum |a||b| (the forward-error-bound form of relative error; tests/util.py)."""
    import numpy as np
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(absdot.astype(np.float64), 1e-30)))


def _survey_rel_err(got, want):
    """max |got - want| / max(|want|, 1e-3 max |want|) (tests/util.py)."""
    import numpy as np
    want = want.astype(np.float64)
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), 1e-3 * np.max(np.abs(want)))))


def parity_leg(samples):
    """The benchmark's own results on sampled images of the timed batch against the reference CPU backend (checker, all host
    threads): both error figures per mode, for the bench line's config.parity.
    samples: dict(x, d, w, idx, modes={mode: (y[idx], dx[idx])}) as numpy arrays."""
    import numpy as np
    from oracle import Oracle
    try:
        ref = Oracle("reference", threads=os.cpu_count() or 1)
    except FileNotFoundError:
        ref = Oracle("port", threads=os.cpu_count() or 1)
    c = CFG
    x, d, w = samples["x"], samples["d"], samples["w"]
    zb = np.zeros((1, c["K"]), np.float32)
    want_y, mag_y = ref.conv_forward(x, w, zb, 3, 3, 1, 1, 1, 1), ref.conv_forward(np.abs(x), np.abs(w), zb, 3, 3, 1, 1, 1, 1)
    shape = (c["C"], c["H"], c["W"])
    want_dx, mag_dx = ref.conv_backward(d, w, zb, shape, 3, 3, 1, 1, 1, 1), ref.conv_backward(np.abs(d), np.abs(w), zb, shape, 3, 3, 1, 1, 1, 1)
    out = dict(checker="reference CPU backend (oracle/_ref)" if ref.kind == "reference" else "CPU restatement (oracle/)",
               sample="forward and backward-data of images %s of the timed batch" % list(samples["idx"]),
               tolerance="2e-3 (tf32) / 1e-4 (tf32x3) on dot_rel_err = |err| / sum|a||b|; survey_rel_err = |err| / max(|want|, 1e-3 max|want|) is reported beside it")
    for mode, (y, dx) in samples["modes"].items():
        out[mode] = dict(forward=dict(dot_rel_err=_dot_rel_err(y, want_y, mag_y), survey_rel_err=_survey_rel_err(y, want_y)),
                         backward_data=dict(dot_rel_err=_dot_rel_err(dx, want_dx, mag_dx), survey_rel_err=_survey_rel_err(dx, want_dx)))
    return out


def cpu_baseline(seconds_budget=25.0):
    """Single-core reference CPU backend on a bounded sample of the workload (whole samples until ~budget)."""
    import numpy as np
    from oracle import Oracle
    try:
        ref = Oracle("reference")
        kind = "reference"
    except FileNotFoundError:
        ref = Oracle("port")
        kind = "port"
    c = CFG
    r = np.random.default_rng(5)
    wt = r.normal(0, (2.0 / (c["C"] * 9)) ** 0.5, (1, c["K"], c["C"] * 9)).astype(np.float32)
    zb = np.zeros((1, c["K"]), np.float32)
    n = 0
    t0 = time.perf_counter()
    while True:
        x = r.normal(0, 1, (1, c["C"], c["H"], c["W"])).astype(np.float32)
        d = r.normal(0, 1, (1, c["K"], c["H"], c["W"])).astype(np.float32)
        ref.conv_forward(x, wt, zb, 3, 3, 1, 1, 1, 1)
        ref.conv_backward(d, wt, zb, (c["C"], c["H"], c["W"]), 3, 3, 1, 1, 1, 1)
        ref.conv_wgrad(np.zeros((1, c["K"], c["C"] * 9), np.float32), zb, x, d, 3, 3, 1, 1, 1, 1)
        n += 1
        dt = time.perf_counter() - t0
        if dt > seconds_budget * 0.6 or n >= 8:
            break
    return dict(value=flops_per_sample(c) * n / dt / 1e12, unit="TFLOP/s", cores=1, kind=kind, host_cores=os.cpu_count(),
                sample=f"{n} of {c['batch']} samples of the workload, fwd+bwd+wgrad, single thread, {dt:.1f} s")


def dcgan_cpu_baseline(images=2):
    """The combined DCGAN step (generator and discriminator chains, forward + backward + weight gradients) on the CPU twin
    built from the reference CPU backend's tensor routines, single thread, on a few images."""
    import numpy as np
    import torch
    from cuda_cnn_gan_vae_b200.nets import dcgan_discriminator, dcgan_generator
    from oracle import Oracle
    from oracle.net_twin import OracleNet
    try:
        port, kind = Oracle("reference"), "reference"
    except FileNotFoundError:
        port, kind = Oracle("port"), "port"
    G, D = dcgan_generator(images), dcgan_discriminator(images)
    tg, td = OracleNet(port, G), OracleNet(port, D)
    r = np.random.default_rng(7)
    z = r.standard_normal((images, 1, 100, 1)).astype(np.float32)
    labels = r.integers(0, 2, (images, 1, 1, 1)).astype(np.float32)
    t0 = time.perf_counter()
    fake = tg.forward(z)
    out = td.forward(fake)
    d_image = td.backward((out.reshape(labels.shape) - labels).astype(np.float32), need_input_error=True)
    tg.backward(d_image)
    dt = time.perf_counter() - t0
    del torch
    return dict(value=images / dt, unit="img/s", cores=1, kind=kind, host_cores=os.cpu_count(),
                sample=f"{images} images through generator + discriminator fwd+bwd+dW (no optimiser), single thread, {dt:.1f} s")


class _L2Flush:
    """Writes a buffer larger than L2 (126 MB) so that the next timed launch finds none of its operands cached."""

    def __init__(self, torch):
        self.buf = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.buf.zero_()


def _timed_with_flush(torch, fn, flush, iters, warmup=3):
    """Mean device time of fn in ms: one CUDA-event pair per call, an L2 flush before every call (outside the pair)."""
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(iters):
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


CFG1 = dict(B=16, C=3, H=64, W=64, K=32, k=3)


def cfg1_flops():
    c = CFG1
    return 3 * 2.0 * c["B"] * c["K"] * c["C"] * c["k"] * c["k"] * c["H"] * c["W"]


def cfg1_inputs():
    import numpy as np
    c = CFG1
    r = np.random.default_rng(1)
    x = r.uniform(-1, 1, (c["B"], c["C"], c["H"], c["W"])).astype(np.float32)
    wt = r.normal(0, (2.0 / (c["C"] * 9)) ** 0.5, (1, 1, c["K"], c["C"] * 9)).astype(np.float32)
    d = r.normal(0, 1, (c["B"], c["K"], c["H"], c["W"])).astype(np.float32)
    return x, wt, d


def cfg1_gpu(torch, ops, iters=30):
    """The CPU-runnable configuration (batch 16 of 3x64x64 U[-1,1], 32 filters 3x3 s1 p1, He-normal weights, zero bias,
    N(0,1) error; seed 1): one step = the convolution layer's Forward and TrainingBackward.  Device-resident and through
    host buffers, L2 flushed before every step (the operands are far smaller than L2)."""
    c = CFG1
    x, wt, d = cfg1_inputs()
    hx, hd = torch.from_numpy(x).pin_memory(), torch.from_numpy(d).pin_memory()
    X, D, WT = hx.cuda(), hd.cuda(), torch.from_numpy(wt).cuda()
    bias = torch.zeros(1, c["K"], 1, 1, device="cuda")
    y, dx = torch.empty_like(D), torch.empty_like(X)
    dk, db = torch.empty_like(WT), torch.empty_like(bias)
    hres = torch.empty(dk.numel() + db.numel()).pin_memory()
    layer = ops.ConvLayer(c["C"], c["H"], c["W"], c["K"], 3, 3, 1, 1, 1, 1, c["B"])
    flush = _L2Flush(torch)

    def step():
        layer.forward(y, X, WT, bias)
        layer.backward(dx, dk, db, D, X, WT, accumulate=False)

    def e2e_step():
        X.copy_(hx, non_blocking=True)
        D.copy_(hd, non_blocking=True)
        step()
        hres[:dk.numel()].copy_(dk.view(-1), non_blocking=True)
        hres[dk.numel():].copy_(db.view(-1), non_blocking=True)

    out = dict(workload="single convolution layer: batch 16 of 3x64x64 U[-1,1], 32 filters 3x3 s1 p1, fwd+bwd-data+wgrad (BASELINE configs[0])",
               flops_per_step=cfg1_flops(), unit="TFLOP/s", l2="flushed before every step")
    for name, mode in (("tf32x3", ops.TF32X3), ("tf32", ops.TF32), ("fp32", ops.FP32)):
        ops.set_precision(mode)
        ms = _timed_with_flush(torch, step, flush, iters)
        out[name] = dict(value=cfg1_flops() / (ms * 1e-3) / 1e12, ms_per_step=ms, path="tcgen05" if ops.last_path() == ops.PATH_TCGEN05 else "cuda cores")
    ops.set_precision(ops.TF32)
    ms = _timed_with_flush(torch, e2e_step, flush, iters)
    out["e2e"] = dict(value=cfg1_flops() / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=ms, h2d_bytes_per_step=int((hx.numel() + hd.numel()) * 4),
                      d2h_bytes_per_step=int(hres.numel() * 4), note="image and error from pinned host memory, dW|dB read back; plain-TF32 mode")
    ops.stream_status()
    layer.close()
    return out


def cfg1_cpu(steps=3, threads=1):
    """The same configuration, WHOLE, on the reference CPU backend: forward, backward-data with a zero bias, per-sample
    weight gradients reduced over the batch (the layer's sequence, netlayer/cnetlayerconvolution.cu.h:310,484-508)."""
    import numpy as np
    from oracle import Oracle
    try:
        ref, kind = Oracle("reference", threads=threads), "reference"
    except FileNotFoundError:
        ref, kind = Oracle("port", threads=threads), "port"
    c = CFG1
    x, wt, d = cfg1_inputs()
    zb = np.zeros((1, c["K"]), np.float32)

    def step():
        ref.conv_forward(x, wt[0], zb, 3, 3, 1, 1, 1, 1)
        ref.conv_backward(d, wt[0], zb, (c["C"], c["H"], c["W"]), 3, 3, 1, 1, 1, 1)
        dk, db = ref.conv_wgrad(np.zeros((c["B"], c["K"], c["C"] * 9), np.float32), np.zeros((c["B"], c["K"]), np.float32), x, d, 3, 3, 1, 1, 1, 1)
        return dk.sum(0), db.sum(0)

    step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dict(value=cfg1_flops() / dt / 1e12, unit="TFLOP/s", ms_per_step=dt * 1e3, cores=threads, kind=kind, host_cores=os.cpu_count(),
                same_config=True, sample="the whole configuration (batch 16), %d steps" % steps)


def vae_bench(torch, ops, lib, timed, steps, world=1):
    """BASELINE configs[3]: the convolutional VAE training step at batch 128 of 3x128x128 per GPU (encoder 32-64-128-256 with
    max-pooling, two Linear heads to 256, reparameterisation with supplied noise, mirror decoder, MSE + KL errors, Adam)."""
    from cuda_cnn_gan_vae_b200.nets import VAEStep
    B = 128
    gen = torch.Generator(device="cuda").manual_seed(41)
    hx = torch.rand(B, 3, 128, 128).pin_memory()
    heps = torch.randn(B, 1, 256, 1).pin_memory()
    x, eps = hx.cuda(), heps.cuda()
    hres = torch.empty(1).pin_memory()
    out = dict(unit="img/s", per_gpu_batch=B, workload="conv VAE train step: batch 128 of 3x128x128 U[0,1], encoder 3x3 convs 32-64-128-256 + 2x2 max-pool, "
               "Linear heads to 256-d mean / log-variance, reparameterisation with N(0,1) noise, mirror decoder with upsampling, MSE + KL, Adam (BASELINE configs[3])")
    del gen
    for name, mode in (("tf32x3", ops.TF32X3), ("tf32", ops.TF32)):
        ops.set_precision(mode)
        step = VAEStep(B, world=world)
        n0 = lib.b200_launch_count()
        step(x, eps)
        launches = lib.b200_launch_count() - n0
        ms, clocks, _, _ = timed(lambda: step(x, eps), max(3, steps // 2), 3)
        ops.stream_status()
        out[name] = dict(value=B * world / (ms * 1e-3), ms_per_step=ms, gpu_launches=int(launches))
        out["parameters"] = int(sum(net.parameter_count for net in step.nets))

        if mode == ops.TF32:
            def e2e_step():
                x.copy_(hx, non_blocking=True)
                eps.copy_(heps, non_blocking=True)
                x_hat = step(x, eps)
                hres.copy_(x_hat.view(-1)[:1], non_blocking=True)
                torch.cuda.current_stream().synchronize()
            ms, _, _, _ = timed(e2e_step, max(3, steps // 2), 2)
            out["e2e"] = dict(value=B * world / (ms * 1e-3), unit="img/s", ms_per_step=ms, h2d_bytes_per_step=int((hx.numel() + heps.numel()) * 4 * world),
                              d2h_bytes_per_step=4 * world, note="images and noise from pinned host memory every step; plain-TF32 mode")
        del step
        torch.cuda.empty_cache()
    out["value"] = out["tf32"]["value"]
    return out


def vae_cpu_baseline(images=1):
    """The same step (no optimiser) on the CPU twin built from the reference CPU backend's routines, single thread."""
    import numpy as np
    from cuda_cnn_gan_vae_b200.nets import VAEStep
    from oracle import Oracle
    from oracle.net_twin import OracleNet
    try:
        ref, kind = Oracle("reference"), "reference"
    except FileNotFoundError:
        ref, kind = Oracle("port"), "port"
    port = Oracle("port")
    step = VAEStep(images)
    enc, mu_t, lv_t, dec = (OracleNet(ref, net) for net in step.nets)
    r = np.random.default_rng(9)
    x = r.uniform(0, 1, (images, 3, 128, 128)).astype(np.float32)
    eps = r.standard_normal((images, 256)).astype(np.float32)
    t0 = time.perf_counter()
    feat = enc.forward(x)
    mu, lv = mu_t.forward(feat), lv_t.forward(feat)
    z, _ = port.vae_forward(mu.reshape(images, -1), lv.reshape(images, -1), eps)
    x_hat = dec.forward(z.reshape(images, 1, 256, 1))
    n = float(x[0].size)
    d_z = dec.backward(ref.binary("sub", x_hat, x, 2.0 / n, 2.0 / n), need_input_error=True)
    d_mu, d_lv = port.vae_backward(d_z.reshape(images, -1), mu.reshape(images, -1), lv.reshape(images, -1), eps, 1.0)
    e = ref.binary("add", mu_t.backward(d_mu.reshape(images, 1, 256, 1), need_input_error=True),
                   lv_t.backward(d_lv.reshape(images, 1, 256, 1), need_input_error=True))
    enc.backward(e)
    dt = time.perf_counter() - t0
    return dict(value=images / dt, unit="img/s", cores=1, kind=kind, host_cores=os.cpu_count(),
                sample=f"{images} image(s) through encoder, heads, decoder fwd+bwd+dW (no optimiser), single thread, {dt:.1f} s")


def gemm_bench(torch, ops, peak_gbs, iters=10):
    """The Linear layers' three products (netlayer/cnetlayerlinear.cu.h:262-278, 415-445) at the shapes of the configurations:
    out = W x (Mul), prev = W^T d (TransponseMul), dW = D^T X (TransponseMul over the batch).  These products are bound by the
    bytes of their largest operand (a few FLOP per byte): algorithmic bytes = every operand and the result once / device
    time with L2 flushed, against the measured HBM copy bandwidth."""
    shapes = [("dcgan generator: 100 -> 8192, batch 64", 64, 8192, 100), ("dcgan discriminator: 8192 -> 1, batch 64", 64, 1, 8192),
              ("vae heads: 16384 -> 256, batch 128", 128, 256, 16384), ("vae decoder input: 256 -> 16384, batch 128", 128, 16384, 256)]
    flush = _L2Flush(torch)
    gen = torch.Generator(device="cuda").manual_seed(3)
    out = dict(unit="GB/s", peak=peak_gbs, peak_source="hbm_gbs (copy bandwidth), of measured", l2="flushed before every call", shapes=[])
    for mode_name, mode in (("tf32", ops.TF32), ("tf32x3", ops.TF32X3)):
        ops.set_precision(mode)
        for name, B, n_out, n_in in shapes:
            Wm = torch.randn(1, 1, n_out, n_in, device="cuda", generator=gen) * (2.0 / n_in) ** 0.5
            x = torch.randn(B, 1, n_in, 1, device="cuda", generator=gen)
            d = torch.randn(B, 1, n_out, 1, device="cuda", generator=gen)
            h, prev, dw = torch.empty(B, 1, n_out, 1, device="cuda"), torch.empty(B, 1, n_in, 1, device="cuda"), torch.empty(1, 1, n_out, n_in, device="cuda")
            cases = (("forward", lambda: ops.CTensorMath.Mul(h, Wm, x)),
                     ("backward", lambda: ops.CTensorMath.TransponseMul(prev, Wm, d)),
                     ("weight_gradient", lambda: ops.CTensorMath.TransponseMul(dw, d.view(1, 1, B, n_out), x.view(1, 1, B, n_in))))
            entry = dict(layer=name, mode=mode_name)
            for cname, fn in cases:
                ms = _timed_with_flush(torch, fn, flush, iters)
                nbytes = 4.0 * (n_out * n_in + B * n_in + B * n_out)
                gbs = nbytes / (ms * 1e-3) / 1e9
                entry[cname] = dict(ms=ms, tflops=2.0 * B * n_out * n_in / (ms * 1e-3) / 1e12, algorithmic_mb=nbytes / 1e6, achieved_gbs=gbs,
                                    frac=gbs / peak_gbs, path="tcgen05" if ops.last_path() == ops.PATH_TCGEN05 else "cuda cores")
            out["shapes"].append(entry)
    ops.stream_status()
    return out


def hbm_kernels(torch, ops, peak_gbs, iters=5):
    """The memory-bound kernels around the contractions on tensors well beyond L2 (256 MiB of fp32 activations: the
    VAE encoder's first feature map, 128 x 32 x 128 x 128): algorithmic bytes (every input read once, every output
    written once) / CUDA-event time, against the measured HBM copy bandwidth."""
    W, Z, Y, X = 128, 32, 128, 128
    n = Z * Y * X
    gen = torch.Generator(device="cuda").manual_seed(17)
    a = torch.randn(W, Z, Y, X, device="cuda", generator=gen)
    b = torch.randn(W, Z, Y, X, device="cuda", generator=gen)
    o1, o2 = torch.empty_like(a), torch.empty_like(a)
    stat = [torch.rand(1, Z, Y, X, device="cuda", generator=gen) + 0.5 for _ in range(3)]
    s_out = [torch.empty(1, Z, Y, X, device="cuda") for _ in range(5)]
    bn_s = [torch.rand(1, 2 * Z, Y, X, device="cuda", generator=gen) + 0.5 for _ in range(7)]
    bias = torch.randn(1, Z, 1, 1, device="cuda", generator=gen)
    half = torch.empty(W, Z, Y // 2, X // 2, device="cuda")
    pos = torch.empty(W, Z, Y // 2, X // 2, 2, dtype=torch.int32, device="cuda")
    planes = torch.empty(W, Z, 1, 1, device="cuda")
    flat = lambda t: t.view(1, 1, 1, -1)
    lib = ops.load()
    P, S, chk = ops._ptr, ops._stream, ops._check
    F = 4.0 * W * n                                    # bytes of one full activation tensor
    st = 4.0 * n
    cases = [
        # batch normalisation at the DCGAN batch: the same 256 MiB viewed as 64 x (2 n) elements
        ("bn_forward", lambda: chk(lib.b200_bn_forward(P(o1), P(o2), P(bn_s[2]), P(bn_s[3]), P(bn_s[4]), P(bn_s[5]), P(bn_s[6]), P(a),
                                                       P(bn_s[0]), P(bn_s[1]), W // 2, 2 * n, 0.9, 1e-6, S())), 3 * F + 14 * st),
        ("bn_backward", lambda: chk(lib.b200_bn_backward(P(o1), P(bn_s[2]), P(bn_s[3]), P(a), P(b), P(bn_s[0]), P(bn_s[1]), W // 2, 2 * n, 1, S())),
         3 * F + 12 * st),
        ("bias_activation", lambda: ops.CTensorApplyFunc.BiasActivation(o1, bias, "leaky_relu", 0.2), 2 * F),
        ("activation_backward", lambda: ops.CTensorApplyFunc.Backward(o1, a, b, "leaky_relu", 0.2), 3 * F),
        ("maxpool", lambda: ops.CTensorMath.MaxPooling(half, pos, a, 2, 2), F + F / 4 + 2 * F / 4),
        ("maxpool_backward", lambda: ops.CTensorMath.MaxPoolingBackward(o1, pos, half, 2, 2), F + F / 4 + 2 * F / 4),
        ("upsample", lambda: ops.CTensorMath.UpSampling(o1, half, 2, 2), F + F / 4),
        ("downsample", lambda: ops.CTensorMath.DownSampling(half, a, 2, 2), F + F / 4),
        ("summ_xy", lambda: ops.CTensorMath.SummXY(planes, a), F),
        ("add_sum_w", lambda: ops.CTensorMath.AddSumW(s_out[0], s_out[0], a), F + 2 * st),
        ("add", lambda: ops.CTensorMath.Add(o1, a, b, 0.5, 0.25), 3 * F),
        ("adam", lambda: ops.CTensorMath.Adam(flat(o1), flat(a), flat(b), flat(o2), 64, 1e-3, 0.9, 0.999, 1e-8, 2), 7 * F),
    ]
    out = {}
    for name, fn, nbytes in cases:
        if name == "adam":
            o2.abs_()                                  # the second-moment operand must not be negative
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = dict(ms=ms, algorithmic_mb=nbytes / 1e6, achieved_gbs=gbs, frac=gbs / peak_gbs)
    ops.stream_status()
    return dict(unit="GB/s", peak=peak_gbs, peak_source="hbm_gbs (copy bandwidth), of measured", tensor="128x32x128x128 fp32 (256 MiB), beyond L2",
                kernels=out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=CFG["batch"], help="global batch (default: the headline 1024)")
    ap.add_argument("--cpu-threads", type=int, default=64)
    ap.add_argument("--skip-cpu", action="store_true", help="leave out the cpu_baseline leg")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-dcgan", action="store_true", help="leave out the DCGAN training-step measurement")
    ap.add_argument("--skip-hbm", action="store_true", help="leave out the memory-bound kernel measurements")
    ap.add_argument("--skip-extra", action="store_true", help="leave out the cfg1, VAE and Linear-product measurements (single GPU only)")
    ap.add_argument("--vae-only", action="store_true", help="run only the VAE training-step measurement (profiling aid)")
    ap.add_argument("--conv-layer", default=None, metavar="C,H,W,K,k,s,p,B",
                    help="run only Forward + TrainingBackward of one convolution layer of this geometry in plain TF32 (profiling aid)")
    ap.add_argument("--hbm-only", action="store_true", help="run only the memory-bound kernel measurements (profiling aid)")
    ap.add_argument("--dcgan-batch", type=int, default=64, help="images per GPU in the DCGAN step")
    ap.add_argument("--dcgan-fused", action="store_true", help="batch normalisation and the function layer after it as one fused layer (comparison aid)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="several ranks: sum the gradients with the library's own NVLink peer-memory kernels (default) or with NCCL")
    ap.add_argument("--dcgan-overlap", action="store_true", help="run the discriminator's exchange on a side stream beside the generator's backward pass (comparison aid)")
    ap.add_argument("--dcgan-eager", action="store_true", help="launch the DCGAN step eagerly instead of replaying its CUDA graph (profiling aid)")
    args = ap.parse_args()
    keep_stdout_clean()
    if args.warmup < 3 and args.impl == "b200":
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from cuda_cnn_gan_vae_b200 import ops
    from cuda_cnn_gan_vae_b200.lib import load

    lib = load()
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.hbm_only:
        emit(json.dumps(dict(hbm_kernels=hbm_kernels(torch, ops, measured_peaks()["hbm"], iters=2))))
        return
    if args.conv_layer:
        Cc, H, W, K, k, s_, p_, B = (int(v) for v in args.conv_layer.split(","))
        ops.set_precision(ops.TF32)
        oy, ox = (H - k + 2 * p_) // s_ + 1, (W - k + 2 * p_) // s_ + 1
        x, d = torch.randn(B, Cc, H, W, device="cuda"), torch.randn(B, K, oy, ox, device="cuda")
        wt, bias = torch.randn(1, 1, K, Cc * k * k, device="cuda") * (2.0 / (Cc * k * k)) ** 0.5, torch.zeros(1, K, 1, 1, device="cuda")
        y, dx, dk, db = torch.empty_like(d), torch.empty_like(x), torch.empty_like(wt), torch.empty_like(bias)
        layer = ops.ConvLayer(Cc, H, W, K, k, k, s_, s_, p_, p_, B)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(args.warmup + args.steps):
            if i == args.warmup:
                e0.record()
            layer.forward(y, x, wt, bias)
            layer.backward(dx, dk, db, d, x, wt, accumulate=False)
        e1.record()
        torch.cuda.synchronize()
        ops.stream_status()
        ms = e0.elapsed_time(e1) / max(1, args.steps)
        flops = 3 * 2.0 * B * K * Cc * k * k * oy * ox
        emit(json.dumps(dict(conv_layer=args.conv_layer, mode="tf32", ms_per_step=ms, value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s")))
        return
    c = dict(CFG, batch=args.batch)
    assert c["batch"] % world == 0, "global batch must divide over the ranks"
    B = c["batch"] // world
    Cc, H, W, K, k = c["C"], c["H"], c["W"], c["K"], c["k"]
    gen = torch.Generator(device="cuda").manual_seed(5 + rank)
    x = torch.randn(B, Cc, H, W, device="cuda", generator=gen)
    delta = torch.randn(B, K, H, W, device="cuda", generator=gen)
    wgen = torch.Generator(device="cuda").manual_seed(5)
    wt = torch.randn(1, 1, K, Cc * k * k, device="cuda", generator=wgen) * (2.0 / (Cc * k * k)) ** 0.5
    bias = torch.zeros(1, K, 1, 1, device="cuda")
    if world > 1:
        dist.broadcast(wt, 0)                       # weights replicated from rank 0 at start-up
    y = torch.empty(B, K, H, W, device="cuda")
    dx = torch.empty(B, Cc, H, W, device="cuda")
    from cuda_cnn_gan_vae_b200.dp import GradArena, PeerBuffer, arena_layout
    exchange_note = None
    if world > 1 and args.exchange == "peer":
        # the peer-memory exchange proves itself on this box before anything is timed with it: all ranks map one another's
        # memory and sum small integers; a rank that cannot sends every rank to NCCL, and the line says so
        probe = PeerBuffer(1 << 16, strict=False)
        why = probe.failed or probe.self_test()
        if not probe.failed:
            probe.close()
        if why:
            args.exchange = "nccl"
            exchange_note = "peer-memory exchange not usable on this box (%s): NCCL used instead" % why
    shapes = {"dW": (1, 1, K, Cc * k * k), "dB": (1, K, 1, 1)}
    peer = None
    if world > 1 and args.exchange == "peer":
        peer = PeerBuffer(arena_layout(shapes)[1])      # the arena lives in memory every rank maps: the library's kernel sums it over NVLink
    grads = GradArena(shapes, "cuda", peer.buffer[:arena_layout(shapes)[1]] if peer else None)   # contiguous dW | dB, summed as one buffer
    arena, dk, db = grads.buffer, grads.views["dW"], grads.views["dB"]

    def sum_over_ranks():
        if peer is not None:
            ops._check(lib.b200_allreduce(peer.comm, 0, arena.numel(), 0, ops._stream()))
        else:
            grads.all_reduce()
    step_flops = flops_per_sample(c) * c["batch"]

    layer = ops.ConvLayer(Cc, H, W, K, k, k, 1, 1, 1, 1, B)

    side = torch.cuda.Stream() if world > 1 else None

    def step():
        # the layer's Forward and TrainingBackward (netlayer/cnetlayerconvolution.cu.h:310,484): forward convolution, then the
        # batch-summed weight/bias gradient written into the arena and the backward-data convolution.  With several ranks
        # the gradients come first and their all-reduce runs on a side stream while the input error is computed (the
        # library packs the output error once for the two calls).
        layer.forward(y, x, wt, bias)
        if world > 1:
            layer.backward(None, dk, db, delta, x, wt, accumulate=False)
            main = torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                sum_over_ranks()
            layer.backward(dx, None, None, delta, x, wt)
            main.wait_stream(side)
        else:
            layer.backward(dx, dk, db, delta, x, wt, accumulate=False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, sample_clocks=False):
        for _ in range(warmup):
            fn()
        barrier()
        sampler = ClockSampler(local_rank) if sample_clocks else None
        lib.b200_profile_read(None, None)
        n0 = lib.b200_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        w1 = time.time()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        clocks = sampler.stop(w0, w1) if sampler else None
        launches = (lib.b200_launch_count() - n0) // steps
        kms, kn = C.c_double(0), C.c_int(0)
        lib.b200_profile_read(C.byref(kms), C.byref(kn))
        # tensor-core kernel time of one step (sum over its launches) and the launches it took
        return ms.item() / steps, clocks, launches, ((kms.value / steps, kn.value / steps) if kn.value else None)

    if args.vae_only:
        del x, delta, y, dx
        torch.cuda.empty_cache()
        emit(json.dumps(dict(vae=vae_bench(torch, ops, lib, timed, args.steps))))
        return
    peaks = measured_peaks()
    tf32_peak = peaks["bf16_sustained"] / 2.0
    results = {}
    sample_idx = [0, B // 3, B // 2, B - 1]
    samples = dict(idx=sample_idx, modes={})
    for mode_name, mode in (("tf32x3", ops.TF32X3), ("tf32", ops.TF32)):
        ops.set_precision(mode)
        lib.b200_profile_tensor_core(1)
        ms, clocks, launches, tc_time = timed(step, args.steps, args.warmup, sample_clocks=True)
        tc_ms_per_step, tc_launches = tc_time if tc_time else (None, None)
        kernel_ms = tc_ms_per_step / tc_launches if tc_time else None
        lib.b200_profile_tensor_core(0)
        ops.stream_status()
        if rank == 0 and world == 1 and not args.skip_cpu:
            samples["modes"][mode_name] = (y[sample_idx].cpu().numpy(), dx[sample_idx].cpu().numpy())
        # flops of an average launch: the three products of a step are equal; large layers run the forward and the
        # backward-data product as several launches (batch chunks pipelined against the pack), so the step's flops are
        # divided over the launches it actually took
        per_launch_flops = step_flops / world / (tc_launches or 3.0)
        # dram__bytes_read+write per tc_kernel launch from the committed ncu capture at batch 128, scaled by the units of a launch
        per_image, traffic_source = profiled_traffic()
        traffic = per_image * B * 3.0 / (tc_launches or 3.0) if per_image else None
        achieved = per_launch_flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms else None
        # the sustained peak was taken at a lower SM clock than this run holds under the same power cap: the fraction at
        # equal clock says how much of the tensor pipe the kernel uses, the plain fraction how fast it is
        run_mhz = (clocks or {}).get("sm_mhz")
        equal_clock = (achieved / tf32_peak * peaks["sm_mhz"] / run_mhz) if (achieved and run_mhz and peaks.get("sm_mhz")) else None
        results[mode_name] = dict(
            value=step_flops / (ms * 1e-3) / 1e12, ms_per_step=ms, clocks=clocks, gpu_launches=int(launches),
            roofline=dict(bound="tensor", achieved=achieved, peak=tf32_peak, unit="TFLOP/s",
                          frac=(achieved / tf32_peak) if achieved else None, traffic=traffic if mode == ops.TF32 else None,
                          traffic_source=traffic_source if mode == ops.TF32 else None,
                          frac_of_burst=(achieved / (peaks["bf16_burst"] / 2.0)) if (achieved and peaks.get("bf16_burst")) else None,
                          kernel="tc_kernel (tcgen05 implicit GEMM), mean over the forward, backward-data and weight-gradient launches of a step",
                          kernel_ms=kernel_ms, kernel_launches_per_step=tc_launches, kernel_ms_per_step=tc_ms_per_step, mma_per_product=3 if mode == ops.TF32X3 else 1,
                          peak_sm_mhz=peaks.get("sm_mhz"), frac_at_equal_clock=equal_clock,
                          tensor_pipe_frac=(achieved * (3 if mode == ops.TF32X3 else 1) / tf32_peak) if achieved else None,
                          peak_source=f"{peaks['source']}: bf16_tflops_sustained / 2 (kind::tf32 issues at half the bf16 rate), of measured"))

    # end to end through the C-ABI with host buffers (plain TF32 and 3xTF32 share the copies; measured in the headline mode)
    e2e = None
    if not args.skip_e2e:
        ops.set_precision(ops.TF32)
        hx = torch.empty(x.shape, pin_memory=True).copy_(x)
        hd = torch.empty(delta.shape, pin_memory=True).copy_(delta)
        hres = torch.empty(arena.shape, pin_memory=True)

        # The batch goes through in micro-batches: the host -> device copy of micro-batch i+1 (copy stream) runs while
        # micro-batch i is in the layer (forward, then backward accumulating dW|dB into the arena), so the step costs about
        # what the copies cost.  The public call sequence is the reference's gradient accumulation over mini-batches.
        chunks = 8 if B % 8 == 0 and B >= 64 else 1
        cb = B // chunks
        layer_mb = ops.ConvLayer(Cc, H, W, K, k, k, 1, 1, 1, 1, cb) if chunks > 1 else layer
        copy_stream = torch.cuda.Stream()
        arrived = [torch.cuda.Event() for _ in range(chunks)]

        def e2e_step():
            main = torch.cuda.current_stream()
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                for i in range(chunks):
                    sl = slice(i * cb, (i + 1) * cb)
                    x[sl].copy_(hx[sl], non_blocking=True)
                    delta[sl].copy_(hd[sl], non_blocking=True)
                    arrived[i].record(copy_stream)
            for i in range(chunks):
                sl = slice(i * cb, (i + 1) * cb)
                main.wait_event(arrived[i])
                layer_mb.forward(y[sl], x[sl], wt, bias)
                layer_mb.backward(dx[sl], dk, db, delta[sl], x[sl], wt, accumulate=(i > 0))
            sum_over_ranks()
            hres.copy_(arena, non_blocking=True)
            main.synchronize()

        ms, _, _, _ = timed(e2e_step, max(3, args.steps // 2), 2)
        e2e = dict(value=step_flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=ms,
                   h2d_bytes_per_step=int((hx.numel() + hd.numel()) * 4 * world), d2h_bytes_per_step=int(hres.numel() * 4 * world),
                   micro_batches=chunks,
                   note="image and delta copied from pinned host memory in micro-batches that overlap the layer calls, dW|dB read back, every step; plain-TF32 mode")
        ops.stream_status()

    # ---- DCGAN training step (generator + discriminator chains), 64 images per GPU -------------------------------
    dcgan = None
    if not args.skip_dcgan:
        from cuda_cnn_gan_vae_b200.nets import DCGANStep
        gb = args.dcgan_batch
        hz = torch.randn(gb, 1, 100, 1, generator=torch.Generator().manual_seed(11 + rank)).pin_memory()
        hl = (torch.rand(gb, 1, 1, 1, generator=torch.Generator().manual_seed(13 + rank)) < 0.5).float().pin_memory()
        z, labels = hz.cuda(), hl.cuda()
        hout = torch.empty(gb, 1, 1, 1).pin_memory()
        dcgan = dict(unit="img/s", per_gpu_batch=gb, global_batch=gb * world, scaling="weak",
                     step="G forward, D forward on the generated images, D backward + dW, G backward + dW, all-reduce of both "
                          "gradient arenas, Adam on both nets; LeakyReLU slope 0.2, per-element batch normalisation; the launches "
                          "up to the all-reduce are replayed from a CUDA graph captured after two eager steps")
        for mode_name, mode in (("tf32x3", ops.TF32X3), ("tf32", ops.TF32)):
            ops.set_precision(mode)
            trainer = DCGANStep(gb, world=world, use_graph=not args.dcgan_eager, fused=args.dcgan_fused,
                                update="fused" if args.exchange == "peer" else "nccl", overlap=args.dcgan_overlap)   # a graph is captured in the precision mode of its first steps
            dcgan["parameters"] = dict(generator=trainer.G.parameter_count, discriminator=trainer.D.parameter_count)
            n0 = lib.b200_launch_count()
            trainer(z, labels)                            # eager: every launch of the step is counted once
            per_step = lib.b200_launch_count() - n0

            def dcgan_step():
                trainer(z, labels)

            ms, clocks, _, _ = timed(dcgan_step, args.steps, max(args.warmup, 3), sample_clocks=True)
            ops.stream_status()
            dcgan[mode_name] = dict(value=gb * world / (ms * 1e-3), ms_per_step=ms, gpu_launches=int(per_step), clocks=clocks,
                                    cuda_graph=trainer.graph is not None)

        def dcgan_e2e_step():
            z.copy_(hz, non_blocking=True)
            labels.copy_(hl, non_blocking=True)
            hout.copy_(trainer(z, labels).view(gb, 1, 1, 1), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        ms, _, _, _ = timed(dcgan_e2e_step, args.steps, 2)
        ops.stream_status()
        dcgan["e2e"] = dict(value=gb * world / (ms * 1e-3), unit="img/s", ms_per_step=ms, h2d_bytes_per_step=int((hz.numel() + hl.numel()) * 4 * world),
                            d2h_bytes_per_step=int(hout.numel() * 4 * world), note="noise and labels from pinned host memory, discriminator outputs read back; plain-TF32 mode")
        dcgan["value"] = dcgan["tf32"]["value"]
        if world > 1 and gb % world == 0:
            # the same global batch of 64 images split over the ranks (strong scaling), for comparison with the weak-scaling figure
            ops.set_precision(ops.TF32)
            del trainer
            small = DCGANStep(gb // world, world=world, use_graph=not args.dcgan_eager, fused=args.dcgan_fused,
                              update="fused" if args.exchange == "peer" else "nccl", overlap=args.dcgan_overlap)
            zs, ls = z[:gb // world].contiguous(), labels[:gb // world].contiguous()
            ms, _, _, _ = timed(lambda: small(zs, ls), args.steps, max(args.warmup, 3))
            ops.stream_status()
            dcgan["strong_scaling"] = dict(global_batch=gb, per_gpu_batch=gb // world, value=gb / (ms * 1e-3), ms_per_step=ms, unit="img/s", mode="tf32")
            del small

    if samples["modes"]:
        samples.update(x=x[sample_idx].cpu().numpy(), d=delta[sample_idx].cpu().numpy(), w=wt.cpu().numpy()[0])
    cfg1 = vae = gemm = None
    if world == 1 and not args.skip_extra:
        x = delta = y = dx = None
        torch.cuda.empty_cache()
        cfg1 = cfg1_gpu(torch, ops)
        vae = vae_bench(torch, ops, lib, timed, args.steps)
        gemm = gemm_bench(torch, ops, peaks["hbm"])

    hbm = None
    if not args.skip_hbm and world == 1:
        x = delta = y = dx = None
        torch.cuda.empty_cache()
        hbm = hbm_kernels(torch, ops, peaks["hbm"])

    if rank == 0:
        head = results["tf32"]
        line = dict(metric=METRIC, value=head["value"], unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=head["ms_per_step"], higher_is_better=True, scaling="strong", vs_baseline=None, dtype="tf32",
                    data="synthetic",
                    config=dict(workload="dp_conv_sweep: batch %d of 256x32x32 N(0,1), 256 filters 3x3 s1 p1, fwd+bwd-data+wgrad%s"
                                % (c["batch"], " + sum of dW|dB over the ranks" if world > 1 else ""),
                                global_batch=c["batch"], per_gpu_batch=B, parallelism=f"dp{world}",
                                exchange=(("library kernels over NVLink peer memory (b200_allreduce, b200_allreduce_adam)" if args.exchange == "peer"
                                           else "NCCL all-reduce") if world > 1 else None), exchange_note=exchange_note, l2="inputs exceed L2 (1 GiB tensors)",
                                parity="tf32: 2e-3, tf32x3: 1e-4 on dot_rel_err vs the reference CPU backend (tests/test_gpu_full_size.py); measured on this run's batch when the CPU leg runs",
                                flops_per_step=step_flops),
                    clocks=head["clocks"], gpu_launches=head["gpu_launches"], roofline=head["roofline"], e2e=e2e,
                    tf32x3=results["tf32x3"], dcgan=dcgan, cfg1=cfg1, vae=vae, gemm=gemm, hbm_kernels=hbm)
        if not args.skip_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline()
            if samples["modes"]:
                line["config"]["parity"] = parity_leg(samples)
            if dcgan is not None:
                dcgan["cpu_baseline"] = dcgan_cpu_baseline()
            if cfg1 is not None:
                cfg1["cpu_baseline"] = cfg1_cpu()
                cfg1["vs_cpu_baseline_same_config"] = dict(device_ratio=cfg1["tf32"]["value"] / cfg1["cpu_baseline"]["value"],
                                                           e2e_ratio=cfg1["e2e"]["value"] / cfg1["cpu_baseline"]["value"])
            if vae is not None:
                vae["cpu_baseline"] = vae_cpu_baseline()
        emit(json.dumps(line))
    if world > 1:
        # Leave without tearing the process group down: destroying NCCL communicators while CUDA graphs that hold
        # captured collectives are alive can block for minutes; every rank has finished its work at this barrier.
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
