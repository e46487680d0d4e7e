#!/usr/bin/env python
"""Benchmark of the Winograd / DWM forward-convolution path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload vgg16|cfg2]

Workload (default): BASELINE config 5 -- the 13-convolution VGG-16 stack (3x3/s1/p1, ReLU, five
2x2 max-pools), fp16, input 3x224x224 ~ U(0,1), Kaiming-normal weights, a global batch of 256 images
cut into contiguous shards over the N ranks (256 / 128 / 64 / 32 per GPU at N = 1 / 2 / 4 / 8: strong
scaling, as the configuration is stated; `--scaling weak` gives every rank 256 images instead).
Synthetic data, random weights; every rank holds its own shard, no collective on the data path.
A step is one pass of the stack over the rank's shard.  One JSON line is printed by rank 0:

  value      images/s of the whole job with the batch resident in HBM (CUDA-graph replay of the stack,
             CUDA events, max over ranks)
  e2e        the same through the public API from pinned host memory: H2D copy of the batch, the
             stack, D2H copy of the result, every step
  layers     per-layer device time, effective direct-conv TFLOP/s and two roofline fractions,
             t_roof / t with t_roof = max(F_gemm / TC_peak, B_alg / HBM_peak): `roof_frac` takes F_gemm of
             the algorithm that ran, `roof_frac_contract` the multiply-adds of the algorithm the configuration
             names (F(4x4,3x3) for 2-D 3x3 stride-1 layers, the DWM piece table at m = 2 otherwise) -- the
             second cannot be raised by switching to a more wasteful decomposition
  roofline   the kernel class with the largest share of device time, measured with CUDA events around
             every launch of an instrumented pass (winoconv_forward_timed); `frac` and `frac_contract` as above
  errors     per layer, on a two-image sample: E_B / E_A / E_C and the 99.9th percentile of the engine against
             the float64 direct convolution of the layer's own input, beside the same figures for the
             reference's tile algebra evaluated on the CPU on the same tensors
  cpu_baseline  the reference's torch-level Winograd algebra (oracle restatement) timed on this host's
             cores on a bounded sample of the same workload

`--impl reference` times that CPU restatement alone (the reference's own Python modules need the
reference checkout, which does not travel to the GPU box, and its CUDA path has no 2-D 3x3 entry).
With N > 1 this file is launched by torchrun (one rank per GPU); run directly with --gpus N it
re-launches itself that way.
"""
import argparse
import json
import math
import os
import socket
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu capture
# kept with the profile summaries (None until a capture exists for that kernel and workload).
NCU_TRAFFIC_PER_IMAGE = {
    # rowfused_kernel, C = K = 256 at 56 x 56 (VGG layers 6-7): 169.1 MB for 64 images in the capture kept in
    # profiles/rowfused_pair_c256_k256_56_ncu.md; traffic grows in proportion to the images of a launch
    # (algorithmic bytes of that layer: 3.2 MB per image; part of y is still dirty in L2 when the kernel ends)
    ("vgg16", "rowfused_kernel"): (169.1e6 / 64, "ncu capture of the 256->256 56x56 layer at 64 images, scaled by images per launch"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg16", choices=["vgg16", "cfg1", "cfg2", "cfg3a", "cfg3b", "cfg4", "conv", "gemm", "mma-rate"],
                    help="vgg16 = BASELINE configs[4] (the headline); cfg1..cfg4 = the single-layer configs[0..3]; conv = --shape; "
                         "gemm = the per-position batched GEMM of cfg1 / cfg2 / cfg3b / cfg4 beside torch.bmm (cuBLAS) on the same box; "
                         "mma-rate = clocks per tcgen05.mma by accumulator width, issuing threads and operand placement")
    ap.add_argument("--shape", default="256,256,56,3", help="--workload conv: C,K,HW,kernel (stride 1, 'same' padding, fp16)")
    ap.add_argument("--batch", type=int, default=0, help="global batch (default: what the configuration names: 256 for vgg16)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the global batch is cut into shards over the ranks (the stated configuration); "
                         "weak: every rank gets the whole batch")
    ap.add_argument("--clock-csv", default="", help="write the clock samples of this rank to this file")
    ap.add_argument("--skip-errors", action="store_true", help="skip the per-layer error columns (CPU work on rank 0)")
    ap.add_argument("--algo", default="auto", choices=["auto", "row", "fused", "staged"],
                    help="fused: one tcgen05 kernel per layer, F(2x2,3x3); staged: three kernels per pass, F(4x4,3x3)")
    ap.add_argument("--product", default="f32", choices=["f32", "f16"], help="dtype of the staged algorithm's products M")
    ap.add_argument("--engine", default="auto", choices=["auto", "simt", "tcgen05", "tf32", "tf32x3"],
                    help="GEMM engine of the staged algorithm (single-layer workloads)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the cpu_baseline sample")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------
# clocks: sample nvidia-smi while the timed regions run
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, sampled while the timed regions run.

    Reads NVML from a thread of this process every few milliseconds (the timed regions of the default run
    last ~0.1 s, shorter than nvidia-smi's start-up); falls back to an `nvidia-smi -lms` child when the NVML
    module is missing.  Only samples taken inside a `with sampler.window():` block enter the summary.
    Reading only: no clock, power or mode setting is touched.
    """
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index, csv_path=""):
        self.gpu = gpu_index
        self.csv_path = csv_path          # where the caller wants the samples kept (optional)
        self.proc = None
        self.thread = None
        self.samples = []        # (t, sm_mhz, power_w, reason bitmask)
        self.windows = []        # (t0, t1)
        self.sm_max = None
        self._stop = False

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def start(self):
        try:
            pynvml, h = self._nvml_handle()
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop:
                    try:
                        sm = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                        rs = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                        self.samples.append((time.perf_counter(), sm, pw, rs))
                    except Exception:
                        pass
                    time.sleep(0.003)

            import threading
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            import tempfile
            self.fh = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.gpu)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    class _Window:
        def __init__(self, owner):
            self.owner = owner

        def __enter__(self):
            self.t0 = time.perf_counter()

        def __exit__(self, *exc):
            self.owner.windows.append((self.t0, time.perf_counter()))
            return False

    def window(self):
        return ClockSampler._Window(self)

    def stop(self):
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            inside = [s for s in self.samples if any(t0 <= s[0] <= t1 for t0, t1 in self.windows)]
            used = inside if inside else self.samples
            if self.csv_path:
                try:
                    with open(self.csv_path, "w") as fh:
                        fh.write("t_s,sm_mhz,power_w,reasons_mask,in_timed_region\n")
                        for smp in self.samples:
                            fh.write("%.6f,%.0f,%.1f,0x%x,%d\n" % (smp[0], smp[1], smp[2], smp[3], int(smp in inside)))
                except Exception:
                    pass
            if not used:
                return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"]}
            mask = 0
            for smp in used:
                mask |= smp[3]
            reasons = sorted(n for n, bit in self.REASON_BITS.items() if mask & bit)
            return {"sm_mhz": statistics.median(s[1] for s in used), "sm_max_mhz": self.sm_max, "reasons": reasons,
                    "power_w_max": max(s[2] for s in used), "samples": len(used),
                    "sampled": "NVML every ~3 ms inside the timed regions" if inside else "NVML, whole run"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = open(self.fh.name).readlines()
        if self.csv_path:
            try:
                with open(self.csv_path, "w") as fh:
                    fh.writelines(lines)
            except Exception:
                pass
        os.unlink(self.fh.name)
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm), "sampled": "nvidia-smi -lms 25, whole run"}


# ---------------------------------------------------------------------------------------------------
# the CPU arm (cpu_baseline and --impl reference)
# ---------------------------------------------------------------------------------------------------
def vgg_weights(dtype, seed=100):
    from oracle import winograd_oracle as wo
    return [wo.kaiming_normal((k, c, 3, 3), seed + i).to(dtype) for i, (c, k) in enumerate(wo.VGG16_CHANNELS)]


def cpu_vgg_images_per_s(seconds_budget, chunk=2):
    """Reference-style fp32 F(2x2,3x3) Winograd on the host cores over a bounded sample of the workload."""
    import torch
    from oracle import winograd_oracle as wo
    torch.set_num_threads(os.cpu_count() or 1)
    ws = vgg_weights(torch.float32)
    g = torch.Generator().manual_seed(0)
    x = torch.rand(chunk, 3, 224, 224, generator=g)
    wo.vgg16_winograd_cpu(x[:1], ws)                     # warm-up (thread pools, allocator)
    images, t0 = 0, time.perf_counter()
    while True:
        wo.vgg16_winograd_cpu(x, ws)
        images += chunk
        el = time.perf_counter() - t0
        if el >= seconds_budget or images >= 256:
            break
    return images / el, images, el, torch.get_num_threads()


def cpu_cfg2_layers_per_s(seconds_budget):
    import torch
    from oracle import winograd_oracle as wo
    torch.set_num_threads(os.cpu_count() or 1)
    x = torch.randn(32, 256, 28, 28, generator=torch.Generator().manual_seed(0))
    w = wo.kaiming_normal((256, 256, 3, 3), 1)
    wo.winograd_conv_cpu(x[:2], w, padding=1)
    n, t0 = 0, time.perf_counter()
    while True:
        wo.winograd_conv_cpu(x, w, padding=1, tile_m=2)
        n += 1
        el = time.perf_counter() - t0
        if el >= seconds_budget:
            break
    return n / el, n, el, torch.get_num_threads()


def run_reference(args):
    """The reference arm: its torch-level Winograd path (CPU restatement) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import winograd_oracle as wo
    torch.set_num_threads(os.cpu_count() or 1)
    chunk = 2
    if args.workload == "vgg16":
        ws = vgg_weights(torch.float32)
        x = torch.rand(chunk, 3, 224, 224, generator=torch.Generator().manual_seed(0))
        step = lambda: wo.vgg16_winograd_cpu(x, ws)
        units, metric, unit = chunk, "vgg16_conv_images_per_s", "images/s"
        workload = "vgg16_conv_stack_3x224x224 (BASELINE configs[4])"
        sample = f"{chunk} images per step, fp32 F(2x2,3x3), CPU"
    else:
        x = torch.randn(32, 256, 28, 28, generator=torch.Generator().manual_seed(0))
        w = wo.kaiming_normal((256, 256, 3, 3), 1)
        step = lambda: wo.winograd_conv_cpu(x, w, padding=1, tile_m=2)
        units, metric, unit = 32, "conv_images_per_s", "images/s"
        workload = "conv3x3_n32_c256_k256_28x28 (BASELINE configs[1])"
        sample = "the full layer per step, fp32 F(2x2,3x3), CPU"
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    el = time.perf_counter() - t0
    value = units * args.steps / el
    cores = torch.get_num_threads()
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * el / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "device": "host CPU", "sample": sample},
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------
def relaunch_under_torchrun(args):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
    sys.exit(subprocess.call(cmd))


ALGO_NAMES = {0: "auto", 1: "staged", 2: "fused", 3: "row"}


def describe_algorithms(layers):
    """What ran, from the plans themselves (never from the command line)."""
    from pytorch_winoconv_b200 import capi
    text = {
        capi.ALGO_ROW: "DWM 1x3 row pieces, F(2,3) along W, one fused tcgen05 kernel per layer",
        capi.ALGO_FUSED: "F(2x2,3x3) fused: gather + transforms + tcgen05 GEMM in one kernel per layer",
    }
    out = []
    for c in layers:
        a = int(c.info.algo)
        if a in text:
            d = text[a]
        else:
            m = max(int(v) for v in c.info.tile_m)
            eng = {capi.GEMM_TCGEN05: "tcgen05 GEMM", capi.GEMM_TF32: "tcgen05 tf32 GEMM",
                   capi.GEMM_TF32X3: "tcgen05 GEMM, three tf32 products of a hi / lo split per multiply"}.get(
                       int(c.info.gemm_engine), "fp32 FMA GEMM")
            d = (f"F({m}x{m},3x3)" if int(c.info.n_pieces) == 1 and c.ndim == 2 else f"DWM pieces of F({m},r)") + \
                f" staged: input transform, {eng}, output transform; products fp32"
        if d not in out:
            out.append(d)
    return "; ".join(out)


def layer_errors(args, layers, x_host, dev):
    """Per layer, on the first two images: the engine against the float64 direct convolution of the layer's own
    input, and the reference's tile algebra (CPU; every intermediate rounded to half for 16-bit layers, the way
    its conv16 does) against the same oracle on the same tensors.  The reference algebra runs at the tile the
    configuration names (F(4x4,3x3) is fed the matrices its own generator gives for (0, +-1, +-2))."""
    import torch
    import torch.nn.functional as F
    from oracle import winograd_oracle as wo
    from pytorch_winoconv_b200 import capi, engine
    n_s = min(2, int(x_host.shape[0]))
    h = x_host[:n_s].to(dev)
    rows = []
    for li, big in enumerate(layers):
        nd = big.ndim
        epi = int(big.desc.epilogue)
        relu, pool = bool(epi & capi.EPI_RELU), bool(epi & capi.EPI_POOL2)
        stride, pad = tuple(big.desc.stride)[3 - nd:], tuple(big.desc.pad)[3 - nd:]
        w = big._w_keepalive
        conv = engine.WinoConv((n_s,) + tuple(big.in_shape[1:]), w, stride=stride, padding=pad,
                               tile_m=max(int(v) for v in big.info.tile_m) if int(big.info.algo) == capi.ALGO_STAGED else 2,
                               bias=big.bias, relu=relu, pool2=pool, algo=int(big.info.algo))
        y = conv(h)
        torch.cuda.synchronize(dev)
        to_nchw = (0, nd + 1) + tuple(range(1, nd + 1))
        hin, wc = h.permute(*to_nchw).cpu(), w.cpu()

        def finish(t):
            t = torch.relu(t) if relu else t
            return F.max_pool2d(t, 2) if pool else t

        o = finish(wo.direct_conv_f64(hin, wc, stride=stride, padding=pad))
        ks = tuple(wc.shape[2:])
        f43 = nd == 2 and ks == (3, 3) and tuple(stride) == (1, 1) and args.workload != "cfg1"
        half = h.dtype != torch.float32
        ref = finish(wo.winograd_conv_cpu(hin, wc, stride=list(stride), padding=list(pad), tile_m=4 if f43 else 2,
                                          fp16=half).double())
        e = wo.error_metrics(y.permute(*to_nchw).cpu(), o, percentile=True)
        r = wo.error_metrics(ref, o, percentile=True)
        rows.append({"layer": li + 1, "engine": {k: float("%.3g" % v) for k, v in e.items()},
                     "reference_algebra": {k: float("%.3g" % v) for k, v in r.items()},
                     "reference_tile": "F(4x4,3x3)" if f43 else "F(2,r) pieces", "images": n_s})
        h = y
    return {"metric": "E_B = max |y-o| / max(|o|, rms o); E_A = max|d| / max|o|; E_C = mean |d|/|o|; P999 of the E_B ratio; "
                      "o = float64 direct convolution of the layer's input",
            "tolerance_E_B": 1e-3 if x_host.dtype == torch.float32 else 2e-2, "layers": rows}


def run_gemm_compare(args):
    """winoconv_gemm_batched beside torch.bmm (the library GEMM the reference calls through cublas{S,H}gemmBatched,
    src/base_conv_launchers.cu:362-367) on the [positions, tiles, C] x [positions, C, K] shapes of the staged path.
    A side measurement: one JSON line, no contract keys."""
    import torch
    from pytorch_winoconv_b200 import capi, engine
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    capi.check(capi.lib().winoconv_device_check(), "winoconv_device_check")
    shapes = [("cfg1 F(2x2,3x3) fp32", 16, 6272, 64, 64, torch.float32),
              ("cfg2 F(4x4,3x3) fp16", 36, 1568, 256, 256, torch.float16),
              ("cfg3b 5x5 pieces fp16", 49, 25088, 128, 128, torch.float16),
              ("cfg4 F(2,3)^3 fp16", 64, 50176, 64, 64, torch.float16)]
    rows = []
    for name, pos, tiles, c, k, dt in shapes:
        g = torch.Generator().manual_seed(0)
        v = torch.randn(pos, tiles, c, generator=g).to(dt).to(dev)
        u = (torch.randn(pos, k, c, generator=g) / c ** 0.5).to(dt).to(dev)
        m = torch.empty(pos, tiles, k, dtype=torch.float32, device=dev)
        ut = u.transpose(1, 2).contiguous()
        stream = torch.cuda.current_stream(dev).cuda_stream
        engines = ([("fp32 fma", capi.GEMM_SIMT), ("tf32", capi.GEMM_TF32), ("tf32 x3", capi.GEMM_TF32X3)]
                   if dt == torch.float32 else [("tcgen05 f16, fp32 products", capi.GEMM_TCGEN05)])
        calls = [(n, (lambda e=e: capi.gemm_batched(engine.dtype_code(dt), capi.F32, e, pos, tiles, c, k, v.data_ptr(),
                                                    u.data_ptr(), m.data_ptr(), stream))) for n, e in engines]
        if dt != torch.float32:      # what cuBLAS writes here: products rounded to the input dtype
            m16 = torch.empty(pos, tiles, k, dtype=dt, device=dev)
            calls.append(("tcgen05 f16, f16 products", lambda: capi.gemm_batched(engine.dtype_code(dt), engine.dtype_code(dt),
                                                                                  capi.GEMM_TCGEN05, pos, tiles, c, k, v.data_ptr(),
                                                                                  u.data_ptr(), m16.data_ptr(), stream)))
        calls.append(("torch.bmm (cuBLAS), out in the input dtype", lambda: torch.bmm(v, ut)))
        if dt == torch.float32:
            def bmm_tf32():
                torch.backends.cuda.matmul.allow_tf32 = True
                torch.bmm(v, ut)
                torch.backends.cuda.matmul.allow_tf32 = False
            calls.append(("torch.bmm (cuBLAS), tf32 allowed", bmm_tf32))
        flops = 2.0 * pos * tiles * c * k
        res = {}
        for n, fn in calls:
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize(dev)
            us = 1e3 * e0.elapsed_time(e1) / args.steps
            res[n] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1)}
        rows.append({"shape": name, "positions": pos, "tiles": tiles, "c": c, "k": k, "engines": res})
    print(json.dumps({"workload": "gemm", "steps": args.steps, "note": "eager launches, CUDA events; m in fp32 for the engine", "rows": rows}), flush=True)


def run_mma_rate(args):
    """The calibration probe behind the planner's accumulator width: clocks per tcgen05.mma (M = 128 per SM, K = 16)."""
    import torch
    from pytorch_winoconv_b200 import capi
    torch.cuda.set_device(0)
    rows = []
    for pair in (False, True):
        for a_tmem in (False, True):
            for thr in (1, 2, 4):
                for n in (16, 32, 64, 128, 256):
                    try:
                        total, issue = capi.probe_mma_rate(pair, a_tmem, n, thr, 512)
                    except capi.WinoconvError as exc:
                        if exc.status == capi.ERR_UNSUPPORTED:      # the accumulators of that many threads do not fit
                            continue
                        raise
                    rows.append({"cta_pair": pair, "a_operand": "tmem" if a_tmem else "smem", "threads": thr, "n": n,
                                 "clocks_per_mma": round(total, 1), "issue_clocks_per_mma_one_thread": round(issue, 1),
                                 "ideal_clocks": n / 2})
    print(json.dumps({"workload": "mma-rate", "m_rows_per_sm": 128, "k": 16, "rows": rows}), flush=True)


def run_ours(args):
    if args.workload == "gemm":
        return run_gemm_compare(args)
    if args.workload == "mma-rate":
        return run_mma_rate(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        relaunch_under_torchrun(args)
    import torch
    import torch.distributed as dist
    from pytorch_winoconv_b200 import capi, engine, sharding

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a B200: the engine has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    capi.check(capi.lib().winoconv_device_check(), "winoconv_device_check")
    peaks, peaks_kind = load_peaks()

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()

    # ---- build the workload ------------------------------------------------------------------
    g = torch.Generator().manual_seed(1234 + rank)

    def shard_of(global_batch):
        """This rank's share of the global batch: a contiguous shard (strong scaling) or all of it (weak)."""
        if args.scaling == "weak" or world == 1:
            return global_batch
        lo, hi = sharding.shard_bounds(global_batch, world, rank)
        if hi <= lo:
            raise RuntimeError(f"global batch {global_batch} leaves rank {rank} of {world} without an image")
        return hi - lo

    if args.workload == "vgg16":
        global_batch = args.batch or 256
        batch = shard_of(global_batch)
        ws = [w.to(dev) for w in vgg_weights(torch.float16)]
        fused = args.algo in ("row", "fused")
        algo_code = {"auto": capi.ALGO_AUTO, "row": capi.ALGO_ROW, "fused": capi.ALGO_FUSED, "staged": capi.ALGO_STAGED}[args.algo]
        # auto: the library's own choice per layer (tile_m = 0)
        model = engine.VGG16ConvStack(ws, batch, tile_m=0 if args.algo == "auto" else (2 if fused else 4), algo=algo_code,
                                      product_dtype=torch.float16 if (args.product == "f16" and not fused) else None)
        x_host = torch.rand(batch, 224, 224, 3, generator=g).half().pin_memory()
        layers = model.layers
        workload = "vgg16_conv_stack_3x224x224 (BASELINE configs[4])"
        metric = "vgg16_conv_images_per_s"
    else:
        from oracle import winograd_oracle as wo   # Kaiming-normal helper only; nothing timed runs in the oracle
        # single-layer workloads: BASELINE configs[0..3] by name, or --shape
        named = {
            #        batch, C,   K,   spatial,        kernel,    stride, pad, dtype,         tile_m, input
            "cfg1":  (8,   64,  64,  (56, 56),       (3, 3),    1,      1,   torch.float32, 2,      "normal"),
            "cfg2":  (32,  256, 256, (28, 28),       (3, 3),    1,      1,   torch.float16, 4,      "normal"),
            "cfg3a": (64,  3,   64,  (224, 224),     (7, 7),    2,      3,   torch.float16, 2,      "uniform"),
            "cfg3b": (32,  128, 128, (56, 56),       (5, 5),    1,      2,   torch.float16, 2,      "normal"),
            "cfg4":  (8,   64,  64,  (16, 56, 56),   (3, 3, 3), 1,      1,   torch.float16, 2,      "normal"),
        }
        if args.workload in named:
            nb, cc, kk, sp, ks, stride, pad, dt, tm, dist_kind = named[args.workload]
            global_batch = args.batch or nb
            batch = shard_of(global_batch)
        else:
            cc, kk, hw_, ksz_ = tuple(int(v) for v in args.shape.split(","))
            sp, ks, stride, pad, dt, tm, dist_kind = (hw_, hw_), (ksz_, ksz_), 1, ksz_ // 2, torch.float16, (4 if ksz_ == 3 else 2), "normal"
            global_batch = args.batch or 32
            batch = shard_of(global_batch)
        hw = sp[-1]
        ksz = ks[-1]
        w = wo.kaiming_normal((kk, cc) + tuple(ks), 1).to(dt).to(dev)
        fused = args.algo in ("fused", "row")
        # auto: the algorithm the config names (cfg2: staged F(4x4,3x3)); otherwise what the engine picks for 2-wide tiles
        if args.algo == "auto":
            algo_code = capi.ALGO_STAGED if (tm == 4 or dt == torch.float32) else capi.ALGO_AUTO
        else:
            algo_code = {"row": capi.ALGO_ROW, "fused": capi.ALGO_FUSED, "staged": capi.ALGO_STAGED}[args.algo]
        conv = engine.WinoConv((batch,) + tuple(sp) + (cc,), w, stride=stride, padding=pad,
                               tile_m=2 if (fused or tm == 2) else 4, algo=algo_code,
                               gemm_engine={"auto": capi.GEMM_AUTO, "simt": capi.GEMM_SIMT, "tcgen05": capi.GEMM_TCGEN05,
                                            "tf32": capi.GEMM_TF32, "tf32x3": capi.GEMM_TF32X3}[args.engine],
                               product_dtype=torch.float16 if (args.product == "f16" and not fused and dt == torch.float16) else None)
        out_buf = torch.empty(conv.out_shape, dtype=dt, device=dev)

        class _Single:
            layers = [conv]
            out_shape = conv.out_shape
            launches_per_call = conv.launches_per_call
            direct_flops = conv.info.direct_flops
            _graph = None

            def forward(self, x):
                return conv(x, out=out_buf)

            __call__ = forward
            capture = engine.VGG16ConvStack.capture
            replay = engine.VGG16ConvStack.replay
            acts = [out_buf]

        model = _Single()
        x_host = (torch.rand if dist_kind == "uniform" else torch.randn)((batch,) + tuple(sp) + (cc,), generator=g).to(dt).pin_memory()
        layers = model.layers
        names = {"cfg1": "conv3x3_n8_c64_k64_56x56_fp32_f23 (BASELINE configs[0])",
                 "cfg2": "conv3x3_n32_c256_k256_28x28_f43 (BASELINE configs[1])",
                 "cfg3a": "conv7x7_s2_n64_c3_k64_224x224_dwm (BASELINE configs[2]a)",
                 "cfg3b": "conv5x5_n32_c128_k128_56x56_dwm (BASELINE configs[2]b)",
                 "cfg4": "conv3x3x3_n8_c64_k64_16x56x56 (BASELINE configs[3])"}
        workload = names.get(args.workload, f"conv{ksz}x{ksz}_n{global_batch}_c{cc}_k{kk}_{hw}x{hw}")
        metric = "conv_images_per_s"
    x_dev = x_host.to(dev, non_blocking=True)
    io_dtype = x_host.dtype
    y_host = torch.empty(model.out_shape, dtype=io_dtype).pin_memory()
    y_probe = torch.empty(model.out_shape, dtype=io_dtype, device=dev)
    torch.cuda.synchronize(dev)

    use_graph = not args.no_graph
    if use_graph:
        model.capture(x_dev)
        step = lambda: model.replay()
    else:
        step = lambda: model(x_dev)

    sampler = ClockSampler(local_rank, args.clock_csv)
    sampler.start()

    # ---- region 1: inputs resident in HBM ---------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler.window():
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    ms_local = e0.elapsed_time(e1)
    ms = sharding.max_over_ranks(ms_local)
    total_images = sharding.sum_over_ranks(batch)
    value = total_images * args.steps / (ms / 1e3)

    # ---- region 2: end to end from pinned host memory ---------------------------------------------
    # Every step copies its batch host -> device and its result device -> host.  The copies run on their own
    # streams: H2D into two alternating input buffers, so the copy of step i+1 overlaps the kernels of step i; the
    # result is moved to one of two staging buffers (device to device) and read back from there while the next
    # step computes.  All copies of the K timed steps lie between the two events.
    main = torch.cuda.current_stream(dev)
    copy_stream = torch.cuda.Stream(device=dev)
    d2h_stream = torch.cuda.Stream(device=dev)
    x_bufs = [x_dev, torch.empty_like(x_dev)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    y_stage = [torch.empty_like(y_probe), torch.empty_like(y_probe)]
    staged = [torch.cuda.Event() for _ in range(2)]
    read_back = [torch.cuda.Event() for _ in range(2)]

    def issue_copy(i):
        b = i % 2
        copy_stream.wait_event(consumed[b])
        with torch.cuda.stream(copy_stream):
            x_bufs[b].copy_(x_host, non_blocking=True)
            copied[b].record(copy_stream)

    def run_e2e(n_steps):
        for b in range(2):
            consumed[b].record(main)
            read_back[b].record(main)
        copy_stream.wait_stream(main)
        d2h_stream.wait_stream(main)
        issue_copy(0)
        for i in range(n_steps):
            b = i % 2
            if i + 1 < n_steps:
                issue_copy(i + 1)
            main.wait_event(copied[b])
            y = model.forward(x_bufs[b])
            consumed[b].record(main)
            main.wait_event(read_back[b])          # the staging buffer's previous read-back has finished
            y_stage[b].copy_(y, non_blocking=True)
            staged[b].record(main)
            d2h_stream.wait_event(staged[b])
            with torch.cuda.stream(d2h_stream):
                y_host.copy_(y_stage[b], non_blocking=True)
                read_back[b].record(d2h_stream)
        main.wait_stream(copy_stream)
        main.wait_stream(d2h_stream)

    run_e2e(3)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler.window():
        f0.record()
        run_e2e(args.steps)
        f1.record()
        barrier()
    ms_e2e = sharding.max_over_ranks(f0.elapsed_time(f1))
    e2e_value = total_images * args.steps / (ms_e2e / 1e3)
    clocks = sampler.stop()

    # ---- region 3: the same steps with every layer's filter transform inside (what a caller pays who hands over
    # fresh weights on every call, as the reference's operators do; device-resident inputs, eager launches)
    def step_with_filter_transform():
        for conv in layers:
            conv.set_weight(conv._w_keepalive)
        return model.forward(x_dev)

    for _ in range(2):
        step_with_filter_transform()
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0.record()
    for _ in range(args.steps):
        step_with_filter_transform()
    h1.record()
    barrier()
    ms_wft = sharding.max_over_ranks(h0.elapsed_time(h1))

    # ---- instrumented pass: CUDA events around every launch ---------------------------------------
    # Two roofline numerators per layer: the multiply-adds of the algorithm that ran (`roof_frac`), and those of the
    # algorithm the configuration names (`roof_frac_contract`): F(4x4,3x3) for a 2-D 3x3 stride-1 layer (F(2x2,3x3)
    # for configs[0], which names it), the DWM piece table at m = 2 otherwise -- both 2 * positions * tiles * C * K --
    # with the same compulsory bytes x + w + y.
    def contract_info(conv):
        d = capi.Desc.from_buffer_copy(bytes(conv.desc))
        ks, st = tuple(d.ker_size), tuple(d.stride)
        f43 = conv.ndim == 2 and ks[1:] == (3, 3) and st[1:] == (1, 1) and args.workload != "cfg1"
        d.algo, d.tile_m, d.gemm_engine, d.product_dtype = capi.ALGO_STAGED, (4 if f43 else 2), capi.GEMM_AUTO, capi.F32
        return capi.plan(d), ("F(4x4,3x3)" if f43 else "DWM pieces, m = 2")

    reps = 3
    stage_names = ["input_transform", "gemm", "output_transform"]
    per_layer = []
    single_layer = args.workload != "vgg16"
    esz_io = x_host.element_size()
    # a kernel timed alone is held against the burst figure, one inside a long step against the sustained one;
    # fp32 layers run their products as fp32 FMA: nominal 75 TFLOP/s
    tc_peak_16 = peaks["bf16_tflops"] if single_layer else peaks["bf16_tflops_sustained"]

    def product_peak(conv):
        """TFLOP/s the layer's multiply-adds can be held against: the 16-bit tensor peak; for fp32 inputs half of it
        per tf32 product (a third of that when every multiply-add is three products of a hi / lo split), or the
        nominal 75 TFLOP/s of fp32 FMA for the FMA kernel."""
        if io_dtype != torch.float32:
            return tc_peak_16, "tensor"
        eng = int(conv.info.gemm_engine)
        if eng == capi.GEMM_TF32:
            return tc_peak_16 / 2, "tensor (tf32)"
        if eng == capi.GEMM_TF32X3:
            return tc_peak_16 / 6, "tensor (3 x tf32)"
        return 75.0, "fp32-fma"
    h = x_dev
    for li, conv in enumerate(layers):
        acc = [0.0, 0.0, 0.0]
        n_launch = 0
        conv.timed(h)                                    # warm
        for _ in range(reps):
            out, st, n_launch = conv.timed(h)
            acc = [a + s_ for a, s_ in zip(acc, st)]
        st = [a / reps for a in acc]
        info = conv.info
        cinfo, cname = contract_info(conv)
        t_ms = sum(st)
        mma_peak, mma_bound = product_peak(conv)
        t_tc = info.gemm_flops / (mma_peak * 1e12) * 1e3
        t_hbm = info.algorithmic_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        t_tc_c = cinfo.gemm_flops / (mma_peak * 1e12) * 1e3
        # the configuration's compulsory bytes count the convolution's own output (before a fused pool), as its table does
        b_contract = float(esz_io) * (math.prod(conv.in_shape) + conv._w_keepalive.numel()
                                      + conv.in_shape[0] * int(conv.desc.k_out) * math.prod(int(v) for v in info.conv_out_size))
        t_hbm_c = b_contract / (peaks["hbm_gbs"] * 1e9) * 1e3
        per_layer.append({"layer": li + 1, "c": int(conv.desc.c_in), "k": int(conv.desc.k_out),
                          "hw": int(conv.in_shape[-2]), "ms": round(t_ms, 4), "stage_ms": [round(v, 4) for v in st],
                          "launches": n_launch, "algo": ALGO_NAMES[int(info.algo)],
                          "eff_tflops": round(info.direct_flops / (t_ms * 1e-3) / 1e12, 2),
                          "gemm_tflops": round(info.gemm_flops / (st[1] * 1e-3) / 1e12, 2),
                          "roof_ms": round(max(t_tc, t_hbm), 4), "roof_bound": mma_bound if t_tc >= t_hbm else "hbm",
                          "roof_frac": round(max(t_tc, t_hbm) / t_ms, 4),
                          "contract": cname, "roof_ms_contract": round(max(t_tc_c, t_hbm_c), 5),
                          "roof_bound_contract": "tensor" if t_tc_c >= t_hbm_c else "hbm",
                          "roof_frac_contract": round(max(t_tc_c, t_hbm_c) / t_ms, 4)})
        h = out
    stage_tot = [sum(l["stage_ms"][i] for l in per_layer) for i in range(3)]
    # Time per kernel class over the step (a stack may mix algorithms: AUTO takes staged F(4x4,3x3) for some layers and
    # the row-piece kernel for the rest): the dominant class is the one the roofline object describes.
    esz = x_host.element_size()
    classes = {}      # kernel -> [ms, launches, algorithmic flops, algorithmic bytes]

    def add(kernel, ms, flops=0.0, nbytes=0.0, launches=1):
        c = classes.setdefault(kernel, [0.0, 0, 0.0, 0.0])
        c[0] += ms; c[1] += launches; c[2] += flops; c[3] += nbytes

    for l, conv in zip(per_layer, layers):
        a = int(conv.info.algo)
        if a == capi.ALGO_ROW:
            add("rowfused_kernel", l["stage_ms"][1], flops=conv.info.gemm_flops)
        elif a == capi.ALGO_FUSED:
            add("fused23_kernel", l["stage_ms"][1], flops=conv.info.gemm_flops)
        else:
            passes = max(l["launches"] // 3, 1)
            f43_16 = io_dtype != torch.float32 and max(int(v) for v in conv.info.tile_m) == 4
            add("input_f43_tma_kernel" if f43_16 else "input_transform_kernel", l["stage_ms"][0],
                nbytes=float(esz) * math.prod(conv.in_shape), launches=passes)      # it must read x once
            if io_dtype == torch.float32:
                add("gemm_simt_kernel" if product_peak(conv)[1] == "fp32-fma" else "gemm_persistent_kernel",
                    l["stage_ms"][1], flops=conv.info.gemm_flops, launches=passes)
            else:
                add("gemm_persistent_kernel", l["stage_ms"][1], flops=conv.info.gemm_flops, launches=passes)
            add("output_f43_tma_kernel" if f43_16 and not (int(conv.desc.epilogue) & capi.EPI_POOL2) else "output_transform_kernel",
                l["stage_ms"][2], nbytes=float(esz) * math.prod(conv.out_shape), launches=passes)   # it must write y once
    kernel = max(classes, key=lambda k_: classes[k_][0])
    dom_ms, n_dom_launch, dom_flops, dom_bytes = classes[kernel]
    if dom_flops > 0:
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12
        if io_dtype == torch.float32:
            peak, bound = product_peak(layers[0])
            unit = "TFLOP/s"
        else:
            peak, unit, bound = tc_peak_16, "TFLOP/s", "tensor"
    else:
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        peak, unit, bound = peaks["hbm_gbs"], "GB/s", "hbm"
    traffic, traffic_source = None, None
    if (args.workload, kernel) in NCU_TRAFFIC_PER_IMAGE:
        per_image, traffic_source = NCU_TRAFFIC_PER_IMAGE[(args.workload, kernel)]
        traffic = per_image * batch
    step_roof_ms = sum(l["roof_ms"] for l in per_layer)
    step_roof_ms_contract = sum(l["roof_ms_contract"] for l in per_layer)
    roofline = {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
                "frac": round(achieved / peak, 4),
                "frac_contract": round(step_roof_ms_contract / sum(l["ms"] for l in per_layer), 4),
                "frac_contract_note": "sum over layers of max(F_gemm of the algorithm the configuration names / tensor peak, "
                                      "(x + w + convolution output bytes) / HBM peak), divided by the layers' measured time",
                "traffic": traffic, "traffic_source": traffic_source,
                "kernel": kernel, "launches_per_step": n_dom_launch,
                "avg_launch_us": round(1e3 * dom_ms / max(n_dom_launch, 1), 2),
                "kernel_share": {k_: round(v[0] / sum(c[0] for c in classes.values()), 4) for k_, v in classes.items()},
                "peak_source": f"MEASURED_PEAKS.json ({peaks_kind}; {'burst' if single_layer else 'sustained'} bf16 figure, copy bandwidth)",
                "stage_share": {n: round(t / sum(stage_tot), 4) for n, t in zip(stage_names, stage_tot)}}

    # ---- per-layer error beside the reference algebra's error, on a two-image sample (rank 0 of a 1-GPU run) ----
    errors = None
    if rank == 0 and world == 1 and not args.skip_errors:
        errors = layer_errors(args, layers, x_host, dev)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        if args.workload == "vgg16":
            v, n, el, cores = cpu_vgg_images_per_s(args.cpu_seconds)
            cpu_baseline = {"value": round(v, 3), "unit": "images/s", "cores": cores, "kind": "port",
                            "sample": f"{n} images of the same stack in {el:.1f} s, fp32 F(2x2,3x3) tile algebra "
                                      "(reference torch-level path restated in oracle/)"}
        elif args.workload == "cfg2":
            v, n, el, cores = cpu_cfg2_layers_per_s(args.cpu_seconds)
            cpu_baseline = {"value": round(v * 32, 3), "unit": "images/s", "cores": cores, "kind": "port",
                            "sample": f"{n} passes of the same layer in {el:.1f} s, fp32 F(2x2,3x3), CPU"}

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    flops_per_image = model.direct_flops / batch
    line = {
        "metric": metric, "value": round(value, 2), "unit": "images/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32" if io_dtype == torch.float32 else "f16", "data": "synthetic",
        "config": {"workload": workload, "per_gpu_batch": batch, "global_batch": int(total_images),
                   "parallelism": f"batch shards x{world}, no collective", "launch": "cuda_graph" if use_graph else "eager",
                   "l2": "activations and scratch of every step exceed the 126 MB L2 (inputs larger than L2)",
                   "weights": "filter transforms precomputed outside the timed region",
                   "accumulate": "fp32",
                   "winograd": describe_algorithms(layers)},
        "effective_tflops": round(value * flops_per_image / 1e12, 2),
        "with_filter_transform": {"value": round(total_images * args.steps / (ms_wft / 1e3), 2), "unit": "images/s",
                                  "ms_per_step": round(ms_wft / args.steps, 4),
                                  "note": "every layer's filter transform re-run inside each step, eager launches"},
        "step_roofline_frac": round(step_roof_ms / (ms / args.steps), 4),
        "step_roofline_frac_contract": round(step_roof_ms_contract / (ms / args.steps), 4),
        "e2e": {"value": round(e2e_value, 2), "unit": "images/s", "ms_per_step": round(ms_e2e / args.steps, 4),
                "h2d_bytes_per_step": int(x_host.numel() * x_host.element_size() * world),
                "d2h_bytes_per_step": int(y_host.numel() * y_host.element_size() * world)},
        "gpu_launches": int(model.launches_per_call * args.steps * world),   # all ranks, timed region of `value`
        "roofline": roofline, "cpu_baseline": cpu_baseline, "clocks": clocks, "layers": per_layer, "errors": errors,
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
