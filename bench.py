"""Benchmark of the quantization-simulation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 2): the weight of a Llama-3-8B MLP linear, [14336, 4096] bfloat16,
N(0, 0.02) with 0.1 % of the entries scaled 20x; one *step* is quantize-dequantize forward +
backward (input, scale and offset gradients) of that weight under three encodings: per-channel
symmetric int8, blockwise int4 (block 64) and LPBQ (int4 blocks, 8-bit per-channel scale).
Metric: algorithmic GB/s = 10 bytes per element and encoding / time (2 read + 2 written forward,
2 + 2 read and 2 written backward).

* ``value``: inputs resident in HBM, kernels launched through the C ABI on the current stream.
* ``e2e``: the same step through the public module API (``aimet_b200.quantizer``) with HOST
  buffers: pinned weight and upstream gradient copied in, parameter gradients and a checksum read
  back, inside the timed region.
* ``roofline``: the dominant kernel (backward), timed with CUDA events inside the timed region.
* ``cpu_baseline`` / ``--impl reference``: the CPU oracle (a restatement of the reference's torch
  path) on the host cores, on a bounded row-sample of the same weight.

With N > 1 every rank runs the same step on its own weight (independent layers: no collective),
reported as weak scaling; the calibration figure shards its batches over the ranks and
all-reduces min/max and histogram counts.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS, BLOCK = 14336, 4096, 64
BYTES_PER_ELEM = 10  # fwd 2 + 2, bwd 2 + 2 + 2 (bfloat16)
VARIANTS = ("per_channel_int8", "blockwise_int4", "lpbq_int4")


def make_weight(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    w = w * (1 + 19 * (torch.rand(rows, cols, generator=g) < 0.001))
    dy = torch.randn(rows, cols, generator=g)
    return w.to(torch.bfloat16), dy.to(torch.bfloat16)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def profile_traffic(key):
    """dram bytes per launch of the dominant kernel, copied from an ncu capture (profiles/*.md)."""
    path = os.path.join(ROOT, "profiles", "qdq_kernels_cfg2.md")
    if not os.path.exists(path):
        return None
    m = re.search(rf"^{key}\s*:\s*([0-9.eE+]+)", open(path).read(), flags=re.M)
    return float(m.group(1)) if m else None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# device-resident step through the C ABI
# --------------------------------------------------------------------------------------------
class ResidentStep:
    def __init__(self, w, dy, dev):
        from aimet_b200 import _lib
        from aimet_b200.quantizer import GroupedBlockQuantizeDequantize, QuantizeDequantize

        self.lib, self._lib = _lib.lib, _lib
        self.dev = dev
        self.w, self.dy = w.to(dev), dy.to(dev)
        self.y, self.gx = torch.empty_like(self.w), torch.empty_like(self.w)
        self.io = _lib.AB_BF16
        self.st = torch.cuda.current_stream(dev).cuda_stream
        rows, cols = w.shape
        nblk = cols // BLOCK
        self.enc = {}
        # encodings come from the public modules (calibration is not part of the timed step)
        mods = {
            "per_channel_int8": QuantizeDequantize((rows, 1), 8, True),
            "blockwise_int4": QuantizeDequantize((rows, nblk), 4, True, block_size=(1, BLOCK)),
            "lpbq_int4": GroupedBlockQuantizeDequantize((rows, nblk), 4, True, decompressed_bw=8,
                                                        block_size=(1, BLOCK), block_grouping=(1, -1)),
        }
        for name, q in mods.items():
            q = q.to(dev)
            with q.compute_encodings():
                q(self.w)
            with torch.no_grad():
                scale = q.get_scale().contiguous()
                offset = q.get_offset().contiguous()
            lay = _lib.make_layout([rows, cols], [1, cols] if name == "per_channel_int8" else [1, BLOCK])
            ct = _lib.AB_F32 if name == "per_channel_int8" else _lib.AB_BF16
            e = dict(scale=scale, offset=offset, lay=lay, ct=ct, qmin=q.qmin, qmax=q.qmax,
                     gs=torch.empty_like(scale), go=torch.empty_like(scale))
            if name == "lpbq_int4":
                with torch.no_grad():
                    raw = super(GroupedBlockQuantizeDequantize, q).get_scale().contiguous()
                    pcs = q.get_per_channel_scale().contiguous()
                e.update(raw=raw, pcs=pcs, zero=torch.zeros_like(pcs), lay_s=_lib.make_layout([rows, nblk], [1, nblk]),
                         g_raw=torch.empty_like(raw), g_pcs=torch.empty_like(pcs))
            self.enc[name] = e
        nb = max(self.lib.aimet_b200_backward_scratch_bytes(e["lay"], self.io) for e in self.enc.values())
        nb = max(nb, self.lib.aimet_b200_backward_scratch_bytes(self.enc["lpbq_int4"]["lay_s"], _lib.AB_F32), 16)
        self.scratch = torch.empty(nb, dtype=torch.uint8, device=dev)
        self.bwd_events = []

    def _ok(self, rc):
        if rc != 0:
            raise RuntimeError(self._lib.last_error())

    def run(self, record=False):
        lib, p = self.lib, torch.Tensor.data_ptr
        self.st = torch.cuda.current_stream(self.dev).cuda_stream  # the capture stream while a graph is recorded
        for name in VARIANTS:
            e = self.enc[name]
            if name == "lpbq_int4":  # block scales = integer multiples of the per-channel scale
                self._ok(lib.aimet_b200_quantize_dequantize(p(e["raw"]), p(e["scale"]), p(e["pcs"]), p(e["zero"]),
                                                            e["lay_s"], self._lib.AB_F32, self._lib.AB_F32, 0, 1, 16,
                                                            0.0, self.st))
            self._ok(lib.aimet_b200_quantize_dequantize(p(self.w), p(self.y), p(e["scale"]), p(e["offset"]), e["lay"],
                                                        self.io, e["ct"], 0, e["qmin"], e["qmax"], 0.0, self.st))
            if record:
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            self._ok(lib.aimet_b200_quantize_dequantize_backward(
                p(self.w), p(self.dy), p(e["scale"]), p(e["offset"]), e["lay"], self.io, e["ct"], 0, e["qmin"],
                e["qmax"], 0.0, p(self.gx), p(e["gs"]), None, p(self.scratch), self.scratch.numel(), self.st))
            if record:
                ev1.record()
                self.bwd_events.append((ev0, ev1))
            if name == "lpbq_int4":  # gradient of the block scales flows on to the raw scales
                self._ok(lib.aimet_b200_quantize_dequantize_backward(
                    p(e["raw"]), p(e["gs"]), p(e["pcs"]), p(e["zero"]), e["lay_s"], self._lib.AB_F32,
                    self._lib.AB_F32, 0, 1, 16, 0.0, p(e["g_raw"]), p(e["g_pcs"]), None, p(self.scratch),
                    self.scratch.numel(), self.st))


    def run_backward_only(self):
        """The three backward launches of a step on their own (same tensors, same encodings)."""
        lib, p = self.lib, torch.Tensor.data_ptr
        self.st = torch.cuda.current_stream(self.dev).cuda_stream
        for name in VARIANTS:
            e = self.enc[name]
            self._ok(lib.aimet_b200_quantize_dequantize_backward(
                p(self.w), p(self.dy), p(e["scale"]), p(e["offset"]), e["lay"], self.io, e["ct"], 0, e["qmin"],
                e["qmax"], 0.0, p(self.gx), p(e["gs"]), None, p(self.scratch), self.scratch.numel(), self.st))


# --------------------------------------------------------------------------------------------
# end-to-end step through the public API with host buffers
# --------------------------------------------------------------------------------------------
class HostStep:
    def __init__(self, w, dy, dev):
        from aimet_b200.quantizer import GroupedBlockQuantizeDequantize, QuantizeDequantize

        self.dev = dev
        self.w_host, self.dy_host = w.pin_memory(), dy.pin_memory()
        rows, cols = w.shape
        nblk = cols // BLOCK
        self.mods = [
            QuantizeDequantize((rows, 1), 8, True).to(dev),
            QuantizeDequantize((rows, nblk), 4, True, block_size=(1, BLOCK)).to(dev),
            GroupedBlockQuantizeDequantize((rows, nblk), 4, True, decompressed_bw=8, block_size=(1, BLOCK),
                                           block_grouping=(1, -1)).to(dev),
        ]
        wd = w.to(dev)
        for q in self.mods:
            with q.compute_encodings():
                q(wd)
        self.h2d = (self.w_host.numel() + self.dy_host.numel()) * 2
        self.d2h = 0

    def _compute(self, w, dy):
        outs = []
        for q in self.mods:
            wi = w.detach().requires_grad_(True)
            q.min.grad = q.max.grad = None
            y = q(wi)
            y.backward(dy)
            outs += [q.min.grad.flatten(), q.max.grad.flatten(), torch.sum(wi.grad, dtype=torch.float32).reshape(1)]
        return torch.cat(outs)

    def run(self):
        # one step: the weight and the upstream gradient come from pinned host memory once, then the
        # three encodings run on them; parameter gradients and a checksum go back to the host
        w = self.w_host.to(self.dev, non_blocking=True)
        dy = self.dy_host.to(self.dev, non_blocking=True)
        res = self._compute(w, dy).cpu()
        self.d2h = res.numel() * 4
        return res

    def run_many(self, steps):
        """``steps`` steps with the copies of step i+1 (a second stream, a second pair of device
        buffers) overlapping the kernels of step i.  Every step still copies its own inputs from
        pinned host memory and reads its own result back."""
        main = torch.cuda.current_stream(self.dev)
        copier = torch.cuda.Stream(self.dev)
        bufs = [(torch.empty_like(self.w_host, device=self.dev), torch.empty_like(self.dy_host, device=self.dev))
                for _ in range(2)]
        ready = [torch.cuda.Event() for _ in range(2)]
        free = [torch.cuda.Event() for _ in range(2)]

        def prefetch(i):
            b = i % 2
            with torch.cuda.stream(copier):
                if i >= 2:
                    copier.wait_event(free[b])
                bufs[b][0].copy_(self.w_host, non_blocking=True)
                bufs[b][1].copy_(self.dy_host, non_blocking=True)
                ready[b].record(copier)

        results, pinned, done = [], [None, None], [torch.cuda.Event() for _ in range(2)]
        prefetch(0)
        for i in range(steps):
            b = i % 2
            if i + 1 < steps:
                prefetch(i + 1)
            main.wait_event(ready[b])
            out = self._compute(*bufs[b])
            free[b].record(main)
            if pinned[b] is None:
                pinned[b] = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
            pinned[b].copy_(out, non_blocking=True)  # this step's result, read back asynchronously
            done[b].record(main)
            if i >= 1:  # the host picks up the previous step's result while this one runs
                done[1 - b].synchronize()
                results.append(pinned[1 - b].clone())
        done[(steps - 1) % 2].synchronize()
        results.append(pinned[(steps - 1) % 2].clone())
        self.d2h = results[-1].numel() * 4
        return results


# --------------------------------------------------------------------------------------------
# CPU oracle leg
# --------------------------------------------------------------------------------------------
def cpu_step(sample_rows):
    """One step of the workload on a row sample through the CPU oracle.  Returns seconds."""
    from oracle import affine as OA
    from oracle import encoding_analyzer as OE
    from oracle import quantizer as OQ

    w, dy = make_weight(sample_rows, COLS, seed=2000)
    nblk = COLS // BLOCK
    encs = []
    for shape, bw, block in (((sample_rows, 1), 8, None), ((sample_rows, nblk), 4, (1, BLOCK)), ((sample_rows, nblk), 4, (1, BLOCK))):
        steps = 2**bw - 1
        qmin, qmax = -((steps + 1) // 2), steps // 2
        mn, mx = OE.minmax_collect(w, shape, block)
        mn, mx = OE.minmax_encodings(mn, mx, steps, True)
        encs.append((mn.float(), mx.float(), qmin, qmax, block))
    t0 = time.perf_counter()
    for i, (mn, mx, qmin, qmax, block) in enumerate(encs):
        scale, offset = OQ.scale_offset_from_min_max(mn, mx, qmin, qmax, True)
        if i == 2:
            scale, _ = OQ.lpbq_scale(scale, 4, 8, (1, -1))
        OA.quantize_dequantize(w, scale, offset, qmin, qmax, block)
        OA.quantize_dequantize_backward(w, dy, scale, offset, qmin, qmax, block)
    return time.perf_counter() - t0


def cpu_baseline(sample_rows=1024, repeats=3):
    torch.set_num_threads(os.cpu_count() or 1)
    cpu_step(sample_rows)
    times = [cpu_step(sample_rows) for _ in range(repeats)]
    t = statistics.median(times)
    gbs = 3 * sample_rows * COLS * BYTES_PER_ELEM / t / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_rows} of {ROWS} rows of the weight, all three encodings, median of {repeats} runs"}


# --------------------------------------------------------------------------------------------
# secondary figures: calibration (config 3) and SeqMSE (config 5)
# --------------------------------------------------------------------------------------------
def student_t_batch(gen, hot, dev, tokens=16 * 2048, channels=4096, df=3):
    z = torch.randn((tokens, channels), device=dev, generator=gen)
    chi = torch.randn((tokens, channels, df), device=dev, generator=gen).pow_(2).sum(-1)
    x = z / torch.sqrt(chi / df)
    x[:, hot] *= 50
    return x.to(torch.bfloat16).view(16, 2048, channels)


def calibration_figure(dev, rank, world, num_batches=64):
    """SQNR calibration of config 3: ``num_batches`` activation batches [16,2048,4096] bf16 (Student-t,
    df 3, 32 channels x50) dealt round-robin to the ranks; two-phase exact histogram (min/max
    all-reduce, 2048-bin int64 count all-reduce), then the 17x21 asymmetric candidate sweep."""
    import torch.distributed as dist

    from aimet_b200 import distributed as D
    from aimet_b200 import encoding_analyzer as EA

    gen = torch.Generator(device=dev).manual_seed(3000)
    hot = torch.randperm(4096, device=dev, generator=gen)[:32]
    mine = D.my_batches(num_batches, rank, world)
    batches = []
    for b in range(num_batches):  # every rank draws the same stream and keeps its own share
        x = student_t_batch(gen, hot, dev)
        if b in mine:
            batches.append(x)
    group = dist.group.WORLD if world > 1 else None

    def run():
        an = EA.SqnrEncodingAnalyzer((), num_bins=2048)
        D.calibrate_histogram(an, batches, group)
        return an.compute_encodings(255, False)

    run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        enc = run()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    tokens = num_batches * 16 * 2048
    peaks, kind = measured_peaks()
    bytes_moved = num_batches * 16 * 2048 * 4096 * 2 * 2  # two passes over every batch
    # the reference's own calling pattern: update_stats batch after batch (range growth + merge)
    seq = EA.SqnrEncodingAnalyzer((), num_bins=2048)
    seq.update_stats(batches[0])
    torch.cuda.synchronize()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for x in batches:
        seq.update_stats(x)
    s1.record()
    torch.cuda.synchronize()
    seq_ms = s0.elapsed_time(s1)
    sequential = {"tokens_per_s_per_gpu": len(batches) * 16 * 2048 / (seq_ms * 1e-3), "ms_per_batch": seq_ms / len(batches),
                  "what": "analyzer.update_stats on this rank's batches one after the other (no exchange)"}
    return {"sequential_update_stats": sequential, "metric": "calibration_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "ms": ms,
            "batches": num_batches, "batch_shape": [16, 2048, 4096], "analyzer": "SQNR, 2048 bins, 17x21 asymmetric candidates",
            "algorithmic_bytes": bytes_moved, "achieved_GBps_per_gpu": bytes_moved / world / (ms * 1e-3) / 1e9,
            "frac_of_" + kind + "_hbm": bytes_moved / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "encoding_min_max": [float(enc[0]), float(enc[1])]}


def seqmse_figure(dev, rank, world, m=8192, n=4096, k=4096, cands=20):
    """Config 5: reconstruction loss of 20 candidates for a [4096,4096] bf16 weight on 8192 tokens;
    output channels split across ranks."""
    import torch.distributed as dist

    from aimet_b200 import distributed as D
    from aimet_b200.seq_mse import linear_loss_all_candidates

    gen = torch.Generator(device=dev).manual_seed(5000)
    x = torch.randn((m, k), device=dev, generator=gen)
    x[:, torch.randperm(k, device=dev, generator=gen)[:20]] *= 30
    x = x.to(torch.bfloat16)
    lo, hi = D.shard_range(n, rank, world)
    w = (torch.randn((n, k), device=dev, generator=gen) * 0.02).to(torch.bfloat16)[lo:hi].contiguous()
    fr = torch.linspace(0.5, 1.0, cands, device=dev)  # BASELINE's candidate grid: [0.5 max, max]
    smax = w.float().abs().amax(1, keepdim=True) / 7
    wq = torch.stack([(torch.clamp(torch.round(w.float() / (smax * f)), -8, 7) * (smax * f)).to(torch.bfloat16) for f in fr])
    for _ in range(2):
        linear_loss_all_candidates(x, x, w, wq, "mse")
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        loss = linear_loss_all_candidates(x, x, w, wq, "mse")
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops = 2.0 * m * n * k * cands
    peaks, kind = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {"metric": "seqmse_candidate_TFLOPs", "value": tf, "unit": "TFLOP/s (whole job)", "ms": ms,
            "shape": {"tokens": m, "out": n, "in": k, "candidates": cands}, "per_gpu_TFLOPs": tf / world,
            "frac_of_" + kind + "_bf16_burst": tf / world / peaks["bf16_tflops"],
            "frac_of_sustained": tf / world / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]),
            "best_index_histogram": torch.bincount(loss.argmin(0), minlength=cands).tolist()}


def resnet50_figure(dev, batch=256):
    """Config 4: forward of a random-init ResNet-50 at batch 256 (224x224 fp32, N(0,1)) with per-channel
    int8 weight QDQ and per-tensor int8 QDQ on the input and output of all 54 conv / linear layers
    (the reference's QuantSim model builder is replaced by ``aimet_b200.nn.quantize_model``).
    QDQ share = 1 - plain forward time / quantized forward time."""
    try:
        import torchvision
    except ImportError:
        return {"unavailable": "torchvision is not installed"}
    from aimet_b200 import nn as qnn

    torch.manual_seed(4000)
    model = torchvision.models.resnet50(weights=None).eval().to(dev)
    x = torch.randn(batch, 3, 224, 224, device=dev)

    def timed(m, reps=5):
        with torch.no_grad():
            for _ in range(2):
                m(x)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                m(x)
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    plain_ms = timed(model)
    qmodel = qnn.quantize_model(model)
    with torch.no_grad(), qnn.compute_encodings(qmodel):
        qmodel(x[:32])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.no_grad(), qnn.compute_encodings(qmodel):  # model-level calibration, timed on its second run
        qmodel(x[:64])
        qmodel(x[64:128])
    torch.cuda.synchronize()
    calib_ms = (time.perf_counter() - t0) * 1e3
    quant_ms = timed(qmodel)
    layers = list(qnn.quantized_layers(qmodel))
    act_elems, w_elems = 0, 0
    hooks = []

    def count(_m, inp, out):
        nonlocal act_elems
        act_elems += inp[0].numel() + out.numel()

    for layer in layers:
        hooks.append(layer.register_forward_hook(count))
        w_elems += layer.weight.numel()
    with torch.no_grad():
        qmodel(x)
    for h in hooks:
        h.remove()
    qdq_bytes = act_elems * 8  # the quantized weights are kept across forwards (25.5 M elements, once)
    peaks, kind = measured_peaks()
    qdq_ms = quant_ms - plain_ms
    return {"metric": "quantsim_resnet50_images_per_s", "value": batch / (quant_ms * 1e-3), "unit": "images/s",
            "batch": batch, "quantized_layers": len(layers), "forward_ms": quant_ms, "plain_forward_ms": plain_ms,
            "qdq_ms": qdq_ms, "qdq_share": qdq_ms / quant_ms, "qdq_algorithmic_bytes": qdq_bytes,
            "weight_elements": w_elems, "weight_qdq": "kept across forwards while weight and range are unchanged",
            "calibration_ms_128_images": calib_ms,
            "qdq_achieved_GBps": qdq_bytes / (qdq_ms * 1e-3) / 1e9,
            "qdq_frac_of_" + kind + "_hbm": qdq_bytes / (qdq_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}


def base_config(n_gpus):
    return {"workload": "configs[1]: Llama-3-8B MLP weight [14336,4096] bf16 QDQ fwd+bwd: per-channel int8 + "
                        "blockwise int4 (block 64) + LPBQ (int4, 8-bit per-channel scale), scale grads on",
            "elements_per_step": 3 * ROWS * COLS, "algorithmic_bytes_per_element": BYTES_PER_ELEM,
            "l2": "inputs larger than L2: 470 MB touched per encoding vs 126 MB L2",
            "parallelism": f"replicated layers x{n_gpus}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    rows = 512
    for _ in range(args.warmup):
        cpu_step(rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(rows)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = 3 * rows * COLS * BYTES_PER_ELEM / dt / 1e9
    sample = f"each step = {rows} of {ROWS} rows of the weight, all three encodings, CPU oracle (restated torch path)"
    print(json.dumps({
        "impl": "reference", "metric": "qdq_fwd_bwd_algorithmic_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": base_config(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from aimet_b200 import _lib

    w, dy = make_weight(ROWS, COLS, seed=2000 + rank)
    resident = ResidentStep(w, dy, dev)
    host = HostStep(w, dy, dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident: the step's launches are captured once and replayed as a CUDA graph ----
    for _ in range(3):
        resident.run()
    barrier()
    before = _lib.lib.aimet_b200_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        resident.run()
    launches_per_step = _lib.lib.aimet_b200_launch_count() - before
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            graph.replay()
        end.record()
        barrier()
        ms = start.elapsed_time(end)
        # the same steps once more, launched one by one with events around every backward launch:
        # the per-launch duration behind `roofline`
        for _ in range(args.steps):
            resident.run(record=True)
        torch.cuda.synchronize()
        # and the backward launches alone, back to back (3 per step), between two events: the
        # kernel's duration without the idle time an isolated launch has around it
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        resident.run_backward_only()
        b0.record()
        for _ in range(args.steps):
            resident.run_backward_only()
        b1.record()
        torch.cuda.synchronize()
        bwd_tight = b0.elapsed_time(b1) / (3 * args.steps)
        if ms < 300:  # keep the sampler alive long enough to see clocks under load
            t_end = time.time() + 0.4
            while time.time() < t_end:
                graph.replay()
            torch.cuda.synchronize()
    launches = launches_per_step * args.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    step_bytes = 3 * ROWS * COLS * BYTES_PER_ELEM
    value = world * step_bytes / (ms_step * 1e-3) / 1e9

    bwd_ms = [a.elapsed_time(b) for a, b in resident.bwd_events]
    bwd_single = sum(bwd_ms) / len(bwd_ms)
    bwd_avg = bwd_tight
    peaks, peak_kind = measured_peaks()
    achieved = ROWS * COLS * 6 / (bwd_avg * 1e-3) / 1e9

    # ---- end to end through the module API with host buffers ----
    for _ in range(2):
        host.run()
    barrier()
    e2e_steps = max(2, min(args.steps, 10))
    t0 = time.perf_counter()
    host.run_many(e2e_steps)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * step_bytes / float(t.item()) / 1e9

    if rank == 0:
        out = {
            "metric": "qdq_fwd_bwd_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": base_config(world),
            "launch": "the step's kernel launches (C-ABI calls) are captured once and replayed as one CUDA graph",
            "roofline": {"bound": "hbm", "kernel": "k_bwd_seg (quantize-dequantize backward, bf16, [14336,4096])",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_source": f"{peak_kind} copy bandwidth",
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "frac_of_nominal_8TBps": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": ROWS * COLS * 6, "avg_launch_us": bwd_avg * 1e3,
                         "timed_in": "after the graph replays: K x 3 backward launches back to back between two "
                                     "CUDA events (352 MB touched per launch, larger than L2)",
                         "isolated_launch_us": bwd_single * 1e3,
                         "isolated_launch_note": "the same K steps launched one by one with events around every "
                                                 "backward launch (includes the idle time around a lone launch)",
                         "traffic": profile_traffic("bwd_dram_bytes_per_launch")},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": host.h2d, "d2h_bytes_per_step": host.d2h,
                    "ms_per_step": e2e_s * 1e3,
                    "overlap": "the copies of step i+1 run on a second stream while step i computes"},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "frac_of_measured_hbm": value / world / peaks["hbm_gbs"],
        }
        if world == 1 and not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline()
    extras = {}
    if not args.no_extras:
        del resident, host
        torch.cuda.empty_cache()
        extras["calibration"] = calibration_figure(dev, rank, world)
        torch.cuda.empty_cache()
        extras["seqmse"] = seqmse_figure(dev, rank, world)
        if world == 1:  # a model forward does not shard: replicas only
            torch.cuda.empty_cache()
            extras["quantsim_resnet50"] = resnet50_figure(dev)
    if rank == 0:
        out.update(extras)
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_kernels_only(steps, case):
    """A few eager resident steps and nothing else: the small, fixed launch sequence that the ncu
    captures under ``profiles/`` are taken from (``qdq``: 8 launches per step, see
    ResidentStep.run; ``calibration``: a two-phase SQNR calibration over 4 config-3 batches)."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if case == "calibration":
        from aimet_b200 import distributed as D
        from aimet_b200 import encoding_analyzer as EA

        gen = torch.Generator(device=dev).manual_seed(3000)
        hot = torch.randperm(4096, device=dev, generator=gen)[:32]
        batches = [student_t_batch(gen, hot, dev) for _ in range(4)]
        for _ in range(steps):
            an = EA.SqnrEncodingAnalyzer((), num_bins=2048)
            D.calibrate_histogram(an, batches, None)
            an.compute_encodings(255, False)
        torch.cuda.synchronize()
        print(json.dumps({"kernels_only_steps": steps, "case": case}))
        return
    w, dy = make_weight(ROWS, COLS, seed=2000)
    resident = ResidentStep(w, dy, dev)
    for _ in range(steps):
        resident.run()
    torch.cuda.synchronize()
    print(json.dumps({"kernels_only_steps": steps}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-oracle baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the calibration and SeqMSE figures")
    ap.add_argument("--kernels-only", type=int, default=0, metavar="STEPS",
                    help="run STEPS eager resident steps and exit (for profiler captures)")
    ap.add_argument("--kernels-case", default="qdq", choices=["qdq", "calibration"])
    args = ap.parse_args()
    if args.kernels_only:
        run_kernels_only(args.kernels_only, args.kernels_case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
