#!/usr/bin/env python
"""Benchmark of the hot path: whole-network inference throughput on N B200s of one node.

    python bench.py --gpus N --steps K --warmup W [--workload tinyyolov2|dscnn]
    python bench.py --impl reference ...      # the reference's CPU code on the host cores

A step is one pass of the layer chain over one batch of seeded synthetic inputs
(Tiny-YOLOv2 fp32: 64 images of 3x416x416 per GPU, i.e. the 512-image batch of the
configuration sharded over 8 GPUs; DS-CNN uint8: 4096 images of 1x49x10 per GPU).  Images
are independent, so ranks share nothing on the data path (weak scaling, no collective).
Prints ONE JSON line on rank 0.  Without --workload the line is the Tiny-YOLOv2 measurement and
carries the DS-CNN measurement (same fields) under "workloads".

The K steps of --steps are timed as one round between two barriers; rounds are repeated until at
least a second has been timed, and the median round is what the line reports (the fastest one is
there too), with the SM clock sampled over the whole span.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "tinyyolov2": dict(dtype="f32", per_gpu_batch=64, seed=4,
                       desc="Tiny-YOLOv2 fp32 3x416x416, 512 images over 8 GPUs = 64 per GPU"),
    "dscnn": dict(dtype="u8", per_gpu_batch=4096, seed=1,
                  desc="DS-CNN uint8 1x49x10, batch 4096 per GPU"),
    # the other configurations (parity-test cases; benchable on request)
    "resnet8": dict(dtype="f32", per_gpu_batch=1024, seed=0, desc="ResNet-8 fp32 3x32x32, batch 1024 per GPU"),
    "mobilenet": dict(dtype="f32", per_gpu_batch=2048, seed=2,
                      desc="MobileNet-v1 x0.25 fp32 3x96x96, batch 2048 per GPU"),
    "mobilenet_u8": dict(dtype="u8", per_gpu_batch=2048, seed=2,
                         desc="MobileNet-v1 x0.25 uint8 3x96x96, batch 2048 per GPU"),
}
METRIC = "inferences/s"


def config_of(workload, batch, world):
    """The `config` object of a JSON line: the same for the GPU arm and the reference arm."""
    wl = WORKLOADS[workload]
    small = wl["dtype"] == "u8"
    return {"workload": wl["desc"], "per_gpu_batch": batch, "global_batch": batch * world,
            "l2": ("the network input rotates over more batches than the 126 MB L2 holds; the activations "
                   "between the layers of a step (32 MB per layer at batch 4096) are produced and consumed "
                   "inside L2 by design, so per-layer figures of this workload are L2 figures"
                   if small else
                   "per-step input (133 MB) and every activation exceed the 126 MB L2; no flush needed"),
            "graph": "whole network captured in one CUDA graph per GPU"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=float(p["hbm_gbs"]), tensor=float(p["bf16_tflops_sustained"]),
                    tensor_burst=float(p["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


def make_layers(workload):
    from smallframework_b200 import networks
    if workload == "tinyyolov2":
        return networks.tiny_yolov2(seed=4)
    if workload == "dscnn":
        return networks.ds_cnn(seed=1)
    if workload == "resnet8":
        return networks.resnet8(seed=0)
    return networks.mobilenet_v1_025(seed=2, dtype="u8" if workload.endswith("u8") else "f32")


def make_input(workload, layers, batch, seed):
    """Seeded synthetic inputs, already in the packed layout (first layer: HWC interleaved)."""
    from smallframework_b200 import networks, packing
    c, h, w = networks.input_shape(layers)
    rng = np.random.default_rng(seed + 1000)
    if WORKLOADS[workload]["dtype"] == "f32":
        x = rng.random((batch, c, h, w), dtype=np.float32)
    else:
        x = rng.integers(0, 256, (batch, c, h, w), dtype=np.uint8)
    return packing.pack_activation(x)


# ------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------- CPU reference
def reference_layers(layers, platform_cb, dtype):
    """The layer list in the form oracle/bindings.Ref.run_chain takes, weights packed for the
    CPU platform's blocking."""
    from oracle.bindings import Quant, shape
    from smallframework_b200 import packing
    out = []
    for L in layers:
        s = shape(L["C"], L["K"], L["H"], L["W"], L["Fh"], L["Fw"], L["stride"], L["pads"], platform_cb)
        d = dict(op=L["op"], s=s, act=L.get("act", 0), slope=L.get("slope", 0.0))
        if L["op"] == "conv":
            w, b, _ = packing.pad_output_channels(L["w"], L.get("b"), platform_cb)
            s.K = w.shape[0]
            d["filt"] = packing.pack_conv_filter(w, platform_cb, platform_cb)
            if dtype == "f32":
                d["bias"] = b
        elif L["op"] == "dwconv":
            d["filt"] = packing.pack_dw_filter(L["w"], platform_cb)
            if dtype == "f32" and L.get("b") is not None:
                d["bias"] = L["b"]
        if "q" in L:
            q = L["q"]
            d["q"] = Quant(q["zero_in"], q["zero_filt"], q["lshift"], q["rshift"], q["multiplier"], 0)
        out.append(d)
    return out


def has_avx2():
    try:
        return " avx2 " in open("/proc/cpuinfo").read() and " fma " in open("/proc/cpuinfo").read()
    except OSError:
        return False


def time_reference(workload, layers, threads, budget_s=12.0, max_images=4096):
    """Times the reference's own CPU implementation (compiled from its headers into
    oracle/_ref) on a bounded sample of the workload.  Returns dict(value, cores, kind,
    sample, platform).  fp32 runs the AVX2 platform (ZEN2) when the host has AVX2+FMA, else
    the scalar REF platform; uint8 exists on REF only."""
    from oracle.bindings import Ref
    from smallframework_b200 import networks
    dtype = WORKLOADS[workload]["dtype"]
    if dtype == "f32":
        platform = "zen2" if has_avx2() else "ref"
    else:
        platform = "ref"
        # the reference has no quint8 average pool and no per-channel bias: time the
        # convolution chain it does have (stem + 4 x (dw, pw)); the pool and the 64->12
        # dense layer are under 0.2 % of the arithmetic
        layers = [L for L in layers if L["op"] in ("conv", "dwconv") and L["name"] != "dense"]
    ref = Ref(platform)
    cb = ref.float_cb if dtype == "f32" else ref.quint8_cb
    rl = reference_layers(layers, cb, dtype)
    from smallframework_b200 import packing
    c, h, w = networks.input_shape(layers)
    rng = np.random.default_rng(5)
    x = rng.random((c, h, w), dtype=np.float32) if dtype == "f32" else rng.integers(0, 256, (c, h, w), dtype=np.uint8)
    xp = packing.pack_activation(x, cb)
    last = rl[-1]["s"]
    ho, wo = last.out_hw()
    out_elems = (last.K if rl[-1]["op"] == "conv" else last.C) * ho * wo
    tag = "f32" if dtype == "f32" else "u8"
    n0 = threads if dtype == "u8" else 1
    sec, _ = ref.run_chain(rl, xp, n0, threads, out_elems, tag)          # warm-up + probe
    per_image = max(sec / n0, 1e-6)
    images = int(min(max_images, max(n0, budget_s / per_image)))
    if dtype == "u8":
        images = max(threads, images // threads * threads)
    sec, _ = ref.run_chain(rl, xp, images, threads, out_elems, tag)
    return dict(value=images / sec, unit=METRIC, cores=threads, kind="reference", platform=platform,
                sample=f"{images} images of the same layer chain through the reference's "
                       f"{platform.upper()} platform in {sec:.2f} s"
                       + ("" if dtype == "f32" else " (convolution layers only: stem + 4 x (dw, pw))"))


def reference_line(args, workload):
    """The reference's own CPU implementation of one workload on this host's cores, as a JSON line."""
    layers = make_layers(workload)
    threads = os.cpu_count() or 1
    per = []
    for _ in range(max(args.warmup, 0) + max(args.steps, 1)):
        per.append(time_reference(workload, layers, threads,
                                  budget_s=max(2.0, 40.0 / (args.steps + args.warmup))))
    timed = per[max(args.warmup, 0):]
    v = float(np.mean([p["value"] for p in timed]))
    wl = WORKLOADS[workload]
    return {
        "impl": "reference", "metric": METRIC, "value": v, "unit": METRIC, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / v if v else None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"],
        "data": "synthetic (seeded), random-init weights",
        "config": config_of(workload, args.batch or wl["per_gpu_batch"], max(args.gpus, 1)),
        "cpu_baseline": dict(timed[-1], value=v),
        "e2e": {"value": v, "unit": METRIC, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    line = reference_line(args, args.workload or "tinyyolov2")
    if not args.workload:
        line["workloads"] = {"dscnn": reference_line(args, "dscnn")}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- GPU arm
def measured_pipes(torch):
    """tera-ops/s of the fp32 FMA pipe and of the tf32 / i8 tensor pipes of this GPU, from the
    library's resident-operand probes (small_b200_peak_probe), next to what the nominal ratios to the
    measured bf16 GEMM would give."""
    from smallframework_b200 import _lib
    peaks = load_peaks()
    out = {}
    for kind, name in ((0, "ffma"), (1, "tf32"), (2, "i8")):
        v = C.c_double(0.0)
        _lib.check(_lib.lib().small_b200_peak_probe(kind, C.byref(v)))
        out[name] = v.value
    floor = {}
    for kind, name in ((3, "tf32_m128_n32"), (4, "i8_m128_n32")):
        v = C.c_double(0.0)
        _lib.check(_lib.lib().small_b200_peak_probe(kind, C.byref(v)))
        floor[name] = round(v.value, 1)
    out["mma_floor_cycles_per_instruction"] = floor
    torch.cuda.synchronize()
    out["assumed"] = {"tf32": peaks["tensor_burst"] / 2.0, "i8": peaks["tensor_burst"] * 2.0}
    out["how"] = "resident-operand issue loops: FFMA chains in registers; tcgen05.mma M128 N256 from shared memory, 2 issuing threads per SM"
    return out


def h2d_bandwidth(l, check, dst_ptr, host_ptr, nbytes, stream, torch, min_bytes=2e8):
    """Upload alone: pinned host memory -> device, GB/s, per rank."""
    reps = max(3, int(min_bytes // max(nbytes, 1)))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    check(l.small_b200_memcpy_h2d(dst_ptr, host_ptr, nbytes, stream.cuda_stream))
    e0.record(stream)
    for _ in range(reps):
        check(l.small_b200_memcpy_h2d(dst_ptr, host_ptr, nbytes, stream.cuda_stream))
    e1.record(stream)
    stream.synchronize()
    return nbytes * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9


def measure_workload(args, workload, env, pipes):
    """One workload on this rank's GPU: resident rounds, end-to-end rounds, per-layer report."""
    torch, dist, world, rank, local = env
    from smallframework_b200 import _lib, networks, sharding
    from smallframework_b200._lib import check, lib
    wl = WORKLOADS[workload]
    batch = args.batch or wl["per_gpu_batch"]
    layers = make_layers(workload)
    chain = networks.Chain(layers, batch, wl["dtype"], fuse_u8=not args.no_fuse_u8)
    l = lib()
    st = chain.stream.cuda_stream

    # host side: pinned input / output staging through the C ABI
    xp = make_input(workload, layers, batch, wl["seed"] + rank)
    in_bytes = xp.nbytes
    hin, hout = C.c_void_p(), C.c_void_p()
    alloc_in = l.small_b200_malloc_host_upload if args.upload_memory == "wc" else l.small_b200_malloc_host
    check(alloc_in(in_bytes, C.byref(hin)))
    C.memmove(hin, xp.ctypes.data, in_bytes)
    check(l.small_b200_memcpy_h2d(chain.x.data_ptr(), hin, in_bytes, st))
    chain.stream.synchronize()
    # resident leg: the input rotates over copies of the batch that together exceed L2 (a network whose
    # whole input is a few MB would otherwise be timed on an L2-resident input)
    copies = 2 if in_bytes > 160e6 / 2 else int(min(96, -(-160e6 // in_bytes)))
    inputs = [chain.x] + [chain.x.clone() for _ in range(copies - 1)]
    chain.capture(inputs)
    out_bytes = chain.y.numel() * chain.y.element_size()
    check(l.small_b200_malloc_host(out_bytes, C.byref(hout)))
    chain.stream.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_round(fn, steps, finish=None):
        """exactly `steps` steps between two barriers; device time, max over ranks"""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(chain.stream)
        for _ in range(steps):
            fn()
        if finish:
            finish()  # work of these steps on other streams is inside the timed span
        e1.record(chain.stream)
        chain.stream.synchronize()
        barrier()
        return sharding.max_over_ranks(e0.elapsed_time(e1), device="cuda")

    def timed(fn, steps, budget_s, finish=None):
        first = timed_round(fn, steps, finish)
        rounds = int(min(400, max(1, budget_s * 1e3 / max(first, 1e-3))))
        if world > 1:  # every rank must run the same number of rounds
            t = torch.tensor([rounds], device="cuda")
            dist.broadcast(t, 0)
            rounds = int(t.item())
        ms = [first] + [timed_round(fn, steps, finish) for _ in range(rounds - 1)]
        return float(np.median(ms)), float(np.min(ms)), len(ms), float(np.sum(ms))

    step_no = [0]

    def step_resident():
        chain.launch(step_no[0])
        step_no[0] += 1

    # End to end: every step copies its batch from pinned host memory and reads its result back.
    # Three streams: the upload of step i+1 (into the other of two input buffers, which the recorded
    # graphs read directly) and the download of step i-1's result (from a small device copy of it)
    # both overlap the graph of step i.
    copy_stream, down_stream = torch.cuda.Stream(), torch.cuda.Stream()
    y_stage = [torch.empty_like(chain.y) for _ in range(2)]
    hout2 = C.c_void_p()
    check(l.small_b200_malloc_host(out_bytes, C.byref(hout2)))
    houts = [hout, hout2]
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_y = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]
    e2e_count = [0]

    def step_e2e():
        i = e2e_count[0] & 1
        e2e_count[0] += 1
        copy_stream.wait_event(ev_free[i])          # input buffer i was consumed two steps ago
        check(l.small_b200_memcpy_h2d(inputs[i].data_ptr(), hin, in_bytes, copy_stream.cuda_stream))
        ev_up[i].record(copy_stream)
        chain.stream.wait_event(ev_up[i])
        chain.launch(i)                             # graph i reads input buffer i
        ev_free[i].record(chain.stream)
        chain.stream.wait_event(ev_down[i])         # result copy i went to the host two steps ago
        check(l.small_b200_memcpy_d2d(y_stage[i].data_ptr(), chain.y.data_ptr(), out_bytes, st))
        ev_y[i].record(chain.stream)
        down_stream.wait_event(ev_y[i])
        check(l.small_b200_memcpy_d2h(houts[i], y_stage[i].data_ptr(), out_bytes, down_stream.cuda_stream))
        ev_down[i].record(down_stream)

    def finish_e2e():
        for ev in ev_down:
            chain.stream.wait_event(ev)

    for _ in range(max(args.warmup, 3)):
        step_resident()
    budget = args.min_seconds
    with ClockSampler(local) as clk:
        ms, ms_min, rounds, span_ms = timed(step_resident, args.steps, budget)
        for _ in range(2):
            step_e2e()
        ms_e2e, ms_e2e_min, rounds_e2e, span_e2e = timed(step_e2e, args.steps, budget, finish_e2e)
    h2d_gbs = h2d_bandwidth(l, check, inputs[1].data_ptr(), hin, in_bytes, copy_stream, torch)
    # the same upload with every rank of the box uploading at once: what the host side (memory, root
    # complexes) gives one GPU when all of them pull, i.e. the ceiling of the end-to-end leg at this N
    h2d_all = None
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        mine = h2d_bandwidth(l, check, inputs[1].data_ptr(), hin, in_bytes, copy_stream, torch, min_bytes=1.5e9)
        t = torch.tensor([mine, -mine, mine], dtype=torch.float64, device="cuda")
        parts = [t.clone() for _ in range(world)]
        dist.all_gather(parts, t)
        vals = [float(p[0]) for p in parts]
        h2d_all = {"per_rank_min_gbs": round(min(vals), 2), "per_rank_max_gbs": round(max(vals), 2),
                   "aggregate_gbs": round(sum(vals), 1)}
    # The final host gather (outside the timed spans): every rank's result for its own batch goes to
    # rank 0, which recomputes each shard from that rank's seed on its own GPU and compares the bytes.
    shards_verified = None
    if world > 1:
        check(l.small_b200_memcpy_h2d(chain.x.data_ptr(), hin, in_bytes, st))
        chain.launch(0)
        chain.stream.synchronize()
        feats = chain.y.numel() // batch
        gathered = sharding.gather_to_host(chain.y.reshape(batch, feats), batch * world, 0)
        if rank == 0:
            shards_verified = 0
            for r in range(world):
                xr = make_input(workload, layers, batch, wl["seed"] + r)
                chain.x.copy_(torch.from_numpy(xr).reshape(-1))
                torch.cuda.synchronize()
                chain.launch(0)
                chain.stream.synchronize()
                mine = chain.y.reshape(batch, feats).cpu()
                shards_verified += int(torch.equal(mine, gathered[r * batch:(r + 1) * batch]))
    if world > 1:
        dist.barrier()
    images_per_round = batch * world * args.steps
    clocks = clk.summary()
    res = {
        "metric": METRIC, "value": images_per_round / (ms * 1e-3), "unit": METRIC, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "ms_per_step_min": ms_min / args.steps, "rounds": rounds, "timed_s": round((span_ms + span_e2e) * 1e-3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"],
        "data": "synthetic (seeded), random-init weights",
        "config": config_of(workload, batch, world),
        "e2e": {"value": images_per_round / (ms_e2e * 1e-3), "unit": METRIC, "h2d_bytes_per_step": in_bytes,
                "d2h_bytes_per_step": out_bytes, "ms_per_step": ms_e2e / args.steps,
                "ms_per_step_min": ms_e2e_min / args.steps, "rounds": rounds_e2e, "h2d_gbs": round(h2d_gbs, 2),
                "h2d_ms_alone": round(in_bytes / (h2d_gbs * 1e9) * 1e3, 4),
                "overlap": "upload of the next batch and download of the previous result overlap the current step "
                           "(three streams, two input buffers read directly by the recorded graphs)"},
        "gpu_launches": chain.kernels_per_step * args.steps * (rounds + rounds_e2e),
        "kernels_per_step": chain.kernels_per_step,
        "clocks": clocks,
    }
    if h2d_all is not None:
        # a step cannot be shorter than its upload at the bandwidth a rank gets when all ranks upload
        bound_ms = in_bytes / (h2d_all["per_rank_min_gbs"] * 1e9) * 1e3
        h2d_all["upload_bound_ms_per_step"] = round(bound_ms, 4)
        h2d_all["upload_bound_value"] = round(batch * world / (max(bound_ms, ms / args.steps) * 1e-3), 1)
        h2d_all["e2e_of_upload_bound"] = round(res["e2e"]["value"] / h2d_all["upload_bound_value"], 3)
        res["e2e"]["all_ranks_uploading"] = h2d_all
    if shards_verified is not None:
        res["host_gather"] = {"shards": world, "shards_bit_identical_to_rank0_recomputation": shards_verified}
    if rank == 0:
        res.update(per_layer_report(chain, layers, batch, wl, clocks, torch, pipes))
    if world > 1:
        dist.barrier()
    if rank == 0 and world == 1 and not args.no_cpu_baseline and workload in ("tinyyolov2", "dscnn"):
        try:
            res["cpu_baseline"] = time_reference(workload, layers, os.cpu_count() or 1)
        except Exception as e:  # the checker library is absent: say so, do not hide it
            res["cpu_baseline"] = {"value": None, "unit": METRIC, "cores": 0, "kind": "reference",
                                   "sample": f"unavailable: {e}"}
    torch.cuda.synchronize()
    check(l.small_b200_free_host(hin)); check(l.small_b200_free_host(hout)); check(l.small_b200_free_host(hout2))
    del chain, y_stage, inputs
    torch.cuda.empty_cache()
    return res


def cpp_boundary_leg():
    """Throughput through the reference's own object API (small::TinyYoloV2<FloatBuffer> built from the
    reference's headers against this platform, BatchScope(64) + InferenceGraph): the driver under
    tests/reference_drivers/_build, when it has been built, with the tensor-core convolution on and
    off.  inferences/s from its 'ms per image' line."""
    exe = os.path.join(ROOT, "tests", "reference_drivers", "_build", "bin", "model_graph")
    if not os.path.exists(exe):
        return {"unavailable": "tests/reference_drivers/_build/bin/model_graph is not built"}
    out = {"api": "small::TinyYoloV2<FloatBuffer>::inference under small::b200::BatchScope(64) + InferenceGraph",
           "note": "the reference's model has no bias and ReLU; same convolution shapes as the benchmark network"}
    for key, flag in (("tensor_cores", "1"), ("cuda_cores_only", "0")):
        try:
            r = subprocess.run([exe, "416", "64", "20"], env=dict(os.environ, SMALL_B200_TENSOR_CORE=flag),
                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
            ms = [float(line.split("graph")[1].split("ms per image")[0]) for line in r.stdout.splitlines()
                  if "images: graph" in line]
            out[key] = {"inferences_per_s": 1e3 / ms[0], "ms_per_image": ms[0], "rc": r.returncode} if ms else \
                {"unavailable": r.stdout[-200:]}
        except Exception as e:
            out[key] = {"unavailable": str(e)}
    return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    env = (torch, dist, world, rank, local)
    pipes = measured_pipes(torch)
    primary = args.workload or "tinyyolov2"
    line = measure_workload(args, primary, env, pipes)
    if rank == 0:
        line["pipes_measured"] = pipes
    if not args.workload:
        # the second half of the metric: DS-CNN uint8, same fields
        other = measure_workload(args, "dscnn", env, pipes)
        line["workloads"] = {"dscnn": other}
        if rank == 0 and world == 1 and not args.no_cpp_boundary:
            line["cpp_boundary"] = cpp_boundary_leg()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_one_layer(args):
    """Launches one layer of the workload alone (after running the chain once so that its input
    holds real activations): the command ncu captures, one kernel class at a time."""
    import torch

    from smallframework_b200 import _lib, networks
    args.workload = args.workload or "tinyyolov2"
    wl = WORKLOADS[args.workload]
    batch = args.batch or 8
    layers = make_layers(args.workload)
    chain = networks.Chain(layers, batch, wl["dtype"], fuse_u8=not args.no_fuse_u8)
    xp = make_input(args.workload, layers, batch, wl["seed"])
    chain.x.copy_(torch.from_numpy(xp).reshape(-1))
    chain.enqueue()
    chain.stream.synchronize()
    idx = [i for i, L in enumerate(layers) if L.get("name") == args.profile_layer]
    if not idx:
        raise SystemExit(f"no layer named {args.profile_layer!r}: " + ", ".join(L["name"] for L in layers))
    i = idx[0]
    io = chain.io_plan()[i]
    if io is None:
        raise SystemExit(f"{args.profile_layer} runs inside its producer's kernel: profile that layer")
    st = chain.stream.cuda_stream
    for _ in range(args.steps):
        chain.enqueue_layer(i, io[0], io[1], st)
    chain.stream.synchronize()
    print(json.dumps({"profile_layer": args.profile_layer, "batch": batch, "launches": args.steps,
                      "device_status": _lib.device_status()}))


def run_layer_sweep(args):
    """The single-layer sweep: the 13 convolutions of YOLOv3-tiny at 416x416, fp32, each built,
    run and timed alone at the given batch (default 256) and charged against its roofline like
    the layers of a network.  Prints one JSON line with a row per layer; it is a report of layer
    times, not an inferences/s figure."""
    import torch

    from smallframework_b200 import networks
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if int(os.environ.get("RANK", "0")) != 0:
        return
    batch = args.batch or 256
    wl = dict(dtype="f32")
    rows, total_ms, total_flops = [], 0.0, 0.0
    pipes = measured_pipes(torch)
    with ClockSampler(0) as clk:
        for layers in networks.yolov3_tiny_convs(seed=3):
            chain = networks.Chain(layers, batch, "f32")
            c, h, w = networks.input_shape(layers)
            g = torch.Generator(device="cuda").manual_seed(3)
            chain.x.copy_(torch.rand(chain.x.numel(), device="cuda", generator=g) * 2 - 1)
            chain.enqueue()
            chain.stream.synchronize()
            rep = per_layer_report(chain, layers, batch, wl, {"sm_mhz": 1965.0}, torch, pipes)
            row = rep["layers"][0]
            L = layers[0]
            row["shape"] = f"{L['C']}->{L['K']} {L['Fh']}x{L['Fw']} @{L['H']}"
            rows.append(row)
            total_ms += row["ms"]
            total_flops += row["tflops"] * row["ms"]
            del chain
            torch.cuda.empty_cache()
    peaks = load_peaks()
    print(json.dumps({
        "workload": f"YOLOv3-tiny convolution layers, fp32, 416x416, batch {batch}, each timed alone",
        "data": "synthetic (seeded): inputs U[-1,1), weights N(0, 0.05)", "dtype": "f32",
        "sum_ms": round(total_ms, 4), "mean_tflops": round(total_flops / total_ms, 2) if total_ms else None,
        "peaks": {"hbm_gbs": peaks["hbm"], "bf16_tflops_burst": peaks["tensor_burst"], "source": peaks["source"]},
        "pipes_measured": pipes,
        "clocks": clk.summary(), "layers": rows}), flush=True)


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of a layer's launch from a one-pass ncu
# capture at the bench size: (layer, batch) -> (bytes, summary under profiles/, date of the capture).
# A capture belongs to the kernel as it was that day; the line reports the provenance with the number.
MEASURED_TRAFFIC = {
    ("conv8", 64): (210.6e6, "conv_tf32x3_kernel_conv8_batch16.md", "2026-11-25"),
}


def kernel_class(chain, i, L, dtype):
    """Which kernel runs layer i (with the layers it absorbs) and what bounds it."""
    follow = chain.absorbed(i)
    if L["op"] == "conv":
        if dtype == "f32":
            if chain.prepared[i] is not None:
                return "conv_tf32x3_kernel (tcgen05 kind::tf32, 3xTF32)" + (" + 2x2 max pool" if follow else ""), "tf32x3"
            name = "conv2d_first_f32_kernel (FFMA)" if L["C"] < 16 else "conv2d_f32_kernel (FFMA)"
            return name + (" + 2x2 max pool" if follow else ""), "ffma"
        if follow:
            tail = "depthwise 3x3 on tcgen05" if len(follow) == 1 else "global average pool + dense"
            return f"block_u8_tc_kernel (tcgen05 kind::i8 {'im2col first layer' if L['C'] == 1 else '1x1'} -> {tail})", "i8"
        pw = (L["Fh"] == 1 and L["Fw"] == 1 and L["stride"] == 1 and L["C"] % 32 == 0 and L["C"] <= 256)
        if pw:
            return "pw_u8_tc_kernel (tcgen05 kind::i8)", "i8"
        ho, wo = networks_out_hw(L)
        if L["C"] == 1 and L["Fw"] <= 4 and L["Fh"] <= 16 and ho * wo <= 128 and L["K"] <= 128:
            return "stem_u8_tc_kernel (im2col in shared memory + tcgen05 kind::i8)", "i8"
        if L["C"] * L["Fh"] * L["Fw"] > 32 or (L["C"] >= 16 and L["K"] >= 32):
            return "conv_u8_ring_kernel (implicit GEMM, tcgen05 kind::i8)", "i8"
        return "conv2d_u8_onestep_kernel (dp4a, streaming)", "stream"
    if L["op"] == "dwconv" and dtype == "u8":
        rows = L["Fh"] == 3 and L["Fw"] == 3 and L["stride"] == 1
        return ("dwconv3x3_u8_rows_kernel (dp4a)" if rows else "dwconv_u8_dp4a_kernel"), "stream"
    return {"dwconv": "window_f32_kernel (depthwise)", "maxpool": "max pool", "avgpool": "average pool",
            "softmax": "softmax", "alias": "alias"}[L["op"]], "stream"


def networks_out_hw(L):
    from smallframework_b200.networks import _out_hw
    return _out_hw(L)


def per_layer_report(chain, layers, batch, wl, clocks, torch, pipes=None):
    """Times every launch of the step alone with CUDA events on the launching stream and charges it
    against its roofline: t_roof = max(flops / pipe peak, bytes / HBM peak).  Pipe peaks are MEASURED on
    this GPU (small_b200_peak_probe): the fp32 FMA pipe for CUDA-core convolutions, one third of the tf32
    tensor rate for the 3xTF32 convolution (three MMAs per product), the i8 tensor rate for uint8
    tensor-core layers.  A launch that runs several layers (a producer and what it absorbs) is charged the
    flops of all of them and the bytes it has to move: the first layer's input, the last one's output, all
    the weights.  fp32 layers at their batch read inputs far larger than L2; the uint8 networks' layers are
    L2-resident here as they are inside a step (see config.l2)."""
    from smallframework_b200 import networks
    peaks = load_peaks()
    if pipes is None:
        pipes = measured_pipes(torch)
    pipe_tops = {"ffma": pipes["ffma"], "tf32x3": pipes["tf32"] / 3.0, "i8": pipes["i8"],
                 "cuda_u8": pipes["ffma"], "stream": pipes["ffma"]}
    elt = chain.elt
    st = chain.stream.cuda_stream
    reps = 5
    rows = []
    plan = chain.io_plan()
    work = {}
    for i, L in enumerate(layers):
        if L["op"] == "alias":
            continue
        if plan[i] is None:
            rows.append({"layer": L.get("name", L["op"]), "kernel": "runs inside " + layers[chain.fused_into[i]]["name"],
                         "ms": 0.0, "tflops": 0.0, "gbs": 0.0, "bound": "fused", "roofline_frac": None})
            continue
        src, dst = plan[i]
        for _ in range(2):
            chain.enqueue_layer(i, src, dst, st)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(chain.stream)
        for _ in range(reps):
            chain.enqueue_layer(i, src, dst, st)
        e1.record(chain.stream)
        chain.stream.synchronize()
        ms = e0.elapsed_time(e1) / reps
        group = [i] + chain.absorbed(i)
        flops = wbytes = 0
        for k in group:
            f, _, w = networks.algorithmic_work(layers[k], elt)
            flops += f
            wbytes += w
        first, last = layers[group[0]], layers[group[-1]]
        ho, wo = networks_out_hw(last)
        abytes = (first["C"] * first["H"] * first["W"] + networks.padded(last["K"]) * ho * wo) * elt
        flops *= batch
        nbytes = abytes * batch + wbytes
        work[len(rows)] = (flops, nbytes)
        kname, kcls = kernel_class(chain, i, L, wl["dtype"])
        t_flop = flops / (pipe_tops[kcls] * 1e12)
        t_mem = nbytes / (peaks["hbm"] * 1e9)
        rows.append({"layer": "+".join(layers[k].get("name", layers[k]["op"]) for k in group), "kernel": kname,
                     "ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 3),
                     "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
                     "bound": ("tensor" if kcls in ("tf32x3", "i8") else "fp32 pipe") if t_flop > t_mem else "hbm",
                     "pipe": kcls, "roofline_frac": round(max(t_flop, t_mem) / (ms * 1e-3), 4)})
    top = max(range(len(rows)), key=lambda i: rows[i]["ms"])
    flops, nbytes = work[top]
    kcls = rows[top]["pipe"]
    traffic = MEASURED_TRAFFIC.get((rows[top]["layer"], batch))
    src = None if traffic is None else {"profile": "profiles/" + traffic[1], "captured": traffic[2]}
    if rows[top]["bound"] != "hbm":
        achieved = flops / (rows[top]["ms"] * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["tensor_burst"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tensor_burst"], "traffic": None if traffic is None else traffic[0],
                "traffic_source": src, "kernel": rows[top]["kernel"], "layer": rows[top]["layer"],
                "peak_source": f"dense bf16 GEMM, burst (the kernel is timed alone), of {peaks['source']}",
                "pipe": {"peak": pipe_tops[kcls], "frac": achieved / pipe_tops[kcls],
                         "note": {"tf32x3": "fp32 result from three tf32 MMAs per product: one third of the tf32 "
                                            "tensor rate measured on this GPU in this run",
                                  "ffma": "fp32 FMA pipe measured on this GPU in this run",
                                  "i8": "i8 tensor rate measured on this GPU in this run"}.get(kcls, "")}}
    else:
        achieved = nbytes / (rows[top]["ms"] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": achieved / peaks["hbm"], "traffic": None if traffic is None else traffic[0],
                "traffic_source": src, "kernel": rows[top]["kernel"],
                "layer": rows[top]["layer"], "peak_source": f"copy bandwidth, of {peaks['source']}"}
    return {"roofline": roof, "layers": rows}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="", choices=[""] + sorted(WORKLOADS) + ["yolov3tiny_layers"],
                    help="default: Tiny-YOLOv2 as the line, DS-CNN under 'workloads'")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="rounds of --steps steps are repeated until this much has been timed, per leg")
    ap.add_argument("--no-cpp-boundary", action="store_true")
    ap.add_argument("--upload-memory", default="pinned", choices=["pinned", "wc"],
                    help="host staging memory of the end-to-end leg's input: pinned, or pinned write-combined")
    ap.add_argument("--no-fuse-u8", action="store_true",
                    help="uint8 networks: one kernel per layer instead of the fused block kernels")
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the configuration's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-layer", default="",
                    help="run only this layer (by name) --steps times on a small batch: the ncu target")
    args = ap.parse_args()
    if args.workload == "yolov3tiny_layers":
        run_layer_sweep(args)
    elif args.profile_layer:
        run_one_layer(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
