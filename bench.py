#!/usr/bin/env python
"""Headline benchmark: VGG-16 forward inference, global batch 256, fp32 semantics
with TF32 tensor-core contractions, on N B200 GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload vgg16|alexnet|resnet50|lstm2] [--math tf32|tf32x3|fp32]

A step is one forward pass of the whole network over the batch (each rank runs
its contiguous slice with replicated weights; for N>1 the step ends with the one
collective of the path, an NCCL all-gather of the logits).  `value` is images/s
with the batch resident in HBM; `e2e` is the same metric through the C-ABI
hand-off calls (nb_network_submit_u8 / nb_network_submit_host + nb_network_wait):
every step copies that step's pinned host batch in -- decoded 8-bit images for
the image networks, as the reference holds them before its float conversion --
and the probabilities out, the copy of step i+1 overlapping the pass of step i.
Inputs and weights are seeded synthetic tensors with ImageNet shapes and value
range (uniform 8-bit images / 255, He-normal weights).

`--impl reference` times the reference's own CPU implementation (the binary
under oracle/_ref, compiled from the reference sources) on a bounded sample of
the same workload on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WEIGHT_SEED, INPUT_SEED = 3000, 3001
UNIT = {"vgg16": "images/s", "alexnet": "images/s", "resnet50": "images/s", "lstm2": "sequences/s"}
DEFAULT_BATCH = {"vgg16": 256, "alexnet": 16, "resnet50": 256, "lstm2": 64}
CPU_SAMPLE = {"vgg16": 8, "alexnet": 16, "resnet50": 16, "lstm2": 8}     # units per CPU-baseline forward


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_burst=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def ncu_traffic(workload: str, math: str, world: int, kernel: str):
    """DRAM bytes per launch of `kernel` from the table of ncu captures (nebula_b200/ncu_traffic.json), or (None, why)."""
    p = ROOT / "nebula_b200" / "ncu_traffic.json"
    if world != 1 or not p.exists():
        return None, "no capture for this configuration"
    for row in json.loads(p.read_text()).get("captures", []):
        if row["workload"] == workload and row["math"] == math and row["kernel"] == kernel:
            return row["dram_bytes_per_launch"], row["source"]
    return None, "no capture for this configuration"


def make_workload(name: str, batch: int):
    from nebula_b200 import workloads
    return workloads.WORKLOADS[name](batch=batch)


# ----------------------------------------------------------------- CPU baseline
def run_cpu_reference(wl_name: str, reps: int, warm: int):
    """Times network_t::forward() of the compiled reference (OpenBLAS build, all
    host cores) on a bounded sample of the workload.  Returns a dict or raises."""
    import numpy as np
    from oracle import oracle as O
    flavour = "oblas" if O.ref_binary("oblas") else ("custom" if O.ref_binary("custom") else None)
    sample = CPU_SAMPLE[wl_name]
    wl = make_workload(wl_name, sample)
    cores = os.cpu_count() or 1
    w = wl.make_weights(WEIGHT_SEED)
    x = wl.make_input(INPUT_SEED)
    if flavour is None:
        # no compiled reference on this machine: time the plain-C restatement instead
        O.lib().nbo_set_threads(min(cores, 64))
        times = []
        for _ in range(warm + reps):
            t0 = time.perf_counter()
            O.forward_network(wl.cfg, w, x)
            times.append((time.perf_counter() - t0) * 1e3)
        kind, used = "port", min(cores, 64)
    else:
        _, info = O.run_reference(wl.cfg, w, x, recurrent=wl.recurrent, flavour=flavour, threads=min(cores, 64),
                                  reps=warm + reps)
        times = info["forward_ms"]
        kind, used = "reference", info["threads"]
    timed = times[warm:]
    ms = statistics.median(timed)
    return dict(value=sample / (ms / 1e3), ms_per_step=ms, cores=used, kind=kind,
                sample=f"{sample} {wl.unit} of {wl_name} per forward, median of {len(timed)} timed forward() calls "
                       f"after {warm} warm-up, {'OpenBLAS 0.3.15' if flavour == 'oblas' else 'in-tree GEMM'} build",
                unit=UNIT[wl_name])


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl_name = args.workload
    batch = args.batch or DEFAULT_BATCH[wl_name]
    try:
        r = run_cpu_reference(wl_name, max(1, args.steps), max(0, args.warmup))
    except Exception as e:  # the checker could not be built or run here
        print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
        return
    line = {
        "impl": "reference", "metric": f"{wl_name} forward inference throughput", "value": round(r["value"], 3),
        "unit": r["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(r["ms_per_step"], 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{wl_name}_b{batch}", "global_batch": batch, "note": "reference CPU path on host cores"},
        "cpu_baseline": {"value": round(r["value"], 3), "unit": r["unit"], "cores": r["cores"], "kind": r["kind"],
                         "sample": r["sample"]},
        "e2e": {"value": round(r["value"], 3), "unit": r["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------- GPU arm
def gpu_arm(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from nebula_b200 import api, sharding

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    wl_name = args.workload
    batch = args.batch or DEFAULT_BATCH[wl_name]
    lo, hi = sharding.shard_bounds(batch, world, rank)
    my = hi - lo
    if my == 0:
        raise SystemExit(f"rank {rank} has no units: global batch {batch} < world size {world}")
    full = make_workload(wl_name, batch)
    wl = full.with_batch(my)

    handle = api.Handle(local, args.math)
    net = api.Network(handle, wl.cfg)
    weights = full.make_weights(WEIGHT_SEED)
    net.load_weights(weights)
    del weights
    images = not full.recurrent
    if images:
        # decoded 8-bit images [B,H,W,C] (BGR), and the reference's float conversion of the same images
        # (models/networks/convolutional.cc:386-398) for the device-resident leg: both legs compute the same thing
        Bf, Cf, Hf, Wf = full.input_shape
        u8_full = np.random.default_rng(INPUT_SEED).integers(0, 256, size=(Bf, Hf, Wf, Cf), dtype=np.uint8)
        u8 = np.ascontiguousarray(u8_full[lo:hi])
        del u8_full
        x_host = (u8.astype(np.float64) / 255.0).astype(np.float32).transpose(0, 3, 1, 2)
        x_host = np.ascontiguousarray(x_host[:, ::-1] if Cf == 3 else x_host)
        x_pin = torch.from_numpy(u8).pin_memory()
    else:
        x_host_full = full.make_input(INPUT_SEED)
        x_host = sharding.shard_input(x_host_full, world, rank, full.recurrent)
        del x_host_full
        x_pin = torch.from_numpy(x_host).pin_memory()
    x_dev = torch.from_numpy(x_host).to(dev)
    out_pins = [torch.empty(net.output_size, dtype=torch.float32).pin_memory() for _ in range(2)]
    classes = full.classes
    rows = net.logits_size // classes
    pending = []        # logits all-gathers in flight (they overlap the next step's pass)

    def gather_logits():
        """The one collective of the path, started behind the pass and not waited for until two steps later."""
        lg = net.logits(device=dev).view(rows, classes)
        if full.recurrent:
            lg = lg.view(-1, my, classes).permute(1, 0, 2).reshape(my, -1).contiguous()
        pending.append(sharding.gather_rows(lg, batch, world, rank, async_op=True))
        while len(pending) > 2:
            pending.pop(0).wait()

    def drain():
        while pending:
            pending.pop(0).wait()

    def step_device():
        net.forward(x_dev)
        if world > 1:
            gather_logits()

    step_no = [0]

    def step_host():
        out = out_pins[step_no[0] & 1]
        step_no[0] += 1
        if images:
            net.submit_u8(x_pin, out)
        else:
            net.submit_host(x_pin, out)
        if world > 1:
            gather_logits()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        net.wait()          # pipelined submissions: every output is in host memory
        drain()             # ... and every gather has finished (the waits are stream-side)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    W, K = max(3, args.warmup), max(1, args.steps)
    # N > 1: a pass is a few dozen launches of a millisecond or two in total, so it is replayed as one CUDA graph and
    # the per-kernel event timing (which needs the kernels launched one by one) runs as a second region of K steps.
    # N = 1: one region, kernels launched one by one with their event pairs, value and roofline from the same steps.
    separate_profile = world > 1
    net.set_graph(separate_profile)
    for _ in range(W):
        step_device()
    drain()
    handle.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = handle.launch_count()
    if not separate_profile:
        handle.profile_begin()
    total_ms = timed(step_device, K)
    launches = handle.launch_count() - launches0
    if separate_profile:
        handle.profile_begin()
        timed(step_device, K)
    prof = handle.profile_end()
    clocks = sampler.stop() if rank == 0 else None
    handle.synchronize()

    for _ in range(3):
        step_host()
    net.wait()
    drain()
    e2e_ms = timed(step_host, K)
    handle.synchronize()

    if world > 1:
        t = torch.tensor([float(launches)], device=dev, dtype=torch.float64)
        dist.all_reduce(t)
        launches = int(t.item())

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = total_ms / K
        value = batch / (ms_per_step / 1e3)
        e2e = batch / (e2e_ms / K / 1e3)
        # dominant kernel: the tcgen05 contraction (all convolutions with C >= 32 and the FC layers)
        tf32_peak = peaks["bf16_sustained"] / 2.0
        if args.math == "tf32x3":
            tf32_peak /= 3.0
        # dominant kernel: whichever tensor-core contraction kernel took more device time in the timed region
        kernels = {"gemm_tf32_tcgen05_kernel": ("tc_ms", "tc_flops", "tc_launches"),
                   "conv3x3_halo_tcgen05_kernel": ("halo_ms", "halo_flops", "halo_launches")}
        dom = max(kernels, key=lambda k: prof[kernels[k][0]])
        other = [k for k in kernels if k != dom][0]
        d_ms, d_fl, d_n = (prof[f] for f in kernels[dom])
        o_ms, o_fl, o_n = (prof[f] for f in kernels[other])
        achieved = d_fl / (d_ms / 1e3) / 1e12 if d_ms > 0 else 0.0
        # dram__bytes_read + dram__bytes_write per launch of the dominant kernel: not something a run can measure on
        # itself; taken from the table of ncu captures kept with the package (null when this workload has none)
        traffic, traffic_source = ncu_traffic(f"{wl_name}_b{batch}", args.math, world, dom)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            try:
                cpu = run_cpu_reference(wl_name, 2, 1)
                cpu = {"value": round(cpu["value"], 3), "unit": cpu["unit"], "cores": cpu["cores"], "kind": cpu["kind"],
                       "sample": cpu["sample"]}
            except Exception as e:
                cpu = {"value": None, "unit": UNIT[wl_name], "cores": 0, "kind": "port",
                       "sample": f"unavailable: {type(e).__name__}: {e}"[:200]}
        line = {
            "metric": f"{wl_name} forward inference throughput", "value": round(value, 2), "unit": UNIT[wl_name],
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"tf32": "tf32", "tf32x3": "3xtf32", "fp32": "f32"}[args.math], "data": "synthetic",
            "config": {"workload": f"{wl_name}_b{batch}", "global_batch": batch, "per_gpu_batch": my,
                       "parallelism": f"batch-sharded replicas x{world}, logits all-gather" if world > 1 else "single GPU",
                       "l2": "inputs and activations larger than L2 (no flush needed)",
                       "storage": "fp32, NHWC internal"},
            "e2e": {"value": round(e2e, 2), "unit": UNIT[wl_name],
                    "h2d_bytes_per_step": int(x_pin.numel() * x_pin.element_size() * world),
                    "d2h_bytes_per_step": int(out_pins[0].numel() * 4 * world),
                    "input": "decoded 8-bit images, pinned" if images else "fp32 sequences, pinned",
                    "api": "nb_network_submit_u8 + nb_network_wait" if images else "nb_network_submit_host + nb_network_wait",
                    "pipelined": "copy of step i+1 overlaps the pass of step i (two device input slots)"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(tf32_peak, 1), "unit": "TFLOP/s",
                         "frac": round(achieved / tf32_peak, 4) if tf32_peak else None, "traffic": traffic,
                         "traffic_unit": "bytes per launch (ncu dram read+write)", "traffic_source": traffic_source,
                         "timed_in": "a second region of the same K steps, kernels launched one by one" if separate_profile
                                     else "the region `value` comes from",
                         "kernel": dom,
                         "launches_per_step": d_n / K, "kernel_ms_per_step": round(d_ms / K, 4),
                         "other_tensor_kernel": {"kernel": other, "launches_per_step": o_n / K,
                                                 "ms_per_step": round(o_ms / K, 4),
                                                 "achieved": round(o_fl / (o_ms / 1e3) / 1e12, 2) if o_ms > 0 else 0.0},
                         "all_tensor_kernels": {"ms_per_step": round((d_ms + o_ms) / K, 4),
                                                "achieved": round((d_fl + o_fl) / ((d_ms + o_ms) / 1e3) / 1e12, 2)
                                                if d_ms + o_ms > 0 else 0.0},
                         "peak_source": f"{peaks['source']}: bf16 cuBLAS sustained {peaks['bf16_sustained']} TFLOP/s / 2 "
                                        "(dense TF32 rate is half the bf16 rate)" + (" / 3 products" if args.math == "tf32x3" else ""),
                         "other_contraction_ms_per_step": round(prof["simt_ms"] / K, 4)},
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    net.close()
    handle.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="nebula_b200", choices=["nebula_b200", "reference"])
    ap.add_argument("--workload", default="vgg16", choices=list(UNIT))
    ap.add_argument("--batch", type=int, default=0, help="global batch (default: the benchmark configuration's)")
    ap.add_argument("--math", default="tf32", choices=["tf32", "tf32x3", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
