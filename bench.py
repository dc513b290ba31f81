"""Benchmark of the MSDA hot path (forward + zero-buffer backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2_m2f_1024_bf16] [--batch-per-gpu B]

A step is one forward plus one backward of the operator over one batch of synthetic input
(Mask2Former pixel-decoder shapes; see deformops_b200/workloads.py).  Metric: queries per
second, fwd+bwd, whole job (all ranks).  One process per GPU; batch-sharded, no collective on
the data path (torch.distributed is used only for the barrier and the max over ranks).

Legs, all inside one run:
  value     inputs resident in HBM, forward and backward launched through the C ABI,
            timed with CUDA events on the launching stream around exactly K steps.
            Consecutive steps use different input sets (3 sets rotate), so nothing a step
            reads is left in L2 by the previous one ("inputs larger than L2").
  roofline  per-kernel CUDA-event durations sampled inside the same timed region.
  e2e       the same step through the public operator (registry.msda + autograd) with HOST
            (pinned) input and output buffers; copies inside the timed region.
  cpu_baseline  the CPU restatement of the reference's eager PyTorch path on a bounded
            sample, rank 0 at N=1 only.

``--impl reference`` times only the CPU restatement (the reference has no GPU-free binary
to ship; its eager CPU path is Python on torch), on rank 0.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "MSDA fwd+bwd queries/sec"
UNIT = "queries/s"
NUM_SETS = 3  # rotating input sets


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2_m2f_1024_bf16")
    ap.add_argument("--batch-per-gpu", type=int, default=None,
                    help="samples per GPU (default: the workload's batch)")
    ap.add_argument("--global-batch", type=int, default=None,
                    help="fixed global batch split evenly over the GPUs (strong scaling)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-sequential", action="store_true",
                    help="e2e leg without overlap: upload, compute, download one after another")
    ap.add_argument("--no-scratch", action="store_true",
                    help="backward without the replica scratch (every level adds straight into grad_value)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-caller-path", action="store_true",
                    help="skip the leg that times the layer-level call (fused vs torch arithmetic)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0,
                    help="target CPU time of the cpu_baseline sample")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs
    (read-only queries, every few milliseconds, from a helper thread)."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
               "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].strip().isdigit():
                    phys = int(ids[self.index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
            self._thread = threading.Thread(target=self._pump, daemon=True)
            self._thread.start()
        except Exception:  # noqa: BLE001 - no NVML: the summary says "unsampled"
            self._thread = None
        return self

    def _pump(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"], "samples": 0}
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


# ------------------------------------------------------------------------------------------
# CPU restatement of the reference's eager path (cpu_baseline and --impl reference)
# ------------------------------------------------------------------------------------------
def cpu_eager_sample(workload_name: str, target_seconds: float, reps: int = 3):
    """Time fwd+bwd of the eager restatement on single samples of the workload, float32."""
    from deformops_b200.workloads import make_workload
    from oracle.msda_eager_port import eager_forward_backward

    torch.set_num_threads(os.cpu_count() or 1)
    w = make_workload(workload_name, batch=1, first_sample=0)
    Q = w.sampling_locations.shape[1]
    args = (w.value.float(), w.spatial_shapes, w.level_start_index, w.sampling_locations,
            w.attention_weights.float(), w.grad_output.float())
    t0 = time.perf_counter()
    eager_forward_backward(*args)  # warm-up, also sizes the sample
    first = time.perf_counter() - t0
    reps = max(1, min(reps, int(target_seconds / max(first, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        eager_forward_backward(*args)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {
        "value": Q / best, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
        "sample": (f"1 sample of {workload_name} (Q={Q}) in float32, fwd+bwd, torch eager "
                   f"restatement of the reference's CPU path, best of {reps} after 1 warm-up"),
        "seconds_per_sample": best,
    }


def run_reference_arm(args):
    """--impl reference: only rank 0 works; each step is one single-sample fwd+bwd on the CPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from deformops_b200.workloads import CONFIGS, make_workload
    from oracle.msda_eager_port import eager_forward_backward

    torch.set_num_threads(os.cpu_count() or 1)
    w = make_workload(args.workload, batch=1)
    Q = w.sampling_locations.shape[1]
    a = (w.value.float(), w.spatial_shapes, w.level_start_index, w.sampling_locations,
         w.attention_weights.float(), w.grad_output.float())
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 1))
    for _ in range(warm):
        eager_forward_backward(*a)
    t0 = time.perf_counter()
    for _ in range(steps):
        eager_forward_backward(*a)
    dt = (time.perf_counter() - t0) / steps
    value = Q / dt
    cfg = CONFIGS[args.workload]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "levels": cfg["levels"], "heads": cfg["heads"],
                   "head_dim": cfg["head_dim"], "points": cfg["points"],
                   "sample": "1 sample per step on the host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": "port",
                         "sample": f"{steps} steps of 1 sample (Q={Q}) float32 fwd+bwd, torch eager "
                                   "restatement of the reference's CPU path"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    from deformops_b200._loader import load_library
    from deformops_b200.ops import DTYPE_CODES, launch_counter
    from deformops_b200.registry import Backend, msda
    from deformops_b200.workloads import CONFIGS, make_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = CONFIGS[args.workload]
    if args.global_batch is not None:
        assert args.global_batch % world == 0
        B = args.global_batch // world
        scaling = "strong"
    else:
        B = args.batch_per_gpu or cfg["batch"]
        scaling = "weak"

    shim = load_library()
    sets = []
    for r in range(NUM_SETS):
        w = make_workload(args.workload, batch=B, first_sample=(rank * NUM_SETS + r) * B, seed=0)
        host = {k: getattr(w, k).pin_memory() for k in
                ("value", "sampling_locations", "attention_weights", "grad_output")}
        d = {k: v.to(device, non_blocking=True) for k, v in host.items()}
        d["shapes"] = w.spatial_shapes.to(device)
        d["starts"] = w.level_start_index.to(device)
        d["out"] = torch.empty(w.grad_output.shape, dtype=w.value.dtype, device=device)
        d["grad_value"] = torch.empty_like(d["value"])
        d["grad_loc"] = torch.empty_like(d["sampling_locations"])
        d["grad_attn"] = torch.empty_like(d["attention_weights"])
        sets.append((w, host, d))
    w0 = sets[0][0]
    Bq, S, G, D, Q, L, K = w0.dims
    fwd_bytes, bwd_bytes = w0.algorithmic_bytes()
    code = DTYPE_CODES[w0.value.dtype]
    stream = torch.cuda.current_stream()
    sptr = ctypes.c_void_p(stream.cuda_stream)

    # scratch for the replica accumulators of a 16-bit grad_value (see msda_b200_backward)
    nscratch = 0 if args.no_scratch else shim.scratch_bytes(Bq, S, G, D, Q, L, K, code)
    scratch = torch.empty(max(nscratch // 4, 1), dtype=torch.float32, device=device)
    scr = _p(scratch) if nscratch else None

    def abi_step(d, ev=None):
        st = shim.forward(_p(d["value"]), _p(d["shapes"]), _p(d["starts"]),
                          _p(d["sampling_locations"]), _p(d["attention_weights"]), _p(d["out"]),
                          Bq, S, G, D, Q, L, K, code, 0, local_rank, sptr)
        if ev:
            ev[1].record(stream)
        # one call = clear (memset, or the prepare kernel) + backward kernel (+ finalize kernel)
        st |= shim.backward(_p(d["value"]), _p(d["shapes"]), _p(d["starts"]),
                            _p(d["sampling_locations"]), _p(d["attention_weights"]),
                            _p(d["grad_output"]), _p(d["grad_value"]), _p(d["grad_loc"]),
                            _p(d["grad_attn"]), scr, nscratch, 0, Bq, S, G, D, Q, L, K, code, 0, 1,
                            local_rank, sptr)
        if st != 0:
            raise RuntimeError(shim.last_error())

    # ---- value: resident inputs, K steps between one pair of events --------------------
    for i in range(args.warmup):
        abi_step(sets[i % NUM_SETS][2])
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        start.record(stream)
        for i in range(args.steps):
            abi_step(sets[i % NUM_SETS][2])
        stop.record(stream)
        barrier()
    ms_total = start.elapsed_time(stop)
    clock_summary = clocks.summary()

    # ---- roofline: per-kernel durations, events around each launch, same rotation ---------
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        evs[i][0].record(stream)
        abi_step(sets[i % NUM_SETS][2], evs[i])
        evs[i][2].record(stream)
    barrier()
    fwd_all = [e[0].elapsed_time(e[1]) for e in evs]
    bwd_all = [e[1].elapsed_time(e[2]) for e in evs]
    fwd_ms, bwd_ms = statistics.mean(fwd_all), statistics.mean(bwd_all)
    spread = {"forward_median": statistics.median(fwd_all), "forward_min": min(fwd_all),
              "backward_call_median": statistics.median(bwd_all), "backward_call_min": min(bwd_all)}

    # ---- e2e: public operator, host buffers, copies inside the timed region --------------
    e2e = None
    if not args.no_e2e:
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

        def e2e_step(host, d, sink):
            """One step through the public operator with host buffers.  The batch is walked
            sample by sample so that the upload of sample i+1 (copy stream), the kernels of
            sample i (caller's stream) and the download of sample i-1 (second copy stream)
            overlap; every byte still crosses PCIe inside the timed region."""
            if args.e2e_sequential:
                chunks = [slice(0, Bq)]
            else:
                chunks = [slice(i, i + 1) for i in range(Bq)]
            for c in chunks:
                with torch.cuda.stream(s_in):
                    ins = [host[k][c].to(device, non_blocking=True) for k in
                           ("value", "sampling_locations", "attention_weights", "grad_output")]
                stream.wait_stream(s_in)
                for t in ins:
                    t.record_stream(stream)
                v, l, a = (t.requires_grad_(True) for t in ins[:3])
                out = msda(v, d["shapes"], d["starts"], l, a, backend=Backend.CUDA)
                out.backward(ins[3])
                s_out.wait_stream(stream)
                with torch.cuda.stream(s_out):
                    for key, t in (("out", out.detach()), ("grad_value", v.grad),
                                   ("grad_loc", l.grad), ("grad_attn", a.grad)):
                        t.record_stream(s_out)
                        sink[key][c].copy_(t, non_blocking=True)
            stream.wait_stream(s_out)           # the step ends when its results are on the host

        sink = {"out": torch.empty(sets[0][2]["out"].shape, dtype=w0.value.dtype).pin_memory(),
                "grad_value": torch.empty(w0.value.shape, dtype=w0.value.dtype).pin_memory(),
                "grad_loc": torch.empty(w0.sampling_locations.shape).pin_memory(),
                "grad_attn": torch.empty(w0.attention_weights.shape, dtype=w0.value.dtype).pin_memory()}
        e2e_steps = max(3, min(args.steps, 20))
        for i in range(3):
            e2e_step(sets[i % NUM_SETS][1], sets[i % NUM_SETS][2], sink)
        barrier()
        launch_counter.reset()
        s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record(stream)
        for i in range(e2e_steps):
            e2e_step(sets[i % NUM_SETS][1], sets[i % NUM_SETS][2], sink)
        t2.record(stream)
        barrier()
        e2e_ms = s2.elapsed_time(t2) / e2e_steps
        # the host buffers must hold what the resident path computes for the same inputs
        last = sets[(e2e_steps - 1) % NUM_SETS][2]
        abi_step(last)
        torch.cuda.synchronize()
        if not (torch.equal(sink["out"], last["out"].cpu())
                and torch.equal(sink["grad_loc"], last["grad_loc"].cpu())):
            raise RuntimeError("e2e leg: results on the host differ from the resident path")
        h2d = sum(h.numel() * h.element_size() for h in sets[0][1].values())
        d2h = sum(t.numel() * t.element_size() for t in sink.values())
        e2e = {"ms": e2e_ms, "h2d": h2d, "d2h": d2h, "steps": e2e_steps}

    # ---- caller path: what a deformable-attention layer does around the operator -------------
    # Same sampling pattern, expressed the way a layer holds it: raw logits, reference points
    # and offsets in the value dtype.  (a) torch computes softmax and ref + offsets / (W, H),
    # then the linear operator runs (what the reference's Hugging Face module does);
    # (b) one fused call.  Forward + backward through autograd, resident inputs.
    caller = None
    if world == 1 and not args.no_caller_path:
        from deformops_b200.registry import locations_from_offsets, msda_from_offsets

        d0 = sets[0][2]
        gen = torch.Generator(device=device).manual_seed(1)
        ref = torch.rand((Bq, Q, L, 2), device=device, generator=gen)
        wh = d0["shapes"].flip(-1).to(torch.float32)[None, None, None, :, None, :]
        offsets = ((d0["sampling_locations"] - ref[:, :, None, :, None, :]) * wh).to(w0.value.dtype)
        leaves = [d0["value"].detach().clone().requires_grad_(),
                  offsets.requires_grad_(),
                  d0["attention_weights"].detach().clone().requires_grad_()]

        def torch_arithmetic():
            v, off, logits = leaves
            weights = torch.softmax(logits, -1)
            loc = locations_from_offsets(ref, off, d0["shapes"])
            return msda(v, d0["shapes"], d0["starts"], loc, weights)

        def fused():
            v, off, logits = leaves
            return msda_from_offsets(v, d0["shapes"], d0["starts"], ref, off, logits, softmax=True)

        caller = {}
        for name, fn in (("torch_arithmetic_ms", torch_arithmetic), ("fused_ms", fused)):
            n = max(3, min(args.steps, 20))
            for _ in range(3):
                torch.autograd.grad(fn(), leaves, d0["grad_output"])
            torch.cuda.synchronize()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record(stream)
            for _ in range(n):
                torch.autograd.grad(fn(), leaves, d0["grad_output"])
            c1.record(stream)
            torch.cuda.synchronize()
            caller[name] = c0.elapsed_time(c1) / n
        caller["what"] = ("fwd+bwd of softmax + location arithmetic + operator, offsets in the "
                          "value dtype; torch_arithmetic = elementwise passes in torch around "
                          "the linear operator, fused = one msda_from_offsets call")
        del leaves, offsets, ref

    # ---- max over ranks -------------------------------------------------------------------
    stats = torch.tensor([ms_total, fwd_ms, bwd_ms, e2e["ms"] if e2e else 0.0],
                         device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_total, fwd_ms, bwd_ms, e2e_ms = stats.tolist()

    if rank == 0:
        ms_per_step = ms_total / args.steps
        queries = world * Bq * Q
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peak, peak_kind = json.loads(peaks_file.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_kind = 6650.0, "fallback"
        traffic = None
        tfile = ROOT / "profiles" / "dram_traffic.json"
        if tfile.exists():
            entry = json.loads(tfile.read_text()).get("msda_backward", {})
            per_query = entry.get("dram_bytes_per_query")
            if per_query:
                traffic = per_query * Bq * Q
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": queries / (ms_per_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": {0: "f32", 1: "f16", 2: "bf16"}[code],
            "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": Bq, "queries": Q,
                       "levels": cfg["levels"], "heads": G, "head_dim": D, "points": K,
                       "l2": f"{NUM_SETS} input sets rotate between steps (each step touches "
                             f"{(fwd_bytes + bwd_bytes) / 1e6:.0f} MB, L2 is 126 MB); no flush",
                       "parallelism": f"batch-sharded x{world}, no collective"},
            "clocks": clock_summary,
            "gpu_launches": (4 if nscratch else 2) * args.steps,
            "kernels_ms": {"forward": fwd_ms, "backward_call": bwd_ms, **spread,
                           "backward_call_launches": ("prepare + backward + finalize kernels"
                                                      if nscratch else "memset + backward kernel")},
            "roofline": {"bound": "hbm", "kernel": "msda backward (whole call, grad_value clear included)", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "traffic": traffic,
                         "algorithmic_bytes": bwd_bytes,
                         "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                     "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                                     "algorithmic_bytes": fwd_bytes},
                         "fwd_bwd_vs_8TBs": (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 8e12},
        }
        if e2e:
            line["e2e"] = {"value": queries / (e2e_ms * 1e-3), "unit": UNIT,
                           "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                           "ms_per_step": e2e_ms, "steps": e2e["steps"],
                           "api": "deformops_b200.registry.msda + autograd, pinned host buffers",
                           "pipeline": ("whole batch, no overlap" if args.e2e_sequential else
                                        "per-sample chunks; upload, kernels and download on "
                                        "three streams")}
        if caller:
            line["caller_path"] = caller
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_eager_sample(args.workload, args.cpu_seconds)
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
