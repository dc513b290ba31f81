"""Benchmark of the MSDA hot path (forward + zero-buffer backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2_m2f_1024_bf16] [--batch-per-gpu B] [--repeats R]

A step is one forward plus one backward of the operator over one batch of synthetic input
(Mask2Former pixel-decoder shapes; see deformops_b200/workloads.py).  Metric: queries per
second, fwd+bwd, whole job (all ranks).  One process per GPU; batch-sharded, no collective on
the data path (torch.distributed is used only for the barrier and the max over ranks).

Legs, all inside one run:
  value        inputs resident in HBM, forward and backward launched through the C ABI; K steps
               between one pair of CUDA events on the launching stream, repeated R times back
               to back; the median repeat is reported, min and max beside it.  Consecutive
               steps use different input sets (3 sets rotate), so nothing a step reads is left
               in L2 by the previous one ("inputs larger than L2").
  roofline     per-kernel CUDA-event durations sampled in a second pass over the same steps.
  e2e          the same step through the public operator (registry.msda + autograd) with HOST
               (pinned) input and output buffers, copies inside the timed region; beside it a
               copy-only leg (same copies, no kernels) that shows what the host side allows.
  config4      the scaling configuration: global batch 64 split evenly over the ranks, timed
               the same way (max over ranks); every rank also checks the results on its own
               slice against the reference's CUDA kernel (or the C oracle on one sample when
               that library was not built) and the run fails if a tolerance is exceeded.
  floors       N=1: what kernels reach that only gather the operator's rows, only add into them
               (packed reductions, and the copy engine's bulk reductions), or do both and
               nothing else, on the operator's own addresses; plus the issue rates of
               tensor-core instructions and shared-memory row updates (bench-only library,
               not part of libmsda_b200.so).
  gpu_baseline N=1: the reference's own GPU implementations on this GPU and these inputs - its
               CUDA kernels (production float32-accumulate and 16-bit-atomics builds) and its
               Triton backend - with peak memory beside ours.
  cpu_baseline the reference's eager CPU path on a bounded sample, rank 0 at N=1 only.

``--impl reference`` times only the reference's eager CPU path, on rank 0.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import statistics
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
CONFIG4_GLOBAL_BATCH = 64
E2E_REPEATS = 5        # the end-to-end region is run this many times, the median reported
# stated tolerances, max|a-b| / max|b|: (output, gradients)
TOLERANCES = {torch.float32: (1e-5, 1e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-2, 1e-2)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10,
                    help="how many times the --steps-step timed region is run back to back")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2_m2f_1024_bf16")
    ap.add_argument("--batch-per-gpu", type=int, default=None,
                    help="samples per GPU (default: the workload's batch)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-config4", action="store_true")
    ap.add_argument("--no-floors", action="store_true")
    ap.add_argument("--no-gpu-baseline", action="store_true")
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

    def __init__(self, index: int, period_s: float = 0.002):
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
# The reference's eager CPU path (cpu_baseline and --impl reference)
# ------------------------------------------------------------------------------------------
def reference_package():
    """Import the reference's own package from ``oracle/_ref/py`` (staged by
    ``oracle/build_ref.py`` where a checkout exists); None when it was not staged."""
    from oracle import build_ref

    staged = build_ref.staged_package()
    if staged is None:
        return None
    if str(staged) not in sys.path:
        sys.path.insert(0, str(staged))
    try:
        import deformops  # noqa: F401
        from deformops import registry
    except Exception:  # noqa: BLE001 - an unusable copy counts as absent
        return None
    return registry


def cpu_eager_step(workload_name: str):
    """Returns ``(step, Q, kind, what)``: ``step()`` runs fwd+bwd of ONE sample of the workload
    in float32 through the reference's eager CPU backend (kind "reference"), or through the
    restatement of it in ``oracle/msda_eager_port.py`` when the package is not staged (kind
    "port")."""
    from deformops_b200.workloads import make_workload

    torch.set_num_threads(os.cpu_count() or 1)
    w = make_workload(workload_name, batch=1, first_sample=0)
    Q = w.sampling_locations.shape[1]
    value, loc = w.value.float(), w.sampling_locations
    attn, grad_out = w.attention_weights.float(), w.grad_output.float()
    registry = reference_package()
    if registry is not None:
        def step():
            v, l, a = (t.detach().clone().requires_grad_(True) for t in (value, loc, attn))
            out = registry.msda(v, w.spatial_shapes, w.level_start_index, l, a,
                                backend=registry.Backend.EAGER)
            out.backward(grad_out)
            return out

        return step, Q, "reference", "deformops.registry.msda(backend=EAGER) + autograd"
    from oracle.msda_eager_port import eager_forward_backward

    def step():
        return eager_forward_backward(value, w.spatial_shapes, w.level_start_index, loc, attn, grad_out)

    return step, Q, "port", "torch restatement of the reference's eager CPU path"


def cpu_eager_sample(workload_name: str, target_seconds: float, reps: int = 3):
    """Time fwd+bwd of the eager CPU path on single samples of the workload, float32."""
    step, Q, kind, what = cpu_eager_step(workload_name)
    t0 = time.perf_counter()
    step()  # warm-up, also sizes the sample
    first = time.perf_counter() - t0
    reps = max(1, min(reps, int(target_seconds / max(first, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {
        "value": Q / best, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
        "sample": (f"1 sample of {workload_name} (Q={Q}) in float32, fwd+bwd, {what}, "
                   f"best of {reps} after 1 warm-up"),
        "seconds_per_sample": best,
    }


def workload_config(name, cfg, batch_per_gpu, world, extra=None):
    levels = cfg["levels"]
    out = {"workload": name, "batch_per_gpu": batch_per_gpu,
           "queries": cfg.get("num_queries") or sum(h * w for h, w in levels), "levels": levels,
           "heads": cfg["heads"], "head_dim": cfg["head_dim"], "points": cfg["points"],
           "parallelism": f"batch-sharded x{world}, no collective"}
    out.update(extra or {})
    return out


def run_reference_arm(args):
    """--impl reference: only rank 0 works; each step is one single-sample fwd+bwd on the CPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from deformops_b200.workloads import CONFIGS

    step, Q, kind, what = cpu_eager_step(args.workload)
    steps, warm = max(1, args.steps), max(1, args.warmup)
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = Q / dt
    cfg = CONFIGS[args.workload]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, cfg, args.batch_per_gpu or cfg["batch"],
                                  int(os.environ.get("WORLD_SIZE", "1")),
                                  {"sample": "each step is 1 sample (of the batch) on the host CPU, "
                                             "float32; the value is queries of that sample per second"}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": kind,
                         "sample": f"{steps} steps of 1 sample (Q={Q}) float32 fwd+bwd, {what}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def bind_host_threads(local_rank: int, local_world: int) -> int:
    """Give every rank of a node its own share of the host cores (copies issued by 8 ranks from
    the same cores were one cause of a slow end-to-end leg) and size torch's thread pool to it."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        share = max(1, len(cores) // max(local_world, 1))
        mine = cores[local_rank * share:(local_rank + 1) * share] or cores
        if local_world > 1:
            os.sched_setaffinity(0, mine)
        torch.set_num_threads(max(1, len(mine)))
        return len(mine)
    except (AttributeError, OSError):
        return os.cpu_count() or 1


class AbiCall:
    """Forward and backward of one batch through the C ABI on preallocated buffers."""

    def __init__(self, shim, w, device, local_rank, stream):
        from deformops_b200.ops import DTYPE_CODES

        self.shim, self.local_rank, self.stream = shim, local_rank, stream
        self.sptr = ctypes.c_void_p(stream.cuda_stream)
        self.dims = w.dims
        B, S, G, D, Q, L, K = w.dims
        self.code = DTYPE_CODES[w.value.dtype]
        self.nscratch = shim.scratch_bytes(B, S, G, D, Q, L, K, self.code)
        self.scratch = torch.empty(max(self.nscratch, 16), dtype=torch.uint8, device=device)

    def buffers(self, w, device):
        d = {k: getattr(w, k).to(device) for k in
             ("value", "sampling_locations", "attention_weights", "grad_output")}
        d["shapes"] = w.spatial_shapes.to(device)
        d["starts"] = w.level_start_index.to(device)
        d["out"] = torch.empty(w.grad_output.shape, dtype=w.value.dtype, device=device)
        d["grad_value"] = torch.empty_like(d["value"])
        d["grad_loc"] = torch.empty_like(d["sampling_locations"])
        d["grad_attn"] = torch.empty_like(d["attention_weights"])
        return d

    def forward(self, d):
        B, S, G, D, Q, L, K = self.dims
        st = self.shim.forward(_p(d["value"]), _p(d["shapes"]), _p(d["starts"]),
                               _p(d["sampling_locations"]), _p(d["attention_weights"]),
                               _p(d["out"]), B, S, G, D, Q, L, K, self.code, 0, self.local_rank,
                               self.sptr)
        if st != 0:
            raise RuntimeError(self.shim.last_error())

    def backward(self, d):
        # one call = header memset + prepare kernel + backward kernel + finalize kernel
        B, S, G, D, Q, L, K = self.dims
        st = self.shim.backward(_p(d["value"]), _p(d["shapes"]), _p(d["starts"]),
                                _p(d["sampling_locations"]), _p(d["attention_weights"]),
                                _p(d["grad_output"]), _p(d["grad_value"]), _p(d["grad_loc"]),
                                _p(d["grad_attn"]), _p(self.scratch) if self.nscratch else None,
                                self.nscratch, 0, B, S, G, D, Q, L, K, self.code, 0, 1,
                                self.local_rank, self.sptr)
        if st != 0:
            raise RuntimeError(self.shim.last_error())

    def step(self, d, ev=None):
        self.forward(d)
        if ev:
            ev[1].record(self.stream)
        self.backward(d)


def rel_err(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def parity_vs_reference_cuda(d, dtype):
    """Worst max|a-b|/max|b| of this rank's out / grad_value / grad_loc / grad_attn (already in
    `d`) against the reference's own CUDA kernel run here on the same slice - its float32
    result, which is what the tolerances are stated against.  Falls back to the float64 C
    oracle on the slice's first sample when that library was not built."""
    from oracle import ref_cuda

    ins = (d["value"], d["shapes"], d["starts"], d["sampling_locations"], d["attention_weights"])
    if ref_cuda.available("msda_fp32acc"):
        f32 = [t.float() if t.is_floating_point() else t for t in ins]
        r_out = ref_cuda.forward(*f32)
        r_gv, r_gl, r_ga = ref_cuda.backward(*f32, d["grad_output"].float())
        against = "reference CUDA kernel msda_fp32acc in float32, whole slice"
        got = (d["out"], d["grad_value"], d["grad_loc"], d["grad_attn"])
        loc = d["sampling_locations"]
    else:
        from oracle import msda_oracle as orc

        one = [t[:1].cpu() if t.dim() > 2 else t.cpu() for t in ins]
        r_out = torch.from_numpy(orc.forward(*one))
        r_gv, r_gl, r_ga = (torch.from_numpy(x) for x in orc.backward(*one, d["grad_output"][:1].cpu()))
        against = "float64 C oracle, first sample of the slice"
        got = tuple(d[k][:1].cpu() for k in ("out", "grad_value", "grad_loc", "grad_attn"))
        loc = d["sampling_locations"][:1].cpu()
    # grad_loc is one-sided where a sample lies exactly on a pixel; the float32 rounding of
    # loc*size-0.5 decides the side, so points that close to a pixel are left out of its bar
    wh = torch.flip(d["shapes"], [-1]).to(loc.device).double()[None, None, None, :, None, :]
    pix = loc.double() * wh - 0.5
    keep = ((pix - pix.round()).abs() >= 1e-4).all(-1, keepdim=True)
    errs = {"out": rel_err(got[0], r_out.reshape(got[0].shape)),
            "grad_value": rel_err(got[1], r_gv.reshape(got[1].shape)),
            "grad_loc": rel_err(got[2] * keep, r_gl.reshape(got[2].shape) * keep),
            "grad_attn": rel_err(got[3], r_ga.reshape(got[3].shape))}
    tol_out, tol_grad = TOLERANCES[dtype]
    ok = errs["out"] <= tol_out and all(errs[k] <= tol_grad for k in ("grad_value", "grad_loc", "grad_attn"))
    return errs, ok, against


def timed_steps(fn, steps, stream, barrier, repeats=1):
    """CUDA-event time of `steps` calls of fn(i), `repeats` times back to back; ms per repeat."""
    out = []
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record(stream)
        for i in range(steps):
            fn(i)
        b.record(stream)
        barrier()
        out.append(a.elapsed_time(b))
    return out


def floors_leg(w, device, stream):
    """Throughput of the operator's own gather and reduction addresses through kernels that do
    nothing else, and of back-to-back tensor-core instructions (bench-only library)."""
    from deformops_b200._build import build_floors_library

    lib = ctypes.CDLL(str(build_floors_library()))
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    lib.floors_red_rows.argtypes = [vp, vp, i64, ctypes.c_int, vp]
    lib.floors_red_rows_on.argtypes = [vp, vp, i64, ctypes.c_int, vp]
    lib.floors_bulk_red_rows.argtypes = [vp, vp, i64, ctypes.c_int, vp]
    lib.floors_gather_rows.argtypes = [vp, vp, i64, vp, vp]
    lib.floors_gather_red_rows.argtypes = [vp, vp, vp, i64, ctypes.c_int, ctypes.c_int, vp]
    lib.floors_mma.argtypes = [ctypes.c_int, vp, ctypes.POINTER(i64), vp]
    lib.floors_smem_rmw.argtypes = [ctypes.c_int, ctypes.c_int, vp, ctypes.POINTER(i64), vp]
    B, S, G, D, Q, L, K = w.dims
    loc = w.sampling_locations.to(device)
    shapes, starts = w.spatial_shapes.to(device), w.level_start_index.to(device)
    Hs, Ws = shapes[:, 0].view(1, 1, 1, L, 1), shapes[:, 1].view(1, 1, 1, L, 1)
    x0 = torch.floor(loc[..., 0] * Ws - 0.5).long()
    y0 = torch.floor(loc[..., 1] * Hs - 0.5).long()
    b = torch.arange(B, device=device).view(B, 1, 1, 1, 1)
    g = torch.arange(G, device=device).view(1, 1, G, 1, 1)
    offs, oks = [], []
    for dy in (0, 1):
        for dx in (0, 1):
            x, y = x0 + dx, y0 + dy
            oks.append((x >= 0) & (x < Ws) & (y >= 0) & (y < Hs))
            offs.append(((b * S + starts.view(1, 1, 1, L, 1) + y * Ws + x) * G + g) * D)
    # order of the kernels' own accesses: sample, query, point, corner, head
    off = torch.stack(offs, -1).permute(0, 1, 3, 4, 5, 2)
    ok = torch.stack(oks, -1).permute(0, 1, 3, 4, 5, 2)
    rows = off[ok].to(torch.int32).contiguous()
    n = rows.numel()
    del off, ok, offs, oks
    sp = ctypes.c_void_p(stream.cuda_stream)
    sink = torch.zeros(16, dtype=torch.int32, device=device)
    dst = torch.zeros(B * S * G * D, dtype=torch.float16, device=device)
    src = w.value.to(device).contiguous()

    def median_ms(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        return statistics.median(timed_steps(lambda i: fn(), 1, stream, torch.cuda.synchronize, reps))

    red_ms = median_ms(lambda: lib.floors_red_rows(vp(dst.data_ptr()), vp(rows.data_ptr()), n, 1, sp))
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    red_by_sms = {str(k): n / (median_ms(lambda k=k: lib.floors_red_rows_on(
        vp(dst.data_ptr()), vp(rows.data_ptr()), n, k, sp)) * 1e-3) for k in (sms, sms // 2, sms // 4)}
    if lib.floors_bulk_red_rows(vp(dst.data_ptr()), vp(rows.data_ptr()), n, 1, sp) != 0:
        raise RuntimeError("floors_bulk_red_rows refused its arguments")
    bulk_by_piece = {str(64 * k): n // 8 * 8 / (median_ms(lambda k=k: lib.floors_bulk_red_rows(
        vp(dst.data_ptr()), vp(rows.data_ptr()), n, k, sp)) * 1e-3) for k in (1, 2, 4)}
    gat_ms = median_ms(lambda: lib.floors_gather_rows(vp(src.data_ptr()), vp(rows.data_ptr()), n,
                                                      vp(sink.data_ptr()), sp))
    # with the shared memory the backward kernel holds per CTA at this shape, so that L1 is as small
    from deformops_b200._loader import load_library
    from deformops_b200.ops import DTYPE_CODES

    grid_, threads_, smem_f, smem_b = ctypes.c_int64(), ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64()
    if load_library().launch_geometry(B, G, D, Q, L, K, DTYPE_CODES[w.value.dtype], 0, grid_, threads_,
                                      smem_f, smem_b) != 0:
        raise RuntimeError("launch geometry refused the workload's shape")
    bwd_smem = min(int(smem_b.value), 48 * 1024)
    # rows of one query on average, rounded up to whole instructions of eight rows
    block_rows = (-(-n // (B * Q)) + 7) // 8 * 8
    if lib.floors_gather_red_rows(vp(src.data_ptr()), vp(dst.data_ptr()), vp(rows.data_ptr()), n,
                                  block_rows, bwd_smem, sp) != 0:
        raise RuntimeError("floors_gather_red_rows refused its arguments")
    both_ms = median_ms(lambda: lib.floors_gather_red_rows(vp(src.data_ptr()), vp(dst.data_ptr()),
                                                           vp(rows.data_ptr()), n, block_rows, bwd_smem, sp))
    cnt = i64(0)
    mma_ms = median_ms(lambda: lib.floors_mma(2000, vp(sink.data_ptr()), ctypes.byref(cnt), sp))
    mma_rate = cnt.value / (mma_ms * 1e-3)
    rmw_ms = median_ms(lambda: lib.floors_smem_rmw(2000, 96, vp(sink.data_ptr()), ctypes.byref(cnt), sp))
    rmw_rate = cnt.value / (rmw_ms * 1e-3)
    return {
        "what": "kernels that only issue the operator's gathers / reductions for one call of "
                "this workload (64-byte rows at the addresses of its in-bounds bilinear corners, "
                "in the kernels' order), and back-to-back tensor-core / shared-memory updates",
        "corner_rows": n,
        "gather_rows_ms": gat_ms, "gather_rows_per_s": n / (gat_ms * 1e-3),
        "red_f16x2_rows_ms": red_ms, "red_f16x2_rows_per_s": n / (red_ms * 1e-3),
        "gather_red_rows_ms": both_ms, "gather_red_idle_smem_bytes_per_cta": bwd_smem,
        "red_f16x2_rows_per_s_by_issuing_sms": red_by_sms,
        "bulk_reduce_f16_rows_per_s_by_piece_bytes": bulk_by_piece,
        "mma_m16n8k16_per_s": mma_rate,
        "smem_row_updates_per_s": rmw_rate,
        "reading": "a forward cannot finish before gather_rows_ms; a backward that adds every "
                   "corner row into global memory cannot finish before red_f16x2_rows_ms, nor, as it must "
                   "gather the same rows first, before gather_red_rows_ms; the "
                   "reduction rate falls in proportion to the SMs that issue, so the limit is each "
                   "SM's path to L2 (one 64-byte row in about four cycles), not L2's reduction units; "
                   "the copy engine's bulk reductions leave the SM no faster",
    }


def gpu_baseline_leg(sets, abi, device, stream, iters):
    """The reference's own GPU implementations on this GPU, same rotating inputs: CUDA-event
    time of a forward and of a backward call as a user of that library gets them, and the peak
    of torch-allocated memory during one forward + backward."""
    from oracle import ref_cuda

    B, Q, K = abi.dims[0], abi.dims[4], abi.dims[6]
    sync = torch.cuda.synchronize

    def t5(d):
        return d["value"], d["shapes"], d["starts"], d["sampling_locations"], d["attention_weights"]

    def median_ms(fn):
        for i in range(3):
            fn(sets[i % NUM_SETS])
        return statistics.median(timed_steps(lambda i: fn(sets[i % NUM_SETS]), 1, stream, sync, iters))

    # name -> (forward call, backward call or None, forward+backward call)
    impls = {}
    ours = torch.ops.deformops_b200

    def pair(fwd, bwd):
        def both(d):
            fwd(d)
            bwd(d)
        return fwd, bwd, both

    impls["this library (private torch ops, allocation included)"] = pair(
        lambda d: ours.msda_forward(*t5(d), 128, K, 0, 0),
        lambda d: ours.msda_backward(*t5(d), d["grad_output"], 128, K, 0, 0))
    for prefix in ref_cuda.PREFIXES:
        if ref_cuda.available(prefix):
            impls[f"reference CUDA {prefix}"] = pair(
                lambda d, p=prefix: ref_cuda.forward(*t5(d), prefix=p),
                lambda d, p=prefix: ref_cuda.backward(*t5(d), d["grad_output"], prefix=p))
    registry = reference_package()
    if registry is not None:
        def triton_forward(d):
            with torch.no_grad():
                return registry.msda(*t5(d), backend=registry.Backend.TRITON)

        def triton_both(d):
            v, l, a = (d[k].detach().requires_grad_(True) for k in
                       ("value", "sampling_locations", "attention_weights"))
            out = registry.msda(v, d["shapes"], d["starts"], l, a, backend=registry.Backend.TRITON)
            torch.autograd.grad(out, [v, l, a], d["grad_output"])

        impls["reference Triton (registry.msda backend=TRITON + autograd)"] = (
            triton_forward, None, triton_both)

    rows = {}
    for name, (fwd, bwd, both) in impls.items():
        try:
            f_ms = median_ms(fwd)
            b_ms = median_ms(bwd) if bwd is not None else median_ms(both) - f_ms
            sync()
            torch.cuda.reset_peak_memory_stats(device)
            base = torch.cuda.memory_allocated(device)
            both(sets[0])
            sync()
            peak = torch.cuda.max_memory_allocated(device) - base
            rows[name] = {"forward_ms": f_ms, "backward_ms": b_ms,
                          "fwd_bwd_queries_per_s": B * Q / ((f_ms + b_ms) * 1e-3),
                          "peak_bytes": int(peak)}
        except Exception as exc:  # noqa: BLE001 - a baseline that cannot run is reported, not fatal
            rows[name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    return {"what": "forward call / backward call, median of CUDA-event times, 3 input sets "
                    "rotating (Triton: backward = forward+backward through autograd minus "
                    "forward); peak_bytes = torch max_memory_allocated delta over one forward + "
                    "backward (outputs, gradients and scratch included)",
            "results": rows}


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    from deformops_b200._loader import load_library
    from deformops_b200.registry import Backend, msda
    from deformops_b200.sharding import shard_batch
    from deformops_b200.workloads import CONFIGS, make_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    host_threads = bind_host_threads(local_rank, local_world)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = CONFIGS[args.workload]
    B = args.batch_per_gpu or cfg["batch"]

    # one rank of a node builds a stale library, the others wait for it
    if local_rank == 0:
        load_library()
    barrier()
    shim = load_library()
    stream = torch.cuda.current_stream()

    sets, hosts = [], []
    for r in range(NUM_SETS):
        w = make_workload(args.workload, batch=B, first_sample=(rank * NUM_SETS + r) * B, seed=0)
        if r == 0:
            w0 = w
            abi = AbiCall(shim, w, device, local_rank, stream)
        hosts.append({k: getattr(w, k).pin_memory() for k in
                      ("value", "sampling_locations", "attention_weights", "grad_output")})
        sets.append(abi.buffers(w, device))
    Bq, S, G, D, Q, L, K = w0.dims
    fwd_bytes, bwd_bytes = w0.algorithmic_bytes()
    dtype = w0.value.dtype

    # ---- value: resident inputs, K steps between one pair of events, R repeats -----------------
    for i in range(max(args.warmup, 3)):
        abi.step(sets[i % NUM_SETS])
    with ClockSampler(local_rank) as clocks:
        repeats_ms = timed_steps(lambda i: abi.step(sets[i % NUM_SETS]), args.steps, stream, barrier,
                                 max(1, args.repeats))
        # ---- roofline: per-kernel durations, events around each call, same rotation ------------
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
        barrier()
        for i in range(args.steps):
            evs[i][0].record(stream)
            abi.step(sets[i % NUM_SETS], evs[i])
            evs[i][2].record(stream)
        barrier()
    ms_total = statistics.median(repeats_ms)
    clock_summary = clocks.summary()
    fwd_all = [e[0].elapsed_time(e[1]) for e in evs]
    bwd_all = [e[1].elapsed_time(e[2]) for e in evs]
    fwd_ms, bwd_ms = statistics.mean(fwd_all), statistics.mean(bwd_all)
    spread = {"forward_median": statistics.median(fwd_all), "forward_min": min(fwd_all),
              "backward_call_median": statistics.median(bwd_all), "backward_call_min": min(bwd_all)}

    # ---- e2e: public operator, host buffers, copies inside the timed region --------------------
    e2e = None
    if not args.no_e2e:
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        sink = {"out": torch.empty(sets[0]["out"].shape, dtype=dtype).pin_memory(),
                "grad_value": torch.empty(w0.value.shape, dtype=dtype).pin_memory(),
                "grad_loc": torch.empty(w0.sampling_locations.shape).pin_memory(),
                "grad_attn": torch.empty(w0.attention_weights.shape, dtype=dtype).pin_memory()}
        keys_in = ("value", "sampling_locations", "attention_weights", "grad_output")

        def e2e_step(host, d, compute=True):
            """One step with host buffers.  The batch is walked sample by sample so that the
            upload of sample i+1 (copy stream), the kernels of sample i (caller's stream) and
            the download of sample i-1 (second copy stream) overlap; every byte still crosses
            PCIe inside the timed region.  compute=False: the same copies without the kernels
            (device buffers of the resident leg stand in for the results)."""
            for c in (slice(i, i + 1) for i in range(Bq)):
                with torch.cuda.stream(s_in):
                    ins = [host[k][c].to(device, non_blocking=True) for k in keys_in]
                stream.wait_stream(s_in)
                for t in ins:
                    t.record_stream(stream)
                if compute:
                    v, l, a = (t.requires_grad_(True) for t in ins[:3])
                    out = msda(v, d["shapes"], d["starts"], l, a, backend=Backend.CUDA)
                    out.backward(ins[3])
                    results = (("out", out.detach()), ("grad_value", v.grad), ("grad_loc", l.grad),
                               ("grad_attn", a.grad))
                else:
                    results = tuple((k, d[k][c]) for k in ("out", "grad_value", "grad_loc", "grad_attn"))
                s_out.wait_stream(stream)
                with torch.cuda.stream(s_out):
                    for key, t in results:
                        t.record_stream(s_out)
                        sink[key][c].copy_(t, non_blocking=True)
            stream.wait_stream(s_out)           # the step ends when its results are on the host

        e2e_steps = max(3, min(args.steps, 20))
        for i in range(3):
            e2e_step(hosts[i % NUM_SETS], sets[i % NUM_SETS])
        # the host side (other tenants of the machine, the allocator) makes this leg noisier than
        # the device-timed one: several repeats, the median reported with the spread beside it
        e2e_all = [t / e2e_steps for t in timed_steps(
            lambda i: e2e_step(hosts[i % NUM_SETS], sets[i % NUM_SETS]), e2e_steps, stream, barrier,
            E2E_REPEATS)]
        e2e_ms = statistics.median(e2e_all)
        # the host buffers must hold what the resident path computes for the same inputs
        last = sets[(e2e_steps - 1) % NUM_SETS]
        abi.step(last)
        torch.cuda.synchronize()
        if not (torch.equal(sink["out"], last["out"].cpu())
                and torch.equal(sink["grad_loc"], last["grad_loc"].cpu())):
            raise RuntimeError("e2e leg: results on the host differ from the resident path")
        copy_all = [t / e2e_steps for t in timed_steps(
            lambda i: e2e_step(hosts[i % NUM_SETS], sets[i % NUM_SETS], False), e2e_steps, stream,
            barrier, E2E_REPEATS)]
        copy_ms = statistics.median(copy_all)
        h2d = sum(h.numel() * h.element_size() for h in hosts[0].values())
        d2h = sum(t.numel() * t.element_size() for t in sink.values())
        e2e = {"ms": e2e_ms, "copy_ms": copy_ms, "h2d": h2d, "d2h": d2h, "steps": e2e_steps,
               "ms_all": e2e_all, "copy_all": copy_all}
        del sink

    # ---- config 4: global batch 64 over the ranks, timed and checked per rank --------------------
    config4 = None
    if not args.no_config4 and CONFIG4_GLOBAL_BATCH % world == 0:
        shard = shard_batch(CONFIG4_GLOBAL_BATCH, world, rank)
        count = shard.batch
        w4 = make_workload(args.workload, batch=count, first_sample=10_000 + shard.first_sample, seed=0)
        abi4 = AbiCall(shim, w4, device, local_rank, stream)
        d4 = abi4.buffers(w4, device)
        for _ in range(2):
            abi4.step(d4)
        steps4 = max(3, min(args.steps, 10))
        ms4 = statistics.median(timed_steps(lambda i: abi4.step(d4), steps4, stream, barrier, 3)) / steps4
        errs, ok, against = parity_vs_reference_cuda(d4, dtype)
        f4, b4 = w4.algorithmic_bytes()
        config4 = {"ms": ms4, "errs": errs, "ok": ok, "against": against, "batch_per_gpu": count,
                   "bytes": f4 + b4}
        del d4, abi4, w4
        torch.cuda.empty_cache()

    # ---- caller path: what a deformable-attention layer does around the operator -------------
    # Same sampling pattern, expressed the way a layer holds it: raw logits, reference points
    # and offsets in the value dtype.  (a) torch computes softmax and ref + offsets / (W, H),
    # then the linear operator runs (what the reference's Hugging Face module does);
    # (b) one fused call.  Forward + backward through autograd, resident inputs.
    caller = None
    if world == 1 and not args.no_caller_path:
        from deformops_b200.registry import locations_from_offsets, msda_from_offsets

        d0 = sets[0]
        gen = torch.Generator(device=device).manual_seed(1)
        ref = torch.rand((Bq, Q, L, 2), device=device, generator=gen)
        wh = d0["shapes"].flip(-1).to(torch.float32)[None, None, None, :, None, :]
        offsets = ((d0["sampling_locations"] - ref[:, :, None, :, None, :]) * wh).to(dtype)
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
            caller[name] = timed_steps(lambda i: torch.autograd.grad(fn(), leaves, d0["grad_output"]),
                                       n, stream, torch.cuda.synchronize)[0] / n
        caller["what"] = ("fwd+bwd of softmax + location arithmetic + operator, offsets in the "
                          "value dtype; torch_arithmetic = elementwise passes in torch around "
                          "the linear operator, fused = one msda_from_offsets call")
        del leaves, offsets, ref

    floors = gpu_baseline = None
    if world == 1 and not args.no_floors:
        try:
            floors = floors_leg(w0, device, stream)
        except Exception as exc:  # noqa: BLE001 - the floors are context, not the measurement
            floors = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    if world == 1 and not args.no_gpu_baseline:
        try:
            gpu_baseline = gpu_baseline_leg(sets, abi, device, stream, max(5, min(args.steps, 20)))
        except Exception as exc:  # noqa: BLE001 - the baselines are context, not the measurement
            gpu_baseline = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}

    # ---- max over ranks -------------------------------------------------------------------
    stats = torch.tensor([ms_total, fwd_ms, bwd_ms, e2e["ms"] if e2e else 0.0,
                          e2e["copy_ms"] if e2e else 0.0, config4["ms"] if config4 else 0.0,
                          min(repeats_ms), max(repeats_ms)]
                         + ([config4["errs"][k] for k in ("out", "grad_value", "grad_loc", "grad_attn")]
                            if config4 else [0.0] * 4)
                         + [0.0 if (config4 is None or config4["ok"]) else 1.0],
                         device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    (ms_total, fwd_ms, bwd_ms, e2e_ms, copy_ms, ms4, rep_min, rep_max, e_out, e_gv, e_gl, e_ga,
     parity_failed) = stats.tolist()

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
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {torch.float32: "f32", torch.float16: "f16",
                                           torch.bfloat16: "bf16"}[dtype],
            "data": "synthetic",
            "config": workload_config(args.workload, cfg, Bq, world, {
                "l2": f"{NUM_SETS} input sets rotate between steps (each step touches "
                      f"{(fwd_bytes + bwd_bytes) / 1e6:.0f} MB, L2 is 126 MB); no flush",
                "host_threads_per_rank": host_threads}),
            "repeats": {"count": len(repeats_ms), "ms_per_step_median": ms_per_step,
                        "ms_per_step_min": rep_min / args.steps, "ms_per_step_max": rep_max / args.steps},
            "clocks": clock_summary,
            "gpu_launches": 4 * args.steps,
            "kernels_ms": {"forward": fwd_ms, "backward_call": bwd_ms, **spread,
                           "backward_call_launches": "header memset + prepare, backward and finalize kernels"},
            "roofline": {"bound": "hbm", "kernel": "msda backward (whole call, grad_value clear included)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
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
                           "ms_per_step": e2e_ms, "steps": e2e["steps"], "repeats": E2E_REPEATS,
                           "ms_per_step_repeats_rank0": [round(t, 4) for t in e2e["ms_all"]],
                           "copy_only_ms_per_step_repeats_rank0": [round(t, 4) for t in e2e["copy_all"]],
                           "api": "deformops_b200.registry.msda + autograd, pinned host buffers",
                           "pipeline": "per-sample chunks; upload, kernels and download on three streams",
                           "copy_only_ms_per_step": copy_ms,
                           "copy_only_gbs_per_rank": (e2e["h2d"] + e2e["d2h"]) / (copy_ms * 1e-3) / 1e9,
                           "copy_only_gbs_all_ranks": world * (e2e["h2d"] + e2e["d2h"]) / (copy_ms * 1e-3) / 1e9}
        if config4:
            q4 = CONFIG4_GLOBAL_BATCH * Q
            gbs = config4["bytes"] / (ms4 * 1e-3) / 1e9
            line["config4"] = {
                "what": f"global batch {CONFIG4_GLOBAL_BATCH} of this workload split evenly over the "
                        "ranks, resident inputs, device-timed, max over ranks (strong scaling)",
                "global_batch": CONFIG4_GLOBAL_BATCH, "batch_per_gpu": config4["batch_per_gpu"],
                "ms_per_step": ms4, "value": q4 / (ms4 * 1e-3), "unit": UNIT,
                "hbm_gbs_per_gpu": gbs, "frac_of_peak": gbs / peak, "frac_of_8TBs": gbs / 8000.0}
            line["parity"] = {"against": config4["against"], "max_over_ranks": {
                "out": e_out, "grad_value": e_gv, "grad_loc": e_gl, "grad_attn": e_ga},
                "tolerance": {"out": TOLERANCES[dtype][0], "gradients": TOLERANCES[dtype][1]},
                "ok": parity_failed == 0.0}
        if caller:
            line["caller_path"] = caller
        if floors:
            line["floors"] = floors
        if gpu_baseline:
            line["gpu_baseline"] = gpu_baseline
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_eager_sample(args.workload, args.cpu_seconds)
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.destroy_process_group()
    if parity_failed != 0.0:
        sys.exit(3)


if __name__ == "__main__":
    main()
