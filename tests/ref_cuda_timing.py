"""TEST INFRASTRUCTURE - time the reference's own CUDA kernels on this GPU, beside ours.

Not collected by pytest.  Usage on a GPU box where ``oracle/_ref`` has been built:

    python tests/ref_cuda_timing.py [--workload cfg2_m2f_1024_bf16] [--iters 20] [--out FILE]

For each implementation it reports CUDA-event times of the forward call and of the backward
call as a user of that library gets them (the reference's production configuration includes
its float32 upcasts, its zero-filled outputs and its cast-back passes, exactly as its
autograd closure performs them: ``_msda_bridge.py:232-259``, ``msda_launch.cuh:188-273``).
Three input sets rotate so that no step finds its inputs in L2.
"""

from __future__ import annotations

import argparse
import json
import pathlib
import statistics
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2_m2f_1024_bf16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    from deformops_b200.workloads import make_workload
    from oracle import ref_cuda

    dev = torch.device("cuda", 0)
    sets = []
    for r in range(3):
        w = make_workload(args.workload, first_sample=r * 16)
        sets.append(dict(value=w.value.to(dev), shapes=w.spatial_shapes.to(dev),
                         starts=w.level_start_index.to(dev), loc=w.sampling_locations.to(dev),
                         attn=w.attention_weights.to(dev), go=w.grad_output.to(dev)))
    B, S, G, D, Q, L, K = w.dims

    def timed(fn):
        for i in range(3):
            fn(sets[i % 3])
        torch.cuda.synchronize()
        ts = []
        for i in range(args.iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(sets[i % 3])
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    def t5(s):
        return s["value"], s["shapes"], s["starts"], s["loc"], s["attn"]

    import deformops_b200  # noqa: F401  (registers torch.ops.deformops_b200)

    ours = torch.ops.deformops_b200
    impls = {"ours": (lambda s: ours.msda_forward(*t5(s), 128, K, 0, 0),
                      lambda s: ours.msda_backward(*t5(s), s["go"], 128, K, 0, 0))}
    for prefix in ref_cuda.PREFIXES:
        if ref_cuda.available(prefix):
            impls[f"reference {prefix}"] = (
                lambda s, p=prefix: ref_cuda.forward(*t5(s), prefix=p),
                lambda s, p=prefix: ref_cuda.backward(*t5(s), s["go"], prefix=p))
    rows = {}
    for name, (fwd, bwd) in impls.items():
        f_ms, b_ms = timed(fwd), timed(bwd)
        rows[name] = {"forward_ms": f_ms, "backward_ms": b_ms,
                      "fwd_bwd_queries_per_s": B * Q / ((f_ms + b_ms) * 1e-3)}
        print(f"{name:32s} fwd {f_ms:8.3f} ms   bwd {b_ms:8.3f} ms   "
              f"{rows[name]['fwd_bwd_queries_per_s'] / 1e6:8.2f} M queries/s")
    result = {"workload": args.workload, "dims": dict(B=B, S=S, G=G, D=D, Q=Q, L=L, K=K),
              "gpu": torch.cuda.get_device_name(0), "iters": args.iters, "results": rows,
              "note": "both sides are timed through their private torch ops, output allocation included"}
    if args.out:
        pathlib.Path(args.out).write_text(json.dumps(result, indent=1))


if __name__ == "__main__":
    main()
