"""GPU tests of the operator surface: functional, autograd, custom ops, operand hygiene."""

from __future__ import annotations

import pathlib

import numpy as np
import pytest
import torch

from oracle import msda_oracle as orc
from tests._abi import abi_backward, abi_forward, dev, to_np
from tests._golden import load, rel_err

pytestmark = pytest.mark.gpu


def _case(name="small_b", dtype=torch.float32):
    c = load(name)
    t = {k: dev(c[k], dtype) for k in ("value", "loc", "attn_linear", "attn_logits", "grad_out")}
    t["loc"] = dev(c["loc"], torch.float32)
    t["shapes"], t["starts"] = dev(c["spatial_shapes"]), dev(c["level_start_index"])
    return c, t


@pytest.mark.parametrize("method", ["linear", "softmax"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_functional_autograd_equals_abi(method, dtype):
    from deformops_b200.registry import Backend, msda

    _, t = _case(dtype=dtype)
    attn = t["attn_logits"] if method == "softmax" else t["attn_linear"]
    v, l, a = (x.clone().requires_grad_(True) for x in (t["value"], t["loc"], attn))
    out = msda(v, t["shapes"], t["starts"], l, a, method=method, backend=Backend.CUDA)
    out.backward(t["grad_out"])
    e_out = abi_forward(t["value"], t["shapes"], t["starts"], t["loc"], attn, softmax=method == "softmax")
    e_gv, e_gl, e_ga = abi_backward(t["value"], t["shapes"], t["starts"], t["loc"], attn,
                                    t["grad_out"], softmax=method == "softmax")
    assert torch.equal(out, e_out)
    assert torch.equal(l.grad, e_gl) and torch.equal(a.grad, e_ga)
    tol = 1e-6 if dtype == torch.float32 else 2e-2  # atomics reorder grad_value sums
    torch.testing.assert_close(v.grad, e_gv, rtol=tol, atol=tol)
    assert v.grad.dtype == dtype and l.grad.dtype == torch.float32 and a.grad.dtype == dtype


def test_non_contiguous_split_weights_int32_tables_and_16bit_locations():
    """Any memory layout, (B,Q,G,L,K) weights, int32 level tables, low-precision locations."""
    from deformops_b200.registry import msda

    c, t = _case("small_b")
    B, Q, G, L, K, _ = c["loc"].shape
    value = t["value"].transpose(1, 2).contiguous().transpose(1, 2)      # strided view
    padded = torch.zeros(*t["loc"].shape[:-1], 3, device="cuda")
    padded[..., :2] = t["loc"]
    loc = padded[..., :2]                                                # strided view
    attn5 = t["attn_linear"].view(B, Q, G, L, K)
    v, l, a = (x.detach().requires_grad_(True) for x in (value, loc, attn5))
    assert not v.is_contiguous() and not l.is_contiguous()
    out = msda(v, t["shapes"].int(), t["starts"].int(), l, a)
    out.backward(t["grad_out"])
    assert rel_err(to_np(out), c["linear_out_eager"]) < 1e-5
    assert a.grad.shape == attn5.shape
    assert rel_err(to_np(a.grad).reshape(B, Q, G, L * K), c["linear_grad_attn"]) < 1e-4
    assert rel_err(to_np(v.grad), c["linear_grad_value"]) < 1e-4
    assert rel_err(to_np(l.grad), c["linear_grad_loc"]) < 1e-4

    # bf16 locations are widened to float32 before the kernel; the gradient returns as bf16
    lb = t["loc"].bfloat16().requires_grad_(True)
    vb = t["value"].bfloat16()
    ab = t["attn_linear"].bfloat16()
    ob = msda(vb, t["shapes"], t["starts"], lb, ab)
    ob.float().sum().backward()
    assert lb.grad.dtype == torch.bfloat16
    e = orc.forward(vb.cpu(), c["spatial_shapes"], c["level_start_index"], lb.detach().cpu(), ab.cpu())
    assert rel_err(to_np(ob), e) < 1e-2


def test_public_ops_no_grad_inference_and_vmap():
    from deformops_b200.registry import msda

    c, t = _case("small_b")
    args = (t["value"], t["shapes"], t["starts"], t["loc"], t["attn_linear"])
    ref = msda(*args)
    with torch.no_grad():
        assert torch.equal(torch.ops.deformops_b200.msda(*args), ref)
    with torch.inference_mode():
        assert torch.equal(torch.ops.deformops_b200.msda(*args), ref)
    sm = torch.ops.deformops_b200.msda_softmax(t["value"], t["shapes"], t["starts"], t["loc"],
                                               t["attn_logits"])
    assert rel_err(to_np(sm), c["softmax_out_eager"]) < 1e-5
    # vmap over an extra leading axis folds into the batch: one kernel run, same numbers
    stacked = [torch.stack([x, x * 1.0]) for x in (t["value"], t["loc"], t["attn_linear"])]
    out = torch.vmap(torch.ops.deformops_b200.msda, in_dims=(0, None, None, 0, 0))(
        stacked[0], t["shapes"], t["starts"], stacked[1], stacked[2])
    assert out.shape == (2, *ref.shape)
    assert torch.equal(out[0], ref) and torch.equal(out[1], ref)
    with pytest.raises(ValueError, match="shared"):
        torch.vmap(torch.ops.deformops_b200.msda, in_dims=(0, 0, None, 0, 0))(
            stacked[0], torch.stack([t["shapes"]] * 2), t["starts"], stacked[1], stacked[2])


def test_opcheck_private_and_public_ops():
    _, t = _case("small_a")
    K = t["loc"].shape[4]
    v, l, a = (x.clone().requires_grad_(True) for x in (t["value"], t["loc"], t["attn_linear"]))
    torch.library.opcheck(torch.ops.deformops_b200.msda_forward.default,
                          (v, t["shapes"], t["starts"], l, a, 128, K, 0, 0))
    torch.library.opcheck(torch.ops.deformops_b200.msda_softmax_forward.default,
                          (v, t["shapes"], t["starts"], l, a, 128, K, 0, 0))
    torch.library.opcheck(torch.ops.deformops_b200.msda_backward.default,
                          (t["value"], t["shapes"], t["starts"], t["loc"], t["attn_linear"],
                           t["grad_out"], 128, K, 0, 0),
                          test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(torch.ops.deformops_b200.msda.default,
                          (v, t["shapes"], t["starts"], l, a),
                          test_utils=("test_schema", "test_faketensor", "test_aot_dispatch_static"))


def test_fake_tensor_backward_and_compile():
    from torch._subclasses.fake_tensor import FakeTensorMode

    from deformops_b200.registry import msda

    c, t = _case("small_b")
    with FakeTensorMode(allow_non_fake_inputs=False) as mode:
        f = {k: mode.from_tensor(x) for k, x in t.items()}
        v, l, a = (f[k].clone().requires_grad_(True) for k in ("value", "loc", "attn_linear"))
        out = torch.ops.deformops_b200.msda(v, f["shapes"], f["starts"], l, a)
        out.sum().backward()
        assert v.grad.shape == v.shape and l.grad.shape == l.shape and a.grad.shape == a.shape

    compiled = torch.compile(lambda *xs: msda(*xs), backend="aot_eager", fullgraph=True)
    args = (t["value"], t["shapes"], t["starts"], t["loc"], t["attn_linear"])
    assert torch.equal(compiled(*args), msda(*args))


def test_errors_before_launch():
    from deformops_b200 import NoBackendError
    from deformops_b200.registry import Backend, msda

    _, t = _case("small_b")
    args = [t["value"], t["shapes"], t["starts"], t["loc"], t["attn_linear"]]
    with pytest.raises(TypeError):
        msda(*args, backend="cuda")
    with pytest.raises(TypeError):
        msda(*args, bogus=1)
    with pytest.raises(TypeError):
        msda(args[0], args[1])
    with pytest.raises(ValueError):
        msda(args[0], args[1], args[2], args[3][:, :, :1], args[4])
    with pytest.raises(ValueError):
        msda(args[0], args[1], args[2], args[3], args[4].double())
    with pytest.raises(NoBackendError):
        msda(*args, backend=Backend.TRITON)
    with pytest.raises(NoBackendError):
        msda(args[0][..., :7].contiguous(), *args[1:])      # 7 channels: no 16-byte vectors
    with pytest.raises(NoBackendError):
        msda(*[a.cpu() for a in args])


def test_empty_calls_return_zeros_without_launch():
    from deformops_b200.ops import launch_counter
    from deformops_b200.registry import msda

    _, t = _case("small_b")
    launch_counter.reset()
    out = msda(t["value"], t["shapes"], t["starts"], t["loc"][:, :0], t["attn_linear"][:, :0])
    assert out.shape == (t["value"].shape[0], 0, t["value"].shape[2] * t["value"].shape[3])
    out = msda(t["value"][:0], t["shapes"], t["starts"], t["loc"][:0], t["attn_linear"][:0])
    assert out.numel() == 0 and launch_counter.kernels == 0


def test_autocast_keeps_float32_locations():
    from deformops_b200.registry import msda

    c, t = _case("small_b", torch.bfloat16)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = msda(t["value"], t["shapes"], t["starts"], t["loc"], t["attn_linear"])
    assert out.dtype == torch.bfloat16
    e = orc.forward(t["value"].cpu(), c["spatial_shapes"], c["level_start_index"], t["loc"].cpu(),
                    t["attn_linear"].cpu())
    assert rel_err(to_np(out), e) < 1e-2


def test_forward_and_backward_replay_from_a_cuda_graph():
    """The call path never synchronises with the host and reads the level table on the device,
    so forward + backward can be captured once and replayed on new data."""
    from deformops_b200.registry import msda

    _, t = _case("small_b", torch.bfloat16)
    value = t["value"].clone().requires_grad_(True)
    loc = t["loc"].clone().requires_grad_(True)
    attn = t["attn_linear"].clone().requires_grad_(True)

    def step():
        out = msda(value, t["shapes"], t["starts"], loc, attn)
        grads = torch.autograd.grad(out, [value, loc, attn], t["grad_out"])
        return out, grads

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):          # warm-up outside capture: library load, allocator
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, grads = step()
    with torch.no_grad():                   # new inputs in the captured buffers
        value.mul_(0.5)
        loc.add_(0.01)
    graph.replay()
    torch.cuda.synchronize()
    e_out, e_grads = step()
    assert torch.equal(out, e_out)
    assert torch.equal(grads[1], e_grads[1]) and torch.equal(grads[2], e_grads[2])
    torch.testing.assert_close(grads[0], e_grads[0], rtol=2e-2, atol=2e-2)


def test_large_call_replays_from_a_cuda_graph():
    """A backward call long enough to launch its second and third kernel as programmatic
    dependents of the one before (2^21 (query, head, point) triples and up) is captured and
    replayed like any other: the replay on new data equals an ordinary call on that data."""
    from deformops_b200.registry import msda
    from deformops_b200.workloads import make_workload

    w = make_workload("cfg2_m2f_1024_bf16", batch=2).to("cuda")
    B, S, G, D, Q, L, K = w.dims
    assert B * Q * G * L * K >= 1 << 21
    value = w.value.clone().requires_grad_(True)
    loc = w.sampling_locations.clone().requires_grad_(True)
    attn = w.attention_weights.clone().requires_grad_(True)

    def step():
        out = msda(value, w.spatial_shapes, w.level_start_index, loc, attn)
        return out, torch.autograd.grad(out, [value, loc, attn], w.grad_output)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, grads = step()
    with torch.no_grad():
        value.mul_(0.5)
        loc.add_(0.003)
    for _ in range(3):                      # several replays: the dependency edges hold every time
        graph.replay()
    torch.cuda.synchronize()
    e_out, e_grads = step()
    assert torch.equal(out, e_out)
    assert torch.equal(grads[1], e_grads[1]) and torch.equal(grads[2], e_grads[2])
    torch.testing.assert_close(grads[0].float(), e_grads[0].float(), rtol=2e-2, atol=2e-2)


def test_export_and_dynamo_record_the_public_op():
    """torch.export keeps the public op in the graph and decomposes it to the private forward op;
    Dynamo traces the functional without a graph break (dynamic query count included)."""
    from deformops_b200.registry import msda

    _, t = _case("small_b")
    args = (t["value"], t["shapes"], t["starts"], t["loc"], t["attn_linear"])

    class Layer(torch.nn.Module):
        def forward(self, value, shapes, starts, loc, attn):
            return msda(value, shapes, starts, loc, attn, method="softmax")

    exported = torch.export.export(Layer(), args)
    targets = [str(n.target) for n in exported.graph.nodes if n.op == "call_function"]
    assert any("deformops_b200.msda_softmax" in x for x in targets), targets
    decomposed = exported.run_decompositions()
    targets = [str(n.target) for n in decomposed.graph.nodes if n.op == "call_function"]
    assert any("deformops_b200.msda_softmax_forward" in x for x in targets), targets
    assert torch.equal(decomposed.module()(*args), Layer()(*args))

    seen = []

    def backend(gm, example_inputs):
        seen.extend(str(n.target) for n in gm.graph.nodes if n.op == "call_function")
        return gm.forward

    compiled = torch.compile(Layer(), backend=backend, fullgraph=True, dynamic=True)
    out = compiled(*args)
    assert torch.equal(out, Layer()(*args))
    assert any("deformops_b200.msda_softmax" in x for x in seen), seen
    fewer = (t["value"], t["shapes"], t["starts"], t["loc"][:, :5], t["attn_linear"][:, :5])
    assert torch.equal(compiled(*fewer), Layer()(*fewer))


def test_aot_inductor_package_in_fresh_processes_with_and_without_python_registration(tmp_path):
    """An AOTInductor package of a module that calls the operator is compiled in one child
    process and run in two others.  The first imports ``deformops_b200`` (which registers the
    ops and their CUDA implementations over ctypes) - the recipe the reference documents for
    its CUDA operators (``docs/export.md``: "needs their library loaded first").  The second
    never imports the package: it loads ``libmsda_b200_torch.so`` (csrc/torch_binding.cpp),
    which registers the private operators with the dispatcher natively, runs the same package
    and calls the backward operator directly; results equal the Python-registered ones."""
    import os
    import shutil
    import subprocess
    import sys

    from deformops_b200._build import TORCH_BINDING_PATH, build_torch_binding

    if not TORCH_BINDING_PATH.exists():
        build_torch_binding()
    c, t = _case("small_b")
    K = t["loc"].shape[4]
    torch.save({k: torch.as_tensor(c[k]) for k in ("value", "spatial_shapes", "level_start_index",
                                                   "loc", "attn_logits", "grad_out")},
               tmp_path / "in.pt")
    root = pathlib.Path(__file__).resolve().parents[1]
    env = dict(os.environ)
    if shutil.which("g++"):
        env["CXX"] = shutil.which("g++")
    compile_script = f"""
import torch
from deformops_b200.registry import msda
c = torch.load(r'{tmp_path / 'in.pt'}')
args = tuple(c[k].cuda() for k in ("value", "spatial_shapes", "level_start_index", "loc", "attn_logits"))
class Layer(torch.nn.Module):
    def forward(self, value, shapes, starts, loc, attn):
        return msda(value, shapes, starts, loc, attn, method="softmax") * 2.0
torch.save(Layer()(*args).cpu(), r'{tmp_path / 'expected.pt'}')
exported = torch.export.export(Layer(), args)
torch._inductor.aoti_compile_and_package(exported, package_path=r'{tmp_path / 'layer.pt2'}')
print('compiled')
"""
    native_script = f"""
import sys, torch
torch.ops.load_library(r'{TORCH_BINDING_PATH}')
c = torch.load(r'{tmp_path / 'in.pt'}')
args = tuple(c[k].cuda() for k in ("value", "spatial_shapes", "level_start_index", "loc", "attn_logits"))
runner = torch._inductor.aoti_load_package(r'{tmp_path / 'layer.pt2'}')
out = runner(*args)
torch.cuda.synchronize()
assert torch.equal(out.cpu(), torch.load(r'{tmp_path / 'expected.pt'}'))
grads = torch.ops.deformops_b200.msda_softmax_backward(*args, c["grad_out"].cuda(), 128, {K}, 0, 0)
torch.save([g.cpu() for g in grads], r'{tmp_path / 'native_grads.pt'}')
assert 'deformops_b200' not in sys.modules
print('native-ok')
"""
    done = subprocess.run([sys.executable, "-c", compile_script], cwd=root, env=env,
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "compiled" in done.stdout, done.stderr[-3000:]
    python_script = f"""
import torch
import deformops_b200
from deformops_b200._loader import loaded
c = torch.load(r'{tmp_path / 'in.pt'}')
args = tuple(c[k].cuda() for k in ("value", "spatial_shapes", "level_start_index", "loc", "attn_logits"))
runner = torch._inductor.aoti_load_package(r'{tmp_path / 'layer.pt2'}')
out = runner(*args)
torch.cuda.synchronize()
assert torch.equal(out.cpu(), torch.load(r'{tmp_path / 'expected.pt'}'))
assert loaded()
print('python-ok')
"""
    done = subprocess.run([sys.executable, "-c", python_script], cwd=root, env=env,
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "python-ok" in done.stdout, done.stderr[-3000:]
    done = subprocess.run([sys.executable, "-c", native_script], cwd=tmp_path, env=env,
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "native-ok" in done.stdout, done.stderr[-3000:]
    native = torch.load(tmp_path / "native_grads.pt")
    mine = torch.ops.deformops_b200.msda_softmax_backward(
        t["value"], t["shapes"], t["starts"], t["loc"], t["attn_logits"], t["grad_out"], 128, K,
        0, 0)
    assert torch.equal(native[1], mine[1].cpu()) and torch.equal(native[2], mine[2].cpu())
    torch.testing.assert_close(native[0], mine[0].cpu(), rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
def test_aot_inductor_package_of_the_default_layer_runs_without_python_registration(tmp_path):
    """The layer's default path fuses the location arithmetic into the operator
    (``deformops_b200::msda_offsets_forward``).  A package exported from it must run in a process
    that only loads ``libmsda_b200_torch.so``: the native library registers the offsets
    operators too."""
    import os
    import shutil
    import subprocess
    import sys

    from deformops_b200._build import TORCH_BINDING_PATH, build_torch_binding

    if not TORCH_BINDING_PATH.exists():
        build_torch_binding()
    root = pathlib.Path(__file__).resolve().parents[1]
    env = dict(os.environ)
    if shutil.which("g++"):
        env["CXX"] = shutil.which("g++")
    compile_script = f"""
import torch
from deformops_b200.nn import MultiScaleDeformAttn2d
torch.manual_seed(0)
levels = [(8, 8), (4, 4)]
S = sum(h * w for h, w in levels)
layer = MultiScaleDeformAttn2d(64, num_heads=2, num_levels=2, num_points=4).cuda().eval()
args = (torch.randn(2, S, 64, device="cuda"), torch.rand(2, S, 2, 2, device="cuda"),
        torch.randn(2, S, 64, device="cuda"), torch.tensor(levels, device="cuda"),
        torch.tensor([0, 64], device="cuda"))
torch.save([a.cpu() for a in args], r'{tmp_path / 'in.pt'}')
with torch.no_grad():
    torch.save(layer(*args).cpu(), r'{tmp_path / 'expected.pt'}')
    exported = torch.export.export(layer, args)
text = "".join(str(m.graph) for m in exported.graph_module.modules() if hasattr(m, "graph"))
assert "msda_offsets_forward" in text, text
torch._inductor.aoti_compile_and_package(exported, package_path=r'{tmp_path / 'layer.pt2'}')
print('compiled')
"""
    native_script = f"""
import sys, torch
torch.ops.load_library(r'{TORCH_BINDING_PATH}')
args = tuple(a.cuda() for a in torch.load(r'{tmp_path / 'in.pt'}'))
runner = torch._inductor.aoti_load_package(r'{tmp_path / 'layer.pt2'}')
out = runner(*args)
torch.cuda.synchronize()
torch.testing.assert_close(out.cpu(), torch.load(r'{tmp_path / 'expected.pt'}'), rtol=1e-5, atol=1e-6)
assert 'deformops_b200' not in sys.modules
print('native-ok')
"""
    # (the second process starts where the package cannot even be imported from)
    for script, word, cwd in ((compile_script, "compiled", root), (native_script, "native-ok", tmp_path)):
        done = subprocess.run([sys.executable, "-c", script], cwd=cwd, env=env,
                              capture_output=True, text=True, timeout=900)
        assert done.returncode == 0 and word in done.stdout, done.stderr[-3000:]


@pytest.mark.gpu
def test_reference_op_names_run_these_kernels_in_a_process_without_the_reference():
    """A program written against ``torch.ops.deformops.msda`` (the reference's public name) runs
    on this library alone after ``define_reference_op_names()``: same numbers as our own op,
    gradients included."""
    import subprocess
    import sys

    code = (
        "import torch, deformops_b200\n"
        "from deformops_b200.ops import define_reference_op_names\n"
        "from deformops_b200.workloads import make_workload\n"
        "assert define_reference_op_names()\n"
        "w = make_workload(dict(batch=2, levels=[(8, 8), (4, 4)], heads=4, head_dim=32, points=4,\n"
        "                       dtype=torch.float32), seed=2).to('cuda')\n"
        "def run(op, attn):\n"
        "    leaves = [t.detach().clone().requires_grad_() for t in (w.value, w.sampling_locations, attn)]\n"
        "    out = op(leaves[0], w.spatial_shapes, w.level_start_index, leaves[1], leaves[2])\n"
        "    return (out, *torch.autograd.grad(out, leaves, w.grad_output))\n"
        "for name, attn in (('msda', w.attention_weights), ('msda_softmax', w.attention_logits)):\n"
        "    a = run(getattr(torch.ops.deformops, name), attn)\n"
        "    b = run(getattr(torch.ops.deformops_b200, name), attn)\n"
        "    assert all(torch.equal(x, y) for x, y in zip(a[:1] + a[2:], b[:1] + b[2:]))\n"
        "    torch.testing.assert_close(a[1], b[1], rtol=1e-5, atol=1e-6)\n"
        "print('ok')\n")
    root = __import__("pathlib").Path(__file__).resolve().parents[1]
    res = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
