"""CPU tests: operand validation, method resolution, registry errors, op schemas, the C ABI's
exported symbols and pure-host entry points, fake-tensor wiring.  No kernel is launched."""

from __future__ import annotations

import ctypes
import pathlib
import re
import subprocess
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _operands(B=2, S=20, G=2, D=8, Q=5, L=2, K=3, dtype=torch.float32, device="cpu"):
    value = torch.zeros(B, S, G, D, dtype=dtype, device=device)
    shapes = torch.tensor([[4, 4], [2, 2]], dtype=torch.int64, device=device)[:L]
    starts = torch.tensor([0, 16], dtype=torch.int64, device=device)[:L]
    loc = torch.zeros(B, Q, G, L, K, 2, device=device)
    attn = torch.zeros(B, Q, G, L * K, dtype=dtype, device=device)
    return [value, shapes, starts, loc, attn]


# ---- validation (mirrors the reference's ValueError conventions) ---------------------------
def test_check_msda_call_accepts_flat_and_split_weights():
    from deformops_b200.core.sanitize import check_msda_call

    ops = _operands()
    check_msda_call(*ops)
    ops[4] = ops[4].view(2, 5, 2, 2, 3)
    check_msda_call(*ops)
    ops[3] = ops[3].bfloat16()      # locations may differ in dtype
    check_msda_call(*ops)


@pytest.mark.parametrize("mutate, match", [
    (lambda o: o.__setitem__(0, o[0][0]), "value must have 4"),
    (lambda o: o.__setitem__(1, o[1][:, :1]), "height, width"),
    (lambda o: o.__setitem__(2, o[2][:1]), "one entry per level"),
    (lambda o: o.__setitem__(3, o[3][:1]), "batch of value"),
    (lambda o: o.__setitem__(3, o[3][:, :, :1]), "heads of value"),
    (lambda o: o.__setitem__(3, o[3][..., :1]), r"\(x, y\) pair"),
    (lambda o: o.__setitem__(4, o[4][:, :3]), "queries"),
    (lambda o: o.__setitem__(4, o[4][..., :5]), "levels x points"),
    (lambda o: o.__setitem__(1, o[1].float()), "integer tensor"),
    (lambda o: o.__setitem__(4, o[4].double()), "mixed input dtypes"),
    (lambda o: o.__setitem__(3, o[3].long()), "floating-point"),
    (lambda o: o.__setitem__(2, o[2].to("meta")), "one device"),
])
def test_check_msda_call_rejects(mutate, match):
    from deformops_b200.core.sanitize import check_msda_call

    ops = _operands()
    mutate(ops)
    with pytest.raises(ValueError, match=match):
        check_msda_call(*ops)


def test_level_table_value_checks_only_when_enabled(monkeypatch):
    from deformops_b200.core.sanitize import check_msda_call

    ops = _operands()
    ops[2] = torch.tensor([0, 15])           # not the prefix sum
    check_msda_call(*ops)                     # metadata-only by default: no host read
    monkeypatch.setenv("DEFORMOPS_VALIDATE", "1")
    with pytest.raises(ValueError, match="prefix sum"):
        check_msda_call(*ops)
    ops[2] = torch.tensor([0, 16])
    ops[0] = torch.zeros(2, 21, 2, 8)
    with pytest.raises(ValueError, match="tile the value tensor"):
        check_msda_call(*ops)
    ops[0] = torch.zeros(2, 20, 2, 8)
    ops[1] = torch.tensor([[4, 4], [0, 4]])
    with pytest.raises(ValueError, match="positive"):
        check_msda_call(*ops)


def test_method_resolution():
    from deformops_b200.core.runtime import Method, resolve_method

    assert resolve_method(None) is Method.LINEAR
    assert resolve_method(None, softmax=True) is Method.SOFTMAX
    assert resolve_method("linear", softmax=True) is Method.LINEAR      # explicit wins
    assert resolve_method(Method.SOFTMAX) is Method.SOFTMAX
    assert Method.SOFTMAX == "softmax"
    with pytest.raises(ValueError):
        resolve_method("mean")


# ---- registry surface ----------------------------------------------------------------------
def test_registry_errors_on_cpu():
    from deformops_b200 import NoBackendError
    from deformops_b200.registry import Backend, MSDABackend, msda

    ops = _operands()
    with pytest.raises(NoBackendError, match="no CPU path"):
        msda(*ops)
    with pytest.raises(NoBackendError, match="not part of this build"):
        msda(*ops, backend=Backend.EAGER)
    with pytest.raises(TypeError, match="string"):
        msda(*ops, backend="cuda")
    with pytest.raises(TypeError, match="unexpected keyword"):
        msda(*ops, tile=3)
    with pytest.raises(TypeError, match="positionally"):
        msda(ops[0], ops[1], ops[2])
    with pytest.raises(ValueError):
        msda(ops[0], ops[1], ops[2], ops[3], ops[4][:, :1])
    assert isinstance(msda.backend, MSDABackend) and msda.backend.name == "cuda_b200"


def test_context_and_supports():
    from deformops_b200.registry import MSDAContext, Method, msda, supports_context, unsupported_reason

    ctx = msda.context_of(*_operands(), method="softmax")
    assert (ctx.num_levels, ctx.num_heads, ctx.num_points, ctx.head_dim) == (2, 2, 3, 8)
    assert ctx.method is Method.SOFTMAX and ctx.num_queries == 5 and not ctx.is_training
    assert not supports_context(ctx) and "CUDA" in unsupported_reason(ctx)
    import dataclasses

    gpu = dataclasses.replace(ctx, device=torch.device("cuda", 0), sm_version=(10, 0))
    assert supports_context(gpu)
    assert "sm_100a" in unsupported_reason(dataclasses.replace(gpu, sm_version=(9, 0)))
    assert "multiple" in unsupported_reason(dataclasses.replace(gpu, head_dim=6))
    assert supports_context(dataclasses.replace(gpu, dtype=torch.float64, head_dim=3))
    assert "int32" in unsupported_reason(dataclasses.replace(gpu, dtype=torch.int32))
    assert "levels" in unsupported_reason(dataclasses.replace(gpu, num_levels=17))
    # num_queries is not part of equality (varying resolutions share one context)
    assert dataclasses.replace(gpu, num_queries=7) == gpu and isinstance(gpu, MSDAContext)


def test_apply_msda_method_shapes():
    from deformops_b200.registry import apply_msda_method

    a = torch.randn(2, 3, 4, 6)
    assert torch.allclose(apply_msda_method(a, "softmax").sum(-1), torch.ones(2, 3, 4))
    a5 = a.view(2, 3, 4, 2, 3)
    assert torch.allclose(apply_msda_method(a5, "softmax").flatten(-2), apply_msda_method(a, "softmax"))
    assert apply_msda_method(a, "linear") is a
    with pytest.raises(ValueError):
        apply_msda_method(a[0], "softmax")


# ---- torch.library wiring -----------------------------------------------------------------
def test_op_schemas_exist_and_match_reference_signature():
    import deformops_b200  # noqa: F401

    ns = torch.ops.deformops_b200
    fwd = str(ns.msda_forward.default._schema)
    assert "Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn" in fwd
    assert "int chunk_step, int K, int channels_per_thread, int threads_per_block) -> Tensor" in fwd
    bwd = str(ns.msda_softmax_backward.default._schema)
    assert "Tensor grad_output" in bwd and "-> (Tensor, Tensor, Tensor)" in bwd
    pub = str(ns.msda.default._schema)
    assert pub.endswith("(Tensor value, Tensor spatial_shapes, Tensor level_start_index, "
                        "Tensor sampling_locations, Tensor attention_weights) -> Tensor")
    assert hasattr(ns, "msda_softmax") and hasattr(ns, "msda_softmax_forward")


def test_fake_tensors_need_no_gpu_and_no_kernel():
    from torch._subclasses.fake_tensor import FakeTensorMode

    import deformops_b200  # noqa: F401

    with FakeTensorMode():
        ops = _operands(dtype=torch.bfloat16, device="cuda")
        out = torch.ops.deformops_b200.msda(*ops)
        assert out.shape == (2, 5, 16) and out.dtype == torch.bfloat16 and out.device.type == "cuda"
        out = torch.ops.deformops_b200.msda_softmax(*ops)
        assert out.shape == (2, 5, 16)
        gv, gl, ga = torch.ops.deformops_b200.msda_backward(*ops, out, 128, 3, 0, 0)
        assert gv.shape == ops[0].shape and gl.dtype == torch.float32 and ga.dtype == torch.bfloat16


def test_private_op_on_cpu_tensors_fails_loudly():
    import deformops_b200  # noqa: F401

    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.deformops_b200.msda_forward(*_operands(), 128, 3, 0, 0)


def test_import_defines_ops_without_loading_the_library():
    code = ("import deformops_b200, torch, deformops_b200._loader as l;"
            "assert hasattr(torch.ops.deformops_b200, 'msda');"
            "assert not l.loaded(); print('ok')")
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr


# ---- the C ABI ------------------------------------------------------------------------------
def _declared_functions():
    text = (ROOT / "include" / "msda_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msda_b200_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from deformops_b200._loader import Shim, load_library

    shim = load_library()
    declared = _declared_functions()
    assert len(declared) >= 6
    assert sorted(Shim.SYMBOLS) == declared            # the loader binds exactly the header
    for name in declared:
        assert hasattr(shim.lib, name), name
    header_version = int(re.search(r"#define MSDA_B200_ABI_VERSION (\d+)",
                                   (ROOT / "include" / "msda_b200.h").read_text()).group(1))
    assert shim.lib.msda_b200_abi_version() == header_version


def test_loader_is_memoised_and_thread_safe():
    import threading

    from deformops_b200._loader import load_library

    got = []
    threads = [threading.Thread(target=lambda: got.append(load_library())) for _ in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert all(g is got[0] for g in got)


def test_missing_library_raises_typed_error(monkeypatch, tmp_path):
    import deformops_b200._loader as loader
    from deformops_b200 import KernelUnavailableError

    monkeypatch.setattr(loader, "_shim", None)
    monkeypatch.setenv("DEFORMOPS_B200_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(KernelUnavailableError, match="no CPU path"):
        loader.load_library()
    bad = tmp_path / "bad.so"
    bad.write_bytes(b"not an ELF file")
    monkeypatch.setenv("DEFORMOPS_B200_LIBRARY", str(bad))
    with pytest.raises(KernelUnavailableError, match="cannot load"):
        loader.load_library()


def test_host_only_entry_points():
    """Shape validation, launch geometry and scratch sizing never touch the device."""
    from deformops_b200._loader import load_library

    shim = load_library()
    null = ctypes.c_void_p(0)
    grid, threads = ctypes.c_int64(), ctypes.c_int()
    sf, sb = ctypes.c_int64(), ctypes.c_int64()
    # headline shape: bf16, 8 heads x 32 channels, 3 levels x 4 points, 4 x 21504 queries
    assert shim.launch_geometry(4, 8, 32, 21504, 3, 4, 2, 0, grid, threads, sf, sb) == 0
    assert threads.value == 256 and grid.value == 4 * 21504 // 8     # one warp per query
    # 8 warps x 8 pairs x (12 points x 2 words + 1 word of padding) x 16 bytes of descriptors
    assert sf.value == 8 * 8 * (2 * 12 + 1) * 16 and sb.value > sf.value
    assert shim.scratch_bytes(4, 21504, 8, 32, 21504, 3, 4, 2) == 256 + 2 * 4 * (21504 * 256 + 3 * 344064)
    assert shim.scratch_bytes(4, 21504, 8, 32, 21504, 3, 4, 0) == 0
    # statuses and messages
    assert shim.launch_geometry(1, 1, 12, 1, 1, 1, 2, 0, grid, threads, sf, sb) == -2
    assert "multiple of 8" in shim.last_error()
    assert shim.launch_geometry(1, 1, 8, 1, 17, 1, 2, 0, grid, threads, sf, sb) == -2
    assert shim.launch_geometry(1, 1, 8, 1, 1, 1, 9, 0, grid, threads, sf, sb) == -1
    assert shim.forward(null, null, null, null, null, null, 1, 4, 1, 8, 1, 1, 1, 2, 0, -1, null) == -1
    assert "null" in shim.last_error()
    assert shim.forward(null, null, null, null, null, null, 0, 4, 1, 8, 1, 1, 1, 2, 0, -1, null) == 0
    big = 1 << 24
    assert shim.forward(null, null, null, null, null, null, 1, big, 8, 32, 1, 1, 1, 2, 0, -1, null) == -2
    assert "2^31" in shim.last_error()


def test_error_message_is_thread_local():
    import threading

    from deformops_b200._loader import load_library

    shim = load_library()
    null = ctypes.c_void_p(0)
    shim.forward(null, null, null, null, null, null, 1, 4, 1, 12, 1, 1, 1, 2, 0, -1, null)
    seen = []
    t = threading.Thread(target=lambda: seen.append(shim.last_error()))
    t.start()
    t.join()
    assert seen == [""] and "multiple of 8" in shim.last_error()


def test_register_into_reference_registry():
    """With the reference package importable, the adapter becomes its Backend.CUDA."""
    from oracle import build_ref

    ref_sources = build_ref.staged_package()
    if ref_sources is None:
        pytest.skip("reference package not staged (oracle/build_ref.py needs a checkout)")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch\n"
        "from deformops_b200.integrations.reference_registry import register_into_deformops, supports\n"
        "ref = register_into_deformops()\n"
        "from deformops.registry import Backend\n"
        "from deformops.registry.msda import MSDAContext, Method\n"
        "ctx = MSDAContext(device=torch.device('cuda', 0), num_levels=3, num_heads=8, num_points=4,\n"
        "                  dtype=torch.bfloat16, sm_version=(10, 0), is_training=True, num_queries=5,\n"
        "                  method=Method.LINEAR, head_dim=32)\n"
        "assert supports(ctx)\n"
        "import dataclasses\n"
        "assert not supports(dataclasses.replace(ctx, sm_version=(9, 0)))\n"
        "print(ref.load(Backend.CUDA))\n" % str(ref_sources))
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "libmsda_b200.so" in res.stdout


def test_reference_op_names_can_be_offered_without_the_reference():
    """``define_reference_op_names`` defines ``deformops::msda`` / ``deformops::msda_softmax`` with
    the public schema, once; in a fresh process so that no other test's imports interfere."""
    code = (
        "import torch, deformops_b200\n"
        "from deformops_b200.ops import define_reference_op_names\n"
        "assert define_reference_op_names() is True\n"
        "assert define_reference_op_names() is False\n"
        "for name in ('msda', 'msda_softmax'):\n"
        "    ours = getattr(torch.ops.deformops_b200, name).default._schema\n"
        "    theirs = getattr(torch.ops.deformops, name).default._schema\n"
        "    assert str(ours).split('(', 1)[1] == str(theirs).split('(', 1)[1]\n"
        "print('ok')\n")
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
