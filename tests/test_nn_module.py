"""``MultiScaleDeformAttn2d`` and ``run_msda``: parameters, checkpoints, location math (CPU) and
end-to-end parity with a pure-torch evaluation of the same layer (GPU)."""

from __future__ import annotations

import pathlib
import subprocess
import sys

import pytest
import torch

from deformops_b200.nn import MultiScaleDeformAttn2d

ROOT = pathlib.Path(__file__).resolve().parents[1]
LEVELS = [(8, 6), (4, 3), (2, 2)]


def _tables(device="cpu"):
    shapes = torch.tensor(LEVELS, dtype=torch.int64, device=device)
    sizes = shapes[:, 0] * shapes[:, 1]
    return shapes, torch.cumsum(sizes, 0) - sizes, int(sizes.sum())


def test_constructor_checks_and_parameter_shapes():
    m = MultiScaleDeformAttn2d(64, 48, 32, num_heads=4, num_levels=3, num_points=2)
    assert m.proj_offset.weight.shape == (4 * 3 * 2 * 2, 64)
    assert m.proj_weights.weight.shape == (4 * 3 * 2, 64)
    assert m.proj_value.weight.shape == (64, 48) and m.proj_output.weight.shape == (32, 64)
    assert m.method == "softmax" and m.chunk_step == 128 and m.backend is None
    for bad in (dict(dim=0), dict(num_heads=0), dict(num_levels=-1), dict(num_points=0),
                dict(dim=66), dict(dim=48, num_heads=4)):   # 48/4 = 12 is not a power of two
        kw = dict(dim=64, num_heads=4, num_levels=3, num_points=2)
        kw.update(bad)
        with pytest.raises(ValueError):
            MultiScaleDeformAttn2d(kw.pop("dim"), **kw)


def test_detr_initialisation():
    m = MultiScaleDeformAttn2d(32, num_heads=8, num_levels=2, num_points=4)
    assert not m.proj_offset.weight.any() and not m.proj_weights.weight.any()
    assert not m.proj_weights.bias.any() and not m.proj_value.bias.any()
    bias = m.proj_offset.bias.view(8, 2, 4, 2)
    # point k sits (k+1) steps along its head's direction; head 0 points along +x
    assert torch.allclose(bias[0, :, :, 0], torch.tensor([1., 2., 3., 4.]).expand(2, 4))
    assert torch.allclose(bias[0, :, :, 1], torch.zeros(2, 4), atol=1e-6)
    assert torch.allclose(bias[:, 0, 1], 2 * bias[:, 0, 0])
    assert torch.allclose(bias[:, 0, 0].abs().amax(-1), torch.ones(8))


def test_state_dict_round_trip_and_detr_key_rename():
    m = MultiScaleDeformAttn2d(32, num_heads=4, num_levels=2)
    sd = m.state_dict()
    assert set(sd) == {f"{n}.{p}" for n in ("proj_offset", "proj_weights", "proj_value", "proj_output")
                       for p in ("weight", "bias")}
    m2 = MultiScaleDeformAttn2d(32, num_heads=4, num_levels=2)
    m2.load_state_dict(sd)
    # a Deformable-DETR checkpoint (no version metadata) uses the old names
    rename = {"proj_offset": "sampling_offsets", "proj_weights": "attention_weights",
              "proj_value": "value_proj", "proj_output": "output_proj"}
    old = {f"{rename[k.split('.')[0]]}.{k.split('.')[1]}": torch.randn_like(v) for k, v in sd.items()}
    m3 = MultiScaleDeformAttn2d(32, num_heads=4, num_levels=2)
    m3.load_state_dict(dict(old))
    assert torch.equal(m3.proj_offset.weight, old["sampling_offsets.weight"])
    assert torch.equal(m3.proj_output.bias, old["output_proj.bias"])
    # nested under a parent module the prefix is honoured
    parent = torch.nn.Sequential(MultiScaleDeformAttn2d(32, num_heads=4, num_levels=2))
    parent.load_state_dict({f"0.{k}": v for k, v in old.items()})
    assert torch.equal(parent[0].proj_value.weight, old["value_proj.weight"])


def test_sampling_location_math():
    shapes, _, _ = _tables()
    m = MultiScaleDeformAttn2d(32, num_heads=4, num_levels=3, num_points=2)
    q = torch.randn(2, 5, 32)
    p2 = torch.rand(2, 5, 3, 2)
    loc = m.sampling_locations(q, p2, shapes)
    off = m.proj_offset(q).view(2, 5, 4, 3, 2, 2)
    for l, (h, w) in enumerate(LEVELS):
        expect = p2[:, :, None, l, None, :] + off[:, :, :, l] / torch.tensor([w, h])
        assert torch.allclose(loc[:, :, :, l], expect, atol=1e-6)
    p4 = torch.rand(2, 5, 3, 4)
    loc4 = m.sampling_locations(q, p4, shapes)
    expect = p4[:, :, None, :, None, :2] + off / 2 * p4[:, :, None, :, None, 2:] * 0.5
    assert torch.allclose(loc4, expect, atol=1e-6)
    with pytest.raises(ValueError):
        m.sampling_locations(q, torch.rand(2, 5, 3, 3), shapes)


def test_matches_reference_module_parameter_for_parameter():
    """Where the reference package is importable: same init, same state-dict, same locations."""
    from oracle import build_ref

    ref = build_ref.staged_package()
    if ref is None:
        pytest.skip("reference package not staged (oracle/build_ref.py needs a checkout)")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch\n"
        "from deformops.nn import MultiScaleDeformAttn2d as Ref\n"
        "from deformops_b200.nn import MultiScaleDeformAttn2d as Ours\n"
        "torch.manual_seed(0); r = Ref(64, num_heads=8, num_levels=3, num_points=4)\n"
        "torch.manual_seed(0); o = Ours(64, num_heads=8, num_levels=3, num_points=4)\n"
        "assert r.state_dict().keys() == o.state_dict().keys()\n"
        "assert torch.allclose(r.proj_offset.bias, o.proj_offset.bias, atol=1e-6)\n"
        "o.load_state_dict(r.state_dict()); r.load_state_dict(o.state_dict())\n"
        "print('ok')\n" % str(ref))
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]


def test_run_msda_derives_level_starts_and_accepts_backend_objects():
    from deformops_b200.integrations import run_msda

    seen = {}

    class Probe:
        name = "probe"

        def supports(self, context):
            return True

        def forward(self, value, shapes, starts, loc, attn, chunk_step, method):
            seen.update(starts=starts, chunk_step=chunk_step, method=method)
            return value.new_zeros(value.shape[0], loc.shape[1], value.shape[2] * value.shape[3])

    shapes, starts, S = _tables()
    out = run_msda(torch.zeros(1, S, 2, 8), shapes, None, torch.zeros(1, 3, 2, 3, 4, 2),
                   torch.zeros(1, 3, 2, 12), chunk_step=64, backend=Probe())
    assert out.shape == (1, 3, 16) and torch.equal(seen["starts"], starts)
    assert seen["chunk_step"] == 64 and seen["method"] == "linear"


# ---- GPU ---------------------------------------------------------------------------------------
def _torch_layer(m, q, p, v, shapes, starts, padding_mask=None):
    """The same layer evaluated with the pure-torch restatement of the operator."""
    from oracle.msda_eager_port import eager_forward

    B, Q, _ = q.shape
    value = m.proj_value(v)
    if padding_mask is not None:
        value = value.masked_fill(padding_mask[..., None], 0.0)
    value = value.view(B, v.shape[1], m.num_heads, m.dim // m.num_heads)
    w = m.proj_weights(q).view(B, Q, m.num_heads, m.num_levels * m.num_points)
    loc = m.sampling_locations(q, p, shapes)
    out = eager_forward(value, shapes, starts, loc, w, softmax=m.method == "softmax")
    return m.proj_output(out)


@pytest.mark.gpu
@pytest.mark.parametrize("method", ["softmax", "linear"])
@pytest.mark.parametrize("boxes", [False, True])
def test_layer_forward_backward_matches_torch_evaluation(method, boxes):
    torch.manual_seed(3)
    shapes, starts, S = _tables("cuda")
    m = MultiScaleDeformAttn2d(64, num_heads=4, num_levels=3, num_points=4, method=method).cuda()
    with torch.no_grad():   # leave the all-zero init so that offsets and weights depend on q
        m.proj_offset.weight.normal_(std=0.5)
        m.proj_weights.weight.normal_(std=0.5)
    q = torch.randn(2, 7, 64, device="cuda", requires_grad=True)
    v = torch.randn(2, S, 64, device="cuda", requires_grad=True)
    p = torch.rand(2, 7, 3, 4 if boxes else 2, device="cuda")
    mask = torch.zeros(2, S, dtype=torch.bool, device="cuda")
    mask[1, -5:] = True
    out = m(q, p, v, shapes, starts, mask)
    ref = _torch_layer(m, q, p, v, shapes, starts, mask)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    g = torch.randn_like(out)
    grads = torch.autograd.grad(out, [q, v, *m.parameters()], g, retain_graph=True)
    ref_grads = torch.autograd.grad(ref, [q, v, *m.parameters()], g)
    for a, b in zip(grads, ref_grads):
        torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-4)


@pytest.mark.gpu
def test_layer_with_backend_object_and_bf16_autocast():
    from deformops_b200.registry import Backend, msda

    shapes, starts, S = _tables("cuda")
    torch.manual_seed(4)
    m = MultiScaleDeformAttn2d(64, num_heads=2, num_levels=3, backend=msda.backend).cuda()
    m2 = MultiScaleDeformAttn2d(64, num_heads=2, num_levels=3, backend=Backend.CUDA).cuda()
    m2.load_state_dict(m.state_dict())
    q, v = torch.randn(1, 9, 64, device="cuda"), torch.randn(1, S, 64, device="cuda")
    p = torch.rand(1, 9, 3, 2, device="cuda")
    assert torch.equal(m(q, p, v, shapes, starts), m2(q, p, v, shapes, starts))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = m(q, p, v, shapes, starts)
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out.float(), m(q, p, v, shapes, starts), rtol=5e-2, atol=5e-2)
