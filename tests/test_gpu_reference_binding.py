"""The sm_100a kernels driven through the REFERENCE's own Python package.

``deformops_b200.integrations.reference_registry.register_into_deformops`` makes the call a
backend module of the reference makes at import time (``msda.register(Backend.CUDA, ...)``,
``sources/deformops/registry/_dispatch.py:169-205``).  From then on every caller of the
reference reaches these kernels.  The tests run them that way - the functional
``deformops.registry.msda(..., backend=Backend.CUDA)``, the layer
``deformops.nn.MultiScaleDeformAttn2d`` and the Hugging Face replacements installed by
``deformops.integrations.transformers.patch`` inside a tiny Mask2Former and a tiny
Deformable-DETR - and compare outputs AND gradients with the reference's eager backend, the
way the reference pins its own CUDA backend (``tests/deformops/test_public_ops.py:348-385``,
``tests/deformops/models/test_backend_matrix.py:61-76``, ``models/_tiny.py:44-96``).

The reference package is not part of this repository: ``oracle/build_ref.py`` stages an
unmodified copy under ``oracle/_ref/py`` wherever a checkout is available, and the tests skip
without it.
"""

from __future__ import annotations

import copy
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    """The reference package with this library registered as its ``Backend.CUDA``."""
    from oracle import build_ref

    staged = build_ref.staged_package()
    if staged is None:
        pytest.skip("reference package not staged (oracle/build_ref.py needs a checkout)")
    if str(staged) not in sys.path:
        sys.path.insert(0, str(staged))
    import deformops  # noqa: F401
    from deformops.registry import Backend

    from deformops_b200.integrations.reference_registry import register_into_deformops

    registry_msda = register_into_deformops()
    return registry_msda, Backend


def _operands(dtype, seed=0, batch=2):
    from deformops_b200.workloads import make_workload

    cfg = dict(batch=batch, levels=[(12, 10), (6, 5), (3, 3)], heads=4, head_dim=32, points=4,
               dtype=dtype)
    w = make_workload(cfg, seed=seed)
    dev = torch.device("cuda")
    return (w.value.to(dev), w.spatial_shapes.to(dev), w.level_start_index.to(dev),
            w.sampling_locations.to(dev), w.attention_weights.to(dev),
            w.attention_logits.to(dev), w.grad_output.to(dev))


@pytest.mark.parametrize("method", ["linear", "softmax"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_registry_msda_with_cuda_backend_runs_these_kernels(ref, dtype, method):
    from deformops_b200.ops import launch_counter

    registry_msda, Backend = ref
    value, shapes, starts, loc, weights, logits, grad_out = _operands(dtype)
    attn = logits if method == "softmax" else weights

    def run(backend):
        leaves = [t.detach().clone().requires_grad_(True) for t in (value, loc, attn)]
        out = registry_msda(leaves[0], shapes, starts, leaves[1], leaves[2], method=method,
                            backend=backend)
        grads = torch.autograd.grad(out, leaves, grad_out)
        return out, grads

    launch_counter.reset()
    out, grads = run(Backend.CUDA)
    assert launch_counter.kernels >= 2, "the call did not reach libmsda_b200.so"
    e_out, e_grads = run(Backend.EAGER)
    # (the eager backend computes 16-bit inputs in float32 and may return that: compare values)
    assert out.dtype == dtype
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(out.float(), e_out.float(), **tol)
    for got, want, leaf in zip(grads, e_grads, (value, loc, attn)):
        assert got.dtype == leaf.dtype and got.shape == want.shape
        scale = want.float().abs().max().clamp_min(1e-6)
        bar = 1e-4 if dtype == torch.float32 else 2e-2
        assert ((got.float() - want.float()).abs().max() / scale).item() <= bar


def test_reference_layer_on_these_kernels_matches_eager(ref):
    from deformops.nn import MultiScaleDeformAttn2d

    _, Backend = ref
    torch.manual_seed(0)
    levels = [(8, 8), (4, 4)]
    S = sum(h * w for h, w in levels)
    layer = MultiScaleDeformAttn2d(64, num_heads=2, num_levels=2, num_points=4,
                                   backend=Backend.CUDA).cuda()
    twin = copy.deepcopy(layer)
    twin.backend = Backend.EAGER
    q = torch.randn(2, S, 64, device="cuda")
    v = torch.randn(2, S, 64, device="cuda")
    p = torch.rand(2, S, 2, 2, device="cuda")
    shapes = torch.tensor(levels, device="cuda")
    starts = torch.tensor([0, 64], device="cuda")
    g = torch.randn(2, S, 64, device="cuda")
    results = []
    for module in (layer, twin):
        out = module(q, p, v, shapes, starts)
        grads = torch.autograd.grad(out, list(module.parameters()), g)
        results.append((out, grads))
    torch.testing.assert_close(results[0][0], results[1][0], rtol=1e-4, atol=1e-5)
    for got, want in zip(results[0][1], results[1][1]):
        torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-4)


# ---- tiny random-weight models (shapes after the reference's tests/deformops/models/_tiny.py) ----
def _tiny_mask2former():
    from transformers import Mask2FormerConfig, Mask2FormerForUniversalSegmentation
    from transformers.models.swin.configuration_swin import SwinConfig

    backbone = SwinConfig(image_size=64, patch_size=4, embed_dim=8, depths=[1, 1, 1, 1],
                          num_heads=[1, 1, 1, 1], window_size=2, out_indices=[1, 2, 3, 4])
    config = Mask2FormerConfig(feature_size=32, mask_feature_size=32, hidden_dim=32,
                               num_attention_heads=4, encoder_layers=1, decoder_layers=1,
                               encoder_feedforward_dim=64, dim_feedforward=64, num_queries=10,
                               backbone_config=backbone)
    return (Mask2FormerForUniversalSegmentation(config),
            lambda out: (out.class_queries_logits, out.masks_queries_logits))


def _tiny_deformable_detr():
    from transformers import DeformableDetrConfig, DeformableDetrForObjectDetection, ResNetConfig

    config = DeformableDetrConfig(
        backbone_config=ResNetConfig(embedding_size=16, hidden_sizes=[16, 24, 32, 48],
                                     depths=[1, 1, 1, 1],
                                     out_features=["stage2", "stage3", "stage4"]),
        use_pretrained_backbone=False, d_model=32, encoder_layers=1, decoder_layers=2,
        encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=64,
        decoder_ffn_dim=64, num_queries=10, num_feature_levels=4)
    return DeformableDetrForObjectDetection(config), lambda out: (out.logits, out.pred_boxes)


def _attention_parameters(model):
    return {name: parameter for name, parameter in model.named_parameters()
            if any(key in name for key in ("sampling_offsets", "attention_weights"))}


def _run_model(net, outputs_of, patch, backend):
    model = patch(copy.deepcopy(net).cuda(), backend=backend).eval()
    image = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(1)).cuda()
    outputs = outputs_of(model(pixel_values=image))
    loss = sum((o.float() * torch.linspace(-1, 1, o.numel(), device="cuda").view_as(o)).sum()
               for o in outputs)
    loss.backward()
    grads = {k: p.grad.detach().float().cpu() for k, p in _attention_parameters(model).items()}
    return [o.detach().float().cpu() for o in outputs], grads


@pytest.mark.parametrize("name", ["mask2former", "deformable_detr"])
def test_patched_models_match_eager_in_outputs_and_attention_gradients(ref, name):
    pytest.importorskip("transformers")
    try:
        from deformops.integrations.transformers import patch
    except ImportError as exc:   # the installed transformers lacks the classes it replaces
        pytest.skip(str(exc))
    from deformops_b200.ops import launch_counter

    _, Backend = ref
    torch.manual_seed(0)
    try:
        net, outputs_of = _tiny_mask2former() if name == "mask2former" else _tiny_deformable_detr()
    except Exception as exc:  # noqa: BLE001 - model classes differ between transformers versions
        pytest.skip(f"cannot build the tiny {name}: {exc}")
    want_out, want_grads = _run_model(net, outputs_of, patch, Backend.EAGER)
    launch_counter.reset()
    got_out, got_grads = _run_model(net, outputs_of, patch, Backend.CUDA)
    assert launch_counter.kernels > 0, "the patched model did not reach libmsda_b200.so"
    assert want_grads, "the model has no deformable attention parameters"
    for got, want in zip(got_out, want_out, strict=True):
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    assert got_grads.keys() == want_grads.keys()
    for key, want in want_grads.items():
        torch.testing.assert_close(got_grads[key], want, rtol=1e-3, atol=1e-4, msg=key)
