"""Hugging Face integration: ``patch(model)`` swaps the attention modules (CPU) and the patched
modules / a tiny random-weight Mask2Former agree with upstream Hugging Face (GPU)."""

from __future__ import annotations

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _tiny_mask2former():
    from transformers import Mask2FormerConfig, Mask2FormerForUniversalSegmentation, SwinConfig

    backbone = SwinConfig(image_size=64, patch_size=4, embed_dim=8, depths=[1, 1, 1, 1],
                          num_heads=[1, 1, 1, 1], window_size=2, out_indices=[1, 2, 3, 4])
    config = Mask2FormerConfig(feature_size=32, mask_feature_size=32, hidden_dim=32,
                               num_attention_heads=4, encoder_layers=2, decoder_layers=1,
                               encoder_feedforward_dim=64, dim_feedforward=64, num_queries=10,
                               backbone_config=backbone)
    torch.manual_seed(0)
    return Mask2FormerForUniversalSegmentation(config).eval()


def test_patch_replaces_modules_and_shares_parameters():
    import transformers.models.mask2former.modeling_mask2former as hf

    from deformops_b200.integrations import transformers as ours

    model = _tiny_mask2former()
    originals = [m for m in model.modules()
                 if isinstance(m, hf.Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention)]
    assert len(originals) == 2
    names_before = sorted(n for n, _ in model.named_parameters())
    ours.patch(model)
    patched = [m for m in model.modules()
               if isinstance(m, ours.Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention)]
    assert len(patched) == 2
    assert sorted(n for n, _ in model.named_parameters()) == names_before
    for old, new in zip(originals, patched):
        assert new.value_proj.weight is old.value_proj.weight        # same tensors, no copy
        assert new.sampling_offsets is old.sampling_offsets
    ours.patch(model)                                                  # idempotent
    assert sum(isinstance(m, hf.Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention)
               for m in model.modules()) == 2


@pytest.mark.gpu
@pytest.mark.parametrize("coords", [2, 4])
def test_pixel_decoder_attention_matches_hugging_face(coords):
    import transformers.models.mask2former.modeling_mask2former as hf

    from deformops_b200.integrations import transformers as ours

    torch.manual_seed(1)
    levels = [(8, 8), (4, 4), (2, 2)]
    S = sum(h * w for h, w in levels)
    up = hf.Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention(64, 4, 3, 4).cuda()
    mine = ours.Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention(64, 4, 3, 4).cuda()
    mine.load_state_dict(up.state_dict())
    h = torch.randn(2, S, 64, device="cuda", requires_grad=True)
    pos = torch.randn(2, S, 64, device="cuda")
    ref = torch.rand(2, S, 3, coords, device="cuda")
    starts = torch.tensor([0, 64, 80], device="cuda")
    mask = torch.zeros(2, S, dtype=torch.bool, device="cuda")
    mask[0, :3] = True
    kw = dict(attention_mask=mask, encoder_hidden_states=h, position_embeddings=pos,
              reference_points=ref, spatial_shapes_list=levels, level_start_index=starts)
    out_up, w_up = up(h, output_attentions=True, **kw)
    out_me, w_me = mine(h, output_attentions=True, **kw)
    torch.testing.assert_close(out_me, out_up, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(w_me, w_up, rtol=1e-5, atol=1e-6)
    assert mine(h, **kw)[1] is None
    g = torch.randn_like(out_up)
    grads_up = torch.autograd.grad(out_up, [h, *up.parameters()], g)
    grads_me = torch.autograd.grad(out_me, [h, *mine.parameters()], g)
    for a, b in zip(grads_me, grads_up):
        torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-4)


@pytest.mark.gpu
def test_deformable_detr_core_matches_hugging_face():
    import transformers.models.deformable_detr.modeling_deformable_detr as hf

    from deformops_b200.integrations import transformers as ours

    torch.manual_seed(2)
    levels = [(6, 5), (3, 3)]
    S = sum(h * w for h, w in levels)
    value = torch.randn(2, S, 4, 16, device="cuda")
    loc = torch.rand(2, 7, 4, 2, 4, 2, device="cuda") * 1.2 - 0.1
    attn = torch.randn(2, 7, 4, 8, device="cuda").softmax(-1).view(2, 7, 4, 2, 4)
    shapes = torch.tensor(levels, device="cuda")
    starts = torch.tensor([0, 30], device="cuda")
    expect = hf.MultiScaleDeformableAttention()(value, shapes, levels, starts, loc, attn, 64)
    got = ours.MultiScaleDeformableAttention()(value, shapes, levels, starts, loc, attn, 64)
    torch.testing.assert_close(got, expect, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_tiny_mask2former_patched_equals_unpatched():
    from deformops_b200.integrations import transformers as ours
    from deformops_b200.ops import launch_counter

    model = _tiny_mask2former().cuda()
    pixels = torch.randn(2, 3, 64, 64, device="cuda")
    with torch.no_grad():
        before = model(pixel_values=pixels)
    ours.patch(model)
    launch_counter.reset()
    with torch.no_grad():
        after = model(pixel_values=pixels)
    assert launch_counter.kernels == 2                      # one forward kernel per encoder layer
    torch.testing.assert_close(after.masks_queries_logits, before.masks_queries_logits,
                               rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(after.class_queries_logits, before.class_queries_logits,
                               rtol=1e-3, atol=1e-4)
