"""Seeded synthetic MSDA workloads with the shapes of the pixel-decoder use case.

Stands in for the Mask2Former / Deformable-DETR encoder inputs the benchmark
configurations are named after: no dataset item is used, only their shapes and
value distributions.

* ``value ~ N(0, 1)``, shape ``(B, S, G, D)``.
* Encoder queries enumerate the pixels of every level (level-major, row-major),
  so ``Q == S``.  The reference point of the query at pixel ``(x, y)`` of an
  ``H x W`` level is ``((x + 0.5) / W, (y + 0.5) / H)``, shared by all sampled
  levels; ``sampling_locations = reference point + N(0, 0.05^2)`` independently
  per (batch, query, head, level, point, axis), kept in float32.
* Decoder queries (``num_queries`` given) draw reference points uniformly from
  ``[0, 1]^2`` per (batch, query).
* ``attention_weights = softmax over L*K of N(0, 1)`` logits, cast to the value
  dtype; the raw logits are kept for the in-kernel-softmax variant.
* ``grad_output ~ N(0, 1)``, shape ``(B, Q, G*D)``.

Every sample is generated from its own generator seeded with
``(seed, global sample index)``, so a batch slice held by one rank is identical
no matter how many ranks share the global batch.
"""

from __future__ import annotations

import dataclasses
from typing import Sequence

import torch

__all__ = ["CONFIGS", "Workload", "level_tables", "make_workload", "encoder_reference_points"]

#: Named shapes: levels are (height, width) rows; "dtype" is the value dtype.
CONFIGS: dict[str, dict] = {
    # CPU-runnable case
    "cfg0_cpu_fp32": dict(batch=2, levels=[(32, 32), (16, 16), (8, 8)], heads=8, head_dim=32,
                          points=4, dtype=torch.float32),
    # Mask2Former pixel decoder, 512 x 512 input
    "cfg1_m2f_512_bf16": dict(batch=8, levels=[(64, 64), (32, 32), (16, 16)], heads=8,
                              head_dim=32, points=4, dtype=torch.bfloat16),
    # Mask2Former pixel decoder, 1024 x 1024 input (headline, 21 504 queries per sample)
    "cfg2_m2f_1024_bf16": dict(batch=4, levels=[(128, 128), (64, 64), (32, 32)], heads=8,
                               head_dim=32, points=4, dtype=torch.bfloat16),
    # Deformable-DETR encoder
    "cfg3_detr_enc_fp16": dict(batch=4, levels=[(100, 134), (50, 67), (25, 34), (13, 17)],
                               heads=8, head_dim=32, points=4, dtype=torch.float16),
    "cfg3_detr_enc_fp32": dict(batch=4, levels=[(100, 134), (50, 67), (25, 34), (13, 17)],
                               heads=8, head_dim=32, points=4, dtype=torch.float32),
    # Deformable-DETR decoder cross-attention: 300 queries over the same value tensor
    "cfg3_detr_dec_fp16": dict(batch=4, levels=[(100, 134), (50, 67), (25, 34), (13, 17)],
                               heads=8, head_dim=32, points=4, dtype=torch.float16,
                               num_queries=300),
}


@dataclasses.dataclass
class Workload:
    """One batch of operator inputs plus the upstream gradient."""

    value: torch.Tensor               # (B, S, G, D)
    spatial_shapes: torch.Tensor      # (L, 2) int64, rows (H, W)
    level_start_index: torch.Tensor   # (L,) int64
    sampling_locations: torch.Tensor  # (B, Q, G, L, K, 2) float32
    attention_weights: torch.Tensor   # (B, Q, G, L*K) value dtype, normalised
    attention_logits: torch.Tensor    # (B, Q, G, L*K) value dtype, raw
    grad_output: torch.Tensor         # (B, Q, G*D)

    @property
    def dims(self) -> tuple[int, int, int, int, int, int, int]:
        B, S, G, D = self.value.shape
        _, Q, _, L, K, _ = self.sampling_locations.shape
        return B, S, G, D, Q, L, K

    def to(self, device, non_blocking: bool = False) -> "Workload":
        return Workload(*[getattr(self, f.name).to(device, non_blocking=non_blocking)
                          for f in dataclasses.fields(self)])

    def algorithmic_bytes(self) -> tuple[int, int]:
        """Compulsory bytes of one forward and one backward call.

        Forward: value, locations and weights read once, output written once.
        Backward: value, locations, weights and grad_output read once;
        grad_value, grad_loc and grad_attn written once.
        """
        B, S, G, D, Q, L, K = self.dims
        e = self.value.element_size()
        e_loc = self.sampling_locations.element_size()
        P = L * K
        val = B * S * G * D * e
        loc = B * Q * G * P * 2 * e_loc
        att = B * Q * G * P * e
        out = B * Q * G * D * e
        return val + loc + att + out, (val + loc + att + out) + (val + loc + att)


def level_tables(levels: Sequence[tuple[int, int]], device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """``spatial_shapes`` (L,2) and ``level_start_index`` (L,), both int64."""
    shapes = torch.tensor(list(levels), dtype=torch.int64, device=device).reshape(-1, 2)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cumsum(sizes, 0) - sizes
    return shapes, starts


def encoder_reference_points(levels: Sequence[tuple[int, int]]) -> torch.Tensor:
    """Pixel-centre reference points ``(S, 2)`` as (x, y), level-major then row-major."""
    pts = []
    for h, w in levels:
        ys = (torch.arange(h, dtype=torch.float32) + 0.5) / h
        xs = (torch.arange(w, dtype=torch.float32) + 0.5) / w
        gy, gx = torch.meshgrid(ys, xs, indexing="ij")
        pts.append(torch.stack([gx.reshape(-1), gy.reshape(-1)], -1))
    return torch.cat(pts, 0)


def _one_sample(index: int, seed: int, levels, heads, head_dim, points, num_queries, ref_enc):
    gen = torch.Generator(device="cpu")
    gen.manual_seed((seed * 1_000_003 + index) & 0x7FFFFFFFFFFFFFFF)
    S = sum(h * w for h, w in levels)
    L = len(levels)
    value = torch.randn(S, heads, head_dim, generator=gen)
    if num_queries is None:
        ref = ref_enc
    else:
        ref = torch.rand(num_queries, 2, generator=gen)
    Q = ref.shape[0]
    offsets = torch.randn(Q, heads, L, points, 2, generator=gen) * 0.05
    loc = ref.view(Q, 1, 1, 1, 2) + offsets
    logits = torch.randn(Q, heads, L * points, generator=gen)
    grad_out = torch.randn(Q, heads * head_dim, generator=gen)
    return value, loc, logits, grad_out


def make_workload(name_or_cfg, *, batch: int | None = None, first_sample: int = 0,
                  seed: int = 0, device="cpu") -> Workload:
    """Build a workload by config name (see :data:`CONFIGS`) or from a dict.

    ``batch`` overrides the config's batch; ``first_sample`` is the global index
    of this slice's first sample (for batch sharding across ranks).
    """
    cfg = dict(CONFIGS[name_or_cfg]) if isinstance(name_or_cfg, str) else dict(name_or_cfg)
    levels = [tuple(x) for x in cfg["levels"]]
    heads, head_dim, points = cfg["heads"], cfg["head_dim"], cfg["points"]
    dtype = cfg.get("dtype", torch.float32)
    num_queries = cfg.get("num_queries")
    B = cfg["batch"] if batch is None else batch
    ref_enc = encoder_reference_points(levels) if num_queries is None else None
    vals, locs, logit_list, gos = [], [], [], []
    for i in range(B):
        v, l, a, g = _one_sample(first_sample + i, seed, levels, heads, head_dim, points,
                                 num_queries, ref_enc)
        vals.append(v)
        locs.append(l)
        logit_list.append(a)
        gos.append(g)
    shapes, starts = level_tables(levels)
    logits32 = torch.stack(logit_list)
    wl = Workload(
        value=torch.stack(vals).to(dtype),
        spatial_shapes=shapes,
        level_start_index=starts,
        sampling_locations=torch.stack(locs),
        attention_weights=torch.softmax(logits32, -1).to(dtype),
        attention_logits=logits32.to(dtype),
        grad_output=torch.stack(gos).to(dtype),
    )
    return wl.to(device) if str(device) != "cpu" else wl
