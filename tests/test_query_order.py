"""Space-filling-curve query ordering (``deformops_b200.query_order``)."""

from __future__ import annotations

import pytest
import torch

from deformops_b200.core.runtime import Method
from deformops_b200.query_order import ReorderingBackend, curve_index, query_permutation
from deformops_b200.registry import MSDABackend


def _grid(bits):
    n = 1 << bits
    ys, xs = torch.meshgrid(torch.arange(n), torch.arange(n), indexing="ij")
    cells = n - 1
    return xs.flatten(), ys.flatten(), xs.flatten() / cells, ys.flatten() / cells


def test_morton_is_bit_interleaving():
    ix, iy, x, y = _grid(4)
    got = curve_index(x, y, "morton", bits=4)
    want = torch.zeros_like(ix)
    for b in range(4):
        want |= ((ix >> b) & 1) << (2 * b)
        want |= ((iy >> b) & 1) << (2 * b + 1)
    assert torch.equal(got, want)
    assert sorted(got.tolist()) == list(range(256))


@pytest.mark.parametrize("bits", [1, 3, 5])
def test_hilbert_visits_every_cell_once_moving_one_step_at_a_time(bits):
    ix, iy, x, y = _grid(bits)
    d = curve_index(x, y, "hilbert", bits=bits)
    n = 1 << bits
    assert sorted(d.tolist()) == list(range(n * n))
    order = torch.argsort(d)
    step = (ix[order][1:] - ix[order][:-1]).abs() + (iy[order][1:] - iy[order][:-1]).abs()
    assert torch.all(step == 1)


def test_curve_index_clamps_and_rejects():
    d = curve_index(torch.tensor([-3.0, 7.0, float("nan")]), torch.tensor([0.0, 1.0, 0.5]), "morton")
    assert d[0] == 0 and d[1] == (1 << 20) - 1
    with pytest.raises(ValueError):
        curve_index(torch.zeros(1), torch.zeros(1), "peano")
    with pytest.raises(ValueError):
        curve_index(torch.zeros(1), torch.zeros(1), bits=40)


class _RowSum(MSDABackend):
    """Stand-in backend: one output row per query that depends on that query alone."""

    name = "rowsum"

    def supports(self, context):
        return True

    def forward(self, value, spatial_shapes, level_start_index, sampling_locations,
                attention_weights, chunk_step, method):
        self.seen = sampling_locations.detach().clone()
        return sampling_locations.sum(dim=(2, 3, 4, 5)).unsqueeze(-1) * attention_weights.sum(
            dim=(2, 3)).unsqueeze(-1) * torch.ones(1, 1, 4)


@pytest.mark.parametrize("curve", ["morton", "hilbert"])
def test_reordering_backend_is_transparent_and_differentiable(curve):
    torch.manual_seed(0)
    B, Q, G, L, K = 2, 33, 2, 2, 3
    loc = torch.rand(B, Q, G, L, K, 2, requires_grad=True)
    attn = torch.rand(B, Q, G, L * K, requires_grad=True)
    inner = _RowSum()
    backend = ReorderingBackend(curve, inner=inner)
    assert backend.name == f"rowsum+{curve}" and backend.supports(None)
    out = backend.forward(None, None, None, loc, attn, 128, Method.LINEAR)
    want = _RowSum().forward(None, None, None, loc, attn, 128, Method.LINEAR)
    torch.testing.assert_close(out, want)
    # the wrapped backend saw the queries in curve order
    perm = query_permutation(loc, curve)
    assert sorted(perm[0].tolist()) == list(range(Q))
    centre = inner.seen.mean(dim=(2, 3, 4))
    keys = curve_index(centre[..., 0], centre[..., 1], curve)
    assert torch.all(keys[:, 1:] >= keys[:, :-1])
    g1 = torch.autograd.grad(out.sum(), [loc, attn])
    g2 = torch.autograd.grad(want.sum(), [loc, attn])
    for a, b in zip(g1, g2):
        torch.testing.assert_close(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("curve", ["morton", "hilbert"])
def test_reordered_kernels_give_the_same_rows(curve):
    from deformops_b200.registry.msda import CudaBackend
    from deformops_b200.workloads import make_workload

    w = make_workload("cfg3_detr_dec_fp16", batch=2).to("cuda")
    args = (w.spatial_shapes, w.level_start_index)
    leaves = [t.detach().clone().requires_grad_() for t in
              (w.value, w.sampling_locations, w.attention_weights)]
    plain = CudaBackend().forward(leaves[0], *args, leaves[1], leaves[2], 128, Method.LINEAR)
    sorted_ = ReorderingBackend(curve).forward(leaves[0], *args, leaves[1], leaves[2], 128,
                                               Method.LINEAR)
    assert torch.equal(plain, sorted_)            # a query's row does not depend on its position
    g1 = torch.autograd.grad(plain, leaves, w.grad_output)
    g2 = torch.autograd.grad(sorted_, leaves, w.grad_output)
    assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2])
    # grad_value sums the same terms in another order (16-bit reductions)
    err = (g1[0].float() - g2[0].float()).abs().max() / g1[0].float().abs().max()
    assert err <= 1e-2
