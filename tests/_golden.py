"""Loader for the fixtures under tests/golden (made by tests/golden/make_golden.py)."""

from __future__ import annotations

import pathlib

import numpy as np

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"

#: fixtures that store their inputs
FULL_CASES = ["boundary", "small_a", "small_b", "small_c", "small_d", "k8_d64", "ragged",
              "all_outside"]
METHODS = ["linear", "softmax"]


def load(name: str) -> dict[str, np.ndarray]:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


def attn_for(case: dict, method: str) -> np.ndarray:
    return case["attn_logits"] if method == "softmax" else case["attn_linear"]


def rel_err(actual, expected) -> float:
    """The reference tests' metric: max|a-b| / max(max|b|, tiny)."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    if expected.size == 0:
        return 0.0
    return float(np.abs(actual - expected).max() / max(np.abs(expected).max(), 1e-30))


def load_cfg0():
    """Configuration 0: inputs regenerated from the seed and checked against the stored checksum."""
    from deformops_b200.workloads import make_workload

    gold = load("cfg0")
    w = make_workload("cfg0_cpu_fp32", seed=0)
    chk = np.array([
        w.value.double().sum().item(), w.sampling_locations.double().sum().item(),
        w.attention_weights.double().abs().sum().item(), w.attention_logits.double().sum().item(),
        w.grad_output.double().sum().item()])
    if not np.allclose(chk, gold["input_checksum"], rtol=1e-12, atol=1e-9):
        raise AssertionError("workload generator no longer reproduces the fixture's inputs")
    return w, gold
