"""The opt-in region-tiled backward kernel (``MSDA_B200_REGION_BACKWARD=1``): same results as
the oracle.  The switch is read once per process, so the check runs in a child process."""

from __future__ import annotations

import os
import pathlib
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]

_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
from deformops_b200.workloads import make_workload
from oracle import msda_oracle as orc
from tests._abi import abi_backward, dev, to_np
from tests._golden import rel_err

def check(cfg, dtype, softmax, tol, batch=None):
    w = make_workload(cfg, batch=batch)
    attn = w.attention_logits if softmax else w.attention_weights
    v, l, a, go = dev(w.value, dtype), dev(w.sampling_locations, torch.float32), dev(attn, dtype), dev(w.grad_output, dtype)
    gv, gl, ga = abi_backward(v, dev(w.spatial_shapes), dev(w.level_start_index), l, a, go, softmax=softmax)
    e = orc.backward(v.cpu(), w.spatial_shapes, w.level_start_index, l.cpu(), a.cpu(), go.cpu(), softmax=softmax)
    errs = [rel_err(to_np(x), y) for x, y in zip((gv, ga), (e[0], e[2]))]
    assert max(errs) <= tol, (cfg, dtype, softmax, errs)
    assert torch.isfinite(gl).all()
    return errs

print(check("cfg1_m2f_512_bf16", torch.bfloat16, False, 1e-2, batch=2))
print(check("cfg1_m2f_512_bf16", torch.bfloat16, True, 1e-2, batch=1))
print(check("cfg3_detr_enc_fp16", torch.float16, False, 1e-2, batch=1))
print(check("cfg0_cpu_fp32", torch.float32, False, 1e-4))
# Q == S but every query samples everywhere (decoder-like locations): windows miss a lot
odd = dict(batch=1, levels=[(9, 7), (5, 4), (3, 2), (1, 1)], heads=8, head_dim=32, points=4,
           dtype=torch.float32)
print(check(odd, torch.float32, True, 1e-4))
print("region kernel ok")
"""


def test_region_backward_matches_oracle():
    env = dict(os.environ, MSDA_B200_REGION_BACKWARD="1")
    res = subprocess.run([sys.executable, "-c", _CHILD % str(ROOT)], cwd=ROOT, env=env,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "region kernel ok" in res.stdout, res.stdout + res.stderr[-3000:]
