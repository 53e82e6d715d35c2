"""GPU parity of the gated attention layer's steps (per-head q/k RMSNorm out of the fused projection
rows, sigmoid output gate) against the oracle and, when the fixture holds them, against the rows the
reference's own ``RMSNorm`` (FlashInfer ``gemma_rmsnorm``) and ``_sigmoid_output_gate`` produced on a
GPU (tests/golden/make_attention_golden.py)."""
import os
import sys

import numpy as np
import pytest
import torch

from async_llm_b200 import attn_layer
from oracle import view_oracle as vo

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_attention_golden as gold  # noqa: E402  (seeded input builder only)

GOLD = os.path.join(HERE, "golden", "attention_golden.npz")


def one_bf16_step(got, want, what):
    g, w = got.float().cpu(), want.float().cpu()
    tol = w.abs() * 2.0 ** -7 + 1e-30
    bad = (g - w).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} values differ by more than one bf16 step"
    frac = (got.cpu() != want.cpu()).float().mean().item()
    assert frac < 0.02, f"{what}: {frac:.3%} of the values are off by a step"


@pytest.mark.parametrize("name", ["d128", "d256"])
def test_qk_norm_and_output_gate(cuda_device, name):
    c = gold.layer_step_inputs()[name]
    n, hq, hkv, d = c["n"], c["hq"], c["hkv"], c["d"]
    qkv = c["qkv"].to(cuda_device)
    qw, kw = (c[k].float().to(cuda_device) for k in ("q_weight", "k_weight"))
    q, k, v = attn_layer.qk_norm(qkv, qw, kw, hq, hkv, d, c["eps"], True)
    gated = attn_layer.output_gate(c["o"].to(cuda_device), qkv, hq, d)
    torch.cuda.synchronize()
    # oracle: the reference's split of the projection rows, then the fp32 formulas
    q_gate, k_in, v_in = c["qkv"].split([2 * hq * d, hkv * d, hkv * d], dim=-1)
    q_gate = q_gate.view(n, hq, 2 * d)
    want_q = vo.qk_rmsnorm(q_gate[..., :d], c["q_weight"], c["eps"]).reshape(n, hq * d)
    want_k = vo.qk_rmsnorm(k_in.reshape(n, hkv, d), c["k_weight"], c["eps"]).reshape(n, hkv * d)
    want_g = vo.sigmoid_output_gate(c["o"].view(n, hq, d), q_gate[..., d:]).reshape(n, hq * d)
    one_bf16_step(q, want_q, "q norm vs oracle")
    one_bf16_step(k, want_k, "k norm vs oracle")
    one_bf16_step(gated, want_g, "output gate vs oracle")
    assert torch.equal(v.cpu(), v_in), "v is a view of the projection rows"
    z = np.load(GOLD) if os.path.exists(GOLD) else {}
    if f"layer/{name}/q" in z:
        bits = lambda key: torch.from_numpy(z[key].copy()).view(torch.bfloat16)
        one_bf16_step(q, bits(f"layer/{name}/q"), "q norm vs reference rows")
        one_bf16_step(k, bits(f"layer/{name}/k"), "k norm vs reference rows")
        one_bf16_step(gated, bits(f"layer/{name}/gated"), "output gate vs reference rows")
        print(f"[layer/{name}] compared with the reference's rows")
    else:
        print(f"[layer/{name}] fixture holds no reference rows for the layer steps; oracle only")
