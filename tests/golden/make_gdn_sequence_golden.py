"""Generate tests/golden/gdn_sequence_golden.npz: the reference Gated DeltaNet LAYER run end to end.

    python tests/golden/make_gdn_sequence_golden.py /path/to/reference

The reference layer ``Qwen3_5GatedDeltaNet`` (minisgl/models/qwen3_5_delta.py:264-490) is built
without its constructor (which needs a distributed context), given seeded weights, and driven on
CPU tensors through its async-reasoning entry points with the reference's own eager
``SharedCacheGDN`` (minisgl/shared_cache/gdn.py) and ``CacheBlock`` objects, with the FLA kernels
switched off so that its torch recurrences run (as the reference's own tests do):

  step "s"       one request prefills 130 tokens into an empty block s              (_forward_ar_prefill)
  step "ab"      two requests prefill 70 and 37 tokens into blocks a and b, both    (_forward_ar_prefill,
                 reading s first                                                     batched segments)
  step "decode"  three workers decode one token: views [s, a], [s, b], [c] writing  (_forward_ar_decode)
                 a, b and the new block c
  step "decode2" the same three workers decode another token

Stored: the layer's output rows of every step (bf16 bit patterns) and, after the last step, block
a's conv window and slices of its summary.  ``sequence_inputs()`` is the seeded input builder the
tests call to rebuild the same weights and activations.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))

HIDDEN, HK, HV, DK, DV, KW = 64, 2, 4, 128, 128, 4
KEY_DIM, VALUE_DIM = HK * DK, HV * DV
CONV_DIM = 2 * KEY_DIM + VALUE_DIM
EPS = 1e-6
STEPS = {"s": [130], "ab": [70, 37], "decode": [1, 1, 1], "decode2": [1, 1, 1]}


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def sequence_inputs():
    """Seeded weights of one GDN layer and the hidden rows of every step (bf16)."""
    g = torch.Generator().manual_seed(707)
    bf = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)
    w = dict(
        w_qkv=bf(CONV_DIM, HIDDEN, scale=HIDDEN ** -0.5), w_z=bf(VALUE_DIM, HIDDEN, scale=HIDDEN ** -0.5),
        w_a=bf(HV, HIDDEN, scale=HIDDEN ** -0.5), w_b=bf(HV, HIDDEN, scale=HIDDEN ** -0.5),
        w_out=bf(HIDDEN, VALUE_DIM, scale=VALUE_DIM ** -0.5), conv_weight=bf(CONV_DIM, 1, KW, scale=0.5),
        A_log=torch.randn(HV, generator=g) * 0.5, dt_bias=torch.randn(HV, generator=g),
        norm_weight=torch.rand(DV, generator=g) + 0.5)
    x = {name: bf(sum(lengths), HIDDEN) for name, lengths in STEPS.items()}
    return w, x


class _Linear:
    def __init__(self, weight):
        self.weight = weight

    def forward(self, x):
        return F.linear(x, self.weight)


def reference_layer(w):
    import minisgl.models.qwen3_5_delta as mod

    mod._fla_chunk = None        # the torch recurrences, as the reference's CPU tests run them
    mod._fla_recurrent = None
    layer = mod.Qwen3_5GatedDeltaNet.__new__(mod.Qwen3_5GatedDeltaNet)
    layer.num_k_heads, layer.num_v_heads, layer.head_k_dim, layer.head_v_dim = HK, HV, DK, DV
    layer.key_dim, layer.value_dim, layer.conv_dim, layer.conv_kernel = KEY_DIM, VALUE_DIM, CONV_DIM, KW
    layer._n_rep, layer._lin_idx = HV // HK, 0
    layer.in_proj_qkv, layer.in_proj_z = _Linear(w["w_qkv"]), _Linear(w["w_z"])
    layer.in_proj_a, layer.in_proj_b = _Linear(w["w_a"]), _Linear(w["w_b"])
    layer.out_proj = _Linear(w["w_out"])
    layer.conv1d = mod._Conv1d.__new__(mod._Conv1d)
    layer.conv1d.weight = w["conv_weight"]
    layer.A_log, layer.dt_bias = w["A_log"], w["dt_bias"]
    layer.norm = mod._GatedRMSNorm.__new__(mod._GatedRMSNorm)
    layer.norm.weight, layer.norm._eps = w["norm_weight"], EPS
    return layer


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "python"))
    from minisgl.shared_cache.gdn import SharedCacheGDN
    from minisgl.shared_cache.shared_block import CacheBlock

    torch.manual_seed(0)
    w, x = sequence_inputs()
    layer = reference_layer(w)
    cpu = torch.device("cpu")
    ar = SharedCacheGDN(num_heads=HV, head_k_dim=DK, head_v_dim=DV, conv_dim=CONV_DIM, conv_kernel=KW, device=cpu)
    s, a, b, c = (CacheBlock(cpu, 16) for _ in range(4))
    out = {}
    with torch.no_grad():
        ar.set_context([[s]], [s], prefill_segments=STEPS["s"])
        out["out_s"] = bf16_bits(layer._forward_ar_prefill(x["s"], ar))
        ar.set_context([[s, a], [s, b]], [a, b], prefill_segments=STEPS["ab"])
        out["out_ab"] = bf16_bits(layer._forward_ar_prefill(x["ab"], ar))
        for name in ("decode", "decode2"):
            ar.set_context([[s, a], [s, b], [c]], [a, b, c])
            out[f"out_{name}"] = bf16_bits(layer._forward_ar_decode(x[name], ar))
    A, Bm = a.linear_affine[0]
    out["a_conv"] = bf16_bits(a.linear_conv_state[0].to(torch.bfloat16))
    out["a_A_rows"] = A[0, :, :4, :].float().numpy()
    out["a_B_rows"] = Bm[0, :, :4, :].float().numpy()
    out["c_conv"] = bf16_bits(c.linear_conv_state[0].to(torch.bfloat16))
    out["c_B_rows"] = c.linear_affine[0][1][0, :, :4, :].float().numpy()
    np.savez_compressed(os.path.join(HERE, "gdn_sequence_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_gdn_sequence_golden.py /path/to/reference")
    main(sys.argv[1])
