"""The Gated DeltaNet LAYER end to end on the GPU against the reference layer's outputs.

tests/golden/gdn_sequence_golden.npz holds what ``Qwen3_5GatedDeltaNet._forward_ar_prefill`` /
``_forward_ar_decode`` (minisgl/models/qwen3_5_delta.py:349-490), run on CPU with the reference's
eager ``SharedCacheGDN``, produced for a four-step sequence (a 130-token prefill, a batched prefill of
two requests reading it, two decode steps of three workers); ``GatedDeltaNetLayer`` runs the same
sequence here through the fused kernels (conv -> gates -> core -> gated norm -> projection, back to
back), eagerly and under fixed-capacity buffers replayed from CUDA graphs."""
import os
import sys

import numpy as np
import pytest
import torch

from async_llm_b200.blocks import CacheBlock
from async_llm_b200.gdn_layer import GatedDeltaNetLayer
from async_llm_b200.view_gdn import GDNDecodeBuffers, GDNPrefillBuffers, SharedCacheGDN

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_gdn_sequence_golden as seq  # noqa: E402  (seeded input builder only)

GOLDEN = np.load(os.path.join(HERE, "golden", "gdn_sequence_golden.npz"))


def from_bits(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def close(got, want_bits, what, atol=2e-2, mean=1e-3):
    """The layer's rows come out of the output projection with magnitudes of a few units, where one
    bf16 step is 2^-7 .. 2^-6: the 2e-2 / 1e-3 bounds (stated for outputs of unit scale) are applied
    relative to the scale of the reference rows."""
    g, w = got.float().cpu(), from_bits(want_bits).float()
    assert g.shape == w.shape, f"{what}: {tuple(g.shape)} vs {tuple(w.shape)}"
    scale = max(1.0, float(w.abs().max()))
    d = (g - w).abs() / scale
    print(f"[{what}] max-abs {float(d.max()) * scale:.3e} mean-abs {float(d.mean()) * scale:.3e} (|ref| max {scale:.3f})")
    assert d.max() <= atol and d.mean() <= mean, (f"{what}: max-abs {float(d.max()) * scale:.3g} mean-abs "
                                                   f"{float(d.mean()) * scale:.3g} at scale {scale:.3g}")


def build(device, engine):
    w, x = seq.sequence_inputs()
    dev = lambda t: t.to(device)
    layer = GatedDeltaNetLayer(0, seq.HK, seq.HV, seq.DK, seq.DV, dev(w["w_qkv"]), dev(w["w_z"]), dev(w["w_a"]),
                               dev(w["w_b"]), dev(w["w_out"]), dev(w["conv_weight"]), w["A_log"], w["dt_bias"],
                               w["norm_weight"], seq.EPS)
    ar = SharedCacheGDN(num_heads=seq.HV, head_k_dim=seq.DK, head_v_dim=seq.DV, conv_dim=seq.CONV_DIM,
                        conv_kernel=seq.KW, device=device, num_k_heads=seq.HK, prefill_engine=engine)
    return layer, ar, {k: dev(v) for k, v in x.items()}


def check_blocks(a, c):
    A, Bm = a.linear_affine[0]
    assert torch.equal(a.linear_conv_state[0].cpu().view(torch.int16), torch.from_numpy(GOLDEN["a_conv"]))
    assert torch.equal(c.linear_conv_state[0].cpu().view(torch.int16), torch.from_numpy(GOLDEN["c_conv"]))
    # summaries: the prefill part came from the chunked engine (bf16 operands) or the fp32 scan
    torch.testing.assert_close(A[0, :, :4, :].cpu(), torch.from_numpy(GOLDEN["a_A_rows"]), atol=1e-2, rtol=2e-2)
    torch.testing.assert_close(Bm[0, :, :4, :].cpu(), torch.from_numpy(GOLDEN["a_B_rows"]), atol=1e-2, rtol=2e-2)
    torch.testing.assert_close(c.linear_affine[0][1][0, :, :4, :].cpu(), torch.from_numpy(GOLDEN["c_B_rows"]),
                               atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("engine", ["chunk_tc", "chunk", "scan"])
def test_layer_sequence_matches_reference_layer(cuda_device, engine):
    layer, ar, x = build(cuda_device, engine)
    s, a, b, c = (CacheBlock(cuda_device, 16) for _ in range(4))

    def prefill(chains, targets, segments, rows):
        ar.set_context(chains, targets, prefill_segments=segments)
        ar.prepare_prefill(1, torch.bfloat16, sum(segments))
        out = layer.forward_ar_prefill(rows, ar)
        ar.finish_prefill(True)
        return out

    close(prefill([[s]], [s], seq.STEPS["s"], x["s"]), GOLDEN["out_s"], f"prefill s/{engine}")
    close(prefill([[s, a], [s, b]], [a, b], seq.STEPS["ab"], x["ab"]), GOLDEN["out_ab"], f"prefill a,b/{engine}")
    for name in ("decode", "decode2"):
        ar.set_context([[s, a], [s, b], [c]], [a, b, c])
        ar.prepare_decode(1, torch.bfloat16)
        out = layer.forward_ar_decode(x[name], ar)
        ar.finish_decode(True)
        close(out, GOLDEN[f"out_{name}"], f"{name}/{engine}")
    torch.cuda.synchronize()
    check_blocks(a, c)


def test_layer_sequence_replayed_from_graphs_with_fixed_buffers(cuda_device):
    # the same sequence with every forward replayed from a CUDA graph captured ONCE on a dummy topology:
    # the step's addresses are planned into fixed-capacity tables (more workers / rows / depth than any
    # step uses), inputs are staged into fixed rows, padding rows and requests publish nothing
    layer, ar, x = build(cuda_device, "chunk_tc")
    CAP_W, CAP_ROWS, DEPTH = 4, 160, 3
    dec = GDNDecodeBuffers(ar, 1, CAP_W, DEPTH, torch.bfloat16)
    pre = GDNPrefillBuffers(ar, 1, CAP_W, DEPTH, torch.bfloat16, CAP_ROWS)
    x_dec = torch.zeros(CAP_W, seq.HIDDEN, dtype=torch.bfloat16, device=cuda_device)
    x_pre = torch.zeros(CAP_ROWS, seq.HIDDEN, dtype=torch.bfloat16, device=cuda_device)

    def capture(prefill):
        dummy = [CacheBlock(cuda_device, 16) for _ in range(2)]
        ar.set_context([[d] for d in dummy], dummy, prefill_segments=[3, 2] if prefill else None)
        if prefill:
            ar.prepare_prefill(1, torch.bfloat16, CAP_ROWS, buffers=pre)
            run = lambda: layer.forward_ar_prefill(x_pre, ar)
        else:
            ar.prepare_decode(1, torch.bfloat16, buffers=dec)
            run = lambda: layer.forward_ar_decode(x_dec, ar)
        run()                                  # warm-up outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = run()
        (ar.finish_prefill if prefill else ar.finish_decode)(False)
        torch.cuda.synchronize()
        return graph, out

    g_pre, out_pre = capture(True)
    g_dec, out_dec = capture(False)
    s, a, b, c = (CacheBlock(cuda_device, 16) for _ in range(4))

    def prefill(chains, targets, segments, rows):
        ar.set_context(chains, targets, prefill_segments=segments)
        ar.prepare_prefill(1, torch.bfloat16, CAP_ROWS, buffers=pre)
        x_pre.zero_()
        x_pre[: rows.shape[0]] = rows
        g_pre.replay()
        ar.finish_prefill(True)
        return out_pre[: rows.shape[0]].clone()

    close(prefill([[s]], [s], seq.STEPS["s"], x["s"]), GOLDEN["out_s"], "graph prefill s")
    close(prefill([[s, a], [s, b]], [a, b], seq.STEPS["ab"], x["ab"]), GOLDEN["out_ab"], "graph prefill a,b")
    for name in ("decode", "decode2"):
        ar.set_context([[s, a], [s, b], [c]], [a, b, c])
        ar.prepare_decode(1, torch.bfloat16, buffers=dec)
        x_dec.zero_()
        x_dec[:3] = x[name]
        g_dec.replay()
        ar.finish_decode(True)
        close(out_dec[:3].clone(), GOLDEN[f"out_{name}"], f"graph {name}")
    torch.cuda.synchronize()
    check_blocks(a, c)
    # capacity errors are raised on the host before anything is copied
    many = [CacheBlock(cuda_device, 16) for _ in range(CAP_W + 1)]
    ar.set_context([[m] for m in many], many)
    with pytest.raises(ValueError, match="exceeds the prepared capacity"):
        ar.prepare_decode(1, torch.bfloat16, buffers=dec)
