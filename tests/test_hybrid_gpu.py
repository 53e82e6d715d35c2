"""The hybrid decoder stack ([GDN, GDN, GDN, attention] pattern) decoding over cache views: the
captured-graph step planned through ``SharedGraphIO`` against the same step run eagerly without
fixed-capacity tables, over several steps with changing topologies and padding rows."""
import pytest
import torch

from async_llm_b200 import AsyncContext
from hybrid_decoder import HybridConfig, HybridDecoder, HybridSession

pytestmark = pytest.mark.gpu


def build(device, dense_fraction):
    cfg = HybridConfig.small()
    model = HybridDecoder(cfg, device, seed=1)
    sess = HybridSession(model, num_pages=400, max_workers=6, depth=3, max_seq_len=1024, dense_fraction=dense_fraction)
    gen = torch.Generator(device=device).manual_seed(5)
    return cfg, sess, gen


@pytest.mark.parametrize("dense_fraction", [0.0, 0.25])
def test_graph_step_matches_eager_step_over_changing_topologies(cuda_device, dense_fraction):
    # two sessions with identical weights and identical synthetic block contents: one runs every step
    # eagerly, the other replays the graph captured once on a dummy topology
    outs = []
    for mode in ("eager", "graph"):
        cfg, sess, gen = build(cuda_device, dense_fraction)
        shared = sess.new_block(300, gen)
        priv = [sess.new_block(n, gen) for n in (40, 77, 130, 9, 65)]
        fresh = sess.new_block(0, gen)
        if mode == "graph":
            sess.capture()
        topologies = [
            [([shared, priv[0]], priv[0]), ([shared, priv[1]], priv[1]), ([shared, priv[2]], priv[2]),
             ([shared, priv[3]], priv[3]), ([shared, priv[4]], priv[4])],
            [([shared, priv[4], priv[0]], priv[0]), ([priv[1]], priv[1]), ([priv[2], shared], priv[2]),
             ([shared], fresh)],
            [([shared, priv[0]], priv[0]), ([shared, priv[1]], priv[1]), ([shared, priv[2]], priv[2]),
             ([shared, priv[3]], priv[3]), ([shared, priv[4]], priv[4]), ([shared, fresh], fresh)],
        ]
        rows = []
        for step, topo in enumerate(topologies):
            contexts = [AsyncContext(cache_view=list(view), output_block=out) for view, out in topo]
            tokens = [(7 * step + 3 * w) % cfg.vocab for w in range(len(contexts))]
            logits = (sess.run_step if mode == "graph" else sess.forward_eager)(contexts, tokens)
            torch.cuda.synchronize()
            sess.sc_attn.check_status()
            rows.append(logits.float().cpu().clone())
        outs.append((rows, [b.num_tokens for b in priv] + [fresh.num_tokens],
                     priv[0].linear_affine[0][1].float().cpu().clone(), fresh.linear_conv_state[0].cpu().clone()))
    (eager_rows, eager_len, eager_B, eager_conv), (graph_rows, graph_len, graph_B, graph_conv) = outs
    assert eager_len == graph_len
    for step, (a, b) in enumerate(zip(eager_rows, graph_rows)):
        assert a.shape == b.shape and torch.isfinite(b).all()
        scale = max(1.0, float(a.abs().max()))
        diff = (a - b).abs() / scale
        # same kernels and the same arithmetic; only the split of the attention work over lanes /
        # tiles differs between a free plan and a fixed-capacity one
        assert diff.max() <= 2e-2 and diff.mean() <= 1e-3, f"step {step}: {float(diff.max())} / {float(diff.mean())}"
    torch.testing.assert_close(graph_B, eager_B, atol=1e-4, rtol=1e-3)
    assert torch.equal(graph_conv, eager_conv)
