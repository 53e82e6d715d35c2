"""Generate the golden fixtures of tests/golden/ from the reference implementation.

Run in a container that holds the reference checkout (it is imported, never copied):

    python tests/golden/make_golden.py /path/to/reference

Fixtures written (all inputs are seeded synthetic tensors):
  rope_golden.npz     apply_rope_correction outputs (minisgl/shared_cache/rope_correction.py)
  plan_golden.json    tables emitted by SharedCacheAttention.prepare / prepare_prefill_batch and
                      SharedCacheSession._plan_decode_writes with the FlashInfer wrappers replaced
                      by recorders (the trick of tests/core/test_attention_metadata.py:63-88)
  gdn_golden.npz      _recurrent_gated_delta_rule / _chunk_gated_delta_rule outputs
                      (minisgl/models/qwen3_5_delta.py) and gdn_affine update / compose results
  gdn_bf16_golden.npz  SharedCacheGDN(state_dtype=bfloat16) eager capture / compose results
                      (minisgl/shared_cache/gdn.py:127-269)
  gdn_layer_golden.npz  _decode_conv_silu, Qwen3_5GatedDeltaNet._gates and _GatedRMSNorm.forward outputs
                      (minisgl/models/qwen3_5_delta.py:232-263,296-299) on seeded bf16 inputs
  merge_golden.npz    KV pools, page lists, span overrides and recurrent summaries after
                      SharedCacheSession.merge_blocks / append_block (minisgl/shared_cache/session.py),
                      run on CPU tensors with a list-backed page allocator
"""
import json
import os
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def make_rope(ref):
    from minisgl.shared_cache.rope_correction import apply_rope_correction

    g = torch.Generator().manual_seed(101)
    out = {}
    for name, (n, h, d, max_pos, base, dtype) in {
        "bf16_d128": (33, 4, 128, 4096, 1e6, torch.bfloat16),
        "bf16_d256": (17, 2, 256, 2048, 1e7, torch.bfloat16),
        "bf16_d64": (9, 3, 64, 64, 1e4, torch.bfloat16),
    }.items():
        inv = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.float) / d))
        fr = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv)
        cache = torch.cat((fr.cos(), fr.sin()), dim=-1)
        x = torch.randn(n, h, d, generator=g).to(dtype)
        delta = torch.randint(-max_pos - 5, max_pos + 5, (n,), generator=g)
        delta[0], delta[1], delta[2] = 0, max_pos - 1, -(max_pos - 1)
        y = apply_rope_correction(x, delta, cache)
        out[f"{name}_x"] = bf16_bits(x)
        out[f"{name}_delta"] = delta.numpy()
        out[f"{name}_y"] = bf16_bits(y)
        out[f"{name}_meta"] = np.array([max_pos, base])
    # interleaved mRoPE: 3-axis positions and text positions, signed (query corrections)
    from minisgl.shared_cache.attention import SharedCacheAttention

    for name, (n, h, d, rd, section, base) in {
        "mrope_d128_r64": (21, 3, 128, 64, (11, 11, 10), 1e7),
        "mrope_d256_r64": (13, 2, 256, 64, (11, 11, 10), 1e7),
        "mrope_d128_r128": (9, 2, 128, 128, (24, 20, 20), 1e6),
    }.items():
        a = SharedCacheAttention.__new__(SharedCacheAttention)
        a.device, a.rotary_dim, a.mrope_section = torch.device("cpu"), rd, section
        a._mrope_inv_freq = 1.0 / (base ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        x = torch.randn(n, h, d, generator=g).to(torch.bfloat16)
        pos3 = torch.randint(0, 3000, (3, n), generator=g)
        pos1 = torch.randint(-3000, 3000, (n,), generator=g)
        pos1[0] = 0
        out[f"{name}_x"] = bf16_bits(x)
        out[f"{name}_pos3"], out[f"{name}_pos1"] = pos3.numpy(), pos1.numpy()
        out[f"{name}_y3"] = bf16_bits(a._rope_mrope(x, pos3))
        out[f"{name}_y1"] = bf16_bits(a._rope_mrope(x, pos1))
        out[f"{name}_meta"] = np.array([rd, base, *section])
    np.savez_compressed(os.path.join(HERE, "rope_golden.npz"), **out)


class Plans:
    def plan(self, **kwargs):
        self.last = {k: (v.tolist() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()
                     if k in ("indptr", "indices", "last_page_len", "seq_lens", "qo_indptr",
                              "paged_kv_indptr", "paged_kv_indices", "paged_kv_last_page_len",
                              "max_token_per_sequence", "causal", "page_size")}


def reference_attention(page_size):
    from minisgl.shared_cache.attention import SharedCacheAttention

    a = SharedCacheAttention.__new__(SharedCacheAttention)
    a.device, a.dtype = torch.device("cpu"), torch.bfloat16
    a.num_qo_heads, a.num_kv_heads, a.head_dim = 8, 2, 64
    a.page_size = page_size
    a._plan_event = SimpleNamespace(synchronize=lambda: None, record=lambda: None)
    a.wrapper, a.aux_wrapper = Plans(), Plans()
    a.prefill_ctx_wrapper, a.prefill_self_wrapper = Plans(), Plans()
    return a


def strip_pin():
    for name in ("tensor", "arange", "ones", "empty"):
        original = getattr(torch, name)

        def cpu_only(*args, _original=original, **kwargs):
            kwargs.pop("pin_memory", None)
            return _original(*args, **kwargs)

        setattr(torch, name, cpu_only)
    torch.Tensor.pin_memory = lambda self: self


# Topologies are described symbolically so the test can rebuild them with its own classes:
#   blocks: name -> (pages, length[, span override]) ; views / writes by name
DECODE_TOPOLOGIES = {
    "cross_readers": {
        "blocks": {"common": ([7, 2], "P+1", 1), "left": ([11], "P"), "right": ([], 0), "empty": ([], 0)},
        "views": [["common", "empty", "right", "left"], ["common", "left", "common"]],
        "writes": ["left", "right"],
    },
    "shared_prefix": {
        "blocks": {"s": ([3, 9, 4], "2*P+3"), "a": ([5], 1), "b": ([6, 8], "P+2"), "c": ([], 0)},
        "views": [["s", "a"], ["s", "b"], ["s", "c"], ["s"]],
        "writes": ["a", "b", "c", "c2"],
        "extra_blocks": {"c2": ([10], "P-1")},
    },
    "thinker_writer": {
        "blocks": {"p": ([1, 2], "2*P"), "t": ([3], 2), "w": ([4], "P")},
        "views": [["p", "w", "t"], ["p", "t", "w"]],
        "writes": ["t", "w"],
    },
}


def length_of(expr, P):
    return int(eval(str(expr), {"P": P}))


def build_topology(topo, P, CacheBlock):
    blocks = {}
    spec = dict(topo["blocks"])
    spec.update(topo.get("extra_blocks", {}))
    for name, item in spec.items():
        pages, length = item[0], length_of(item[1], P)
        b = CacheBlock(torch.device("cpu"), P)
        n_pages = -(-length // P) if length else 0
        pages = list(pages)[:n_pages] if n_pages <= len(pages) else list(pages) + [40 + i for i in range(n_pages - len(pages))]
        b.page_starts = [p * P for p in pages]
        b.num_tokens = length
        if len(item) > 2:
            b.mrope_span_override = item[2]
        blocks[name] = b
    return blocks


def make_plans(ref):
    strip_pin()
    from minisgl.shared_cache.attention import PrefillSpec
    from minisgl.shared_cache.session import SharedCacheSession
    from minisgl.shared_cache.shared_block import CacheBlock
    from minisgl.shared_cache.worker_group import WorkerGroup

    out = {"decode": [], "prefill": []}
    for name, topo in DECODE_TOPOLOGIES.items():
        for P in (1, 4, 16):
            blocks = build_topology(topo, P, CacheBlock)
            views = [[blocks[n] for n in v] for v in topo["views"]]
            writes = [blocks[n] for n in topo["writes"]]
            group = WorkerGroup(cache_structure=views, write_to=writes)
            session = SharedCacheSession.__new__(SharedCacheSession)
            session.page_size, session.device = P, torch.device("cpu")
            fresh = iter(range(60, 200))
            session.page_allocator = SimpleNamespace(
                alloc_pages=lambda n: torch.tensor([next(fresh) * P for _ in range(n)], dtype=torch.int32))
            pending, slots, positions = session._plan_decode_writes(group)
            a = reference_attention(P)
            meta = a.prepare(group, pending, slots)
            out["decode"].append({
                "topology": name, "page_size": P,
                "pending": [pending[id(b)] for b in writes],
                "slots": slots.tolist(), "positions": list(positions),
                "sub_worker": meta.sub_worker.tolist(), "sub_loc": meta.sub_loc.tolist(),
                "pad_slot": meta.pad_slot.tolist(), "max_segments": meta.max_segments,
                "n_main": meta.n_main, "n_aux": meta.n_aux,
                "main": getattr(a.wrapper, "last", None), "aux": getattr(a.aux_wrapper, "last", None),
            })
    # prefill: requests over a shared context pool
    for P in (1, 4, 16):
        for case_id, (ctx_lens, new_lens, prefix) in enumerate([
            ([[5, 9], [9], []], [3, 7, 4], [0, 2, 0]),
            ([[2 * P + 1, P, 3]], [P + 5], [P - 1 if P > 1 else 0]),
        ]):
            pool = {}
            specs, desc = [], []
            page_cursor = 100
            for r, (lens, S, T) in enumerate(zip(ctx_lens, new_lens, prefix)):
                ctx = []
                for L in lens:
                    if L not in pool:
                        b = CacheBlock(torch.device("cpu"), P)
                        n_pages = -(-L // P)
                        b.page_starts = [(page_cursor + i) * P for i in range(n_pages)]
                        page_cursor += n_pages
                        b.num_tokens = L
                        pool[L] = b
                    ctx.append(pool[L])
                n_self_pages = -(-(T + S) // P)
                self_pages = torch.tensor([(page_cursor + i) * P for i in range(n_self_pages)], dtype=torch.int32)
                page_cursor += n_self_pages
                specs.append(PrefillSpec(ctx, self_pages, S, T))
                desc.append({"ctx_lens": lens, "ctx_pages": [[s // P for s in b.page_starts] for b in ctx],
                             "self_pages": (self_pages // P).tolist(), "num_new": S, "prefix": T})
            a = reference_attention(P)
            meta = a.prepare_prefill_batch(specs)
            out["prefill"].append({
                "page_size": P, "case": case_id, "requests": desc,
                "sub_worker": meta.sub_worker.tolist(), "sub_loc": meta.sub_loc.tolist(),
                "pad_slot": meta.pad_slot.tolist(), "max_segments": meta.max_segments,
                "n_ctx_rows": meta.n_ctx_rows, "last_indices": meta.last_indices.tolist(),
                "num_rows": meta.num_workers,
                "ctx": getattr(a.prefill_ctx_wrapper, "last", None),
                "self": getattr(a.prefill_self_wrapper, "last", None),
            })
    with open(os.path.join(HERE, "plan_golden.json"), "w") as f:
        json.dump(out, f)


def make_gdn(ref):
    from minisgl.models.qwen3_5_delta import _chunk_gated_delta_rule, _recurrent_gated_delta_rule
    from minisgl.shared_cache.gdn_affine import compose_gdn_affines, init_gdn_affine, update_affine_summary

    g = torch.Generator().manual_seed(404)
    out = {}
    B, T, H, dk, dv = 2, 150, 3, 32, 32
    q = torch.randn(B, T, H, dk, generator=g).to(torch.bfloat16)
    k = torch.randn(B, T, H, dk, generator=g).to(torch.bfloat16)
    v = torch.randn(B, T, H, dv, generator=g).to(torch.bfloat16)
    gate = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=g))
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g))
    s0 = torch.randn(B, H, dk, dv, generator=g) * 0.1
    o_chunk, s_chunk = _chunk_gated_delta_rule(q, k, v, gate, beta, chunk_size=64, initial_state=s0)
    o_rec, s_rec = _recurrent_gated_delta_rule(q, k, v, gate, beta, s0)
    o1, s1 = _recurrent_gated_delta_rule(q[:, :1], k[:, :1], v[:, :1], gate[:, :1], beta[:, :1], s0)
    for name, t in {"q": q, "k": k, "v": v, "o_chunk": o_chunk, "o_rec": o_rec, "o1": o1}.items():
        out[name] = bf16_bits(t)
    for name, t in {"g": gate, "beta": beta, "s0": s0, "s_chunk": s_chunk, "s_rec": s_rec, "s1": s1}.items():
        out[name] = t.float().numpy()
    # affine summaries: per-token update over 5 tokens, then compose of two blocks
    A, Bm = init_gdn_affine(batch_size=B, num_heads=H, d_k=dk, d_v=dv, device="cpu")
    kn = k.float()
    kn = kn * torch.rsqrt((kn * kn).sum(-1, keepdim=True) + 1e-6)
    for t in range(5):
        A, Bm = update_affine_summary(A_hat=A, B_hat=Bm, k=kn[:, t], v=v[:, t].float(),
                                      alpha=gate[:, t].exp(), beta=beta[:, t])
    out["aff_A5"], out["aff_B5"] = A.numpy(), Bm.numpy()
    A2, B2 = init_gdn_affine(batch_size=B, num_heads=H, d_k=dk, d_v=dv, device="cpu")
    for t in range(5, 9):
        A2, B2 = update_affine_summary(A_hat=A2, B_hat=B2, k=kn[:, t], v=v[:, t].float(),
                                       alpha=gate[:, t].exp(), beta=beta[:, t])
    Ac, Bc = compose_gdn_affines(A_first=A, B_first=Bm, A_second=A2, B_second=B2)
    out["aff_Ac"], out["aff_Bc"] = Ac.numpy(), Bc.numpy()
    np.savez_compressed(os.path.join(HERE, "gdn_golden.npz"), **out)


# ---- bf16 summary storage ---------------------------------------------------------------------
BF16_CASE = dict(H=2, dk=128, dv=128, block_tokens={"a": 12, "b": 30, "c": 0, "w0": 3, "w1": 0, "w2": 0},
                 chains=[["a", "c", "b", "w0"], ["b", "w1"], ["c"]], targets=["w0", "w1", "w2"], new_tokens=2)


def gdn_bf16_inputs():
    """Seeded tokens of the bf16-summary case: per block its tokens, then new_tokens per worker."""
    c = BF16_CASE
    g = torch.Generator().manual_seed(808)
    H, dk, dv = c["H"], c["dk"], c["dv"]

    def tokens(T):
        k = torch.randn(T, H, dk, generator=g).to(torch.bfloat16)
        v = torch.randn(T, H, dv, generator=g).to(torch.bfloat16)
        alpha = torch.sigmoid(torch.randn(T, H, generator=g) + 2.0)
        beta = torch.sigmoid(torch.randn(T, H, generator=g))
        return k, v, alpha, beta

    data = {name: tokens(T) for name, T in c["block_tokens"].items()}
    data["new"] = tokens(len(c["targets"]) * c["new_tokens"])
    return data


def make_gdn_bf16(ref):
    """Reference SharedCacheGDN(state_dtype=bfloat16), eager path on CPU: summaries captured block by
    block, the chains composed, two more tokens captured into the write blocks."""
    from minisgl.shared_cache.gdn import SharedCacheGDN
    from minisgl.shared_cache.shared_block import CacheBlock

    c = BF16_CASE
    H, dk, dv = c["H"], c["dk"], c["dv"]
    data = gdn_bf16_inputs()
    cpu = torch.device("cpu")
    ar = SharedCacheGDN(num_heads=H, head_k_dim=dk, head_v_dim=dv, conv_dim=2 * H * dk + H * dv, conv_kernel=4,
                        device=cpu, state_dtype=torch.bfloat16)
    blocks = {name: CacheBlock(cpu, 16) for name in c["block_tokens"]}
    out = {}
    for name, T in c["block_tokens"].items():
        if T == 0:
            continue
        k, v, alpha, beta = data[name]
        ar.set_context([[blocks[name]]], [blocks[name]])
        ar.capture_token_affines(0, k[None], v[None], alpha[None], beta[None])
        A, Bm = blocks[name].linear_affine[0]
        assert A.dtype == torch.bfloat16
        out[f"{name}_A"], out[f"{name}_B"] = bf16_bits(A), bf16_bits(Bm)
    chains = [[blocks[n] for n in ch] for ch in c["chains"]]
    targets = [blocks[n] for n in c["targets"]]
    ar.set_context(chains, targets)
    out["S0"] = ar.compose_initial_recurrent_state(0, torch.float32).numpy()
    k, v, alpha, beta = data["new"]
    W, n = len(targets), c["new_tokens"]
    ar.capture_token_affines(0, k.view(W, n, H, dk), v.view(W, n, H, dv), alpha.view(W, n, H), beta.view(W, n, H))
    for w, t in enumerate(targets):
        A, Bm = t.linear_affine[0]
        out[f"new{w}_A"], out[f"new{w}_B"] = bf16_bits(A), bf16_bits(Bm)
    np.savez_compressed(os.path.join(HERE, "gdn_bf16_golden.npz"), **out)


# ---- block merge / append -------------------------------------------------------------------
MERGE_SHAPE = dict(layers=2, pages=24, P=4, Hkv=2, D=64, max_pos=256, base=1e4, H=2, dk=8, dv=8)


def merge_inputs(CacheBlock):
    """Seeded pools, two blocks and their recurrent summaries; the tests rebuild exactly these with
    their own CacheBlock class."""
    c = MERGE_SHAPE
    g = torch.Generator().manual_seed(505)
    pool = torch.randn(2, c["layers"], c["pages"], c["P"], c["Hkv"], c["D"], generator=g).to(torch.bfloat16)
    inv = 1.0 / (c["base"] ** (torch.arange(0, c["D"], 2, dtype=torch.float) / c["D"]))
    fr = torch.einsum("i,j -> ij", torch.arange(c["max_pos"], dtype=torch.float), inv)
    cos_sin = torch.cat((fr.cos(), fr.sin()), dim=-1)
    left, right = CacheBlock(torch.device("cpu"), c["P"]), CacheBlock(torch.device("cpu"), c["P"])
    left.page_starts = [5 * c["P"], 2 * c["P"]]
    left.num_tokens = 6
    left.mrope_span_override = 9
    left.token_ids = [11, 12, 13, 14, 15, 16]
    right.page_starts = [9 * c["P"], 1 * c["P"]]
    right.num_tokens = 5
    right.token_ids = [21, 22, 23, 24, 25]
    aff = lambda: (torch.randn(1, c["H"], c["dk"], c["dk"], generator=g) * 0.3,
                   torch.randn(1, c["H"], c["dv"], c["dk"], generator=g) * 0.3)
    left_aff = {0: aff(), 2: aff()}
    right_aff = {0: aff(), 1: aff()}
    left_conv = {0: torch.randn(6, 3, generator=g), 2: torch.randn(6, 3, generator=g)}
    right_conv = {0: torch.randn(6, 3, generator=g)}
    free = [p * c["P"] for p in (7, 3, 11, 0, 8, 4, 6, 10)]
    return pool, cos_sin, left, right, left_aff, right_aff, left_conv, right_conv, free


def make_merge(ref):
    from minisgl.shared_cache.attention import SharedCacheAttention
    from minisgl.shared_cache.session import SharedCacheSession
    from minisgl.shared_cache.shared_block import CacheBlock

    c = MERGE_SHAPE
    out = {}

    def fresh_session():
        pool, cos_sin, left, right, la, ra, lc, rc, free = merge_inputs(CacheBlock)
        left._replace_linear_states(dict(la), dict(lc))
        right._replace_linear_states(dict(ra), dict(rc))
        a = SharedCacheAttention.__new__(SharedCacheAttention)
        a.mrope_section, a.rotary_dim, a.head_dim, a.cos_sin_cache = None, c["D"], c["D"], cos_sin
        s = SharedCacheSession.__new__(SharedCacheSession)
        s.device, s.page_size, s.sc_attn, s.sc_gdn = torch.device("cpu"), c["P"], a, None
        s.kv_cache = SimpleNamespace(num_layers=c["layers"], k_cache=lambda i: pool[0, i], v_cache=lambda i: pool[1, i])
        free = list(free)
        s.page_allocator = SimpleNamespace(
            alloc_pages=lambda n: torch.tensor([free.pop(0) for _ in range(n)], dtype=torch.int32))
        return s, pool, left, right

    def record(tag, pool, block):
        out[f"{tag}_pool"] = bf16_bits(pool)
        out[f"{tag}_pages"] = np.array(block.page_starts, np.int64)
        out[f"{tag}_meta"] = np.array([block.num_tokens, -1 if block.mrope_span_override is None
                                       else block.mrope_span_override], np.int64)
        out[f"{tag}_tokens"] = np.array(block.token_ids, np.int64)
        for layer, (A, B) in block.linear_affine.items():
            out[f"{tag}_A{layer}"], out[f"{tag}_B{layer}"] = A.numpy(), B.numpy()
        for layer, conv in block.linear_conv_state.items():
            out[f"{tag}_conv{layer}"] = conv.numpy()

    s, pool, left, right = fresh_session()
    record("merge", pool, s.merge_blocks(left, right))
    s, pool, left, right = fresh_session()
    record("append", pool, s.append_block(left, right))
    s, pool, left, right = fresh_session()
    record("self_append", pool, s.append_block(left, left))
    s, pool, left, right = fresh_session()
    right.num_tokens, right.page_starts, right.token_ids = 0, [], []
    record("merge_empty_right", pool, s.merge_blocks(left, right))
    np.savez_compressed(os.path.join(HERE, "merge_golden.npz"), **out)


PREFILL_CONV_LENGTHS = (7, 2, 1)


def gdn_layer_inputs():
    """Seeded inputs of the GDN layer steps; the tests rebuild exactly these."""
    g = torch.Generator().manual_seed(606)
    W, conv_dim, k, Hv, dv = 5, 96, 4, 6, 128
    bf = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)
    return dict(prior=bf(W, conv_dim, k), qkv=bf(W, conv_dim), weight=bf(conv_dim, 1, k, scale=0.5),
                a=bf(W, Hv, scale=3.0), b=bf(W, Hv, scale=2.0), A_log=torch.randn(Hv, generator=g),
                dt_bias=torch.randn(Hv, generator=g) * 8.0, core=bf(W, Hv, dv, scale=2.0), z=bf(W, Hv, dv),
                norm_weight=torch.rand(dv, generator=g) + 0.5, eps=1e-6,
                prefill_qkv=bf(sum(PREFILL_CONV_LENGTHS), conv_dim),
                prefill_prior=bf(len(PREFILL_CONV_LENGTHS), conv_dim, k))


def make_gdn_layer(ref):
    from minisgl.models.qwen3_5_delta import Qwen3_5GatedDeltaNet, _decode_conv_silu, _GatedRMSNorm

    d = gdn_layer_inputs()
    out = {}
    for tag, prior in (("with_state", d["prior"]), ("no_state", torch.zeros_like(d["prior"]))):
        conv_in = torch.cat([prior, d["qkv"].unsqueeze(-1)], dim=-1)
        out[f"qkv2_{tag}"] = bf16_bits(_decode_conv_silu(conv_in, d["weight"]))
        out[f"state_{tag}"] = bf16_bits(conv_in[..., -d["weight"].shape[-1]:])
    layer = Qwen3_5GatedDeltaNet.__new__(Qwen3_5GatedDeltaNet)
    layer.A_log, layer.dt_bias = d["A_log"], d["dt_bias"]
    beta, gate = layer._gates(d["a"], d["b"])
    out["beta"], out["g"] = bf16_bits(beta), gate.numpy()
    norm = _GatedRMSNorm.__new__(_GatedRMSNorm)
    norm.weight, norm._eps = d["norm_weight"], d["eps"]
    out["normed"] = bf16_bits(norm.forward(d["core"], d["z"]))
    # prefill conv of three requests (lengths 7, 2, 1: the short ones mix prior state into the new
    # state), with and without a prior state, through the reference's own convolution and slicing
    from minisgl.models.qwen3_5_delta import _prefill_conv_silu
    import torch.nn.functional as F

    k = d["weight"].shape[-1]
    for tag in ("prior", "fresh"):
        offset = 0
        for r, length in enumerate(PREFILL_CONV_LENGTHS):
            conv_in = d["prefill_qkv"][offset: offset + length].transpose(0, 1).unsqueeze(0)
            offset += length
            if tag == "prior":
                ctx_tail = d["prefill_prior"][r: r + 1, :, -(k - 1):]
                full_input = torch.cat([ctx_tail, conv_in], dim=-1)
                conv_out = _prefill_conv_silu(full_input, d["weight"], padding=k - 1)
                qkv2 = conv_out[..., k - 1: k - 1 + length]
                new_state = full_input[..., -k:]
            else:
                qkv2 = _prefill_conv_silu(conv_in, d["weight"], padding=k - 1)[..., :length]
                pad = k - length
                new_state = F.pad(conv_in, (pad, 0)) if pad >= 0 else conv_in[..., -k:]
            out[f"prefill_{tag}_qkv2_{r}"] = bf16_bits(qkv2.squeeze(0).transpose(0, 1))
            out[f"prefill_{tag}_state_{r}"] = bf16_bits(new_state.squeeze(0))
    np.savez_compressed(os.path.join(HERE, "gdn_layer_golden.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "python"))
    make_rope(ref)
    make_gdn(ref)
    make_gdn_bf16(ref)
    make_merge(ref)
    make_gdn_layer(ref)
    make_plans(ref)
    print("golden fixtures written to", HERE)
