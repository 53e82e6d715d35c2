"""CPU restatement of the cache-view attention path (torch, fp32 accumulation).

TEST INFRASTRUCTURE: the checker the CUDA kernels are compared with, and the timed CPU baseline.

Pinning status
--------------
* ``rope_mrope``      -- PINNED: bit-equal to the reference ``SharedCacheAttention._rope_mrope``
                         (minisgl/shared_cache/attention.py:257-280) on ``tests/golden/rope_golden.npz``
                         (``mrope_*`` entries, generated from the reference).
* ``rope_delta``      -- PINNED: bit-equal to the reference ``apply_rope_correction``
                         (minisgl/shared_cache/rope_correction.py:15-54) on the committed golden
                         vectors ``tests/golden/rope_*.npz`` (generated from the reference).
* ``plan_decode`` / ``plan_prefill`` -- PINNED: equal to the tables the reference planners emit
                         (minisgl/shared_cache/attention.py:282-622), golden ``tests/golden/plan_*.json``.
* ``view_decode`` / ``view_prefill`` -- PINNED on ``tests/golden/attention_golden.npz``: output rows
  of the unmodified reference ``SharedCacheAttention.prepare`` / ``prepare_prefill_batch`` +
  ``forward`` (minisgl/shared_cache/attention.py:282-752; its attention core is the third-party
  ``flashinfer`` paged decode / prefill kernels with backend "fa2" and ``merge_states``) run on a
  B200 on the seeded cases of ``tests/attention_cases.py`` by ``tests/golden/make_attention_golden.py``
  (FlashInfer 0.6.11.post2 -- the reference pins 0.6.17 -- and the reference's own ``MHAKVCache``
  store kernel).  ``tests/test_attention_golden_cpu.py`` compares this restatement with those rows
  (max-abs 1e-4 .. 4e-3, i.e. one bf16 step of the output magnitude; the keys it stores are equal bit
  for bit).  The restatement: softmax(q.k^T / sqrt(D)) in fp32 over each paged segment, outputs
  combined by log-sum-exp weights, which equals one softmax over the concatenated view
  (attention.py:4-41 module docstring, :624-752).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- RoPE
def make_cos_sin_cache(rotary_dim: int, max_pos: int, base: float) -> torch.Tensor:
    """``[max_pos, rotary_dim]`` fp32, cos then sin (minisgl/layers/rotary.py:24-32)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def rope_delta(x: torch.Tensor, delta: torch.Tensor, cos_sin: torch.Tensor,
               rotary_dim: Optional[int] = None) -> torch.Tensor:
    """Rotate ``x [N, heads, D]`` by signed integer offsets ``delta [N]``.

    Follows rope_correction.py:33-54: table row ``min(|delta|, max_pos-1)``, sin negated for
    negative offsets, fp32 products and sums, cast back; with ``rotary_dim < D`` only the first
    ``rotary_dim`` dims rotate (attention.py:250-255).
    """
    D = x.shape[-1]
    rd = D if rotary_dim is None else rotary_dim
    half = rd // 2
    idx = delta.abs().clamp(max=cos_sin.shape[0] - 1).long()
    cos = cos_sin[idx, :half].unsqueeze(1)
    sin = cos_sin[idx, half:rd].unsqueeze(1)
    sin = torch.where((delta < 0).view(-1, 1, 1), -sin, sin)
    a = x[..., :half].to(cos.dtype)
    b = x[..., half:rd].to(cos.dtype)
    rot = torch.cat((cos * a - sin * b, cos * b + sin * a), dim=-1).to(x.dtype)
    if rd == D:
        return rot
    return torch.cat((rot, x[..., rd:]), dim=-1)


def mrope_inv_freq(rotary_dim: int, base: float) -> torch.Tensor:
    """Frequencies of the interleaved mRoPE rotation (attention.py:170-174)."""
    return 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def rope_mrope(x: torch.Tensor, corrections: torch.Tensor, inv_freq: torch.Tensor,
               mrope_section: Sequence[int], rotary_dim: int) -> torch.Tensor:
    """Interleaved 3-axis mRoPE of ``x [N, heads, D]`` at positions ``[N]`` or ``[3, N]``.

    Follows attention.py:257-280: the angles of axis 0 everywhere, those of axis 1 (2) at
    frequencies ``1, 4, 7, ...`` (``2, 5, 8, ...``) below ``3 * section``; cos and sin are cast to
    ``x``'s dtype and the products and the sum are formed in that dtype."""
    pos = corrections.float()
    pos3 = pos if pos.dim() == 2 else pos[None, :].expand(3, -1)
    freqs3 = pos3[:, :, None] * inv_freq[None, None, :]
    freqs = freqs3[0].clone()
    for dim, offset in ((1, 1), (2, 2)):
        idx = slice(offset, mrope_section[dim] * 3, 3)
        freqs[..., idx] = freqs3[dim][..., idx]
    emb = torch.cat((freqs, freqs), dim=-1)
    cos = emb.cos().to(x.dtype)[:, None, :]
    sin = emb.sin().to(x.dtype)[:, None, :]
    x_rot, x_pass = x[..., :rotary_dim], x[..., rotary_dim:]
    x1, x2 = x_rot[..., : rotary_dim // 2], x_rot[..., rotary_dim // 2:]
    x_rot = x_rot * cos + torch.cat((-x2, x1), dim=-1) * sin
    return torch.cat([x_rot, x_pass], dim=-1)


def mrope_cos_sin_cache(rotary_dim: int, max_pos: int, base: float) -> torch.Tensor:
    """``[max_pos, rotary_dim]`` fp32 table whose row p holds the cos | sin that ``rope_mrope``
    computes on the fly for position p (same products ``p * inv_freq`` in fp32)."""
    freqs = torch.arange(max_pos, dtype=torch.float32)[:, None] * mrope_inv_freq(rotary_dim, base)[None, :]
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


# --------------------------------------------------------------------------- KV store
def store_kv(k_pool: torch.Tensor, v_pool: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
             positions: Optional[torch.Tensor], out_loc: torch.Tensor, cos_sin: Optional[torch.Tensor],
             rotary_dim: Optional[int] = None) -> None:
    """Rotate ``k [n, Hkv, D]`` at ``positions`` and write k, v to ``pool.view(-1, Hkv, D)[out_loc]``;
    negative slots are skipped (attention.py:645-649, kernel/csrc/jit/store.cu:41-52)."""
    kf = k_pool.view(-1, k_pool.shape[-2], k_pool.shape[-1])
    vf = v_pool.view(-1, v_pool.shape[-2], v_pool.shape[-1])
    kr = k.reshape(k.shape[0], kf.shape[1], kf.shape[2])
    if positions is not None:
        kr = rope_delta(kr, positions, cos_sin, rotary_dim)
    vr = v.reshape(v.shape[0], vf.shape[1], vf.shape[2])
    keep = out_loc >= 0
    kf[out_loc[keep].long()] = kr[keep]
    vf[out_loc[keep].long()] = vr[keep]


# --------------------------------------------------------------------------- planners
def plan_decode(group, new_page_for_block: Dict[int, Optional[int]], new_token_slots: Sequence[int],
                page_size: int) -> Dict[str, list]:
    """Per-(worker, segment) sub-requests of one decode step (attention.py:302-372, 430-433).

    Returns the reference's tables: main/aux sub-request lists and the scatter slots.
    """
    P = page_size
    written = set(new_page_for_block)
    main = {"worker": [], "loc": [], "slot": [], "pages": [], "seq_len": [], "last_page_len": []}
    aux = {"worker": [], "loc": [], "slot": [], "kv_slot": []}
    widest = 0
    for w, (view, wt) in enumerate(zip(group.cache_structure, group.write_to)):
        lengths = [b.num_tokens + (id(b) in written) for b in view]
        spans = [b.mrope_span + (id(b) in written) for b in view]
        total, before, n_seg = sum(spans), 0, 0
        for b, length, span in zip(view, lengths, spans):
            if length:
                pages = [s // P for s in b.page_starts]
                extra = new_page_for_block.get(id(b))
                if extra is not None:
                    pages.append(extra // P)
                main["worker"].append(w)
                main["loc"].append(total - before - 1)
                main["slot"].append(n_seg)
                main["pages"].append(pages)
                main["seq_len"].append(length)
                main["last_page_len"].append(length - (len(pages) - 1) * P)
                n_seg += 1
            before += span
        if not any(b is wt for b in view):
            aux["worker"].append(w)
            aux["loc"].append(wt.mrope_span)
            aux["slot"].append(n_seg)
            aux["kv_slot"].append(int(new_token_slots[w]))
            n_seg += 1
        widest = max(widest, n_seg)
    sub_worker = main["worker"] + aux["worker"]
    sub_slot = main["slot"] + aux["slot"]
    return {
        "main": main, "aux": aux, "max_segments": widest,
        "sub_worker": sub_worker, "sub_loc": main["loc"] + aux["loc"],
        "pad_slot": [w * widest + s for w, s in zip(sub_worker, sub_slot)],
    }


# --------------------------------------------------------------------------- attention core
def _gather_segment(k_pool, v_pool, pages: List[int], length: int, page_size: int, tok0: int = 0):
    kf = k_pool.view(-1, k_pool.shape[-2], k_pool.shape[-1])
    vf = v_pool.view(-1, v_pool.shape[-2], v_pool.shape[-1])
    pg = torch.tensor(pages, dtype=torch.long)
    slots = (pg[:, None] * page_size + torch.arange(page_size)[None, :]).reshape(-1)[tok0: tok0 + length]
    return kf[slots], vf[slots]


def attend_segments(q_rows: torch.Tensor, segments: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]],
                    num_kv_heads: int, sm_scale: float) -> torch.Tensor:
    """One query position against several segments.

    ``segments`` holds ``(q_rot [Hq, D] bf16, K [L, Hkv, D], V [L, Hkv, D], mask [L] or None)``.
    Scores are fp32 dot products of the bf16-rounded rotated query with the stored keys;
    the softmax runs over the concatenation (== per-segment softmax + LSE merge).
    Returns fp32 ``[Hq, D]``.
    """
    Hq, D = q_rows.shape
    g = Hq // num_kv_heads
    scores, values = [], []
    for q_rot, K, V, mask in segments:
        qf = q_rot.float().view(num_kv_heads, g, D)
        s = torch.einsum("hgd,lhd->hgl", qf, K.float()) * sm_scale
        if mask is not None:
            s = s.masked_fill(~mask.view(1, 1, -1), float("-inf"))
        scores.append(s)
        values.append(V.float())
    s = torch.cat(scores, dim=-1)
    p = torch.softmax(s, dim=-1)
    v = torch.cat(values, dim=0)
    out = torch.einsum("hgl,lhd->hgd", p, v)
    return out.reshape(Hq, D)


def view_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, group,
                new_page_for_block: Dict[int, Optional[int]], new_token_slots: Sequence[int],
                cos_sin: torch.Tensor, num_q_heads: int, rotary_dim: Optional[int] = None,
                sm_scale: Optional[float] = None) -> torch.Tensor:
    """Decode attention over each worker's view; the new K/V must already be in the pool.

    ``q [W, Hq*D]`` unrotated bf16.  Returns fp32 ``[W, Hq*D]`` (attention.py:651-703).
    """
    _, P, Hkv, D = k_pool.shape
    scale = D ** -0.5 if sm_scale is None else sm_scale
    plan = plan_decode(group, new_page_for_block, new_token_slots, P)
    W = len(group.write_to)
    qh = q.view(W, num_q_heads, D)
    per_worker: List[list] = [[] for _ in range(W)]
    m = plan["main"]
    for w, loc, pages, length in zip(m["worker"], m["loc"], m["pages"], m["seq_len"]):
        K, V = _gather_segment(k_pool, v_pool, pages, length, P)
        q_rot = rope_delta(qh[w: w + 1], torch.tensor([loc]), cos_sin, rotary_dim)[0]
        per_worker[w].append((q_rot, K, V, None))
    a = plan["aux"]
    for w, loc, slot in zip(a["worker"], a["loc"], a["kv_slot"]):
        K, V = _gather_segment(k_pool, v_pool, [slot // P], 1, P, tok0=slot % P)
        q_rot = rope_delta(qh[w: w + 1], torch.tensor([loc]), cos_sin, rotary_dim)[0]
        per_worker[w].append((q_rot, K, V, None))
    out = torch.zeros(W, num_q_heads, D, dtype=torch.float32)
    for w in range(W):
        out[w] = attend_segments(qh[w], per_worker[w], Hkv, scale)
    return out.view(W, -1)


def plan_prefill(specs, page_size: int) -> Dict[str, list]:
    """Reference tables of a batched view-conditioned prefill (attention.py:507-550).

    ``specs`` are objects with ``context`` (blocks), ``self_page_starts``, ``num_new``,
    ``self_prefix_len``, ``self_prefix_span``.
    """
    P = page_size
    widest = max(len(s.context) + 1 for s in specs)
    ctx = {"rows": [], "slot": [], "loc": [], "pages": [], "q_len": [], "seq_len": [], "last_page_len": []}
    own = {"rows": [], "slot": [], "loc": [], "pages": [], "q_len": [], "seq_len": [], "last_page_len": []}
    last, offset = [], 0
    for spec in specs:
        S, T = int(spec.num_new), int(spec.self_prefix_len)
        T_span = T if spec.self_prefix_span is None else int(spec.self_prefix_span)
        spans = [b.mrope_span for b in spec.context]
        self_offset = sum(spans) + T_span
        rows = list(range(offset, offset + S))
        prefix = 0
        for j, (block, span) in enumerate(zip(spec.context, spans)):
            ctx["rows"] += rows
            ctx["slot"] += [j] * S
            ctx["loc"] += [i + self_offset - prefix for i in range(S)]
            ctx["pages"].append([s // P for s in block.page_starts])
            ctx["q_len"].append(S)
            ctx["seq_len"].append(block.num_tokens)
            ctx["last_page_len"].append(block.last_page_len)
            prefix += span
        pages = [int(s) // P for s in spec.self_page_starts.tolist()]
        own["rows"] += rows
        own["slot"] += [len(spec.context)] * S
        own["loc"] += [i + T_span for i in range(S)]
        own["pages"].append(pages)
        own["q_len"].append(S)
        own["seq_len"].append(T + S)
        own["last_page_len"].append(T + S - (len(pages) - 1) * P)
        last.append(offset + S - 1)
        offset += S
    gather = ctx["rows"] + own["rows"]
    slot = ctx["slot"] + own["slot"]
    return {"ctx": ctx, "self": own, "max_segments": widest, "num_rows": offset,
            "sub_worker": gather, "sub_loc": ctx["loc"] + own["loc"],
            "pad_slot": [r * widest + s for r, s in zip(gather, slot)],
            "n_ctx_rows": len(ctx["rows"]), "last_indices": last}


def view_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, specs,
                 cos_sin: torch.Tensor, num_q_heads: int, rotary_dim: Optional[int] = None,
                 sm_scale: Optional[float] = None, mrope=None) -> torch.Tensor:
    """View-conditioned prefill; the new K/V must already be in the pool.

    Row ``i`` of request ``r`` attends to every token of each context block (query rotated by
    ``i + self_offset - prefix_j``) and to tokens ``0 .. T+i`` of its own block (query rotated by
    ``i + T_span``); one fp32 softmax over the concatenation (attention.py:705-752, :586-587 for
    the end-aligned causal mask).  Returns fp32 ``[N, Hq*D]``.

    ``mrope = (inv_freq, mrope_section)`` switches the query rotation to the interleaved 3-axis
    form: a request's ``spec.mrope_rel [3, S]`` (token index on all axes without one) replaces the
    token index in both rotations, the causal mask stays on token indices (attention.py:118-127,
    :516-537).
    """
    def rotate(x, rel_tok, rel3, shift):
        if mrope is None:
            return rope_delta(x, rel_tok + shift, cos_sin, rotary_dim)
        return rope_mrope(x, rel3 + shift, mrope[0], mrope[1], D if rotary_dim is None else rotary_dim)

    _, P, Hkv, D = k_pool.shape
    scale = D ** -0.5 if sm_scale is None else sm_scale
    N = sum(int(s.num_new) for s in specs)
    qh = q.view(N, num_q_heads, D)
    out = torch.zeros(N, num_q_heads, D, dtype=torch.float32)
    g = num_q_heads // Hkv
    offset = 0
    for spec in specs:
        S, T = int(spec.num_new), int(spec.self_prefix_len)
        T_span = T if spec.self_prefix_span is None else int(spec.self_prefix_span)
        spans = [b.mrope_span for b in spec.context]
        self_offset = sum(spans) + T_span
        rel = torch.arange(S)
        rel3 = getattr(spec, "mrope_rel", None)
        rel3 = rel.view(1, -1).expand(3, -1) if rel3 is None else rel3.long()
        scores, values = [], []
        prefix = 0
        qs = qh[offset: offset + S]
        for block, span in zip(spec.context, spans):
            K, V = _gather_segment(k_pool, v_pool, [s // P for s in block.page_starts], block.num_tokens, P)
            q_rot = rotate(qs, rel, rel3, self_offset - prefix)
            s_ = torch.einsum("shgd,lhd->shgl", q_rot.float().view(S, Hkv, g, D), K.float()) * scale
            scores.append(s_)
            values.append(V.float())
            prefix += span
        pages = [int(s) // P for s in spec.self_page_starts.tolist()]
        K, V = _gather_segment(k_pool, v_pool, pages, T + S, P)
        q_rot = rotate(qs, rel, rel3, T_span)
        s_ = torch.einsum("shgd,lhd->shgl", q_rot.float().view(S, Hkv, g, D), K.float()) * scale
        visible = torch.arange(T + S)[None, :] <= (T + rel)[:, None]
        s_ = s_.masked_fill(~visible[:, None, None, :], float("-inf"))
        scores.append(s_)
        values.append(V.float())
        p = torch.softmax(torch.cat(scores, dim=-1), dim=-1)
        v = torch.cat(values, dim=0)
        out[offset: offset + S] = torch.einsum("shgl,lhd->shgd", p, v).reshape(S, num_q_heads, D)
        offset += S
    return out.view(N, -1)


def plain_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, slot_rows: Sequence[Sequence[int]],
                    extend_lens: Sequence[int], num_q_heads: int, sm_scale: Optional[float] = None) -> torch.Tensor:
    """Causal paged attention of ordinary (view-less) batches: what the reference's stock backends
    compute (minisgl/attention/fi.py:176-188, FlashInfer paged prefill with ``causal=True`` /
    paged decode over ``page_table[table_idx, :device_len]``, page size 1).

    Request ``r`` has keys at token slots ``slot_rows[r]`` (all already in the pool, the new ones
    last) and ``extend_lens[r]`` query rows; query row ``i`` sees keys ``0 .. len - extend + i``.
    ``q [rows, Hq*D]`` is used as given (the layer rotated it).  Returns fp32 ``[rows, Hq*D]``.
    """
    Hkv, D = k_pool.shape[-2], k_pool.shape[-1]
    scale = D ** -0.5 if sm_scale is None else sm_scale
    g = num_q_heads // Hkv
    kf, vf = k_pool.reshape(-1, Hkv, D).float(), v_pool.reshape(-1, Hkv, D).float()
    rows = sum(int(e) for e in extend_lens)
    qh = q.reshape(rows, num_q_heads, D).float()
    out = torch.zeros(rows, num_q_heads, D)
    off = 0
    for slots, S in zip(slot_rows, extend_lens):
        S = int(S)
        idx = torch.as_tensor(list(slots), dtype=torch.long)
        L = idx.numel()
        K, V = kf[idx], vf[idx]
        s_ = torch.einsum("shgd,lhd->shgl", qh[off: off + S].view(S, Hkv, g, D), K) * scale
        visible = torch.arange(L)[None, :] <= (L - S + torch.arange(S))[:, None]
        s_ = s_.masked_fill(~visible[:, None, None, :], float("-inf"))
        out[off: off + S] = torch.einsum("shgl,lhd->shgd", torch.softmax(s_, dim=-1), V).reshape(S, num_q_heads, D)
        off += S
    return out.view(rows, -1)


# --------------------------------------------------------------------------- gated attention layer steps
def qk_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, weight_plus_one: bool = True) -> torch.Tensor:
    """Per-head RMSNorm of ``x [..., D]``: ``x * rsqrt(mean(x^2) + eps) * (weight [+ 1])`` in fp32, one cast
    back -- the published semantics of FlashInfer's ``gemma_rmsnorm`` / ``rmsnorm``, which the reference's
    ``RMSNorm`` calls (minisgl/layers/norm.py:8-22; used at models/qwen3_5_attn.py:53-54,113-114)."""
    xf = x.float()
    w = weight.float() + (1.0 if weight_plus_one else 0.0)
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w).to(x.dtype)


def sigmoid_output_gate(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``(o.float() * gate.float().sigmoid()).to(o.dtype)`` (models/qwen3_5_attn.py:21-23)."""
    return (o.float() * gate.float().sigmoid()).to(o.dtype)
