"""Seeded synthetic cache-view workloads (the shapes of the benchmark configurations).

Everything is generated on the CPU from ``torch.Generator`` seeds so that the CUDA path, the CPU
oracle and the golden fixtures see identical bits; ``ViewCase.to(device)`` moves a case to the GPU.
Pool pages are dealt from a seeded random permutation, so page tables are never contiguous.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from async_llm_b200.blocks import CacheBlock, WorkerGroup


def cos_sin_table(rotary_dim: int, max_pos: int, base: float) -> torch.Tensor:
    """fp32 ``[max_pos, rotary_dim]`` RoPE table, cos half then sin half (neox layout)."""
    inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
    ang = torch.arange(max_pos, dtype=torch.float)[:, None] * inv[None, :]
    return torch.cat((ang.cos(), ang.sin()), dim=-1)


def rotate_rows(x: torch.Tensor, pos: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """neox rotation of ``x [N, H, D]`` at non-negative positions (fp32 math, cast back)."""
    half = table.shape[1] // 2
    c = table[pos, :half].unsqueeze(1)
    s = table[pos, half:].unsqueeze(1)
    a, b = x[..., :half].float(), x[..., half: 2 * half].float()
    rot = torch.cat((c * a - s * b, c * b + s * a), dim=-1).to(x.dtype)
    return rot if 2 * half == x.shape[-1] else torch.cat((rot, x[..., 2 * half:]), dim=-1)


@dataclass
class ViewCase:
    """A pool, its blocks and one decode step's inputs."""

    page_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    rope_base: float
    max_pos: int
    num_pages: int
    k_pool: torch.Tensor          # [num_pages, P, Hkv, D] bf16 (rotated keys)
    v_pool: torch.Tensor
    cos_sin: torch.Tensor         # [max_pos, D] fp32
    blocks: Dict[str, CacheBlock]
    views: List[List[str]]
    writes: List[str]
    q: torch.Tensor               # [W, Hq*D] bf16, unrotated
    k_new: torch.Tensor           # [W, Hkv*D] bf16, unrotated
    v_new: torch.Tensor
    free_pages: List[int] = field(default_factory=list)   # page-start slots still unused

    @property
    def group(self) -> WorkerGroup:
        return WorkerGroup(
            cache_structure=[[self.blocks[n] for n in view] for view in self.views],
            write_to=[self.blocks[n] for n in self.writes],
        )

    def plan_writes(self):
        """Destination slot / pending page / write position of each worker's new token, the
        arithmetic of SharedCacheSession._plan_decode_writes (session.py:1102-1141)."""
        pending: Dict[int, Optional[int]] = {}
        fresh = list(self.free_pages)
        slots, positions = [], []
        targets = [self.blocks[n] for n in self.writes]
        need = [b for b in targets if not b.has_capacity]
        grant = {id(b): fresh[i] for i, b in enumerate(need)}
        for b in targets:
            pending[id(b)] = grant.get(id(b))
        for b in targets:
            start = pending[id(b)] if pending[id(b)] is not None else b.page_starts[-1]
            slots.append(start + b.num_tokens % self.page_size)
            positions.append(b.mrope_span)
        return pending, torch.tensor(slots, dtype=torch.int32), torch.tensor(positions, dtype=torch.int32)

    def kv_bytes_compulsory(self) -> int:
        """Distinct KV bytes one decode step must read (every block counted once, post-append)."""
        written = {id(self.blocks[n]) for n in self.writes}
        seen, toks = set(), 0
        for view in self.views:
            for n in view:
                b = self.blocks[n]
                if id(b) not in seen:
                    seen.add(id(b))
                    toks += b.num_tokens + (id(b) in written)
        for n in self.writes:
            if id(self.blocks[n]) not in seen:
                seen.add(id(self.blocks[n]))
                toks += 1
        return toks * 2 * self.num_kv_heads * self.head_dim * 2

    def kv_bytes_logical(self) -> int:
        """KV bytes summed per request view (what a per-request kernel streams)."""
        written = {id(self.blocks[n]) for n in self.writes}
        toks = 0
        for view, wname in zip(self.views, self.writes):
            toks += sum(self.blocks[n].num_tokens + (id(self.blocks[n]) in written) for n in view)
            if wname not in view:
                toks += 1
        return toks * 2 * self.num_kv_heads * self.head_dim * 2


def make_view_case(
    *, lengths: Dict[str, int], views: Sequence[Sequence[str]], writes: Sequence[str],
    num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, rope_base: float,
    seed: int, max_pos: Optional[int] = None, spare_pages: int = 0, kv_std: float = 0.5,
) -> ViewCase:
    g = torch.Generator().manual_seed(seed)
    P = page_size
    W = len(views)
    need_pages = sum(-(-L // P) for L in lengths.values()) + W + spare_pages
    num_pages = need_pages + 1  # + dummy page, as the engine allocates (engine.py:70-76)
    perm = torch.randperm(need_pages, generator=g).tolist()
    max_pos = max_pos or (max(lengths.values()) + sum(lengths.values()) + 64)
    table = cos_sin_table(head_dim, max_pos, rope_base)
    k_pool = torch.zeros(num_pages, P, num_kv_heads, head_dim, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    kf, vf = k_pool.view(-1, num_kv_heads, head_dim), v_pool.view(-1, num_kv_heads, head_dim)
    blocks: Dict[str, CacheBlock] = {}
    cursor = 0
    for name, L in lengths.items():
        b = CacheBlock(torch.device("cpu"), P)
        n_pages = -(-L // P)
        b.page_starts = [p * P for p in perm[cursor: cursor + n_pages]]
        cursor += n_pages
        b.num_tokens = L
        blocks[name] = b
        if L:
            slots = b.token_slots_tensor().long()
            k = (torch.randn(L, num_kv_heads, head_dim, generator=g) * kv_std).to(torch.bfloat16)
            v = (torch.randn(L, num_kv_heads, head_dim, generator=g) * kv_std).to(torch.bfloat16)
            kf[slots] = rotate_rows(k, torch.arange(L), table)
            vf[slots] = v
    free_pages = [p * P for p in perm[cursor:]]
    q = torch.randn(W, num_q_heads * head_dim, generator=g).to(torch.bfloat16)
    k_new = (torch.randn(W, num_kv_heads * head_dim, generator=g) * kv_std).to(torch.bfloat16)
    v_new = (torch.randn(W, num_kv_heads * head_dim, generator=g) * kv_std).to(torch.bfloat16)
    return ViewCase(
        page_size=P, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
        rope_base=rope_base, max_pos=max_pos, num_pages=num_pages, k_pool=k_pool, v_pool=v_pool,
        cos_sin=table, blocks=blocks, views=[list(v) for v in views], writes=list(writes), q=q,
        k_new=k_new, v_new=v_new, free_pages=free_pages,
    )


def config1_decode(page_size: int = 16, seed: int = 1000) -> ViewCase:
    """Decode parity case: 4 requests, Hq16/Hkv4/D128, private blocks of 512/1024/256 tokens,
    request r reads its three blocks rotated by r mod 3 and writes the last one; theta 1e6."""
    lengths, views, writes = {}, [], []
    for r in range(4):
        names = [f"r{r}b{j}" for j in range(3)]
        for n, L in zip(names, (512, 1024, 256)):
            lengths[n] = L
        rot = names[r % 3:] + names[: r % 3]
        views.append(rot)
        writes.append(rot[-1])
    return make_view_case(lengths=lengths, views=views, writes=writes, num_q_heads=16,
                          num_kv_heads=4, head_dim=128, page_size=page_size, rope_base=1e6, seed=seed)


def config2_decode(page_size: int = 16, seed: int = 2000, requests: int = 64,
                   shared_len: int = 8192, private_len: int = 2048, num_q_heads: int = 16,
                   num_kv_heads: int = 2, head_dim: int = 256, spare_pages: int = 0) -> ViewCase:
    """Shared-prefix decode: every request sees ``[shared, private_i]`` and writes ``private_i``;
    Hq16/Hkv2/D256, theta 1e7."""
    lengths = {"shared": shared_len}
    views, writes = [], []
    for r in range(requests):
        lengths[f"p{r}"] = private_len
        views.append(["shared", f"p{r}"])
        writes.append(f"p{r}")
    return make_view_case(lengths=lengths, views=views, writes=writes, num_q_heads=num_q_heads,
                          num_kv_heads=num_kv_heads, head_dim=head_dim, page_size=page_size,
                          rope_base=1e7, seed=seed, spare_pages=spare_pages)


# --------------------------------------------------------------------------- device driver
class DeviceView:
    """A ``ViewCase`` resident on one GPU behind the public pool / attention classes."""

    def __init__(self, case: ViewCase, device: torch.device, num_layers: int = 1, dense_engine=None):
        from types import SimpleNamespace

        from async_llm_b200.kvpool import MHAKVCache
        from async_llm_b200.view_attention import SharedCacheAttention

        self.case = case
        self.device = torch.device(device)
        self.pool = MHAKVCache(case.num_kv_heads, num_layers, case.head_dim, case.num_pages,
                               case.page_size, torch.bfloat16, self.device)
        for layer in range(num_layers):
            self.pool.k_cache(layer).copy_(case.k_pool)
            self.pool.v_cache(layer).copy_(case.v_pool)
        self.attn = SharedCacheAttention(
            self.pool, case.cos_sin.to(self.device), case.num_q_heads, case.num_kv_heads,
            case.head_dim, case.page_size, torch.bfloat16, self.device, dense_engine=dense_engine,
        )
        self.q = case.q.to(self.device)
        self.k_new = case.k_new.to(self.device)
        self.v_new = case.v_new.to(self.device)
        self._ns = SimpleNamespace

    def plan(self):
        """Host planning of one decode step; returns the batch object ``forward`` consumes."""
        pending, slots, positions = self.case.plan_writes()
        meta = self.attn.prepare(self.case.group, pending, slots)
        return self._ns(attn_metadata=meta, positions=positions.to(self.device),
                        out_loc=slots.to(self.device), mrope_positions=None)

    def decode(self, batch=None, layer_id: int = 0) -> torch.Tensor:
        batch = self.plan() if batch is None else batch
        return self.attn.forward(self.q, self.k_new, self.v_new, layer_id, batch)


# --------------------------------------------------------------------------- prefill workloads
@dataclass
class PrefillCase:
    """A pool with context blocks and one batched view-conditioned prefill's inputs."""

    page_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    num_pages: int
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    cos_sin: torch.Tensor
    blocks: Dict[str, CacheBlock]
    requests: List[dict]          # {"context": [names], "write": name, "num_new": S}
    q: torch.Tensor               # [N, Hq*D] unrotated
    k_new: torch.Tensor           # [N, Hkv*D] unrotated
    v_new: torch.Tensor
    positions: torch.Tensor       # [N] int32 block-relative write positions
    out_loc: torch.Tensor         # [N] int32 physical slots
    self_pages: List[torch.Tensor]  # per request: complete post-write page-start list of its block

    def specs(self):
        from async_llm_b200.view_attention import PrefillSpec

        out = []
        for req, pages in zip(self.requests, self.self_pages):
            wb = self.blocks[req["write"]]
            out.append(PrefillSpec([self.blocks[n] for n in req["context"]], pages, req["num_new"],
                                   wb.num_tokens, None))
        return out

    def flops(self) -> float:
        total = 0.0
        for req in self.requests:
            S = req["num_new"]
            ctx = sum(self.blocks[n].num_tokens for n in req["context"])
            T = self.blocks[req["write"]].num_tokens
            total += 4.0 * self.num_q_heads * self.head_dim * S * (ctx + T + (S + 1) / 2)
        return total


def make_prefill_case(*, lengths: Dict[str, int], requests: Sequence[dict], num_q_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, rope_base: float, seed: int,
                      kv_std: float = 0.5) -> PrefillCase:
    """``lengths`` gives every block's current token count (write blocks may be non-empty: the
    prefill extends them); each request appends ``num_new`` tokens to its ``write`` block."""
    g = torch.Generator().manual_seed(seed)
    P = page_size
    extra = {r["write"]: r["num_new"] for r in requests}
    need_pages = sum(-(-(L + extra.get(n, 0)) // P) for n, L in lengths.items()) + 4
    num_pages = need_pages + 1
    perm = torch.randperm(need_pages, generator=g).tolist()
    max_pos = sum(lengths.values()) + sum(extra.values()) + 64
    table = cos_sin_table(head_dim, max_pos, rope_base)
    k_pool = torch.zeros(num_pages, P, num_kv_heads, head_dim, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    kf, vf = k_pool.view(-1, num_kv_heads, head_dim), v_pool.view(-1, num_kv_heads, head_dim)
    blocks: Dict[str, CacheBlock] = {}
    cursor = 0
    for name, L in lengths.items():
        b = CacheBlock(torch.device("cpu"), P)
        n_pages = -(-L // P)
        b.page_starts = [p * P for p in perm[cursor: cursor + n_pages]]
        cursor += n_pages
        b.num_tokens = L
        blocks[name] = b
        if L:
            slots = b.token_slots_tensor().long()
            k = (torch.randn(L, num_kv_heads, head_dim, generator=g) * kv_std).to(torch.bfloat16)
            v = (torch.randn(L, num_kv_heads, head_dim, generator=g) * kv_std).to(torch.bfloat16)
            kf[slots] = rotate_rows(k, torch.arange(L), table)
            vf[slots] = v
    positions, out_loc, self_pages = [], [], []
    for req in requests:
        wb, S = blocks[req["write"]], req["num_new"]
        fresh = wb.pages_needed(S)
        new_starts = [p * P for p in perm[cursor: cursor + fresh]]
        cursor += fresh
        all_starts = list(wb.page_starts) + new_starts
        self_pages.append(torch.tensor(all_starts, dtype=torch.int32))
        T = wb.num_tokens
        for i in range(T, T + S):
            out_loc.append(all_starts[i // P] + i % P)
            positions.append(i)
    N = len(out_loc)
    q = torch.randn(N, num_q_heads * head_dim, generator=g).to(torch.bfloat16)
    k_new = (torch.randn(N, num_kv_heads * head_dim, generator=g) * kv_std).to(torch.bfloat16)
    v_new = (torch.randn(N, num_kv_heads * head_dim, generator=g) * kv_std).to(torch.bfloat16)
    return PrefillCase(page_size=P, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                       head_dim=head_dim, num_pages=num_pages, k_pool=k_pool, v_pool=v_pool,
                       cos_sin=table, blocks=blocks, requests=[dict(r) for r in requests], q=q,
                       k_new=k_new, v_new=v_new, positions=torch.tensor(positions, dtype=torch.int32),
                       out_loc=torch.tensor(out_loc, dtype=torch.int32), self_pages=self_pages)


def config3_prefill(page_size: int = 16, seed: int = 3000, requests: int = 16, chunk: int = 512,
                    pool_blocks: int = 24, min_len: int = 1024, max_len: int = 8192,
                    max_context: int = 32768, num_q_heads: int = 32, num_kv_heads: int = 8,
                    head_dim: int = 128) -> PrefillCase:
    """View-conditioned prefill: every request appends ``chunk`` tokens to its own empty block and
    attends to 2-6 blocks drawn from a shared pool (lengths U[min_len, max_len], total context
    capped at ``max_context``); Hq32/Hkv8/D128, theta 1e6."""
    g = torch.Generator().manual_seed(seed)
    lengths = {f"c{i}": int(torch.randint(min_len, max_len + 1, (1,), generator=g)) for i in range(pool_blocks)}
    reqs = []
    for r in range(requests):
        n = int(torch.randint(2, 7, (1,), generator=g))
        names = [f"c{int(i)}" for i in torch.randperm(pool_blocks, generator=g)[:n]]
        while sum(lengths[x] for x in names) > max_context - chunk and len(names) > 1:
            names.pop()
        lengths[f"w{r}"] = 0
        reqs.append({"context": names, "write": f"w{r}", "num_new": chunk})
    return make_prefill_case(lengths=lengths, requests=reqs, num_q_heads=num_q_heads,
                             num_kv_heads=num_kv_heads, head_dim=head_dim, page_size=page_size,
                             rope_base=1e6, seed=seed + 1)


class DevicePrefill:
    """A ``PrefillCase`` resident on one GPU behind the public pool / attention classes."""

    def __init__(self, case: PrefillCase, device: torch.device, dense_engine=None):
        from types import SimpleNamespace

        from async_llm_b200.kvpool import MHAKVCache
        from async_llm_b200.view_attention import SharedCacheAttention

        self.case = case
        self.device = torch.device(device)
        self.pool = MHAKVCache(case.num_kv_heads, 1, case.head_dim, case.num_pages, case.page_size,
                               torch.bfloat16, self.device)
        self.pool.k_cache(0).copy_(case.k_pool)
        self.pool.v_cache(0).copy_(case.v_pool)
        self.attn = SharedCacheAttention(self.pool, case.cos_sin.to(self.device), case.num_q_heads,
                                         case.num_kv_heads, case.head_dim, case.page_size,
                                         torch.bfloat16, self.device, dense_engine=dense_engine)
        self.q, self.k_new, self.v_new = (t.to(self.device) for t in (case.q, case.k_new, case.v_new))
        self._ns = SimpleNamespace

    def plan(self):
        meta = self.attn.prepare_prefill_batch(self.case.specs())
        return self._ns(attn_metadata=meta, positions=self.case.positions.to(self.device),
                        out_loc=self.case.out_loc.to(self.device), mrope_positions=None)

    def forward(self, batch=None) -> torch.Tensor:
        batch = self.plan() if batch is None else batch
        return self.attn.forward(self.q, self.k_new, self.v_new, 0, batch)


# --------------------------------------------------------------------------- GDN workloads
def gdn_tokens(n: int, num_k_heads: int, num_v_heads: int, dk: int, dv: int, seed: int):
    """Seeded GDN layer inputs for ``n`` tokens: q, k ~ N(0,1) L2-normalised, v ~ N(0,1) (bf16),
    g = logsigmoid(N(0,1)), beta = sigmoid(N(0,1)) (fp32)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(n, num_k_heads, dk, generator=g), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(n, num_k_heads, dk, generator=g), dim=-1).to(torch.bfloat16)
    v = torch.randn(n, num_v_heads, dv, generator=g).to(torch.bfloat16)
    gate = torch.nn.functional.logsigmoid(torch.randn(n, num_v_heads, generator=g))
    beta = torch.sigmoid(torch.randn(n, num_v_heads, generator=g))
    return q, k, v, gate, beta


def gdn_random_summary(num_v_heads: int, dk: int, dv: int, seed: int, device):
    """A plausible block summary without running a scan: a contraction-like A_hat and a small B_hat."""
    g = torch.Generator().manual_seed(seed)
    A = (0.9 * torch.eye(dk) + 0.01 * torch.randn(dk, dk, generator=g)).expand(1, num_v_heads, dk, dk).clone()
    Bm = 0.05 * torch.randn(1, num_v_heads, dv, dk, generator=g)
    return A.to(device), Bm.to(device)
