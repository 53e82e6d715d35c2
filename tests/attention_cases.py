"""Seeded attention cases shared by the reference-output fixture and the parity tests.

``tests/golden/make_attention_golden.py`` runs the reference implementation on these cases (on a GPU,
its attention core is FlashInfer) and stores its output rows; the parity tests rebuild the same cases
from the same seeds and compare the CPU oracle and the CUDA kernels with the stored rows.
"""
import benchcases as wl

EDGE_LENGTHS = {"common": 17, "left": 16, "right": 0, "empty": 0, "solo": 1, "tail": 33, "out": 5}
EDGE_VIEWS = [["common", "empty", "right", "left"], ["common", "left", "common"], ["solo"],
              ["tail", "common"], ["common"]]
EDGE_WRITES = ["left", "right", "solo", "tail", "out"]

PREFILL_LENGTHS = {"a": 70, "b": 129, "c": 5, "w0": 0, "w1": 37, "w2": 0}
PREFILL_REQS = [{"context": ["a", "b"], "write": "w0", "num_new": 45},
                {"context": ["b", "c", "a"], "write": "w1", "num_new": 33},
                {"context": [], "write": "w2", "num_new": 70}]


def _edge(D, hq, hkv):
    return wl.make_view_case(lengths=EDGE_LENGTHS, views=EDGE_VIEWS, writes=EDGE_WRITES, num_q_heads=hq,
                             num_kv_heads=hkv, head_dim=D, page_size=16, rope_base=1e6, seed=7)


def _small_prefill(D, hq, hkv, page_size):
    return wl.make_prefill_case(lengths=PREFILL_LENGTHS, requests=PREFILL_REQS, num_q_heads=hq,
                                num_kv_heads=hkv, head_dim=D, page_size=page_size, rope_base=1e6, seed=5)


# name -> zero-argument builder of a ViewCase (one decode step)
DECODE_CASES = {
    "config1_p16": lambda: wl.config1_decode(page_size=16),
    "config1_p1": lambda: wl.config1_decode(page_size=1),
    "config1_p64": lambda: wl.config1_decode(page_size=64),
    "shared_prefix_small_p16": lambda: wl.config2_decode(page_size=16, requests=6, shared_len=700, private_len=333),
    "edge_d128_gqa4": lambda: _edge(128, 8, 2),
    "edge_d256_gqa8": lambda: _edge(256, 8, 1),
    "config2_full": lambda: wl.config2_decode(page_size=16),
}

# name -> zero-argument builder of a PrefillCase (one batched view-conditioned prefill)
PREFILL_CASES = {
    "small_d128_p16": lambda: _small_prefill(128, 8, 2, 16),
    "small_d256_p16": lambda: _small_prefill(256, 8, 1, 16),
    "small_d128_p1": lambda: _small_prefill(128, 8, 2, 1),
    "config3_reduced": lambda: wl.config3_prefill(requests=4, chunk=96, pool_blocks=6, min_len=100,
                                                  max_len=400, max_context=1400),
    "config3_4of16": lambda: wl.config3_prefill(requests=4),
}
