"""Host side of the attention-backend plugin: planning of ordinary batches, registration."""
import numpy as np
import pytest
import torch

from async_llm_b200 import B200AttnBackend, MHAKVCache
from async_llm_b200.attention_backend import register
from async_llm_b200.attention_base import BaseAttnBackend
from attention_backend_cases import make_batch, make_plain_case


def cpu_backend(case):
    pool = MHAKVCache(case.hkv, 1, case.d, case.k_pool.shape[0], case.page_size, torch.bfloat16, torch.device("cpu"))
    be = B200AttnBackend(case.config, pool, case.table)
    be.op._lanes, be.op._lane_width = 64, 4
    return be


def test_backend_implements_the_plugin_interface():
    assert issubclass(B200AttnBackend, BaseAttnBackend)
    for name in ("forward", "prepare_metadata", "init_capture_graph", "prepare_for_capture", "prepare_for_replay"):
        assert callable(getattr(B200AttnBackend, name))


def test_decode_batch_becomes_one_streamed_segment_per_request():
    case = make_plain_case([(100, 1), (37, 1), (1, 1)])
    be = cpu_backend(case)
    batch = make_batch(case, "decode", torch.device("cpu"))
    be.prepare_metadata(batch)
    inner = batch.attn_metadata.inner
    assert inner.phase == "decode" and inner.n_main == 3 and inner.n_aux == 0 and inner.max_segments == 1
    # every request's segment is its slot row, post-append (page size 1: slots are the page numbers)
    t = inner.tables
    want = np.concatenate([case.table[r.table_idx, : r.device_len].numpy() for r in case.reqs])
    assert t.main_seq_lens == [101, 38, 2]
    assert np.array_equal(np.asarray(t.main_indices), want)
    assert torch.equal(batch.attn_metadata.get_last_indices(3), torch.arange(3))


def test_prefill_batch_becomes_context_free_prefill_specs():
    case = make_plain_case([(0, 45), (37, 33), (0, 70)])
    be = cpu_backend(case)
    batch = make_batch(case, "prefill", torch.device("cpu"))
    be.prepare_metadata(batch)
    inner = batch.attn_metadata.inner
    assert inner.phase == "prefill_batch" and inner.n_ctx_rows == 0
    seg = inner.plan.host["segments"]
    # one causal, end-aligned segment per request over prefix + new tokens
    assert seg[:, 2].tolist() == [45, 70, 70] and seg[:, 4].tolist() == [0, 37, 0]
    assert batch.attn_metadata.get_last_indices(3).tolist() == [44, 77, 147]


def test_registration_in_the_host_registry():
    try:
        import sys, os
        here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        for path in (os.environ.get("ASYNC_LLM_REFERENCE_PYTHON"),
                     os.path.join(os.path.dirname(here), "reference", "python")):   # a checkout beside this repository
            if path and os.path.isdir(os.path.join(path, "minisgl")) and path not in sys.path:
                sys.path.insert(0, path)
        from minisgl.attention import SUPPORTED_ATTENTION_BACKENDS, validate_attn_backend
    except Exception as exc:   # noqa: BLE001
        pytest.skip(f"host framework not importable here: {exc}")
    assert register("b200") and register("b200")        # idempotent
    assert validate_attn_backend("b200", allow_auto=False) == "b200"
    assert "b200" in SUPPORTED_ATTENTION_BACKENDS.supported_names()
    assert callable(SUPPORTED_ATTENTION_BACKENDS["b200"])
