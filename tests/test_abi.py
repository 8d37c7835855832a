"""The drop-in boundary without a GPU: the library loads, exports every symbol the headers
declare (the reference's loader refuses a library missing any of them, cuda.rs:24-47),
reports ABI version 6, and its host-only entry points behave like the reference's."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from system1_omni_b200 import lib as L
from system1_omni_b200 import model as M

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:cs1|s1)_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(cs1):
    names = declared("cs1_ops.h") + declared("s1_executor.h") + declared("s1_dispatch.h")
    # the 45 entry points of the reference's ops.h plus the ones only this library has
    assert len(declared("cs1_ops.h")) == 45 + len(L.NOT_IN_REFERENCE)
    for name in names:
        assert hasattr(cs1, name), name
        assert name in L.SIGNATURES, f"{name} has no Python binding"
    assert sorted(L.SIGNATURES) == sorted(names)


def test_reference_symbol_list_matches():
    """The names the reference's loader binds (its api! block), kept as text."""
    want = """cs1_abi_version cs1_error_string cs1_set_device cs1_malloc cs1_free cs1_stream_create cs1_stream_sync
    cs1_stream_destroy cs1_graph_begin cs1_graph_end cs1_graph_launch cs1_graph_destroy cs1_upload cs1_download
    cs1_copy_dd cs1_copy2d cs1_embed cs1_rms_norm cs1_add_rms_norm cs1_gated_rms_norm cs1_gdn_conv cs1_gdn_gates
    cs1_gdn_workspace_floats cs1_gdn_prefill cs1_gdn_prefill_x cs1_attn_prep cs1_attention cs1_attention_gated
    cs1_attention_gated_prefix cs1_sigmoid_gate cs1_silu_mul cs1_gemm_create cs1_gemm_destroy cs1_gemm
    cs1_vision_linear cs1_gemm_f32 cs1_vision_norm cs1_vision_position cs1_vision_rope cs1_vision_attention
    cs1_vision_bias cs1_vision_gelu cs1_vision_add cs1_vision_to_float cs1_vision_lora_add""".split()
    assert len(want) == 45
    assert sorted(want) == [n for n in declared("cs1_ops.h") if n not in L.NOT_IN_REFERENCE]


def test_abi_version_and_error_strings(cs1):
    assert cs1.cs1_abi_version() == 6
    for code in (0, 1, 2, 700, 1000, 1015, 2000, 2001, 2002, 123456):
        s = cs1.cs1_error_string(code)
        assert isinstance(s, bytes) and len(s) > 0


def test_workspace_size_is_monotone_and_covers_smaller_windows(cs1):
    for h in (3, 16, 48):
        prev = 0
        for t in (0, 1, 63, 64, 65, 1024, 2048, 16384):
            n = cs1.cs1_gdn_workspace_floats(t, h)
            assert n >= prev
            prev = n
    # one query at the scratch capacity serves every shorter window (model.rs:456)
    # and is smaller than the reference's 1.6 GiB at its largest prompt (no per-chunk state is stored)
    assert cs1.cs1_gdn_workspace_floats(16384, 48) * 4 < 1 << 30


def test_host_heads_match_the_reference_known_answers(cs1):
    # tests/open_jev/head.rs:5-18, tests/cua_s1/head.rs:4-23
    assert M.DecisionHead(np.array([16_777_216.0, 1.0, -16_777_216.0], np.float32), 0.25).score([1, 1, 1]) == 1.25
    assert M.DecisionHead(np.array([16_777_216.0, 1.0], np.float32), -16_777_216.0).score([1, 1]) == 0.0
    with pytest.raises(ValueError):
        M.DecisionHead(np.array([np.finfo(np.float32).max], np.float32)).score([2.0])
    with pytest.raises(ValueError):
        M.DecisionHead(np.array([np.finfo(np.float32).max], np.float32)).score([np.nan])
    letters = [16_777_216.0, 1.0, -16_777_216.0, 16_777_216.0, 1.0, 0.0, np.nan, np.nan, np.nan]
    assert list(M.letter_logits(letters, [1.0, 1.0, 1.0], 2)) == [1.0, 16_777_216.0]
    assert list(M.letter_logits(letters, [1.0, 1.0, 1.0], 1)) == [1.0]
    with pytest.raises(ValueError):
        M.letter_logits([np.nan], [1.0], 1)


def test_host_batching_and_decision(cs1):
    lengths = [2048, 2048, 1, 5000, 3] + [4] * 17
    got = M.ranges(lengths)
    assert got == [range(0, 2), range(2, 3), range(3, 4), range(4, 20), range(20, 22)]
    assert M.ranges([]) == []
    mode, probs = M.answer([1.0, 3.0, 3.0, 0.5])
    assert mode == 1 and abs(probs.sum() - 1) < 1e-12
    with pytest.raises(ValueError):
        M.answer([1.0, np.inf])
    with pytest.raises(ValueError):
        M.answer([1.0, 2.0], temperature=0.0)


def test_host_logic_agrees_with_the_oracle(cs1):
    import oracle as O
    rng = np.random.default_rng(3)
    for _ in range(20):
        lengths = rng.integers(1, 6000, rng.integers(1, 60)).astype(np.int32)
        assert [(r.start, r.stop) for r in M.ranges(lengths)] == O.batch_ranges(lengths)
        w = rng.normal(size=(5, 64)).astype(np.float32)
        h = rng.normal(size=64).astype(np.float32)
        assert np.array_equal(M.head_logits(w, h), O.letter_logits(w, h, 5))
        logits = rng.normal(size=7).astype(np.float32)
        logits[3] = logits[5] = logits.max() + 1      # a tie
        m1, p1 = M.answer(logits, 0.7)
        m2, p2 = O.decide(logits, 0.7)
        assert m1 == m2 == 3 and np.array_equal(p1, p2)


def test_token_balanced_assignment(cs1):
    rng = np.random.default_rng(0)
    lengths = np.exp(rng.uniform(np.log(512), np.log(16384), 64)).astype(np.int32)
    for ranks in (1, 2, 4, 8):
        where = M.assign_requests(lengths, ranks, a=1.0, b=1e-4)
        assert where.min() >= 0 and where.max() < ranks
        cost = lengths + 1e-4 * lengths.astype(np.float64) ** 2
        loads = np.array([cost[where == r].sum() for r in range(ranks)])
        assert loads.max() <= cost.sum() / ranks + cost.max()      # the greedy bound
        assert sorted(np.concatenate([np.flatnonzero(where == r) for r in range(ranks)])) == list(range(64))


def test_config_parsing_follows_the_reference_checks():
    hf = {"text_config": {
        "hidden_size": 2560, "intermediate_size": 9728, "num_hidden_layers": 4, "num_attention_heads": 16,
        "num_key_value_heads": 4, "head_dim": 256, "rms_norm_eps": 1e-6, "max_position_embeddings": 262144,
        "layer_types": ["linear_attention"] * 3 + ["full_attention"], "hidden_act": "silu", "vocab_size": 151936,
        "linear_num_key_heads": 16, "linear_num_value_heads": 32, "linear_key_head_dim": 128,
        "linear_value_head_dim": 128, "linear_conv_kernel_dim": 4,
        "rope_parameters": {"rope_theta": 1e7, "partial_rotary_factor": 0.25, "rope_type": "default"}}}
    cfg = M.Config.from_hf(hf)
    assert cfg.rotary_half == 32 and cfg.key_dim == 2048 and cfg.value_dim == 4096 and cfg.full_attention == [
        False, False, False, True]
    bad = {"text_config": dict(hf["text_config"], linear_conv_kernel_dim=3)}
    with pytest.raises(ValueError):
        M.Config.from_hf(bad)
    bad = {"text_config": dict(hf["text_config"], hidden_act="gelu")}
    with pytest.raises(ValueError):
        M.Config.from_hf(bad)
    bad = {"text_config": dict(hf["text_config"], layer_types=["sliding"] * 4)}
    with pytest.raises(ValueError):
        M.Config.from_hf(bad)
