"""Safetensors checkpoint reading (Weights::load, model.rs:239-315): prefix search, single file
and index + shards, dtype / size / presence checks, and a round trip through the device arena.
The files are written here with numpy in the published layout (8-byte little-endian header
length, JSON header, data)."""
import ctypes as C
import json
import os
import struct

import numpy as np
import pytest

from helpers import random_weights, tiny_config
from system1_omni_b200 import lib as L


def write_safetensors(path, tensors, dtypes=None):
    """tensors: name -> uint16 (bf16 bits) or float32 array."""
    header, blobs, at = {"__metadata__": {"format": "pt"}}, [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        dtype = (dtypes or {}).get(name, "BF16" if a.dtype == np.uint16 else "F32")
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [at, at + a.nbytes]}
        blobs.append(a.tobytes())
        at += a.nbytes
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def hf_config(cfg):
    return {"text_config": {
        "head_dim": cfg.head_dim, "layer_types": cfg.layer_types, "num_hidden_layers": len(cfg.layer_types),
        "hidden_act": "silu", "attn_output_gate": True, "attention_bias": False, "linear_conv_kernel_dim": 4,
        "rope_parameters": {"rope_type": "default", "rope_theta": cfg.rope_theta,
                            "partial_rotary_factor": 2 * cfg.rotary_half / cfg.head_dim},
        "hidden_size": cfg.hidden, "intermediate_size": cfg.intermediate, "num_attention_heads": cfg.heads,
        "num_key_value_heads": cfg.kv_heads, "linear_num_key_heads": cfg.lin_k_heads,
        "linear_num_value_heads": cfg.lin_v_heads, "vocab_size": cfg.vocab, "rms_norm_eps": cfg.eps,
        "max_position_embeddings": cfg.max_positions, "linear_key_head_dim": 128, "linear_value_head_dim": 128}}


def inspect(directory, index=-1):
    lib = L.load()
    prefix, name, dtype = C.create_string_buffer(64), C.create_string_buffer(256), C.create_string_buffer(16)
    n, rank, nbytes = C.c_int(), C.c_int(), C.c_uint64()
    shape = (C.c_uint64 * 8)()
    code = lib.s1_checkpoint_inspect(os.fsencode(directory), prefix, 64, C.byref(n), index, name, 256, dtype, 16,
                                     C.byref(rank), shape, C.byref(nbytes))
    return code, prefix.value.decode(), n.value, name.value.decode(), dtype.value.decode(), list(shape)[:rank.value], nbytes.value


def test_prefix_search_and_listing(tmp_path, cs1):
    rng = np.random.default_rng(0)
    t = {"model.language_model.embed_tokens.weight": rng.integers(0, 65535, (6, 8)).astype(np.uint16),
         "model.language_model.layers.0.mlp.down_proj.weight": rng.integers(0, 65535, (8, 16)).astype(np.uint16),
         "model.visual.patch_embed.weight": rng.standard_normal((4, 4)).astype(np.float32),
         "lm_head.weight": rng.integers(0, 65535, (6, 8)).astype(np.uint16)}
    write_safetensors(tmp_path / "model.safetensors", t)
    code, prefix, n, *_ = inspect(tmp_path)
    assert (code, prefix, n) == (0, "model.language_model.", 2)
    seen = {}
    for i in range(n):
        code, _, _, name, dtype, shape, nbytes = inspect(tmp_path, i)
        assert code == 0
        seen[name] = (dtype, shape, nbytes)
    assert seen == {"embed_tokens.weight": ("BF16", [6, 8], 96), "layers.0.mlp.down_proj.weight": ("BF16", [8, 16], 256)}
    assert inspect(tmp_path, 2)[0] == 3000


def test_index_with_shards_and_bare_names(tmp_path, cs1):
    a = {"embed_tokens.weight": np.zeros((4, 8), np.uint16)}
    b = {"norm.weight": np.ones(8, np.uint16), "layers.0.input_layernorm.weight": np.ones(8, np.uint16)}
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", a)
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", b)
    index = {"metadata": {"total_size": 1}, "weight_map": {
        "embed_tokens.weight": "model-00001-of-00002.safetensors", "norm.weight": "model-00002-of-00002.safetensors",
        "layers.0.input_layernorm.weight": "model-00002-of-00002.safetensors"}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    code, prefix, n, *_ = inspect(tmp_path)
    assert (code, prefix, n) == (0, "", 3)


def test_malformed_checkpoints_are_refused(tmp_path, cs1):
    assert inspect(tmp_path)[0] == 3004                                   # no file at all
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00")
    assert inspect(tmp_path)[0] == 3005                                   # shorter than its length field
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    assert inspect(tmp_path)[0] == 3005                                   # header longer than the file
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", 9) + b'{"a": [1}')
    assert inspect(tmp_path)[0] == 3005                                   # not JSON
    text = json.dumps({"model.embed_tokens.weight": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 64]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    assert inspect(tmp_path)[0] == 3005                                   # data range past the end
    write_safetensors(tmp_path / "model.safetensors", {"model.norm.weight": np.ones(8, np.uint16)})
    assert inspect(tmp_path)[0] == 3007                                   # no embed_tokens.weight under any prefix


def test_malformed_headers_are_refused(tmp_path, cs1):
    def header(obj_text, data=b""):
        raw = obj_text if isinstance(obj_text, bytes) else obj_text.encode()
        (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(raw)) + raw + data)
        return inspect(tmp_path)[0]

    good = {"model.embed_tokens.weight": {"dtype": "BF16", "shape": [4, 8], "data_offsets": [0, 64]}}
    assert header(json.dumps(good), b"\0" * 64) == 0
    # a header that ends inside a literal, or inside a string
    assert header('{"a": t') == 3005
    assert header('{"a": nul') == 3005
    assert header('{"a": "xy') == 3005
    assert header('{"a": "\\u00') == 3005
    # begin past end, a fractional offset, a negative extent
    bad = json.loads(json.dumps(good))
    bad["model.embed_tokens.weight"]["data_offsets"] = [64, 0]
    assert header(json.dumps(bad), b"\0" * 64) == 3005
    assert header(json.dumps(good).replace("[0, 64]", "[0, 64.5]"), b"\0" * 64) == 3005
    assert header(json.dumps(good).replace("[4, 8]", "[-4, 8]"), b"\0" * 64) == 3005
    # two tensors that share bytes
    two = dict(good)
    two["model.norm.weight"] = {"dtype": "BF16", "shape": [8], "data_offsets": [56, 72]}
    assert header(json.dumps(two), b"\0" * 72) == 3005
    two["model.norm.weight"]["data_offsets"] = [64, 80]
    assert header(json.dumps(two), b"\0" * 80) == 0
    # an escaped name is decoded: "model.embed_tokens.w\u0065ight"
    esc = json.dumps(good).replace("weight", "w\\u0065ight")
    assert "\\u0065" in esc
    assert header(esc, b"\0" * 64) == 0


def export_manifest(hidden, **over):
    m = {"format": "open-jev-text-merged/1", "model_id": "open-jev-9b", "base_revision": "r1", "checkpoint_revision": "r2",
         "temperature": 1.7, "max_length": 4096, "chat_prefix": "<|im_start|>user\n", "chat_suffix": "<|im_end|>\n",
         "head_weight": [0.25 * i - 1.0 for i in range(hidden)], "head_bias": -0.125}
    m.update(over)
    return m


def read_export(directory, hidden):
    lib = L.load()
    w = np.zeros(hidden, np.float32)
    bias, temp, length, mid = C.c_float(), C.c_double(), C.c_int(), C.create_string_buffer(64)
    code = lib.s1_export_read(os.fsencode(directory), hidden, w.ctypes.data_as(C.c_void_p), C.byref(bias), C.byref(temp),
                              C.byref(length), mid, 64)
    return code, w, bias.value, temp.value, length.value, mid.value.decode()


def test_export_manifest(tmp_path, cs1):
    """open_jev_export.json as Engine::load and DecisionHead::load read it (engine.rs:21-46,
    executor.rs:21-54): head, bias, temperature, length cap; the reference's refusals."""
    from system1_omni_b200 import model as M
    hidden = 12
    assert read_export(tmp_path, hidden)[0] == 3004                      # no manifest: not an export
    path = tmp_path / "open_jev_export.json"
    path.write_text(json.dumps(export_manifest(hidden)) + "\n")
    code, w, bias, temp, length, mid = read_export(tmp_path, hidden)
    assert (code, bias, temp, length, mid) == (0, -0.125, 1.7, 4096, "open-jev-9b")
    assert np.array_equal(w, np.array([0.25 * i - 1.0 for i in range(hidden)], np.float32))
    # the head as the worker applies it: float64 accumulation, float32 result, bias added in float32
    last = np.linspace(-1, 1, hidden).astype(np.float32)
    score = M.DecisionHead(w, bias).score(last)
    assert score == np.float32(np.float32(np.dot(w.astype(np.float64), last.astype(np.float64))) + np.float32(bias))
    for over in ({"format": "something-else/1"}, {"temperature": 0.0}, {"temperature": "hot"}, {"max_length": 0},
                 {"max_length": 16385}, {"head_weight": [1.0] * (hidden - 1)}, {"head_weight": [1.0] * (hidden - 1) + ["x"]},
                 {"head_bias": None}, {"chat_prefix": 3}, {"head_weight": [1e39] + [0.0] * (hidden - 1)}):
        path.write_text(json.dumps(export_manifest(hidden, **over)))
        assert read_export(tmp_path, hidden)[0] in (3005, 3008), over
    path.write_text("{")
    assert read_export(tmp_path, hidden)[0] == 3005


@pytest.mark.gpu
def test_model_from_checkpoint_matches_set_tensors(tmp_path, cs1):
    from system1_omni_b200 import model as M
    cfg = tiny_config()
    weights = random_weights(cfg, seed=4)
    names = sorted(weights)
    half = len(names) // 2
    shards = [{"model." + n: weights[n] for n in names[:half]}, {"model." + n: weights[n] for n in names[half:]}]
    shards[1]["lm_head.weight"] = np.zeros((cfg.vocab, cfg.hidden), np.float32)      # outside the prefix: ignored
    shards[1]["model.mtp.fc.weight"] = np.zeros((8, 8), np.uint16)                   # inside, no place for it: skipped
    wmap = {}
    for i, shard in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-00002.safetensors"
        write_safetensors(tmp_path / fname, shard)
        wmap.update({n: fname for n in shard})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wmap}))
    (tmp_path / "config.json").write_text(json.dumps(hf_config(cfg)))

    loaded = M.Model.from_checkpoint(str(tmp_path))
    direct = M.Model(cfg)
    direct.set_tensors(weights)
    try:
        assert loaded.cfg == cfg
        ids = np.random.default_rng(0).integers(0, cfg.vocab, 90).tolist()
        assert np.array_equal(loaded.forward(ids), direct.forward(ids))
        assert np.array_equal(loaded.get_tensor("layers.1.linear_attn.A_log"), weights["layers.1.linear_attn.A_log"])
    finally:
        loaded.close()
        direct.close()

    # a float16 tensor of the decoder, a missing one and a mis-sized one are refused, by name
    def attempt(mutate):
        bad = {n: dict(s) for n, s in zip(("a", "b"), shards)}
        dtypes = mutate(bad) or {}
        for key, fname in (("a", "model-00001-of-00002.safetensors"), ("b", "model-00002-of-00002.safetensors")):
            write_safetensors(tmp_path / fname, bad[key], dtypes)
        with pytest.raises(L.CudaError) as err:
            M.Model.from_checkpoint(str(tmp_path))
        return str(err.value)

    victim = "model." + names[0]
    assert "3006" in attempt(lambda b: {victim: "F16"})
    msg = attempt(lambda b: (b["a"].pop(victim), None)[1])
    assert "3007" in msg and names[0] in msg
    msg = attempt(lambda b: b["a"].update({victim: np.zeros(3, np.uint16)}))
    assert "3003" in msg and names[0] in msg
    # a matrix of the right byte count but transposed is refused too (the reference compares shapes)
    matrix = "model.layers.0.mlp.down_proj.weight"
    key = "a" if matrix in shards[0] else "b"
    msg = attempt(lambda b: b[key].update({matrix: np.ascontiguousarray(b[key][matrix].T)}))
    assert "3003" in msg and "down_proj" in msg
    # a tensor under the prefix that the decoder does not use must still be bfloat16
    assert "3006" in attempt(lambda b: b["b"].update({"model.mtp.fc.weight": np.zeros((8, 8), np.float32)}))
