"""Host-side mirror of the reference's model executor interface over the C ABI.

`Config` follows Config::load (src/models/qwen3_5/native/src/model.rs:50-180), `Model` the
public methods of Model (model.rs:622, 763, 769), `DecisionHead` / `letter_logits` the
workers' CPU heads (open_jev executor.rs:56-68, cua_s1 executor.rs:61-78), `ranges`
batching::ranges (open_jev batching.rs:9-25) and `answer` contract::answer's decision
(contract.rs:227-247). All arithmetic happens in libqwen3_5_cuda.so; this file only marshals.
"""
import ctypes as C
import json
import os
from dataclasses import dataclass, field
from typing import List

import numpy as np

from . import lib as L


@dataclass
class Config:
    hidden: int
    intermediate: int
    layer_types: List[str]
    heads: int
    kv_heads: int
    head_dim: int
    rotary_half: int
    lin_k_heads: int
    lin_v_heads: int
    vocab: int
    eps: float = 1e-6
    rope_theta: float = 1e7
    max_positions: int = 262144
    lin_k_dim: int = 128
    lin_v_dim: int = 128

    @property
    def n_layers(self):
        return len(self.layer_types)

    @property
    def key_dim(self):
        return self.lin_k_heads * 128

    @property
    def value_dim(self):
        return self.lin_v_heads * 128

    @property
    def full_attention(self):
        return [t == "full_attention" for t in self.layer_types]

    def shape_dict(self):
        return dict(hidden=self.hidden, intermediate=self.intermediate, layer_types=list(self.layer_types),
                    heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim, rotary_half=self.rotary_half,
                    lin_k_heads=self.lin_k_heads, lin_v_heads=self.lin_v_heads, vocab=self.vocab, eps=self.eps,
                    rope_theta=self.rope_theta)

    @classmethod
    def from_hf(cls, root):
        """Parse a Hugging Face config.json dict with the checks of model.rs:50-180 that apply here."""
        c = root.get("text_config", root)
        rope = c.get("rope_parameters") or {}
        partial = rope.get("partial_rotary_factor", c.get("partial_rotary_factor", 1.0))
        head_dim = int(c["head_dim"])
        types = list(c["layer_types"])
        for t in types:
            if t not in ("full_attention", "linear_attention"):
                raise ValueError(f"unknown layer type {t!r}")
        if len(types) != int(c["num_hidden_layers"]):
            raise ValueError("layer_types does not match num_hidden_layers")
        if c.get("hidden_act") != "silu":
            raise ValueError("hidden_act is not silu")
        if not c.get("attn_output_gate", True):
            raise ValueError("attention without the output gate")
        if c.get("attention_bias") is True:
            raise ValueError("attention with bias")
        if rope.get("rope_type", "default") != "default":
            raise ValueError(f"rope type {rope.get('rope_type')}")
        if int(c["linear_conv_kernel_dim"]) != 4:
            raise ValueError("conv kernel is not 4")
        theta = rope.get("rope_theta", c.get("rope_theta"))
        if theta is None:
            raise ValueError("rope_theta")
        cfg = cls(hidden=int(c["hidden_size"]), intermediate=int(c["intermediate_size"]), layer_types=types,
                  heads=int(c["num_attention_heads"]), kv_heads=int(c["num_key_value_heads"]), head_dim=head_dim,
                  rotary_half=int(head_dim * partial) // 2, lin_k_heads=int(c["linear_num_key_heads"]),
                  lin_v_heads=int(c["linear_num_value_heads"]), vocab=int(c["vocab_size"]),
                  eps=float(c["rms_norm_eps"]), rope_theta=float(theta),
                  max_positions=int(c["max_position_embeddings"]), lin_k_dim=int(c["linear_key_head_dim"]),
                  lin_v_dim=int(c["linear_value_head_dim"]))
        if cfg.head_dim not in (128, 256) or cfg.lin_k_dim != 128 or cfg.lin_v_dim != 128:
            raise ValueError(f"head dims {cfg.head_dim} / {cfg.lin_k_dim} / {cfg.lin_v_dim}")
        if not (0 < cfg.max_positions <= 1 << 24):
            raise ValueError("unsupported max_position_embeddings")
        if cfg.kv_heads <= 0 or cfg.heads % cfg.kv_heads:
            raise ValueError("attention heads")
        if cfg.lin_k_heads <= 0 or cfg.lin_v_heads % cfg.lin_k_heads:
            raise ValueError("linear attention heads")
        if cfg.hidden % 8:
            raise ValueError("hidden size")
        return cfg

    @classmethod
    def load(cls, directory):
        with open(os.path.join(directory, "config.json")) as f:
            return cls.from_hf(json.load(f))


def tensor_shapes(cfg):
    """Checkpoint tensor names (without the model prefix) and shapes, as Model::load expects them."""
    h, I, kd, vd, hv = cfg.hidden, cfg.intermediate, cfg.key_dim, cfg.value_dim, cfg.lin_v_heads
    hq, hk, hd = cfg.heads, cfg.kv_heads, cfg.head_dim
    out = {"embed_tokens.weight": (cfg.vocab, h), "norm.weight": (h,)}
    for i, kind in enumerate(cfg.layer_types):
        p = f"layers.{i}."
        out[p + "input_layernorm.weight"] = (h,)
        out[p + "post_attention_layernorm.weight"] = (h,)
        out[p + "mlp.gate_proj.weight"] = (I, h)
        out[p + "mlp.up_proj.weight"] = (I, h)
        out[p + "mlp.down_proj.weight"] = (h, I)
        if kind == "full_attention":
            out[p + "self_attn.q_proj.weight"] = (hq * hd * 2, h)
            out[p + "self_attn.k_proj.weight"] = (hk * hd, h)
            out[p + "self_attn.v_proj.weight"] = (hk * hd, h)
            out[p + "self_attn.o_proj.weight"] = (h, hq * hd)
            out[p + "self_attn.q_norm.weight"] = (hd,)
            out[p + "self_attn.k_norm.weight"] = (hd,)
        else:
            out[p + "linear_attn.in_proj_qkv.weight"] = (2 * kd + vd, h)
            out[p + "linear_attn.in_proj_z.weight"] = (vd, h)
            out[p + "linear_attn.in_proj_b.weight"] = (hv, h)
            out[p + "linear_attn.in_proj_a.weight"] = (hv, h)
            out[p + "linear_attn.conv1d.weight"] = (2 * kd + vd, 1, 4)
            out[p + "linear_attn.A_log"] = (hv,)
            out[p + "linear_attn.dt_bias"] = (hv,)
            out[p + "linear_attn.norm.weight"] = (128,)
            out[p + "linear_attn.out_proj.weight"] = (h, vd)
    return out


class Prefix:
    """Device-side state of a captured prefix; owned by the model that captured it."""

    def __init__(self, handle, length):
        self.handle, self.length = handle, length

    @property
    def nbytes(self):
        return int(L.load().s1_prefix_bytes(self.handle)) if self.handle else 0

    def close(self):
        if self.handle:
            L.load().s1_prefix_destroy(self.handle)
            self.handle = None


class Model:
    """One decoder on one GPU: weights, scratch, stream, GEMM handle and graph cache."""

    def __init__(self, cfg: Config, device=0):
        self.cfg = cfg
        self.device = device
        self._flags = (C.c_ubyte * cfg.n_layers)(*[int(f) for f in cfg.full_attention])
        c = L.S1Config(cfg.hidden, cfg.intermediate, cfg.n_layers, cfg.heads, cfg.kv_heads, cfg.head_dim,
                       cfg.rotary_half, cfg.lin_k_heads, cfg.lin_v_heads, cfg.vocab, cfg.max_positions, cfg.eps,
                       cfg.rope_theta, self._flags)
        self.handle = C.c_void_p()
        L.check(L.load().s1_model_create(C.byref(c), device, C.byref(self.handle)), "model create")

    def close(self):
        if getattr(self, "handle", None) and self.handle.value:
            L.load().s1_model_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self):
        return C.c_void_p(L.load().s1_model_stream(self.handle))

    @property
    def weight_bytes(self):
        return L.load().s1_model_weight_bytes(self.handle)

    @classmethod
    def from_checkpoint(cls, directory, device=0):
        """Model::load (model.rs:622-705): config.json + safetensors files of a checkpoint directory."""
        model = cls(Config.load(directory), device=device)
        offender = C.create_string_buffer(256)
        code = L.load().s1_model_load_checkpoint(model.handle, os.fsencode(directory), offender, 256)
        if code != 0:
            model.close()
            raise L.CudaError(code, f"load checkpoint ({offender.value.decode() or directory})")
        return model

    def init_random(self, seed=0, std=0.02):
        L.check(L.load().s1_model_init_random(self.handle, seed, std), "init random")

    def set_tensors(self, tensors):
        """tensors: name -> uint16 (bf16 bits) numpy array."""
        for name, a in tensors.items():
            a = np.ascontiguousarray(a)
            assert a.dtype == np.uint16, name
            L.check(L.load().s1_model_set_tensor(self.handle, name.encode(), a.ctypes.data_as(C.c_void_p), a.nbytes),
                    f"set tensor {name}")

    def get_tensor(self, name):
        shape = tensor_shapes(self.cfg)[name]
        ptr, nbytes = C.c_void_p(), C.c_size_t()
        L.check(L.load().s1_model_tensor(self.handle, name.encode(), C.byref(ptr), C.byref(nbytes)), "tensor")
        out = np.empty(shape, np.uint16)
        assert out.nbytes == nbytes.value
        L.check(L.load().cs1_download(out.ctypes.data_as(C.c_void_p), ptr, out.nbytes, self.stream), "download")
        return out

    def enable_graphs(self, on=True):
        L.check(L.load().s1_model_enable_graphs(self.handle, int(on)), "graphs")

    def set_exact_packing(self, on=True):
        """Bit-identical results for a prompt alone or in a pack (slower); see s1_executor.h."""
        L.check(L.load().s1_model_set_exact_packing(self.handle, int(on)), "exact packing")

    def set_overlap_tokens(self, tokens):
        """Passes of at most `tokens` tokens launch every kernel as a programmatic dependent of the one
        before it, longer ones only the GEMMs; tokens < 0: plain stream order."""
        L.check(L.load().s1_model_set_overlap_tokens(self.handle, int(tokens)), "overlap tokens")

    def set_fused_mlp(self, on=True):
        """Gate/up projection + SiLU-multiply as one kernel (default) or as the two operators."""
        L.check(L.load().s1_model_set_fused_mlp(self.handle, int(on)), "fused mlp")

    def graph_stats(self):
        r, c, e = C.c_int(), C.c_int(), C.c_int()
        L.check(L.load().s1_model_graph_stats(self.handle, C.byref(r), C.byref(c), C.byref(e)), "graph stats")
        return {"replays": r.value, "captures": c.value, "enabled": bool(e.value)}

    def forward_batch(self, inputs, want_layers=False):
        """inputs: list of token id sequences. Returns float32 [n, hidden] (and bf16 [L, T, hidden])."""
        lengths = np.array([len(x) for x in inputs], np.int32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(x, np.int64) for x in inputs]) if len(inputs) else
                                   np.zeros(0, np.int64))
        if ids.size and (ids.min() < 0 or ids.max() >= 2 ** 31):
            raise ValueError("token id outside the vocabulary")
        ids = ids.astype(np.int32)
        last = np.zeros((len(inputs), self.cfg.hidden), np.float32)
        layers = np.zeros((self.cfg.n_layers, int(lengths.sum()), self.cfg.hidden), np.uint16) if want_layers else None
        code = L.load().s1_model_forward_batch(
            self.handle, ids.ctypes.data_as(C.c_void_p), lengths.ctypes.data_as(C.c_void_p), len(inputs),
            last.ctypes.data_as(C.c_void_p), None if layers is None else layers.ctypes.data_as(C.c_void_p))
        L.check(code, "forward_batch")
        return (last, layers) if want_layers else last

    # ---- prefix capture / continuation (PrefixState, model.rs:557-588, 954-1073) ----
    def capture_prefix(self, ids):
        """Run a prefix (a positive multiple of 64 tokens) once and keep its per-layer state on
        the device. Returns a Prefix to pass to forward_continue; release it with .close()."""
        ids = np.ascontiguousarray(np.asarray(ids, np.int64))
        if ids.size and (ids.min() < 0 or ids.max() >= 2 ** 31):
            raise ValueError("token id outside the vocabulary")
        ids = ids.astype(np.int32)
        handle = C.c_void_p()
        L.check(L.load().s1_prefix_create(self.handle, int(ids.size), C.byref(handle)), "prefix create")
        prefix = Prefix(handle, int(ids.size))
        try:
            L.check(L.load().s1_model_prefix_capture(self.handle, ids.ctypes.data_as(C.c_void_p), int(ids.size), handle),
                    "prefix capture")
        except Exception:
            prefix.close()
            raise
        return prefix

    def forward_continue(self, prefix, candidates):
        """candidates: token id sequences that each continue the captured prefix. Returns the
        final-norm hidden state of every candidate's last token, float32 [n, hidden] - what
        forward_batch returns for the prompts prefix + candidate."""
        lengths = np.array([len(x) for x in candidates], np.int32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(x, np.int64) for x in candidates]) if len(candidates)
                                   else np.zeros(0, np.int64))
        if ids.size and (ids.min() < 0 or ids.max() >= 2 ** 31):
            raise ValueError("token id outside the vocabulary")
        ids = ids.astype(np.int32)
        last = np.zeros((len(candidates), self.cfg.hidden), np.float32)
        L.check(L.load().s1_model_forward_continue(self.handle, prefix.handle, ids.ctypes.data_as(C.c_void_p),
                                                   lengths.ctypes.data_as(C.c_void_p), len(candidates),
                                                   last.ctypes.data_as(C.c_void_p)), "forward_continue")
        return last

    def forward_flat(self, ids, lengths):
        """The same pass on an int32 array used in place (e.g. a view of pinned host memory)."""
        assert ids.dtype == np.int32 and ids.flags["C_CONTIGUOUS"]
        lengths = np.ascontiguousarray(lengths, dtype=np.int32)
        last = np.zeros((lengths.size, self.cfg.hidden), np.float32)
        L.check(L.load().s1_model_forward_batch(self.handle, ids.ctypes.data_as(C.c_void_p),
                                                lengths.ctypes.data_as(C.c_void_p), lengths.size,
                                                last.ctypes.data_as(C.c_void_p), None), "forward_batch")
        return last

    def forward(self, ids):
        return self.forward_batch([ids])[0]

    def forward_device(self, ids_device, lengths):
        """Queue a pass over ids already on the device; returns the device pointer of the last rows."""
        lengths = np.ascontiguousarray(lengths, dtype=np.int32)
        out = C.c_void_p()
        L.check(L.load().s1_model_forward_device(self.handle, ids_device, lengths.ctypes.data_as(C.c_void_p),
                                                 lengths.size, C.byref(out)), "forward_device")
        return out

    def synchronize(self):
        L.check(L.load().s1_model_sync(self.handle), "sync")


def head_logits(weights, last, bias=None):
    """float32 logits [n_classes] of one last-token row; raises on a non-finite logit."""
    weights = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1, np.asarray(last).size)
    last = np.ascontiguousarray(last, dtype=np.float32)
    n = weights.shape[0]
    b = None if bias is None else np.ascontiguousarray(np.broadcast_to(np.asarray(bias, np.float32), (n,)))
    out = np.zeros(n, np.float32)
    code = L.load().s1_head_logits(weights.ctypes.data_as(C.c_void_p), None if b is None else b.ctypes.data_as(C.c_void_p),
                                   last.ctypes.data_as(C.c_void_p), last.size, n, out.ctypes.data_as(C.c_void_p))
    if code == 3001:
        raise ValueError("non-finite decision score")
    L.check(code, "head")
    return out


@dataclass
class DecisionHead:
    """The scalar head of the Open-Jev worker: score = f32(sum_f64 w*h) + bias."""
    weights: np.ndarray
    bias: float = 0.0

    def score(self, last):
        return head_logits(self.weights, last, self.bias)[0]


@dataclass
class Export:
    """A merged Open-Jev export's manifest, open_jev_export.json (engine.rs:21-46): the trained
    scalar head, the calibration temperature of contract::answer and the prompt length cap."""
    head: DecisionHead
    temperature: float
    max_length: int
    model_id: str

    @classmethod
    def load(cls, directory, hidden):
        w = np.zeros(hidden, np.float32)
        bias, temp, length, mid = C.c_float(), C.c_double(), C.c_int(), C.create_string_buffer(128)
        L.check(L.load().s1_export_read(os.fsencode(directory), hidden, w.ctypes.data_as(C.c_void_p), C.byref(bias),
                                        C.byref(temp), C.byref(length), mid, 128), "export manifest")
        return cls(DecisionHead(w, bias.value), temp.value, length.value, mid.value.decode())

    def decide(self, last_rows):
        """(index of the chosen candidate, probabilities) from the candidates' last-token rows."""
        scores = np.array([self.head.score(row) for row in last_rows], np.float32)
        return answer(scores, self.temperature)


def letter_logits(letters, last, n_options):
    last = np.asarray(last, np.float32)
    letters = np.asarray(letters, np.float32).reshape(-1, last.size)[:n_options]
    try:
        return head_logits(letters, last)
    except ValueError:
        raise ValueError("non-finite probabilities")


def ranges(lengths):
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    starts = np.zeros(max(1, lengths.size), np.int32)
    n = L.load().s1_batch_ranges(lengths.ctypes.data_as(C.c_void_p), lengths.size, starts.ctypes.data_as(C.c_void_p))
    edges = [int(s) for s in starts[:n]] + [int(lengths.size)]
    return [range(edges[i], edges[i + 1]) for i in range(n)]


def answer(logits, temperature=1.0):
    """(argmax with first-maximum ties, probabilities) of the calibrated softmax."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    probs = np.zeros(logits.size, np.float64)
    mode = L.load().s1_decide(logits.ctypes.data_as(C.c_void_p), logits.size, float(temperature),
                              probs.ctypes.data_as(C.c_void_p))
    if mode < 0:
        raise ValueError("invalid logits or temperature")
    return mode, probs


def assign_requests(lengths, n_ranks, a=1.0, b=0.0):
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    out = np.zeros(lengths.size, np.int32)
    L.check(L.load().s1_assign_requests(lengths.ctypes.data_as(C.c_void_p), lengths.size, n_ranks, a, b,
                                        out.ctypes.data_as(C.c_void_p)), "assign")
    return out
