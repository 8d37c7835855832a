"""ctypes binding of libqwen3_5_cuda.so: the cs1_* C ABI and the s1_* additions.

The role of the reference's Rust loader (src/models/qwen3_5/native/src/cuda.rs:24-190):
resolve every entry point, check the ABI version, turn non-zero codes into errors, and own
device buffers. There is no fallback: if the library is missing or a symbol does not
resolve, loading raises.
"""
import ctypes as C
import os

import numpy as np

ABI_VERSION = 6
_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqwen3_5_cuda.so")

vp, sz, i32, f32, f64 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_double
vpp = C.POINTER(C.c_void_p)
ip = C.POINTER(C.c_int)


class S1Config(C.Structure):
    _fields_ = [("hidden", i32), ("intermediate", i32), ("n_layers", i32), ("heads", i32), ("kv_heads", i32),
                ("head_dim", i32), ("rotary_half", i32), ("lin_k_heads", i32), ("lin_v_heads", i32), ("vocab", i32),
                ("max_positions", i32), ("eps", f32), ("rope_theta", f64), ("full_attention", C.POINTER(C.c_ubyte))]


# name -> (restype, argtypes); every cs1_* symbol of include/cs1_ops.h and s1_* of include/s1_executor.h
# and include/s1_dispatch.h
SIGNATURES = {
    "cs1_abi_version": (C.c_uint32, []),
    "cs1_error_string": (C.c_char_p, [i32]),
    "cs1_set_device": (i32, [i32]),
    "cs1_malloc": (i32, [vpp, sz]),
    "cs1_free": (i32, [vp]),
    "cs1_stream_create": (i32, [vpp]),
    "cs1_stream_sync": (i32, [vp]),
    "cs1_stream_destroy": (i32, [vp]),
    "cs1_graph_begin": (i32, [vp]),
    "cs1_graph_end": (i32, [vp, vpp]),
    "cs1_graph_launch": (i32, [vp, vp]),
    "cs1_graph_destroy": (i32, [vp]),
    "cs1_upload": (i32, [vp, vp, sz, vp]),
    "cs1_download": (i32, [vp, vp, sz, vp]),
    "cs1_copy_dd": (i32, [vp, vp, sz, vp]),
    "cs1_copy2d": (i32, [vp, sz, vp, sz, sz, sz, vp]),
    "cs1_embed": (i32, [vp, vp, vp, i32, i32, vp]),
    "cs1_rms_norm": (i32, [vp, vp, vp, i32, i32, f32, vp]),
    "cs1_add_rms_norm": (i32, [vp, vp, vp, vp, i32, i32, f32, vp]),
    "cs1_gated_rms_norm": (i32, [vp, vp, i32, vp, vp, i32, i32, i32, f32, vp]),
    "cs1_gdn_conv": (i32, [vp, i32, vp, vp, vp, vp, i32, i32, i32, vp]),
    "cs1_gdn_gates": (i32, [vp, vp, i32, vp, vp, vp, vp, i32, i32, vp]),
    "cs1_gdn_workspace_floats": (sz, [i32, i32]),
    "cs1_gdn_prefill": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp]),
    "cs1_gdn_prefill_x": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp, vp, vp]),
    "cs1_gdn_prefill_static": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp]),
    "cs1_attn_prep": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp]),
    "cs1_attention": (i32, [vp, vp, vp, i32, vp, i32, i32, i32, i32, f32, vp]),
    "cs1_attention_gated": (i32, [vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, f32, vp]),
    "cs1_attention_gated_prefix": (i32, [vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, f32, i32, vp]),
    "cs1_sigmoid_gate": (i32, [vp, vp, sz, vp]),
    "cs1_silu_mul": (i32, [vp, i32, vp, i32, i32, vp]),
    "cs1_gemm_create": (vp, [sz]),
    "cs1_gemm_destroy": (None, [vp]),
    "cs1_gemm": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "cs1_vision_linear": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "cs1_gemm_f32": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "cs1_vision_norm": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "cs1_vision_position": (i32, [vp, vp, vp, vp, i32, vp]),
    "cs1_vision_rope": (i32, [vp, vp, vp, vp, vp, i32, vp]),
    "cs1_vision_attention": (i32, [vp, vp, vp, vp, i32, vp]),
    "cs1_vision_bias": (i32, [vp, vp, sz, i32, vp]),
    "cs1_vision_gelu": (i32, [vp, sz, i32, vp]),
    "cs1_vision_add": (i32, [vp, vp, sz, vp]),
    "cs1_vision_to_float": (i32, [vp, vp, sz, vp]),
    "cs1_vision_lora_add": (i32, [vp, vp, sz, f32, vp]),
    # additions
    "s1_device_count": (i32, [ip]),
    "s1_event_create": (i32, [vpp]),
    "s1_event_destroy": (i32, [vp]),
    "s1_event_record": (i32, [vp, vp]),
    "s1_event_sync": (i32, [vp]),
    "s1_event_elapsed_ms": (i32, [vp, vp, C.POINTER(f32)]),
    "s1_host_alloc": (i32, [vpp, sz]),
    "s1_host_free": (i32, [vp]),
    "s1_upload_async": (i32, [vp, vp, sz, vp]),
    "s1_download_async": (i32, [vp, vp, sz, vp]),
    "s1_memset_async": (i32, [vp, i32, sz, vp]),
    "s1_device_sync": (i32, []),
    "s1_mem_info": (i32, [C.POINTER(sz), C.POINTER(sz)]),
    "s1_gemm_plain": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "s1_gemm_plan_override": (i32, [i32, i32, i32, i32]),
    "s1_gemm_tcgen05": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "s1_gemm_tc5_status": (i32, [ip]),
    "s1_gemm_tc5_cluster_room": (i32, [i32, i32]),
    "s1_gemm_unsplit": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "s1_attn_tc5_status": (i32, [ip]),
    "s1_gdn_status": (i32, [ip]),
    "s1_l2norm_heads": (i32, [vp, vp, C.c_longlong, f32, vp]),
    "s1_gdn_conv_gates": (i32, [vp, i32, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32, vp]),
    "s1_checkpoint_inspect": (i32, [C.c_char_p, C.c_char_p, C.c_size_t, ip, i32, C.c_char_p, C.c_size_t, C.c_char_p,
                                    C.c_size_t, ip, vp, vp]),
    "s1_model_load_checkpoint": (i32, [vp, C.c_char_p, C.c_char_p, C.c_size_t]),
    "s1_model_unfilled": (i32, [vp, C.c_char_p, C.c_size_t]),
    "s1_model_tensor_shape": (i32, [vp, C.c_char_p, ip, vp]),
    "s1_export_read": (i32, [C.c_char_p, i32, vp, C.POINTER(f32), C.POINTER(f64), ip, C.c_char_p, C.c_size_t]),
    "s1_gemm_swiglu": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "s1_model_set_exact_packing": (i32, [vp, i32]),
    "s1_model_set_overlap_tokens": (i32, [vp, i32]),
    "s1_set_dependent_launch": (i32, [i32]),
    "s1_model_set_fused_mlp": (i32, [vp, i32]),
    "s1_attention_gated_shared_prefix": (i32, [vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp]),
    "s1_prefix_create": (i32, [vp, i32, vp]),
    "s1_prefix_destroy": (None, [vp]),
    "s1_prefix_bytes": (C.c_size_t, [vp]),
    "s1_prefix_len": (i32, [vp]),
    "s1_model_prefix_capture": (i32, [vp, vp, i32, vp]),
    "s1_model_forward_continue": (i32, [vp, vp, vp, vp, i32, vp]),
    "s1_model_create": (i32, [C.POINTER(S1Config), i32, vpp]),
    "s1_model_destroy": (None, [vp]),
    "s1_model_set_tensor": (i32, [vp, C.c_char_p, vp, sz]),
    "s1_model_tensor": (i32, [vp, C.c_char_p, vpp, C.POINTER(sz)]),
    "s1_model_init_random": (i32, [vp, C.c_uint64, f32]),
    "s1_model_weight_bytes": (sz, [vp]),
    "s1_model_stream": (vp, [vp]),
    "s1_model_enable_graphs": (i32, [vp, i32]),
    "s1_model_graph_stats": (i32, [vp, ip, ip, ip]),
    "s1_model_forward_batch": (i32, [vp, vp, vp, i32, vp, vp]),
    "s1_model_forward_device": (i32, [vp, vp, vp, i32, vpp]),
    "s1_model_sync": (i32, [vp]),
    "s1_model_profile": (i32, [vp, i32]),
    "s1_model_profile_read": (i32, [vp, vp, vp, vp]),
    "s1_gemm_engine": (i32, [vp, vp, vp, i32, i32, i32]),
    "s1_head_logits": (i32, [vp, vp, vp, i32, i32, vp]),
    "s1_decide": (i32, [vp, i32, f64, vp]),
    "s1_batch_ranges": (i32, [vp, i32, vp]),
    "s1_assign_requests": (i32, [vp, i32, i32, f64, f64, vp]),
    "s1_gdn_conv_gates_batch": (i32, [vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32, vp]),
    "s1_attn_prep_batch": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, f32, vp]),
    "s1_attention_gated_batch": (i32, [vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, vp, vp, i32, i32, i32, i32, f32, vp]),
    "s1_gdn_prefill_batch": (i32, [vp, vp, vp, vp, vp, vp, vp, C.c_size_t, vp, vp, i32, i32, i32, f32, vp, vp, vp]),
    "s1_assign_requests_weighted": (i32, [vp, i32, i32, f64, f64, vp, vp]),
    "s1_device_status": (i32, [ip, ip, ip]),
    "s1_selftest_wait_runs_out": (i32, [i32, vp]),
    "s1_model_config": (i32, [vp, C.POINTER(S1Config)]),
    "s1_model_reserve": (i32, [vp, i32]),
    "s1_model_forward_queue": (i32, [vp, vp, vp, i32, vp]),
    "s1_model_read_rows": (i32, [vp, vp, vp, sz]),
    # include/s1_dispatch.h
    "s1_dispatch_create": (i32, [i32, i32, i32, C.c_char_p, C.c_char_p, vpp]),
    "s1_dispatch_destroy": (None, [vp]),
    "s1_dispatch_set_cost": (i32, [vp, f64, f64]),
    "s1_dispatch_layout": (i32, [vp, i32, i32, f64, f64, i32, vp, vp, ip, vp]),
    "s1_dispatch_layout_weighted": (i32, [vp, i32, i32, f64, f64, vp, i32, vp, vp, ip, vp]),
    "s1_dispatch_set_speed": (i32, [vp, vp, i32]),
    "s1_dispatch_candidates": (i32, [vp, vp, vp, vp, vp, i32, vp, vp, i32, vp, vp]),
    "s1_dispatch_plan": (i32, [vp, vp, vp, i32, i32]),
    "s1_dispatch_info": (i32, [vp, ip, C.POINTER(C.c_longlong), ip, vp]),
    "s1_dispatch_local": (i32, [vp, vp, vp]),
    "s1_dispatch_stage": (i32, [vp, vp]),
    "s1_dispatch_upload": (i32, [vp]),
    "s1_dispatch_enqueue": (i32, [vp, i32]),
    "s1_dispatch_pack_ms": (i32, [vp, vp]),
    "s1_dispatch_collect": (i32, [vp, vp, vp, vp, C.POINTER(f64)]),
    "s1_dispatch_barrier": (i32, [vp]),
    "s1_dispatch_allreduce_max": (i32, [vp, vp, i32]),
    "s1_dispatch_allgather": (i32, [vp, vp, i32, vp]),
}

_LIB = None
# cs1_* entry points of this library that the reference's ABI does not have
NOT_IN_REFERENCE = {"cs1_gdn_prefill_static"}


class CudaError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: error {code}: {error_string(code)}")


def load(path=None):
    """dlopen the library once per process, bind every symbol and check the ABI version."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = path or os.environ.get("CUA_S1_CUDA_LIB") or LIB_PATH
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} is missing: build it with `python -m system1_omni_b200.build`")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a symbol does not resolve
        fn.restype = res
        fn.argtypes = args
    version = lib.cs1_abi_version()
    if version != ABI_VERSION:
        raise RuntimeError(f"{path} has ABI version {version}, expected {ABI_VERSION}")
    _LIB = lib
    return lib


def error_string(code):
    s = load().cs1_error_string(int(code))
    return s.decode() if s else "?"


def check(code, what):
    if code != 0:
        raise CudaError(code, what)


def set_device(device):
    check(load().cs1_set_device(int(device)), "set device")


def device_count():
    n = C.c_int(0)
    code = load().s1_device_count(C.byref(n))
    return n.value if code == 0 else 0


class Stream:
    def __init__(self):
        self.handle = C.c_void_p()
        check(load().cs1_stream_create(C.byref(self.handle)), "stream")

    def sync(self):
        check(load().cs1_stream_sync(self.handle), "stream sync")

    def __del__(self):
        if getattr(self, "handle", None) and _LIB is not None:
            _LIB.cs1_stream_destroy(self.handle)
            self.handle = None


class Event:
    def __init__(self):
        self.handle = C.c_void_p()
        check(load().s1_event_create(C.byref(self.handle)), "event")

    def record(self, stream):
        check(load().s1_event_record(self.handle, stream.handle if isinstance(stream, Stream) else stream), "record")

    def sync(self):
        check(load().s1_event_sync(self.handle), "event sync")

    def elapsed_ms(self, later):
        ms = C.c_float(0)
        check(load().s1_event_elapsed_ms(self.handle, later.handle, C.byref(ms)), "elapsed")
        return ms.value

    def __del__(self):
        if getattr(self, "handle", None) and _LIB is not None:
            _LIB.s1_event_destroy(self.handle)
            self.handle = None


class DeviceBuffer:
    """A device allocation released on drop (cuda.rs DeviceBuffer)."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        self.ptr = C.c_void_p()
        check(load().cs1_malloc(C.byref(self.ptr), max(self.nbytes, 1)), "malloc")

    def at(self, offset=0):
        return C.c_void_p(self.ptr.value + int(offset))

    def __del__(self):
        if getattr(self, "ptr", None) and self.ptr.value and _LIB is not None:
            _LIB.cs1_free(self.ptr)
            self.ptr = None


def to_device(array, stream, offset_elems=0):
    """Upload a numpy array; offset_elems leaves that many elements of padding in front."""
    a = np.ascontiguousarray(array)
    pad = offset_elems * a.itemsize
    buf = DeviceBuffer(a.nbytes + pad)
    if a.nbytes:
        check(load().cs1_upload(buf.at(pad), a.ctypes.data_as(C.c_void_p), a.nbytes, stream.handle), "upload")
    return buf


def from_device(buf, shape, dtype, stream, offset_bytes=0):
    out = np.empty(shape, dtype)
    if out.nbytes:
        check(load().cs1_download(out.ctypes.data_as(C.c_void_p), buf.at(offset_bytes), out.nbytes, stream.handle),
              "download")
    return out


def device_status():
    """(gemm, attention, delta rule) error words of the current device after a device sync; cleared."""
    g, a, d = C.c_int(0), C.c_int(0), C.c_int(0)
    check(load().s1_device_status(C.byref(g), C.byref(a), C.byref(d)), "device status")
    return g.value, a.value, d.value


def gemm_status():
    code = C.c_int(0)
    check(load().s1_gemm_tc5_status(C.byref(code)), "gemm status")
    return code.value


def attn_status():
    code = C.c_int(0)
    check(load().s1_attn_tc5_status(C.byref(code)), "attention status")
    return code.value


def gdn_status():
    code = C.c_int(0)
    check(load().s1_gdn_status(C.byref(code)), "delta-rule status")
    return code.value


def load_other(path):
    """Bind a second library that exports the same cs1_* ABI (the reference's own build, for
    side-by-side runs). Only the cs1_* symbols are bound; nothing is cached."""
    other = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        if name.startswith("cs1_") and name not in NOT_IN_REFERENCE:
            fn = getattr(other, name)
            fn.restype = res
            fn.argtypes = args
    if other.cs1_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{path}: ABI version {other.cs1_abi_version()}")
    return other
