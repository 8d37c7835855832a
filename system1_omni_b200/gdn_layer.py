"""One Gated DeltaNet layer's mixer on the device, operator by operator through the C ABI:

    in_proj GEMM [qkv | z | b | a] -> causal conv1d(k=4) + SiLU + split -> beta / log-decay gates
    -> chunked gated delta rule (q, k L2-normalised inside) -> gated RMSNorm with SiLU(z) -> out_proj GEMM

the sequence of the reference's layer loop for a linear-attention layer
(src/models/qwen3_5/native/src/model.rs:1160-1235). This is the "single Gated DeltaNet layer
prefill" configuration: batch 1, T tokens, 16 q/k heads and 16 v heads of 128 by default.
"""
import ctypes as C

import numpy as np

from . import lib as L


class GdnLayer:
    def __init__(self, hidden=2048, k_heads=16, v_heads=16, max_tokens=2048, eps=1e-6, stream=None):
        self.lib = L.load()
        self.hidden, self.hk, self.hv, self.eps = hidden, k_heads, v_heads, eps
        self.kd, self.vd = k_heads * 128, v_heads * 128
        self.conv = 2 * self.kd + self.vd
        self.gdn_in = self.conv + self.vd + 2 * v_heads
        self.cap = max_tokens
        self.stream = stream or L.Stream()
        self.gemm = self.lib.cs1_gemm_create(32 << 20)
        if not self.gemm:
            raise RuntimeError("cs1_gemm_create failed")
        T = max_tokens
        nb = lambda n: L.DeviceBuffer(n)
        self.w_in, self.w_out = nb(self.gdn_in * hidden * 2), nb(hidden * self.vd * 2)
        self.w_conv, self.a_log, self.dt_bias, self.w_norm = nb(self.conv * 4 * 2), nb(v_heads * 2), nb(v_heads * 2), nb(256)
        self.proj, self.q, self.k, self.v = nb(T * self.gdn_in * 2), nb(T * self.kd * 2), nb(T * self.kd * 2), nb(T * self.vd * 2)
        self.beta, self.g, self.o, self.n = nb(T * v_heads * 2), nb(T * v_heads * 4), nb(T * self.vd * 2), nb(T * self.vd * 2)
        self.ws = nb(self.lib.cs1_gdn_workspace_floats(T, v_heads) * 4)
        self.y = nb(T * hidden * 2)

    def close(self):
        if self.gemm:
            self.lib.cs1_gemm_destroy(self.gemm)
            self.gemm = None

    def set_weights(self, in_proj, conv, a_log, dt_bias, norm, out_proj):
        """bf16 bit patterns: in_proj [gdn_in, hidden] (qkv | z | b | a stacked), conv [conv, 4],
        a_log [hv], dt_bias [hv], norm [128], out_proj [hidden, vd]."""
        for buf, a in ((self.w_in, in_proj), (self.w_conv, conv), (self.a_log, a_log), (self.dt_bias, dt_bias),
                       (self.w_norm, norm), (self.w_out, out_proj)):
            a = np.ascontiguousarray(a)
            assert a.dtype == np.uint16 and a.nbytes <= buf.nbytes
            L.check(self.lib.cs1_upload(buf.at(), a.ctypes.data_as(C.c_void_p), a.nbytes, self.stream.handle), "upload")

    def forward(self, x_dev, T):
        """Queue the layer on x_dev (bf16 [T, hidden] on the device); the result lands in self.y."""
        lib, st = self.lib, self.stream.handle
        z = self.proj.at(self.conv * 2)
        b = self.proj.at((self.conv + self.vd) * 2)
        a = self.proj.at((self.conv + self.vd + self.hv) * 2)
        L.check(lib.cs1_gemm(self.gemm, x_dev, self.w_in.at(), self.proj.at(), T, self.gdn_in, self.hidden,
                             self.gdn_in, st), "in_proj")
        L.check(lib.cs1_gdn_conv(self.proj.at(), self.gdn_in, self.w_conv.at(), self.q.at(), self.k.at(), self.v.at(),
                                 T, self.kd, self.vd, st), "conv")
        L.check(lib.cs1_gdn_gates(b, a, self.gdn_in, self.a_log.at(), self.dt_bias.at(), self.beta.at(), self.g.at(),
                                  T, self.hv, st), "gates")
        L.check(lib.cs1_gdn_prefill(self.q.at(), self.k.at(), self.v.at(), self.g.at(), self.beta.at(), self.o.at(),
                                    self.ws.at(), T, self.hv, self.hk, 128 ** -0.5, st), "delta rule")
        L.check(lib.cs1_gated_rms_norm(self.o.at(), z, self.gdn_in, self.w_norm.at(), self.n.at(), T, self.hv, 128,
                                       self.eps, st), "gated norm")
        L.check(lib.cs1_gemm(self.gemm, self.n.at(), self.w_out.at(), self.y.at(), T, self.hidden, self.vd,
                             self.hidden, st), "out_proj")
        return self.y
