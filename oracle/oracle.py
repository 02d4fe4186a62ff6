"""ctypes bindings for the CPU oracle (oracle/oracle.cpp) and, when built, the
reference's own quantizer (oracle/_ref/libref_quants.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
cpu_baseline / reference arm of bench.py. The product package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libref_quants.so")

u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
u32, u64, f32, i32, vp = C.c_uint32, C.c_uint64, C.c_float, C.c_int, C.c_void_p


def reference_tree():
    """Path of a vkllama source tree to build the reference's own quantizer from: the
    VKLLAMA_REFERENCE environment variable, else a `reference` folder beside this repository's
    parent; None when neither holds src/core/quants.h."""
    cands = [os.environ.get("VKLLAMA_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "src", "core", "quants.h")):
            return c
    return None


def build(force=False):
    """Compile liboracle.so (and oracle/_ref when the reference tree is here)."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    ref = reference_tree()
    if ref and (force or not os.path.exists(_REF)):
        subprocess.check_call(["make", "-C", _HERE, "ref", "REF=" + ref], stdout=subprocess.DEVNULL)


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_LIB)

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("orc_threads", i32)
    sig("orc_set_threads", None, i32)
    sig("orc_synth_normal_f32", None, u64, u64, u64, u64, f32, f32, f32p)
    sig("orc_synth_normal_f16", None, u64, u64, u64, u64, f32, f32, u16p)
    sig("orc_synth_tokens", None, u64, u64, u64, u32, u32p)
    sig("orc_q8_0_quantize34", None, f32p, u8p, u64, u64)
    sig("orc_q8_0_quantize36", None, f32p, u8p, u64, u64)
    sig("orc_q8_0_dequantize34", None, u8p, f32p, u64, u64)
    sig("orc_synth_q8_0", None, u64, u64, u64, u64, f32, f32, u8p)
    sig("orc_matmul_q8_0", None, u16p, u8p, u16p, u32, u32, u32, f32, f32, i32)
    sig("orc_kqv_q8_0", None, u16p, u8p, u8p, u8p, u16p, u16p, u16p, u32, u32, u32)
    sig("orc_ffn_up_gate_q8_0", None, u16p, u8p, u8p, u16p, u32, u32, u32)
    sig("orc_feed_forward_q8_0", None, u16p, u8p, u8p, u8p, u16p, u32, u32, u32)
    sig("orc_feed_forward_f16", None, u16p, u16p, u16p, u16p, u16p, u32, u32, u32)
    for n in ("orc_matmul_tb_f16", "orc_matmul_nn_f16"):
        sig(n, None, u16p, u16p, u16p, u32, u32, u32, u32, u64, u64, u64, u64, u64, u64, f32, f32, i32)
    sig("orc_softmax_f16", None, u16p, u16p, u32, u32, u32, i32, u32)
    sig("orc_rope_table", None, u32, u32, f32p, f32p)
    sig("orc_rope_f16", None, u16p, u32, u32, u32, u32, f32p, f32p)
    sig("orc_update_kvcache_f16", None, u16p, u16p, u32, u32, u32, u32, u32, u32)
    sig("orc_rms_norm_f16", None, u16p, f32p, u16p, u32, u32, f32)
    sig("orc_add_f16", None, u16p, u16p, u64)
    sig("orc_embedding_q8_0", None, u8p, u32p, u16p, u32, u32, u32, u32)
    sig("orc_embedding_f16", None, u16p, u32p, u16p, u32, u32, u32, u32)
    sig("orc_argmax_f16", None, u16p, u32p, u32, u32)
    sig("orc_argmax_f32", u32, f32p, u32)
    sig("orc_transpose_f16", None, u16p, u16p, u32, u32, u32)
    sig("orc_attn_create", vp, u32, u32, u32)
    sig("orc_attn_destroy", None, vp)
    sig("orc_attn_kcache", C.POINTER(C.c_uint16), vp)
    sig("orc_attn_vcache", C.POINTER(C.c_uint16), vp)
    sig("orc_attn_forward_q8_0", None, vp, u16p, u8p, u8p, u8p, u8p, u32, u32, i32, u16p)
    sig("orc_model_create", vp, u32, u32, u32, u32, u32, u32, f32, f32)
    sig("orc_model_destroy", None, vp)
    sig("orc_model_synth", None, vp, u64, f32, f32)
    sig("orc_model_synth_f16", None, vp, u64, f32, f32)
    sig("orc_model_weight", vp, vp, u32, u32, C.POINTER(u64))
    sig("orc_model_kcache", C.POINTER(C.c_uint16), vp, u32)
    sig("orc_model_vcache", C.POINTER(C.c_uint16), vp, u32)
    sig("orc_block_forward", None, vp, u32, u16p, u32, u32, i32, u16p)
    sig("orc_model_forward", None, vp, u32p, u32, u32, f32p, vp)
    sig("orc_model_generate", None, vp, u32p, u32, u32, u32p, f32p)
    _lib = L
    return L


_ref = None


def ref():
    """The reference's own quantizer, or None when oracle/_ref was never built."""
    global _ref
    if _ref is not None:
        return _ref
    build()
    if not os.path.exists(_REF):
        return None
    R = C.CDLL(_REF)
    R.ref_q8_0_quantize.restype = i32
    R.ref_q8_0_quantize.argtypes = [f32p, np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS"), C.c_size_t, C.c_size_t]
    R.ref_q8_0_dequantize.restype = i32
    R.ref_q8_0_dequantize.argtypes = [np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS"), f32p, C.c_size_t, C.c_size_t]
    R.ref_q8_0_bytes_per_block.restype = C.c_uint
    R.ref_fp32_to_fp16.restype = C.c_ushort
    R.ref_fp32_to_fp16.argtypes = [f32]
    R.ref_fp16_to_fp32.restype = f32
    R.ref_fp16_to_fp32.argtypes = [C.c_ushort]
    _ref = R
    return R


# ---- thin numpy helpers -----------------------------------------------------
SLOTS = dict(attn_norm=0, wq=1, wk=2, wv=3, wo=4, ffn_norm=5, gate=6, up=7, down=8)
GLOBALS = dict(tok_embd=0, output_norm=1, output=2)


def f16(a):
    """uint16 bit patterns -> float32 values."""
    return np.asarray(a, np.uint16).view(np.float16).astype(np.float32)


def bits(a):
    """float array -> fp16 bit patterns (round to nearest even)."""
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def synth_f32(seed, tensor, n, mean=0.0, std=1.0, first=0):
    out = np.empty(n, np.float32)
    lib().orc_synth_normal_f32(seed, tensor, first, n, mean, std, out)
    return out


def synth_f16(seed, tensor, n, mean=0.0, std=1.0, first=0):
    out = np.empty(n, np.uint16)
    lib().orc_synth_normal_f16(seed, tensor, first, n, mean, std, out)
    return out


def threads():
    """OpenMP threads the oracle's loops run on."""
    return int(lib().orc_threads())


def set_threads(n):
    lib().orc_set_threads(int(n))


def synth_tokens(seed, tensor, n, vocab):
    out = np.empty(n, np.uint32)
    lib().orc_synth_tokens(seed, tensor, n, vocab, out)
    return out


def synth_q8_0(seed, tensor, rows, K, mean=0.0, std=0.02):
    out = np.empty(rows * ((K + 31) // 32) * 34, np.uint8)
    lib().orc_synth_q8_0(seed, tensor, rows, K, mean, std, out)
    return out


def quantize34(x):
    x = np.ascontiguousarray(x, np.float32)
    h, w = x.shape
    out = np.empty(h * ((w + 31) // 32) * 34, np.uint8)
    lib().orc_q8_0_quantize34(x, out, h, w)
    return out


def quantize36(x):
    x = np.ascontiguousarray(x, np.float32)
    h, w = x.shape
    out = np.empty(h * ((w + 31) // 32) * 36, np.uint8)
    lib().orc_q8_0_quantize36(x, out, h, w)
    return out


def matmul_q8_0(x, w, M, N, K, scale=1.0, bias=0.0, act=0):
    y = np.empty(M * N, np.uint16)
    lib().orc_matmul_q8_0(np.ascontiguousarray(x), w, y, M, N, K, scale, bias, act)
    return y.reshape(M, N)


class Model:
    """Synthetic Llama-2-shaped model held by the oracle."""

    def __init__(self, dim, heads, ffn, vocab, layers, maxlen, eps=1e-5, final_eps=1e-6,
                 seed=0, wstd=0.02, nstd=0.01, fp16=False):
        self.cfg = dict(dim=dim, heads=heads, ffn=ffn, vocab=vocab, layers=layers,
                        maxlen=maxlen, eps=eps, final_eps=final_eps)
        self.fp16 = fp16
        self.L = lib()
        self.h = self.L.orc_model_create(dim, heads, ffn, vocab, layers, maxlen, eps, final_eps)
        (self.L.orc_model_synth_f16 if fp16 else self.L.orc_model_synth)(self.h, seed, wstd, nstd)

    def weight(self, layer, slot):
        """Raw bytes (34-byte blocks or dense fp16; fp32 for norms) as a numpy view."""
        n = u64(0)
        p = self.L.orc_model_weight(self.h, layer, slot, C.byref(n))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,))

    def kcache(self, layer):
        c = self.cfg
        return np.ctypeslib.as_array(self.L.orc_model_kcache(self.h, layer),
                                     shape=(c["heads"], c["maxlen"], c["dim"] // c["heads"]))

    def vcache(self, layer):
        c = self.cfg
        return np.ctypeslib.as_array(self.L.orc_model_vcache(self.h, layer),
                                     shape=(c["heads"], c["maxlen"], c["dim"] // c["heads"]))

    def block(self, layer, x, T, offset, clip=False):
        out = np.empty((1 if clip else T) * self.cfg["dim"], np.uint16)
        self.L.orc_block_forward(self.h, layer, np.ascontiguousarray(x), T, offset, int(clip), out)
        return out.reshape(-1, self.cfg["dim"])

    def forward(self, toks, offset, want_hidden=False):
        toks = np.ascontiguousarray(toks, np.uint32)
        logits = np.empty(self.cfg["vocab"], np.float32)
        hid = np.empty(self.cfg["dim"], np.uint16) if want_hidden else None
        self.L.orc_model_forward(self.h, toks, len(toks), offset, logits,
                                 hid.ctypes.data if want_hidden else None)
        return (logits, hid) if want_hidden else logits

    def generate(self, prompt, n_gen):
        prompt = np.ascontiguousarray(prompt, np.uint32)
        ids = np.empty(n_gen, np.uint32)
        gap = np.empty(n_gen, np.float32)
        self.L.orc_model_generate(self.h, prompt, len(prompt), n_gen, ids, gap)
        return ids, gap

    def close(self):
        if self.h:
            self.L.orc_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- generic ops outside the token loop (numpy restatements of the shaders; fp16 bit patterns in and out) ----
def elementwise(x_bits, y, op):
    """src/shaders/element_wise_fp16.comp:19-48 (two tensors) and element_wise_constant_fp16.comp:19-44
    (tensor and scalar): fp32 arithmetic, one rounding to fp16. op 0 add, 1 sub, 2 mul, 3 div."""
    a = f16(x_bits)
    b = f16(y) if isinstance(y, np.ndarray) else np.float32(y)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = [a + b, a - b, a * b, a / b][op]
    return bits(r.astype(np.float32)).reshape(np.asarray(x_bits).shape)


def concat(inputs, axis):
    """src/ops/concat.cpp:115-170 + src/shaders/concat_fp16.comp:27-49: plain copies at growing offsets."""
    return np.concatenate([np.asarray(t, np.uint16) for t in inputs], axis=axis)


def reduce(x_bits, op):
    """src/shaders/reduce_fp16.comp:24-76 with src/ops/reduce.h:96-99: per row, 32 lane-strided fp32 partial
    results (max and min start from the row's first value), combined in lane order, times 1/W for the mean
    (op 3), one rounding to fp16. [c,h,w] -> [c,h,1]."""
    x = f16(x_bits)
    C, H, W = x.shape
    k = 0 if op == 3 else op
    out = np.empty((C, H, 1), np.float32)
    for c in range(C):
        rows = x[c]
        lanes = []
        for l in range(32):
            part = rows[:, l::32]
            if k == 0:
                acc = np.zeros(H, np.float32)
                for j in range(part.shape[1]):
                    acc = (acc + part[:, j]).astype(np.float32)
            else:
                acc = rows[:, 0].copy()
                for j in range(part.shape[1]):
                    acc = np.maximum(acc, part[:, j]) if k == 1 else np.minimum(acc, part[:, j])
            lanes.append(acc)
        tot = lanes[0]
        for l in range(1, 32):
            tot = (tot + lanes[l]).astype(np.float32) if k == 0 else (np.maximum(tot, lanes[l]) if k == 1 else np.minimum(tot, lanes[l]))
        out[c, :, 0] = tot * (np.float32(1.0) / np.float32(W) if op == 3 else np.float32(1.0))
    return bits(out)


def read_kvcache(cache_bits, offset, length):
    """src/shaders/read_kvcache_fp16.comp: out[c, y, :] = cache[c, (y + offset) % H, :]."""
    c = np.asarray(cache_bits, np.uint16)
    idx = (np.arange(length) + offset) % c.shape[1]
    return np.ascontiguousarray(c[:, idx, :])


def matmul_broadcast(a_bits, b_bits, broadcast_type, transpose_b, scale=1.0, bias=0.0, act=0):
    """src/shaders/matmul_broadcast{0,1,2}_fp16_v2.comp: per channel C = act(A . B(^T) * scale + bias) with fp32
    accumulation; type 1 shares one B among the channels of A, type 2 one A among the channels of B."""
    a, b = f16(a_bits), f16(b_bits)
    C = max(a.shape[0], b.shape[0])
    outs = []
    for c in range(C):
        ac = a[0 if broadcast_type == 2 else c]
        bc = b[0 if broadcast_type == 1 else c]
        v = (ac.astype(np.float64) @ (bc.T if transpose_b else bc).astype(np.float64)).astype(np.float32) * np.float32(scale) + np.float32(bias)
        if act == 1:
            v = v / (1.0 + np.exp(-v))
        outs.append(v)
    return bits(np.stack(outs).astype(np.float32))
