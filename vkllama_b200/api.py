"""ctypes bindings of include/vkllama_b200.h with the reference's class names."""
import ctypes as C
import os

import numpy as np

FP32, FP16, UINT32, INT8, Q8_0 = 0, 1, 2, 3, 4
_NP = {FP32: np.float32, FP16: np.uint16, UINT32: np.uint32, INT8: np.int8, Q8_0: np.uint8}

_HERE = os.path.dirname(os.path.abspath(__file__))
# the in-tree build; VKLLAMA_B200_LIB names another build of the same library (A/B comparisons)
_LIB_PATH = os.environ.get("VKLLAMA_B200_LIB") or os.path.join(_HERE, "libvkllama_b200.so")
_lib = None

vp, u32, u64, i32, f32, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_size_t
pvp = C.POINTER(C.c_void_p)


class VklError(RuntimeError):
    """A non-zero status from the C ABI (code = absl::StatusCode number)."""

    def __init__(self, code, msg):
        super().__init__("[%d] %s" % (code, msg))
        self.code = code
        self.message = msg


class ModelConfig(C.Structure):
    _fields_ = [("dim", u32), ("heads", u32), ("ffn", u32), ("vocab", u32), ("layers", u32),
                ("maxlen", u32), ("eps", f32), ("final_eps", f32), ("weight_dtype", i32),
                ("tp_rank", i32), ("tp_size", i32)]


def library_path():
    return _LIB_PATH


def load_library():
    """Load the in-tree shared library; raises when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ImportError("%s is missing: run `python -m vkllama_b200.build` (needs nvcc); "
                          "there is no fallback path" % _LIB_PATH)
    L = C.CDLL(_LIB_PATH)
    L.vkl_last_error.restype = C.c_char_p
    L.vkl_kernel_launches.restype = u64
    sigs = {
        "vkl_device_create": [i32, pvp], "vkl_device_destroy": [vp],
        "vkl_device_info": [vp, C.c_char_p, C.POINTER(i32), C.POINTER(sz)],
        "vkl_device_pool_bytes": [vp, C.POINTER(sz)],
        "vkl_tensor_create": [vp, i32, i32, i32, i32, pvp], "vkl_tensor_retain": [vp],
        "vkl_tensor_release": [vp], "vkl_tensor_view": [vp, sz, sz, sz, pvp],
        "vkl_tensor_reshape": [vp, sz, sz, sz], "vkl_tensor_shape": [vp, C.POINTER(u32)],
        "vkl_tensor_dtype": [vp, C.POINTER(i32)], "vkl_tensor_bytes": [vp, C.POINTER(sz)],
        "vkl_tensor_device_ptr": [vp, pvp],
        "vkl_command_create": [vp, pvp], "vkl_command_destroy": [vp], "vkl_command_begin": [vp],
        "vkl_command_end": [vp], "vkl_command_submit": [vp], "vkl_command_wait": [vp],
        "vkl_command_submit_and_wait": [vp], "vkl_command_elapsed_us": [vp, C.POINTER(f32)],
        "vkl_command_stream": [vp, pvp], "vkl_argmax_noalloc": [vp, u32, u32, vp, vp], "vkl_command_upload": [vp, vp, sz, vp],
        "vkl_command_download": [vp, vp, vp, sz],
        "vkl_op_init": [vp], "vkl_op_time": [vp, C.POINTER(u64)], "vkl_op_destroy": [vp],
        "vkl_matmul_create": [vp, vp, vp, f32, f32, i32, i32, i32, i32, i32, pvp],
        "vkl_matmul_run": [vp, vp, vp, pvp],
        "vkl_matmul_run_many": [C.POINTER(vp), sz, vp, sz, C.POINTER(f32)],
        "vkl_feed_forward_create": [vp, vp, vp, vp, vp, i32, i32, pvp], "vkl_feed_forward_run": [vp, vp, pvp],
        "vkl_mha_create": [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, pvp],
        "vkl_mha_run": [vp, vp, sz, pvp], "vkl_mha_caches": [vp, pvp, pvp],
        "vkl_update_kvcache_create": [vp, vp, i32, pvp], "vkl_update_kvcache_run": [vp, vp, vp, u32],
        "vkl_rms_norm_create": [vp, vp, vp, f32, i32, pvp], "vkl_rms_norm_run": [vp, vp, pvp],
        "vkl_rope_create": [vp, vp, i32, i32, i32, pvp], "vkl_rope_run": [vp, vp, sz, pvp],
        "vkl_softmax_create": [vp, vp, i32, f32, i32, pvp], "vkl_softmax_run": [vp, vp, sz, pvp],
        "vkl_argop_create": [vp, vp, i32, i32, pvp], "vkl_argop_run": [vp, vp, pvp],
        "vkl_embedding_create": [vp, vp, vp, u32, i32, pvp], "vkl_embedding_run": [vp, vp, pvp],
        "vkl_elementwise_create": [vp, vp, i32, i32, pvp], "vkl_elementwise_run": [vp, vp, vp, pvp],
        "vkl_transpose_create": [vp, vp, i32, i32, pvp], "vkl_transpose_run": [vp, vp, pvp],
        "vkl_slice_create": [vp, vp, i32, pvp],
        "vkl_slice_run": [vp, vp, C.POINTER(u32), C.POINTER(u32), pvp],
        "vkl_cast_create": [vp, vp, i32, i32, pvp], "vkl_cast_run": [vp, vp, pvp],
        "vkl_q8_0_quantize": [vp, vp, sz, sz], "vkl_q8_0_quantize36": [vp, vp, sz, sz],
        "vkl_q8_0_dequantize": [vp, vp, sz, sz], "vkl_q8_0_blocks36_to_34": [vp, vp, sz],
        "vkl_q8_0_quantize_device": [vp, vp, vp],
        "vkl_tensor_fill_synthetic": [vp, vp, u64, u64, f32, f32],
        "vkl_model_create": [vp, C.POINTER(ModelConfig), pvp], "vkl_model_destroy": [vp],
        "vkl_model_set_weight": [vp, C.c_char_p, i32, vp, sz],
        "vkl_model_synth_weights": [vp, u64, f32, f32],
        "vkl_model_forward": [vp, vp, sz, sz, vp],
        "vkl_model_generate": [vp, vp, sz, sz, vp, C.POINTER(f32), C.POINTER(f32)],
        "vkl_model_last_token": [vp, C.POINTER(u32)], "vkl_model_read_kv": [vp, u32, vp, vp], "vkl_model_write_kv": [vp, u32, vp, vp],
        "vkl_model_block_forward": [vp, u32, vp, sz, sz, vp],
        "vkl_model_decode_profile": [vp, u32, sz, C.POINTER(f32)],
        "vkl_model_decode_trace": [vp, u32, sz, vp, sz, C.POINTER(u32), C.POINTER(u32), vp],
        "vkl_model_tp_buffer": [vp, pvp, C.POINTER(sz)], "vkl_model_tp_connect": [vp, pvp, i32],
        "vkl_model_set_wait_limit": [vp, u32],
        "vkl_ipc_export": [vp, C.c_char_p], "vkl_ipc_open": [vp, C.c_char_p, pvp],
        "vkl_model_topk": [vp, u32, vp, vp],
        "vkl_gguf_open": [C.c_char_p, pvp], "vkl_gguf_close": [vp],
        "vkl_gguf_counts": [vp, C.POINTER(u32), C.POINTER(sz), C.POINTER(sz)],
        "vkl_gguf_get_u32": [vp, C.c_char_p, C.POINTER(u32)], "vkl_gguf_get_f32": [vp, C.c_char_p, C.POINTER(f32)],
        "vkl_gguf_get_string": [vp, C.c_char_p, C.c_char_p, sz],
        "vkl_gguf_tensor": [vp, sz, C.c_char_p, C.c_char_p, sz, C.POINTER(u32), C.POINTER(u64), C.POINTER(u32), pvp, C.POINTER(sz)],
        "vkl_model_load_gguf": [vp, vp, u32, i32, i32, pvp],
        "vkl_sampler_create": [i32, sz, f32, u64, pvp], "vkl_sampler_destroy": [vp],
        "vkl_sampler_sample": [vp, vp, sz, C.POINTER(i32)],
        "vkl_sampler_sample_candidates": [vp, vp, vp, sz, C.POINTER(i32)],
    }
    for name, args in sigs.items():
        f = getattr(L, name)
        f.restype = i32
        f.argtypes = args
    _lib = L
    return L


def _ck(status):
    if status != 0:
        raise VklError(status, load_library().vkl_last_error().decode("utf-8", "replace"))


def kernel_launches():
    return int(load_library().vkl_kernel_launches())


def _ptr(a):
    return a.ctypes.data_as(vp)


# ---- host quantizer ---------------------------------------------------------
def q8_0_quantize(x):
    x = np.ascontiguousarray(x, np.float32)
    h, w = x.shape
    out = np.empty(h * ((w + 31) // 32) * 34, np.uint8)
    _ck(load_library().vkl_q8_0_quantize(_ptr(x), _ptr(out), h, w))
    return out


def q8_0_quantize36(x):
    x = np.ascontiguousarray(x, np.float32)
    h, w = x.shape
    out = np.empty(h * ((w + 31) // 32) * 36, np.uint8)
    _ck(load_library().vkl_q8_0_quantize36(_ptr(x), _ptr(out), h, w))
    return out


def q8_0_dequantize(blocks34, h, w):
    b = np.ascontiguousarray(blocks34, np.uint8)
    out = np.empty((h, w), np.float32)
    _ck(load_library().vkl_q8_0_dequantize(_ptr(b), _ptr(out), h, w))
    return out


def blocks36_to_34(blocks36):
    b = np.ascontiguousarray(blocks36, np.uint8)
    n = b.size // 36
    out = np.empty(n * 34, np.uint8)
    _ck(load_library().vkl_q8_0_blocks36_to_34(_ptr(b), _ptr(out), n))
    return out


# ---- core -------------------------------------------------------------------
class Device:
    """GPUDevice (src/core/gpu_device.h)."""

    def __init__(self, dev=0):
        self.L = load_library()
        self.h = vp()
        _ck(self.L.vkl_device_create(dev, C.byref(self.h)))

    def info(self):
        name = C.create_string_buffer(256)
        sms, mem = i32(), sz()
        _ck(self.L.vkl_device_info(self.h, name, C.byref(sms), C.byref(mem)))
        return name.value.decode(), sms.value, mem.value

    def pool_bytes(self):
        """Released device memory currently kept for reuse."""
        n = sz()
        _ck(self.L.vkl_device_pool_bytes(self.h, C.byref(n)))
        return n.value

    def close(self):
        if self.h:
            self.L.vkl_device_destroy(self.h)
            self.h = None


class Tensor:
    """Tensor (src/core/tensor.h): a reference-counted handle."""

    def __init__(self, c=0, h=0, w=0, dev=None, dtype=FP32, _handle=None, _borrowed=False):
        self.L = load_library()
        self.dev = dev
        if _handle is not None:
            self.h = _handle
            if _borrowed:
                _ck(self.L.vkl_tensor_retain(self.h))
        else:
            self.h = vp()
            _ck(self.L.vkl_tensor_create(dev.h, c, h, w, dtype, C.byref(self.h)))

    def create(self):  # allocation happens in the constructor; kept for API parity
        return self

    def shape_constant(self):
        o = (u32 * 6)()
        _ck(self.L.vkl_tensor_shape(self.h, o))
        return tuple(o)

    def shape(self):
        return self.shape_constant()[:3]

    def channels(self):
        return self.shape_constant()[0]

    def height(self):
        return self.shape_constant()[1]

    def width(self):
        return self.shape_constant()[2]

    def dtype(self):
        d = i32()
        _ck(self.L.vkl_tensor_dtype(self.h, C.byref(d)))
        return d.value

    def bytes(self):
        b = sz()
        _ck(self.L.vkl_tensor_bytes(self.h, C.byref(b)))
        return b.value

    def view(self, c, h, w):
        out = vp()
        _ck(self.L.vkl_tensor_view(self.h, c, h, w, C.byref(out)))
        return Tensor(dev=self.dev, _handle=out)

    def reshape(self, c, h, w):
        _ck(self.L.vkl_tensor_reshape(self.h, c, h, w))
        return self

    def device_ptr(self):
        p = vp()
        _ck(self.L.vkl_tensor_device_ptr(self.h, C.byref(p)))
        return p.value

    def __del__(self):
        try:
            if self.h:
                self.L.vkl_tensor_release(self.h)
                self.h = None
        except Exception:
            pass


class Command:
    """Command (src/core/command.h): begin / ops / end / submit / wait."""

    def __init__(self, dev):
        self.L = load_library()
        self.dev = dev
        self.h = vp()
        self._keep = []
        _ck(self.L.vkl_command_create(dev.h, C.byref(self.h)))

    def init(self):
        return self

    def begin(self):
        _ck(self.L.vkl_command_begin(self.h))

    def end(self):
        _ck(self.L.vkl_command_end(self.h))

    def submit(self):
        _ck(self.L.vkl_command_submit(self.h))

    def wait(self):
        _ck(self.L.vkl_command_wait(self.h))
        self._keep.clear()

    def submit_and_wait(self):
        _ck(self.L.vkl_command_submit_and_wait(self.h))
        self._keep.clear()

    def elapsed_us(self):
        t = f32()
        _ck(self.L.vkl_command_elapsed_us(self.h, C.byref(t)))
        return t.value

    def stream(self):
        """The command's cudaStream_t as an integer."""
        s = vp()
        _ck(self.L.vkl_command_stream(self.h, C.byref(s)))
        return s.value

    def upload(self, arr, tensor):
        a = np.ascontiguousarray(arr)
        self._keep.append(a)
        _ck(self.L.vkl_command_upload(self.h, _ptr(a), a.nbytes, tensor.h))

    def download(self, tensor, out=None):
        """Returns a numpy array that is filled when wait() returns."""
        if out is None:
            dt = tensor.dtype()
            if dt == Q8_0:
                out = np.empty(tensor.bytes(), np.uint8)
            else:
                out = np.empty(tensor.shape(), _NP[dt])
        self._keep.append(out)
        _ck(self.L.vkl_command_download(self.h, tensor.h, _ptr(out), out.nbytes))
        return out

    def fill_synthetic(self, tensor, seed, tensor_id, mean, std):
        _ck(self.L.vkl_tensor_fill_synthetic(self.h, tensor.h, seed, tensor_id, mean, std))

    def q8_0_quantize(self, src_fp32, dst_q8):
        _ck(self.L.vkl_q8_0_quantize_device(self.h, src_fp32.h, dst_q8.h))

    def close(self):
        if self.h:
            self.L.vkl_command_destroy(self.h)
            self.h = None

    def __enter__(self):
        self.begin()
        return self

    def __exit__(self, et, ev, tb):
        if et is None:
            self.end()
            self.submit_and_wait()
        else:
            try:
                self.end()
                self.submit_and_wait()
            except VklError:
                pass
        return False


# ---- ops --------------------------------------------------------------------
class Op:
    """class Op (src/ops/op.h:14-25)."""

    def __init__(self, dev, command):
        self.L = load_library()
        self.dev, self.command = dev, command
        self.h = vp()

    def init(self):
        _ck(self.L.vkl_op_init(self.h))
        return self

    def time(self):
        t = u64()
        _ck(self.L.vkl_op_time(self.h, C.byref(t)))
        return t.value

    def _out(self, handle):
        return Tensor(dev=self.dev, _handle=handle, _borrowed=True)

    def __del__(self):
        try:
            if self.h:
                self.L.vkl_op_destroy(self.h)
                self.h = None
        except Exception:
            pass


def _h(t):
    return t.h if t is not None else None


class MatMul(Op):
    def __init__(self, dev, command, weight=None, scale=1.0, bias=0.0, act=0, broadcast_type=0,
                 transpose_b=False, a_dtype=FP16, b_dtype=FP16):
        super().__init__(dev, command)
        self.weight = weight
        _ck(self.L.vkl_matmul_create(dev.h, command.h, _h(weight), scale, bias, act, broadcast_type,
                                     int(transpose_b), a_dtype, b_dtype, C.byref(self.h)))

    def __call__(self, a, b=None):
        out = vp()
        _ck(self.L.vkl_matmul_run(self.h, a.h, _h(b), C.byref(out)))
        return self._out(out)


def matmul_run_many(ops, a, reps, timed=False):
    """Benchmark helper: `reps` weight-form MatMul calls on `a`, rotating over `ops`. With
    `timed` the calls run as one CUDA graph and the mean device time per call (us) is returned."""
    arr = (vp * len(ops))(*[o.h for o in ops])
    us = f32(0.0)
    _ck(load_library().vkl_matmul_run_many(arr, len(ops), a.h, reps, C.byref(us) if timed else None))
    return us.value if timed else None


class FeedForward(Op):
    def __init__(self, dev, command, w1, w2, w3, transposed_weight=False, dtype=FP16):
        super().__init__(dev, command)
        self.w = (w1, w2, w3)
        _ck(self.L.vkl_feed_forward_create(dev.h, command.h, _h(w1), _h(w2), _h(w3), int(transposed_weight), dtype,
                                           C.byref(self.h)))

    def __call__(self, x):
        out = vp()
        _ck(self.L.vkl_feed_forward_run(self.h, x.h, C.byref(out)))
        return self._out(out)


class MultiHeadAttentionV2(Op):
    def __init__(self, dev, command, wk, wq, wv, wo, maxlen, dim, transposed_weight=False, dtype=FP16,
                 use_kvcache=False, clip_output=False):
        super().__init__(dev, command)
        self.w = (wk, wq, wv, wo)
        _ck(self.L.vkl_mha_create(dev.h, command.h, _h(wk), _h(wq), _h(wv), _h(wo), maxlen, dim,
                                  int(transposed_weight), dtype, int(use_kvcache), int(clip_output), C.byref(self.h)))

    def __call__(self, x, offset=0):
        out = vp()
        _ck(self.L.vkl_mha_run(self.h, x.h, offset, C.byref(out)))
        return self._out(out)

    def caches(self):
        k, v = vp(), vp()
        _ck(self.L.vkl_mha_caches(self.h, C.byref(k), C.byref(v)))
        return self._out(k), self._out(v)


class UpdateKVCache(Op):
    def __init__(self, dev, command, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_update_kvcache_create(dev.h, command.h, dtype, C.byref(self.h)))

    def __call__(self, cache, kv, offset):
        _ck(self.L.vkl_update_kvcache_run(self.h, cache.h, kv.h, offset))


class RMSNorm(Op):
    def __init__(self, dev, command, weight, eps=1e-3, dtype=FP16):
        super().__init__(dev, command)
        self.weight = weight
        _ck(self.L.vkl_rms_norm_create(dev.h, command.h, _h(weight), eps, dtype, C.byref(self.h)))

    def __call__(self, x):
        out = vp()
        _ck(self.L.vkl_rms_norm_run(self.h, x.h, C.byref(out)))
        return self._out(out)


class Rope(Op):
    def __init__(self, dev, command, maxlen, dim, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_rope_create(dev.h, command.h, maxlen, dim, dtype, C.byref(self.h)))

    def __call__(self, q, offset=0):
        out = vp()
        _ck(self.L.vkl_rope_run(self.h, q.h, offset, C.byref(out)))
        return self._out(out)


class Softmax(Op):
    def __init__(self, dev, command, seq_mask=False, temp=1.0, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_softmax_create(dev.h, command.h, int(seq_mask), temp, dtype, C.byref(self.h)))

    def __call__(self, a, offset=0):
        out = vp()
        _ck(self.L.vkl_softmax_run(self.h, a.h, offset, C.byref(out)))
        return self._out(out)


class ArgOp(Op):
    def __init__(self, dev, command, op_type=0, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_argop_create(dev.h, command.h, op_type, dtype, C.byref(self.h)))

    def __call__(self, x):
        out = vp()
        _ck(self.L.vkl_argop_run(self.h, x.h, C.byref(out)))
        return self._out(out)


class ArgMax(ArgOp):
    def __init__(self, dev, command, dtype=FP16):
        super().__init__(dev, command, 0, dtype)


class ArgMin(ArgOp):
    def __init__(self, dev, command, dtype=FP16):
        super().__init__(dev, command, 1, dtype)


class Embedding(Op):
    def __init__(self, dev, command, vocab, UNK, dtype=FP16):
        super().__init__(dev, command)
        self.vocab = vocab
        _ck(self.L.vkl_embedding_create(dev.h, command.h, _h(vocab), UNK, dtype, C.byref(self.h)))

    def __call__(self, indices):
        out = vp()
        _ck(self.L.vkl_embedding_run(self.h, indices.h, C.byref(out)))
        return self._out(out)


class ElementWise(Op):
    def __init__(self, dev, command, type=0, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_elementwise_create(dev.h, command.h, type, dtype, C.byref(self.h)))

    def __call__(self, x, y):
        out = vp()
        if isinstance(y, (int, float)):  # ElementWise::operator()(Tensor, float): in place in x
            _ck(self.L.vkl_elementwise_run_scalar(self.h, x.h, f32(float(y)), C.byref(out)))
        else:
            _ck(self.L.vkl_elementwise_run(self.h, x.h, y.h, C.byref(out)))
        return self._out(out)


class Concat(Op):
    """Concat(dev, command, num, axis, dtype) (src/ops/concat.h:10-17)."""

    def __init__(self, dev, command, num, axis, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_concat_create(dev.h, command.h, num, axis, dtype, C.byref(self.h)))

    def __call__(self, inputs):
        arr = (vp * len(inputs))(*[t.h for t in inputs])
        out = vp()
        _ck(self.L.vkl_concat_run(self.h, arr, len(inputs), C.byref(out)))
        return self._out(out)


class Reduce(Op):
    """Reduce(dev, command, op_type, dtype): 0 sum, 1 max, 2 min, 3 mean (src/ops/reduce.h:18-67)."""

    def __init__(self, dev, command, op_type, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_reduce_create(dev.h, command.h, op_type, dtype, C.byref(self.h)))

    def __call__(self, a):
        out = vp()
        _ck(self.L.vkl_reduce_run(self.h, a.h, C.byref(out)))
        return self._out(out)


class ReadKVCache(Op):
    """ReadKVCache(dev, command) (src/ops/read_kvcache_op.h:10-16)."""

    def __init__(self, dev, command):
        super().__init__(dev, command)
        _ck(self.L.vkl_read_kvcache_create(dev.h, command.h, C.byref(self.h)))

    def __call__(self, cache, offset, length):
        out = vp()
        _ck(self.L.vkl_read_kvcache_run(self.h, cache.h, offset, length, C.byref(out)))
        return self._out(out)


class Transpose(Op):
    def __init__(self, dev, command, type=0, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_transpose_create(dev.h, command.h, type, dtype, C.byref(self.h)))

    def __call__(self, x):
        out = vp()
        _ck(self.L.vkl_transpose_run(self.h, x.h, C.byref(out)))
        return self._out(out)


class Slice(Op):
    def __init__(self, dev, command, dtype=FP16):
        super().__init__(dev, command)
        _ck(self.L.vkl_slice_create(dev.h, command.h, dtype, C.byref(self.h)))

    def __call__(self, x, starts, extents):
        out = vp()
        _ck(self.L.vkl_slice_run(self.h, x.h, (u32 * 3)(*starts), (u32 * 3)(*extents), C.byref(out)))
        return self._out(out)


class Cast(Op):
    def __init__(self, dev, command, from_dtype, to_dtype):
        super().__init__(dev, command)
        _ck(self.L.vkl_cast_create(dev.h, command.h, from_dtype, to_dtype, C.byref(self.h)))

    def __call__(self, x):
        out = vp()
        _ck(self.L.vkl_cast_run(self.h, x.h, C.byref(out)))
        return self._out(out)


# ---- model ------------------------------------------------------------------
LAYER_TENSORS = ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate",
                 "ffn_up", "ffn_down")


class Model:
    """vkllama::Model (models/llama2.h:322-854)."""

    def __init__(self, dev, dim, heads, ffn, vocab, layers, maxlen, eps=1e-5, final_eps=1e-6,
                 weight_dtype=Q8_0, tp_rank=0, tp_size=1):
        self.L = load_library()
        self.dev = dev
        self.cfg = ModelConfig(dim, heads, ffn, vocab, layers, maxlen, eps, final_eps, weight_dtype,
                               tp_rank, tp_size)
        self.h = vp()
        _ck(self.L.vkl_model_create(dev.h, C.byref(self.cfg), C.byref(self.h)))

    @classmethod
    def from_gguf(cls, dev, gguf, maxlen=0, tp_rank=0, tp_size=1):
        """Model::init from an open GGUF file (models/llama2.h:348-681)."""
        self = cls.__new__(cls)
        self.L = load_library()
        self.dev = dev
        self.h = vp()
        _ck(self.L.vkl_model_load_gguf(dev.h, gguf.h, maxlen, tp_rank, tp_size, C.byref(self.h)))
        heads, layers, eps, ctx = gguf.u32("llama.attention.head_count"), gguf.u32("llama.block_count"), \
            gguf.f32("llama.attention.layer_norm_rms_epsilon"), gguf.u32("llama.context_length")
        emb, outw = gguf.tensor("token_embd.weight"), gguf.tensor("output.weight")
        ffn = gguf.tensor("blk.0.ffn_gate.weight")["dims"][1] if layers else emb["dims"][0]
        self.cfg = ModelConfig(emb["dims"][0], heads, ffn, emb["dims"][1], layers, min(maxlen, ctx) if maxlen else ctx, eps, 1e-6,
                               {0: FP32, 1: FP16, 8: Q8_0}[outw["type"]], tp_rank, max(1, tp_size))
        return self

    def topk(self, k):
        """The k largest logits of the last step and their ids, selected on the device."""
        vals, ids = np.empty(k, np.float32), np.empty(k, np.uint32)
        _ck(self.L.vkl_model_topk(self.h, k, _ptr(vals), _ptr(ids)))
        return vals, ids

    def set_weight(self, name, dtype, data):
        a = np.ascontiguousarray(data)
        _ck(self.L.vkl_model_set_weight(self.h, name.encode(), dtype, _ptr(a), a.nbytes))

    def synth_weights(self, seed, wstd=0.02, nstd=0.01):
        _ck(self.L.vkl_model_synth_weights(self.h, seed, wstd, nstd))

    def __call__(self, toks, offset, out=None):
        """Model::operator()(toks, offset) -> fp32 logits of the last token (into `out` when given: a loop that
        reuses its buffer spares the allocator a 128 KB mapping per token)."""
        t = np.ascontiguousarray(toks, np.uint32)
        n = self.cfg.vocab // max(1, self.cfg.tp_size)
        if out is None:
            out = np.empty(n, np.float32)
        elif out.dtype != np.float32 or out.size != n or not out.flags.c_contiguous:
            raise ValueError("out must be a contiguous float32 array of %d elements" % n)
        _ck(self.L.vkl_model_forward(self.h, _ptr(t), t.size, offset, _ptr(out)))
        return out

    forward = __call__

    def generate(self, prompt, n_gen):
        p = np.ascontiguousarray(prompt, np.uint32)
        ids = np.empty(n_gen, np.uint32)
        pre, dec = f32(), f32()
        _ck(self.L.vkl_model_generate(self.h, _ptr(p), p.size, n_gen, _ptr(ids), C.byref(pre), C.byref(dec)))
        return ids, pre.value, dec.value

    def last_token(self):
        t = u32()
        _ck(self.L.vkl_model_last_token(self.h, C.byref(t)))
        return t.value

    def kv_shape(self):
        c = self.cfg
        return (c.heads // max(1, c.tp_size), c.maxlen, c.dim // c.heads)

    def read_kv(self, layer):
        k = np.empty(self.kv_shape(), np.uint16)
        v = np.empty(self.kv_shape(), np.uint16)
        _ck(self.L.vkl_model_read_kv(self.h, layer, _ptr(k), _ptr(v)))
        return k, v

    def write_kv(self, layer, k, v):
        k = np.ascontiguousarray(k, np.uint16)
        v = np.ascontiguousarray(v, np.uint16)
        _ck(self.L.vkl_model_write_kv(self.h, layer, _ptr(k), _ptr(v)))

    def block_forward(self, layer, x, offset):
        x = np.ascontiguousarray(x, np.uint16)
        T = x.size // self.cfg.dim
        out = np.empty((T, self.cfg.dim), np.uint16)
        _ck(self.L.vkl_model_block_forward(self.h, layer, _ptr(x), T, offset, _ptr(out)))
        return out

    def decode_profile(self, token, offset):
        """Per-kernel-class device microseconds of one decode step (see the header)."""
        out = (f32 * 20)()
        _ck(self.L.vkl_model_decode_profile(self.h, token, offset, out))
        return list(out)

    def decode_trace(self, token, offset):
        """(stamps [nops, grid, 8] in ns, kinds [nops]) of one traced decode step (see the header)."""
        nops, grid = u32(), u32()
        _ck(self.L.vkl_model_decode_trace(self.h, token, offset, None, 0, C.byref(nops), C.byref(grid), None))
        out = np.zeros((nops.value, grid.value, 8), np.uint64)
        kinds = np.zeros(nops.value, np.uint32)
        _ck(self.L.vkl_model_decode_trace(self.h, token, offset, _ptr(out), out.size, C.byref(nops), C.byref(grid), _ptr(kinds)))
        return out, kinds

    def set_wait_limit(self, polls):
        """Bound of every wait inside the decode kernel, in polls (0 = default)."""
        _ck(self.L.vkl_model_set_wait_limit(self.h, polls))

    def tp_buffer(self):
        """(device pointer, bytes) of this rank's exchange buffer."""
        p, n = vp(), sz()
        _ck(self.L.vkl_model_tp_buffer(self.h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def tp_connect_pointers(self, ptrs):
        """Connect with already mapped peer pointers, indexed by rank (own entry ignored)."""
        arr = (vp * len(ptrs))(*[vp(x) for x in ptrs])
        _ck(self.L.vkl_model_tp_connect(self.h, arr, len(ptrs)))

    def tp_export(self):
        """CUDA IPC handle (64 bytes) of this rank's exchange buffer."""
        p, n = vp(), sz()
        _ck(self.L.vkl_model_tp_buffer(self.h, C.byref(p), C.byref(n)))
        h = C.create_string_buffer(64)
        _ck(self.L.vkl_ipc_export(p, h))
        return h.raw

    def tp_connect(self, handles):
        """handles[r] = IPC handle of rank r's exchange buffer (own entry ignored)."""
        ptrs = (vp * len(handles))()
        opened = self.__dict__.setdefault("_tp_opened", {})  # a handle is mapped once; reconnecting reuses the mapping
        for r, hb in enumerate(handles):
            if r == self.cfg.tp_rank:
                continue
            if hb not in opened:
                q = vp()
                _ck(self.L.vkl_ipc_open(self.dev.h, C.create_string_buffer(hb, 64), C.byref(q)))
                opened[hb] = q.value
            ptrs[r] = opened[hb]
        _ck(self.L.vkl_model_tp_connect(self.h, ptrs, len(handles)))

    def close(self):
        if self.h:
            self.L.vkl_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- checkpoint container and samplers ---------------------------------------------------
class Gguf:
    """Read-only GGUF file as the reference's app opens it (app/llama2_infer.cpp:46-73)."""

    def __init__(self, path):
        self.L = load_library()
        self.h = vp()
        _ck(self.L.vkl_gguf_open(os.fsencode(path), C.byref(self.h)))

    def counts(self):
        v, nk, nt = u32(), sz(), sz()
        _ck(self.L.vkl_gguf_counts(self.h, C.byref(v), C.byref(nk), C.byref(nt)))
        return v.value, nk.value, nt.value

    def u32(self, key):
        v = u32()
        _ck(self.L.vkl_gguf_get_u32(self.h, key.encode(), C.byref(v)))
        return v.value

    def f32(self, key):
        v = f32()
        _ck(self.L.vkl_gguf_get_f32(self.h, key.encode(), C.byref(v)))
        return v.value

    def string(self, key, cap=4096):
        b = C.create_string_buffer(cap)
        _ck(self.L.vkl_gguf_get_string(self.h, key.encode(), b, cap))
        return b.value.decode("utf-8", "replace")

    def tensor(self, name_or_index):
        """dict(name, dims (row length first, as in GGUF), type (GGML id), data (uint8 view of the mapping))."""
        nm = C.create_string_buffer(512)
        nd, dims, ty, data, nb = u32(), (u64 * 4)(), u32(), vp(), sz()
        byname = isinstance(name_or_index, str)
        _ck(self.L.vkl_gguf_tensor(self.h, 0 if byname else name_or_index, name_or_index.encode() if byname else None, nm, 512,
                                   C.byref(nd), dims, C.byref(ty), C.byref(data), C.byref(nb)))
        arr = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nb.value,)) if nb.value else np.empty(0, np.uint8)
        return {"name": nm.value.decode(), "dims": [int(dims[i]) for i in range(nd.value)], "type": ty.value, "data": arr}

    def close(self):
        if self.h:
            self.L.vkl_gguf_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Sampler:
    def __init__(self, kind, topk, topp, seed):
        self.L = load_library()
        self.h = vp()
        _ck(self.L.vkl_sampler_create(kind, topk, topp, seed, C.byref(self.h)))

    def sample(self, logits):
        a = np.ascontiguousarray(logits, np.float32)
        out = i32()
        _ck(self.L.vkl_sampler_sample(self.h, _ptr(a), a.size, C.byref(out)))
        return out.value

    def sample_candidates(self, values, ids):
        v, i = np.ascontiguousarray(values, np.float32), np.ascontiguousarray(ids, np.uint32)
        out = i32()
        _ck(self.L.vkl_sampler_sample_candidates(self.h, _ptr(v), _ptr(i), v.size, C.byref(out)))
        return out.value

    def close(self):
        if self.h:
            self.L.vkl_sampler_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TopkSampler(Sampler):
    """TopkSampler(topk = 40) (models/samplers.h:27-35)."""

    def __init__(self, topk=40, seed=0):
        super().__init__(0, topk, 1.0, seed)


class TopPSampler(Sampler):
    """TopPSampler(p) (models/samplers.h:37-45)."""

    def __init__(self, p, seed=0):
        super().__init__(1, 0, p, seed)
