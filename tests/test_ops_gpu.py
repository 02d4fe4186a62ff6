"""Per-op parity of the CUDA ops (through the C ABI) against the CPU oracle, at
the reference's own test shapes (tests/test_*.cpp of vkllama) and at the
Llama-2-7B shapes. Tolerance: max |a-b| / max |b| <= 1e-2 on fp16 outputs;
Q8_0 codes and scales, indices and copies are compared bit for bit."""
import numpy as np
import pytest

from oracle import oracle as O
import vkllama_b200 as vk
from util import assert_close, up

pytestmark = pytest.mark.gpu


def run(cmd, fn):
    cmd.begin()
    res = fn()
    cmd.end()
    cmd.submit_and_wait()
    return res


# ---- Q8_0 layout / quantizer ------------------------------------------------
@pytest.mark.parametrize("N,K", [(1, 32), (17, 256), (16, 95), (33, 4096), (4096, 4096)])
def test_q8_0_upload_download_round_trip_is_bit_exact(dev, N, K):
    w = O.synth_q8_0(3, 7, N, K)
    cmd = vk.Command(dev)
    cmd.begin()
    t = up(cmd, dev, w, vk.Q8_0, 1, N, K)
    back = cmd.download(t)
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(back, w)


@pytest.mark.parametrize("N,K", [(3, 95), (64, 4096), (8, 11008)])
def test_device_quantizer_is_bit_exact_with_reference_quantizer(dev, N, K):
    x = O.synth_f32(21, 4, N * K, 0.0, 0.02).reshape(N, K)
    want = O.quantize34(x)  # pinned to the reference's quants.h by the CPU tests
    cmd = vk.Command(dev)
    cmd.begin()
    src = up(cmd, dev, x, vk.FP32, 1, N, K)
    dst = vk.Tensor(1, N, K, dev, vk.Q8_0)
    cmd.q8_0_quantize(src, dst)
    got = cmd.download(dst)
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(got, want)


def test_device_synthetic_generator_matches_host_generator(dev):
    cmd = vk.Command(dev)
    cmd.begin()
    a = vk.Tensor(1, 7, 333, dev, vk.FP32)
    b = vk.Tensor(1, 5, 96, dev, vk.FP16)
    c = vk.Tensor(1, 48, 4096, dev, vk.Q8_0)
    cmd.fill_synthetic(a, 5, 1, 1.0, 0.01)
    cmd.fill_synthetic(b, 5, 2, 0.0, 1.0)
    cmd.fill_synthetic(c, 5, 3, 0.0, 0.02)
    ga, gb, gc = cmd.download(a), cmd.download(b), cmd.download(c)
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(ga.ravel(), O.synth_f32(5, 1, 7 * 333, 1.0, 0.01))
    assert np.array_equal(gb.ravel(), O.synth_f16(5, 2, 5 * 96, 0.0, 1.0))
    assert np.array_equal(gc, O.synth_q8_0(5, 3, 48, 4096, 0.0, 0.02))


# ---- MatMul with a Q8_0 weight (tests/test_matmul.cpp Q8_0 cases; 7B shapes) --
@pytest.mark.parametrize("M,N,K,act", [
    (1, 4096, 4096, 0), (1, 11008, 4096, 0), (1, 4096, 11008, 0), (1, 32000, 4096, 0),
    (2, 4096, 4096, 0), (8, 4096, 4096, 1), (9, 17, 256, 0), (16, 4096, 4096, 0), (33, 1000, 4096, 0),
    (64, 4096, 4096, 0), (100, 256, 11008, 0), (5, 16, 32, 0), (3, 50, 96, 1),
    # from 64 rows on: the tcgen05 GEMM with the dequantising warps, every tile width (32 / 64 / 128 / 256 columns by
    # rows and matrix size), several row tiles, a ragged last column tile, one and two K steps
    (512, 1024, 4096, 0), (512, 11008, 256, 0), (200, 352, 1024, 1), (128, 11008, 128, 0), (64, 40, 64, 0), (130, 2048, 2048, 0)])
def test_matmul_q8_0(dev, M, N, K, act):
    w = O.synth_q8_0(31, 1, N, K)
    x = O.synth_f16(31, 2, M * K).reshape(M, K)
    want = O.matmul_q8_0(x, w, M, N, K, 1.0, 0.0, act)
    cmd = vk.Command(dev)
    cmd.begin()
    tw = up(cmd, dev, w, vk.Q8_0, 1, N, K)
    tx = up(cmd, dev, x, vk.FP16, 1, M, K)
    op = vk.MatMul(dev, cmd, tw, 1.0, 0.0, act, 0, True, vk.FP16, vk.Q8_0).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert got.shape == (1, M, N)
    assert_close(got, want, what="matmul_q8_0 %s" % ((M, N, K),))
    assert op.time() >= 0


def test_matmul_q8_0_k_not_multiple_of_32(dev):
    M, N, K = 3, 20, 95  # tail block padded with zero codes (quants.h:79-84)
    xf = O.synth_f32(8, 1, N * K, 0.0, 0.02).reshape(N, K)
    w = O.quantize34(xf)
    x = O.synth_f16(8, 2, M * K).reshape(M, K)
    want = O.matmul_q8_0(x, w, M, N, K)
    cmd = vk.Command(dev)
    cmd.begin()
    tw = up(cmd, dev, w, vk.Q8_0, 1, N, K)
    tx = up(cmd, dev, x, vk.FP16, 1, M, K)
    op = vk.MatMul(dev, cmd, tw, 1.0, 0.0, 0, 0, True, vk.FP16, vk.Q8_0).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="matmul_q8_0 ragged K")


# ---- MatMul fp16 x fp16 (tests/test_matmul.cpp:191: C1 M9 N9 K128, transpose_b) --
@pytest.mark.parametrize("C,M,N,K,tb", [(1, 9, 9, 128, True), (32, 1, 512, 128, True), (32, 1, 128, 512, False),
                                          (3, 5, 7, 100, False), (2, 4, 6, 70, True)])
def test_matmul_fp16_pair(dev, C, M, N, K, tb):
    a = O.synth_f16(41, 1, C * M * K).reshape(C, M, K)
    bshape = (C, N, K) if tb else (C, K, N)
    b = O.synth_f16(41, 2, C * N * K).reshape(bshape)
    want = np.empty(C * M * N, np.uint16)
    f = O.lib().orc_matmul_tb_f16 if tb else O.lib().orc_matmul_nn_f16
    f(a, b, want, C, M, N, K, M * K, K, N * K, K if tb else N, M * N, N, 0.5, 0.0, 0)
    cmd = vk.Command(dev)
    cmd.begin()
    ta = up(cmd, dev, a, vk.FP16, C, M, K)
    tb_ = up(cmd, dev, b, vk.FP16, *bshape)
    op = vk.MatMul(dev, cmd, None, 0.5, 0.0, 0, 0, tb, vk.FP16, vk.FP16).init()
    got = cmd.download(op(ta, tb_))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="matmul fp16")


def test_matmul_fp16_weight(dev):
    M, N, K = 3, 100, 256
    a = O.synth_f16(42, 1, M * K).reshape(1, M, K)
    w = O.synth_f16(42, 2, N * K, 0.0, 0.02).reshape(1, N, K)
    want = np.empty(M * N, np.uint16)
    O.lib().orc_matmul_tb_f16(a, w, want, 1, M, N, K, M * K, K, N * K, K, M * N, N, 1.0, 0.0, 0)
    cmd = vk.Command(dev)
    cmd.begin()
    ta = up(cmd, dev, a, vk.FP16, 1, M, K)
    tw = up(cmd, dev, w, vk.FP16, 1, N, K)
    op = vk.MatMul(dev, cmd, tw, 1.0, 0.0, 0, 0, True, vk.FP16, vk.FP16).init()
    got = cmd.download(op(ta))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="matmul fp16 weight")


# Many rows with FP16 weights run on the tcgen05 tensor-core GEMM (one pass over the weights);
# ragged M and N exercise the zero-filled tile edges, act/scale/bias the epilogue.
@pytest.mark.parametrize("M,N,K,scale,bias,act", [(32, 128, 64, 1.0, 0.0, 0), (128, 128, 128, 1.0, 0.0, 0),
                                                    (100, 136, 256, 0.5, 0.25, 1), (300, 344, 4096, 1.0, 0.0, 0),
                                                    (512, 4096, 4096, 1.0, 0.0, 0), (129, 11008, 4096, 1.0, 0.0, 0)])
def test_matmul_fp16_weight_many_rows(dev, M, N, K, scale, bias, act):
    a = O.synth_f16(43, 1, M * K).reshape(1, M, K)
    w = O.synth_f16(43, 2, N * K, 0.0, 0.02).reshape(1, N, K)
    want = np.empty(M * N, np.uint16)
    O.lib().orc_matmul_tb_f16(a, w, want, 1, M, N, K, M * K, K, N * K, K, M * N, N, scale, bias, act)
    cmd = vk.Command(dev)
    cmd.begin()
    ta = up(cmd, dev, a, vk.FP16, 1, M, K)
    tw = up(cmd, dev, w, vk.FP16, 1, N, K)
    op = vk.MatMul(dev, cmd, tw, scale, bias, act, 0, True, vk.FP16, vk.FP16).init()
    got = cmd.download(op(ta))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="matmul fp16 weight (tensor-core GEMM)")


@pytest.mark.parametrize("M,dim,hidden", [(5, 64, 96), (64, 128, 256), (100, 4096, 11008)])
def test_feed_forward_fp16(dev, M, dim, hidden):
    gate = O.synth_f16(52, 1, hidden * dim, 0.0, 0.02)
    down = O.synth_f16(52, 2, dim * hidden, 0.0, 0.02)
    upw = O.synth_f16(52, 3, hidden * dim, 0.0, 0.02)
    x = O.synth_f16(52, 4, M * dim).reshape(M, dim)
    want = np.empty(M * dim, np.uint16)
    O.lib().orc_feed_forward_f16(x, gate, down, upw, want, M, dim, hidden)
    cmd = vk.Command(dev)
    cmd.begin()
    w1 = up(cmd, dev, gate, vk.FP16, 1, hidden, dim)
    w2 = up(cmd, dev, down, vk.FP16, 1, dim, hidden)
    w3 = up(cmd, dev, upw, vk.FP16, 1, hidden, dim)
    tx = up(cmd, dev, x, vk.FP16, 1, M, dim)
    op = vk.FeedForward(dev, cmd, w1, w2, w3, True, vk.FP16).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="feed_forward fp16")


# ---- FeedForward (tests/test_feedforward.cpp:143-148 Q8_0: dims 16,8,256,17; 7B) --
@pytest.mark.parametrize("M,dim,hidden", [(64, 32, 256), (1, 4096, 11008), (4, 4096, 11008), (17, 64, 96), (128, 1024, 2752)])
def test_feed_forward_q8_0(dev, M, dim, hidden):
    gate = O.synth_q8_0(51, 1, hidden, dim)
    down = O.synth_q8_0(51, 2, dim, hidden)
    upw = O.synth_q8_0(51, 3, hidden, dim)
    x = O.synth_f16(51, 4, M * dim).reshape(M, dim)
    want = np.empty(M * dim, np.uint16)
    O.lib().orc_feed_forward_q8_0(x, gate, down, upw, want, M, dim, hidden)
    cmd = vk.Command(dev)
    cmd.begin()
    w1 = up(cmd, dev, gate, vk.Q8_0, 1, hidden, dim)
    w2 = up(cmd, dev, down, vk.Q8_0, 1, dim, hidden)
    w3 = up(cmd, dev, upw, vk.Q8_0, 1, hidden, dim)
    tx = up(cmd, dev, x, vk.FP16, 1, M, dim)
    op = vk.FeedForward(dev, cmd, w1, w2, w3, True, vk.Q8_0).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="feed_forward")


# ---- RMSNorm (tests/test_rmsnorm.cpp:100-105: [1,1,128]; 7B rows) -------------
@pytest.mark.parametrize("rows,W,eps", [(1, 128, 1e-3), (1, 4096, 1e-5), (33, 4096, 1e-5), (5, 100, 1e-6)])
def test_rms_norm(dev, rows, W, eps):
    x = O.synth_f16(61, 1, rows * W).reshape(rows, W)
    w = O.synth_f32(61, 2, W, 1.0, 0.01)
    want = np.empty(rows * W, np.uint16)
    O.lib().orc_rms_norm_f16(x, w, want, rows, W, eps)
    cmd = vk.Command(dev)
    cmd.begin()
    tw = up(cmd, dev, w, vk.FP32, 1, 1, W)
    tx = up(cmd, dev, x, vk.FP16, 1, rows, W)
    op = vk.RMSNorm(dev, cmd, tw, eps, vk.FP16).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, tol=2e-3, what="rms_norm")


# ---- Rope (tests/test_rope.cpp:211-217: [32,{8,25,13},100], offsets 0/100/1020) --
@pytest.mark.parametrize("C,H,W,maxlen,offset", [(32, 8, 100, 2048, 0), (32, 25, 100, 1024, 100),
                                                  (32, 13, 100, 2048, 1020), (32, 1, 128, 4096, 511)])
def test_rope(dev, C, H, W, maxlen, offset):
    x = O.synth_f16(71, 1, C * H * W).reshape(C, H, W)
    fc = np.empty(2 * maxlen * W // 2, np.float32)
    fs = np.empty_like(fc)
    O.lib().orc_rope_table(W, 2 * maxlen, fc, fs)
    want = x.copy()
    O.lib().orc_rope_f16(want, C, H, W, offset, fc, fs)
    cmd = vk.Command(dev)
    cmd.begin()
    tx = up(cmd, dev, x, vk.FP16, C, H, W)
    op = vk.Rope(dev, cmd, maxlen, W, vk.FP16).init()
    out = op(tx, offset)
    got = cmd.download(out)
    got_in_place = cmd.download(tx)
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, tol=1e-3, what="rope")
    assert np.array_equal(got, got_in_place)


# ---- Softmax (tests/test_softmax.cpp: [32,62,62], [1,1023,63], [3,1023,51]) ----
@pytest.mark.parametrize("C,H,W,mask", [(32, 62, 62, False), (1, 1023, 63, False), (3, 1023, 51, False),
                                          (32, 62, 62, True), (32, 1, 512, True), (4, 8, 40, True)])
def test_softmax(dev, C, H, W, mask):
    x = O.synth_f16(81, 1, C * H * W).reshape(C, H, W)
    off = W - H if mask else 0
    want = np.empty_like(x)
    O.lib().orc_softmax_f16(x, want, C, H, W, int(mask), off)
    cmd = vk.Command(dev)
    cmd.begin()
    tx = up(cmd, dev, x, vk.FP16, C, H, W)
    op = vk.Softmax(dev, cmd, mask, 1.0, vk.FP16).init()
    got = cmd.download(op(tx, off))
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, want, what="softmax")
    if mask:
        assert np.array_equal(got == 0, want == 0)


# ---- ArgMax / ArgMin (tests/test_argop.cpp: [1 or 3, 1023, 511]; vocab row) -----
@pytest.mark.parametrize("C,H,W", [(1, 1023, 511), (3, 1023, 511), (1, 1, 32000), (1, 2, 5)])
@pytest.mark.parametrize("op_type", [0, 1])
def test_argop(dev, C, H, W, op_type):
    x = O.synth_f16(91, 1, C * H * W).reshape(C, H, W)
    xf = O.f16(x).reshape(C * H, W)
    want = (np.argmax(xf, 1) if op_type == 0 else np.argmin(xf, 1)).astype(np.uint32)  # first index on ties
    cmd = vk.Command(dev)
    cmd.begin()
    tx = up(cmd, dev, x, vk.FP16, C, H, W)
    op = vk.ArgOp(dev, cmd, op_type, vk.FP16).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert got.shape == (C, H, 1)
    assert np.array_equal(got.ravel(), want)
    if op_type == 0:
        o = np.empty(C * H, np.uint32)
        O.lib().orc_argmax_f16(x, o, C * H, W)
        assert np.array_equal(o, want)


def test_argmax_ties_pick_lowest_index(dev):
    x = np.zeros((1, 3, 5000), np.float32)
    x[0, 0, [4000, 77, 4999]] = 2.0
    x[0, 1, :] = 1.0
    x[0, 2, [1024, 1023]] = 3.0
    cmd = vk.Command(dev)
    cmd.begin()
    tx = up(cmd, dev, O.bits(x), vk.FP16, 1, 3, 5000)
    op = vk.ArgMax(dev, cmd, vk.FP16).init()
    got = cmd.download(op(tx))
    cmd.end()
    cmd.submit_and_wait()
    assert got.ravel().tolist() == [77, 0, 1023]


# ---- Embedding (tests/test_embedding.cpp: ids [55x19],[123x128], vocab 20000x64) --
@pytest.mark.parametrize("H,W,VH,VW,q8", [(55, 19, 20000, 64, True), (123, 128, 20000, 64, False),
                                           (1, 1, 32000, 4096, True), (1, 32, 32000, 4096, True)])
def test_embedding(dev, H, W, VH, VW, q8):
    ids = O.synth_tokens(101, 1, H * W, VH + 50)  # some ids >= VH map to UNK
    ids[0] = VH + 7
    unk = 3
    want = np.empty(H * W * VW, np.uint16)
    if q8:
        vocab = O.synth_q8_0(101, 2, VH, VW, 0.0, 1.0)
        O.lib().orc_embedding_q8_0(vocab, ids, want, H * W, VH, VW, unk)
    else:
        vocab = O.synth_f16(101, 2, VH * VW)
        O.lib().orc_embedding_f16(vocab, ids, want, H * W, VH, VW, unk)
    cmd = vk.Command(dev)
    cmd.begin()
    tv = up(cmd, dev, vocab, vk.Q8_0 if q8 else vk.FP16, 1, VH, VW)
    ti = up(cmd, dev, ids, vk.UINT32, 1, H, W)
    op = vk.Embedding(dev, cmd, tv, unk, vk.Q8_0 if q8 else vk.FP16).init()
    got = cmd.download(op(ti))
    cmd.end()
    cmd.submit_and_wait()
    assert got.shape == (H, W, VW)
    assert np.array_equal(got.ravel(), want)  # a dequantised value is one exact product, one rounding


# ---- UpdateKVCache (tests/test_update_kv_cache.cpp: heads 32, seq 25, maxlen 1024, dim 100, wrap) --
@pytest.mark.parametrize("offset", [0, 500, 1022])
def test_update_kvcache_with_wrap(dev, offset):
    C, H, W, HO = 32, 25, 100, 1024
    kv = O.synth_f16(111, 1, C * H * W).reshape(C, H, W)
    cache0 = O.synth_f16(111, 2, C * HO * W).reshape(C, HO, W)
    want = cache0.copy()
    O.lib().orc_update_kvcache_f16(want, kv, C, H, W, HO, W, offset)
    cmd = vk.Command(dev)
    cmd.begin()
    tc = up(cmd, dev, cache0, vk.FP16, C, HO, W)
    tk = up(cmd, dev, kv, vk.FP16, C, H, W)
    op = vk.UpdateKVCache(dev, cmd, vk.FP16).init()
    op(tc, tk, offset)
    got = cmd.download(tc)
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(got, want)


# ---- ElementWise add, Transpose, Slice, Cast ----------------------------------
def test_elementwise_add_writes_into_second_operand(dev):
    x = O.synth_f16(121, 1, 3 * 4096).reshape(1, 3, 4096)
    y = O.synth_f16(121, 2, 3 * 4096).reshape(1, 3, 4096)
    want = y.copy().ravel()
    O.lib().orc_add_f16(x.ravel(), want, want.size)
    cmd = vk.Command(dev)
    cmd.begin()
    tx, ty = up(cmd, dev, x, vk.FP16, 1, 3, 4096), up(cmd, dev, y, vk.FP16, 1, 3, 4096)
    op = vk.ElementWise(dev, cmd, 0, vk.FP16).init()
    out = op(tx, ty)
    got, gy = cmd.download(out), cmd.download(ty)
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(got.ravel(), want) and np.array_equal(gy.ravel(), want)


def test_transpose_slice_cast(dev):
    C, H, W = 5, 7, 33
    x = O.synth_f16(131, 1, C * H * W).reshape(C, H, W)
    cmd = vk.Command(dev)
    cmd.begin()
    tx = up(cmd, dev, x, vk.FP16, C, H, W)
    tr = vk.Transpose(dev, cmd, 0, vk.FP16).init()
    sl = vk.Slice(dev, cmd, vk.FP16).init()
    ca = vk.Cast(dev, cmd, vk.FP16, vk.FP32).init()
    cb = vk.Cast(dev, cmd, vk.FP32, vk.FP16).init()
    g_t = cmd.download(tr(tx))
    g_s = cmd.download(sl(tx, (1, 2, 3), (2, 4, 20)))
    f32 = ca(tx)
    g_c = cmd.download(f32)
    g_b = cmd.download(cb(f32))
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(g_t, x.transpose(1, 0, 2))
    assert np.array_equal(g_s, x[1:3, 2:6, 3:23])
    assert np.array_equal(g_c, O.f16(x).reshape(C, H, W))
    assert np.array_equal(g_b, x)


# ---- MultiHeadAttentionV2 (no working test in the reference; oracle = its op chain) --
@pytest.mark.parametrize("T,offset,clip", [(1, 0, False), (7, 0, False), (1, 7, False), (5, 8, False),
                                            (6, 0, True), (1, 13, True)])
def test_multiheadattention_q8_0_sequence(dev, T, offset, clip):
    heads, dim, maxlen = 4, 64, 32
    Wd = heads * dim
    ws = [O.synth_q8_0(141, i, Wd, Wd, 0.0, 0.05) for i in range(4)]  # wk, wq, wv, wo
    att = O.lib().orc_attn_create(heads, dim, maxlen)
    cmd = vk.Command(dev)
    cmd.begin()
    tw = [up(cmd, dev, w, vk.Q8_0, 1, Wd, Wd) for w in ws]
    op = vk.MultiHeadAttentionV2(dev, cmd, tw[0], tw[1], tw[2], tw[3], maxlen, dim, True, vk.FP16, True, clip).init()
    cmd.end()
    cmd.submit_and_wait()
    # warm both sides with `offset` earlier tokens so the caches hold history
    steps = ([(offset, 0)] if offset else []) + [(T, offset)]
    for (t, off) in steps:
        x = O.synth_f16(141, 10 + off, t * Wd).reshape(t, Wd)
        want = np.empty((1 if clip else t) * Wd, np.uint16)
        O.lib().orc_attn_forward_q8_0(att, x, ws[0], ws[1], ws[2], ws[3], t, off, int(clip), want)
        cmd.begin()
        tx = up(cmd, dev, x, vk.FP16, 1, t, Wd)
        got = cmd.download(op(tx, off))
        cmd.end()
        cmd.submit_and_wait()
    assert_close(got, want, what="mha T=%d offset=%d clip=%s" % (T, offset, clip))
    kc, vc = op.caches()
    cmd.begin()
    gk, gv = cmd.download(kc), cmd.download(vc)
    cmd.end()
    cmd.submit_and_wait()
    ok = np.ctypeslib.as_array(O.lib().orc_attn_kcache(att), shape=(heads, maxlen, dim))
    ov = np.ctypeslib.as_array(O.lib().orc_attn_vcache(att), shape=(heads, maxlen, dim))
    L = min(offset + T, maxlen)
    assert_close(gk[:, :L], ok[:, :L], tol=2e-3, what="kcache")
    assert_close(gv[:, :L], ov[:, :L], tol=2e-3, what="vcache")
    O.lib().orc_attn_destroy(att)


def test_multiheadattention_ring_wrap(dev):
    heads, dim, maxlen = 2, 32, 8
    Wd = heads * dim
    ws = [O.synth_q8_0(151, i, Wd, Wd, 0.0, 0.05) for i in range(4)]
    att = O.lib().orc_attn_create(heads, dim, maxlen)
    cmd = vk.Command(dev)
    cmd.begin()
    tw = [up(cmd, dev, w, vk.Q8_0, 1, Wd, Wd) for w in ws]
    op = vk.MultiHeadAttentionV2(dev, cmd, tw[0], tw[1], tw[2], tw[3], maxlen, dim, True, vk.FP16, True, False).init()
    cmd.end()
    cmd.submit_and_wait()
    off = 0
    for t in (6, 1, 1, 1, 1):  # positions 6..9 pass the end of the 8-row cache
        x = O.synth_f16(151, 10 + off, t * Wd).reshape(t, Wd)
        want = np.empty(t * Wd, np.uint16)
        O.lib().orc_attn_forward_q8_0(att, x, ws[0], ws[1], ws[2], ws[3], t, off, 0, want)
        cmd.begin()
        tx = up(cmd, dev, x, vk.FP16, 1, t, Wd)
        got = cmd.download(op(tx, off))
        cmd.end()
        cmd.submit_and_wait()
        assert_close(got, want, what="mha wrap offset=%d" % off)
        off += t
    O.lib().orc_attn_destroy(att)


# ---- argument checks keep the reference's status categories --------------------
def test_op_errors(dev):
    cmd = vk.Command(dev)
    cmd.begin()
    w32 = vk.Tensor(1, 1, 64, dev, vk.FP32)
    w16 = vk.Tensor(1, 1, 64, dev, vk.FP16)
    x32 = vk.Tensor(1, 2, 64, dev, vk.FP32)
    with pytest.raises(vk.VklError) as e:  # rms_norm.cpp:33: weight must be FP32
        vk.RMSNorm(dev, cmd, w16, 1e-5, vk.FP16).init()
    assert e.value.code == 3
    op = vk.RMSNorm(dev, cmd, w32, 1e-5, vk.FP16).init()
    with pytest.raises(vk.VklError) as e:  # rms_norm.cpp:64: input dtype
        op(x32)
    assert e.value.code == 3
    with pytest.raises(vk.VklError) as e:  # tensor.cpp:279: reshape size mismatch
        x32.reshape(1, 3, 64)
    assert e.value.code == 11
    cache = vk.Tensor(2, 4, 8, dev, vk.FP16)
    kv = vk.Tensor(2, 5, 8, dev, vk.FP16)
    with pytest.raises(vk.VklError) as e:  # update_kv_cache.cpp:40: value larger than cache
        vk.UpdateKVCache(dev, cmd, vk.FP16).init()(cache, kv, 0)
    assert e.value.code == 11
    with pytest.raises(vk.VklError) as e:  # mat_mul.cpp:130: unsupported dtype pair
        vk.MatMul(dev, cmd, None, 1.0, 0.0, 0, 0, True, vk.FP32, vk.FP32).init()
    assert e.value.code == 3
    cmd.end()
    cmd.submit_and_wait()
    with pytest.raises(vk.VklError) as e:  # ops record only between begin() and end()
        op(vk.Tensor(1, 2, 64, dev, vk.FP16))
    assert e.value.code == 9


def test_matmul_run_many_matches_single_calls_and_times_them(dev):
    """The benchmark helper records the same MatMul calls as one-by-one use of the op."""
    M, N, K = 2, 64, 256
    x = O.synth_f16(61, 1, M * K).reshape(M, K)
    ws = [O.synth_q8_0(61, 10 + i, N, K) for i in range(3)]
    want = O.matmul_q8_0(x, ws[2], M, N, K)
    cmd = vk.Command(dev)
    cmd.begin()
    tx = up(cmd, dev, x, vk.FP16, 1, M, K)
    ops = [vk.MatMul(dev, cmd, up(cmd, dev, w, vk.Q8_0, 1, N, K), 1.0, 0.0, 0, 0, True, vk.FP16, vk.Q8_0).init() for w in ws]
    vk.matmul_run_many(ops, tx, 6)                  # allocates the outputs
    us = vk.matmul_run_many(ops, tx, 6, timed=True)  # the same calls as one CUDA graph
    got = cmd.download(ops[2](tx))
    cmd.end()
    cmd.submit_and_wait()
    assert us > 0.0
    assert_close(got, want, what="matmul after run_many")


# 32 rows and more go through the tensor-core tile kernel (64 query rows per CTA): from an
# empty cache, on top of history (chunked prefill) and across the end of the ring.
@pytest.mark.parametrize("T,offset,maxlen", [(100, 0, 256), (70, 90, 256), (64, 100, 128), (33, 0, 64)])
def test_multiheadattention_many_rows(dev, T, offset, maxlen):
    heads, dim = 4, 64
    Wd = heads * dim
    ws = [O.synth_q8_0(161, i, Wd, Wd, 0.0, 0.05) for i in range(4)]  # wk, wq, wv, wo
    att = O.lib().orc_attn_create(heads, dim, maxlen)
    cmd = vk.Command(dev)
    cmd.begin()
    tw = [up(cmd, dev, w, vk.Q8_0, 1, Wd, Wd) for w in ws]
    op = vk.MultiHeadAttentionV2(dev, cmd, tw[0], tw[1], tw[2], tw[3], maxlen, dim, True, vk.FP16, True, False).init()
    cmd.end()
    cmd.submit_and_wait()
    steps = ([(offset, 0)] if offset else []) + [(T, offset)]
    for (t, off) in steps:
        x = O.synth_f16(161, 10 + off, t * Wd).reshape(t, Wd)
        want = np.empty(t * Wd, np.uint16)
        O.lib().orc_attn_forward_q8_0(att, x, ws[0], ws[1], ws[2], ws[3], t, off, 0, want)
        cmd.begin()
        tx = up(cmd, dev, x, vk.FP16, 1, t, Wd)
        got = cmd.download(op(tx, off))
        cmd.end()
        cmd.submit_and_wait()
    assert_close(got, want, what="mha T=%d offset=%d maxlen=%d" % (T, offset, maxlen))


# ---- device memory pool -----------------------------------------------------------------------
def test_released_block_is_not_reused_while_queued_work_still_writes_it(dev):
    """Ops return without synchronising and every command has its own stream. A tensor released on
    command A while A's kernels are still queued must not be handed to command B before they have
    run: B's data would be overwritten by A's late writes."""
    n = 64 * 1024 * 1024  # 128 MB of fp16: the fill kernels below run for a while
    a, b = vk.Command(dev), vk.Command(dev)
    for rep in range(3):
        a.begin()
        ta = vk.Tensor(1, 1, n, dev, vk.FP16)
        for k in range(6):
            a.fill_synthetic(ta, 7, 100 + k, 0.0, 1.0)  # queued on A's stream
        a.end()
        a.submit()
        del ta  # released while A is still running
        b.begin()
        tb = vk.Tensor(1, 1, n, dev, vk.FP16)  # same size class: the pooled block, if it were free
        b.fill_synthetic(tb, 9, 1, 0.0, 1.0)
        got = b.download(tb)
        b.end()
        b.submit_and_wait()
        a.wait()
        assert np.array_equal(got.ravel()[:4096], O.synth_f16(9, 1, 4096)), "rep %d" % rep
        assert np.array_equal(got.ravel()[-4096:], O.synth_f16(9, 1, 4096, first=n - 4096)), "rep %d" % rep
        del tb


def test_pool_is_bounded_under_varying_sizes(dev):
    """Calls with many different row counts land in a bounded set of size classes, and what the
    pool keeps never exceeds its cap (an eighth of the device memory)."""
    cmd = vk.Command(dev)
    cap = dev.info()[2] // 8
    before = dev.pool_bytes()  # other tests' blocks
    cmd.begin()
    for rep in range(3):
        for T in range(1, 200, 3):
            t = vk.Tensor(1, T, 4096, dev, vk.FP16)
            del t
    cmd.end()
    cmd.submit_and_wait()
    kept = dev.pool_bytes()
    assert kept <= cap
    # 67 different sizes between 8 KB and 1.6 MB, three times over: at most one block per size class
    # (a class is at most 25 % over the request) unless a block was still fenced when its size came up again
    assert kept - before <= 2 * 67 * 1.25 * 200 * 4096 * 2


# ---- generic ops outside the token loop, at the reference's own test shapes ---------------------
@pytest.mark.parametrize("op_type", [0, 1, 2, 3])
@pytest.mark.parametrize("scalar", [False, True])
def test_elementwise_all_types_tensor_and_scalar(dev, op_type, scalar):
    """tests/test_elementwise.cpp:178-182: [3,1023,511], add / sub / mul / div, tensor and constant operand."""
    C, H, W = 3, 1023, 511
    x = O.synth_f16(122, 1, C * H * W).reshape(C, H, W)
    y = O.synth_f16(122, 2, C * H * W, mean=2.0, std=0.25).reshape(C, H, W)  # away from zero: a divisor too
    cmd = vk.Command(dev)
    cmd.begin()
    tx, ty = up(cmd, dev, x, vk.FP16, C, H, W), up(cmd, dev, y, vk.FP16, C, H, W)
    op = vk.ElementWise(dev, cmd, op_type, vk.FP16).init()
    if scalar:
        got = cmd.download(op(tx, 1.75))
        same = cmd.download(tx)  # in place in x
    else:
        got = cmd.download(op(tx, ty))
        same = cmd.download(ty)  # in place in the second operand
    cmd.end()
    cmd.submit_and_wait()
    want = O.elementwise(x, 1.75 if scalar else y, op_type)
    assert np.array_equal(got, want) and np.array_equal(same, want)


@pytest.mark.parametrize("axis,shapes", [(0, [(1, 63, 31), (2, 63, 31), (5, 63, 31)]), (1, [(3, 63, 31), (3, 31, 31), (3, 22, 31)]),
                                         (2, [(3, 63, 31), (3, 63, 63), (3, 63, 22)])])
def test_concat(dev, axis, shapes):
    """tests/test_concat.cpp:117-121."""
    ins = [O.synth_f16(123, 10 + i, c * h * w).reshape(c, h, w) for i, (c, h, w) in enumerate(shapes)]
    cmd = vk.Command(dev)
    cmd.begin()
    ts = [up(cmd, dev, a, vk.FP16, *a.shape) for a in ins]
    op = vk.Concat(dev, cmd, len(ins), axis, vk.FP16).init()
    got = cmd.download(op(ts))
    cmd.end()
    cmd.submit_and_wait()
    assert np.array_equal(got, O.concat(ins, axis))
    cmd.begin()
    with pytest.raises(vk.VklError) as e:  # wrong input count
        op(ts[:2])
    assert e.value.code == 3
    bad = vk.Concat(dev, cmd, 2, (axis + 1) % 3, vk.FP16).init()
    with pytest.raises(vk.VklError) as e:  # extents that agree along this test's axis only
        bad([ts[1], ts[2]])
    assert e.value.code == 3
    cmd.end()
    cmd.submit_and_wait()


@pytest.mark.parametrize("op_type", [0, 1, 2, 3])
def test_reduce(dev, op_type):
    """tests/test_reduce.cpp:113-118: [1,1023,511], sum / max / min / mean."""
    C, H, W = 1, 1023, 511
    x = O.synth_f16(124, op_type, C * H * W).reshape(C, H, W)
    cmd = vk.Command(dev)
    cmd.begin()
    op = vk.Reduce(dev, cmd, op_type, vk.FP16).init()
    got = cmd.download(op(up(cmd, dev, x, vk.FP16, C, H, W)))
    cmd.end()
    cmd.submit_and_wait()
    assert got.shape == (C, H, 1)
    assert np.array_equal(got, O.reduce(x, op_type))


@pytest.mark.parametrize("offset,length", [(0, 25), (1010, 25), (1022, 2), (5, 1024)])
def test_read_kvcache_reads_back_what_update_wrote(dev, offset, length):
    """tests/test_update_kv_cache.cpp:61-114: heads 32, maxlen 1024, dim 100; write at an offset (wrapping at the
    end of the ring), read the same rows back."""
    heads, maxlen, dim = 32, 1024, 100
    base = O.synth_f16(125, 1, heads * maxlen * dim).reshape(heads, maxlen, dim)
    kv = O.synth_f16(125, 2, heads * 25 * dim).reshape(heads, 25, dim)
    cmd = vk.Command(dev)
    cmd.begin()
    cache = up(cmd, dev, base, vk.FP16, heads, maxlen, dim)
    vk.UpdateKVCache(dev, cmd, vk.FP16).init()(cache, up(cmd, dev, kv, vk.FP16, heads, 25, dim), 1010)
    rd = vk.ReadKVCache(dev, cmd).init()
    got = cmd.download(rd(cache, offset, length))
    cmd.end()
    cmd.submit_and_wait()
    want_cache = base.copy()
    want_cache[:, (np.arange(25) + 1010) % maxlen] = kv
    assert np.array_equal(got, O.read_kvcache(want_cache, offset, length))
    if (offset, length) == (1010, 25):
        assert np.array_equal(got, kv)
    cmd.begin()
    with pytest.raises(vk.VklError) as e:
        rd(cache, 0, maxlen + 1)
    assert e.value.code == 11
    cmd.end()
    cmd.submit_and_wait()


@pytest.mark.parametrize("C,M,N,K,bt,tb", [(5, 64, 48, 96, 1, True), (5, 64, 48, 96, 2, True), (4, 33, 50, 40, 1, False), (4, 33, 50, 40, 2, False),
                                          (16, 31, 21, 129, 0, True)])
def test_matmul_broadcast_types(dev, C, M, N, K, bt, tb):
    """tests/test_matmul.cpp:121-174 (broadcast 0 / 1 / 2, with and without transposed B), scaled-down shapes."""
    ca, cb = (1 if bt == 2 else C), (1 if bt == 1 else C)
    a = O.synth_f16(126, 1, ca * M * K).reshape(ca, M, K)
    bshape = (cb, N, K) if tb else (cb, K, N)
    b = O.synth_f16(126, 2, cb * N * K, std=0.1).reshape(bshape)
    cmd = vk.Command(dev)
    cmd.begin()
    ta, tbn = up(cmd, dev, a, vk.FP16, *a.shape), up(cmd, dev, b, vk.FP16, *bshape)
    pair = vk.MatMul(dev, cmd, None, 0.5, 0.25, 0, bt, tb, vk.FP16, vk.FP16).init()
    got_pair = cmd.download(pair(ta, tbn))
    wop = vk.MatMul(dev, cmd, tbn, 0.5, 0.25, 1, bt, tb, vk.FP16, vk.FP16).init()  # B as the op's weight, SiLU
    got_w = cmd.download(wop(ta))
    cmd.end()
    cmd.submit_and_wait()
    assert got_pair.shape == (C, M, N)
    assert_close(got_pair, O.matmul_broadcast(a, b, bt, tb, 0.5, 0.25, 0), what="matmul broadcast %d" % bt)
    assert_close(got_w, O.matmul_broadcast(a, b, bt, tb, 0.5, 0.25, 1), what="matmul broadcast %d weight form" % bt)
    wrong = vk.MatMul(dev, cmd, None, 1.0, 0.0, 0, 1 if bt != 1 else 2, tb, vk.FP16, vk.FP16).init()
    if C > 1 and bt != 0:
        cmd.begin()
        with pytest.raises(vk.VklError) as e:
            wrong(ta, tbn)
        assert e.value.code == 3
        cmd.end()
        cmd.submit_and_wait()


def test_tensor_view_through_matmul_keeps_the_parent_strides(dev):
    """src/core/tensor.cpp:294-302: a view narrows the extents and keeps the strides; the attention reads the first L
    rows of every head of the [heads, maxlen, dim] cache through such a view (multiheadattention_v2.cpp:255-275)."""
    heads, maxlen, dim, L, M = 6, 64, 32, 19, 3
    cache = O.synth_f16(127, 1, heads * maxlen * dim).reshape(heads, maxlen, dim)
    q = O.synth_f16(127, 2, heads * M * dim).reshape(heads, M, dim)
    cmd = vk.Command(dev)
    cmd.begin()
    tc, tq = up(cmd, dev, cache, vk.FP16, heads, maxlen, dim), up(cmd, dev, q, vk.FP16, heads, M, dim)
    view = tc.view(heads, L, dim)
    assert view.shape() == (heads, L, dim) and view.shape_constant()[3:] == tc.shape_constant()[3:]  # extents narrowed, strides kept
    scores = vk.MatMul(dev, cmd, None, 1.0 / np.sqrt(dim), 0.0, 0, 0, True, vk.FP16, vk.FP16).init()
    got = cmd.download(scores(tq, view))  # q . K^T over the first L cached rows of every head
    pv = vk.MatMul(dev, cmd, None, 1.0, 0.0, 0, 0, False, vk.FP16, vk.FP16).init()
    p = O.synth_f16(127, 3, heads * M * L, std=0.2).reshape(heads, M, L)
    got_pv = cmd.download(pv(up(cmd, dev, p, vk.FP16, heads, M, L), view))  # P . V with the same kind of view
    cmd.end()
    cmd.submit_and_wait()
    assert_close(got, O.matmul_broadcast(q, cache[:, :L], 0, True, 1.0 / np.sqrt(dim)), what="q.K^T through a view")
    assert_close(got_pv, O.matmul_broadcast(p, cache[:, :L], 0, False), what="P.V through a view")
