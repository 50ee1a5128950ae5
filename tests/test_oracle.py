"""The CPU oracle against the reference's known answers and against itself.

The reference holds one known-answer vector for this path: all-ones operands, every output
equals K (script/ncu-gemv-test.py:29-47, shapes :7-24).  The rest are closed-form cases.
"""
import numpy as np
import pytest

from oracle import oracle as o

# LLaMA-7B/13B and Qwen-14B GEMV shapes of the reference's script (N, K); K values exact in fp16
KAT_SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (5120, 5120), (13824, 5120), (5120, 13824),
              (13696, 5120), (5120, 13696)]


@pytest.mark.parametrize("N,K", KAT_SHAPES)
def test_all_ones_known_answer(N, K):
    n = min(N, 256)  # rows are independent; a slice keeps the CPU suite fast
    W = np.ones((n, K), np.float16)
    x = np.ones((1, K), np.float16)
    assert (o.gemv_fp16_ref(W, x).astype(np.float32) == float(np.float16(K))).all()
    assert (o.gemm_nk(x, W) == K).all()
    assert (o.gemm_kn(x, np.ascontiguousarray(W.T)) == K).all()
    W8 = np.ones((n, K), np.int8)
    assert (o.gemv_int8_ref(W8, x).astype(np.float32) == float(np.float16(K))).all()
    assert (o.gemm_w8a16_nk(x, W8) == K).all()


def _rand(N, K, M, seed):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    return W, x


@pytest.mark.parametrize("N,K", [(128, 1024), (256, 4096), (128, 11008)])
def test_order_exact_kernels_agree_with_fp32_reference(N, K):
    W, x = _rand(N, K, 8, N + K)
    ref = o.gemm_nk(x, W)
    o.check_tolerance(o.gemv_fp16_ref(W, x[0])[None], ref[:1], "gemv_fp16")
    o.check_tolerance(o.gemv_fp16_bs2_ref(W, x[:2]), ref[:2], "gemv_fp16_bs2")
    o.check_tolerance(o.gemm_fp16_ref(W, x), ref, "gemm_fp16")
    # M=1 of the two-row kernel follows the same order as the one-row kernel
    assert np.array_equal(o.gemv_fp16_bs2_ref(W, x[:2])[0], o.gemv_fp16_ref(W, x[0]))
    # numpy's own fp32 matmul is an independent check of the double-accumulated value
    assert np.abs(ref - x.astype(np.float32) @ W.astype(np.float32).T).max() < 1e-4
    assert np.abs(o.gemm_nk_f32seq(x, W) - ref).max() < 1e-3


def test_layouts_agree():
    W, x = _rand(256, 512, 5, 3)
    assert np.array_equal(o.gemm_kn(x, np.ascontiguousarray(W.T)), o.gemm_nk(x, W))


def test_one_hot_selects_a_weight_column():
    W, _ = _rand(128, 1024, 1, 9)
    for k in (0, 7, 8, 1023):
        x = np.zeros((1, 1024), np.float16)
        x[0, k] = 1
        assert np.array_equal(o.gemv_fp16_ref(W, x), W[:, k])
        assert np.array_equal(o.gemm_nk(x, W)[0], W[:, k].astype(np.float32))


def test_int8_reference_semantics():
    rng = np.random.default_rng(5)
    N, K = 128, 2048
    W8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    x = rng.standard_normal((2, K)).astype(np.float16)
    s = (rng.uniform(0.5, 1.5, N) / 127).astype(np.float16)
    exact = x.astype(np.float64) @ W8.astype(np.float64).T
    assert np.allclose(o.gemm_w8a16_nk(x, W8), exact, rtol=1e-6, atol=1e-3)
    assert np.allclose(o.gemm_w8a16_nk(x, W8, s), exact * s.astype(np.float64), rtol=1e-6, atol=1e-5)
    # the reference launches its kernel with scale 1 / zero-point 0 (hk/fastgemv.cu:50-59)
    y = o.gemv_int8_ref(W8, x[0])
    o.check_tolerance(y[None], o.gemm_w8a16_nk(x[:1], W8), "gemv_quantized_int8")
    # a zero point shifts every weight
    y_zp = o.gemv_int8_ref(W8, x[0], 1.0, 3.0).astype(np.float64)
    want = x[0].astype(np.float64) @ (W8.astype(np.float64) - 3.0).T
    assert np.allclose(y_zp, want, rtol=2e-3, atol=0.5)


def test_tolerance_rule():
    ref = np.array([[0.0, 0.5, 100.0]], np.float32)
    assert o.tolerance_excess(ref + np.array([[0.009, -0.009, 0.9]], np.float32), ref) < 1.0
    assert o.tolerance_excess(ref + np.array([[0.011, 0, 0]], np.float32), ref) > 1.0
    assert o.tolerance_excess(ref + np.array([[0, 0, 1.1]], np.float32), ref) > 1.0
    assert o.tolerance_excess(np.array([[np.nan, 0, 0]], np.float32), ref) == float("inf")
    with pytest.raises(AssertionError):
        o.check_tolerance(ref + 1, ref)


def test_a_dropped_k_block_is_caught():
    """The tolerance is tight enough that losing one 64-wide k-block fails."""
    W, x = _rand(128, 4096, 4, 21)
    ref = o.gemm_nk(x, W)
    x2 = x.copy()
    x2[:, 640:704] = 0
    assert o.tolerance_excess(o.gemm_nk(x2, W), ref) > 1.0


@pytest.mark.parametrize("M,N,K,bz", [(8, 8192, 8192, 4), (16, 8192, 8192, 1), (8, 4096, 4096, 8),
                                      (8, 4096, 4224, 1), (8, 4096, 4352, 2), (8, 4096, 4608, 4),
                                      (1, 11008, 4096, 1)])
def test_reference_splitk_choice(M, N, K, bz):
    """hk/edgemm.cu:287-305, values worked out by hand from the thresholds."""
    assert o.ref_splitk_bt(M, N, K) == bz


def test_quantiser_restatement():
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((32, 512)) / 20).astype(np.float16)
    W[5] = 0                                  # all-zero row: scale 1, zeros
    W[6, 0] = np.float16(3.0)                 # the row maximum maps to +-127
    q, s = o.quantize_rows_w8(W)
    assert q.dtype == np.int8 and s.dtype == np.float16
    assert int(q.min()) >= -127 and int(q.max()) <= 127
    assert float(s[5]) == 1.0 and not q[5].any()
    assert abs(int(q[6, 0])) == 127
    # reconstruction error is at most half a quantisation step (plus the fp16 rounding of the scale)
    err = np.abs(q.astype(np.float32) * s[:, None].astype(np.float32) - W.astype(np.float32))
    assert (err <= 0.51 * s[:, None].astype(np.float32) + 1e-6).all()
    # independent numpy restatement
    sf = s.astype(np.float32)[:, None]
    assert np.array_equal(q, np.clip(np.rint(W.astype(np.float32) / sf), -127, 127).astype(np.int8))


def _unpack_w4(W4):
    q = np.empty((W4.shape[0], W4.shape[1] * 2), np.int32)
    q[:, 0::2] = W4 & 0x0F   # even k in the low nibble (uint4_2::getX, hk/utility.cuh:22-24)
    q[:, 1::2] = W4 >> 4     # odd k in the high nibble (getY, :26-28)
    return q


def test_int4_reference_semantics():
    rng = np.random.default_rng(8)
    N, K = 128, 2048
    W4 = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    x = rng.standard_normal((2, K)).astype(np.float16)
    q = _unpack_w4(W4).astype(np.float64)
    for zp in (0, 8, 11):
        exact = x.astype(np.float64) @ (q - zp).T
        assert np.allclose(o.gemm_w4a16_nk(x, W4, None, zp), exact, rtol=1e-6, atol=1e-3)
    # one scale per channel, one scale per 128 k
    s1 = (rng.uniform(0.5, 1.5, N) / 8).astype(np.float16)
    assert np.allclose(o.gemm_w4a16_nk(x, W4, s1, 8), (x.astype(np.float64) @ (q - 8).T) * s1.astype(np.float64),
                       rtol=1e-6, atol=1e-4)
    sg = (rng.uniform(0.5, 1.5, (N, K // 128)) / 8).astype(np.float16)
    wdq = (q - 8) * np.repeat(sg.astype(np.float64), 128, axis=1)
    assert np.allclose(o.gemm_w4a16_nk(x, W4, sg, 8), x.astype(np.float64) @ wdq.T, rtol=1e-6, atol=1e-4)
    # the reference's kernel (scalar scale and zero point) sits within the tolerance of that reference
    y = o.gemv_int4_ref(W4, x[0], 0.0625, 8.0)
    o.check_tolerance(y[None], o.gemm_w4a16_nk(x[:1], W4, np.full(N, 0.0625, np.float16), 8), "gemv_quantized_int4")
    # all-ones known answer: every output is K * (15 - zero_point) * scale
    ones = np.ones(K, np.float16)
    y1 = o.gemv_int4_ref(np.full((N, K // 2), 0xFF, np.uint8), ones, 0.03125, 8.0)
    assert np.array_equal(y1, np.full(N, K * 7 * 0.03125, np.float16))


def test_int4_quantiser_restatement():
    rng = np.random.default_rng(4)
    W = (rng.standard_normal((16, 512)) / 20).astype(np.float16)
    W[3] = 0
    for groups in (1, 4):
        q4, s = o.quantize_rows_w4(W, groups)
        assert q4.shape == (16, 256) and s.shape == (16, groups)
        q = _unpack_w4(q4)
        assert (q[3] == 8).all() and (s[3] == 1.0).all()
        sf = np.repeat(s.astype(np.float32), 512 // groups, axis=1)
        assert np.array_equal(q, np.clip(np.rint(W.astype(np.float32) / sf) + 8, 0, 15).astype(np.int32))
        err = np.abs((q - 8) * sf - W.astype(np.float32))
        assert (err <= 0.51 * sf + 1e-6).all()
        assert q.max() == 15 and q.min() >= 1  # the maximum maps to +7, nothing below -7
