"""Parity of the CUDA fused dequant+GEMV (through the C ABI) with the CPU oracle's
QLinear::matvec on the same inputs."""
import numpy as np
import pytest

from conftest import assert_close, dequant_dense, random_qlinear

pytestmark = pytest.mark.gpu


def test_known_answer_basic(l2):
    IN, OUT, GS = 4096, 2048, 128  # src/gptq_test.rs:23-27,40-53
    q = l2.QLinear(np.full((OUT, IN // 8), 1985229328, np.int32), np.zeros((OUT // 8, IN // GS), np.int32),
                   np.full((OUT, IN // GS), 10.0, np.float32), np.arange(IN, dtype=np.int32), GS)
    y = q.matvec(np.full(IN, 10.0, np.float32))
    assert np.all(y == 1024000.0)


def test_known_answer_zero_nibbles(l2):
    IN, OUT, GS = 4096, 2048, 128  # src/kernel.py:100-103
    q = l2.QLinear(np.zeros((OUT, IN // 8), np.int32), np.full((OUT // 8, IN // GS), 1985229328, np.int32),
                   np.full((OUT, IN // GS), -1.0, np.float32), np.arange(IN, dtype=np.int32), GS)
    y = q.matvec(np.ones(IN, np.float32))
    assert np.array_equal(y, np.array([IN * ((o % 8) + 1) for o in range(OUT)], np.float32))


@pytest.mark.parametrize("gs", [32, 64, 128])
@pytest.mark.parametrize("in_f,out_f", [(128, 8), (256, 64), (1408, 40), (2048, 1000)])
def test_small_shapes(l2, orc, gs, in_f, out_f):
    rng = np.random.default_rng(in_f + out_f + gs)
    qw, qz, sc, gi = random_qlinear(rng, in_f, out_f, gs)
    x = rng.standard_normal((3, in_f)).astype(np.float32)
    y = l2.QLinear(qw, qz, sc, gi, gs).matvec(x)
    assert_close(y, orc.qlinear_matvec(qw, qz, sc, gi, gs, x), rel=1e-4, abs_=5e-4, what="gemv vs oracle")
    assert_close(y, x.astype(np.float64) @ dequant_dense(qw, qz, sc, gi, gs).T, rel=1e-4, abs_=5e-4, what="gemv vs dense")


# the (K, N) shapes of the isolated QLinear benchmark: 7B, 13B and 70B projections
SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096), (5120, 13824), (8192, 28672), (28672, 8192), (8192, 1024)]


@pytest.mark.parametrize("gs", [64, 128])
@pytest.mark.parametrize("K,N", SHAPES)
def test_model_shapes(l2, orc, gs, K, N):
    rng = np.random.default_rng(K * 7 + N + gs)
    qw, qz, sc, gi = random_qlinear(rng, K, N, gs)
    q = l2.QLinear(qw, qz, sc, gi, gs)
    for M in (1, 4):
        x = rng.standard_normal((M, K)).astype(np.float32)
        y = q.matvec(x)
        assert_close(y, orc.qlinear_matvec(qw, qz, sc, gi, gs, x), rel=1e-4, abs_=1e-3, what="K%d N%d M%d" % (K, N, M))
    # linearity, a size-independent property: W(a x1 + x2) = a W x1 + W x2
    x1, x2 = rng.standard_normal((2, K)).astype(np.float32)
    lhs = q.matvec(2.0 * x1 + x2).astype(np.float64)
    rhs = 2.0 * q.matvec(x1).astype(np.float64) + q.matvec(x2)
    assert_close(lhs, rhs, rel=1e-4, abs_=2e-3, what="linearity")
    # bit-reproducible from call to call
    assert np.array_equal(q.matvec(x1), q.matvec(x1))


@pytest.mark.parametrize("gs", [64, 128])
@pytest.mark.parametrize("K,N", SHAPES)
def test_model_shapes_batched(l2, orc, gs, K, N):
    # the batched (tcgen05) path at the benchmark's batch sizes: one pass, a full pass, several passes, and a ragged batch;
    # on the large shapes the groups of a matrix are split over several CTAs per tile as well
    rng = np.random.default_rng(K * 11 + N + gs)
    qw, qz, sc, gi = random_qlinear(rng, K, N, gs)
    q = l2.QLinear(qw, qz, sc, gi, gs)
    for M in (16, 64, 256, 37):
        x = rng.standard_normal((M, K)).astype(np.float32)
        y = q.matvec(x)
        assert_close(y, orc.qlinear_matvec(qw, qz, sc, gi, gs, x), rel=1e-4, abs_=1e-3, what="K%d N%d M%d" % (K, N, M))
    # a row of a batch equals the same row alone (B = 1 goes through the GEMV kernel): same integers, same scale order
    x = rng.standard_normal((5, K)).astype(np.float32)
    assert_close(q.matvec(x)[3], q.matvec(x[3]), rel=1e-5, abs_=1e-4, what="batched row vs single row")


def test_bad_arguments(l2):
    rng = np.random.default_rng(0)
    qw, qz, sc, gi = random_qlinear(rng, 256, 64, 64)
    with pytest.raises(l2.L2Error):
        l2.QLinear(qw, qz, sc, gi, 48)
    gi_bad = gi.copy()
    gi_bad[0] = gi_bad[1]
    with pytest.raises(l2.L2Error):
        l2.QLinear(qw, qz, sc, gi_bad, 64)
