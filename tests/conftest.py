import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "llama2.rs_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def l2():
    """The product's Python surface; builds the C-ABI library on first use if it is missing."""
    lib_path = os.path.join(ROOT, "llama2.rs_b200", "libllama2_b200.so")
    if not os.path.exists(lib_path):
        sys.path.insert(0, os.path.join(ROOT, "llama2.rs_b200"))
        import build as _build
        _build.build()
    import llama2_rs
    return llama2_rs


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.lib()
    return oracle


def tiny_config(l2, group_size=64, n_kv_heads=2, n_layers=2, dim=256, hidden=512, vocab=512, seq_len=64):
    c = l2.Config()
    c.dim, c.hidden_dim, c.n_layers, c.n_heads = dim, hidden, n_layers, dim // 128
    c.n_kv_heads, c.vocab_size, c.seq_len, c.group_size = n_kv_heads, vocab, seq_len, group_size
    return c


def random_qlinear(rng, in_f, out_f, gs):
    """A QLinear record with the value distributions of the synthetic checkpoint."""
    groups = in_f // gs
    qweight = rng.integers(0, 2**32, size=(out_f, in_f // 8), dtype=np.uint32).view(np.int32)
    znib = rng.integers(6, 10, size=(out_f // 8, groups, 8), dtype=np.uint32)
    qzeros = np.zeros((out_f // 8, groups), np.uint32)
    for j in range(8):
        qzeros |= znib[:, :, j] << np.uint32(4 * j)
    scales = rng.uniform(0.002, 0.02, size=(out_f, groups)).astype(np.float32)
    perm = rng.permutation(in_f)
    g_idx = perm // gs
    g_index = np.argsort(g_idx, kind="stable").astype(np.int32)
    return qweight, qzeros.view(np.int32), scales, g_index


def dequant_dense(qweight, qzeros, scales, g_index, gs):
    """Independent check: dense f64 [OUT][IN] matrix in natural input order."""
    out_f, words = qweight.shape
    in_f = words * 8
    q = np.zeros((out_f, in_f), np.int64)
    qw = qweight.view(np.uint32)
    for j in range(8):
        q[:, j::8] = (qw >> np.uint32(4 * j)) & 15
    qz = qzeros.view(np.uint32)
    z = np.zeros((out_f, in_f // gs), np.int64)
    for r in range(8):
        z[r::8, :] = ((qz >> np.uint32(4 * r)) & 15) + 1
    w_perm = (q - np.repeat(z, gs, axis=1)) * np.repeat(scales.astype(np.float64), gs, axis=1)
    w = np.zeros_like(w_perm)
    w[:, g_index] = w_perm  # permuted position p reads input g_index[p]
    return w


def assert_close(got, want, rel=1e-2, abs_=1e-3, what=""):
    """The parity bound of the token loop: |got - want| <= abs + rel * |want|."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    bound = abs_ + rel * np.abs(want)
    bad = err > bound
    assert not bad.any(), "%s: %d of %d outside tolerance, worst |err| %.3g at %s (want %.6g got %.6g)" % (
        what, bad.sum(), bad.size, err.max(), np.unravel_index(err.argmax(), err.shape),
        want.flat[err.argmax()], got.flat[err.argmax()])
