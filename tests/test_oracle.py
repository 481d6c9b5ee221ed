"""Pins the CPU oracle: known-answer vectors derived from the reference's constant fixtures,
an independent dequantise-then-matmul check, and the quirks of the reference arithmetic."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import assert_close, dequant_dense, random_qlinear, tiny_config

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_known_answer_basic(orc):
    # src/gptq_test.rs:40-53 basic(): qweight 0x76543210, scales 10, qzeros 0 (zero point 1), x 10
    IN, OUT, GS = 4096, 64, 128
    qweight = np.full((OUT, IN // 8), 1985229328, np.int32)
    qzeros = np.zeros((OUT // 8, IN // GS), np.int32)
    scales = np.full((OUT, IN // GS), 10.0, np.float32)
    g_index = np.arange(IN, dtype=np.int32)
    y = orc.qlinear_matvec(qweight, qzeros, scales, g_index, GS, np.full(IN, 10.0, np.float32))
    assert np.all(y == 100.0 * (IN // 8) * sum(j - 1 for j in range(8)))  # 1 024 000


def test_known_answer_zero_nibbles(orc):
    # src/kernel.py:100-103 / src/gptq_test.rs:56-62: qweight 0, scales -1, qzeros 0x76543210, x 1
    IN, OUT, GS = 4096, 64, 128
    qweight = np.zeros((OUT, IN // 8), np.int32)
    qzeros = np.full((OUT // 8, IN // GS), 1985229328, np.int32)
    scales = np.full((OUT, IN // GS), -1.0, np.float32)
    g_index = np.arange(IN, dtype=np.int32)
    y = orc.qlinear_matvec(qweight, qzeros, scales, g_index, GS, np.ones(IN, np.float32))
    assert np.array_equal(y, np.array([IN * ((o % 8) + 1) for o in range(OUT)], np.float32))


@pytest.mark.parametrize("gs", [32, 64, 128])
@pytest.mark.parametrize("B", [1, 2, 5])
def test_qlinear_vs_dense(orc, gs, B):
    rng = np.random.default_rng(gs * 10 + B)
    IN, OUT = 512, 72
    qw, qz, sc, gi = random_qlinear(rng, IN, OUT, gs)
    x = rng.standard_normal((B, IN)).astype(np.float32)
    y = orc.qlinear_matvec(qw, qz, sc, gi, gs, x)
    want = x.astype(np.float64) @ dequant_dense(qw, qz, sc, gi, gs).T
    assert_close(y, want, rel=1e-5, abs_=1e-5, what="qlinear vs dense")


def test_batch_rows_independent(orc):
    rng = np.random.default_rng(3)
    qw, qz, sc, gi = random_qlinear(rng, 256, 64, 64)
    x = rng.standard_normal((4, 256)).astype(np.float32)
    yb = orc.qlinear_matvec(qw, qz, sc, gi, 64, x)
    for b in range(4):
        assert np.array_equal(yb[b], orc.qlinear_matvec(qw, qz, sc, gi, 64, x[b]))


def test_rope_rotate_half_in_place(orc):
    # src/models.rs:106-116: the second half is rotated with the NEW first half
    hs, pos = 128, 7
    rng = np.random.default_rng(0)
    q = rng.standard_normal(2 * hs).astype(np.float32)
    k = rng.standard_normal(hs).astype(np.float32)
    q0, k0 = q.copy(), k.copy()
    L = orc.lib()
    L.orc_rope(q.ctypes.data_as(C.POINTER(C.c_float)), k.ctypes.data_as(C.POINTER(C.c_float)), pos, 2, 1, hs)
    i = np.arange(hs // 2)
    freq = (1.0 / np.power(np.float32(10000.0), (2 * i).astype(np.float32) / np.float32(hs))).astype(np.float32)
    ang = (np.float32(pos) * freq).astype(np.float64)
    c, s = np.cos(ang), np.sin(ang)
    for h in range(2):
        a, b = q0[h * hs:h * hs + 64].astype(np.float64), q0[h * hs + 64:(h + 1) * hs].astype(np.float64)
        na = a * c - b * s
        nb = b * c + na * s
        np.testing.assert_allclose(q[h * hs:h * hs + 64], na, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(q[h * hs + 64:(h + 1) * hs], nb, rtol=1e-5, atol=1e-6)
    a, b = k0[:64].astype(np.float64), k0[64:].astype(np.float64)
    np.testing.assert_allclose(k[:64], a * c - b * s, rtol=1e-5, atol=1e-6)
    # textbook RoPE would give b*c + a*s for the second half; the reference does not
    assert not np.allclose(q[64:128], q0[64:128] * c + q0[:64] * s, atol=1e-3)


def test_argmax_last_max_wins(orc):
    v = np.array([1.0, 5.0, 2.0, 5.0, 0.0], np.float32)
    assert orc.lib().orc_argmax(v.ctypes.data_as(C.POINTER(C.c_float)), 5) == 3


def test_random_matches_xorshift_star(orc):
    seed = C.c_uint64(1)
    s = 1
    for _ in range(5):
        s ^= s >> 12
        s = (s ^ (s << 25)) & (2**64 - 1)
        s ^= s >> 27
        want = ((s * 0x2545F4914F6CDD1D) & (2**64 - 1)) >> 32
        assert orc.lib().orc_random_u32(C.byref(seed)) == want
    assert seed.value == s


def test_sample_cdf_walk(orc):
    p = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    L = orc.lib()
    for s0 in (1, 2, 3, 99):
        seed = C.c_uint64(s0)
        seed2 = C.c_uint64(s0)
        r = L.orc_random_f32(C.byref(seed2))
        want = int(np.searchsorted(np.cumsum(p, dtype=np.float32), r, side="right"))
        assert L.orc_sample(C.byref(seed), p.ctypes.data_as(C.POINTER(C.c_float)), 4) == min(want, 3)


def test_layout_sizes(orc):
    # payload sizes of the three model sizes (size_of::<QTransformerWeights>())
    sizes = {("7B", 128): 4520919044, ("13B", 128): 8110493700, ("70B", 64): 41166864388}
    dims = {"7B": (4096, 11008, 32, 32, 32), "13B": (5120, 13824, 40, 40, 40), "70B": (8192, 28672, 80, 64, 8)}
    for (name, gs), want in sizes.items():
        d, h, l, nh, kv = dims[name]
        cfg = orc.make_config(dim=d, hidden_dim=h, n_layers=l, n_heads=nh, n_kv_heads=kv, vocab_size=32000, seq_len=2048, group_size=gs)
        assert orc.weights_bytes(cfg) == want


def test_prefill_ladder_matches_single_steps(orc, l2):
    # "Should lead to identical results" (src/inference.rs:12-15)
    cfg = tiny_config(l2, group_size=64, n_kv_heads=1)
    payload = l2.synth_fill(cfg, 20240)
    m = orc.Model(cfg, payload)
    prompt = np.random.default_rng(7).integers(0, cfg.vocab_size, 21).astype(np.int32)
    a = m.generate_ids(prompt, 40, use_prefill=True, trace_logits=True)
    b = m.generate_ids(prompt, 40, use_prefill=False, trace_logits=True)
    assert a["pos0"] == 20 and b["pos0"] == 0  # 16 + 4 positions pre-filled, one prompt position left
    assert np.array_equal(a["tokens"], b["tokens"][20:])
    assert_close(a["logits"], b["logits"][20:], rel=1e-4, abs_=1e-5, what="prefill vs steps")
    assert np.array_equal(b["tokens"][:21], prompt[:21])  # teacher forcing


def test_steps_beyond_seq_len_rejected(orc, l2):
    cfg = tiny_config(l2)
    m = orc.Model(cfg, l2.synth_fill(cfg, 1))
    with pytest.raises(ValueError):
        m.generate_ids([1, 2, 3], cfg.seq_len + 1)


def test_oracle_matches_golden(orc, l2):
    g = np.load(os.path.join(GOLDEN, "tiny_generate.npz"))
    cfg = tiny_config(l2, group_size=int(g["group_size"]), n_kv_heads=int(g["n_kv_heads"]))
    m = orc.Model(cfg, l2.synth_fill(cfg, int(g["seed"])))
    r = m.generate_ids(g["prompt"], int(g["steps"]), trace_logits=True)
    assert np.array_equal(r["tokens"], g["tokens"])
    assert_close(r["logits"], g["logits"], rel=1e-5, abs_=1e-6, what="oracle vs golden")
