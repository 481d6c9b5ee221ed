"""Host-side logic that needs no GPU: the C ABI surface, the load-time repack (an exact
re-ordering), the tokenizer, and loud failure when no CUDA device is present."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

from conftest import ROOT, dequant_dense, random_qlinear, tiny_config


def test_every_declared_symbol_is_exported(l2):
    header = open(os.path.join(ROOT, "include", "llama2_b200.h")).read()
    declared = set(re.findall(r"\b(l2_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    for name in sorted(declared):
        assert hasattr(l2.lib, name), name
    assert declared == set(l2._lib.SIGNATURES), declared ^ set(l2._lib.SIGNATURES)


def emulate_device_gemv(rec, tiles, in_f, out_f, gs, x_perm):
    """numpy model of the kernel's view of the device layout (tiles of 16 rows, units of one group):
    y[o] = sum_g scale * sum_k (q - z) x."""
    G, W = in_f // gs, gs // 32
    rec = rec.reshape(tiles, G, 64 * W + 20)
    qw = rec[:, :, :64 * W].reshape(tiles, G, 2, 32, W)
    meta = rec[:, :, 64 * W:]
    sc = meta[:, :, :16].copy().view(np.float32)
    zr = meta[:, :, 16:18]
    assert not meta[:, :, 18:].any()
    y = np.zeros(out_f)
    for o in range(out_f):
        tile, h, r = o // 16, (o % 16) // 8, o % 8
        for g in range(G):
            z = int((zr[tile, g, h] >> np.uint32(4 * r)) & 15) + 1
            acc = 0.0
            for t in range(4):
                for i in range(W):
                    word = int(qw[tile, g, h, r * 4 + t, i])
                    k0 = g * gs + (t * W + i) * 8
                    for j in range(8):
                        acc += (((word >> (4 * j)) & 15) - z) * float(x_perm[k0 + j])
            y[o] += float(sc[tile, g, o % 16]) * acc
    return y


@pytest.mark.parametrize("gs,in_f,out_f", [(32, 96, 16), (64, 256, 24), (128, 1408, 8)])
def test_repack_is_exact(l2, orc, gs, in_f, out_f):
    rng = np.random.default_rng(in_f)
    qweight, qzeros, scales, g_index = random_qlinear(rng, in_f, out_f, gs)
    order = rng.permutation(out_f).astype(np.int32)
    for rows in (None, order):
        pq = C.POINTER(C.c_uint32)()
        tiles, uw = C.c_int(0), C.c_int(0)
        l2.check(l2.lib.l2_debug_repack(in_f, out_f, gs, l2._lib.as_i32p(qweight), l2._lib.as_i32p(qzeros), l2._lib.as_f32p(scales),
                                        l2._lib.as_i32p(rows) if rows is not None else None,
                                        C.byref(pq), C.byref(tiles), C.byref(uw)))
        g = in_f // gs
        assert tiles.value == (out_f + 15) // 16
        assert uw.value == 64 * (gs // 32) + 20
        rec = np.ctypeslib.as_array(pq, shape=(tiles.value * g * uw.value,)).copy()
        l2.lib.l2_host_free(pq)
        qw = rec.reshape(-1, uw.value)[:, :64 * (gs // 32)].ravel()
        x = rng.standard_normal(in_f).astype(np.float32)
        y = emulate_device_gemv(rec, tiles.value, in_f, out_f, gs, x[g_index])
        want = orc.qlinear_matvec(qweight, qzeros, scales, g_index, gs, x).astype(np.float64)
        if rows is not None:
            want = want[rows]
        np.testing.assert_allclose(y, want, rtol=2e-5, atol=2e-5)
        # the nibbles are carried over bit for bit: the multiset of words is unchanged, padding rows are zero
        assert np.array_equal(np.sort(qw[qw != 0]), np.sort(qweight.view(np.uint32)[qweight.view(np.uint32) != 0]))


def test_repack_rejects_bad_arguments(l2):
    rng = np.random.default_rng(0)
    qweight, qzeros, scales, g_index = random_qlinear(rng, 64, 8, 32)
    bad = np.zeros(8, np.int32)
    pq, gp, uw = C.POINTER(C.c_uint32)(), C.c_int(0), C.c_int(0)
    rc = l2.lib.l2_debug_repack(64, 8, 32, l2._lib.as_i32p(qweight), l2._lib.as_i32p(qzeros), l2._lib.as_f32p(scales),
                                l2._lib.as_i32p(bad), C.byref(pq), C.byref(gp), C.byref(uw))
    assert rc == -1 and b"permutation" in l2.lib.l2_last_error()


def write_tokenizer(path, vocab):
    with open(path, "wb") as f:
        f.write(struct.pack("i", max(len(v.encode()) for v, _ in vocab)))
        for s, score in vocab:
            b = s.encode()
            f.write(struct.pack("fi", score, len(b)))
            f.write(b)


def test_tokenizer_merges_by_best_score(l2, tmp_path):
    # 260 filler entries so that str_lookup's "index >= 260 first" rule is exercised
    vocab = [("<f%d>" % i, 0.0) for i in range(260)]
    vocab[5] = ("a", -1.0)  # shadowed by the later "a"
    vocab += [(" ", -1.0), ("a", -2.0), ("b", -3.0), ("ab", -0.5), (" a", -0.2), (" ab", -0.1), ("abb", -4.0), ("é", -1.0)]
    path = tmp_path / "tok.bin"
    write_tokenizer(path, vocab)
    t = l2.Tokenizer(path, vocab_size=len(vocab))
    base = 260
    assert t.bpe_encode("a") == [base + 1]          # not entry 5
    assert t.bpe_encode(" ab") == [base + 5]        # " "+"a" (-0.2) first, then " a"+"b" -> " ab"
    assert t.bpe_encode("abb") == [base + 6]  # "ab" first, then "ab"+"b" = "abb" (-4.0 > -1e10) still merges
    assert t.bpe_encode("é a") == [base + 7, base + 4]
    assert t.bpe_encode("") == []
    with pytest.raises(l2.L2Error):
        t.bpe_encode("z")
    assert t.piece(1, base + 4) == "a"    # leading space stripped after START
    assert t.piece(2, base + 4) == " a"


def test_tokenizer_abb_merge_rule(l2, tmp_path):
    # merging continues while any adjacent pair is in the vocabulary (src/tokenizer.rs:63-107)
    vocab = [("<f%d>" % i, 0.0) for i in range(260)] + [("a", 0.0), ("b", 0.0), ("ab", 1.0), ("abb", 0.5)]
    path = tmp_path / "tok2.bin"
    write_tokenizer(path, vocab)
    t = l2.Tokenizer(path, vocab_size=len(vocab))
    assert t.bpe_encode("abb") == [263]


def test_reference_tokenizer_file_if_present(l2):
    # the reference checkout, when it sits next to this repository
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "tokenizer.bin")
    if not os.path.exists(path):
        pytest.skip("reference tokenizer.bin not available")
    t = l2.Tokenizer(path)
    ids = t.bpe_encode(" The only thing")
    assert len(ids) >= 3 and all(0 <= i < 32000 for i in ids)
    assert "".join(t.piece(1 if k == 0 else 0, i) for k, i in enumerate(ids)) == "The only thing"


def test_no_gpu_fails_loudly(l2):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    cfg = tiny_config(l2)
    with pytest.raises(l2.L2Error) as e:
        l2.LlamaModel.synthetic(cfg, 1)
    assert e.value.code == -3 and "no CPU fallback" in str(e.value)
    rng = np.random.default_rng(0)
    with pytest.raises(l2.L2Error):
        l2.QLinear(*random_qlinear(rng, 64, 8, 32), group_size=32)


def test_random_matches_oracle(l2, orc):
    a, b = l2.Random(12345), C.c_uint64(12345)
    for _ in range(10):
        assert a.random_u32() == orc.lib().orc_random_u32(C.byref(b))
    assert a.random() == orc.lib().orc_random_f32(C.byref(b))


def test_bench_workloads_and_prefill_report():
    """bench.py's workload table and the prefill roofline arithmetic (no GPU: a stand-in for the model handle)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.WORKLOADS["7b"] == ("7B", 128, 32, 256) and bench.WORKLOADS["70b"] == ("70B", 64, 64, 256)
    assert bench.WORKLOADS["70b-long"][2] + bench.WORKLOADS["70b-long"][3] == 2048  # the prompt and the decoded tokens fill the cache

    class Cfg:
        dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size = 4096, 11008, 32, 32, 32, 32000

    class Model:
        decode_bytes = 3991027712

    r = bench.prefill_report(Model, Cfg, 30, 4.4, False, 6549.4, 1642.0, "measured")
    assert r["weight_passes"] == 1 and r["executed_mma_inflation"] == 3
    flops = 2.0 * 32 * (4 * 4096 * 4096 + 3 * 4096 * 11008) * 30
    assert abs(r["tflops"] - flops / 4.4e-3 / 1e12) < 1e-6
    qbytes = 3991027712 - 4.0 * 32000 * 4096 - 4.0 * 65 * 4096
    assert abs(r["weight_gbs"] - qbytes / 4.4e-3 / 1e9) < 1e-6
    # 130 positions need three passes of up to 64; under NCCL tensor parallelism every position is a pass
    assert bench.prefill_report(Model, Cfg, 130, 10.0, False, 6549.4, 1642.0, "measured")["weight_passes"] == 3
    assert bench.prefill_report(Model, Cfg, 130, 10.0, True, 6549.4, 1642.0, "measured")["weight_passes"] == 130
    # a vocabulary-parallel rank streams a slice of the classifier: its QLinear bytes are what is left of its decode bytes
    half = bench.prefill_report(Model, Cfg, 30, 4.4, False, 6549.4, 1642.0, "measured", cls_rows=16000)
    assert half["weight_gbs"] > r["weight_gbs"]
