"""The .bin layout (export.py:83-119, src/gptq.rs:34-84): synthetic writer -> loader round trip,
value distributions of the synthetic checkpoint, header rules."""
import os
import struct

import numpy as np
import pytest

from conftest import tiny_config


def qlinear_fields(payload, off_words, in_f, out_f, gs):
    w = payload.view(np.uint32)
    g = in_f // gs
    n = [out_f * in_f // 8, (out_f // 8) * g, out_f * g, in_f]
    o = off_words
    qweight = w[o:o + n[0]].reshape(out_f, in_f // 8); o += n[0]
    qzeros = w[o:o + n[1]].reshape(out_f // 8, g); o += n[1]
    scales = w[o:o + n[2]].view(np.float32).reshape(out_f, g); o += n[2]
    g_index = w[o:o + n[3]].view(np.int32); o += n[3]
    return qweight, qzeros, scales, g_index, o


def test_preset_sizes(l2):
    want = {("7B", 128): 4520919044, ("13B", 128): 8110493700, ("70B", 64): 41166864388}
    for (name, gs), size in want.items():
        c = l2.preset_config(name, gs)
        assert l2.checkpoint_bytes(c) == size
    c = l2.preset_config("70B", 64)
    assert (c.n_heads, c.n_kv_heads) == (64, 8)
    with pytest.raises(l2.L2Error):
        l2.preset_config("30B", 128)


def test_file_round_trip(l2, orc, tmp_path):
    cfg = tiny_config(l2, group_size=32, n_kv_heads=1)
    path = tmp_path / "tiny.bin"
    l2.synth_write_file(cfg, 5, path)
    payload = l2.synth_fill(cfg, 5)
    raw = np.fromfile(path, np.uint8)
    assert raw.size == 28 + l2.checkpoint_bytes(cfg)
    header = struct.unpack("7i", raw[:28].tobytes())
    # export.py:83-87: n_kv_heads repeats n_heads, vocab is written negative
    assert header == (cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_heads, -cfg.vocab_size, cfg.seq_len)
    assert np.array_equal(raw[28:], payload)
    # the oracle's loader (Config::load + mmap cast) reads it with the feature values supplied
    m = orc.Model.open(path, attn_groups=2, group_size=32)
    assert m.cfg.n_kv_heads == 1 and m.cfg.vocab_size == cfg.vocab_size
    with pytest.raises(ValueError):
        orc.Model.open(path, attn_groups=1, group_size=32)  # wrong feature set -> size assert fails


def test_synthetic_distributions(l2):
    cfg = tiny_config(l2, group_size=64, n_kv_heads=2)
    p = l2.synth_fill(cfg, 20240)
    f = p.view(np.float32)
    D, V, L = cfg.dim, cfg.vocab_size, cfg.n_layers
    assert f[0] == np.float32(1e-5)
    emb = f[1:1 + V * D]
    assert abs(emb.mean()) < 2e-3 and abs(emb.std() - 0.02) < 1e-3
    att = f[1 + V * D:1 + V * D + L * D]
    assert abs(att.mean() - 1.0) < 5e-3 and abs(att.std() - 0.02) < 3e-3
    qweight, qzeros, scales, g_index, _ = qlinear_fields(p, 1 + V * D + L * D, D, D, 64)
    nib = np.stack([(qweight >> np.uint32(4 * j)) & 15 for j in range(8)])
    counts = np.bincount(nib.ravel(), minlength=16)
    assert counts.min() > 0.9 * nib.size / 16 and counts.max() < 1.1 * nib.size / 16
    znib = np.stack([(qzeros >> np.uint32(4 * j)) & 15 for j in range(8)])
    assert znib.min() == 6 and znib.max() == 9
    assert scales.min() >= 0.002 and scales.max() <= 0.02 and abs(scales.mean() - 0.011) < 1e-3
    # g_index = stable argsort of a group assignment: a permutation, ascending inside every group
    assert np.array_equal(np.sort(g_index), np.arange(D))
    assert np.all(np.diff(g_index.reshape(-1, 64), axis=1) > 0)
    assert not np.array_equal(g_index, np.arange(D))
    # the same seed gives the same bytes, another seed does not
    assert np.array_equal(p, l2.synth_fill(cfg, 20240))
    assert not np.array_equal(p, l2.synth_fill(cfg, 20241))


def test_bad_sizes_are_errors(l2):
    cfg = tiny_config(l2)
    buf = np.zeros(100, np.uint8)
    import ctypes as C
    assert l2.lib.l2_synth_fill(C.byref(cfg), 1, buf.ctypes.data_as(C.c_void_p), 100, 1) == -2
    assert b"100 bytes" in l2.lib.l2_last_error()
    bad = tiny_config(l2, group_size=48)
    assert l2.checkpoint_bytes(bad) > 0
    with pytest.raises(l2.L2Error):
        l2.synth_fill(bad, 1)
