"""Parity of the CUDA RoPE + cache append + GQA attention kernel (through the C ABI, on device
buffers) with the oracle's rope + multihead_attention (src/models.rs:100-176)."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu
HS = 128


def oracle_attention(orc, q, k, v, kc, vc, pos, n_heads, n_kv_heads):
    L = orc.lib()
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    q, k, kc, vc = q.copy(), k.copy(), kc.copy(), vc.copy()
    L.orc_rope(f(q), f(k), pos, n_heads, n_kv_heads, HS)
    kc[pos] = k.reshape(n_kv_heads, HS)
    vc[pos] = v.reshape(n_kv_heads, HS)
    out = np.zeros(n_heads * HS, np.float32)
    L.orc_attention(f(out), f(q), f(vc), f(kc), pos, n_heads, n_kv_heads, HS)
    return out, kc, vc


def run_gpu(l2, q, k, v, kc, vc, pos, n_heads, n_kv_heads, seq):
    import torch
    cos, sin = np.zeros((seq, HS // 2), np.float32), np.zeros((seq, HS // 2), np.float32)
    l2.check(l2.lib.l2_rope_table(seq, l2._lib.as_f32p(cos), l2._lib.as_f32p(sin)))
    d = lambda a: torch.from_numpy(a).cuda()
    dq, dk, dv, dkc, dvc, dcos, dsin = map(d, (q, k, v, kc, vc, cos, sin))
    out = torch.zeros(n_heads * HS, device="cuda")
    ws = torch.empty(l2.lib.l2_attention_workspace_bytes(n_heads, n_kv_heads), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    l2.check(l2.lib.l2_attention_decode_dev(n_heads, n_kv_heads, pos, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dkc.data_ptr(),
                                            dvc.data_ptr(), dcos.data_ptr(), dsin.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), st))
    torch.cuda.synchronize()
    return out.cpu().numpy(), dkc.cpu().numpy(), dvc.cpu().numpy()


@pytest.mark.parametrize("n_heads,n_kv_heads", [(2, 2), (4, 2), (8, 2), (32, 32), (64, 8)])
@pytest.mark.parametrize("pos", [0, 1, 63, 64, 300, 1023])
def test_attention_matches_oracle(l2, orc, n_heads, n_kv_heads, pos):
    seq = 1024
    rng = np.random.default_rng(n_heads * 1000 + pos)
    q = rng.standard_normal(n_heads * HS).astype(np.float32)
    k = rng.standard_normal(n_kv_heads * HS).astype(np.float32)
    v = rng.standard_normal(n_kv_heads * HS).astype(np.float32)
    kc = np.zeros((seq, n_kv_heads, HS), np.float32)
    vc = np.zeros((seq, n_kv_heads, HS), np.float32)
    kc[:pos] = rng.standard_normal((pos, n_kv_heads, HS)) * 0.5
    vc[:pos] = rng.standard_normal((pos, n_kv_heads, HS))
    want, wkc, wvc = oracle_attention(orc, q, k, v, kc, vc, pos, n_heads, n_kv_heads)
    got, gkc, gvc = run_gpu(l2, q, k, v, kc, vc, pos, n_heads, n_kv_heads, seq)
    assert_close(got, want, rel=1e-4, abs_=1e-5, what="attention output")
    assert_close(gkc[pos], wkc[pos], rel=1e-6, abs_=1e-6, what="appended key (RoPE)")
    assert np.array_equal(gvc[pos], wvc[pos])
    assert np.array_equal(gkc[:pos], kc[:pos]) and not gkc[pos + 1:].any()  # nothing else is touched


def test_attention_bad_arguments(l2):
    rc = l2.lib.l2_attention_decode_dev(6, 4, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1 << 30, None)
    assert rc == -1 and b"divide" in l2.lib.l2_last_error()
    rc = l2.lib.l2_attention_decode_dev(4, 4, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 16, None)
    assert rc == -1 and b"workspace" in l2.lib.l2_last_error()
