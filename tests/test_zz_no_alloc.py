"""The attention entry point for callers that cannot allocate device memory
(l2_attention_decode_noalloc) against the workspace-taking entry point (l2_attention_decode_dev).

Such callers -- a serving loop whose device memory all belongs to its own pool, a plug-in that is
only handed pointers into that pool, code holding a lock under which the CUDA allocator must not
run -- pass inputs and outputs only; the kernel's split-sequence scratch is a fixed array inside the
library.  The array is shared by all calls and keeps the previous call's contents, so this test
makes two different calls in a row and checks both.  It is collected last on purpose."""
import numpy as np
import pytest

from conftest import assert_close
from test_gpu_attention import oracle_attention

pytestmark = pytest.mark.gpu
HS = 128


def _inputs(rng, n_heads, n_kv_heads, pos, seq):
    q = rng.standard_normal(n_heads * HS).astype(np.float32)
    k = rng.standard_normal(n_kv_heads * HS).astype(np.float32)
    v = rng.standard_normal(n_kv_heads * HS).astype(np.float32)
    kc = np.zeros((seq, n_kv_heads, HS), np.float32)
    vc = np.zeros((seq, n_kv_heads, HS), np.float32)
    kc[:pos] = rng.standard_normal((pos, n_kv_heads, HS)) * 0.5
    vc[:pos] = rng.standard_normal((pos, n_kv_heads, HS))
    return q, k, v, kc, vc


def test_noalloc_matches_workspace_entry_point_twice(l2, orc):
    import torch
    seq = 1024
    cos, sin = np.zeros((seq, HS // 2), np.float32), np.zeros((seq, HS // 2), np.float32)
    l2.check(l2.lib.l2_rope_table(seq, l2._lib.as_f32p(cos), l2._lib.as_f32p(sin)))
    dcos, dsin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    st = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(2024)
    # two calls in a row with different shapes and split counts: the second must not see the first's leftovers
    for n_heads, n_kv_heads, pos in [(64, 8, 1000), (32, 32, 130), (4, 2, 0)]:
        q, k, v, kc, vc = _inputs(rng, n_heads, n_kv_heads, pos, seq)
        d = lambda a: torch.from_numpy(a).cuda()
        outs, caches = [], []
        for noalloc in (False, True):
            dq, dk, dv, dkc, dvc = map(d, (q, k, v, kc, vc))
            out = torch.zeros(n_heads * HS, device="cuda")
            if noalloc:
                call = lambda kcache, vcache, o: l2.lib.l2_attention_decode_noalloc(
                    n_heads, n_kv_heads, pos, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), kcache.data_ptr(), vcache.data_ptr(),
                    dcos.data_ptr(), dsin.data_ptr(), o.data_ptr(), st)
                # a warm-up call on scratch copies first (the very first call on a device looks the array's address up and
                # may load the module), then the device's free memory as the driver reports it must not move across the
                # checked call: torch's own counters would not see a cudaMalloc made inside the library
                l2.check(call(dkc.clone(), dvc.clone(), torch.zeros_like(out)))
                torch.cuda.synchronize()
                free_before = torch.cuda.mem_get_info()[0]
                rc = call(dkc, dvc, out)
                torch.cuda.synchronize()
                assert torch.cuda.mem_get_info()[0] == free_before
            else:
                ws = torch.empty(l2.lib.l2_attention_workspace_bytes(n_heads, n_kv_heads), dtype=torch.uint8, device="cuda")
                rc = l2.lib.l2_attention_decode_dev(n_heads, n_kv_heads, pos, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dkc.data_ptr(),
                                                    dvc.data_ptr(), dcos.data_ptr(), dsin.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), st)
            l2.check(rc)
            torch.cuda.synchronize()
            outs.append(out.cpu().numpy())
            caches.append((dkc.cpu().numpy(), dvc.cpu().numpy()))
        # same kernel, same split geometry, fixed summation order: the tolerance of the attention tests, and in fact equal
        np.testing.assert_allclose(outs[1], outs[0], rtol=1e-4, atol=1e-5)
        assert np.array_equal(outs[1], outs[0])
        assert np.array_equal(caches[1][0], caches[0][0]) and np.array_equal(caches[1][1], caches[0][1])
        assert np.abs(outs[1]).max() > 0
        # and against the CPU oracle's rope + multihead_attention (src/models.rs:100-176), the tolerance of the attention tests
        want, want_kc, want_vc = oracle_attention(orc, q, k, v, kc, vc, pos, n_heads, n_kv_heads)
        assert_close(outs[1], want, rel=1e-4, abs_=1e-5, what="no-alloc attention vs oracle, %d heads pos %d" % (n_heads, pos))
        assert_close(caches[1][0][pos], want_kc[pos], rel=1e-6, abs_=1e-6, what="appended key (RoPE)")
        assert np.array_equal(caches[1][1][pos], want_vc[pos])


def test_noalloc_rejects_shapes_beyond_the_builtin_scratch(l2):
    rc = l2.lib.l2_attention_decode_noalloc(128, 128, 0, 1, 1, 1, 1, 1, 1, 1, 1, None)
    assert rc == -1
    msg = l2.lib.l2_last_error()
    assert b"exceed the built-in scratch" in msg and b"l2_attention_decode_dev" in msg
