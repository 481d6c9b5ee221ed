"""The tensor-parallel data flow on CPU ranks (gloo, world size 2): every projection split by
output rows with l2_tp_rows, vectors re-assembled by all-gather.  Uses the oracle's QLinear on row
slices, so it checks the sharding scheme and the w1/w3 row re-ordering, not the CUDA kernels."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, random_qlinear


def _worker(rank, world, port, out):
    sys.path.insert(0, os.path.join(ROOT, "llama2.rs_b200"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch
    import torch.distributed as dist
    import llama2_rs as l2
    import oracle as orc
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    D, H, gs = 256, 512, 64
    rng = np.random.default_rng(5)  # the same weights on every rank
    w1, w3, w2 = random_qlinear(rng, D, H, gs), random_qlinear(rng, D, H, gs), random_qlinear(rng, H, D, gs)
    x = rng.standard_normal(D).astype(np.float32)

    def rows(total):
        r0, n = C.c_int(0), C.c_int(0)
        l2.check(l2.lib.l2_tp_rows(total, rank, world, C.byref(r0), C.byref(n)))
        return r0.value, n.value

    def sliced(q, sel):  # QLinear restricted to the output rows `sel` (whole blocks of 8 rows)
        qweight, qzeros, scales, g_index = q
        nib = np.stack([(qzeros.view(np.uint32)[sel // 8] >> (4 * (sel % 8)).astype(np.uint32)[:, None]) & 15])[0]
        z = np.zeros((len(sel) // 8, qzeros.shape[1]), np.uint32)
        for j in range(len(sel)):
            z[j // 8] |= nib[j].astype(np.uint32) << np.uint32(4 * (j % 8))
        return qweight[sel], z.view(np.int32), scales[sel], g_index

    def gather(part, total):
        parts = [torch.zeros(total // world) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(part.astype(np.float32)))
        return torch.cat(parts).numpy()

    # w1/w3 rows are stored in w2's K order, so a rank's slice of the SwiGLU output is a contiguous
    # slice of w2's permuted input
    order = w2[3]
    r0, n = rows(H)
    sel = order[r0:r0 + n]
    a = orc.qlinear_matvec(*sliced(w1, sel), gs, x)
    b = orc.qlinear_matvec(*sliced(w3, sel), gs, x)
    hb_perm = gather((a * (1.0 / (1.0 + np.exp(-a)))) * b, H)      # all-gather of the SwiGLU output
    hb = np.zeros(H, np.float32)
    hb[order] = hb_perm                                               # back to natural order for the oracle's own gather
    r0, n = rows(D)
    y = gather(orc.qlinear_matvec(*sliced(w2, np.arange(r0, r0 + n)), gs, hb), D)
    # single-process reference
    fa, fb = orc.qlinear_matvec(*w1, gs, x), orc.qlinear_matvec(*w3, gs, x)
    want = orc.qlinear_matvec(*w2, gs, ((fa * (1.0 / (1.0 + np.exp(-fa)))) * fb).astype(np.float32))
    out.put((rank, bool(np.array_equal(y, want)), float(np.abs(y - want).max())))
    dist.destroy_process_group()


def test_row_split_all_gather_equals_single_process():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29533, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
    assert all(ok for _, ok, _ in res), res


def test_tp_rows_rejects_ragged_splits(l2):
    r0, n = C.c_int(0), C.c_int(0)
    assert l2.lib.l2_tp_rows(8192, 3, 8, C.byref(r0), C.byref(n)) == 0 and (r0.value, n.value) == (3072, 1024)
    assert l2.lib.l2_tp_rows(1000, 0, 8, C.byref(r0), C.byref(n)) == -1


def test_splits_of_the_70b_shapes_at_every_world_size(l2):
    """What the tensor-parallel kernels assume about a rank's share: whole 16-row tiles of every projection, heads and kv heads
    divided evenly, slices that are contiguous and cover the matrix; and the vocabulary slices of the classifier
    (rows V r / T .. V (r + 1) / T) cover 0..V without overlap."""
    cfg = l2.preset_config("70B", 64)
    kv = cfg.dim * cfg.n_kv_heads // cfg.n_heads
    for world in (1, 2, 4, 8):
        assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0
        for total in (cfg.dim, kv, cfg.hidden_dim):
            end = 0
            for rank in range(world):
                r0, n = C.c_int(0), C.c_int(0)
                assert l2.lib.l2_tp_rows(total, rank, world, C.byref(r0), C.byref(n)) == 0
                assert r0.value == end and n.value == total // world and n.value % 16 == 0 and r0.value % 16 == 0
                end = r0.value + n.value
            assert end == total
        edges = [cfg.vocab_size * r // world for r in range(world + 1)]
        assert edges[0] == 0 and edges[-1] == cfg.vocab_size and all(b > a for a, b in zip(edges, edges[1:]))
        # a rank's kv heads are whole heads of 128 values inside the full-width cache row
        assert (kv // world) % 128 == 0
