"""One rank of the tensor-parallel parity check; run under torch.distributed.run with N ranks.
Each rank owns 1/N of every matrix's rows on its own GPU and must reproduce the CPU oracle's
per-step logits and greedy stream, bit-identically across ranks."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "llama2.rs_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))
import llama2_rs as l2  # noqa: E402
import oracle as orc  # noqa: E402
from conftest import assert_close, tiny_config  # noqa: E402


def run_case(cfg, rank, world, steps, n_prompt, seed, direct, ties=False):
    payload = l2.synth_fill(cfg, seed)
    V, D = cfg.vocab_size, cfg.dim
    if ties:
        # The classifier is the last V x D floats of the file (src/gptq.rs:65).  Eight rows below the middle of the vocabulary
        # are copied onto the eight rows above it and both sets scaled up, so that the largest logit is often an exact tie
        # between a row of one rank's slice and a row of the next rank's: the last maximum must win (src/util.rs:39-46).
        wcls = payload[-V * D * 4:].view(np.float32).reshape(V, D)
        wcls[V // 2 - 8:V // 2] *= np.float32(4.0)
        wcls[V // 2:V // 2 + 8] = wcls[V // 2 - 8:V // 2]
    gpu = l2.LlamaModel.from_blob(cfg, payload, device=rank, tp=(rank, world))
    if direct:
        # peer memory: every rank maps every other rank's activation pool; the token kernel stores into all of them
        handles = [None] * world
        dist.all_gather_object(handles, gpu.tp_pool_handle())
        for r in range(world):
            gpu.tp_pool_attach(r, handles[r])
    else:
        ids = [l2.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        gpu.tp_connect(ids[0])
    if ties:
        # (on the model's first run state: under peer memory only that one runs as the token kernel)
        # temperature sampling: softmax over all ranks' logits, CDF walk in index order, one draw per token (src/util.rs:102-113)
        st = l2.RunState(gpu)
        L = orc.lib()
        import ctypes as C
        agree = 0
        for sd in range(1, 21):
            rnd = l2.Random(sd)
            nxt, logits = l2.decode_step(gpu, st, 7, 0, temperature=0.8, random=rnd, want_logits=True)
            p = (logits / np.float32(0.8)).astype(np.float32)
            L.orc_softmax(p.ctypes.data_as(C.POINTER(C.c_float)), p.size)
            sv = C.c_uint64(sd)
            want_tok = L.orc_sample(C.byref(sv), p.ctypes.data_as(C.POINTER(C.c_float)), p.size)
            assert rnd.seed == sv.value
            agree += int(nxt == want_tok)
            picks = [None] * world
            dist.all_gather_object(picks, int(nxt))
            assert len(set(picks)) == 1, "ranks sampled different tokens: %s" % picks
        assert agree >= 19, "sampled tokens differ from the oracle's in %d of 20 draws" % (20 - agree)
        st.close()
    prompt = np.random.default_rng(seed).integers(0, cfg.vocab_size, n_prompt).astype(np.int32)
    got = l2.generate_ids(gpu, prompt, steps, trace_logits=True)
    fast = l2.generate_ids(gpu, prompt, steps)
    want = orc.Model(cfg, payload).generate_ids(prompt, steps, trace_logits=True)
    assert got["pos0"] == want["pos0"]
    assert_close(got["logits"], want["logits"], what="rank %d logits" % rank)
    assert np.array_equal(got["tokens"], want["tokens"]) and np.array_equal(fast["tokens"], want["tokens"])
    # bit-identical on every rank: nothing is summed across ranks
    mine = torch.from_numpy(got["logits"].copy())
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(mine, ref), "rank %d differs from rank 0" % rank
    if ties:
        free = got["tokens"][n_prompt - got["pos0"]:]  # tokens chosen by argmax, not forced by the prompt
        assert not ((free >= V // 2 - 8) & (free < V // 2)).any(), "the first of two equal maxima was chosen"
        assert ((free >= V // 2) & (free < V // 2 + 8)).any(), "the tie case never occurred: the test checks nothing"
    gpu.close()


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(rank)
    cfg = tiny_config(l2, group_size=64, n_kv_heads=2, dim=512, hidden=1024, n_layers=2)
    cfg.n_heads, cfg.n_kv_heads = 4, world if world in (1, 2, 4) else 4
    big = l2.preset_config("70B", 64)  # the real 70B projection shapes and GQA, two layers, small vocabulary
    big.n_layers, big.vocab_size, big.seq_len = 2, 2048, 128
    for direct in (False, True):  # NCCL all-gathers between per-operator kernels; stores into peer memory from the token kernel
        run_case(cfg, rank, world, steps=40, n_prompt=21, seed=11, direct=direct)
        run_case(big, rank, world, steps=24, n_prompt=9, seed=12, direct=direct)
        run_case(cfg, rank, world, steps=48, n_prompt=5, seed=13, direct=direct, ties=True)  # classifier split over the ranks (peer memory) or replicated (NCCL)
        dist.barrier()
        if rank == 0:
            print("tp parity ok (%s)" % ("peer memory" if direct else "nccl"), flush=True)
    dist.barrier()
    if rank == 0:
        print("tp parity ok on %d ranks" % world)


if __name__ == "__main__":
    main()
