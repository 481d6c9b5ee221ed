"""The benchmark configurations at full depth against the CPU oracle (per-step logits within 1e-2 relative /
1e-3 absolute, identical greedy stream for at least 64 free-running tokens), the text-level generate(), and a
bounded device-side wait that really runs out.

The oracle decodes the 7B model at 10-20 tokens per second on a GPU box's host cores, so the 7B case costs seconds;
13B runs a shorter stream; 70B (41 GB of synthetic weights, minutes of CPU time) runs only with L2_TEST_70B=1."""
import os
import struct

import numpy as np
import pytest

from conftest import assert_close, tiny_config

pytestmark = pytest.mark.gpu
WEIGHT_SEED, PROMPT_SEED = 20240, 7  # the seeds of the benchmark harness


def run_config(l2, orc, name, gs, n_prompt, n_free):
    cfg = l2.preset_config(name, gs)
    payload = l2.synth_fill(cfg, WEIGHT_SEED)
    gpu = l2.LlamaModel.from_blob(cfg, payload)
    cpu = orc.Model(cfg, payload)
    prompt = np.random.default_rng(PROMPT_SEED).integers(0, cfg.vocab_size, n_prompt).astype(np.int32)
    steps = n_prompt + n_free
    want = cpu.generate_ids(prompt, steps, trace_logits=True)   # the prompt goes through the 64/32/16/8/4/2 ladder
    got = l2.generate_ids(gpu, prompt, steps, trace_logits=True)
    assert got["pos0"] == want["pos0"]
    assert_close(got["logits"], want["logits"], what="%s per-step logits" % name)
    free = n_prompt - got["pos0"]  # positions of the B=1 loop that are still teacher-forced
    assert np.array_equal(got["tokens"], want["tokens"])
    assert len(got["tokens"]) - free >= n_free
    fast = l2.generate_ids(gpu, prompt, steps)  # the device-resident loop
    assert np.array_equal(fast["tokens"], want["tokens"])
    gpu.close()


def test_config0_7b_g128_full_depth(l2, orc):
    # Llama2-7B GPTQ 4-bit g128 act-order, seed 20240, 32-token prompt through batched prefill, 64 free-running greedy tokens
    run_config(l2, orc, "7B", 128, 32, 64)


def test_config2_13b_g128_full_depth(l2, orc):
    # Llama2-13B g128: 128-token prompt through batched prefill, then 16 greedy tokens (the oracle runs ~5 tokens per second)
    run_config(l2, orc, "13B", 128, 128, 16)


@pytest.mark.skipif(not os.environ.get("L2_TEST_70B"), reason="70B at full depth takes minutes of CPU time: set L2_TEST_70B=1")
def test_config3_70b_g64_full_depth(l2, orc):
    run_config(l2, orc, "70B", 64, 64, 8)


def write_tokenizer(path, vocab):
    """tokenizer.bin as the reference reads it (src/tokenizer.rs:22-44): i32 max length, then per token f32 score, i32 length, bytes."""
    with open(path, "wb") as f:
        f.write(struct.pack("i", max(len(v.encode()) for v, _ in vocab)))
        for s, score in vocab:
            b = s.encode()
            f.write(struct.pack("fi", score, len(b)))
            f.write(b)


def test_text_generate_matches_generate_ids(l2, tmp_path):
    # generate(model, tokenizer, prompt, steps, random, temperature) (src/inference.rs:49-57, src/lib.rs:111-131):
    # encodes " " + prompt, runs the id-level loop and maps ids to pieces with the leading-space rule after START
    cfg = tiny_config(l2, group_size=64, n_kv_heads=1)
    letters = " Theonlytigabcdfmprsuvw"
    vocab = [("<f%d>" % i, 0.0) for i in range(260)] + [(ch, -10.0 - i) for i, ch in enumerate(letters)]
    vocab += [(" T", -1.0), ("he", -1.5), (" The", -0.5), (" o", -2.0), ("nl", -2.5), (" on", -1.8), ("ly", -2.2), (" only", -0.7), (" th", -1.2), ("in", -1.4), ("ing", -0.9), (" thing", -0.6)]
    vocab += [("<p%d>" % i, -50.0) for i in range(cfg.vocab_size - len(vocab))]
    path = tmp_path / "tok.bin"
    write_tokenizer(path, vocab)
    tok = l2.Tokenizer(path, vocab_size=cfg.vocab_size)
    model = l2.LlamaModel.from_blob(cfg, l2.synth_fill(cfg, 3))
    prompt = " The only thing"
    ids = tok.bpe_encode(" " + prompt.strip())
    assert len(ids) >= 3 and all(0 <= i < cfg.vocab_size for i in ids)
    steps = 40
    ms, pieces = l2.generate(model, tok, prompt, steps, l2.Random(1), 0.0)
    r = l2.generate_ids(model, ids, steps, l2.Random(1), 0.0, use_prefill=model.prefill())
    assert isinstance(ms, int) and len(pieces) == len(r["tokens"]) == steps - r["pos0"]
    token = l2.START if r["pos0"] == 0 else ids[r["pos0"] - 1]
    for piece, nxt in zip(pieces, r["tokens"]):
        assert piece == tok.piece(token, int(nxt))
        token = int(nxt)
    # the prompt comes back as text (teacher forcing), with the space after START stripped when the loop starts at position 0
    n_forced = len(ids) - r["pos0"]
    assert "".join(pieces[:n_forced]) == "".join(tok.piece(ids[r["pos0"] + i - 1] if r["pos0"] + i > 0 else l2.START, ids[r["pos0"] + i]) for i in range(n_forced))
    # sampling with a temperature is reproducible from the seed
    a = l2.generate(model, tok, prompt, steps, l2.Random(5), 0.8)[1]
    b = l2.generate(model, tok, prompt, steps, l2.Random(5), 0.8)[1]
    assert a == b


def test_bounded_wait_runs_out_and_the_device_stays_usable(l2, orc):
    # A tensor-parallel rank whose peer never launches: the token kernel polls for the peer's part of the attention
    # output, which nothing writes; after 2^12 polls it gives up by itself, the call returns L2_ESTATUS, the state
    # refuses further calls until it is reset, and the device keeps working.  The peer's pool is a plain buffer of
    # this process (nothing waits on this rank either: no second kernel is involved).
    import torch
    cfg = tiny_config(l2, group_size=64, n_kv_heads=2, dim=512, hidden=1024)
    cfg.n_heads = 4
    payload = l2.synth_fill(cfg, 5)
    m = l2.LlamaModel.from_blob(cfg, payload, tp=(0, 2), poll_limit_log2=12)
    m.tp_pool_handle()
    peer_pool = torch.zeros(m.tp_pool_bytes(), dtype=torch.uint8, device="cuda")
    m.tp_pool_attach_ptr(1, peer_pool.data_ptr())
    st = l2.RunState(m)
    with pytest.raises(l2.L2Error) as e:
        l2.decode_step(m, st, 5, 0)
    assert e.value.code == -6 and "device status" in str(e.value)
    with pytest.raises(l2.L2Error) as e:  # latched: no forward until the state is reset
        l2.decode_step(m, st, 5, 0)
    assert e.value.code == -6 and "l2_state_reset" in str(e.value)
    st.reset()
    with pytest.raises(l2.L2Error) as e:  # the peer is still absent: the wait runs out again, cleanly
        l2.decode_step(m, st, 5, 0)
    assert e.value.code == -6 and "device status" in str(e.value)
    st.close()
    with pytest.raises(l2.L2Error) as e:  # the device-resident loop (no host round trip per token) reports it as well
        l2.generate_ids(m, [], 4)
    assert e.value.code == -6
    m.close()
    # the context is intact: a single-GPU model of the same shape matches the oracle afterwards
    gpu = l2.LlamaModel.from_blob(cfg, payload)
    want = orc.Model(cfg, payload).generate_ids([3, 4, 5], 24, trace_logits=True)
    got = l2.generate_ids(gpu, [3, 4, 5], 24, trace_logits=True)
    assert_close(got["logits"], want["logits"], what="logits after a timed-out launch")
    assert np.array_equal(got["tokens"], want["tokens"])
