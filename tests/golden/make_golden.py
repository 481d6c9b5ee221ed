"""Writes tests/golden/tiny_generate.npz: prompt, greedy tokens and per-step logits of the CPU
oracle on the seeded tiny checkpoint.  The reference (nightly Rust) cannot be run here, so these
vectors pin the oracle against regressions and give the GPU tests a fixture that does not need
the oracle at run time.  Usage: python tests/golden/make_golden.py"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "llama2.rs_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import llama2_rs as l2  # noqa: E402
import oracle as orc  # noqa: E402
from conftest import tiny_config  # noqa: E402

SEED, GS, KVH, STEPS = 20240, 64, 1, 48
cfg = tiny_config(l2, group_size=GS, n_kv_heads=KVH)
payload = l2.synth_fill(cfg, SEED)
prompt = np.random.default_rng(7).integers(0, cfg.vocab_size, 12).astype(np.int32)
r = orc.Model(cfg, payload).generate_ids(prompt, STEPS, trace_logits=True)
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_generate.npz"),
                    seed=SEED, group_size=GS, n_kv_heads=KVH, steps=STEPS, prompt=prompt, pos0=r["pos0"],
                    tokens=r["tokens"], logits=r["logits"].astype(np.float32))
print("wrote tiny_generate.npz:", r["tokens"])
