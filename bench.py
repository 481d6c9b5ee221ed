#!/usr/bin/env python
"""Benchmark of the llama2.rs token loop on B200: batch-1 greedy decode tok/s (and prefill tok/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload 7b|13b|70b|70b-long] [--impl ours|reference]

With one GPU visible the default workload is the 7B configuration the metric is quoted on.  Inside a scaling run (several
GPUs visible, or launched by torch.distributed.run with one rank per GPU) the default is the 70B configuration, the one
that shards: tensor parallel over all N ranks (the token kernel stores into every rank's memory over NVLink), at every N
including 1, so that the per-N values form the strong-scaling curve.  `--workload 7b|13b` on N > 1 GPUs runs independent
replicas (batch-1 decode of a model that fits one GPU has nothing to exchange; `scaling` is "weak").

A step is one pass of the workload: a seeded random prompt through prefill, then the decode
loop (the headline configuration for 7B: 32 prompt tokens, 256 greedy tokens).  `value` is decode tok/s with
weights, KV cache and the loop state resident in HBM (CUDA events on the launching stream);
`e2e` is the same loop driven token by token through the C ABI with host buffers (l2_decode_step:
token and position go host->device and the chosen token comes back every step).  Weights are a
seeded synthetic checkpoint in the reference's .bin layout (there are no real weights offline).

--impl reference times the CPU restatement of the reference's rayon+SIMD path (oracle/, the
reference itself is nightly Rust and cannot be built here) on the host cores, on a bounded sample
of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "llama2.rs_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

WORKLOADS = {  # name: (model size, group size, prompt tokens, decode tokens)  -- the benchmark configurations
    "7b": ("7B", 128, 32, 256),
    "13b": ("13B", 128, 128, 512),
    "70b": ("70B", 64, 64, 256),
    # long-context stress case: the prompt fills three quarters of the 2048-entry KV cache, the decode tokens the rest
    "70b-long": ("70B", 64, 1536, 512),
}
WEIGHT_SEED, PROMPT_SEED = 20240, 7
TOKEN_KERNEL_TRAFFIC_RATIO = 1.022  # DRAM bytes / algorithmic bytes of the token kernel, from its ncu capture


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, which): the driver-written measurement of this pool's B200s, else the fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")):
            if any(r[3 + i] == "Active" for r in self.rows):
                reasons.append(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def visible_gpus():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=20).stdout
        n = sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        n = 0
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis is not None and vis.strip() != "":
        n = min(n, len([v for v in vis.split(",") if v.strip()])) if n else len([v for v in vis.split(",") if v.strip()])
    return n


def prefill_report(model, cfg, positions, ms, tp, hbm_peak, tensor_peak, peak_kind, cls_rows=None):
    """Batched prefill (the tcgen05 GEMM path) against both rooflines.  Algorithmic flops: 2 * K * N per position and
    QLinear (the classifier is not run in prefill); algorithmic bytes: the QLinear bytes of one pass over the weights per
    chunk of up to 64 positions.  The integer GEMM executes 3 digit columns per position (balanced base-256 digits of the
    activations), i.e. 3x the algorithmic multiply-adds on the int8 pipe."""
    if positions <= 0 or ms <= 0:
        return None
    d, h, L = cfg.dim, cfg.hidden_dim, cfg.n_layers
    kv = d * cfg.n_kv_heads // cfg.n_heads
    flops_per_pos = 2.0 * L * (2 * d * d + 2 * d * kv + 3 * d * h)
    cls_rows = cfg.vocab_size if cls_rows is None else cls_rows  # classifier rows this process streams per token (a slice under tensor parallelism over peer memory)
    qbytes = float(model.decode_bytes) - 4.0 * cls_rows * d - 4.0 * (2 * L + 1) * d  # qweight + qzeros + scales of this process's rows
    passes = positions if tp else (positions + 63) // 64  # tp here: tensor parallel over NCCL, which takes the prompt one position at a time
    tflops = flops_per_pos * positions / (ms * 1e-3) / 1e12
    gbs = qbytes * passes / (ms * 1e-3) / 1e9
    return {"positions": positions, "ms": ms, "weight_passes": passes, "tflops": tflops, "tensor_peak_tflops": tensor_peak,
            "tensor_frac": tflops / tensor_peak, "weight_gbs": gbs, "hbm_frac": gbs / hbm_peak, "peak_kind": peak_kind,
            "executed_mma_inflation": 1 if tp else 3}


def make_prompt(np, n, vocab):
    return np.random.default_rng(PROMPT_SEED).integers(0, vocab, n).astype(np.int32)


class CpuArm:
    """The CPU restatement on a bounded sample of the workload.  Set-up (untimed, once): the checkpoint in host memory
    and the prompt through the reference's 64/32/16/8/4/2 prefill ladder (its own tok/s is reported).  One run() = the
    next `sample_tokens` positions of the greedy B=1 loop; decode tok/s over those positions."""

    def __init__(self, workload, payload=None, cfg=None):
        import numpy as np
        import llama2_rs as l2
        import oracle as orc
        self.np, self.orc = np, orc
        self.workload = workload
        self.size, gs, self.n_prompt, _ = WORKLOADS[workload]
        self.cfg = cfg if cfg is not None else l2.preset_config(self.size, gs)
        self.payload = payload if payload is not None else l2.synth_fill(self.cfg, WEIGHT_SEED)
        self.model = orc.Model(self.cfg, self.payload)
        self.sample_tokens = {"7b": 8, "13b": 4, "70b": 1, "70b-long": 1}[workload]
        self.prompt = make_prompt(np, self.n_prompt, self.cfg.vocab_size)
        self.cores = orc.lib().orc_num_threads()
        self.state = orc.State(self.model)
        # prefill<A> ladder (src/inference.rs:78-127): batches of A rows while pos + A < n_prompt
        self.pos = 0
        t0 = time.perf_counter()
        for a in (64, 32, 16, 8, 4, 2):
            while self.pos + a < self.n_prompt:
                positions = np.arange(self.pos, self.pos + a, dtype=np.int32)
                tokens = np.array([1 if p == 0 else self.prompt[p - 1] for p in positions], np.int32)
                self.model.transformer(self.state, tokens, positions)
                self.pos += a
        self.prefill_s = time.perf_counter() - t0
        self.prefill_positions = self.pos
        self.token = 1 if self.pos == 0 else int(self.prompt[self.pos - 1])
        self.first_pos = self.pos

    def run(self):
        np = self.np
        n, t0 = 0, time.perf_counter()
        for _ in range(self.sample_tokens):
            if self.pos + 1 >= self.cfg.seq_len:
                break
            logits = self.model.transformer(self.state, np.array([self.token], np.int32), np.array([self.pos], np.int32))
            nxt = int(self.prompt[self.pos]) if self.pos < self.n_prompt else int(len(logits) - 1 - np.argmax(logits[::-1]))  # last maximum wins (src/util.rs:39-46)
            self.token, self.pos, n = nxt, self.pos + 1, n + 1
        dt = time.perf_counter() - t0
        prefill_tok_s = self.prefill_positions / max(self.prefill_s, 1e-9)
        return {"value": n / dt, "unit": "tok/s", "cores": self.cores, "kind": "port",
                "sample": "%s synthetic checkpoint; set-up (untimed): %d-token prompt, %d positions through the 64/32/16/8/4/2 prefill ladder (%.0f ms, %.1f tok/s); "
                          "timed: %d B=1 positions per step, context %d..%d so far (the GPU arm averages over contexts up to %d)"
                          % (self.size, self.n_prompt, self.prefill_positions, self.prefill_s * 1e3, prefill_tok_s, self.sample_tokens,
                             self.first_pos, self.pos, self.n_prompt + WORKLOADS[self.workload][3]),
                "prefill_tok_s": prefill_tok_s}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(WORKLOADS),
                    help="auto: 7b when one GPU is visible; 70b inside a scaling run (several GPUs visible or launched by torch.distributed.run), "
                         "tensor-parallel over all ranks when N > 1.  7b/13b on N > 1 GPUs run as independent replicas")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-warmup", type=int, default=3, help="profiling runs may lower the warm-up floor")
    ap.add_argument("--layers", type=int, default=0, help="profiling only: truncate the model to this many layers (not a benchmark number)")
    ap.add_argument("--prompt", type=int, default=0, help="profiling only: prompt tokens instead of the workload's (not a benchmark number)")
    ap.add_argument("--tp-nccl", action="store_true", help="70b on N > 1 GPUs: NCCL all-gathers between per-operator kernels instead of peer-memory stores")
    ap.add_argument("--flags", type=int, default=0, help="L2_FLAG_* bits for the model (8 = one launch per operator instead of one kernel per token)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    auto = args.workload == "auto"
    if auto:
        # One GPU visible: the 7B configuration the metric is quoted on.  Inside a scaling run (launched by torch.distributed.run,
        # or with several GPUs visible -- the N = 1 leg of such a run is a plain `python bench.py --gpus 1` on the multi-GPU box):
        # the 70B configuration, which is the one that shards, at every N including 1, so that the per-N values form the
        # strong-scaling curve of tensor parallelism.
        args.workload = "70b" if ("WORLD_SIZE" in os.environ or visible_gpus() > 1) else "7b"
    tp = world > 1 and args.workload.startswith("70b")  # 70B is sharded over the ranks (tensor parallel); smaller models run as replicas
    size, gs, n_prompt, n_decode = WORKLOADS[args.workload]
    if args.prompt > 0:
        n_prompt = args.prompt
    config = {"workload": "Llama2-%s GPTQ 4-bit g%d act-order, %d-token random prompt, %d greedy decode tokens, batch 1"
                          % (size, gs, n_prompt, n_decode) +
                          (" (default of a scaling run: more than one GPU visible or launched by torch.distributed.run; with one GPU visible the default is the 7B configuration)"
                           if auto and args.workload == "70b" else ""),
              "weights": "seeded synthetic checkpoint (seed %d) in the export.py .bin layout" % WEIGHT_SEED,
              "l2": "weights streamed per token (%s) exceed the 126 MB L2; no flush needed" % size,
              "parallelism": ("tp%d: every QLinear split by output rows, %s" % (world, "NCCL all-gathers in the token graph" if args.tp_nccl else
                                                                                   "token kernel storing into every rank's memory over NVLink")) if tp
              else ("replicas" if world > 1 else "single GPU")}

    if args.impl == "reference":
        if rank != 0:
            return
        if world > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
            # the launcher pins every rank to one OpenMP thread; this arm is one process that should use the host's cores
            os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        steps = max(1, args.steps)
        arm = CpuArm(args.workload)
        vals = [arm.run() for _ in range(max(0, args.warmup) + steps)][-steps:]
        v = sum(x["value"] for x in vals) / len(vals)
        cb = dict(vals[-1], value=v)
        print(json.dumps({"impl": "reference", "metric": "batch-1 decode tok/s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
                          "steps": steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config, "cpu_baseline": cb,
                          "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import llama2_rs as l2

    if world > 1:
        # the ranks exchange a handful of bytes on the host (IPC handles or the NCCL id, the timing maximum): gloo;
        # the data path between the GPUs is the library's own (peer-memory stores, or NCCL with --tp-nccl)
        dist.init_process_group("gloo")
    dev = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev)
    cfg = l2.preset_config(size, gs)
    if args.layers:
        cfg.n_layers = args.layers
        config["truncated_layers"] = args.layers
    if args.prompt > 0:
        config["profiling_prompt"] = args.prompt
    need_payload = rank == 0 and world == 1 and not args.no_cpu_baseline and not args.workload.startswith("70b")
    payload = l2.synth_fill(cfg, WEIGHT_SEED) if need_payload else None
    if payload is not None:
        model = l2.LlamaModel.from_blob(cfg, payload, device=dev, flags=args.flags)
    else:
        model = l2.LlamaModel.synthetic(cfg, WEIGHT_SEED, device=dev, flags=args.flags, tp=(rank, world) if tp else (0, 1))
    if tp and args.tp_nccl:
        ids = [l2.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        model.tp_connect(ids[0])
    elif tp:
        # peer memory: every rank maps every other rank's activation pool; the token kernel stores into all of them
        handles = [None] * world
        dist.all_gather_object(handles, model.tp_pool_handle())
        for r in range(world):
            model.tp_pool_attach(r, handles[r])
    # one persistent kernel per token on a single GPU; one launch per operator under tensor parallelism or on request
    token_kernel = not (tp and args.tp_nccl) and not (args.flags & 8) and not os.environ.get("L2_NO_TOKEN_KERNEL")
    stream = torch.cuda.Stream(device=dev)
    model.set_stream(stream.cuda_stream)
    state = l2.RunState(model)
    prompt = make_prompt(np, n_prompt, cfg.vocab_size)
    total = n_prompt + n_decode

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(timed):
        state.reset()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        with torch.cuda.stream(stream):
            e0.record(stream)
            pos0 = l2.prefill(model, state, prompt)
            e1.record(stream)
            toks = l2.decode_run(model, state, prompt, pos0, total)
            e2.record(stream)
        torch.cuda.synchronize()
        return pos0, toks, e0.elapsed_time(e1), e1.elapsed_time(e2)

    for _ in range(max(args.min_warmup, args.warmup)):
        pos0, toks_ref, _, _ = one_step(False)
    barrier()
    launches0 = l2.lib.l2_launch_count()
    with ClockSampler(dev) as clocks:
        prefill_ms, decode_ms = 0.0, 0.0
        for _ in range(args.steps):
            pos0, toks, pf, dc = one_step(True)
            prefill_ms += pf
            decode_ms += dc
            assert np.array_equal(toks, toks_ref), "decode is not reproducible from step to step"
        dom_ms = None
        if not token_kernel:
            # the dominant kernel alone: w1/w3 + SwiGLU GEMV, cycling through the layers (each launch reads other weights)
            n_dom = 4 * cfg.n_layers
            l2.check(l2.lib.l2_bench_projection(model._h, state._h, 2, 0, cfg.n_layers))
            torch.cuda.synchronize()
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            d0.record(stream)
            l2.check(l2.lib.l2_bench_projection(model._h, state._h, 2, 0, n_dom))
            d1.record(stream)
            torch.cuda.synchronize()
            dom_ms = d0.elapsed_time(d1) / n_dom
    barrier()
    launches = l2.lib.l2_launch_count() - launches0
    n_loop = total - pos0           # positions run by the B=1 loop per step (a few teacher-forced ones first)
    t = torch.tensor([decode_ms, prefill_ms], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    decode_ms, prefill_ms = t.tolist()
    streams = 1 if tp else world  # token streams running side by side: replicas add up, a tensor-parallel group is one
    value = streams * n_loop * args.steps / decode_ms * 1e3

    # end to end: the host drives every token through l2_decode_step (host buffers in and out)
    state.reset()
    l2.prefill(model, state, prompt)
    torch.cuda.synchronize()
    tok = int(prompt[pos0 - 1]) if pos0 > 0 else l2.START
    t0 = time.perf_counter()
    for p in range(pos0, total):
        forced = int(prompt[p]) if p < n_prompt else -1
        tok, _ = l2.decode_step(model, state, tok, p, forced_next=forced)
    e2e_s = time.perf_counter() - t0
    e2e = {"value": streams * n_loop / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 40 * n_loop, "d2h_bytes_per_step": 40 * n_loop,
           "note": "one l2_decode_step call per token: 40-byte loop record up, 40-byte record (chosen token) back"}

    streams_identical = None
    if world > 1:
        if tp:  # every rank of a tensor-parallel group must have produced the same token stream
            all_toks = [None] * world
            dist.all_gather_object(all_toks, [int(t) for t in toks_ref])
            streams_identical = all(t == all_toks[0] for t in all_toks)
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peak, tensor_peak, peak_kind = measured_peaks()
    tok_s = value / streams
    if token_kernel:
        # One persistent kernel per token: it is the dominant (only) kernel.  Algorithmic bytes per launch
        # = the checkpoint bytes one token reads; launch duration = the CUDA-event time per token above.
        roofline = {"bound": "hbm", "kernel": "token_kernel (whole B=1 forward, one launch per token)",
                    "achieved": model.decode_bytes * tok_s / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": model.decode_bytes * tok_s / 1e9 / peak, "peak_kind": peak_kind,
                    # DRAM bytes per launch: ncu capture of the same kernel on a 4-layer model (dram read+write =
                    # 1.022 x its algorithmic bytes), scaled to a full launch by the bytes processed
                    "traffic": int(TOKEN_KERNEL_TRAFFIC_RATIO * model.decode_bytes),
                    "bytes_per_launch": int(model.decode_bytes), "us_per_launch": 1e6 / tok_s}
    else:
        dom_bytes = int(l2.lib.l2_projection_bytes(model._h, 2))
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "gemv_sk_kernel (w1/w3 + SwiGLU)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
                    "bytes_per_launch": dom_bytes, "us_per_launch": dom_ms * 1e3}
    out = {
        "metric": "batch-1 decode tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": max(args.min_warmup, args.warmup), "ms_per_step": (decode_ms + prefill_ms) / args.steps, "higher_is_better": True,
        "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": "f32 activations / int4 weights", "data": "synthetic", "config": config,
        "prefill_tok_s": streams * pos0 * args.steps / max(prefill_ms, 1e-9) * 1e3,
        "prefill": prefill_report(model, cfg, pos0, prefill_ms / args.steps, tp and args.tp_nccl, peak, tensor_peak, peak_kind,
                                  cls_rows=(cfg.vocab_size * (rank + 1) // world - cfg.vocab_size * rank // world) if tp and not args.tp_nccl else None),
        "decode_ms_per_token": decode_ms / (n_loop * args.steps),
        "roofline": roofline,
        "token_roofline": {"bytes_per_token": model.decode_bytes, "achieved_gbs": model.decode_bytes * tok_s / 1e9,
                           "frac_of_8tbs": model.decode_bytes * tok_s / 8e12, "frac_of_measured": model.decode_bytes * tok_s / (peak * 1e9)},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary(),
    }
    if streams_identical is not None:
        out["tp_streams_identical"] = streams_identical
    if not args.no_cpu_baseline and world == 1:  # the CPU leg belongs to the single-GPU line
        try:
            out["cpu_baseline"] = CpuArm(args.workload, payload=payload, cfg=cfg).run()
        except Exception as e:  # the GPU numbers stand even if the CPU leg cannot run
            out["cpu_baseline"] = {"error": str(e)}
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
