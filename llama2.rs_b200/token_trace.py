"""Where one token's time goes inside the one-kernel-per-token path: per-phase clock stamps of every CTA.

Needs a library built with the stamps compiled in (they cost registers, so the normal build leaves them out):

    L2_TK_TRACE=1 python llama2.rs_b200/build.py --force
    python llama2.rs_b200/token_trace.py [7B|13B|70B] [group size] [context] [layers]
    python llama2.rs_b200/build.py --force        # back to the normal build

Runs `context` positions, then one traced token (l2_debug_token_trace), and prints per kind of phase the mean over CTAs
and layers of: waiting for the tagged inputs, scatter into K order + CTA barrier, digit emission + statistics, main loop,
epilogue, and the gap to the start of the next phase; for the attention phase: q/k/v wait + RoPE, scores, values, merge.
Times are SM cycles divided by the SM clock read from the run (globaltimer stamps give the phase spans).
"""
import ctypes as C
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import llama2_rs as l2  # noqa: E402

TRACE_W = 32  # stamps per (CTA, phase)


def main():
    name = sys.argv[1] if len(sys.argv) > 1 else "7B"
    gs = int(sys.argv[2]) if len(sys.argv) > 2 else 128
    ctx = int(sys.argv[3]) if len(sys.argv) > 3 else 160
    cfg = l2.preset_config(name, gs)
    if len(sys.argv) > 4:
        cfg.n_layers = int(sys.argv[4])
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m = l2.LlamaModel.synthetic(cfg, 20240)
    st = l2.RunState(m)
    L = cfg.n_layers
    nph = 1 + 5 * L + 2
    count = sms * nph * TRACE_W
    tok = 5
    for pos in range(ctx):
        tok = l2.decode_step(m, st, tok, pos)[0]
    l2.check(l2.lib.l2_debug_token_trace(st._h, 1, None, count))
    l2.decode_step(m, st, 11, ctx)
    buf = np.zeros(count, dtype=np.uint64)
    l2.check(l2.lib.l2_debug_token_trace(st._h, 0, buf.ctypes.data_as(C.POINTER(C.c_uint64)), count))
    t = buf.reshape(sms, nph, TRACE_W).astype(np.int64)
    if not t[:, 1, 0].any():
        raise SystemExit("no stamps: the library was built without L2_TK_TRACE=1")
    # SM cycles per microsecond from a long span measured both ways on CTA 0
    cyc = (t[0, nph - 2, 0] - t[0, 1, 0]) / ((t[0, nph - 2, 4] - t[0, 1, 4]) / 1e3)
    total = (t[:, nph - 1, 6].max() - t[:, 0, 4].min()) / 1e3
    lo, hi = (1, L - 1) if L > 4 else (0, L)
    layer = np.mean([np.mean(t[:, 1 + 5 * (l + 1), 4] - t[:, 1 + 5 * l, 4]) / 1e3 for l in range(lo, hi - 1)]) if hi - lo > 1 else float("nan")
    print("%s g%d, %d layers, context %d: token %.1f us, layer %.2f us, classifier %.1f us, SM clock %.0f MHz" %
          (name, gs, L, ctx, total, layer, (t[:, nph - 2, 5].max() - t[:, nph - 2, 4].min()) / 1e3, cyc))
    print("GEMV phases, us (mean over CTAs and layers): span = first CTA's start -> last CTA's end")
    print("phase   span | wait inputs  scatter+sync  digits+stats  main loop  epilogue  to next phase | start spread  end spread")
    for off, n in ((0, "qkv"), (2, "wo"), (3, "w13"), (4, "w2")):
        rows = []
        for l in range(lo, hi):
            p = 1 + 5 * l + off
            work = t[:, p, 9] > 0  # CTAs that own tiles of this phase
            r, nxt = t[work, p], t[work, p + 1]
            natural = (r[:, 22] > 0).any()
            polled = r[:, 21] - r[:, 16]
            sync = (r[:, 22] - r[:, 21]) if natural else np.zeros(len(r), np.int64)
            emit = (r[:, 1] - r[:, 22]) if natural else (r[:, 1] - r[:, 21])
            rows.append([(r[:, 5].max() - r[:, 4].min()) / 1e3, np.mean(r[:, 16] - r[:, 0] + polled) / cyc, np.mean(sync) / cyc, np.mean(emit) / cyc,
                         np.mean(r[:, 2] - r[:, 1]) / cyc, np.mean(r[:, 7] - r[:, 2]) / cyc, np.mean(nxt[:, 0] - r[:, 7]) / cyc,
                         (r[:, 4].max() - r[:, 4].min()) / 1e3, (r[:, 5].max() - r[:, 5].min()) / 1e3])
        a = np.mean(np.array(rows), axis=0)
        print("%-5s %6.2f | %11.2f  %12.2f  %12.2f  %9.2f  %8.2f  %13.2f | %12.2f  %10.2f" % ((n,) + tuple(a)))
    print("attention phase, us (CTAs that had an item): span | items | q,k,v wait + RoPE  scores  values  partials + merge")
    rows = []
    for l in range(lo, hi):
        r = t[:, 1 + 5 * l + 1]
        busy = r[:, 13] > 0
        rb = r[busy]
        rows.append([(r[:, 5].max() - r[:, 4].min()) / 1e3, busy.sum(), np.mean(rb[:, 10] - rb[:, 0]) / cyc, np.mean(rb[:, 11] - rb[:, 10]) / cyc,
                     np.mean(rb[:, 12] - rb[:, 11]) / cyc, np.mean(rb[:, 7] - rb[:, 12]) / cyc])
    a = np.mean(np.array(rows), axis=0)
    print("attn  %6.2f | %5.0f | %17.2f  %6.2f  %6.2f  %16.2f" % tuple(a))


if __name__ == "__main__":
    main()
