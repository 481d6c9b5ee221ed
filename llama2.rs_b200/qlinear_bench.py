"""QLinear::matvec<B> alone (src/gptq.rs:94-176) on the projection shapes of Llama-2 7B / 13B / 70B.

    python llama2.rs_b200/qlinear_bench.py                        # every shape, group sizes 64 and 128, B in 1 4 16 64 256
    python llama2.rs_b200/qlinear_bench.py --shape 4096x4096 --gs 128 --m 64 --iters 4   # one case (for a profiler)

Weights have the value distributions of the synthetic checkpoint (nibbles U{0..15}, zero nibbles U{6..9}, scales
U[0.002, 0.02], act-order g_index from a seeded permutation), activations are N(0,1) f32, resident on the device.
Per case one line: microseconds per call (CUDA events on the launching stream, warm-up first), the checkpoint bytes of the
matrix per second, and useful int8 TFLOP/s (2 M K N).  B = 1 runs the GEMV kernel, B >= 2 the tcgen05 GEMM (a call is the
activation quantiser, the GEMM and, where the groups of a tile are split over CTAs, the kernel that adds the slices).
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096), (5120, 13824), (8192, 28672), (28672, 8192), (8192, 1024)]  # (K, N)


def random_qlinear(rng, in_f, out_f, gs):
    groups = in_f // gs
    qweight = rng.integers(0, 2**32, size=(out_f, in_f // 8), dtype=np.uint32).view(np.int32)
    znib = rng.integers(6, 10, size=(out_f // 8, groups, 8), dtype=np.uint32)
    qzeros = np.zeros((out_f // 8, groups), np.uint32)
    for j in range(8):
        qzeros |= znib[:, :, j] << np.uint32(4 * j)
    scales = rng.uniform(0.002, 0.02, size=(out_f, groups)).astype(np.float32)
    g_index = np.argsort(rng.permutation(in_f) // gs, kind="stable").astype(np.int32)
    return qweight, qzeros.view(np.int32), scales, g_index


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="", help="KxN, e.g. 4096x11008 (default: all projection shapes)")
    ap.add_argument("--gs", type=int, default=0, help="group size (default: 64 and 128)")
    ap.add_argument("--m", type=int, default=0, help="batch (default: 1 4 16 64 256)")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    import torch
    import llama2_rs as l2
    if not torch.cuda.is_available():
        raise SystemExit("qlinear_bench needs a GPU: there is no CPU path")
    shapes = [tuple(int(v) for v in args.shape.lower().split("x"))] if args.shape else SHAPES
    for si, (K, N) in enumerate(shapes):
        for gs in ([args.gs] if args.gs else [64, 128]):
            rng = np.random.default_rng(20240 + si)
            qw, qz, sc, gi = random_qlinear(rng, K, N, gs)
            q = l2.QLinear(qw, qz, sc, gi, gs)
            wbytes = N * K // 2 + N * (K // gs) * 4 + (N // 8) * (K // gs) * 4
            for M in ([args.m] if args.m else [1, 4, 16, 64, 256]):
                x = torch.randn(M, K, device="cuda")
                y = torch.empty(M, N, device="cuda")
                s = torch.cuda.Stream()
                with torch.cuda.stream(s):
                    for _ in range(args.warmup):
                        q.matvec_dev(x.data_ptr(), y.data_ptr(), M, s.cuda_stream)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(s)
                    for _ in range(args.iters):
                        q.matvec_dev(x.data_ptr(), y.data_ptr(), M, s.cuda_stream)
                    e1.record(s)
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) / args.iters * 1e3
                passes = (M + 63) // 64
                print("K %5d N %5d g%-3d M %3d: %8.1f us/call  %7.1f GB/s of checkpoint bytes (%d pass%s)  %6.1f TFLOP/s" %
                      (K, N, gs, M, us, wbytes * passes / us / 1e3, passes, "" if passes == 1 else "es", 2.0 * M * K * N / us / 1e6), flush=True)
            del q


if __name__ == "__main__":
    main()
