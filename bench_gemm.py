#!/usr/bin/env python
"""The tcgen05 main loop alone on the shapes of the two gradient GEMMs, beside cuBLAS (torch.matmul) on the same box.

    python bench_gemm.py [--trace] [--wide 1|0]

Shapes: the weight-gradient and input-gradient GEMMs of the Llama-3-8B head (N=32768, H=4096, V=128256) in the default mode
(one token chunk of 10 880 rows) and in the two-sweep mode (one vocabulary slab of 16 128 columns).  For each: TFLOP/s of
this library's kernel (flce_b200_gemm, bf16 in / bf16 out, CTA pairs, 256x512 or 256x256 tiles) and of cuBLAS, timed with
CUDA events over short back-to-back loops (so clocks are near their burst value: compare the two columns, not the absolutes).

--trace loads the cycle-accounting build (python liger-kernel_b200/build.py --trace) and prints, per shape, the share of
a CTA's cycles the MMA warp waited for TMA data / for a free accumulator, the epilogue warps were busy, and the producer
waited for a free stage, plus ideal cycles (8192 FLOP/clk/SM) over measured cycles.
"""

import argparse
import ctypes as C
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "liger-kernel_b200")

SHAPES = [
    # name, A MN-major, B MN-major, M, N, K
    ("dW two-sweep  (dZ^T.X, one slab) ", 1, 1, 16128, 4096, 32768),
    ("dX two-sweep  (dZ.W, one slab)   ", 0, 1, 32768, 4096, 16128),
    ("dW default    (E^T.X', one chunk)", 1, 1, 128256, 4096, 10880),
    ("dX default    (E.W, one chunk)   ", 0, 1, 10880, 4096, 128256),
    ("dW default, X' stored transposed ", 1, 0, 128256, 4096, 10880),
    ("sweep-1 shape (X.W^T), plain store", 0, 0, 10880, 128256, 4096),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--wide", type=int, default=None, help="1: 256x512 tiles (default of the library), 0: 256x256")
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--seconds", type=float, default=0.0,
                    help="time each kernel over a loop this long instead of --iters launches: the power cap settles (about a second) "
                         "and the SM clock sampled meanwhile is printed, so the figures are the sustained ones")
    ap.add_argument("--out", default="bf16", choices=["bf16", "fp32"], help="dtype of D (fp32: the first chunk of a weight gradient)")
    args = ap.parse_args()
    if args.trace:
        os.environ["LIGER_B200_LIB"] = os.path.join(PKG, "liger_kernel_b200", "libflce_b200_trace.so")
    sys.path.insert(0, PKG)
    import numpy as np
    import torch

    sys.path.insert(0, ROOT)
    from bench import ClockSampler

    from liger_kernel_b200 import _lib

    lib = _lib.lib
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def read_trace(flops):
        buf = (C.c_ulonglong * (1024 * 8))()
        lib.flce_b200_debug_clock_trace.argtypes = [C.c_void_p, C.c_int]
        lib.flce_b200_debug_clock_trace(buf, 1024 * 8)
        a = np.array(buf[:sms * 8], dtype=np.float64).reshape(sms, 8)
        lead = a[::2]
        total = a[:, 5].mean()
        ideal = flops / sms / 8192
        return (f"ideal/measured cycles {ideal / total:.3f} | MMA waits: data {lead[:, 0].mean() / total:.3f}, accumulator "
                f"{lead[:, 1].mean() / total:.3f} | epilogue busy {a[:, 3].mean() / total:.3f} | producer waits {a[:, 4].mean() / total:.3f}")

    for wide in ([args.wide] if args.wide is not None else [1, 0]):
        _lib.set_option("wide_tiles", wide)
        print(f"=== {'256x512' if wide else '256x256'} tiles")
        for name, a_mn, b_mn, M, N, K in SHAPES:
            torch.manual_seed(0)
            A = (torch.randn((K, M) if a_mn else (M, K), device="cuda") * 0.1).bfloat16()
            B = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.1).bfloat16()
            D = torch.empty((M, N), device="cuda", dtype=torch.bfloat16 if args.out == "bf16" else torch.float32)
            d_code = 0 if args.out == "bf16" else 2

            def ours():
                _lib.check(lib.flce_b200_gemm(C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(D.data_ptr()), M, N, K,
                                              A.stride(0), B.stride(0), D.stride(0), 0, d_code, a_mn, b_mn, 1, st))

            Dc = D if args.out == "bf16" else torch.empty((M, N), device="cuda", dtype=torch.bfloat16)

            def cublas():
                torch.matmul(A.t() if a_mn else A, B if b_mn else B.t(), out=Dc)

            res, clk = {}, {}
            for tag, fn in (("ours", ours), ("cublas", cublas)):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                iters = args.iters
                if args.seconds > 0:          # calibrate the launch count for the requested duration
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    fn()
                    e1.record()
                    torch.cuda.synchronize()
                    iters = max(4, int(args.seconds * 1e3 / e0.elapsed_time(e1)))
                with ClockSampler(0) as sampler:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(iters):
                        fn()
                    e1.record()
                    torch.cuda.synchronize()
                res[tag] = 2.0 * M * N * K / (e0.elapsed_time(e1) / iters) / 1e9
                clk[tag] = sampler.summary()["sm_mhz"] if args.seconds > 0 else None
            line = f"{name} {M}x{N}x{K}: ours {res['ours']:.0f} TFLOP/s, cuBLAS {res['cublas']:.0f}, ratio {res['ours'] / res['cublas']:.3f}"
            if args.seconds > 0:
                line += f"  (SM clock under load: ours {clk['ours']} MHz, cuBLAS {clk['cublas']} MHz)"
            if args.trace:
                ours()
                torch.cuda.synchronize()
                line += "\n      " + read_trace(2.0 * M * N * K)
            print(line, flush=True)
            del A, B, D
    _lib.check(lib.flce_b200_check_device_status(st))


if __name__ == "__main__":
    main()
