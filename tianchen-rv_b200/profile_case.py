"""Small, self-ending workloads for profiling one kernel at a time.

    python tianchen-rv_b200/profile_case.py gemv [--rows 32000] [--k 4096] [--cols 1] [--launches 6]
    python tianchen-rv_b200/profile_case.py gemm [--rows 11008] [--k 4096] [--tokens 512] [--launches 4]
    python tianchen-rv_b200/profile_case.py dequant | quantize [--rows 4096] [--k 4096]
    python tianchen-rv_b200/profile_case.py silu | rms_norm [--rows 512] [--k 11008]
    python tianchen-rv_b200/profile_case.py repack_gemv | repack_gemv_q8 [--rows 32000] [--k 4096]
    python tianchen-rv_b200/profile_case.py repack_gemm [--rows 11008] [--k 4096] [--tokens 512]

Each case holds well under a few GB on the device and launches the kernel a handful of
times over rotating weight copies larger than the L2, so DRAM counters mean something.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemv", "gemv_q8", "gemm", "dequant", "quantize", "silu", "rms_norm", "repack_gemv",
                                     "repack_gemv_q8", "repack_gemm"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--launches", type=int, default=6)
    args = ap.parse_args()

    import torch

    pkg = entry.load_package()
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(7)
    if args.case in ("gemv", "gemv_q8"):
        rows = args.rows or 32000
        q8w = args.case == "gemv_q8"
        wf = torch.randn((rows, args.k), generator=gen, device="cuda") * 0.02
        w = pkg.quantize_q8_0(wf) if q8w else pkg.quantize_q4_0(wf)
        copies = [w] + [w.clone() for _ in range(max(2, (300 << 20) // w.numel()))]
        x = pkg.quantize_q8_0(torch.randn((args.cols, args.k), generator=gen, device="cuda"))
        y = torch.empty((rows, args.cols), dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.gemv(copies[i % len(copies)], x, q8_weights=q8w, out=y)
    elif args.case in ("repack_gemv", "repack_gemv_q8"):
        # random bytes stand in for the interleaved weights (timing and traffic do not depend on them)
        rows = args.rows or 32000
        q8w = args.case == "repack_gemv_q8"
        nbytes = rows // 16 * (args.k // 32) * (544 if q8w else 288)
        copies = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda", generator=gen)
                  for _ in range(max(3, (300 << 20) // nbytes + 1))]
        x = pkg.quantize_q8_0(torch.randn((1, args.k), generator=gen, device="cuda")).reshape(-1)
        y = torch.empty(rows, dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.repack_gemv(copies[i % len(copies)], x, rows, q8_weights=q8w, out=y)
    elif args.case == "repack_gemm":
        rows = args.rows or 11008
        nb = args.k // 32
        wx = torch.randint(0, 256, (rows // 16 * nb * 288,), dtype=torch.uint8, device="cuda", generator=gen)
        xx = torch.randint(0, 256, (args.tokens // 4 * nb * 136,), dtype=torch.uint8, device="cuda", generator=gen)
        pw = pkg.PreparedX16Weights(wx, args.k, rows)
        out = torch.empty((args.tokens, rows), dtype=torch.float32, device="cuda")
        for _ in range(args.launches):
            pw.gemm(xx, args.tokens, out=out)
    elif args.case == "gemm":
        rows = args.rows or 11008
        w = pkg.quantize_q4_0(torch.randn((rows, args.k), generator=gen, device="cuda") * 0.02)
        x = pkg.quantize_q8_0(torch.randn((args.tokens, args.k), generator=gen, device="cuda"))
        pw = pkg.PreparedWeights(w)
        out = torch.empty((rows, args.tokens), dtype=torch.float32, device="cuda")
        for _ in range(args.launches):
            pkg.gemm(pw, x, out=out)
    elif args.case in ("quantize", "silu", "rms_norm"):
        rows = args.rows or (4096 if args.case == "quantize" else 512)
        k = args.k if (args.case == "quantize" or args.k != 4096) else 11008
        xs = [torch.randn((rows, k), generator=gen, device="cuda") for _ in range(6)]
        out = torch.empty((rows, k), dtype=torch.float32, device="cuda")
        qout = torch.empty((rows, k // 32 * 34), dtype=torch.uint8, device="cuda")
        for i in range(args.launches):
            if args.case == "quantize":
                pkg.quantize_q8_0(xs[i % len(xs)], out=qout)
            elif args.case == "silu":
                pkg.vec_silu(xs[i % len(xs)], out=out)
            else:
                pkg.rms_norm(xs[i % len(xs)], 1e-6, out=out)
    else:
        rows = args.rows or 4096
        q = pkg.quantize_q8_0(torch.randn((rows, args.k), generator=gen, device="cuda") * 0.02)
        copies = [q] + [q.clone() for _ in range(8)]
        out = torch.empty((rows, args.k), dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.dequantize_q8_0(copies[i % len(copies)], out=out)
    torch.cuda.synchronize()
    pkg.check_device_errors()
    print("profile case done")


if __name__ == "__main__":
    main()
