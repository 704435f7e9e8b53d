"""Runs one decode-matmul shape repeatedly over rotating weight copies and prints its time.

    python -m relax_b200.profile_case --m 1 --k 4096 --n 22016 [--group 32] [--asym] [--bits 4]
                                      [--copies 8] [--reps 3]

The weight copies (together larger than L2 by default) are visited round-robin, so every launch
streams its weight from HBM.  Meant for profilers: few launches, a few hundred MB on the device.
"""
import argparse

import torch

import sys; sys.path.insert(0, "/root/repo"); from relax_b200 import ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=22016)
    ap.add_argument("--group", type=int, default=32)
    ap.add_argument("--bits", type=int, default=4, choices=[4, 8])
    ap.add_argument("--asym", action="store_true")
    ap.add_argument("--copies", type=int, default=0, help="0: enough copies to exceed 320 MB")
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)
    wbytes = a.n * a.k * a.bits // 8
    copies = a.copies or max(2, int(320e6 // wbytes) + 1)
    x = torch.randn((a.m, a.k), device=dev, generator=gen).half()
    out = torch.empty((a.m, a.n), device=dev, dtype=torch.float16)
    ws, ss, zs = [], [], []
    for _ in range(copies):
        if a.bits == 4:
            raw = torch.randint(-2**31, 2**31 - 1, (a.n, a.k // 8), dtype=torch.int32, device=dev, generator=gen)
            ws.append(ops.preprocess_weight_q4f16(raw))
            ss.append((torch.rand((a.n, a.k // a.group), device=dev, generator=gen) * 0.009 + 0.001).half())
            zs.append(torch.randint(0, 16, (a.n, a.k // a.group), device=dev, generator=gen).half() if a.asym else None)
        else:
            raw = torch.randint(-127, 128, (a.k, a.n), dtype=torch.int8, device=dev, generator=gen)
            ws.append(ops.preprocess_weight_ft(raw, False))
            ss.append((torch.rand((a.n,), device=dev, generator=gen) * 0.0009 + 0.0001).half())
            zs.append(None)

    def launch(i):
        if a.bits == 4:
            ops.gemm_fp16_q4f16(x, ws[i], ss[i], zs[i], group_size=a.group, out=out)
        else:
            ops.gemm_fp16_ft(x, ws[i], ss[i], 8, out=out)

    for i in range(copies):
        launch(i)
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.reps):
        for i in range(copies):
            launch(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.reps * copies)
    gb = (wbytes + ss[0].numel() * 2 * (2 if a.asym else 1) + a.m * a.k * 2 + a.m * a.n * 2) / 1e9
    print("m=%d k=%d n=%d bits=%d group=%d: %.2f us per launch (eager), %.0f GB/s, %.1f TFLOP/s"
          % (a.m, a.k, a.n, a.bits, a.group, us, gb / (us * 1e-6), 2.0 * a.m * a.k * a.n / (us * 1e-6) / 1e12))


if __name__ == "__main__":
    main()
