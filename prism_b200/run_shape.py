"""Run one kernel family on one shape and print its time: `python -m prism_b200.run_shape gemm_bf16 4096 8192 8192`.

For looking at a shape that the benchmark does not time by itself (a shard of the multi-GPU run on one GPU, a block of
a host plan) with CUDA events or under a profiler.  Inputs are seeded; every launch is timed on its own.

    gemm_bf16 M N K     D = A * B^T, bf16 in and out, C column-major     (prism_b200.runmyh100)
    sgemm M N K         C = 1.5 * A * B + 0.5 * C in fp32, kernel 5       (prism_b200.run_my_kernel)
    scan N              inclusive scan of N uint32 values in place        (prism_b200.launch_scan)
"""
from __future__ import annotations

import argparse

import torch

import prism_b200 as pb


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("family", choices=["gemm_bf16", "sgemm", "scan"])
    ap.add_argument("dims", type=int, nargs="+")
    ap.add_argument("--launches", type=int, default=10)
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args()
    dev = torch.device(a.device)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(1234)
    if a.family == "scan":
        (n,) = a.dims
        x0 = torch.randint(0, 2, (n,), dtype=torch.int32, device=dev, generator=g)
        x = x0.clone()
        ws = pb.scan_workspace(n, dev)
        restore, run = (lambda: x.copy_(x0)), (lambda: pb.launch_scan(n, x, ws))
        work, unit = 8.0 * n, "GB/s"
    else:
        M, N, K = a.dims
        if a.family == "gemm_bf16":
            A = (torch.randn((M, K), device=dev, generator=g) * 0.1).to(torch.bfloat16)
            B = (torch.randn((N, K), device=dev, generator=g) * 0.1).to(torch.bfloat16)
            C = torch.empty((N, M), dtype=torch.bfloat16, device=dev)
            restore, run = (lambda: None), (lambda: pb.runmyh100(M, N, K, A, B, C))
        else:
            A = torch.rand((M, K), device=dev, generator=g) * 2 - 1
            B = torch.rand((K, N), device=dev, generator=g) * 2 - 1
            C0 = torch.rand((M, N), device=dev, generator=g) * 2 - 1
            C = C0.clone()
            restore, run = (lambda: C.copy_(C0)), (lambda: pb.run_my_kernel(5, M, N, K, 1.5, A, B, 0.5, C))
        work, unit = 2.0 * M * N * K, "GFLOP/s"
    times = []
    for _ in range(a.launches):
        restore()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop))
    code, msg = pb.last_error()
    if code:
        raise SystemExit(f"prism_b200: {msg}")
    best, med = min(times), sorted(times)[len(times) // 2]
    print(f"{a.family} {' x '.join(map(str, a.dims))}: median {med:.4f} ms ({work / med / 1e6:.1f} {unit}), "
          f"best {best:.4f} ms ({work / best / 1e6:.1f} {unit}) of {a.launches} launches")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
