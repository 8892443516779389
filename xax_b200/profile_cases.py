"""Small, fixed workloads for profiling single kernels under ncu (one kernel, a few launches, a few
hundred MB on the device, inputs larger than L2):

    python -m xax_b200.profile_cases attn_decode [--variant V] [--batch B] [--context L]
    python -m xax_b200.profile_cases gemm [--plan BN] [--size N]

Each case runs its op three times on seeded inputs, synchronises and checks the device status
word.  ``--variant`` is passed to xaxb_attn_decode_force_variant (0 = default kernel), ``--plan``
to xaxb_gemm_force_plan (0 = planner's choice, 256 = single-CTA 128x256 tiles, 512 = CTA-pair kernel).
"""

from __future__ import annotations

import argparse

import torch

from . import _lib, ops


def attn_decode(variant: int, batch: int, context: int) -> None:
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    hq, hkv, d = 32, 8, 128
    max_len = (context + 127) // 128 * 128
    kc = torch.randn((batch, max_len, hkv, d), generator=g, device=dev, dtype=torch.bfloat16)
    vc = torch.randn((batch, max_len, hkv, d), generator=g, device=dev, dtype=torch.bfloat16)
    q = torch.randn((batch, hq, d), generator=g, device=dev, dtype=torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    ws = ops.attn_decode_workspace(batch, hq, d, max_len, dev)
    out = torch.empty_like(q)
    _lib.load().xaxb_attn_decode_force_variant(variant)
    for _ in range(3):
        ops.attn_decode(q, kc, vc, pos, workspace=ws, out=out)


def gemm(plan: int, n: int) -> None:
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn((n, n), generator=g, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn((n, n), generator=g, device=dev).to(torch.float8_e4m3fn)
    out = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
    _lib.load().xaxb_gemm_force_plan(plan, 1 if plan else 0)
    for _ in range(3):
        ops.gemm_fp8(a, b, None, None, None, out=out)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    p = sub.add_parser("attn_decode")
    p.add_argument("--variant", type=int, default=0)
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--context", type=int, default=2053)
    p = sub.add_parser("gemm")
    p.add_argument("--plan", type=int, default=0)
    p.add_argument("--size", type=int, default=8192)
    args = ap.parse_args()
    if args.case == "attn_decode":
        attn_decode(args.variant, args.batch, args.context)
    else:
        gemm(args.plan, args.size)
    torch.cuda.synchronize()
    _lib.device_status()
    print("ok")


if __name__ == "__main__":
    main()
