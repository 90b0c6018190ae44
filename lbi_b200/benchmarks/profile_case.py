"""Small, self-terminating workloads for ``ncu`` captures of single kernels.

    python -m lbi_b200.benchmarks.profile_case --case attn      # attention pullback: B 2, H 16, T 2048, Dh 64, P 12
    python -m lbi_b200.benchmarks.profile_case --case gemm      # tcgen05 GEMM 32768 x 5632 x 1024 (fc1 forward)
    python -m lbi_b200.benchmarks.profile_case --case dgrad     # tcgen05 GEMM with MN-major B (fc1 dgrad)
    python -m lbi_b200.benchmarks.profile_case --case elementwise   # rmsnorm_bwd / swiglu_bwd / rope over 65536 rows
    python -m lbi_b200.benchmarks.profile_case --case scan      # suffix scan B 8, K 32, R 256
    python -m lbi_b200.benchmarks.profile_case --case attn_fwd  # causal attention forward B 4, H 16, T 4096
    python -m lbi_b200.benchmarks.profile_case --case ssd       # Mamba-2 SSD forward B 2, L 8192, 24 heads, d_state 64
    python -m lbi_b200.benchmarks.profile_case --case ssd_bwd   # SSD forward + backward (permuted scans, decay gradient, tails)
    python -m lbi_b200.benchmarks.profile_case --case mamba_elementwise   # gated RMSNorm and SISO preprocessing, both directions
    python -m lbi_b200.benchmarks.profile_case --case chunk_bwd          # fused chunk backward, Mamba-3 form: 16 directions x B 1, L 1024, 24 heads
    python -m lbi_b200.benchmarks.profile_case --case chunk_bwd_ssd      # fused chunk backward, Mamba-2 form (grouped B / C, weight dt)
    python -m lbi_b200.benchmarks.profile_case --case mamba_glue         # gate, small-tensor fwd / bwd, conv + SiLU fwd / bwd / wgrad
    python -m lbi_b200.benchmarks.profile_case --case small              # interface / scan / optimizer / embedding / CE kernels
    python -m lbi_b200.benchmarks.profile_case --case prep_bwd           # SISO preprocessing backward as the pullback runs it (bf16 cotangents, 16 directions, no bias gradients)

Each case holds well under 2 GB on the device, touches more than the 126 MB L2, launches the kernel of interest a
handful of times and exits.  Typical capture:
    ncu --set full --clock-control none -k regex:pullback_kernel -c 2 -o prof python -m lbi_b200.benchmarks.profile_case --case attn
"""
from __future__ import annotations

import argparse
import math

import torch

from lbi_b200 import ops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["attn", "gemm", "dgrad", "elementwise", "scan", "attn_fwd", "ssd", "ssd_bwd", "mamba_elementwise", "chunk_bwd",
                             "chunk_bwd_ssd", "mamba_glue", "small", "prep_bwd"])
    ap.add_argument("--repeats", type=int, default=2)
    args = ap.parse_args()
    dev = "cuda"
    torch.manual_seed(0)
    if args.case == "attn":
        from lbi_b200.ops.attention import attention_input_pullback_basis

        b, h, t, dh, p = 2, 16, 2048, 64, 12
        q, k, v = (torch.randn(b, h, t, dh, device=dev).bfloat16() for _ in range(3))
        do = torch.randn(b, p, h, t, dh, device=dev).bfloat16()
        for _ in range(args.repeats):
            attention_input_pullback_basis(q, k, v, do, scale=1.0 / math.sqrt(dh), causal=True, kernel_mode="tcgen05_pblock")
    elif args.case in ("gemm", "dgrad"):
        m, n, k = 32768, 5632, 1024
        if args.case == "gemm":
            a = torch.randn(m, k, device=dev).bfloat16()
            w = torch.randn(n, k, device=dev).bfloat16()
            for _ in range(args.repeats):
                ops.ext().gemm(a, w)
        else:
            dy = torch.randn(m, n, device=dev).bfloat16()
            w = torch.randn(n, k, device=dev).bfloat16()
            for _ in range(args.repeats):
                ops.ext().gemm(dy, w, False, True, False, None, 1)
    elif args.case == "elementwise":
        from lbi_b200.backbones.transformer.rope import rope_tables

        rows, reps, dim, hidden = 8192, 8, 1024, 2816
        stream = torch.randn(rows, dim, device=dev)
        rstd = torch.rand(rows, device=dev) + 0.5
        w = torch.ones(dim, device=dev)
        g = torch.randn(rows * reps, dim, device=dev).bfloat16()
        acc = torch.zeros(rows * reps, dim, device=dev)
        u = torch.randn(rows, 2 * hidden, device=dev).bfloat16()
        da = torch.randn(rows * reps, hidden, device=dev).bfloat16()
        qkv = torch.randn(rows * reps, 3 * dim, device=dev).bfloat16()
        cos, sin = rope_tables(2048, 64, 10000.0, torch.device(dev))
        for _ in range(args.repeats):
            ops.rmsnorm_bwd(g, stream, rstd, w, acc, lowp_dtype=torch.bfloat16)
            ops.swiglu_bwd(da, u)
            ops.rope_qkv(qkv, cos, sin, 16, 16, 64, 2048, False, True)
    elif args.case == "attn_fwd":
        from lbi_b200.ops.attention import flash_forward_packed

        b, h, t = 4, 16, 4096
        qkv = torch.randn(b * t, 3 * h * 64, device=dev).bfloat16()
        for _ in range(args.repeats):
            flash_forward_packed(qkv, b, t, h, h, 64, 0.125, kernel_mode="tcgen05")
    elif args.case == "ssd":
        from lbi_b200.ops.ssd import ssd_chunk_scan_cuda

        b, l, h, n = 2, 8192, 24, 64
        x = torch.randn(b, l, h, 64, device=dev).bfloat16()
        dt = torch.rand(b, l, h, device=dev) * 0.1 + 0.001
        a = -(torch.rand(h, device=dev) * 8 + 1)
        bm = (torch.randn(b, l, 1, n, device=dev) * 0.5).bfloat16()
        cm = (torch.randn(b, l, 1, n, device=dev) * 0.5).bfloat16()
        with torch.no_grad():
            for _ in range(args.repeats):
                ssd_chunk_scan_cuda(x, dt, a, bm, cm, D=torch.ones(h, device=dev))
    elif args.case == "ssd_bwd":
        from lbi_b200.ops.ssd import ssd_chunk_scan_cuda

        b, l, h, n = 2, 8192, 24, 128
        x = torch.randn(b, l, h, 64, device=dev).bfloat16().requires_grad_(True)
        dt = (torch.rand(b, l, h, device=dev) * 0.1 + 0.001).requires_grad_(True)
        a = (-(torch.rand(h, device=dev) * 8 + 1)).requires_grad_(True)
        bm = (torch.randn(b, l, 1, n, device=dev) * 0.5).bfloat16().requires_grad_(True)
        cm = (torch.randn(b, l, 1, n, device=dev) * 0.5).bfloat16().requires_grad_(True)
        d = torch.ones(h, device=dev, requires_grad=True)
        gy = torch.randn(b, l, h, 64, device=dev).bfloat16()
        for _ in range(args.repeats):
            y = ssd_chunk_scan_cuda(x, dt, a, bm, cm, D=d)
            torch.autograd.grad(y, (x, dt, a, bm, cm, d), gy)
    elif args.case == "mamba_elementwise":
        from lbi_b200.backbones.mamba3.siso import _WidePrepFunction
        from lbi_b200.backbones.norms import gated_rms_norm

        b, l, h, n = 8, 4096, 24, 128
        x = torch.randn(b, l, h * 64, device=dev).bfloat16().requires_grad_(True)
        z = torch.randn(b, l, h * 64, device=dev).bfloat16().requires_grad_(True)
        w = torch.ones(h * 64, device=dev, requires_grad=True)
        gy = torch.randn(b, l, h * 64, device=dev).bfloat16()
        q = torch.randn(b, l, 1, n, device=dev).bfloat16()
        k = torch.randn(b, l, 1, n, device=dev).bfloat16()
        qb, kb = torch.randn(h, n, device=dev), torch.randn(h, n, device=dev)
        theta = torch.rand(b, l, h, 32, device=dev) * 6.28
        gamma, scale = torch.rand(b, l, h, device=dev), torch.rand(b, l, h, device=dev)
        dqr, dkr, dqk = torch.randn(b, l, h, n, device=dev), torch.randn(b, l, h, n, device=dev), torch.randn(b, l, h, device=dev)
        for _ in range(args.repeats):
            y = gated_rms_norm(x, w, eps=1e-5, z=z, norm_before_gate=True, group_size=64)
            torch.autograd.grad(y, (x, z, w), gy)
            _WidePrepFunction.apply(q, k, qb, kb, theta, gamma, scale)
            ops.ext().siso_prep_bwd(q, k, qb, kb, theta, gamma, scale, dqr, dkr, dqk)
    elif args.case == "prep_bwd":
        b, reps, l, h, n = 2, 16, 1024, 24, 128
        q = torch.randn(b, l, 1, n, device=dev).bfloat16()
        k = torch.randn(b, l, 1, n, device=dev).bfloat16()
        qb, kb = torch.randn(h, n, device=dev), torch.randn(h, n, device=dev)
        theta = torch.rand(b, l, h, 32, device=dev) * 6.28
        gamma, scale = torch.rand(b, l, h, device=dev), torch.rand(b, l, h, device=dev)
        dqr = torch.randn(reps * b, l, h, n, device=dev).bfloat16()
        dkr = torch.randn(reps * b, l, h, n, device=dev).bfloat16()
        dqk = torch.randn(reps * b, l, h, device=dev)
        for _ in range(args.repeats):
            ops.ext().siso_prep_bwd(q, k, qb, kb, theta, gamma, scale, dqr, dkr, dqk, False, False)
    elif args.case in ("chunk_bwd", "chunk_bwd_ssd"):
        from lbi_b200.ops import ssd

        per_head = args.case == "chunk_bwd"
        b, reps, l, h, n = 1, 16, 1024, 24, 128
        g = h if per_head else 1
        v = torch.randn(b, l, h, 64, device=dev).bfloat16()
        bk = (torch.randn(b, l, g, n, device=dev) * 0.4).bfloat16()
        cq = (torch.randn(b, l, g, n, device=dev) * 0.4).bfloat16()
        a = -(torch.rand(b, l, h, device=dev) * 0.08 + 0.002)
        w = None if per_head else torch.rand(b, l, h, device=dev) * 0.1 + 0.01
        skip = torch.randn(b, l, h, device=dev) if per_head else None
        gy = torch.randn(reps * b, l, h, 64, device=dev).bfloat16()
        _, _, states = ssd.scan_generic(v, bk, cq, a, w, None, strict=per_head, per_head=per_head)
        for _ in range(args.repeats):
            ssd.chunk_backward(v, gy, bk, cq, a, w, skip, states, per_head=per_head, strict=per_head, dv_bf16=per_head, dn_bf16=True)
    elif args.case == "mamba_glue":
        from lbi_b200.ops import mamba as mops

        b, reps, l, h, s = 2, 8, 1024, 24, 32
        n = b * l
        y, z = torch.randn(n, 1536, device=dev).bfloat16(), torch.randn(n, 1536, device=dev).bfloat16()
        dyg = torch.randn(reps * n, 1536, device=dev).bfloat16()
        small = mops.siso_small_fwd(*(torch.randn(n, h, device=dev) for _ in range(3)), torch.randn(n, s, device=dev),
                                    torch.randn(h, device=dev) - 2.0, 1e-4, b, l)
        cots = [torch.randn(reps * b, l, h, device=dev) for _ in range(3)]
        dtheta = torch.randn(reps * b, l, h, s, device=dev)
        parts = (3072, 128, 128)
        xc = torch.randn(n, sum(parts), device=dev).bfloat16()
        wc, bc = torch.randn(sum(parts), 4, device=dev) * 0.5, torch.zeros(sum(parts), device=dev)
        for _ in range(args.repeats):
            mops.gate_silu_fwd(y, z)
            mops.gate_silu_bwd(dyg, y, z)
            mops.siso_small_fwd(*(torch.randn(n, h, device=dev) for _ in range(3)), torch.randn(n, s, device=dev),
                                torch.randn(h, device=dev) - 2.0, 1e-4, b, l)
            mops.siso_small_bwd(small, cots[0], dtheta, cots[1], cots[2], out_dtype=torch.bfloat16)
            pre, acts = mops.conv_silu_fwd(xc, wc, bc, b, l, parts)
            d = [torch.randn(reps * n, pp, device=dev).bfloat16() for pp in parts]
            out = torch.empty(reps * n, sum(parts) + 64, device=dev).bfloat16()
            mops.conv_silu_bwd(d, pre, wc, b, l, out, 64)
            mops.conv_silu_wgrad([t[:n] for t in d], pre, xc, 4, b, l)
    elif args.case == "small":
        from lbi_b200.interfaces.vector_mlp import VectorMLPHead, head_forward_cached, head_input_jacobian_t, head_parameter_vjp

        head = VectorMLPHead(1024, 128, 1024).cuda()
        x = torch.randn(4, 1024, device=dev)
        gbasis = torch.randn(4, 128, 128, device=dev)
        sink = {id(p): torch.zeros_like(p) for p in head.parameters()}
        mats = torch.randn(4, 7, 128, 128, device=dev) / 16
        offs = torch.randn(4, 7, 128, device=dev)
        table = torch.randn(32768, 1024, device=dev).bfloat16()
        ids = torch.randint(0, 32768, (32768,), device=dev)
        flat = torch.randn(64 * 1024 * 1024, device=dev)
        m1, m2, sh = torch.zeros_like(flat), torch.zeros_like(flat), torch.zeros(flat.numel(), device=dev, dtype=torch.bfloat16)
        sq = torch.zeros(1, device=dev)
        normed = torch.randn(8192, 1024, device=dev).bfloat16()
        tgt = torch.randint(0, 32768, (8192,), device=dev)
        with torch.no_grad():
            for _ in range(args.repeats):
                yv, cache = head_forward_cached(head, x)
                head_parameter_vjp(head, cache, torch.randn_like(yv), lambda p: sink[id(p)])
                head_input_jacobian_t(head, x, gbasis)
                ops.affine_suffix_scan(mats, offs, seed=offs[:, 0].contiguous())
                ops.ext().matrix_norms(mats.reshape(-1, 128, 128), 8) if hasattr(ops.ext(), "matrix_norms") else None
                rows = ops.embedding_fwd(ids, table, torch.bfloat16)
                ops.embedding_scatter_add(torch.zeros(32768, 1024, device=dev), ids, rows)
                ops.ext().sumsq_(flat, sq)
                ops.ext().adamw_step_(flat, flat * 1e-3, m1, m2, sh, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, sq, 1.0)
                ops.lm_head_cross_entropy(normed, table, tgt, 1.0 / 8192)
                ops.mean_pool_tokens(rows, 16, 2048)
    else:
        mats = torch.randn(8, 32, 256, 256, device=dev) / 16
        for _ in range(args.repeats):
            ops.suffix_scan_pullbacks(mats)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(torch.zeros(1, device=dev)) == 0
    print("done")


if __name__ == "__main__":
    main()
