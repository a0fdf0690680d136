"""Time one kernel of the library in isolation, at the sizes of a configuration.

    python -m infero_b200.tools.kernel_bench KERNEL [--tokens T] [--context L] [--batch B]
        [--reps N] [--hidden 3584 --heads 28 --kv-heads 4 --head-dim 128 --intermediate 18944]

KERNEL: gemm_qkv | gemm_o | gemm_gate_up | gemm_down | gemm_head | attn_prefill | attn_decode
        | attn_decode_fused (bias, rotary, cache append and attention from the q/k/v partial sums)
        | gemm_o_norm | gemm_down_norm (the product adds itself to the residual stream and prepares the norm)
        | norm | rope | swiglu

The kernel runs on several copies of its inputs (enough to exceed the L2 cache), back to back; a
round over all copies is timed with CUDA events after warm-up, and the median time per launch is
reported with the achieved GB/s or TFLOP/s.  The reference times whole passes the same way (crates/model/examples/
prefill_profile.rs:38-55) and per kernel with events (crates/cuda/src/profile.rs:28-130).
This is also the small case to put under ``ncu``: one kernel, a few launches.
"""
from __future__ import annotations

import argparse
import math
import sys


def _copies(bytes_per_copy: int, reps: int) -> int:
    l2 = 160 << 20
    return max(2, min(reps, -(-l2 // max(1, bytes_per_copy)) + 1))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench")
    ap.add_argument("kernel")
    ap.add_argument("--tokens", type=int, default=2048, help="rows of the activation (prefill) or batch (decode)")
    ap.add_argument("--context", type=int, default=4096, help="cached tokens per request (attn_decode)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hidden", type=int, default=3584)
    ap.add_argument("--heads", type=int, default=28)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--intermediate", type=int, default=18944)
    ap.add_argument("--vocab", type=int, default=152064)
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)

    import torch
    from infero_b200 import kernels as K
    from infero_b200.kernels import attention as A
    from infero_b200.kernels import tc_gemm
    K.lib()
    dev = "cuda:0"
    bf = torch.bfloat16
    d, H, Hkv, D, ff = args.hidden, args.heads, args.kv_heads, args.head_dim, args.intermediate
    T = args.tokens
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * scale).to(dtype)

    name = args.kernel
    runs = []          # one callable per copy
    flops = bytes_ = 0.0
    if name in ("gemm_o_norm", "gemm_down_norm"):
        # few rows only: the cluster-summed product that updates the residual stream
        T = min(T, 256) if args.tokens != 2048 else args.batch
        N, Kd = (d, H * D) if name == "gemm_o_norm" else (d, ff)
        n = _copies(N * Kd * 2, args.reps)
        norm_w = rnd(d, dtype=torch.float32) + 1
        for _ in range(n):
            a, w = rnd(T, Kd), rnd(N, Kd, scale=0.02)
            resid = rnd(T, N, dtype=torch.float32)
            runs.append(lambda a=a, w=w, resid=resid: tc_gemm.residual_norm(a, w, resid, None, norm_w))
        flops = 2.0 * T * N * Kd
        bytes_ = 2.0 * (N * Kd + T * Kd) + 10.0 * T * N
    elif name.startswith("gemm_"):
        N, Kd = {"gemm_qkv": ((H + 2 * Hkv) * D, d), "gemm_o": (d, H * D), "gemm_gate_up": (2 * ff, d),
                 "gemm_down": (d, ff), "gemm_head": (args.vocab, d)}[name]
        n = _copies(N * Kd * 2, args.reps)
        for _ in range(n):
            a, w = rnd(T, Kd), rnd(N, Kd, scale=0.02)
            if name == "gemm_gate_up":
                out = torch.empty((T, N // 2), dtype=bf, device=dev)
                runs.append(lambda a=a, w=w, out=out: tc_gemm.gemm_swiglu(a, w, out))
            elif T <= 256:
                runs.append(lambda a=a, w=w: tc_gemm.partials(a, w))
            else:
                out = torch.empty((T, N), dtype=bf, device=dev)
                runs.append(lambda a=a, w=w, out=out: tc_gemm.gemm(a, w, None, out))
        flops = 2.0 * T * N * Kd
        bytes_ = 2.0 * (N * Kd + T * Kd + T * N)
    elif name in ("attn_decode", "attn_prefill", "attn_decode_fused"):
        P = args.page_size
        B = args.batch if name != "attn_prefill" else 1
        L = args.context if name != "attn_prefill" else T
        blocks = -(-L // P)
        pages = B * blocks
        n = _copies(2 * pages * Hkv * P * D * 2, args.reps)
        scale = 1.0 / math.sqrt(D)
        for c in range(n):
            kc, vc = rnd(pages, Hkv, P, D), rnd(pages, Hkv, P, D)
            perm = torch.randperm(pages, generator=torch.Generator().manual_seed(c)).to(torch.int32)
            table = perm.view(B, blocks).to(dev).contiguous()
            if name == "attn_decode_fused":
                width = (H + 2 * Hkv) * D
                splits_in = tc_gemm.plan(B, width, d, dev)[0]
                qkv = K.Partials(rnd(splits_in, B, width, dtype=torch.float32), rnd(width, dtype=torch.float32))
                inv = (1e6 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).to(torch.float32).to(dev)
                out = torch.empty((B, H * D), dtype=bf, device=dev)
                pos = torch.full((B,), L - 1, dtype=torch.int32, device=dev)
                ent = torch.arange(B, dtype=torch.int32, device=dev)
                chunk, splits = A.plan_decode(B, Hkv, H // Hkv, L)
                runs.append(lambda qkv=qkv, out=out, kc=kc, vc=vc, table=table, ent=ent, pos=pos:
                            A.decode_fused(qkv, out, kc, vc, table, ent, pos, inv, H, Hkv, D, P, None, scale, chunk, splits))
            elif name == "attn_decode":
                q = rnd(B, H * D)
                out = torch.empty((B, H * D), dtype=bf, device=dev)
                pos = torch.full((B,), L - 1, dtype=torch.int32, device=dev)
                ent = torch.arange(B, dtype=torch.int32, device=dev)
                runs.append(lambda q=q, out=out, kc=kc, vc=vc, table=table, ent=ent, pos=pos:
                            A.attention_any(q, out, kc, vc, table, ent, pos, H, Hkv, D, P, None, scale,
                                            q_lens=[1] * B, pos0=[L - 1] * B))
            else:
                q = rnd(T, H * D)
                out = torch.empty((T, H * D), dtype=bf, device=dev)
                pos = torch.arange(T, dtype=torch.int32, device=dev)
                ent = torch.zeros(T, dtype=torch.int32, device=dev)
                e_start = torch.zeros(1, dtype=torch.int32, device=dev)
                e_len = torch.full((1,), T, dtype=torch.int32, device=dev)
                e_pos0 = torch.zeros(1, dtype=torch.int32, device=dev)
                runs.append(lambda q=q, out=out, kc=kc, vc=vc, table=table, ent=ent, pos=pos, a=e_start, b=e_len, c_=e_pos0:
                            A.attention_any(q, out, kc, vc, table, ent, pos, H, Hkv, D, P, None, scale,
                                            q_lens=[T], pos0=[0], entry_q_start=a, entry_q_len=b, entry_pos0=c_))
        if name != "attn_prefill":
            bytes_ = 2.0 * B * L * Hkv * D * 2
            flops = 4.0 * B * L * H * D
        else:
            flops = 2.0 * T * T * H * D          # causal
            bytes_ = 2.0 * (2 * T * Hkv * D + 2 * T * H * D)
    elif name == "norm":
        n = _copies(T * d * 8, args.reps)
        w = rnd(d) + 1
        for _ in range(n):
            x, delta = rnd(T, d, dtype=torch.float32), rnd(T, d)
            out = torch.empty((T, d), dtype=bf, device=dev)
            runs.append(lambda x=x, delta=delta, out=out: K.add_rmsnorm(x, delta, w, 1e-6, out))
        bytes_ = T * d * (4 + 2 + 4 + 2)
    elif name == "swiglu":
        n = _copies(T * ff * 6, args.reps)
        for _ in range(n):
            gu = rnd(T, 2 * ff)
            out = torch.empty((T, ff), dtype=bf, device=dev)
            runs.append(lambda gu=gu, out=out: K.swiglu(gu, out))
        bytes_ = T * ff * 6
    elif name == "rope":
        # rotary on q and k in place and the append of k and v to the cache, T tokens of one request
        P = args.page_size
        blocks = -(-T // P)
        n = _copies(T * (H + 2 * Hkv) * D * 2 + 2 * blocks * Hkv * P * D * 2, args.reps)
        inv = (1e6 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).to(torch.float32).to(dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        ent = torch.zeros(T, dtype=torch.int32, device=dev)
        for c in range(n):
            qkv = rnd(T, (H + 2 * Hkv) * D)
            kc = torch.zeros((blocks, Hkv, P, D), dtype=bf, device=dev)
            vc = torch.zeros_like(kc)
            table = torch.randperm(blocks, generator=torch.Generator().manual_seed(c)).to(torch.int32).view(1, blocks).to(dev)
            runs.append(lambda qkv=qkv, kc=kc, vc=vc, table=table:
                        K.rope_cache(qkv, pos, ent, table, inv, kc, vc, H, Hkv, D, P))
        bytes_ = 2.0 * T * D * (2 * (H + Hkv) + 3 * Hkv)       # q and k read and written, v read, k and v appended
    else:
        print(f"kernel_bench: unknown kernel {name!r}", file=sys.stderr)
        return 2

    for i in range(args.warmup):
        runs[i % len(runs)]()
    torch.cuda.synchronize()
    if tc_gemm.error_flag():
        print(f"kernel_bench: {name} raised error flag {tc_gemm.error_flag()} during warm-up (a wait inside the "
              "kernel ran out); not timed", file=sys.stderr)
        return 1
    # one timed repetition = every input copy once, back to back (the launches queue up, so the
    # host's launch cost is hidden behind kernels that take longer than it)
    from .clocks import ClockSampler
    clocks = ClockSampler()
    clocks.on = True
    times = []
    for i in range(args.reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for run in runs:
            run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / len(runs))
    times.sort()
    us = times[len(times) // 2]
    err = tc_gemm.error_flag()
    line = f"{name}: {us:.1f} us per launch, median of {args.reps} rounds over {len(runs)} input copies (min {times[0]:.1f})"
    if bytes_:
        line += f", {bytes_ / us / 1e3:.0f} GB/s"
    if flops:
        line += f", {flops / us / 1e6:.1f} TFLOP/s"
    c = clocks.summary()
    if c.get("sm_mhz"):
        line += f"; SM clock {c['sm_mhz']} MHz of {c['sm_max_mhz']}" + (f" ({', '.join(c['reasons'])})" if c["reasons"] else "")
    print(line + (f"  [error flag {err}]" if err else ""))
    return 0


if __name__ == "__main__":
    sys.exit(main())
