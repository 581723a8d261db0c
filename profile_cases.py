"""Small single-kernel cases for profiling one kernel of the library in isolation.

    python profile_cases.py attn  --L 16384 --H 8  [--iters 3]
    python profile_cases.py gemm  --M 8192 --N 12288 --K 4096 [--epi plain|gated|swiglu]
    python profile_cases.py quant --M 36436 --K 4096 [--kind plain|fp8|normmod|rot|normmod_rot]
    python profile_cases.py prepass --L 16384 --H 8

Each case builds seeded random inputs on the device, runs the kernel `--iters` times and prints the mean time
from CUDA events, so the same command line serves a plain timing run and a profiler capture.
"""
import argparse

import torch

from rapid_h3_b200 import _lib, attn_int8, gemm, quantizers


def _time(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    _lib.check_status()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["attn", "gemm", "quant", "prepass", "conv", "vae", "mma_rate"])
    ap.add_argument("--L", type=int, default=16384)
    ap.add_argument("--H", type=int, default=8)
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=12288)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--epi", default="plain")
    ap.add_argument("--kind", default="plain")
    ap.add_argument("--T", type=int, default=36)
    ap.add_argument("--HH", type=int, default=24)
    ap.add_argument("--WW", type=int, default=42)
    ap.add_argument("--Cin", type=int, default=512)
    ap.add_argument("--Cout", type=int, default=512)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--rotate", action="store_true", help="attn / prepass: the token-scaled numerics")
    ap.add_argument("--rope", action="store_true", help="prepass: with the per-head RMSNorm + RoPE fused in")
    ap.add_argument("--no-stats", action="store_true", help="conv: without the GroupNorm partial sums")
    ap.add_argument("--single-cta", action="store_true", help="gemm / conv / vae: the single-CTA kernels instead of CTA pairs")
    a = ap.parse_args()
    if a.single_cta:
        _lib.lib().rh3_gemm_use_pairs(0)
    g = torch.Generator(device="cuda").manual_seed(0)

    def randn(*shape):
        return torch.randn(*shape, device="cuda", generator=g)

    if a.case == "mma_rate":
        # retire rate of back-to-back tcgen05 MMAs from shared memory, per operand kind; short bursts and a run of
        # about a second (the clocks the GPU holds under its power cap differ between the two)
        import ctypes
        for kind, name in ((0, "int8"), (1, "e4m3"), (2, "bf16")):
            for rnd in (0, 1):
                for groups, reps, label in ((2000, 3, "burst"), (20000, 12, "sustained")):
                    ops = ctypes.c_double(0)

                    def fn():
                        _lib.call("rh3_selftest_mma_rate", kind, groups, rnd, 0, ctypes.addressof(ops), _lib.stream())
                    ms = _time(fn, reps)
                    print(f"mma_rate {name} {'random' if rnd else 'zero'} operands, {label}: {ms:.3f} ms per launch, "
                          f"{ops.value / ms / 1e9:.0f} TOP/s", flush=True)
        # the issuing thread's own cost: the GEMM main loop's issue pattern on zero operands at full clock
        for pattern, name in ((0, "64 MMAs per commit"), (1, "ring, descriptors rebuilt per stage"),
                              (2, "ring, descriptors kept in registers"),
                              (3, "ring, whole warp in the loop, one elected lane issues"), (0, "64 MMAs per commit (again)")):
            ops = ctypes.c_double(0)

            def fn():
                _lib.call("rh3_selftest_mma_rate", 0, 2000, 0, pattern, ctypes.addressof(ops), _lib.stream())
            ms = _time(fn, 3)
            print(f"mma_rate int8 zero operands, {name}: {ms:.3f} ms per launch, {ops.value / ms / 1e9:.0f} TOP/s", flush=True)
        # 128-column MMAs (the convolution's narrow tiles) against 256-column ones, random operands
        for kind, name in ((2, "bf16"), (0, "int8")):
            for pattern, cols in ((0, 256), (4, 128)):
                ops = ctypes.c_double(0)

                def fn():
                    _lib.call("rh3_selftest_mma_rate", kind, 2000, 1, pattern, ctypes.addressof(ops), _lib.stream())
                ms = _time(fn, 3)
                print(f"mma_rate {name} random operands, {cols}-column MMAs: {ms:.3f} ms per launch, {ops.value / ms / 1e9:.0f} TOP/s",
                      flush=True)
        # the GEMM main loop without an epilogue: MMA rate against the bytes an SM takes in per stage
        for src_mb, where in ((48, "L2-resident source (48 MB)"), (2048, "HBM-resident source (2 GB)")):
            src = torch.randint(-127, 128, (src_mb << 20,), device="cuda", dtype=torch.int8)
            for fill in (0, 16384, 32768, 49152):
                ops = ctypes.c_double(0)

                def fn():
                    _lib.call("rh3_selftest_mma_feed", src.data_ptr(), src.numel(), 40000, fill, ctypes.addressof(ops), _lib.stream())
                ms = _time(fn, 3)
                print(f"mma_feed {where}, {fill // 1024} KB per stage: {ms:.3f} ms per launch, {ops.value / ms / 1e9:.0f} TOP/s, "
                      f"{148 * 40000 * fill / ms / 1e9:.1f} TB/s taken in", flush=True)
            del src
        return
    if a.case == "conv":
        from rapid_h3_b200 import vae
        x = randn(1, a.T, a.HH, a.WW, a.Cin).to(torch.bfloat16)
        w = (0.02 * randn(a.Cout, 27, a.Cin)).to(torch.bfloat16)
        ms = _time(lambda: vae.conv3d_causal(x, w, want_stats=a.Cout % 32 == 0 and not a.no_stats), a.iters)
        fl = 2.0 * a.T * a.HH * a.WW * a.Cin * a.Cout * 27
        print(f"conv3d {a.T}x{a.HH}x{a.WW} {a.Cin}->{a.Cout}: {ms:.3f} ms, {fl / ms / 1e9:.1f} TFLOP/s")
        return
    if a.case == "vae":
        from rapid_h3_b200 import vae
        dec = vae.VAEDecoder(seed=0)
        latent = randn(1, 16, a.T, a.HH, a.WW).to(torch.bfloat16)
        ms = _time(lambda: dec.decode(latent), a.iters)
        print(f"vae decode latent 16x{a.T}x{a.HH}x{a.WW}: {ms:.2f} ms, {dec.flops(a.T, a.HH, a.WW) / ms / 1e9:.1f} TFLOP/s")
        return
    if a.case in ("attn", "prepass"):
        q = randn(a.L, a.H, 128).to(torch.bfloat16)
        k = (randn(a.L, a.H, 128) + 2 * randn(1, a.H, 128)).to(torch.bfloat16)
        v = randn(a.L, a.H, 128).to(torch.bfloat16)
        pre_fn = attn_int8.tok_prepass if a.rotate else attn_int8.int8_prepass
        main_fn = attn_int8.attention_tok_pre if a.rotate else attn_int8.attention_pre
        if a.case == "prepass":
            args = ()
            if a.rope:
                w = torch.ones(128, device="cuda", dtype=torch.bfloat16)
                args = (randn(a.L, 48, 2, 2).to(torch.bfloat16), w, w, 1e-5, None, k)
            ms = _time(lambda: pre_fn(q, k, v, *args), a.iters)
            print(f"prepass L={a.L} H={a.H} rotate={a.rotate} rope={a.rope}: {ms:.3f} ms")
            return
        pre = pre_fn(q, k, v)
        out = torch.empty(a.L, a.H, 128, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda: main_fn(pre, out=out), a.iters)
        print(f"attn L={a.L} H={a.H} rotate={a.rotate}: {ms:.3f} ms, {4 * a.L * a.L * 128 * a.H / ms / 1e9:.1f} TFLOP/s")
    elif a.case == "gemm":
        xq = torch.randint(-127, 128, (a.M, a.K), device="cuda", dtype=torch.int8, generator=g)
        wq = torch.randint(-127, 128, (a.N, a.K), device="cuda", dtype=torch.int8, generator=g)
        xs = torch.rand(a.M, device="cuda", generator=g) * 1e-3
        ws = torch.rand(a.N, device="cuda", generator=g) * 1e-3
        if a.epi == "swiglu":
            out = torch.empty(a.M, a.N // 2, device="cuda", dtype=torch.bfloat16)
            fn = lambda: gemm.int8_gemm_swiglu(xq, xs, wq, ws, out=out)  # noqa: E731
        elif a.epi == "gated":
            resid = randn(a.M, a.N).to(torch.bfloat16)
            gate = randn(a.N).to(torch.bfloat16)
            fn = lambda: gemm.int8_gemm_gated_residual(xq, xs, wq, ws, gate, resid)  # noqa: E731
        else:
            out = torch.empty(a.M, a.N, device="cuda", dtype=torch.bfloat16)
            fn = lambda: gemm.int8_gemm(xq, xs, wq, ws, out=out)  # noqa: E731
        ms = _time(fn, a.iters)
        print(f"gemm {a.epi} M={a.M} N={a.N} K={a.K}: {ms:.3f} ms, {2 * a.M * a.N * a.K / ms / 1e9:.1f} TOP/s")
    else:
        x = randn(a.M, a.K).to(torch.bfloat16)
        if a.kind == "fp8":
            fn = lambda: quantizers.quant_rows(x)  # noqa: E731
        elif a.kind == "rot":
            fn = lambda: quantizers.rot_quant_rows_i8(x)  # noqa: E731
        elif a.kind in ("normmod", "normmod_rot"):
            tab = randn(2, 6 * a.K) * 0.1
            idx = torch.zeros(a.M, dtype=torch.int32, device="cuda")
            w = torch.ones(a.K, device="cuda", dtype=torch.bfloat16)
            fn = lambda: quantizers.norm_mod_rot_quant_rows_i8(x, w, 1e-6, idx, tab[:, :a.K], tab[:, a.K:2 * a.K],
                                                                rotate=a.kind == "normmod_rot")  # noqa: E731
        else:
            fn = lambda: quantizers.quant_rows_i8(x)  # noqa: E731
        ms = _time(fn, a.iters)
        print(f"quant {a.kind} M={a.M} K={a.K}: {ms:.3f} ms, {a.M * a.K * 3 / ms / 1e6:.0f} GB/s (3 B/element)")


if __name__ == "__main__":
    main()
