#!/usr/bin/env python
"""Benchmark of the quantized H3-shaped DiT step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload full|draft|block]

One "step" = one evaluation of the 48-block transformer on the 768x1344x141-frame token grid
(36x24x42 = 36,288 video tokens + 148 audio tokens, CFG batch 2, 512 text tokens), all Linear layers
W8A8 row-wise int8, INT8-QK / FP8-PV attention. For N > 1 (launched by torch.distributed.run) the step is
sequence-parallel: token shards + Ulysses all-to-all around self-attention (strong scaling).
Rank 0 prints ONE JSON line. `--impl reference` times the reference's CPU path (its PyTorch emulation,
restated in oracle/) on the host cores, on a bounded sample extrapolated to a full step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (grid T,H,W, audio tokens, batch, text tokens, blocks)
    "full": ((36, 24, 42), 148, 2, 512, 48),
    "draft": ((36, 17, 29), 148, 2, 512, 48),
    "block": ((36, 24, 42), 148, 1, 512, 1),
}
VAE_LATENT = (16, 36, 24, 42)  # -> RGB 3 x 141 x 768 x 1344


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# DRAM traffic of the self-attention main kernel from one ncu capture (profiles/attn_int8_kernel_dram_block_workload.md):
# dram__bytes_read.sum + dram__bytes_write.sum of the launch at Lq = Lk = 36,436, H = 32, and the first 16 hex digits of
# the SHA-256 of the kernel source the capture was made with. A different source means the figure is stale: the
# bench then reports traffic null instead of a number that no longer belongs to the kernel it times.
ATTN_TRAFFIC = {"bytes": 718.51e6, "lq": 36436, "lk": 36436, "heads": 32, "attn_cu_sha16": "2e9e9add32425609"}


def attn_traffic(alg_bytes_this_launch):
    import hashlib
    src = os.path.join(ROOT, "rapid_h3_b200", "csrc", "attn.cu")
    sha = hashlib.sha256(open(src, "rb").read()).hexdigest()[:16]
    if sha != ATTN_TRAFFIC["attn_cu_sha16"]:
        return None, f"no capture for this kernel source (sha {sha})"
    t = ATTN_TRAFFIC
    ref = t["heads"] * 128 * (t["lq"] + 2 * t["lk"]) + t["heads"] * 128 * 2 * t["lq"]
    return t["bytes"] * alg_bytes_this_launch / ref, "bytes per launch (ncu capture, scaled by operand + output bytes)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------
# CPU port (the oracle) timed on a bounded sample and extrapolated to one full step
# ---------------------------------------------------------------------------------------------------
def cpu_port_step_seconds(workload, rows=1024, attn_rows=256):
    """Seconds per step of the reference's CPU path, extrapolated: row-local work (quantizers, GEMMs,
    epilogues) is timed on `rows` tokens and scaled linearly; attention is timed for one head on
    `attn_rows` query rows against all keys and scaled to H heads x all rows."""
    from oracle import attention as oa
    from oracle import linear as ol
    from oracle import quant as oq
    from rapid_h3_b200.model import H3Config
    cfg = H3Config()
    grid, n_audio, batch, text_len, blocks = WORKLOADS[workload]
    s = grid[0] * grid[1] * grid[2] + n_audio
    d, f = cfg.d_model, cfg.mlp_hidden
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, d, generator=g).to(torch.bfloat16)
    idx = torch.zeros(rows, dtype=torch.int32)
    tab = 0.1 * torch.randn(1, d, generator=g)
    w_norm = torch.ones(d, dtype=torch.bfloat16)

    def qw(n, k):
        return (torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8), torch.rand(1, n, generator=g) * 1e-3)

    t0 = time.perf_counter()
    lin = 0.0
    for n, k, kind in ((3 * d, d, "plain"), (d, d, "gated"), (d, d, "plain"), (d, d, "gated"), (2 * f, d, "swiglu"),
                       (d, f, "gated")):
        wq, ws = qw(n, k)
        a = torch.randn(rows, k, generator=g).to(torch.bfloat16)
        t1 = time.perf_counter()
        if kind == "swiglu" or n == 3 * d:
            xq, xs = oq.norm_mod_quant_rows_i8(a, w_norm[:k], 1e-6, idx, tab[:, :k], tab[:, :k])
        else:
            xq, xs = ol.quantize_rows(a, "int8_rowwise")
        acc = ol.int_mm(xq, wq)
        if kind == "plain":
            ol.dequant(acc, xs, ws)
        elif kind == "gated":
            ol.gated_residual(acc, xs, ws, w_norm[:n], x[:, :n] if n <= d else a[:, :n])
        else:
            ol.swiglu_epilogue(acc, xs, ws)
        lin += time.perf_counter() - t1
    # per-head RMSNorm + 3-D RoPE of q and k (self-attention) and RMSNorm of q (cross-attention), on `rows` tokens
    from oracle import inputs as oi
    rr_rows = min(rows, 2048)
    qk = torch.randn(rr_rows, cfg.heads, 128, generator=g).to(torch.bfloat16)
    rope_tab = oi.rope_table(oi.random_positions(rr_rows, seed=1))
    t1 = time.perf_counter()
    oa.rmsnorm_rope(qk, w_norm[:128], 1e-5, rope_tab)
    oa.rmsnorm_rope(qk, w_norm[:128], 1e-5, rope_tab)
    oa.rmsnorm_rope(qk, w_norm[:128], 1e-5, None)
    t_rr = (time.perf_counter() - t1) * (rows / rr_rows)
    # AdaLN projection of the timestep embedding and the text K/V projection: once per block-sample, not per token
    t1 = time.perf_counter()
    torch.nn.functional.linear(torch.randn(1, d, generator=g).to(torch.bfloat16),
                               torch.randn(6 * d, d, generator=g).to(torch.bfloat16))
    cq, cs = ol.quantize_rows(torch.randn(text_len, cfg.text_dim, generator=g).to(torch.bfloat16), "int8_rowwise")
    wq, ws = qw(2 * d, cfg.text_dim)
    ol.dequant(ol.int_mm(cq, wq), cs, ws)
    t_once = time.perf_counter() - t1
    q, k, v = (torch.randn(s, 1, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    t1 = time.perf_counter()
    pre = oa.prepass(q, k, v)
    t_pre = time.perf_counter() - t1
    t1 = time.perf_counter()
    oa.attention_pre(pre, rows=torch.arange(attn_rows))
    t_attn = time.perf_counter() - t1
    # cross-attention: the same rows against the text keys
    t1 = time.perf_counter()
    oa.attention(q[:attn_rows], k[:text_len], v[:text_len])
    t_cross = time.perf_counter() - t1
    per_block_sample = ((lin + t_rr) * (s / rows) + t_once +
                        cfg.heads * (t_pre + (t_attn + t_cross) * (s / attn_rows)))
    total = per_block_sample * blocks * batch
    return total, {"rows": rows, "attn_rows": attn_rows, "sample_seconds": time.perf_counter() - t0,
                   "linear_s_per_rows": lin, "attn_s_per_head_rows": t_attn, "prepass_s_per_head": t_pre,
                   "rmsnorm_rope_s_per_rows": t_rr, "cross_attn_s_per_head_rows": t_cross, "once_per_block_s": t_once}


# bounded CPU sample shared by the cpu_baseline leg and the --impl reference arm (5-10 s of CPU work per step)
CPU_SAMPLE_ROWS, CPU_SAMPLE_ATTN_ROWS = 12288, 4096


def cpu_baseline_record(workload):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu_port_step_seconds(workload, rows=128, attn_rows=32)  # warm-up
    val, info = cpu_port_step_seconds(workload, rows=CPU_SAMPLE_ROWS, attn_rows=CPU_SAMPLE_ATTN_ROWS)
    return {"value": val, "unit": "s/step", "cores": cores, "kind": "port",
            "sample": (f"row-local ops of one block (quantizers, six GEMMs with their epilogues, RMSNorm + RoPE) on "
                       f"{info['rows']} of the tokens, self- and cross-attention of 1 head on {info['attn_rows']} query "
                       f"rows x all keys, AdaLN and the text K/V projection once ({info['sample_seconds']:.1f} s of CPU "
                       "work), scaled linearly to all rows, heads, blocks and the CFG batch")}


def vae_cpu_seconds():
    """CPU port of the VAE decode (oracle/vae.py): one 512 -> 512 causal conv on a 3 x 24 x 42 slab, scaled by the
    decoder's operation count (convolutions are >95 % of the decode)."""
    from oracle import vae as ov
    from rapid_h3_b200 import vae
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 3, 24, 42, 512, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(512, 27, 512, generator=g)).to(torch.bfloat16)
    ov.conv3d_causal(x[:, :1], w)
    t0 = time.perf_counter()
    ov.conv3d_causal(x, w)
    dt = time.perf_counter() - t0
    dec = vae.VAEDecoder.__new__(vae.VAEDecoder)
    dec.widths, dec.blocks = (512, 256, 128), 2
    return dt * dec.flops(*VAE_LATENT[1:]) / (2.0 * 3 * 24 * 42 * 512 * 512 * 27), dt


def run_reference(args, rank):
    if rank != 0:
        return
    if args.workload == "vae":
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        vals = [vae_cpu_seconds() for _ in range(max(args.steps, 1))]
        val = statistics.median(v for v, _ in vals)
        sample = (f"one 512->512 causal conv3d on a 3x24x42 slab ({vals[0][1]:.1f} s of CPU work per step), scaled by "
                  "the decoder's operation count")
        print(json.dumps({"impl": "reference", "metric": "VAE decode seconds, latent 16x36x24x42 -> RGB 3x141x768x1344",
                          "value": val, "unit": "s/decode", "n_gpus": args.gpus, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": val * 1e3, "higher_is_better": False,
                          "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
                          "config": {"workload": "vae_conv3d_decode", "latent": list(VAE_LATENT)},
                          "cpu_baseline": {"value": val, "unit": "s/decode", "cores": cores, "kind": "port", "sample": sample},
                          "e2e": {"value": val, "unit": "s/decode", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}),
              flush=True)
        return
    grid, n_audio, batch, text_len, blocks = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for _ in range(max(args.warmup, 1)):
        cpu_port_step_seconds(args.workload, rows=128, attn_rows=32)
    vals = []
    for _ in range(args.steps):
        v, info = cpu_port_step_seconds(args.workload, rows=CPU_SAMPLE_ROWS, attn_rows=CPU_SAMPLE_ATTN_ROWS)
        vals.append(v)
    val = statistics.median(vals)
    rec = {"impl": "reference", "metric": "H3 DiT step seconds @768x1344x141f", "value": val, "unit": "s/step",
           "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": val * 1e3,
           "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
           "data": "synthetic", "config": workload_config(args.workload, args.gpus),
           "cpu_baseline": {"value": val, "unit": "s/step", "cores": cores, "kind": "port",
                            "sample": f"per step: row-local ops of one block (quantizers, six GEMMs with their "
                                      f"epilogues, RMSNorm + RoPE) on {CPU_SAMPLE_ROWS} tokens + self- and cross-attention "
                                      f"of 1 head on {CPU_SAMPLE_ATTN_ROWS} query rows x all keys + AdaLN and the text K/V "
                                      f"projection once ({info['sample_seconds']:.1f} s of CPU work), scaled linearly to "
                                      "the full step; the same sample as the cpu_baseline leg of the GPU arm"},
           "e2e": {"value": val, "unit": "s/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(rec), flush=True)


ATTN_TEXT = {"fast": "int8 QK^T (block-64 scales, K smoothing) + fp8 e4m3 PV",
             "reference": "int8 QK^T (per-token scales after a 128-point Hadamard rotation, K smoothing) + u8 P x int8 V "
                          "with a per-tile fold"}


def workload_config(name, n, attn="fast"):
    grid, n_audio, batch, text_len, blocks = WORKLOADS[name]
    return {"workload": f"h3_dit_step_{name}", "token_grid": list(grid), "video_tokens": grid[0] * grid[1] * grid[2],
            "audio_tokens": n_audio, "cfg_batch": batch, "text_tokens": text_len, "blocks": blocks, "d_model": 4096,
            "heads": 32, "head_dim": 128, "mlp_hidden": 16384, "linear": "w8a8 int8 row-wise",
            "attention": ATTN_TEXT[attn],
            "parallelism": "single GPU" if n == 1 else f"sequence-parallel sp{n} (token shards + Ulysses all-to-all)",
            "l2": "every step streams >16 GB of weights and activations, far larger than the 126 MB L2"}


def tensor_probe():
    """Retire rate of back-to-back tcgen05 MMAs from shared memory on pseudo-random operands, held for about a
    second per kind (rh3_selftest_mma_rate): what the tensor pipe sustains under this GPU's power cap for int8 and
    e4m3 operands. MEASURED_PEAKS.json holds no 8-bit figure; this is the live one, reported beside it."""
    import ctypes
    import rapid_h3_b200 as r
    out = {}
    for kind, name in ((0, "int8_tops"), (1, "e4m3_tops")):
        ops = ctypes.c_double(0)

        def fn():
            r._lib.call("rh3_selftest_mma_rate", kind, 20000, 1, 0, ctypes.addressof(ops), r._lib.stream())
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(8):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = round(ops.value * 8 / e0.elapsed_time(e1) / 1e9, 1)
    r._lib.check_status()
    out["note"] = ("128x256x32 MMAs issued back to back by one thread per SM on pseudo-random shared-memory operands, "
                   "8 launches of about 0.1 s, CUDA events")
    return out


def vae_extras(local):
    """The second workload of the path beside the step record: the conv3d VAE decode of the benchmark latent on one
    GPU, latent resident, 3 warm-up + 3 timed decodes (CUDA events)."""
    from rapid_h3_b200 import vae
    c, t, h, w = VAE_LATENT
    dec = vae.VAEDecoder(latent_ch=c, seed=0, device=f"cuda:{local}")
    dev = torch.randn(1, c, t, h, w, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    for _ in range(3):
        dec.decode(dev)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        dec.decode(dev)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 3
    return {"vae_decode_ms": round(ms, 3), "vae_decode_tflops": round(dec.flops(t, h, w) / 1e9 / ms, 1),
            "vae_latent": list(VAE_LATENT)}


def run_vae(args, rank, world, local):
    """VAE decode of the benchmark latent (second workload of the hot path; time-sharded for N > 1)."""
    import torch.distributed as dist
    import rapid_h3_b200 as r
    from rapid_h3_b200 import vae
    c, t, h, w = VAE_LATENT
    dec = vae.VAEDecoder(latent_ch=c, seed=0, device=f"cuda:{local}")
    host = torch.randn(1, c, t, h, w, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).pin_memory()
    sp = vae.TimeShards(t) if world > 1 else None
    t0, t1 = (0, t) if sp is None else (sp.t0, sp.t1)
    dev = host.cuda()[:, :, t0:t1].contiguous()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out_host = None

    def step_e2e():
        nonlocal out_host
        rgb = dec.decode(host[:, :, t0:t1].cuda(non_blocking=True).contiguous(), sp=sp)
        if out_host is None:
            out_host = torch.empty(rgb.shape, dtype=rgb.dtype).pin_memory()
        out_host.copy_(rgb, non_blocking=True)

    def timed(fn, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / k], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(max(args.warmup, 3)):
        dec.decode(dev, sp=sp)
    sampler = ClockSampler(local)
    sampler.start()
    r._lib.launch_count = 0
    ms = timed(lambda: dec.decode(dev, sp=sp), args.steps)
    launches = r._lib.launch_count
    clocks = sampler.stop()
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    r._lib.check_status()
    pk = peaks()
    tflop = dec.flops(t, h, w) / 1e12
    achieved = tflop / (ms / 1e3)
    rec = {"metric": "VAE decode seconds, latent 16x36x24x42 -> RGB 3x141x768x1344", "value": ms / 1e3,
           "unit": "s/decode", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
           "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "vae_conv3d_decode", "latent": list(VAE_LATENT), "widths": [512, 256, 128],
                      "blocks_per_stage": 2, "parallelism": "single GPU" if world == 1 else f"time shards x{world}",
                      "l2": "activations of 0.6-0.9 GB per layer, far larger than the 126 MB L2"},
           "clocks": clocks,
           "e2e": {"value": ms_e2e / 1e3, "unit": "s/decode", "h2d_bytes_per_step": dev.numel() * 2,
                   "d2h_bytes_per_step": out_host.numel() * 2},
           "gpu_launches": launches // max(args.steps, 1) * args.steps,
           "roofline": {"bound": "tensor", "kernel": "conv3d_kernel (whole decode incl. GroupNorm/upsample)",
                        "achieved": achieved * world, "peak": pk["bf16_tflops_sustained"] * world, "unit": "TFLOP/s",
                        "frac": achieved / pk["bf16_tflops_sustained"], "traffic": None,
                        "peak_note": f"{pk['source']} sustained cuBLAS bf16"}}
    if rank == 0:
        print(json.dumps(rec), flush=True)


# ---------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="full", choices=sorted(WORKLOADS) + ["vae"])
    ap.add_argument("--mode", default="int8_rowwise", choices=["int8_rowwise", "int8_rot"],
                    help="linear recipe of the step: un-rotated row-wise int8 (the benchmark configuration) or the "
                         "H256-rotated recipe")
    ap.add_argument("--exchange", default="auto", choices=["nccl", "fused", "auto"],
                    help="N > 1: token <-> head exchanges as NCCL all-to-all, or done by the rope and attention kernels "
                         "themselves (stores into peer buffers); auto = fused, falling back to nccl if the peer "
                         "buffers cannot be set up")
    ap.add_argument("--overlap", default="auto", choices=["auto", "on", "off"],
                    help="run the CFG samples of a step side by side on two streams (auto: when N > 1, where it hides "
                         "the exchanges of the sequence-parallel step)")
    ap.add_argument("--attn", default="fast", choices=["fast", "reference"],
                    help="attention numerics: fast = block-64 Q/K, e4m3 V and P (the headline kernel); reference = "
                         "per-token rotated Q/K, int8 V, u8 P against the tile maximum (the reference's production numerics)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the VAE decode timing added to the N=1 step record")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    import rapid_h3_b200 as r
    from rapid_h3_b200.model import H3Config
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.workload == "vae":
        run_vae(args, rank, world, local)
        if world > 1:
            dist.destroy_process_group()
        return
    grid, n_audio, batch, text_len, blocks = WORKLOADS[args.workload]
    cfg = H3Config(n_blocks=blocks)
    rt = r.step.H3Runtime.random(cfg, seed=0, device=f"cuda:{local}", mode=args.mode)
    r.nodes.ATTN_ROTATE = args.attn == "reference"
    if r.nodes.ATTN_ROTATE and world > 1 and args.exchange == "auto":
        args.exchange = "nccl"   # the token-scaled kernel has no scattering epilogue
    s_total = grid[0] * grid[1] * grid[2] + n_audio
    # the CFG samples of a step are independent: with --overlap each runs on its own stream, and (N > 1) with its own
    # process group and exchange buffers, so one sample's exchanges hide under the other's kernels
    side_by_side = batch > 1 and (args.overlap == "on" or (args.overlap == "auto" and world > 1))
    streams = [torch.cuda.Stream() for _ in range(batch)] if side_by_side else None
    sp = None
    exchange = "none"
    if world > 1:
        groups = [dist.new_group(list(range(world))) for _ in range(batch)] if side_by_side else [None]
        sps = [r.sp.Ulysses(s_total, group=g) for g in groups]
        exchange = "nccl all_to_all_single"
        if args.exchange in ("fused", "auto"):
            try:
                for u in sps:
                    how = u.enable_fused(cfg.heads, cfg.head_dim, torch.device("cuda", local))
                exchange = f"kernel stores into peer buffers ({how})"
            except Exception as e:  # noqa: BLE001
                if args.exchange == "fused":
                    raise
                for u in sps:
                    u.fused = False
                print(f"[bench] peer buffers unavailable ({type(e).__name__}: {e}); using NCCL all-to-all", file=sys.stderr)
        sp = sps if side_by_side else sps[0]
    host = [t.pin_memory() for t in r.step.make_inputs(cfg, grid, n_audio, batch, text_len, seed=0)]
    dev = [t.cuda(non_blocking=True) for t in host]
    rope_dev = dev[3]
    out_host = [torch.empty((batch, cfg.latent_ch) + tuple(grid), dtype=torch.bfloat16).pin_memory(),
                torch.empty((batch, n_audio, cfg.latent_ch), dtype=torch.bfloat16).pin_memory()]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        return rt.step(dev[0], dev[1], dev[2], rope_dev, dev[4], sp=sp, streams=streams)

    def step_e2e():
        lat, aud, temb, ctx = (host[i].cuda(non_blocking=True) for i in (0, 1, 2, 4))
        v, a = rt.step(lat, aud, temb, rope_dev, ctx, sp=sp, streams=streams)
        out_host[0].copy_(v, non_blocking=True)
        out_host[1].copy_(a, non_blocking=True)

    def timed(fn, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / k], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(max(args.warmup, 3)):
        step_resident()
    r._lib.check_status()
    sampler = ClockSampler(local)
    sampler.start()
    r._lib.launch_count = 0
    r.timing.PHASES = {}
    ms_step = timed(step_resident, args.steps)
    launches = r._lib.launch_count
    phases, r.timing.PHASES = r.timing.totals(), None
    clocks = sampler.stop()
    r._lib.check_status()
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    r._lib.check_status()

    # rooflines from CUDA events around the phases of every fused block inside the timed region (timing.PHASES):
    # the dominant kernel (self-attention main kernel), the largest GEMM (fc1 + SwiGLU) and the norm + modulation
    # quantizer; `work` of a phase is its algorithmic operation / byte count
    pk = peaks()
    peak8 = 2.0 * pk["bf16_tflops_sustained"]
    peak_note = (f"2 x {pk['source']} sustained cuBLAS bf16 ({pk['bf16_tflops_sustained']} TF/s): 8-bit operands run "
                 "at twice the bf16 rate; nominal dense INT8/FP8 peak is 4500")
    total_ms = ms_step * args.steps

    def tensor_roof(name, kernel):
        ph = phases.get(name)
        if not ph or ph["ms"] <= 0:
            return None
        achieved = ph["work"] / 1e12 / (ph["ms"] / 1e3)
        return {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peak8, "unit": "TFLOP/s",
                "frac": achieved / peak8, "ms_per_launch": ph["ms"] / ph["n"], "launches": ph["n"],
                "share_of_step": ph["ms"] / total_ms, "peak_note": peak_note, "frac_of_nominal_int8": achieved / 4500.0}

    roof = tensor_roof("attn_self_main", "attn_tok_kernel" if args.attn == "reference" else "attn_int8_kernel")
    if roof and args.attn != "fast":
        roof["traffic"], roof["traffic_unit"] = None, "no capture of the token-scaled kernel"
    elif roof:
        ph = phases["attn_self_main"]
        lq = lk = s_total
        heads_local = cfg.heads // world
        # DRAM bytes of one launch: dram__bytes_read.sum + dram__bytes_write.sum of this kernel from one ncu capture
        # (ATTN_TRAFFIC below), scaled to this launch by its operand + output bytes; dropped when the kernel source
        # has changed since that capture
        def alg_bytes(lq_, lk_, h_):
            return h_ * 128 * (lq_ + 2 * lk_) + h_ * 128 * 2 * lq_
        roof["traffic"], roof["traffic_unit"] = attn_traffic(alg_bytes(lq, lk, heads_local))
    roof_gemm = tensor_roof("gemm_fc1_swiglu", "gemm_pair_kernel<int8, SwiGLU epilogue> (fc1; gemm_w8a8_kernel when CTA pairs are off)")
    roof_quant = None
    ph = phases.get("quant_norm_mod")
    if ph and ph["ms"] > 0:
        gbs = ph["work"] / 1e9 / (ph["ms"] / 1e3)
        roof_quant = {"bound": "hbm", "kernel": "quant_rows_kernel<norm+modulation, int8>", "achieved": gbs,
                      "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                      "ms_per_launch": ph["ms"] / ph["n"], "launches": ph["n"], "share_of_step": ph["ms"] / total_ms,
                      "peak_note": f"{pk['source']} copy bandwidth; 3 algorithmic bytes per element + 4 per row",
                      "frac_of_nominal_8tbs": gbs / 8000.0}
    phase_ms = {k: round(v["ms"] / args.steps, 3) for k, v in sorted(phases.items())}
    exchange_ms = sum(v for k, v in phase_ms.items() if k.startswith("exchange_"))
    h2d = sum(host[i].numel() * host[i].element_size() for i in (0, 1, 2, 4))
    d2h = sum(t.numel() * t.element_size() for t in out_host)
    rec = {"metric": "H3 DiT step seconds @768x1344x141f", "value": ms_step / 1e3, "unit": "s/step", "n_gpus": world,
           "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False,
           "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
           "config": workload_config(args.workload, world, args.attn), "variant": {"linear_mode": args.mode, "attention": args.attn, "exchange": exchange,
                       "cfg_samples": "side by side on two streams" if side_by_side else "one after the other"},
           "clocks": clocks,
           "e2e": {"value": ms_e2e / 1e3, "unit": "s/step", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
           "gpu_launches": launches, "roofline": roof, "roofline_gemm": roof_gemm, "roofline_quant": roof_quant,
           "phases_ms_per_step": phase_ms, "exchange_ms_per_step": round(exchange_ms, 3)}
    if world == 1 and not args.no_extras:
        probe = tensor_probe()
        rec["tensor_probe"] = probe
        if roof:
            # the attention kernel runs half of its operations on int8 and half on e4m3 operands
            mixed = 2.0 / (1.0 / probe["int8_tops"] + 1.0 / probe["e4m3_tops"])
            roof["frac_of_probe"] = roof["achieved"] / (probe["int8_tops"] if args.attn == "reference" else mixed)
        if roof_gemm:
            roof_gemm["frac_of_probe"] = roof_gemm["achieved"] / probe["int8_tops"]
    if world == 1 and args.workload == "full" and not args.no_extras:
        rec["extras"] = vae_extras(local)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            rec["cpu_baseline"] = cpu_baseline_record(args.workload)
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
