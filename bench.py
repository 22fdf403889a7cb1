#!/usr/bin/env python
"""Benchmark of the DiRotQ quantized-linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W]
                    [--workload pixart_int4|pixart_nvfp4|flux_int4|sana_int4|sana_w4a8] [--flux-ffn tp|dp]
    python bench.py --impl reference ...      # the reference's fp32 CPU forward on a bounded sample

One "step" = every wrapped linear of one denoising step of the named DiT (BASELINE config 1 by
default: PixArt-Sigma shapes, 28 blocks x 8 linears, batch 8 x 4096 tokens per GPU), each through
rotate -> split -> 4-bit quantise -> W4A4 GEMM + bf16 branch + dequant + bias.  `value` counts the
algorithmic operations of the linears (2*M*N*D each; the online rotation is overhead, not credited)
over the device time of the step.  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (block fn name, n_blocks, quant, tokens per sample, batch per GPU, description)
    "pixart_int4": ("pixart_block", 28, "int4", 4096, 8,
                    "BASELINE config 1: PixArt-Sigma-shaped step, 28 blocks x (7 INT W4A4 g64 k=64 + ff.net.2 W4A16), "
                    "batch 8 x 4096 tokens per GPU"),
    "pixart_nvfp4": ("pixart_block", 28, "nvfp4", 4096, 8,
                     "BASELINE config 2: same step in NVFP4 W4A4 (E2M1 g16, UE4M3 group scales, fp32 tensor scale)"),
    "sana_int4": ("sana_block", 20, "int4", 1024, 16,
                  "BASELINE config 4 (W4A4): SANA-1.6B-shaped step, 20 blocks x 6 linears (hidden 2240, k=320, per-head "
                  "70 x 32 out-projections), batch 16 x 1024 tokens per GPU"),
    "sana_w4a8": ("sana_block", 20, "int8", 1024, 16,
                  "BASELINE config 4 (W4A8): same step with asymmetric 8-bit activations"),
    # FLUX runs at a FIXED global batch (strong scaling); see dirotq_b200.parallel.FluxLinearStep
    "flux_int4": ("flux_double_block", 57, "int4", 4608, 4,
                  "BASELINE config 3: FLUX.1-dev-shaped step, 19 double-stream (image 4096 + text 512 tokens) + 38 "
                  "single-stream blocks, INT W4A4 g64 k=384, per-head out-projections, K=12288 down-projections "
                  "without rotation, global batch 4"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="pixart_int4", choices=sorted(WORKLOADS))
    ap.add_argument("--blocks", type=int, default=0, help="override the number of blocks (smoke runs only)")
    ap.add_argument("--flux-ffn", default="tp", choices=["tp", "dp"],
                    help="flux_int4 at N > 1: FFN pairs tensor-parallel (all-gather + reduce-scatter) or row-sharded")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fuse-gelu", action="store_true",
                    help="keep the GELU between the FFN linears as a separate PyTorch kernel")
    ap.add_argument("--cache-weight-panel", action="store_true",
                    help="keep each INT4 layer's fp16 weight panel resident (2 bytes per weight) instead of rebuilding it "
                         "from the 4-bit codes on every call")
    ap.add_argument("--exact-int", action="store_true",
                    help="INT4 layers through the exact-integer kind::i8 GEMM instead of the tensor-rate fp16 one")
    ap.add_argument("--profile-case", action="store_true",
                    help="run a small case for ncu instead of the benchmark: one 1152->1152 k=64 layer at M=16384 "
                         "(38 MB in, 38 MB out), INT4 then NVFP4, three forwards each")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's fp32 fused-unrotation forward (oracle port), bounded sample
# ---------------------------------------------------------------------------------------------
def cpu_reference_tflops(workload, steps, warmup, budget_s=20.0):
    """Times dirotq_fused_unrotation._fused_forward (fp32 rotation + fake quant + nn.Linear), restated in
    oracle/dirotq_oracle.py, on one block of the workload at M = 2048 tokens with all host threads."""
    from oracle import dirotq_oracle as O
    from dirotq_b200 import dit
    blk_name, _, quant, _, _, _ = WORKLOADS[workload]
    block = getattr(dit, blk_name)()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    M = 2048
    g = torch.Generator().manual_seed(0)
    x = O.synth_activations(M, block[0].in_f, g).reshape(1, M, -1)
    specs = []
    for ld in block:
        W = (torch.randn(ld.out_f, ld.in_f, generator=g) * 0.02).to(torch.bfloat16)
        b = (torch.randn(ld.out_f, generator=g) * 0.1).to(torch.bfloat16)
        if ld.kind == "w4a16":
            specs.append((ld, None, W, b))
            continue
        cfg = O.QuantCfg(4, 16 if quant == "nvfp4" else 64, True, 1.0, ld.tail, "nvfp4" if quant == "nvfp4" else "int")
        bits = 8 if quant == "int8" else 4
        cfg = O.QuantCfg(bits, cfg.groupsize, bits == 4, 1.0, ld.tail, cfg.quant_dtype)
        U = O.random_orthogonal(ld.in_f, g).float() if ld.kind == "hidden" else None
        Uh = None
        if ld.kind == "perhead":
            Uh = torch.stack([O.random_orthogonal(ld.head_dim, g).float() for _ in range(ld.heads)])
        specs.append((ld, O.LayerSpec(W, b, cfg, rotation=U, rotation_per_head=Uh), W, b))
    ops = sum(dit.linear_ops(ld, M) for ld in block)

    def one_pass():
        ff = None
        for ld, spec, W, b in specs:
            src = x if ld.source == "x" else ff
            if spec is None:
                y = torch.nn.functional.linear(src, W, b)
            else:
                y = O.fused_forward(src, spec, fp32=True)
            if ld.out_f > ld.in_f:
                ff = torch.nn.functional.gelu(y, approximate="tanh")
        return y

    for _ in range(max(1, warmup)):
        one_pass()
    times = []
    t_all = time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > budget_s:
            break
    t = statistics.median(times)
    return {"value": ops / t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"one {blk_name} ({len(block)} linears) at M=2048 tokens, fp32 _fused_forward restated in "
                      f"oracle/, torch CPU {cores} threads, median of {len(times)} passes ({t*1e3:.0f} ms each)"}, t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, t = cpu_reference_tflops(args.workload, args.steps, args.warmup, budget_s=120.0)
    line = {"impl": "reference", "metric": "w4a4_linear_tflops", "value": cb["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "strong" if args.workload.startswith("flux") else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[args.workload][5], "sample": cb["sample"]},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                      stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out = ""
        sm, mx, reasons, pw = [], [], set(), []
        for ln in out.strip().splitlines():
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples under load = upper half by power
        if sm:
            order = sorted(range(len(sm)), key=lambda i: pw[i])
            load = [sm[i] for i in order[len(order) // 2:]]
            return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                    "samples": len(sm), "power_w_max": max(pw)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def run_ours(args):
    import torch.distributed as dist
    from dirotq_b200 import backend, dit, ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    # stdout carries the JSON line only: everything else written to file descriptor 1 until then (library
    # banners such as NCCL's version line included) goes to stderr
    sys.stdout.flush()
    saved_stdout_fd = os.dup(1)
    os.dup2(2, 1)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    blk_name, n_blocks, quant, tokens, batch, desc = WORKLOADS[args.workload]
    if args.blocks:
        n_blocks = args.blocks
    is_flux = args.workload.startswith("flux")
    from dirotq_b200.synth import synth_activations
    import contextlib
    g = torch.Generator().manual_seed(1234 + rank)
    with contextlib.redirect_stdout(sys.stderr):     # stdout carries the JSON line only
        backend.patch_forward()
        if is_flux:
            from dirotq_b200.parallel import FluxLinearStep
            n_double = args.blocks if args.blocks else 19
            step = FluxLinearStep(world, rank, dev, batch=batch, n_double=n_double, n_single=2 * n_double,
                                  ffn=args.flux_ffn, quant=quant)
            backend.preconvert_rotations_to_device(step.layers, dev)
            n_fused = 0 if (args.no_fuse_gelu or args.exact_int) else step.fuse_gelu()
            for lyr in step._flat:                   # the packed device state is all the forward needs
                lyr._b200_explicit = None
                lyr.rotation = lyr.rotation_per_head = None
            torch.cuda.empty_cache()
            n_blocks = 3 * n_double
            M, D, out_f = step.rows_per_rank("single"), 3072, 3072   # rows per GPU (strong scaling: global batch fixed)
            lin_ops, rot_ops = step.ops_per_step()
            lin_ops, rot_ops = lin_ops / world, rot_ops / world      # per-GPU share; the JSON line reports world x this
            x_host = synth_activations(M, D, g).pin_memory()
            y_shape = (M, out_f)
            scaling = "strong"
            l2_note = f"inputs larger than L2 ({len(step._flat)} distinct weight sets per step)"
        else:
            block = getattr(dit, blk_name)()
            M = tokens * batch                           # rows per GPU (weak scaling: fixed per-GPU batch)
            D, out_f = block[0].in_f, block[-1].out_f
            step = dit.LinearPathStep(block, n_blocks, quant, device=dev, seed=1000 + 7919 * rank)
            backend.preconvert_rotations_to_device(step, dev)
            n_fused = 0 if (args.no_fuse_gelu or args.exact_int) else backend.fuse_gelu_modules(step)
            lin_ops, rot_ops = step.ops_per_step(M)
            # step input: synthetic activations with the config-0 distribution, in PINNED host memory
            x_host = synth_activations(M, D, g).reshape(batch, tokens, D).pin_memory()
            y_shape = (batch, tokens, out_f)
            scaling = "weak"
            l2_note = (f"inputs larger than L2 ({M * D * 2 / 1e6:.0f} MB activations + {len(step.layers)} distinct "
                       f"weight sets per step)")
    x_dev = x_host.to(dev, non_blocking=True)
    y_host = torch.empty(*y_shape, dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def step_resident():
        return step(x_dev)

    # end to end: every step copies its input from pinned host memory and its result back; the copies run on side
    # streams (two input buffers) so that they overlap the kernels of the neighbouring steps
    from dirotq_b200.dit import HostStreamedStep
    streamed = HostStreamedStep(step, x_host, y_host, dev)

    def step_e2e():
        return streamed()

    for _ in range(max(3, args.warmup)):
        step_resident()
    ops.check_status(dev)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    torch.cuda.profiler.start()          # lets `ncu --profile-from-start off` see the timed region only
    ms = timed(step_resident, args.steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    step_e2e()
    step_e2e()

    def e2e_steps():
        for _ in range(args.steps):
            step_e2e()
        streamed.finish()                  # the timer's closing event waits for the last result copy
    ms_e2e = timed(e2e_steps, 1) / args.steps
    ops.check_status(dev)

    # roofline pass: the same launches, the dominant kernel bracketed by CUDA events on its stream
    roof = roofline_pass(step, x_dev, M, quant, dev, args.steps) if rank == 0 and not is_flux else None
    if rank == 0 and is_flux:
        roof = roofline_pass_flux(step, x_dev, dev)

    cb = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb, _ = cpu_reference_tflops(args.workload, 10, 1)

    if rank == 0:
        line = {
            "metric": "w4a4_linear_tflops", "value": world * lin_ops / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "e2m1" if quant == "nvfp4" else "s8", "data": "synthetic",
            "config": {"workload": desc, "blocks": n_blocks, "rows_per_gpu": M,
                       "global_batch": batch if is_flux else batch * world,
                       "parallelism": (f"rows/{world} + ffn-{step.ffn}" if is_flux else f"dp{world}"),
                       "gelu": (f"fused into the up-projection GEMM epilogue ({n_fused} layers)" if n_fused
                                else "separate PyTorch kernel"),
                       "l2": l2_note,
                       "linear_gflop_per_step_per_gpu": lin_ops / 1e9, "rotation_gflop_per_step_per_gpu": rot_ops / 1e9},
            "e2e": {"value": world * lin_ops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                    "copies": "pinned host memory, side streams, two device input buffers (dit.HostStreamedStep)"},
            "gpu_launches": step.kernel_launches_per_step() * args.steps,
            "clocks": clocks, "roofline": roof, "cpu_baseline": cb,
        }
    if world > 1:
        dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(saved_stdout_fd, 1)
    os.close(saved_stdout_fd)
    if rank == 0:
        print(json.dumps(line), flush=True)


def roofline_pass(step, x_dev, M, quant, dev, steps):
    """Runs the step's layers through the two C-ABI stages separately and brackets every launch of the
    W4A4 GEMM (the kernel with the largest share of the step) with CUDA events on the launching stream."""
    from dirotq_b200 import ops
    hbm, bf16_burst, bf16_sust, which = measured_peaks()
    pairs = []
    bufs = {}
    ops_total = 0.0
    f16_ws, f16_used = None, False
    bytes_total = 0.0
    k1_pairs, k1_flops, k1_bytes = [], 0.0, 0.0
    nb = len(step.block)
    for _ in range(max(1, min(steps, 2))):
        for idx, lyr in enumerate(step.layers):
            ld = step.block[idx % nb]
            st = getattr(lyr, "_b200_state", None)
            if st is None or ld.source != "x":
                continue
            key = (st.fmt, M)
            if key not in bufs:
                bufs[key] = ops.alloc_act(st.fmt, M, dev)
            buf = bufs[key]
            x2d = x_dev.reshape(M, -1)
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record()
            ops.rotate_quantize(x2d, st.rot_t, st.fmt, out=buf)
            r1.record()
            if st.fmt.num_heads == 0:
                k1_pairs.append((r0, r1))
                k1_flops += 2.0 * M * ld.in_f * ld.in_f
                lay = st.layout
                k1_bytes += 2.0 * M * ld.in_f + 2.0 * ld.in_f * ld.in_f + M * (lay.code_row_bytes + lay.n_chunks * 2
                                                                               + lay.tail_pitch * 2)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if quant == "nvfp4":
                w = ops.PackedWeightNvfp4(st.out_features, st.layout.q_len, st.layout.n_chunks, st.w_tensor_scale,
                                          st.w_codes, st.w_scales)
                ops.gemm_w4a4_nvfp4(buf, w, st.w_tail, st.bias)
            else:
                w = ops.PackedWeightInt4(st.out_features, st.layout.q_len, st.layout.group, st.layout.n_chunks,
                                         st.w_codes, st.w_scales, st.w_sum)
                if st.folded is not None:
                    f16_used = True
                    need = ops.f16_workspace_bytes(buf, 0 if st.folded.panel is not None else st.out_features)
                    if f16_ws is None or f16_ws.numel() < need:
                        f16_ws = torch.empty(need, dtype=torch.uint8, device=dev)
                    ops.gemm_w4a4_int_f16(buf, w, st.folded, st.bias, workspace=f16_ws)
                else:
                    ops.gemm_w4a4_int(buf, w, st.w_tail, st.bias)
            e1.record()
            pairs.append((e0, e1))
            ops_total += 2.0 * M * ld.out_f * ld.in_f
            bytes_total += gemm_algorithmic_bytes(M, ld.out_f, st.layout, quant)
    torch.cuda.synchronize()
    t_ms = sum(a.elapsed_time(b) for a, b in pairs)
    achieved = ops_total / (t_ms * 1e-3) / 1e12
    kname = "gemm_nvfp4_kernel" if quant == "nvfp4" else (
        "gemm_int_f16_kernel (with its fold_expand_kernel or expand_weight_panel_kernel)" if f16_used else "gemm_int_kernel")
    k1 = None
    if k1_pairs:
        k1_ms = sum(a.elapsed_time(b) for a, b in k1_pairs)
        k1 = {"kernel": "rotate_quant_kernel (hidden rotation + split + quantise)", "bound": "tensor",
              "achieved": k1_flops / (k1_ms * 1e-3) / 1e12, "peak": bf16_sust, "unit": "TFLOP/s",
              "frac": k1_flops / (k1_ms * 1e-3) / 1e12 / bf16_sust,
              "hbm_gbs": k1_bytes / (k1_ms * 1e-3) / 1e9, "hbm_peak_gbs": hbm, "hbm_frac": k1_bytes / (k1_ms * 1e-3) / 1e9 / hbm,
              "launches_timed": len(k1_pairs), "avg_launch_us": k1_ms * 1e3 / len(k1_pairs)}
    return {"bound": "tensor", "kernel": kname, "rotate_quantise": k1,
            "achieved": achieved, "peak": bf16_sust, "unit": "TFLOP/s", "frac": achieved / bf16_sust,
            "peak_source": f"{which}: cuBLAS bf16 sustained; the INT4 path computes in fp16 on the same tensor pipe, "
                           "dense FP4 is nominally 4x that figure",
            "launches_timed": len(pairs), "avg_launch_us": t_ms * 1e3 / max(1, len(pairs)),
            "traffic": NCU_TRAFFIC_RATIO * bytes_total / max(1, len(pairs)),
            "traffic_source": f"algorithmic bytes per launch x {NCU_TRAFFIC_RATIO} (dram read + write of one ncu capture of "
                              "the INT4 GEMM at M=16384, N=K=1152 over its algorithmic bytes; traffic grows with M and N)"}


# dram__bytes_read.sum + dram__bytes_write.sum of the captured launch (16.3 MB: the 38 MB of output it wrote
# were still in the 126 MB L2 when the launch ended) / its algorithmic bytes (52 MB); see profiles/
NCU_TRAFFIC_RATIO = 0.31


def gemm_algorithmic_bytes(M, N, lay, quant):
    """Bytes one W4A4 GEMM call must move: activation codes, scale data and tail, the weight's, bias, output."""
    if quant == "nvfp4":
        per_row = lay.code_row_bytes + lay.n_chunks * 4 + lay.tail_pitch * 2
    else:   # codes + 8-byte records per chunk + bf16 scales read by the fold kernel + tail read, written and read again
        per_row = lay.code_row_bytes + lay.n_chunks * (8 + 2 + 8) + lay.tail_pitch * 2 * 3
    w_row = lay.code_row_bytes + lay.n_chunks * 8 + lay.tail_pitch * 2 + 2
    return float(M * per_row + N * w_row + 2 * M * N)


def roofline_pass_flux(step, x_dev, dev):
    """FLUX: the same bracketing over the hidden-rotation attention linears of the single-stream blocks."""
    from dirotq_b200 import ops
    hbm, bf16_burst, bf16_sust, which = measured_peaks()
    pairs, ops_total, buf, f16_ws = [], 0.0, None, None
    M = x_dev.shape[0]
    for stream, ws, wu, wd in step.blocks:
        if stream != "single":
            continue
        for w in ws[:3]:
            st = w._b200_state
            buf = buf if buf is not None else ops.alloc_act(st.fmt, M, dev)
            ops.rotate_quantize(x_dev, st.rot_t, st.fmt, out=buf)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            pw = ops.PackedWeightInt4(st.out_features, st.layout.q_len, st.layout.group, st.layout.n_chunks,
                                      st.w_codes, st.w_scales, st.w_sum)
            if f16_ws is None:
                f16_ws = torch.empty(ops.f16_workspace_bytes(buf, st.out_features), dtype=torch.uint8, device=dev)
            ops.gemm_w4a4_int_f16(buf, pw, st.folded, st.bias, workspace=f16_ws)
            e1.record()
            pairs.append((e0, e1))
            ops_total += 2.0 * M * 3072 * 3072
    torch.cuda.synchronize()
    t_ms = sum(a.elapsed_time(b) for a, b in pairs)
    achieved = ops_total / (t_ms * 1e-3) / 1e12
    return {"bound": "tensor", "kernel": "gemm_int_f16_kernel (with its fold_expand_kernel or expand_weight_panel_kernel)", "achieved": achieved,
            "peak": bf16_sust, "unit": "TFLOP/s", "frac": achieved / bf16_sust,
            "peak_source": f"{which}: cuBLAS bf16 sustained (the kernel computes in fp16 on the same tensor pipe)",
            "launches_timed": len(pairs), "avg_launch_us": t_ms * 1e3 / max(1, len(pairs)),
            "traffic": NCU_TRAFFIC_RATIO * gemm_algorithmic_bytes(M, 3072, st.layout, "int4"),
            "traffic_source": f"algorithmic bytes per launch x {NCU_TRAFFIC_RATIO} (ratio of one ncu capture of the INT4 "
                              "GEMM at M=16384, N=K=1152)"}


def profile_case():
    import contextlib
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    torch.cuda.set_device(0)
    M = 16384
    x = synth_activations(M, 1152, torch.Generator().manual_seed(0)).cuda()
    with contextlib.redirect_stdout(sys.stderr):
        for quant in ("int4", "nvfp4"):
            w = dit.make_wrapped_linear(dit.LayerDef("probe", 1152, 1152, tail=64), quant, 5, "cuda")
            st = backend.prepare_layer(w, "cuda", w._b200_explicit)
            for _ in range(3):
                backend.linear_forward(st, x)
    torch.cuda.synchronize()
    ops.check_status()
    print(json.dumps({"profile_case": "ok", "rows": M}))


if __name__ == "__main__":
    a = parse()
    if a.cache_weight_panel:
        from dirotq_b200 import backend as _backend
        _backend.CACHE_WEIGHT_PANEL = True
    if a.exact_int:
        from dirotq_b200 import backend as _backend
        _backend.INT4_TENSOR_RATE_GEMM = False
    if a.profile_case:
        profile_case()
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
