#!/usr/bin/env python
"""Benchmark of the DiRotQ quantized-linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W]
                    [--workload pixart_int4|pixart_nvfp4|flux_int4|flux_nvfp4|sana_int4|sana_w4a8] [--flux-ffn tp|dp]
    python bench.py --impl reference ...      # the reference's own fp32 CPU forward on a bounded sample

One "step" = every wrapped linear of one denoising step of the named DiT (BASELINE config 1 by default: PixArt-Sigma
shapes, 28 blocks x 8 linears, GLOBAL batch 8 x 4096 tokens split over the GPUs), each through rotate -> split ->
4-bit quantise -> W4A4 GEMM + bf16 branch + dequant + bias.  `value` counts the algorithmic operations of the linears
(2*M*N*D each; the online rotation is overhead, not credited) over the device time of the step.  Prints ONE JSON line
on rank 0.  Beside the headline the line carries: `e2e` (host buffers, copies inside the timed region), `roofline`
(dominant kernel against the measured peak of the pipe it runs on), `cpu_baseline` (the reference's fp32 forward on
the host cores), `denoise_step` (a model-shaped step: the same linears inside attention / norm / modulation glue, with
the path's share of it) and `sub` (NVFP4 FLUX-shaped GEMMs against an FP4 peak, the NVFP4 and FLUX steps; on several
GPUs the tensor-parallel FLUX feed-forwards with their NCCL time).
"""
import argparse
import contextlib
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
    # name: (block fn name, n_blocks, quant, tokens per sample, global batch, model family, description)
    "pixart_int4": ("pixart_block", 28, "int4", 4096, 8, "pixart",
                    "BASELINE config 1: PixArt-Sigma-shaped step, 28 blocks x (7 INT W4A4 g64 k=64 + ff.net.2 W4A16), "
                    "global batch 8 x 4096 tokens"),
    "pixart_nvfp4": ("pixart_block", 28, "nvfp4", 4096, 8, "pixart",
                     "BASELINE config 2: same step in NVFP4 W4A4 (E2M1 g16, UE4M3 group scales, fp32 tensor scale)"),
    "sana_int4": ("sana_block", 20, "int4", 1024, 16, "sana",
                  "BASELINE config 4 (W4A4): SANA-1.6B-shaped step, 20 blocks x 6 linears (hidden 2240, k=320, per-head "
                  "70 x 32 out-projections), global batch 16 x 1024 tokens"),
    "sana_w4a8": ("sana_block", 20, "int8", 1024, 16, "sana",
                  "BASELINE config 4 (W4A8): same step with asymmetric 8-bit activations"),
    "flux_int4": ("flux_double_block", 57, "int4", 4608, 4, "flux",
                  "BASELINE config 3: FLUX.1-dev-shaped step, 19 double-stream (image 4096 + text 512 tokens) + 38 "
                  "single-stream blocks, INT W4A4 g64 k=384, per-head out-projections, K=12288 down-projections "
                  "without rotation, global batch 4"),
    "flux_nvfp4": ("flux_double_block", 57, "nvfp4", 4608, 4, "flux",
                   "FLUX.1-dev-shaped step as config 3, in NVFP4 W4A4 (E2M1 g16, UE4M3 group scales; per-head "
                   "out-projections in blocks of 16 inside each head), K=12288 down-projections without rotation, global batch 4"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="pixart_int4", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): the workload's global batch is split over the GPUs; weak: every GPU runs "
                         "the whole batch (independent replicas)")
    ap.add_argument("--blocks", type=int, default=0, help="override the number of blocks (smoke runs only)")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="override the workload's global batch (experiments: e.g. 1 with --gpus 1 is the per-GPU share of "
                         "the default workload on 8 GPUs)")
    ap.add_argument("--flux-ffn", default="tp", choices=["tp", "dp"],
                    help="flux_int4 at N > 1: FFN pairs tensor-parallel (all-gather + reduce-scatter) or row-sharded")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="skip the sub-records and the model-shaped step")
    ap.add_argument("--no-fuse-gelu", action="store_true",
                    help="keep the GELU between the FFN linears as a separate PyTorch kernel")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel from Python instead of replaying the step from a CUDA graph (resident-input "
                         "timing of the non-FLUX workloads and the model-shaped step)")
    ap.add_argument("--no-fused-glue", action="store_true",
                    help="denoise_step: keep modulated LayerNorm, gated residuals and q/k RMSNorm + rotary embedding as "
                         "chains of PyTorch elementwise kernels instead of the library's single-pass kernels")
    ap.add_argument("--no-fuse-qkv", action="store_true",
                    help="keep to_q / to_k / to_v (and add_*_proj) as three GEMMs on the shared codes instead of one GEMM "
                         "on concatenated weights")
    ap.add_argument("--no-fuse-ffn", action="store_true",
                    help="keep the quantise kernel between an FFN pair's GELU and its un-rotated down-projection instead of "
                         "quantising in the up-projection's GEMM epilogue")
    ap.add_argument("--cache-weight-panel", action="store_true",
                    help="keep each INT4 layer's fp16 weight panel resident (2 bytes per weight) instead of rebuilding it "
                         "from the 4-bit codes on every call")
    ap.add_argument("--no-resident-panels", action="store_true",
                    help="large-batch INT4 layers rebuild their fp16 weight panel on every call (weights stay 0.5 byte each "
                         "in device memory) instead of keeping it while the device's budget for 16-bit weight copies lasts")
    ap.add_argument("--exact-int", action="store_true",
                    help="INT4 layers through the exact-integer kind::i8 GEMM instead of the tensor-rate fp16 one")
    ap.add_argument("--profile-case", default="", nargs="?", const="layers",
                    help="run a small case for ncu instead of the benchmark: 'layers' = one 1152->1152 k=64 layer at "
                         "M=16384, INT4 then NVFP4, three forwards each; 'flux_nvfp4' = one NVFP4 3072->12288 k=384 "
                         "layer at M=4096; 'flux_int4' = one INT4 3072->12288 k=384 layer at M=18432 (its fp16 weight panel, 75 MB, "
                         "does not stay in L2); 'perhead' = one INT4 per-head layer, 70 heads x 32 with 4 high channels each, at "
                         "M=16384; 'quantize' = the quantise-only kernel at M=4096, D=12288; 'glue' = the three "
                         "block-glue kernels on FLUX-shaped tensors (4 x 4096 x 3072)")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own fp32 fused-unrotation forward, bounded sample
# ---------------------------------------------------------------------------------------------
def _config0(seed=0, M=8192, D=1152, N=1152, k=64):
    """BASELINE config 0: one PixArt-Sigma attention linear.  x bf16 [2, 4096, 1152] (N(0,1) + planted rank-32 subspace
    + 8 heavy-tailed channels), orthogonal rotation, INT4 g64 weights with fp16 group scales + 64 bf16 coefficients."""
    from oracle import dirotq_oracle as O
    g = torch.Generator().manual_seed(seed)
    x = O.synth_activations(M, D, g).reshape(2, M // 2, D)
    U = O.random_orthogonal(D, g).float()
    qw = torch.randint(-8, 8, (N, D - k), generator=g)
    sw = (torch.rand(N, (D - k) // 64, generator=g) * 0.015 + 0.005).to(torch.float16).float()
    w_tail = (torch.randn(N, k, generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    w_low = (qw.reshape(N, -1, 64).float() * sw.unsqueeze(-1)).reshape(N, -1)
    W = torch.cat([w_low, w_tail.float()], dim=1).to(torch.bfloat16)
    return x, U, W, bias, k


def cpu_reference_config0(runs=3, warm=1, budget_s=25.0):
    """BASELINE config 0 through the reference's own `_fused_forward` (dirotq_fused_unrotation.py:62-148), imported
    unmodified from oracle/_ref, all host threads: min and median of `runs` forwards and a per-stage split."""
    from oracle import make_ref
    qu, slow, _ = make_ref.load()
    import torch.nn as nn
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, U, W, bias, k = _config0()
    lin = nn.Linear(1152, 1152, bias=True).to(torch.bfloat16)
    lin.weight.data.copy_(W)
    lin.bias.data.copy_(bias)
    w = qu.ActQuantWrapper(lin)
    w.quantizer.configure(bits=4, groupsize=64, sym=True, high_bits_length=k, quant_dtype="int")
    w.rotation = U
    w._unrot_fused = True
    ops = 2.0 * x.shape[0] * x.shape[1] * 1152 * 1152
    with torch.no_grad():
        for _ in range(warm):
            slow._fused_forward(w, x)
        times, t_all = [], time.perf_counter()
        for _ in range(max(1, runs)):
            t0 = time.perf_counter()
            slow._fused_forward(w, x)
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - t_all > budget_s:
                break
        # per-stage split: the same operations the forward runs, timed one after another
        t0 = time.perf_counter()
        xr = (x.float().reshape(-1, 1152) @ U).reshape(x.shape)
        t1 = time.perf_counter()
        w.quantizer.find_params(xr)
        xq = w.quantizer(xr).to(torch.bfloat16)
        w.quantizer.free()
        t2 = time.perf_counter()
        w.module(xq)
        t3 = time.perf_counter()
    t_med, t_min = statistics.median(times), min(times)
    cb = {"value": ops / t_med / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "reference",
          "value_best": ops / t_min / 1e12, "ms_median": t_med * 1e3, "ms_min": t_min * 1e3,
          "stages_ms": {"cast_and_rotation_fp32": (t1 - t0) * 1e3, "find_params_and_quantise": (t2 - t1) * 1e3,
                        "bf16_linear": (t3 - t2) * 1e3},
          "sample": f"BASELINE config 0: one PixArt-Sigma attention linear, x bf16 [2,4096,1152], k=64, INT4 g64 symmetric, "
                    f"through the reference's own dirotq_fused_unrotation._fused_forward (unmodified, oracle/_ref), torch "
                    f"CPU {cores} threads, {warm} warm-up + {len(times)} timed forwards (median; best in value_best)"}
    return cb, t_med


def cpu_port_tflops(workload, steps, warmup, budget_s=20.0):
    """Fallback when oracle/_ref is not populated: the fp32 forward restated in oracle/dirotq_oracle.py on one block of
    the workload at M = 2048 tokens."""
    from oracle import dirotq_oracle as O
    from dirotq_b200 import dit
    blk_name, _, quant = WORKLOADS[workload][:3]
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
        bits = 8 if quant == "int8" else 4
        cfg = O.QuantCfg(bits, 16 if quant == "nvfp4" else 64, bits == 4, 1.0, ld.tail, "nvfp4" if quant == "nvfp4" else "int")
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
            y = torch.nn.functional.linear(src, W, b) if spec is None else O.fused_forward(src, spec, fp32=True)
            if ld.out_f > ld.in_f:
                ff = torch.nn.functional.gelu(y, approximate="tanh")
        return y

    for _ in range(max(1, warmup)):
        one_pass()
    times, t_all = [], time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > budget_s:
            break
    t = statistics.median(times)
    return {"value": ops / t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"one {blk_name} ({len(block)} linears) at M=2048 tokens, fp32 _fused_forward restated in "
                      f"oracle/ (oracle/_ref not populated), torch CPU {cores} threads, median of {len(times)} passes"}, t


def cpu_baseline(workload, steps, warmup, budget_s):
    from oracle import make_ref
    if make_ref.available():
        return cpu_reference_config0(runs=max(3, steps), warm=max(1, min(warmup, 2)), budget_s=budget_s)
    return cpu_port_tflops(workload, steps, warmup, budget_s)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, t = cpu_baseline(args.workload, args.steps, args.warmup, budget_s=120.0)
    line = {"impl": "reference", "metric": "w4a4_linear_tflops", "value": cb["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[args.workload][6], "sample": cb["sample"]},
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
        if sm:   # samples under load = upper half by power
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


def tensor_peak(kind):
    """(peak TFLOP/s, description) of the tensor pipe a kernel kind runs on.  Only bf16 is MEASURED on this pool
    (cuBLAS, seconds-long loop under the power cap); dense FP4 is derived as 4 x that figure, dense INT8 as 2 x."""
    _, _, bf16_sust, which = measured_peaks()
    if kind == "nvfp4":
        return 4.0 * bf16_sust, f"derived: 4 x the {which} cuBLAS bf16 sustained figure ({bf16_sust:.0f} TFLOP/s); no FP4 measurement exists"
    if kind == "i8":
        return 2.0 * bf16_sust, f"derived: 2 x the {which} cuBLAS bf16 sustained figure ({bf16_sust:.0f} TFLOP/s); no INT8 measurement exists"
    return bf16_sust, f"{which}: cuBLAS bf16 sustained (fp16 and bf16 share the pipe and the rate)"


class Dist:
    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", self.local)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def all_true(self, flag: bool) -> bool:
        """True if `flag` holds on every rank (so that all ranks take the same branch around later collectives)."""
        if self.world == 1:
            return bool(flag)
        t = torch.tensor([1 if flag else 0], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def timed(self, fn, steps):
        """Device milliseconds of `steps` calls, bracketed by barrier + synchronize, max over ranks."""
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms


def effective_rotation_ops(layers, block, M):
    """Rotation work that actually runs: sibling layers that reuse the activations of the layer before them
    (to_k / to_v after to_q) rotate nothing."""
    from dirotq_b200 import dit
    nb = len(block)
    tot = 0.0
    for idx, lyr in enumerate(layers):
        st = getattr(lyr, "_b200_state", None)
        if st is None or (st.shared is not None and st.member_id > 0):
            continue
        tot += dit.rotation_ops(block[idx % nb], M)
    return tot


def run_ours(args):
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    D_ = Dist()
    world, rank, dev = D_.world, D_.rank, D_.dev
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    # stdout carries the JSON line only: everything else written to file descriptor 1 until then (library
    # banners such as NCCL's version line included) goes to stderr
    sys.stdout.flush()
    saved_stdout_fd = os.dup(1)
    os.dup2(2, 1)
    torch.cuda.set_device(D_.local)
    if world > 1:
        D_.dist.init_process_group("nccl", device_id=dev)
    blk_name, n_blocks, quant, tokens, gbatch, family, desc = WORKLOADS[args.workload]
    if args.blocks:
        n_blocks = args.blocks
    if args.global_batch:
        gbatch = args.global_batch
    is_flux = args.workload.startswith("flux")
    strong = is_flux or args.scaling == "strong"
    if strong and gbatch % world and not is_flux:
        raise SystemExit(f"global batch {gbatch} does not split over {world} GPUs; use --scaling weak")
    batch = gbatch // world if (strong and not is_flux) else gbatch
    g = torch.Generator().manual_seed(1234 + rank)
    with contextlib.redirect_stdout(sys.stderr):
        backend.patch_forward()
        if is_flux:
            from dirotq_b200.parallel import FluxLinearStep
            n_double = args.blocks if args.blocks else 19
            step = FluxLinearStep(world, rank, dev, batch=gbatch, n_double=n_double, n_single=2 * n_double,
                                  ffn=args.flux_ffn, quant=quant)
            backend.preconvert_rotations_to_device(step.layers, dev)
            n_fused = 0 if (args.no_fuse_gelu or args.exact_int) else step.fuse_gelu()
            n_chained = 0 if args.no_fuse_ffn else step.fuse_ffn_quantise()
            n_qkv = 0 if args.no_fuse_qkv else backend.fuse_sibling_gemms(step.layers)
            for lyr in step._flat:                   # the packed device state is all the forward needs
                lyr._b200_explicit = None
                lyr.rotation = lyr.rotation_per_head = None
            torch.cuda.empty_cache()
            n_blocks = 3 * n_double
            M, D, out_f = step.rows_per_rank("single"), 3072, 3072
            lin_ops, rot_ops = step.ops_per_step()
            lin_ops, rot_ops = lin_ops / world, rot_ops / world      # per-GPU share; the JSON line reports world x this
            x_host = synth_activations(M, D, g).pin_memory()
            y_shape = (M, out_f)
            l2_note = f"inputs larger than L2 ({len(step._flat)} distinct weight sets per step)"
        else:
            block = getattr(dit, blk_name)()
            M = tokens * batch
            D, out_f = block[0].in_f, block[-1].out_f
            step = dit.LinearPathStep(block, n_blocks, quant, device=dev, seed=1000 + 7919 * rank)
            backend.preconvert_rotations_to_device(step, dev)
            n_fused = 0 if (args.no_fuse_gelu or args.exact_int) else backend.fuse_gelu_modules(step)
            n_chained = 0 if args.no_fuse_ffn else backend.fuse_ffn_quantise(step, keep_hidden=False)
            n_qkv = 0 if args.no_fuse_qkv else backend.fuse_sibling_gemms(step)
            lin_ops, _ = step.ops_per_step(M)
            rot_ops = effective_rotation_ops(step.layers, step.block, M)
            x_host = synth_activations(M, D, g).reshape(batch, tokens, D).pin_memory()
            y_shape = (batch, tokens, out_f)
            l2_note = (f"inputs larger than L2 ({M * D * 2 / 1e6:.0f} MB activations + {len(step.layers)} distinct "
                       f"weight sets per step)")
    x_dev = x_host.to(dev, non_blocking=True)
    y_host = torch.empty(*y_shape, dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()

    graphed = [None]

    def step_resident():
        return graphed[0]() if graphed[0] is not None else step(x_dev)

    # end to end: every step copies its input from pinned host memory and its result back; the copies run on side
    # streams (two input buffers) so that they overlap the kernels of the neighbouring steps
    from dirotq_b200.dit import HostStreamedStep
    streamed = HostStreamedStep(step, x_host, y_host, dev)

    for _ in range(max(3, args.warmup)):
        step_resident()
    ops.check_status(dev)
    # small shards (one or two samples per GPU) are short enough for Python's launch cost to show: replay them from a
    # CUDA graph captured once; larger batches gain nothing and keep plain launches
    if not is_flux and not args.no_graph and M <= 8192:
        replay = None
        try:
            from dirotq_b200.dit import GraphedCall
            replay = GraphedCall(lambda: step(x_dev))
            for _ in range(2):
                replay()
            ops.check_status(dev)
        except Exception as e:      # capture is an optimisation, never a requirement
            replay = None
            print(f"CUDA graph capture failed ({type(e).__name__}: {e}); plain launches", file=sys.stderr)
        if D_.all_true(replay is not None):
            # keep whichever form is faster here (max over ranks, so every rank decides alike): replay wins when Python's
            # launch cost shows, plain launches keep their programmatic overlap between consecutive kernels
            t_launch, t_replay = D_.timed(lambda: step(x_dev), 3), D_.timed(replay, 3)
            if t_replay < t_launch:
                graphed[0] = replay
                try:
                    streamed.enable_graphs()             # the end-to-end path replays too (one graph per input buffer)
                except Exception as e:
                    print(f"CUDA graph capture of the streamed step failed ({type(e).__name__}: {e})", file=sys.stderr)
    sampler = ClockSampler(D_.local)
    if rank == 0:
        sampler.start()
    torch.cuda.profiler.start()          # lets `ncu --profile-from-start off` see the timed region only
    ms = D_.timed(step_resident, args.steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    streamed()
    streamed()

    def e2e_steps():
        for _ in range(args.steps):
            streamed()
        streamed.finish()                  # the timer's closing event waits for the last result copy
    ms_e2e = D_.timed(e2e_steps, 1) / args.steps
    ops.check_status(dev)

    # roofline pass: the same launches, the dominant kernel bracketed by CUDA events on its stream
    roof = None
    if rank == 0:
        roof = roofline_pass_flux(step, x_dev, dev) if is_flux else roofline_pass(step, x_dev, M, quant, dev, args.steps,
                                                                                  exact_int=args.exact_int)
    launches = step.kernel_launches_per_step() * args.steps

    # ---- model-shaped step and sub-records ---------------------------------------------------------------------
    denoise, sub = None, {}
    if not args.no_sub and not args.blocks:
        del streamed
        if not is_flux:
            step.blocks = None
        step = None
        torch.cuda.empty_cache()
        with contextlib.redirect_stdout(sys.stderr):
            denoise = denoise_record(D_, family, quant, gbatch, world, strong, args)
            if world == 1:
                sub["nvfp4_flux_gemm"] = sub_nvfp4_flux_gemms(dev)
                if args.workload != "pixart_nvfp4":
                    sub["pixart_nvfp4"] = sub_linear_step(D_, "pixart_nvfp4", 28, not args.no_fuse_ffn, not args.no_fuse_qkv)
                if not is_flux:
                    sub["flux_int4"] = sub_flux_step(D_, 4, "dp", not args.no_fuse_ffn, not args.no_fuse_qkv)
            elif not is_flux:
                sub["flux_int4_tp"] = sub_flux_step(D_, 2, "tp", not args.no_fuse_ffn, not args.no_fuse_qkv)

    cb = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb, _ = cpu_baseline(args.workload, 5, 1, budget_s=25.0)

    if rank == 0:
        int_dtype = "s8" if args.exact_int else "f16"
        line = {
            "metric": "w4a4_linear_tflops", "value": world * lin_ops / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "e2m1" if quant == "nvfp4" else int_dtype, "data": "synthetic",
            "config": {"workload": desc, "blocks": n_blocks, "rows_per_gpu": M, "global_batch": gbatch if strong else gbatch * world,
                       "parallelism": (f"rows/{world} + ffn-{args.flux_ffn if world > 1 else 'dp'}" if is_flux else f"dp{world}"),
                       "arithmetic": ("E2M1 x E2M1 block-scaled (tcgen05 kind::mxf4nvf4), fp32 accumulation" if quant == "nvfp4"
                                      else "int8 x int8 -> int32 per 64-chunk (tcgen05 kind::i8)" if args.exact_int
                                      else "4-bit codes expanded to fp16 beside the tensor core, fp16 x fp16 -> fp32 "
                                           "(tcgen05 kind::f16); the exact-integer kind::i8 route is --exact-int"),
                       "gelu": (f"fused into the up-projection GEMM epilogue ({n_fused} layers)" if n_fused
                                else "separate PyTorch kernel"),
                       "ffn_pairs_quantised_in_epilogue": n_chained, "qkv_groups_as_one_gemm": n_qkv,
                       "execution": ("CUDA graph replay of the step (captured once after the warm-up)" if graphed[0] is not None
                                     else "kernels launched from Python, programmatic dependent launch between them"),
                       "weight_copies": ("4-bit only" if quant == "nvfp4" or args.exact_int else
                                         "4-bit + resident fp16 panels (--cache-weight-panel)" if args.cache_weight_panel else
                                         "4-bit; fp16 panels rebuilt per call (--no-resident-panels)" if args.no_resident_panels
                                         else "4-bit + fp16 panels kept while under a sixteenth of device memory "
                                              f"({backend.resident_weight_copy_bytes() / 2**20:.0f} MiB resident)"),
                       "l2": l2_note,
                       "linear_gflop_per_step_per_gpu": lin_ops / 1e9, "rotation_gflop_per_step_per_gpu": rot_ops / 1e9},
            "e2e": {"value": world * lin_ops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                    "copies": "pinned host memory, side streams, two device input buffers (dit.HostStreamedStep)" + (
                        "; step replayed from a CUDA graph per buffer" if graphed[0] is not None else "")},
            "gpu_launches": launches,
            "clocks": clocks, "roofline": roof, "cpu_baseline": cb, "denoise_step": denoise, "sub": sub or None,
        }
    if world > 1:
        D_.dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(saved_stdout_fd, 1)
    os.close(saved_stdout_fd)
    if rank == 0:
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# model-shaped step, sub-records
# ---------------------------------------------------------------------------------------------
def denoise_record(D_, family, quant, gbatch, world, strong, args):
    """One model-shaped denoising step (dirotq_b200.denoise): the wrapped linears inside attention / norm /
    modulation / residual glue, chained block to block.  Batch-sharded over the GPUs, no collective."""
    from dirotq_b200 import backend, denoise, ops
    dev = D_.dev
    n_blocks = None
    note = "all blocks"
    if family == "flux":                 # 57 blocks at batch 4 take a while to build: a slice of the stack is timed
        n_blocks, note = 3, "3 of 19 double-stream + 6 of 38 single-stream blocks"
    batch = gbatch // world if strong else gbatch
    if batch < 1:
        return {"skipped": f"global batch {gbatch} does not split over {world} GPUs"}
    denoise.FUSED_GLUE = not args.no_fused_glue
    step = denoise.DenoiseStep(family, quant, dev, n_blocks=n_blocks, seed=5000 + 7919 * D_.rank, prepare=True)
    n_fused = 0 if (args.no_fuse_gelu or args.exact_int) else backend.fuse_gelu_modules(step)
    n_chained = 0 if args.no_fuse_ffn else backend.fuse_ffn_quantise(step, keep_hidden=False)
    n_qkv = 0 if args.no_fuse_qkv else backend.fuse_sibling_gemms(step)
    inputs = step.example_inputs(batch, dev, seed=D_.rank)
    ms_graph = None
    with torch.no_grad():
        for _ in range(3):
            step(*inputs)
        ops.check_status(dev)
        ms = D_.timed(lambda: step(*inputs), 4) / 4
        lin_ms = denoise.time_wrapped_linears(step, inputs)
        if not args.no_graph:
            replay = None
            try:
                from dirotq_b200.dit import GraphedCall
                replay = GraphedCall(lambda: step(*inputs))
                replay()
                ops.check_status(dev)
            except Exception as e:
                replay = None
                print(f"CUDA graph capture of the model-shaped step failed ({type(e).__name__}: {e})", file=sys.stderr)
            if D_.all_true(replay is not None):          # every rank takes the timed (collective) branch, or none
                ms_graph = D_.timed(replay, 4) / 4
            del replay
    lin, _ = step.ops_per_step(batch)
    rec = {"family": family, "quant": quant, "blocks": note, "batch_per_gpu": batch, "tokens": step.shape["tokens"],
           "text_tokens": step.shape["text"], "step_ms": ms if ms_graph is None else min(ms, ms_graph),
           "step_ms_launched": ms, "step_ms_graph_replay": ms_graph, "wrapped_linears_ms": lin_ms,
           "linear_path_share": lin_ms / ms if ms > 0 else None,     # both from the launched form
           "linear_tflops_inside_step": D_.world * lin / (lin_ms * 1e-3) / 1e12 if lin_ms > 0 else None,
           "gelu_fused_layers": n_fused, "ffn_pairs_quantised_in_epilogue": n_chained, "qkv_groups_as_one_gemm": n_qkv,
           "launches_per_step": step.kernel_launches_per_step(),
           "glue": ("library single-pass kernels (csrc/glue.cu): modulated LayerNorm, gated residuals, q / k RMSNorm + rotary "
                    "embedding into joint token-major buffers; PyTorch: scaled_dot_product_attention, modulation projections "
                    "(SANA: ReLU linear attention, Mix-FFN convolutions)" if denoise.FUSED_GLUE else
                    "PyTorch bf16: adaLN modulation, LayerNorm / RMSNorm, rotary embedding, scaled_dot_product_attention "
                    "(SANA: ReLU linear attention, Mix-FFN convolutions), residuals"),
           "timing": "CUDA events, 3 warm-up + 4 timed steps, max over ranks; wrapped_linears_ms = events around every "
                     "wrapped-linear call of one further step"}
    del step, inputs
    torch.cuda.empty_cache()
    return rec


def _time_call(fn, n=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def sub_nvfp4_flux_gemms(dev):
    """The NVFP4 W4A4 GEMM alone on the three FLUX linear shapes at M = 16384 (batch 4 x 4096 image tokens), k = 384
    bf16 coefficients: CUDA events around 20 back-to-back launches, operands resident, 3 warm-ups.  Fraction against
    dense FP4 = 4 x the measured bf16 sustained figure (derived)."""
    from dirotq_b200 import ops
    peak, src = tensor_peak("nvfp4")
    out = {"peak_tflops": peak, "peak_source": src, "layers": []}
    g = torch.Generator(device=dev).manual_seed(0)
    M, D, k = 16384, 3072, 384
    x = torch.randn(M, D, generator=g, device=dev).to(torch.bfloat16)
    fmt = ops.ActFormat(ops.NVFP4_HW, D, tail_len=k, group_size=16)
    act = ops.quantize_act(x, fmt)
    lay = act.layout
    for N in (12288, 3072):
        wt = (torch.randn(N, lay.tail_pitch, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        bias = torch.randn(N, generator=g, device=dev).to(torch.bfloat16)
        pk = ops.pack_weight_nvfp4(torch.randn(N, lay.q_len, generator=g, device=dev) * 0.05, 2.0 ** -12)
        ms = _time_call(lambda: ops.gemm_w4a4_nvfp4(act, pk, wt, bias))
        tf = 2.0 * M * N * D / (ms * 1e-3) / 1e12
        tf4 = 2.0 * M * N * lay.q_len / (ms * 1e-3) / 1e12
        out["layers"].append({"shape": f"{D}->{N}", "M": M, "k_bf16": k, "us": ms * 1e3, "tflops": tf, "frac_of_fp4_peak": tf / peak,
                              "tflops_4bit_part_only": tf4,
                              "note": "tflops counts 2*M*N*D over the whole call; one eighth of K runs as bf16 UMMAs at a "
                                      "quarter of the FP4 rate in the same kernel"})
    # the K = 12288 down-projection of the speed path: no rotation, no 16-bit branch (dirotq_b200.dit.flux_double_block with
    # tail 0, as parallel.FluxLinearStep and denoise.py build it)
    D2, N2 = 12288, 3072
    x2 = torch.randn(M, D2, generator=g, device=dev).to(torch.bfloat16)
    fmt2 = ops.ActFormat(ops.NVFP4_HW, D2, tail_len=0, group_size=16)
    act2 = ops.quantize_act(x2, fmt2)
    pk2 = ops.pack_weight_nvfp4(torch.randn(N2, D2, generator=g, device=dev) * 0.05, 2.0 ** -12)
    bias2 = torch.randn(N2, generator=g, device=dev).to(torch.bfloat16)
    ms = _time_call(lambda: ops.gemm_w4a4_nvfp4(act2, pk2, None, bias2))
    tf = 2.0 * M * N2 * D2 / (ms * 1e-3) / 1e12
    out["layers"].append({"shape": f"{D2}->{N2}", "M": M, "k_bf16": 0, "us": ms * 1e3, "tflops": tf, "frac_of_fp4_peak": tf / peak,
                          "tflops_4bit_part_only": tf, "note": "un-rotated down-projection: all of K is 4-bit"})
    # one FLUX block's linears: q, k, v, out (3072 -> 3072 each), up, down
    us = {l["shape"]: l["us"] for l in out["layers"]}
    t_block = 4 * us["3072->3072"] + us["3072->12288"] + us["12288->3072"]
    f_block = 2.0 * M * (4 * 3072 * 3072 + 2 * 3072 * 12288)
    out["flux_block_linears"] = {"us": t_block, "tflops": f_block / t_block / 1e6, "frac_of_fp4_peak": f_block / t_block / 1e6 / peak,
                                 "note": "GEMM time of the six linears of one FLUX block (four 3072 -> 3072, up, down) at M = 16384"}
    ops.check_status(dev)
    return out


def sub_linear_step(D_, workload, n_blocks, chain=True, qkv=True):
    """Another workload's linear-path step on one GPU (resident inputs, 3 warm-up + 5 timed steps)."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    blk_name, _, quant, tokens, gbatch, family, desc = WORKLOADS[workload]
    dev = D_.dev
    block = getattr(dit, blk_name)()
    M = tokens * gbatch
    step = dit.LinearPathStep(block, n_blocks, quant, device=dev, seed=2000)
    backend.preconvert_rotations_to_device(step, dev)
    n_fused = backend.fuse_gelu_modules(step)
    n_chained = backend.fuse_ffn_quantise(step, keep_hidden=False) if chain else 0
    n_qkv = backend.fuse_sibling_gemms(step) if qkv else 0
    x = synth_activations(M, block[0].in_f, torch.Generator().manual_seed(3)).reshape(gbatch, tokens, -1).to(dev)
    for _ in range(3):
        step(x)
    ops.check_status(dev)
    ms = D_.timed(lambda: step(x), 5) / 5
    lin, _ = step.ops_per_step(M)
    peak, src = tensor_peak("nvfp4" if quant == "nvfp4" else "f16")
    rec = {"workload": desc, "blocks": n_blocks, "rows": M, "ms_per_step": ms, "tflops": lin / (ms * 1e-3) / 1e12,
           "frac_of_peak": lin / (ms * 1e-3) / 1e12 / peak, "peak_tflops": peak, "peak_source": src,
           "gelu_fused_layers": n_fused, "ffn_pairs_quantised_in_epilogue": n_chained, "qkv_groups_as_one_gemm": n_qkv,
           "launches_per_step": step.kernel_launches_per_step(),
           "note": "whole linear-path step (rotate + quantise kernels included in the time, only the linears' 2*M*N*D credited)"}
    del step, x
    torch.cuda.empty_cache()
    return rec


def sub_flux_step(D_, n_double, ffn, chain=True, qkv=True):
    """FLUX linear path on a slice of the stack (n_double double-stream blocks on both streams + 2 n_double
    single-stream blocks), fixed global batch 4.  Several GPUs: rows sharded, feed-forwards tensor-parallel; the NCCL
    time is the sum of CUDA-event pairs around every all-gather and reduce-scatter of one step."""
    from dirotq_b200 import backend, ops
    from dirotq_b200.parallel import FluxLinearStep
    from dirotq_b200.synth import synth_activations
    dev, world, rank = D_.dev, D_.world, D_.rank
    step = FluxLinearStep(world, rank, dev, batch=4, n_double=n_double, n_single=2 * n_double, ffn=ffn, quant="int4")
    backend.preconvert_rotations_to_device(step.layers, dev)
    step.fuse_gelu()
    n_chained = step.fuse_ffn_quantise() if chain else 0
    n_qkv = backend.fuse_sibling_gemms(step.layers) if qkv else 0
    for lyr in step._flat:
        lyr._b200_explicit = None
        lyr.rotation = lyr.rotation_per_head = None
    torch.cuda.empty_cache()
    M = step.rows_per_rank("single")
    x = synth_activations(M, 3072, torch.Generator().manual_seed(7 + rank)).to(dev)
    for _ in range(3):
        step(x)
    ops.check_status(dev)
    ms = D_.timed(lambda: step(x), 4) / 4
    rec = {"blocks": f"{n_double} double-stream (image + text) + {2 * n_double} single-stream of 19 + 38", "global_batch": 4,
           "rows_per_gpu": M, "ffn": step.ffn, "ms_per_step": ms,
           "tflops": step.ops_per_step()[0] / (ms * 1e-3) / 1e12, "ffn_pairs_quantised_in_epilogue": n_chained,
           "qkv_groups_as_one_gemm": n_qkv, "launches_per_step": step.kernel_launches_per_step()}
    if world > 1 and step.ffn == "tp":
        step.comm_pairs = []
        step(x)
        torch.cuda.synchronize()
        nccl_ms = sum(a.elapsed_time(b) for a, b in step.comm_pairs)
        t = torch.tensor([nccl_ms], device=dev)
        D_.dist.all_reduce(t, op=D_.dist.ReduceOp.MAX)
        step.comm_pairs = None
        rec.update(nccl_ms_per_step=float(t.item()), nccl_share=float(t.item()) / ms, collectives_per_step=3 * 4 * n_double,
                   overlap="the all-gather of single-stream blocks runs on a side stream beside the attention linears "
                           "(their inputs coincide); nccl_ms is device time of the collectives, overlapped or not")
    del step, x
    torch.cuda.empty_cache()
    return rec


# ---------------------------------------------------------------------------------------------
# roofline
# ---------------------------------------------------------------------------------------------
def roofline_pass(step, x_dev, M, quant, dev, steps, exact_int=False):
    """Runs the step's layers through the two C-ABI stages separately and brackets every launch of the
    W4A4 GEMM (the kernel with the largest share of the step) with CUDA events on the launching stream."""
    from dirotq_b200 import ops
    hbm, _, bf16_sust, which = measured_peaks()
    pairs, bufs = [], {}
    ops_total = bytes_total = 0.0
    f16_ws, f16_used = None, False
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
                                          st.w_codes, st.w_scales, st.w_rowscale)
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
    if quant == "nvfp4":
        kname, kind = "gemm_nvfp4_pair_kernel (CTA pairs; gemm_nvfp4_kernel up to 128 rows)", "nvfp4"
    elif f16_used:
        kname, kind = "gemm_int_f16_kernel (with its fold_expand_kernel or expand_weight_panel_kernel)", "f16"
    else:
        kname, kind = "gemm_int_kernel", "i8"
    peak, peak_src = tensor_peak(kind)
    k1 = None
    if k1_pairs:
        k1_ms = sum(a.elapsed_time(b) for a, b in k1_pairs)
        k1 = {"kernel": "rotate_quant_kernel (hidden rotation + split + quantise)", "bound": "tensor",
              "achieved": k1_flops / (k1_ms * 1e-3) / 1e12, "peak": bf16_sust, "unit": "TFLOP/s",
              "frac": k1_flops / (k1_ms * 1e-3) / 1e12 / bf16_sust,
              "hbm_gbs": k1_bytes / (k1_ms * 1e-3) / 1e9, "hbm_peak_gbs": hbm, "hbm_frac": k1_bytes / (k1_ms * 1e-3) / 1e9 / hbm,
              "launches_timed": len(k1_pairs), "avg_launch_us": k1_ms * 1e3 / len(k1_pairs)}
    n = max(1, len(pairs))
    return {"bound": "tensor", "kernel": kname, "rotate_quantise": k1,
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_src,
            "launches_timed": len(pairs), "avg_launch_us": t_ms * 1e3 / n,
            "algorithmic_bytes_per_launch": bytes_total / n,
            "traffic": None,
            "traffic_estimated": {"bytes_per_launch": NCU_TRAFFIC_RATIO * bytes_total / n,
                                  "how": f"NOT a measurement of this run: algorithmic bytes per launch x {NCU_TRAFFIC_RATIO}, the dram "
                                         "read + write over algorithmic bytes of one ncu capture of the INT4 GEMM at M=16384, N=K=1152 "
                                         "(profiles/); the output of a launch is still in the 126 MB L2 when it ends"}}


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
            if st.fmt.mode == ops.NVFP4_HW:
                pw = ops.PackedWeightNvfp4(st.out_features, st.layout.q_len, st.layout.n_chunks, st.w_tensor_scale,
                                           st.w_codes, st.w_scales, st.w_rowscale)
                ops.gemm_w4a4_nvfp4(buf, pw, st.w_tail, st.bias)
            else:
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
    nvfp4 = st.fmt.mode == ops.NVFP4_HW
    peak, peak_src = tensor_peak("nvfp4" if nvfp4 else "f16")
    return {"bound": "tensor", "kernel": ("gemm_nvfp4_pair_kernel (CTA pairs)" if nvfp4 else
                                          "gemm_int_f16_kernel (with its fold_expand_kernel or expand_weight_panel_kernel)"),
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_src,
            "launches_timed": len(pairs), "avg_launch_us": t_ms * 1e3 / max(1, len(pairs)), "traffic": None,
            "traffic_estimated": {"bytes_per_launch": NCU_TRAFFIC_RATIO * gemm_algorithmic_bytes(M, 3072, st.layout, "nvfp4" if nvfp4 else "int4"),
                                  "how": f"NOT a measurement of this run: algorithmic bytes x {NCU_TRAFFIC_RATIO} (ratio of one ncu "
                                         "capture of the INT4 GEMM at M=16384, N=K=1152)"}}


def profile_case(which):
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    torch.cuda.set_device(0)
    with contextlib.redirect_stdout(sys.stderr):
        if which == "flux_nvfp4":
            M = 4096
            x = synth_activations(M, 3072, torch.Generator().manual_seed(0)).cuda()
            w = dit.make_wrapped_linear(dit.LayerDef("probe", 3072, 12288, tail=384), "nvfp4", 5, "cuda")
            st = backend.prepare_layer(w, "cuda", w._b200_explicit)
            for _ in range(3):
                backend.linear_forward(st, x)
        elif which == "flux_int4":
            M = 18432                                       # FLUX single-stream rows at batch 4: the up-projection
            x = synth_activations(M, 3072, torch.Generator().manual_seed(0)).cuda()
            w = dit.make_wrapped_linear(dit.LayerDef("probe", 3072, 12288, tail=384), "int4", 5, "cuda")
            st = backend.prepare_layer(w, "cuda", w._b200_explicit)
            for _ in range(3):
                backend.linear_forward(st, x)
        elif which == "perhead":
            M = 16384                                       # SANA out-projection: 70 heads x 32, 4 channels per head 16-bit
            x = synth_activations(M, 2240, torch.Generator().manual_seed(0)).cuda()
            w = dit.make_wrapped_linear(dit.LayerDef("probe", 2240, 2240, kind="perhead", tail=4, heads=70, head_dim=32),
                                        "int4", 5, "cuda")
            st = backend.prepare_layer(w, "cuda", w._b200_explicit)
            for _ in range(3):
                backend.linear_forward(st, x)
        elif which == "glue":
            from dirotq_b200 import denoise
            B, T, S, D, H = 4, 4096, 512, 3072, 24         # FLUX-shaped: 151 MB per [B, T, D] tensor
            M = B * T
            g = torch.Generator().manual_seed(0)
            x = synth_activations(M, D, g).reshape(B, T, D).cuda()
            y = synth_activations(M, D, g).reshape(B, T, D).cuda()
            mod = (torch.randn(B, 6 * D, generator=g) * 0.3).to(torch.bfloat16).cuda()[:, None].chunk(6, dim=-1)
            qkv = synth_activations(M, 3 * D, g).cuda()
            q, k, v = [qkv[:, j * D:(j + 1) * D].reshape(B, T, D) for j in range(3)]
            cos, sin = denoise.rope_tables(S + T, D // H, "cuda")
            w = torch.ones(D // H, dtype=torch.bfloat16, device="cuda")
            bufs = tuple(torch.empty(B, S + T, H, D // H, dtype=torch.bfloat16, device="cuda") for _ in range(3))
            for _ in range(3):
                ops.layernorm_modulate(x, mod[1], mod[0])
                ops.gated_residual(x, y, mod[2])
                ops.qkv_norm_rope(q, k, v, H, w, w, cos, sin, out=bufs, t0=S)
        elif which == "quantize":
            M = 4096
            x = synth_activations(M, 12288, torch.Generator().manual_seed(0)).cuda()
            for mode in (ops.INT4_SYM, ops.NVFP4_HW):
                fmt = ops.ActFormat(mode, 12288, tail_len=0, group_size=16 if mode == ops.NVFP4_HW else 64)
                buf = ops.alloc_act(fmt, M, "cuda")
                for _ in range(3):
                    ops.quantize_act(x, fmt, out=buf)
        else:
            M = 16384
            x = synth_activations(M, 1152, torch.Generator().manual_seed(0)).cuda()
            for quant in ("int4", "nvfp4"):
                w = dit.make_wrapped_linear(dit.LayerDef("probe", 1152, 1152, tail=64), quant, 5, "cuda")
                st = backend.prepare_layer(w, "cuda", w._b200_explicit)
                for _ in range(3):
                    backend.linear_forward(st, x)
    torch.cuda.synchronize()
    ops.check_status()
    print(json.dumps({"profile_case": which, "rows": M}))


if __name__ == "__main__":
    a = parse()
    if a.cache_weight_panel:
        from dirotq_b200 import backend as _backend
        _backend.CACHE_WEIGHT_PANEL = True
    if a.no_resident_panels:
        from dirotq_b200 import backend as _backend
        _backend.PANEL_CACHE_BUDGET_FRACTION = 0.0
    if a.exact_int:
        from dirotq_b200 import backend as _backend
        _backend.INT4_TENSOR_RATE_GEMM = False
    if a.profile_case:
        profile_case(a.profile_case)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
