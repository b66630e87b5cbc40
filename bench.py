"""Benchmark of the FP8 MoE prefill layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

One step = one pass of the layer (route -> sort -> up/SiLU/requant/down -> reduce) over one
synthetic prefill batch. N=1 runs the Qwen3.5-35B-A3B-like layer (H=2048, E=256, top-8,
I=512, block-FP8 weights) at T=16384 tokens; N>1 runs the same layer expert-parallel (256/N
experts per rank, all tokens on every rank) with the ranks' partial outputs reduced inside the
kernel or by NCCL after it, whichever was measured faster for that N (--reduce overrides;
--parallel tp selects the tensor-parallel split, --model deepseek the DeepSeek-V3-like layer).
Before anything is timed at N>1 the reduced output of exactly that configuration is checked
against an unfused launch + all-reduce and against the CPU oracle; when the in-kernel reduce was chosen by
the table (not by --reduce fused) and fails that check or leaves a device status, the line says so
(`reduce_fallback`) and kernel + NCCL is checked and timed instead (BENCH_INJECT_FUSED_REJECT=1 exercises
that branch from the host). Prints ONE JSON line (rank 0).
--impl reference times the reference's CPU path (torch MoE on dequantised weights, host cores)
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from unimonomoe_b200 import MonoKernel, synth, tp_fused, variant_path  # noqa: E402

NOMINAL_FP8_TFLOPS = 4500.0
METRIC = "moe_layer_prefill_fp8_tflops"
UNIT = "TFLOP/s"


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p))
        except Exception:
            pass
    return {}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.003)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self) -> dict:
        return {"sm_mhz": (statistics.median(self.samples) if self.samples else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def fp8_gemm_tflops(dev) -> float | None:
    """Library FP8 GEMM throughput (torch._scaled_mm e4m3 x e4m3 8192^3, best of 10): context for the
    roofline, never part of a timed step."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        best = None
        for i in range(13):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if i >= 3:
                best = ms if best is None else min(best, ms)
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


REFERENCE_SAMPLE_TOKENS = 2048   # 64 rows per expert on average; a pass stays within seconds on host cores


def cpu_reference_layer(spec, layer_cpu, hs, threads: int, dtype=torch.float32, with_router=True, with_shared=True):
    """The reference's CPU path for one layer, in torch on `threads` host threads: router linear, softmax
    top-8 with renormalised weights, per expert x @ W13^T -> SiLU(gate)*up -> @ W2^T on dequantised
    block-FP8 weights and the weighted sum (validation/ep4_acc.py:183-217), plus the sigmoid-gated shared
    expert. Returns the layer output."""
    from oracle import cpu_oracle as O
    torch.set_num_threads(threads)
    if with_router:
        logits = torch.nn.functional.linear(hs.to(dtype), layer_cpu["router_w"].to(dtype)).float()
    else:
        logits = layer_cpu["_logits"]
    top = torch.topk(logits, spec.top_k, dim=1)
    w = torch.softmax(logits, 1).gather(1, top.indices)
    w = w / w.sum(1, keepdim=True).clamp(min=1e-30)
    out = O.moe_fp64(hs, top.indices, w, layer_cpu["w13"], layer_cpu["w13_scale"], layer_cpu["w2"],
                     layer_cpu["w2_scale"], dtype=dtype)
    if with_shared and layer_cpu.get("shared") is not None:
        out = out + O.shared_expert_fp(hs, layer_cpu["shared"], dtype=dtype)
    return out


def _cpu_case(spec, tokens):
    layer = synth.make_layer(spec, seed=0, device="cpu", with_shared=True)
    batch = synth.make_batch(spec, layer, tokens, seed=0, device="cpu")
    layer["_logits"] = batch["logits"]
    return layer, batch


def _time_cpu(fn, reps: int) -> float:
    fn()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def time_cpu_baseline(spec, sample_tokens: int, reps: int = 2) -> dict:
    threads = os.cpu_count() or 1
    layer, batch = _cpu_case(spec, sample_tokens)
    sec = _time_cpu(lambda: cpu_reference_layer(spec, layer, batch["hs"], threads), reps)
    fl = synth.routed_flops(spec, sample_tokens)
    return {"value": fl / sec / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample_tokens} tokens of the same layer (all 256 experts): router linear, softmax top-8, routed "
                      f"experts and the gated shared expert in torch fp32 on dequantised weights, median of {reps} "
                      f"passes, {sec * 1e3:.0f} ms per pass; value counts the routed FLOPs only",
            "ms_per_step": sec * 1e3}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = synth.QWEN
    sample = REFERENCE_SAMPLE_TOKENS
    threads = os.cpu_count() or 1
    layer, batch = _cpu_case(spec, sample)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        cpu_reference_layer(spec, layer, batch["hs"], threads)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    # context: the same pass in the oracle's own precision, and the routed experts alone
    sec64 = _time_cpu(lambda: cpu_reference_layer(spec, layer, batch["hs"], threads, dtype=torch.float64), 1)
    sec_routed = _time_cpu(lambda: cpu_reference_layer(spec, layer, batch["hs"], threads, with_router=False,
                                                       with_shared=False), 1)
    flops = synth.routed_flops(spec, sample)
    val = flops / sec / 1e12
    what = (f"{spec.name} MoE layer, reference CPU path (router linear, softmax top-8, routed experts on dequantised "
            f"block-FP8 weights, gated shared expert; torch fp32, {threads} host threads) on a {sample}-token batch "
            f"(the GPU arm runs T={args.tokens})")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": what, "tokens": sample, "gpu_arm_tokens": args.tokens},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} tokens per step: {what}; value counts the routed FLOPs only",
                         "fp64_ms_per_step": sec64 * 1e3, "fp64_value": flops / sec64 / 1e12,
                         "routed_experts_only_ms_per_step": sec_routed * 1e3,
                         "flops_incl_router_and_shared": flops + 2.0 * sample * spec.hidden * spec.experts
                         + 6.0 * sample * spec.hidden * spec.shared_inter},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--model", default="qwen", choices=["qwen", "deepseek"],
                    help="deepseek: DeepSeek-V3-like layer (H=7168, I=2048, grouped sigmoid router), tensor parallel, N=4 or 8")
    ap.add_argument("--parallel", default="auto", choices=["auto", "tp", "ep"],
                    help="N>1: tensor parallel (N=2,4) or expert parallel; auto = ep")
    ap.add_argument("--unfused", action="store_true", help="N>1: same as --reduce nccl")
    ap.add_argument("--reduce", default="auto", choices=["auto", "fused", "nccl"],
                    help="N>1: all-reduce of the ranks' partial outputs inside the kernel (NVLS multimem) or by NCCL "
                         "after it; auto takes what FUSED_REDUCE_WINS records as faster for this split and N")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="after the timed steps, repeat the same launch for this long and report the steady-state "
                         "time and clocks (0: skip)")
    ap.add_argument("--no-verify", action="store_true", help="N>1: skip the pre-timing parity check (profiling runs)")
    ap.add_argument("--chunks", type=int, default=0, help="N>1, in-kernel reduce: chunks the reduce is released in (0: table)")
    ap.add_argument("--sweep", default="", help="N>1, in-kernel reduce: time these 'chunks:ncomm' pairs (comma separated) "
                                                "after the contract line's own run and print them on stderr")
    ap.add_argument("--router", default="logits", choices=["logits", "gemv"],
                    help="logits: the caller's router logits go in (the reference's interface); gemv: the bf16 gate "
                         "weight goes in and the router linear runs inside the launch (no logits cross PCIe in e2e)")
    ap.add_argument("--gather", default="nccl", choices=["nccl", "multimem", "ce"],
                    help="N>1, e2e leg: how the row shards uploaded by the ranks are completed on every GPU: NCCL "
                         "all-gather, multimem stores into symmetric buffers (measured equal at 2 GPUs), or 'ce': every "
                         "rank pushes its rows into the peers' symmetric buffers with copy-engine copies and the ranks "
                         "signal each other with stream-ordered 32-bit writes and waits, so that nothing of the "
                         "exchange needs an SM while the persistent kernel holds them all")
    ap.add_argument("--variant", default=None,
                    help="N=1 only: time another binary of the same geometry, e.g. a development build made with "
                         "`python -m unimonomoe_b200.build qwen_w1_prof` (stall counters) or qwen_w1_abl7 (a piece of "
                         "the work left out: wrong results, used to split the run time)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end leg, the library GEMM probe and the CPU baseline (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else max(args.warmup, 1)
    if args.impl == "reference":
        run_reference(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernel has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    spec = synth.QWEN if args.model == "qwen" else synth.DEEPSEEK
    T = args.tokens
    if args.model == "deepseek":
        if world not in (1, 2, 4, 8):
            raise SystemExit("the DeepSeek-V3 geometry is built for 1, 2, 4 and 8 GPUs (tensor parallel)")
        variant, par = ("ds_w1", "none") if world == 1 else (f"ds_tp{world}", f"tp{world}")
        n = spec.inter // world
        kw = {"inter_slice": (rank * n, (rank + 1) * n), "chunk": 8}
    elif world == 1:
        variant, par, kw = (args.variant or "qwen_w1"), "none", {}
    elif world in (2, 4) and args.parallel == "tp":
        variant, par = f"qwen_tp{world}", f"tp{world}"
        n = spec.inter // world
        kw = {"inter_slice": (rank * n, (rank + 1) * n)}
    else:
        variant, par = f"qwen_ep{world}", f"ep{world}"
        n = spec.experts // world
        kw = {"expert_slice": (rank * n, (rank + 1) * n)}
    mk = MonoKernel(variant_path(variant))
    layer = synth.make_layer(spec, seed=0, device=dev, with_shared=False, **kw)
    emap = synth.expert_map(spec, rank, world, device=dev) if par.startswith("ep") else None
    full_router = layer
    batch = synth.make_batch(spec, full_router, T, seed=0, device=dev)
    out = torch.empty(T, spec.hidden, dtype=torch.bfloat16, device=dev)
    sc = mk.scratch(T, dev)

    # N > 1: the all-reduce of the ranks' partial outputs runs inside the kernel (NVLS multimem through a
    # symmetric pool) when every rank can; otherwise NCCL reduces after the kernel.
    plan = None
    # shape of the in-kernel reduce (chunks, communication CTAs) measured best per group size at T = 16384
    shape_chunks, shape_ncomm = REDUCE_SHAPES.get(world, (8, 32))
    os.environ.setdefault("VLLM_PREFILL_MONOKERNEL_TP_NCOMM", str(shape_ncomm))
    reduce_mode = "nccl" if args.unfused else args.reduce
    if reduce_mode == "auto":
        reduce_mode = "fused" if FUSED_REDUCE_WINS.get((args.model, par[:2], world), True) else "nccl"
    if world > 1:
        # the symmetric pool is built even when NCCL reduces: the parity check before the timing uses it
        plan = tp_fused.FusedTPPlan(mk, dist.group.WORLD, hidden=spec.hidden, max_tokens=T, nslots=2)
        if plan.usable and args.chunks > 0:
            plan.chunks_by_tokens[T] = args.chunks
        elif plan.usable:
            plan.chunks_by_tokens[T] = shape_chunks if T >= 16384 else max(1, shape_chunks // 2)
        if not plan.usable:
            if rank == 0:
                print(f"# fused TP epilogue unavailable ({plan.reason}); reducing with NCCL", file=sys.stderr)
            plan = None
    pool_plan = plan                      # kept for the parity check
    if reduce_mode != "fused":
        plan = None
    reduce_desc = "none" if world == 1 else (
        (f"in-kernel all-reduce ({'direct peer loads' if world == tp_fused.PEER_REDUCE_WORLD else 'NVLS multimem'}), "
         f"{plan.chunks_for(T)} chunks, {plan.ncomm} communication CTAs + every summing CTA once its sums are done")
        if plan is not None else "NCCL all-reduce after the kernel")

    rw16 = None
    if args.router == "gemv":
        if plan is not None:
            raise SystemExit("--router gemv is wired for the unfused launch only: add --unfused")
        rw16 = layer["router_w"].to(torch.bfloat16).contiguous()

    def launch(hs, lg, dst=None):
        if plan is not None:
            slot = 1 if (dst is not None and dst.data_ptr() == plan.pool.base_ptr(1)) else 0
            plan.fused_tp_launch(hs, lg, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], spec.top_k,
                                 True, layer["bias"], expert_map=emap, slot=slot)
        else:
            mk.prefill_impl(hs, lg, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], spec.top_k, True,
                            layer["bias"], out if dst is None else dst, expert_map=emap, scratch=sc, router_weight=rw16)

    def reduce_out(dst=None):
        if world > 1 and plan is None:
            dist.all_reduce(out if dst is None else dst)

    def step():
        launch(batch["hs"], batch["logits"])
        reduce_out()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def warm_up_and_verify():
        """Warm-up steps, the device status of every rank, then the parity check of what is about to be timed.
        Returns (parity or None, reason the configuration must not be timed or None); the same on every rank."""
        for _ in range(args.warmup):
            step()
        barrier()
        why = uniform_status(mk, sc["workspace"], world, dist, dev)
        if why is not None and world == 1:
            raise RuntimeError(why)
        if why is not None or world == 1 or args.no_verify:
            return None, why
        result_now = plan.pool.output(T) if plan is not None else out
        par_info = verify_reduced_output(spec, mk, layer, batch, emap, sc, pool_plan, result_now, world, rank, dist,
                                         dev, par, kw, fused=plan is not None)
        return par_info, (None if par_info["ok"] else "parity check failed")

    reduce_fallback = None
    parity, why = warm_up_and_verify()
    if os.environ.get("BENCH_INJECT_FUSED_REJECT") == "1" and plan is not None and why is None:
        why = "injected by BENCH_INJECT_FUSED_REJECT (host-side test of the fallback)"
    if why is not None and plan is not None and args.reduce == "auto" and not args.unfused:
        # the in-kernel reduce was chosen by the table, not asked for: say what happened and time the launch
        # followed by NCCL instead, behind the same check (a launch that gave up a wait leaves the status word set
        # for the host to read and returns; the next launch starts clean)
        reduce_fallback = {"from": reduce_desc, "why": why, "parity": parity}
        if rank == 0:
            print(f"# in-kernel reduce rejected ({why}); timing kernel + NCCL all-reduce instead", file=sys.stderr)
        plan = None
        reduce_desc = "NCCL all-reduce after the kernel"
        parity, why = warm_up_and_verify()
    if why is not None:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "parity_checked": False, "why": why, "parity": parity,
                              "reduce_fallback": reduce_fallback}), flush=True)
        raise SystemExit(3)

    # ---- device-resident timing: K steps between two events, plus one event pair per kernel launch
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clk:
        barrier()
        e0.record()
        for a, b in evs:
            a.record()
            launch(batch["hs"], batch["logits"])
            b.record()
            reduce_out()
        e1.record()
        barrier()
    total_ms = e0.elapsed_time(e1)
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    mk.check_status(sc["workspace"])
    t = torch.tensor([total_ms, kern_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kern_ms = float(t[0]), float(t[1])
    ms_per_step = total_ms / args.steps
    flops = synth.routed_flops(spec, T)  # whole job: all ranks together
    value = flops / (ms_per_step * 1e-3) / 1e12

    sustained = None
    if args.sustained_seconds > 0:
        sustained = run_sustained(args.sustained_seconds, ms_per_step, launch, reduce_out, batch, barrier, world, dist, dev,
                                  physical_gpu_index(local), flops)
        mk.check_status(sc["workspace"])

    with_shared = None
    if world == 1 and args.model == "qwen" and not args.kernel_only and args.variant is None and mk.has_shared:
        with_shared = time_with_shared_expert(spec, mk, layer, batch, out, sc, args.steps, dev, flops)

    extra = None
    if world in (4, 8) and args.model == "qwen" and args.parallel == "auto" and not args.kernel_only:
        # the north star's other splits, each behind the same parity check: Qwen tensor parallel over 4 GPUs,
        # the DeepSeek-V3-like layer tensor parallel over 8
        extra = time_other_split("qwen" if world == 4 else "deepseek", world, rank, dist, dev, barrier,
                                 8192 if world == 8 else T)

    if args.sweep and plan is not None:
        sweep_reduce_shapes(args.sweep, plan, T, launch, batch, barrier, dist, dev, mk, sc, rank)

    e2e_ms = None
    if not args.kernel_only:
        result = plan.pool.output(T) if plan is not None else out
        # a second output slot (a second slot of the symmetric pool under the fused reduce) lets the next
        # kernel run while the previous result is still going to the host
        second = plan.pool.output(T, 1) if plan is not None else torch.empty_like(out)
        e2e_ms = time_e2e(args, spec, batch, result, launch, reduce_out, world, rank, dist, barrier, dev,
                          with_logits=rw16 is None, second_out=second)
    h2d = batch["hs"].numel() * 2 + (batch["logits"].numel() * 4 if rw16 is None else 0)
    d2h = out.numel() * 2

    phases = None
    if rank == 0:   # of the contract's own launch, before anything else runs through this workspace
        ph = mk.workspace_view(sc["workspace"])["phase_ns"].tolist()
        phases = [round((ph[i + 1] - ph[i]) / 1e3, 1) for i in range(4)]
        stall_counters(mk, sc["workspace"])

    e2e_router_inside = None
    if world == 1 and not args.kernel_only and rw16 is None and args.model == "qwen" and args.variant is None and mk.has_gemv:
        # the same step with the router linear inside the launch (the gate weight stays on the device like every
        # other weight): only the hidden states cross PCIe, the logits are computed, not uploaded
        rw_in = layer["router_w"].to(torch.bfloat16).contiguous()

        def launch_gemv(hs, lg, dst=None):
            mk.prefill_impl(hs, lg, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], spec.top_k, True,
                            layer["bias"], out if dst is None else dst, expert_map=emap, scratch=sc, router_weight=rw_in)
        g_ms = time_e2e(args, spec, batch, out, launch_gemv, reduce_out, world, rank, dist, barrier, dev,
                        with_logits=False, second_out=torch.empty_like(out))
        mk.check_status(sc["workspace"])
        e2e_router_inside = {"value": flops / (g_ms[0] * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": g_ms[0],
                             "serial_ms_per_step": g_ms[1], "h2d_bytes_per_step": batch["hs"].numel() * 2,
                             "d2h_bytes_per_step": d2h,
                             "entry": "launch_prefill_moe_wgmma_q1_gemv: logits = x . W_r^T computed in phase R of the same launch"}

    if rank == 0:
        report(args, spec, T, world, par, variant, value, ms_per_step, kern_ms, flops, e2e_ms, h2d, d2h, clk, dev,
               reduce_desc, phases, sustained, parity, with_shared, extra, reduce_fallback, e2e_router_inside)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


PROF_NAMES = ["tma_wait_emptyB", "mma_wait_fullB", "mma_wait_fullA", "mma_wait_tmem", "mma_wait_inter", "mma_total",
              "gather_wait_emptyA", "phase0_route", "epi_wait_full", "epi_up", "epi_silu", "epi_down", "epi_store",
              "epi_total", "epi_bar", "phase0_quant"]


def stall_counters(mk, workspace) -> None:
    """A binary built with -DMONO_PROFILE leaves per-role clock64 sums in the workspace: print their mean over
    the 148 CTAs, in thousands of cycles, on stderr (the JSON line stays the contract's)."""
    off = mk._int_symbol("prof_offset")
    if off is None:
        return
    raw = workspace.cpu()[off: off + 148 * 64 * 8]
    if raw.numel() != 148 * 64 * 8:
        return
    pr = raw.view(torch.int64).view(148, 64).double()
    if float(pr.sum()) == 0.0:
        return
    print("# stall counters of the last launch, mean over CTAs, kcycles: " +
          ", ".join(f"{n}={pr[:, i].mean().item() / 1e3:.1f}" for i, n in enumerate(PROF_NAMES) if n != "-"),
          file=sys.stderr)
    for row, who in ((16, "epilogue waiting for a full accumulator"), (40, "MMA thread waiting for a free accumulator")):
        h = pr[:, row: row + 24].mean(0) / 1e3
        print(f"# {who}, kcycles by slab of the pass: up " + " ".join(f"{v:.1f}" for v in h[:16].tolist())
              + " | down " + " ".join(f"{v:.1f}" for v in h[16:20].tolist()), file=sys.stderr)


class _CopyEngineGather:
    """All-gather of the ranks' uploaded row shards without any kernel: symmetric input buffers (two slots), every
    rank copies its rows into each peer's buffer with device-to-device copies (copy engines), then raises a
    counter in the peer's memory with a stream-ordered 32-bit write; the consumer's stream waits on those counters
    with a stream-ordered wait. A second set of counters tells the producers that a slot has been read (the kernel
    that used it is finished) before it is overwritten. Counters only grow (use number of the slot)."""

    def __init__(self, batch, rows, nb, world, rank, dist, dev, with_logits):
        self.ok, self.why = False, ""
        self.rows, self.nb, self.world, self.rank, self.with_logits = rows, nb, world, rank, with_logits
        self.use = [0] * nb
        try:
            import torch.distributed._symmetric_memory as sm
            from cuda.bindings import driver as drv
            self.drv = drv
            gname = dist.group.WORLD.group_name
            self.hs = [sm.empty(batch["hs"].shape, dtype=batch["hs"].dtype, device=dev) for _ in range(nb)]
            self.lg = [sm.empty(batch["logits"].shape, dtype=batch["logits"].dtype, device=dev) for _ in range(nb)]
            self.flags = sm.empty((2 * nb * world + 1,), dtype=torch.uint32, device=dev)   # + one word for the self-test
            self.flags.view(torch.int32).zero_()
            torch.cuda.synchronize()
            h_hs = [sm.rendezvous(t, gname) for t in self.hs]
            h_lg = [sm.rendezvous(t, gname) for t in self.lg]
            self.h_flags = sm.rendezvous(self.flags, gname)
            peers = [p for p in range(world) if p != rank]
            self.peers = peers
            self.hs_peer = [{p: h_hs[b].get_buffer(p, batch["hs"].shape, batch["hs"].dtype) for p in peers} for b in range(nb)]
            self.lg_peer = [{p: h_lg[b].get_buffer(p, batch["logits"].shape, batch["logits"].dtype) for p in peers} for b in range(nb)]
            self.flags_peer = {p: self.h_flags.get_buffer(p, (2 * nb * world + 1,), torch.uint32) for p in peers}
            self.flags_flat = self.flags.view(-1)
            # self-test of the two stream memory operations on this rank's own word (already satisfied wait)
            last = 2 * nb * world
            self.h_flags.stream_write_value32(self.flags_flat, last, 7)
            cur = torch.cuda.current_stream()
            (err,) = drv.cuStreamWaitValue32(drv.CUstream(cur.cuda_stream), drv.CUdeviceptr(self.flags_flat.data_ptr() + 4 * last),
                                             7, drv.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ)
            torch.cuda.synchronize()
            if int(err) != 0 or int(self.flags_flat.view(torch.int32)[last].item()) != 7:
                raise RuntimeError(f"stream memory operations not usable here (err {err})")
            dist.barrier()
            self.ok = True
        except Exception as ex:  # noqa: BLE001 - any failure means "use the NCCL path"
            self.why = f"{type(ex).__name__}: {ex}"

    def _idx(self, kind, b, src):
        return (kind * self.nb + b) * self.world + src

    def _wait(self, stream, kind, b, value):
        drv = self.drv
        for p in self.peers:
            addr = self.flags_flat.data_ptr() + 4 * self._idx(kind, b, p)
            (err,) = drv.cuStreamWaitValue32(drv.CUstream(stream.cuda_stream), drv.CUdeviceptr(addr), value,
                                             drv.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ)
            if int(err) != 0:
                raise RuntimeError(f"cuStreamWaitValue32 failed: {err}")

    def _signal(self, kind, b, value):
        for p in self.peers:     # on the current stream, behind the copies / the kernel
            self.h_flags.stream_write_value32(self.flags_peer[p], self._idx(kind, b, self.rank), value)

    def begin(self, b, stream) -> int:
        """Next use of slot b: wait until every peer has read its previous contents. Returns the use number."""
        self.use[b] += 1
        u = self.use[b]
        if u > 1:
            self._wait(stream, 1, b, u - 1)
        return u

    def upload_and_push(self, b, hs_host, lg_host, u) -> None:
        rows = self.rows
        self.hs[b][rows].copy_(hs_host, non_blocking=True)
        if self.with_logits:
            self.lg[b][rows].copy_(lg_host, non_blocking=True)
        for p in self.peers:
            self.hs_peer[b][p][rows].copy_(self.hs[b][rows], non_blocking=True)
            if self.with_logits:
                self.lg_peer[b][p][rows].copy_(self.lg[b][rows], non_blocking=True)
        self._signal(0, b, u)

    def wait_full(self, b, stream, u) -> None:
        self._wait(stream, 0, b, u)

    def release(self, b, u) -> None:
        self._signal(1, b, u)


def time_e2e(args, spec, batch, out, launch, reduce_out, world, rank, dist, barrier, dev, with_logits=True,
             second_out=None) -> tuple:
    """End to end through the public API: host buffers in, host result out, every step's copies inside the
    timed region. Returns (ms per step with the steps software-pipelined, ms per step strictly serial).

    Pipelined: the upload of step i+1, the kernel of step i and the download of step i-1 run on three
    streams over two input slots (and two output slots when `second_out` is given; with one output slot the
    next kernel waits for the download). Every step still moves its own inputs and its own result.

    N > 1: the batch crosses PCIe once, not once per GPU. Rank r uploads rows [r*T/N, (r+1)*T/N) of the
    hidden states and logits, an all-gather over NVLink (multimem stores into symmetric buffers, or NCCL
    where there is no multicast) completes them on every GPU (on the compute
    stream, directly in front of the kernel: a collective that ran beside the persistent kernel could wait
    for a peer whose GPU is occupied by that very kernel), and rank r downloads the same rows of the
    reduced output."""
    T = batch["hs"].shape[0]
    assert T % world == 0
    rows = slice(rank * (T // world), (rank + 1) * (T // world))
    hs_host = batch["hs"][rows].cpu().pin_memory()
    lg_host = batch["logits"][rows].cpu().pin_memory()
    outs = [out] if second_out is None else [out, second_out]
    out_host = [torch.empty(T // world, spec.hidden, dtype=torch.bfloat16).pin_memory() for _ in outs]
    NB = 2
    gather_kind = "none"
    if world > 1:
        # the gathered inputs live in symmetric memory when the platform offers multicast, so that the
        # all-gather is one multimem store per element instead of a ring of copies
        try:
            if args.gather == "nccl":
                raise RuntimeError("NCCL all-gather selected")
            import torch.distributed._symmetric_memory as sm
            gname = dist.group.WORLD.group_name
            hs_dev = [sm.empty(batch["hs"].shape, dtype=batch["hs"].dtype, device=dev) for _ in range(NB)]
            lg_dev = [sm.empty(batch["logits"].shape, dtype=batch["logits"].dtype, device=dev) for _ in range(NB)]
            for t in hs_dev + lg_dev:
                if not int(sm.rendezvous(t, gname).multicast_ptr):
                    raise RuntimeError("no multicast pointer")
            gather_kind = "multimem"
        except Exception as ex:  # plain device buffers and NCCL instead
            if rank == 0 and args.gather != "nccl":
                print(f"# symmetric all-gather unavailable ({ex}); using NCCL", file=sys.stderr)
            gather_kind = "nccl"
        ok = torch.tensor([1 if gather_kind == "multimem" else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # every rank must take the same path
        if int(ok.item()) == 0:
            gather_kind = "nccl"
    ce = None
    if world > 1 and args.gather == "ce":
        ce = _CopyEngineGather(batch, rows, NB, world, rank, dist, dev, with_logits)
        ok = torch.tensor([1 if ce.ok else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            if rank == 0:
                print(f"# copy-engine all-gather unavailable ({ce.why}); using NCCL", file=sys.stderr)
            ce = None
        else:
            gather_kind = "ce"
            hs_dev, lg_dev = ce.hs, ce.lg
    if gather_kind not in ("multimem", "ce"):
        hs_dev = [torch.empty_like(batch["hs"]) for _ in range(NB)]
        lg_dev = [torch.empty_like(batch["logits"]) for _ in range(NB)]
    hs_part = [torch.empty_like(batch["hs"][rows]) for _ in range(NB)] if world > 1 else None
    lg_part = [torch.empty_like(batch["logits"][rows]) for _ in range(NB)] if world > 1 else None
    cur = torch.cuda.current_stream()
    s_in, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(NB)]     # upload of the slot finished
    ev_k = [torch.cuda.Event() for _ in range(NB)]      # the kernel that read the slot finished
    ev_o = [torch.cuda.Event() for _ in outs]           # download of the output slot finished

    def upload(b):
        if world == 1:
            hs_dev[b].copy_(hs_host, non_blocking=True)
            if with_logits:
                lg_dev[b].copy_(lg_host, non_blocking=True)
        else:
            hs_part[b].copy_(hs_host, non_blocking=True)
            if with_logits:
                lg_part[b].copy_(lg_host, non_blocking=True)

    def gather(b):
        if gather_kind == "multimem":
            torch.ops.symm_mem.multimem_all_gather_out(hs_part[b], gname, hs_dev[b])
            if with_logits:
                torch.ops.symm_mem.multimem_all_gather_out(lg_part[b], gname, lg_dev[b])
        elif world > 1:
            dist.all_gather_into_tensor(hs_dev[b], hs_part[b])
            if with_logits:
                dist.all_gather_into_tensor(lg_dev[b], lg_part[b])

    def serial_step():
        if ce is not None:
            u = ce.begin(0, cur)
            ce.upload_and_push(0, hs_host, lg_host, u)
            ce.wait_full(0, cur, u)
            launch(hs_dev[0], lg_dev[0], outs[0])
            reduce_out(outs[0])
            ce.release(0, u)
            out_host[0].copy_(outs[0][rows], non_blocking=True)
            return
        upload(0)
        gather(0)
        launch(hs_dev[0], lg_dev[0], outs[0])
        reduce_out(outs[0])
        out_host[0].copy_(outs[0][rows], non_blocking=True)

    def piped_step(i):
        b, o = i % NB, i % len(outs)
        if ce is not None:
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_k[b])
                u = ce.begin(b, s_in)
                ce.upload_and_push(b, hs_host, lg_host, u)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(ev_in[b])
                s_c.wait_event(ev_o[o])
                ce.wait_full(b, s_c, u)
                launch(hs_dev[b], lg_dev[b], outs[o])
                reduce_out(outs[o])
                ev_k[b].record(s_c)
                ce.release(b, u)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[b])
                out_host[o].copy_(outs[o][rows], non_blocking=True)
                ev_o[o].record(s_out)
            return
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_k[b])
            upload(b)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_c):
            s_c.wait_event(ev_in[b])
            s_c.wait_event(ev_o[o])
            gather(b)
            launch(hs_dev[b], lg_dev[b], outs[o])
            reduce_out(outs[o])
            ev_k[b].record(s_c)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_k[b])
            out_host[o].copy_(outs[o][rows], non_blocking=True)
            ev_o[o].record(s_out)

    def timed(fn, n, piped):
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(cur)
        if piped:
            for st in (s_in, s_c, s_out):
                st.wait_event(e2)
            for e in ev_k + ev_o:
                e.record(cur)
        for i in range(n):
            fn(i) if piped else fn()
        if piped:
            for st in (s_in, s_c, s_out):
                cur.wait_stream(st)
        e3.record(cur)
        barrier()
        t = torch.tensor([e2.elapsed_time(e3) / n], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    n_e2e = max(6, min(args.steps, 20))
    timed(serial_step, 3, False)
    serial_ms = timed(serial_step, n_e2e, False)
    timed(piped_step, 4, True)
    piped_ms = timed(piped_step, n_e2e, True)
    # where a pipelined step's time can go: host time to enqueue one step (Python, ctypes, NCCL enqueue), and the
    # copies alone; the kernel and the all-gather alone are reported beside them
    t0 = time.perf_counter()
    for i in range(8):
        piped_step(i)
    host_enqueue_ms = (time.perf_counter() - t0) / 8 * 1e3
    for st in (s_in, s_c, s_out):
        cur.wait_stream(st)
    barrier()

    def alone(fn, n=5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        barrier()
        return a.elapsed_time(b) / n
    account = {"host_enqueue_ms_per_step": host_enqueue_ms, "h2d_alone_ms": alone(lambda: upload(0)),
               "d2h_alone_ms": alone(lambda: out_host[0].copy_(outs[0][rows], non_blocking=True))}
    gather_ms = 0.0
    if world > 1 and ce is None:   # the all-gather alone, for the record
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(5):
            gather(0)
        g1.record()
        barrier()
        gather_ms = g0.elapsed_time(g1) / 5
    return piped_ms, serial_ms, gather_ms, gather_kind, account


# (model, split, ranks) -> is the reduce inside the kernel faster than NCCL after it? Measured on B200 at
# T=16384 (expert-parallel Qwen-like layer, us per layer in-kernel / NCCL): 2 ranks 597-602 / 625-632, 4 ranks
# 491-496 / 513-516, 8 ranks 402-420 / 514. A split that is not listed takes the in-kernel reduce.
FUSED_REDUCE_WINS = {("qwen", "ep", 2): True, ("qwen", "ep", 4): True, ("qwen", "ep", 8): True}
# ranks -> (chunks, communication CTAs) of the in-kernel reduce at T = 16384 (half the chunks at smaller T)
REDUCE_SHAPES = {2: (2, 32), 4: (4, 16), 8: (4, 32)}   # 8 ranks: 4 chunks 402 us, 8 chunks 416, 16 chunks 459


def sweep_reduce_shapes(spec_text, plan, T, launch, batch, barrier, dist, dev, mk, sc, rank) -> None:
    """Times the fused launch for several (chunks, communication CTAs) shapes of the in-kernel reduce:
    10 launches each after 3 warm-ups, max over ranks, printed on stderr."""
    keep = (plan.chunks_by_tokens.get(T), plan.ncomm)
    for item in spec_text.split(","):
        c, n = (int(x) for x in item.split(":"))
        plan.chunks_by_tokens[T], plan.ncomm = c, n
        for _ in range(3):
            launch(batch["hs"], batch["logits"])
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            launch(batch["hs"], batch["logits"])
        e1.record()
        barrier()
        mk.check_status(sc["workspace"])
        t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ph = mk.workspace_view(sc["workspace"])["phase_ns"].tolist()
        if rank == 0:
            print(f"# reduce shape chunks={c} ncomm={n}: {float(t[0]) * 1e3:.1f} us per layer, phases "
                  f"{[round((ph[i + 1] - ph[i]) / 1e3, 1) for i in range(4)]}", file=sys.stderr, flush=True)
    plan.chunks_by_tokens[T], plan.ncomm = keep


def uniform_status(mk, workspace, world, dist, dev):
    """The kernel's status word of this rank's last launch, agreed over the ranks: None when every rank's launch
    ended cleanly, else a reason (this rank's own, or that another rank reported one). Never raises, so that
    every rank takes the same branch after it."""
    why = None
    try:
        mk.check_status(workspace)
    except RuntimeError as e:
        why = str(e)
    if world > 1:
        flag = torch.tensor([0 if why is None else 1], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()) and why is None:
            why = "device status of another rank"
    return why


def time_other_split(model, world, rank, dist, dev, barrier, T, steps=10) -> dict:
    """One more configuration timed in the same process after the contract's own: the tensor-parallel split of
    the Qwen-like layer (4 GPUs) or of the DeepSeek-V3-like layer (8 GPUs), reduce inside the kernel, behind the
    same parity check as the main run. Returns microseconds per layer (max over ranks) and the check's verdict."""
    spec = synth.QWEN if model == "qwen" else synth.DEEPSEEK
    variant = f"{'qwen' if model == 'qwen' else 'ds'}_tp{world}"
    n = spec.inter // world
    kw = {"inter_slice": (rank * n, (rank + 1) * n), "chunk": 8}
    mk = MonoKernel(variant_path(variant))
    layer = synth.make_layer(spec, seed=0, device=dev, with_shared=False, **kw)
    batch = synth.make_batch(spec, layer, T, seed=0, device=dev)
    sc = mk.scratch(T, dev)
    plan = tp_fused.FusedTPPlan(mk, dist.group.WORLD, hidden=spec.hidden, max_tokens=T, nslots=2)
    if not plan.usable:
        return {"variant": variant, "unavailable": plan.reason}
    if plan.chunks_for(T) == 0:
        plan.chunks_by_tokens[T] = 8 if T >= 16384 else 4

    def go():
        plan.fused_tp_launch(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"],
                             layer["w2_scale"], spec.top_k, True, layer["bias"])
    for _ in range(3):
        go()
    barrier()
    why = uniform_status(mk, sc["workspace"], world, dist, dev)
    if why is not None:
        return {"variant": variant, "tokens": T, "failed": why}
    parity = verify_reduced_output(spec, mk, layer, batch, None, sc, plan, plan.pool.output(T), world, rank, dist, dev,
                                   f"tp{world}", kw, fused=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        go()
    e1.record()
    barrier()
    why = uniform_status(mk, sc["workspace"], world, dist, dev)
    if why is not None:
        return {"variant": variant, "tokens": T, "failed": why}
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    return {"variant": variant, "tokens": T, "us_per_layer": ms * 1e3,
            "tflops": synth.routed_flops(spec, T) / (ms * 1e-3) / 1e12, "reduce": "in-kernel NVLS multimem all-reduce",
            "parity_checked": bool(parity["ok"]), "parity": parity}


def time_with_shared_expert(spec, mk, layer, batch, out, sc, steps, dev, routed_flops) -> dict:
    """Beside the contract's figure (routed experts only): the same launch with the layer's sigmoid-gated
    shared expert computed inside it (I_sh = 512: +12.5 % FLOPs)."""
    from unimonomoe_b200.loader import prepare_shared_expert
    full = synth.make_layer(spec, seed=0, device="cpu", with_shared=True, expert_slice=(0, 8))["shared"]
    sh = prepare_shared_expert(*(full[k].to(dev) for k in ("w13", "w13_scale", "w2", "w2_scale")), full["gate"].to(dev))

    def go():
        mk.prefill_impl(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"],
                        spec.top_k, True, layer["bias"], out, scratch=sc, shared=sh)
    for _ in range(3):
        go()
    torch.cuda.synchronize()
    mk.check_status(sc["workspace"])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        go()
    e1.record()
    torch.cuda.synchronize()
    mk.check_status(sc["workspace"])
    ms = e0.elapsed_time(e1) / steps
    T = batch["hs"].shape[0]
    fl = routed_flops + 6.0 * T * spec.hidden * spec.shared_inter
    return {"us_per_layer": ms * 1e3, "tflops_routed_plus_shared": fl / (ms * 1e-3) / 1e12, "flops": fl}


def run_sustained(seconds, ms_guess, launch, reduce_out, batch, barrier, world, dist, dev, gpu_index, flops) -> dict:
    """The same launch repeated for `seconds`: the steady-state figure under the power cap, with the clocks
    seen. Nothing here touches a clock; time x median SM MHz is the clock-normalised cost."""
    n = max(20, int(seconds * 1e3 / max(ms_guess, 1e-3)))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(gpu_index) as clk:
        barrier()
        e0.record()
        for _ in range(n):
            launch(batch["hs"], batch["logits"])
            reduce_out()
        e1.record()
        barrier()
    t = torch.tensor([e0.elapsed_time(e1) / n], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    c = clk.summary()
    return {"steps": n, "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "sm_mhz_median": c["sm_mhz"],
            "reasons": c["reasons"], "clock_samples": c["samples"],
            "us_times_ghz": (ms * 1e3 * c["sm_mhz"] / 1e3) if c["sm_mhz"] else None}


def _bf16_order_key(t):
    b = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    return torch.where(b >= 0x8000, 0x8000 - b, b)


def verify_reduced_output(spec, mk, layer, batch, emap, sc, pool_plan, result, world, rank, dist, dev, par, shard_kw,
                          fused) -> dict:
    """Before anything is timed on N > 1 GPUs: the reduced output of the configuration that is about to be
    timed (`result`, left there by the warm-up steps) must
      * when the reduce ran inside the kernel: equal, bit for bit, an ordinary launch followed by torch's multimem
        all-reduce (the same in-switch reduction) or, with two ranks, by the correctly rounded fp32 sum of the
        two copies (what the peer-load reduce forms),
      * agree with an ordinary launch + NCCL all-reduce (ulp statistics reported, the largest difference
        bounded against the output's rms: NCCL may sum in another order and round between hops),
      * match the CPU oracle on sampled tokens within the layer's tolerance (rank 0 evaluates every rank's shard).
    Every rank returns the same verdict."""
    T, H = batch["hs"].shape[0], spec.hidden
    got = result.clone()
    info = {}
    plain = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    mk.prefill_impl(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"],
                    spec.top_k, True, layer["bias"], plain, expert_map=emap, scratch=sc, check=True)
    ok = True
    if pool_plan is not None:
        view = pool_plan.pool.output(T, 1)
        view.copy_(plain)
        if world == tp_fused.PEER_REDUCE_WORLD:
            # two ranks: the kernel reads the peer's copy directly and forms the correctly rounded fp32 sum
            # (the in-switch reduction rounds ties differently)
            parts = [torch.empty_like(plain) for _ in range(world)]
            dist.all_gather(parts, plain)
            view.copy_((parts[0].float() + parts[1].float()).to(torch.bfloat16))
            key = "bitwise_equal_to_kernel_plus_correctly_rounded_sum"
        else:
            torch.ops.symm_mem.multimem_all_reduce_(view, "sum", dist.group.WORLD.group_name)
            key = "bitwise_equal_to_kernel_plus_multimem_all_reduce"
        torch.cuda.synchronize()
        info[key] = bool(torch.equal(got.view(torch.int16), view.view(torch.int16)))
        if fused:
            ok = ok and info[key]
    dist.all_reduce(plain)
    d = (_bf16_order_key(got) - _bf16_order_key(plain)).abs()
    rms = float(plain.float().pow(2).mean().sqrt())
    max_abs = float((got.float() - plain.float()).abs().max())
    # NCCL may sum in another order and round between hops: within 2e-2 rms, or, where bf16 values are further
    # apart than that, within one bf16 step per rank
    pf = plain.float()
    step = torch.exp2(torch.floor(torch.log2(pf.abs().clamp(min=2.0 ** -126))) - 7.0)
    close = bool(((got.float() - pf).abs() <= torch.maximum(step * (world * 1.0001), torch.full_like(pf, 2e-2 * rms))).all())
    info["vs_kernel_plus_nccl"] = {"moved": int((d > 0).sum()), "over_1_ulp": int((d > 1).sum()), "max_ulp": int(d.max()),
                                   "max_abs_over_rms": max_abs / max(rms, 1e-30), "within_bound": close}
    ok = ok and close
    if rank == 0:
        import numpy as np
        from oracle import cpu_oracle as O
        n_tok = 64 if H <= 2048 else 8
        toks = np.sort(np.random.RandomState(7).choice(T, n_tok, replace=False)).astype(np.int32)
        ids, w, _ = O.route(batch["logits"], mode=spec.router_mode, bias=layer["bias"])
        q, s = O.quant_act(batch["hs"])
        tot = torch.zeros(n_tok, H)
        n_e = spec.experts // world
        for rr in range(world):
            if par.startswith("ep"):
                kw_r = {"expert_slice": (rr * n_e, (rr + 1) * n_e)}
                ids_r = np.where((ids >= rr * n_e) & (ids < (rr + 1) * n_e), ids - rr * n_e, -1).astype(np.int32)
            else:
                n_i = spec.inter // world
                kw_r = {"inter_slice": (rr * n_i, (rr + 1) * n_i)}
                ids_r = ids
            sh = layer if rr == rank else synth.make_layer(spec, seed=0, device=dev, with_shared=False,
                                                           chunk=shard_kw.get("chunk", 16), **kw_r)
            tot += O.moe_path(toks, q, s, ids_r, w, sh["w13"], sh["w13_scale"], sh["w2"], sh["w2_scale"]).float()
            del sh
        mine = got.float().cpu()[torch.from_numpy(toks).long()]
        m = O.parity_metrics(mine, tot)
        # every element within 2e-2 rms, or (the output is bf16: above 3 rms one bf16 step is wider than that)
        # within one bf16 step per rank's rounding plus the final one
        err = (mine - tot).abs()
        beyond = err > 2e-2 * m["rms_ref"]
        step = torch.exp2(torch.floor(torch.log2(tot.abs().clamp(min=2.0 ** -126))) - 7.0)
        within_steps = bool((err[beyond] <= step[beyond] * (world + 1) * 1.0001).all())
        info["oracle"] = {"tokens": n_tok, **m, "beyond_2e-2_rms": int(beyond.sum()), "those_within_bf16_steps": within_steps}
        ok = ok and m["cos"] >= 0.9995 and within_steps and int(beyond.sum()) <= max(1, tot.numel() * (world + 1) // 10000)
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    info["ok"] = bool(flag.item() == 1.0)
    return info


def report(args, spec, T, world, par, variant, value, ms_per_step, kern_ms, flops, e2e_ms, h2d, d2h, clk, dev,
           reduce_desc, phases=None, sustained=None, parity=None, with_shared=None, extra=None,
           reduce_fallback=None, e2e_router_inside=None) -> None:
    peaks = measured_peaks()
    fp8_lib = fp8_gemm_tflops(dev) if (world == 1 and not args.kernel_only) else None
    if peaks.get("bf16_tflops"):
        peak, peak_src = 2.0 * float(peaks["bf16_tflops"]), "2 x bf16_tflops (burst) of MEASURED_PEAKS.json: no fp8 figure is measured there"
    else:
        peak, peak_src = 2.0 * 1590.0, "2 x 1590 TFLOP/s bf16 fallback"
    achieved = (flops / world) / (kern_ms * 1e-3) / 1e12
    traffic = None
    tp = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tp):
        try:
            traffic = json.load(open(tp)).get(f"{variant}_T{T}")
        except Exception:
            traffic = None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{spec.name} MoE layer prefill, T={T} tokens, H={spec.hidden}, E=256, top-8, "
                               f"I={spec.inter}, block-FP8 [128,128] weights", "tokens": T, "parallelism": par, "variant": variant,
                   "l2_policy": (f"inputs larger than L2: {3 * 256 * spec.hidden * spec.inter / world / 1e6:.0f} MB of "
                                 f"weights per rank + the partial rows stream every step"),
                   "reduce": reduce_desc,
                   "router": ("bf16 router linear inside the launch (its 2*T*H*E FLOPs are not counted)"
                              if args.router == "gemv" else "fp32 logits supplied by the caller")},
        "clocks": clk.summary(),
        "e2e": (None if e2e_ms is None else
                {"value": flops / (e2e_ms[0] * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms[0],
                 "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                 "schedule": "steps software-pipelined over three streams (upload | kernel | download), two input "
                             "slots; every step copies its own inputs and result"
                             + ("" if world == 1 else f"; each rank moves 1/{world} of the rows over PCIe and an "
                                "all-gather over NVLink completes the inputs on every GPU"),
                 "serial_ms_per_step": e2e_ms[1], "serial_value": flops / (e2e_ms[1] * 1e-3) / 1e12,
                 "allgather_ms": e2e_ms[2], "allgather": e2e_ms[3], "account": e2e_ms[4]}),
        "gpu_launches": args.steps,
        "kernel_ms": kern_ms,
        # the last launch on rank 0, from the kernel's own %globaltimer stamps: routing + quantisation,
        # scan + scatter, expert pipeline, slot sum (+ in-kernel reduce)
        "phases_us": phases,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                     "traffic": traffic, "peak_source": peak_src, "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                     "library_fp8_gemm_tflops": fp8_lib},
    }
    if sustained is not None:
        sus_peak = 2.0 * float(peaks.get("bf16_tflops_sustained") or 1400.0)
        sustained["frac_of_2x_bf16_sustained"] = (flops / world) / (sustained["ms_per_step"] * 1e-3) / 1e12 / sus_peak
        sustained["peak_2x_bf16_sustained"] = sus_peak
        line["sustained"] = sustained
    if with_shared is not None:
        line["with_shared_expert"] = with_shared
    if extra is not None:
        line["extra"] = extra
    if e2e_router_inside is not None and line["e2e"] is not None:
        line["e2e"]["router_inside"] = e2e_router_inside
    if world > 1:
        line["parity_checked"] = bool(parity is not None and parity["ok"])
        if reduce_fallback is not None:
            line["reduce_fallback"] = reduce_fallback
        line["parity"] = parity
    if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
        line["cpu_baseline"] = time_cpu_baseline(spec, REFERENCE_SAMPLE_TOKENS)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
