"""Multi-GPU gates of the all-reduce that runs inside the prefill kernel, for tensor-parallel AND
expert-parallel ranks. The predicates follow the reference's validation/tp8_fuse_ab.py,
tp8_fold_gate.py and tp8_soak.py; the expert-parallel arm has no counterpart there (the reference
leaves that reduce to the caller). Launch with torchrun, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 tests/multi_gpu_gates.py --parallel ep --tokens 8192,16384 --ncomm 14,32 --skew 1.0

Gates per (token count, ncomm); every rank must agree:
  g1  the fused entry with ncomm = 0 is bitwise the ordinary kernel                 (tp8_fuse_ab.py:314-323)
  g2  reduce inside the kernel == ordinary kernel + multimem all-reduce, bitwise     (tp8_fuse_ab.py:391-405)
      (two ranks: == the correctly rounded fp32 sum of the two copies, which is what the peer-load reduce forms)
  g3  NCCL all-reduce against the multimem all-reduce, in bf16 ulps (reported)       (tp8_fuse_ab.py:119-124)
  g4  fold: scale 0 returns the reduced residual; 2.5 * routed + residual bitwise == the same fold by the
      ordinary kernel + multimem all-reduce                                          (tp8_fold_gate.py:332-409)
  g5  back-to-back launches without a host synchronisation                           (tp8_soak.py:306-318)
  g6  a sentinel behind T*H in the pool slot is untouched                            (tp8_soak.py:511-536)
  g7  the reduced output against the CPU oracle on 256 sampled tokens (rank 0)       (ep4_acc.py:338-391)
  g8  a captured launch replayed three times                                         (tp8_soak.py:351-402)
Soak (--soak N, off by default), all bitwise against the per-size reference:
  s1  N launches with (tokens, chunks, ncomm) drawn from a seeded generator          (tp8_soak.py:277-303)
  s3  each rank in turn is made late by a few milliseconds of matmuls on its stream  (tp8_soak.py:320-339)
  s7  descending, ascending and alternating sizes through one pool slot              (tp8_soak.py:487-539)
  s8  64 launches leave allocated bytes, reserved bytes and the allocation count unchanged and the pool's
      addresses where they were                                                      (tp8_soak.py:541-583)
  s9  both slots are usable, also alternately; a rank on a different slot than its peers gets a wrong
      result (and no hang), after which both slots still work                        (tp8_soak.py:585-646)
Every device-side wait is bounded, NVLS stays enabled, and no rank is ever killed here.
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from unimonomoe_b200 import MonoKernel, synth, tp_fused, variant_path  # noqa: E402


def bf16_order_key(t: torch.Tensor) -> torch.Tensor:
    """bf16 bit patterns mapped to integers that order like the values (-0 and +0 coincide)."""
    b = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    return torch.where(b >= 0x8000, 0x8000 - b, b)


def ulpstats(a: torch.Tensor, b: torch.Tensor) -> dict:
    d = (bf16_order_key(a) - bf16_order_key(b)).abs()
    return {"moved": int((d > 0).sum()), "max_ulp": int(d.max()), "over_1": int((d > 1).sum()),
            "max_abs": float((a.float() - b.float()).abs().max())}


def same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    return bool(torch.equal(a.contiguous().view(torch.int16), b.contiguous().view(torch.int16)))


class Rig:
    """One rank's kernel, shard, plan and launch helpers."""

    def __init__(self, args):
        dist.init_process_group("nccl")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        local = int(os.environ.get("LOCAL_RANK", self.rank))
        torch.cuda.set_device(local)
        self.dev = torch.device("cuda", local)
        self.gname = dist.group.WORLD.group_name
        self.spec = synth.QWEN if args.model == "qwen" else synth.DEEPSEEK
        fam = "qwen" if args.model == "qwen" else "ds"
        self.parallel = args.parallel
        self.variant = f"{fam}_{args.parallel}{self.world}"
        self.mk = MonoKernel(variant_path(self.variant))
        self.mk.set_wait_timeout_us(5_000_000)
        if args.parallel == "tp":
            n = self.spec.inter // self.world
            self.shard_kw = lambda r: {"inter_slice": (r * n, (r + 1) * n)}
            self.emap = None
        else:
            n = self.spec.experts // self.world
            self.shard_kw = lambda r: {"expert_slice": (r * n, (r + 1) * n)}
            self.emap = synth.expert_map(self.spec, self.rank, self.world, device=self.dev)
        self.layer = synth.make_layer(self.spec, seed=0, device=self.dev, with_shared=False, chunk=8,
                                      **self.shard_kw(self.rank))
        self.plan = tp_fused.FusedTPPlan(self.mk, dist.group.WORLD, hidden=self.spec.hidden, max_tokens=args.max_tokens,
                                         nslots=2)
        assert self.plan.usable, self.plan.reason
        self.skew = args.skew
        self._batches = {}

    def batch(self, T):
        if T not in self._batches:
            self._batches[T] = synth.make_batch(self.spec, self.layer, T, seed=0, device=self.dev, skew=self.skew)
        return self._batches[T]

    def weights(self):
        L = self.layer
        return L["w13"], L["w13_scale"], L["w2"], L["w2_scale"]

    def raw(self, T, out, residual=None, scale=1.0):
        """The kernel without any collective (ncomm = 0), optionally folding scale * routed + residual,
        through the one C entry point that takes every option."""
        b, L, sc = self.batch(T), self.layer, self.mk.scratch(T, self.dev)
        vp = ctypes.c_void_p
        entry = self.mk.lib.launch_prefill_moe_wgmma_q1_ep2
        entry.restype = ctypes.c_int
        rc = entry(vp(b["logits"].data_ptr()), T, 128, vp(sc["workspace"].data_ptr()),
                   ctypes.c_size_t(sc["workspace"].numel()), vp(b["hs"].data_ptr()), vp(sc["act_fp8"].data_ptr()),
                   vp(sc["act_scales"].data_ptr()), vp(L["w13"].data_ptr()), vp(L["w13_scale"].data_ptr()),
                   vp(L["w2"].data_ptr()), vp(L["w2_scale"].data_ptr()), vp(sc["partial"].data_ptr()),
                   vp(sc["topk_ids"].data_ptr()), vp(sc["topk_weights"].data_ptr()), vp(sc["sorted_ids"].data_ptr()),
                   vp(out.data_ptr()), vp(0 if L["bias"] is None else L["bias"].data_ptr()), vp(0), vp(0),
                   0, 1, 1, 0, ctypes.c_uint(0), vp(0), vp(0 if residual is None else residual.data_ptr()),
                   ctypes.c_float(scale), vp(0 if self.emap is None else self.emap.data_ptr()),
                   vp(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, rc
        self.mk.check_status(sc["workspace"])

    def plain(self, T, out):
        b = self.batch(T)
        self.mk.prefill_out(b["hs"], b["logits"], *self.weights(), out, 8, True, self.layer["bias"], check=True,
                            expert_map=self.emap)

    def fused(self, T, C, ncomm, slot=0, residual=None, scale=1.0, check=False):
        b = self.batch(T)
        self.plan.chunks_by_tokens[T] = C
        self.plan.ncomm = ncomm
        out = self.plan.fused_tp_launch(b["hs"], b["logits"], *self.weights(), 8, True, self.layer["bias"],
                                        residual=residual, out_scale=scale, slot=slot, check=check, expert_map=self.emap)
        assert out is not None and self.plan.output_is_fused(out)
        return out

    def status(self, T):
        self.mk.check_status(self.mk.scratch(T, self.dev)["workspace"])

    def all_reduce_like_the_kernel(self, view):
        """The all-reduce the in-kernel reduce must reproduce bit for bit, applied in place to a pool view.
        More than two ranks: torch's multimem all-reduce (the same in-switch reduction). Two ranks: the kernel
        reads the peer's copy directly and adds in fp32 with one round-to-nearest-even, which for two summands is
        THE correctly rounded sum -- computed here from the gathered copies (the switch rounds ties differently:
        its result and NCCL's differ in the last bit of about every sixth element)."""
        if self.world == tp_fused.PEER_REDUCE_WORLD:
            parts = [torch.empty_like(view) for _ in range(self.world)]
            dist.all_gather(parts, view.contiguous())
            view.copy_((parts[0].float() + parts[1].float()).to(torch.bfloat16))
        else:
            torch.ops.symm_mem.multimem_all_reduce_(view, "sum", self.gname)
        torch.cuda.synchronize()

    def reference(self, T, slot=0):
        """Ordinary kernel into the pool view, then the all-reduce: what the fused launch must equal."""
        view = self.plan.pool.output(T, slot)
        self.raw(T, view)
        self.all_reduce_like_the_kernel(view)
        return view.clone()

    def all_agree(self, ok: bool) -> bool:
        t = torch.tensor([1.0 if ok else 0.0], device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() == 1.0)


def default_chunks(T):
    return 8 if T >= 16384 else 4


def valid(T, H, C, nc, caps):
    return C <= caps["tp_max_c"] and nc < caps["grid_size"] and (T * H) % (8 * C) == 0


def gates_for(rig: Rig, T: int, ncomm: int) -> dict:
    spec, dev, plan = rig.spec, rig.dev, rig.plan
    C = default_chunks(T)
    r = {}
    pool_view = plan.pool.output(T)
    tail = plan.pool.slot_buffer(0)[T * spec.hidden:]
    if tail.numel():
        tail.fill_(-7.0)
    # g1
    out_plain = torch.empty(T, spec.hidden, dtype=torch.bfloat16, device=dev)
    rig.plain(T, out_plain)
    rig.raw(T, pool_view)
    r["g1_ncomm0_inert"] = same_bits(out_plain, pool_view)
    # references
    multimem = pool_view.clone()
    rig.all_reduce_like_the_kernel(pool_view)
    ref = pool_view.clone()
    nccl = out_plain.clone()
    dist.all_reduce(nccl)
    symm_view = plan.pool.output(T, 1)
    symm_view.copy_(multimem)
    torch.ops.symm_mem.multimem_all_reduce_(symm_view, "sum", rig.gname)
    torch.cuda.synchronize()
    r["g3_nccl_vs_multimem"] = ulpstats(nccl, symm_view)
    r["g3_reference_vs_nccl"] = ulpstats(ref, nccl)
    # g2
    pool_view.zero_()
    got = rig.fused(T, C, ncomm, check=True)
    torch.cuda.synchronize()
    r["g2_fused_bitwise"] = same_bits(got, ref)
    r["g2_max_abs_diff"] = float((got.float() - ref.float()).abs().max())
    # g5
    ok = True
    for _ in range(3):
        rig.fused(T, C, ncomm)
        rig.fused(T, C, ncomm)
        torch.cuda.synchronize()
        ok = ok and same_bits(pool_view, ref)
    rig.status(T)
    r["g5_back_to_back"] = ok
    # g8: warm up on a side stream, capture, replay; the device-side launch counter advances on every replay
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rig.fused(T, C, ncomm)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        rig.fused(T, C, ncomm)
    ok = True
    for _ in range(3):
        pool_view.zero_()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        ok = ok and same_bits(pool_view, ref)
    rig.status(T)
    del graph
    r["g8_graph_replay"] = ok
    # g6
    r["g6_tail_untouched"] = bool((tail == -7.0).all()) if tail.numel() else True
    # g4
    if plan.fold_shared:
        gen = torch.Generator(device=dev).manual_seed(4242 + T)
        resid = (torch.randn(T, spec.hidden, device=dev, generator=gen) * 0.05).to(torch.bfloat16)
        got0 = rig.fused(T, C, ncomm, residual=resid, scale=0.0, check=True).clone()
        pool_view.copy_(resid)
        rig.all_reduce_like_the_kernel(pool_view)
        r["g4_scale0_is_reduced_residual"] = same_bits(got0, pool_view)
        rig.raw(T, pool_view, resid, 2.5)
        rig.all_reduce_like_the_kernel(pool_view)
        ref_fold = pool_view.clone()
        gotf = rig.fused(T, C, ncomm, residual=resid, scale=2.5, check=True)
        torch.cuda.synchronize()
        r["g4_fold_bitwise"] = same_bits(gotf, ref_fold)
    # g7: rank 0 evaluates the whole layer (every rank's shard) on the CPU for sampled tokens
    if rig.rank == 0:
        from oracle import cpu_oracle as O
        b = rig.batch(T)
        n_tok = 256 if spec.hidden <= 2048 else 32
        toks = np.sort(np.random.RandomState(1).choice(T, n_tok, replace=False)).astype(np.int32)
        ids, w, _ = O.route(b["logits"], mode=spec.router_mode, bias=rig.layer["bias"])
        q, s = O.quant_act(b["hs"])
        tot = torch.zeros(len(toks), spec.hidden)
        n_e = spec.experts // rig.world
        for rr in range(rig.world):
            sh = rig.layer if rr == rig.rank else synth.make_layer(spec, seed=0, device=dev, with_shared=False, chunk=8,
                                                                   **rig.shard_kw(rr))
            if rig.parallel == "tp":
                ids_r = ids
            else:   # this shard's experts under their local ids, everything else unowned
                ids_r = np.where((ids >= rr * n_e) & (ids < (rr + 1) * n_e), ids - rr * n_e, -1).astype(np.int32)
            tot += O.moe_path(toks, q, s, ids_r, w, sh["w13"], sh["w13_scale"], sh["w2"], sh["w2_scale"]).float()
            del sh
        mine = ref.float().cpu()[torch.from_numpy(toks).long()]
        m = O.parity_metrics(mine, tot)
        # within 2e-2 rms, or -- the output is bf16, and above 3 rms one bf16 step is wider than that -- within
        # one bf16 step per rank's rounding plus the final one; such elements have to be rare (one in 10 000
        # per rounding)
        err = (mine - tot).abs()
        beyond = err > 2e-2 * m["rms_ref"]
        step = torch.exp2(torch.floor(torch.log2(tot.abs().clamp(min=2.0 ** -126))) - 7.0)
        m["beyond_2e-2_rms"] = int(beyond.sum())
        r["g7_oracle"] = m
        r["g7_ok"] = bool(m["cos"] >= 0.9995 and (err[beyond] <= step[beyond] * (rig.world + 1) * 1.0001).all()
                          and m["beyond_2e-2_rms"] <= max(1, tot.numel() * (rig.world + 1) // 10000))
    return r


def soak(rig: Rig, tokens, iters: int) -> dict:
    spec, dev, plan, mk = rig.spec, rig.dev, rig.plan, rig.mk
    caps = mk.tp_caps()
    H = spec.hidden
    refs = {T: rig.reference(T) for T in tokens}
    fails, checks = [], 0

    def check(tag, T, C, nc, extra="", slot=0):
        nonlocal checks
        checks += 1
        ok = rig.all_agree(same_bits(refs[T], plan.pool.output(T, slot)))
        if not ok:
            fails.append(f"{tag} T={T} C={C} ncomm={nc} {extra}")
            if rig.rank == 0:
                print("FAIL", fails[-1], flush=True)
        return ok

    # s1: one seeded generator, identical on every rank
    rs = np.random.RandomState(20240607)
    for _ in range(iters):
        T = int(tokens[rs.randint(len(tokens))])
        C = int((1, 2, 4, 8, 16)[rs.randint(5)])
        nc = int((8, 14, 16, 24, 32, 48)[rs.randint(6)])
        if not valid(T, H, C, nc, caps):
            continue
        plan.pool.output(T).zero_()
        rig.fused(T, C, nc)
        torch.cuda.synchronize()
        check("s1", T, C, nc)
    rig.status(tokens[0])
    # s3: each rank late in turn
    big = torch.randn(4096, 4096, device=dev)
    for T in tokens:
        C = default_chunks(T)
        for late in range(rig.world):
            plan.pool.output(T).zero_()
            if rig.rank == late:
                for _ in range(24):
                    big = (big @ big.t()) * 1e-6
            rig.fused(T, C, 14)
            torch.cuda.synchronize()
            check("s3", T, C, 14, f"late={late}")
    del big
    # s7: size orderings through one slot
    order = sorted(tokens, reverse=True) + sorted(tokens) + [max(tokens), min(tokens), max(tokens), min(tokens)]
    for T in order:
        C = default_chunks(T)
        plan.pool.output(T).zero_()
        rig.fused(T, C, 16)
        torch.cuda.synchronize()
        check("s7", T, C, 16, "alternating sizes")
    # s8: nothing allocates, nothing moves
    T, C, nc = max(tokens), default_chunks(max(tokens)), 16
    plan.pool.assert_stable()
    for _ in range(3):
        rig.fused(T, C, nc)
    torch.cuda.synchronize()

    def mem():
        return (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev),
                torch.cuda.memory_stats(dev)["allocation.all.current"])
    before = mem()
    for _ in range(64):
        rig.fused(T, C, nc)
    torch.cuda.synchronize()
    after = mem()
    plan.pool.assert_stable()
    checks += 1
    if not rig.all_agree(before == after):
        fails.append(f"s8 the launch path allocated: {before} -> {after}")
    check("s8", T, C, nc, "after 64 launches")
    # s9: slots
    T, C, nc = min(tokens), default_chunks(min(tokens)), 14
    for slot in range(plan.pool.nslots):
        plan.pool.output(T, slot).zero_()
        rig.fused(T, C, nc, slot=slot)
        torch.cuda.synchronize()
        check("s9 uniform", T, C, nc, f"slot={slot}", slot=slot)
    for rep in range(4):
        slot = rep % plan.pool.nslots
        plan.pool.output(T, slot).zero_()
        rig.fused(T, C, nc, slot=slot)
        torch.cuda.synchronize()
        check("s9 alternating", T, C, nc, f"slot={slot}", slot=slot)
    if plan.pool.nslots >= 2:
        for slot in range(plan.pool.nslots):
            plan.pool.output(T, slot).zero_()
        rig.fused(T, C, nc, slot=1 if rig.rank == 0 else 0)
        torch.cuda.synchronize()
        matched = same_bits(refs[T], plan.pool.output(T, 0))
        t = torch.tensor([1.0 if matched else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        checks += 1
        if t.item() > 0:
            fails.append("s9 a rank on another slot still produced the reference result")
        rig.status(T)
        for slot in range(plan.pool.nslots):
            plan.pool.output(T, slot).zero_()
            rig.fused(T, C, nc, slot=slot)
            torch.cuda.synchronize()
            check("s9 recover", T, C, nc, f"slot={slot}", slot=slot)
    rig.status(T)
    return {"checks": checks, "fails": fails}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="8192,16384")
    ap.add_argument("--model", default="qwen", choices=["qwen", "deepseek"])
    ap.add_argument("--parallel", default="tp", choices=["tp", "ep"])
    ap.add_argument("--ncomm", default="14")
    ap.add_argument("--skew", type=float, default=0.0, help="per-expert logit offset N(0, skew): ragged expert counts")
    ap.add_argument("--soak", type=int, default=0, help="randomised launches of the soak part (0: skip it)")
    ap.add_argument("--soak-tokens", default="2048,4096,8192")
    ap.add_argument("--out", default=os.path.join(os.environ.get("GATES_OUT_DIR", os.path.join(ROOT, "out")), "multi_gpu_gates.json"))
    args = ap.parse_args()
    Ts = [int(t) for t in args.tokens.split(",") if t]
    soak_Ts = [int(t) for t in args.soak_tokens.split(",") if t] if args.soak else []
    args.max_tokens = max(Ts + soak_Ts)
    rig = Rig(args)
    if rig.rank == 0:
        print(f"{rig.variant}: fold={rig.plan.fold_shared} pool: {rig.plan.pool.describe()}", flush=True)
    results, all_ok = {}, True
    for T in Ts:
        for nc in [int(x) for x in args.ncomm.split(",")]:
            r = gates_for(rig, T, nc)
            ok = all(v for v in r.values() if isinstance(v, bool))
            r["all_ranks_ok"] = rig.all_agree(ok)
            all_ok = all_ok and r["all_ranks_ok"]
            results[f"T{T}_ncomm{nc}"] = r
            if rig.rank == 0:
                print(f"T={T} C={default_chunks(T)} ncomm={nc} skew={args.skew}: {json.dumps(r)}", flush=True)
    if args.soak:
        s = soak(rig, soak_Ts, args.soak)
        results["soak"] = s
        all_ok = all_ok and not s["fails"]
        if rig.rank == 0:
            print(f"soak: {s['checks']} checks, {len(s['fails'])} failures {s['fails'][:5]}", flush=True)
    if rig.rank == 0:
        os.makedirs(os.path.dirname(args.out), exist_ok=True)
        json.dump({"world": rig.world, "variant": rig.variant, "skew": args.skew, "results": results, "ok": all_ok},
                  open(args.out, "w"), indent=1)
        print("MULTI-GPU GATES:", "PASS" if all_ok else "FAIL", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if all_ok else 1)


if __name__ == "__main__":
    main()
