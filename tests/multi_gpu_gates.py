"""Multi-GPU gates of the fused tensor-parallel epilogue, after the reference's
validation/tp8_fuse_ab.py, tp8_fold_gate.py and tp8_soak.py. Launch with torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 tests/multi_gpu_gates.py [--tokens 8192,16384]

Gates, per token count (all ranks must agree):
  1. the fused entry with ncomm = 0 is bitwise the ordinary kernel              (tp8_fuse_ab.py:314-323)
  2. FUSED output bitwise == ordinary kernel + multimem all-reduce              (tp8_fuse_ab.py:391-405)
  3. NCCL all-reduce vs multimem all-reduce compared in bf16 ulps               (tp8_fuse_ab.py:119-124)
  4. fold: scale 0 returns the reduced residual; 2.5*routed+residual bitwise == ordinary kernel
     with the same fold + multimem all-reduce                                    (tp8_fold_gate.py:332-409)
  5. back-to-back fused launches without a host sync, bitwise each time          (tp8_soak.py:306-318)
  6. a sentinel tail behind T*H in the pool slot is untouched                    (tp8_soak.py:511-536)
  8. a captured fused launch replayed three times, bitwise each time            (tp8_soak.py:351-402)
  7. summed output against the CPU oracle on sampled tokens (rank 0)
NVLS stays enabled: this test never kills a rank.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from unimonomoe_b200 import MonoKernel, synth, tp_fused, variant_path  # noqa: E402


def ulpstats(a, b):
    d = (a.view(torch.int16).to(torch.int32) - b.view(torch.int16).to(torch.int32)).abs()
    return {"moved": int((d > 0).sum()), "max_ulp": int(d.max()), "over_1": int((d > 1).sum())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="8192,16384")
    ap.add_argument("--model", default="qwen")
    ap.add_argument("--out", default=os.path.join(os.environ.get("GATES_OUT_DIR", os.path.join(ROOT, "out")), "multi_gpu_gates.json"))
    args = ap.parse_args()
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed._symmetric_memory as symm_mem
    gname = dist.group.WORLD.group_name

    spec = synth.QWEN if args.model == "qwen" else synth.DEEPSEEK
    variant = f"{'qwen' if args.model == 'qwen' else 'ds'}_tp{world}"
    mk = MonoKernel(variant_path(variant))
    mk.set_wait_timeout_us(5_000_000)
    n = spec.inter // world
    layer = synth.make_layer(spec, seed=0, device=dev, inter_slice=(rank * n, (rank + 1) * n), with_shared=False, chunk=8)
    Ts = [int(t) for t in args.tokens.split(",")]
    plan = tp_fused.FusedTPPlan(mk, dist.group.WORLD, hidden=spec.hidden, max_tokens=max(Ts))
    if rank == 0:
        print(f"plan usable={plan.usable} reason={plan.reason!r} fold={plan.fold_shared} ncomm={plan.ncomm} "
              f"chunks={plan.chunks_by_tokens} pool: {plan.pool.describe() if plan.pool else None}", flush=True)
    assert plan.usable, plan.reason
    results, all_ok = {}, True
    for T in Ts:
        batch = synth.make_batch(spec, layer, T, seed=0, device=dev)
        out_pool = plan.pool.output(T)
        slot = plan.pool.slot_buffer(0)
        tail = slot[T * spec.hidden:]
        if tail.numel():
            tail.fill_(-7.0)
        nchunk = plan.chunks_for(T) or 4
        plan.chunks_by_tokens[T] = nchunk
        args_k = (batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"])

        def ordinary(residual=None, scale=1.0):
            # the ordinary kernel writing into the pool view (tp_ncomm = 0), then an external reduce
            if residual is None and scale == 1.0:
                mk.prefill_out(*args_k, out_pool, 8, True, layer["bias"], check=True)
            else:
                # same binary, collective switched off, fold applied (the _tp2 entry with ncomm 0)
                sc = mk.scratch(T, dev)
                import ctypes
                vp = ctypes.c_void_p
                rc = mk.lib.launch_prefill_moe_wgmma_q1_tp2(
                    vp(batch["logits"].data_ptr()), T, 128, vp(sc["workspace"].data_ptr()),
                    ctypes.c_size_t(sc["workspace"].numel()), vp(batch["hs"].data_ptr()), vp(sc["act_fp8"].data_ptr()),
                    vp(sc["act_scales"].data_ptr()), vp(layer["w13"].data_ptr()), vp(layer["w13_scale"].data_ptr()),
                    vp(layer["w2"].data_ptr()), vp(layer["w2_scale"].data_ptr()), vp(sc["partial"].data_ptr()),
                    vp(sc["topk_ids"].data_ptr()), vp(sc["topk_weights"].data_ptr()), vp(sc["sorted_ids"].data_ptr()),
                    vp(out_pool.data_ptr()), vp(0 if layer["bias"] is None else layer["bias"].data_ptr()), vp(0), vp(0),
                    0, 1, 1, 0, ctypes.c_uint(0), vp(0), vp(0 if residual is None else residual.data_ptr()),
                    ctypes.c_float(scale), vp(torch.cuda.current_stream().cuda_stream))
                assert rc == 0
                mk.check_status(sc["workspace"])

        r = {}
        # gate 1
        out_plain = torch.empty(T, spec.hidden, dtype=torch.bfloat16, device=dev)
        mk.prefill_out(*args_k, out_plain, 8, True, layer["bias"], check=True)
        ordinary()
        r["g1_ncomm0_inert"] = bool(torch.equal(out_plain.view(torch.int16), out_pool.view(torch.int16)))
        # reference reductions
        torch.ops.symm_mem.multimem_all_reduce_(out_pool, "sum", gname)
        torch.cuda.synchronize()
        ref_symm = out_pool.clone()
        nccl = out_plain.clone()
        dist.all_reduce(nccl)
        r["g3_nccl_vs_multimem"] = ulpstats(nccl, ref_symm)
        # gate 2
        out_pool.zero_()
        got = plan.fused_tp_launch(*args_k, 8, True, layer["bias"], check=True)
        assert got is not None and plan.output_is_fused(got)
        torch.cuda.synchronize()
        r["g2_fused_bitwise"] = bool(torch.equal(got.view(torch.int16), ref_symm.view(torch.int16)))
        r["g2_max_abs_diff"] = float((got.float() - ref_symm.float()).abs().max())
        # gate 5: back to back, no host sync in between
        ok5 = True
        for _ in range(3):
            plan.fused_tp_launch(*args_k, 8, True, layer["bias"])
            plan.fused_tp_launch(*args_k, 8, True, layer["bias"])
            torch.cuda.synchronize()
            ok5 = ok5 and bool(torch.equal(out_pool.view(torch.int16), ref_symm.view(torch.int16)))
        mk.check_status(mk.scratch(T, dev)["workspace"])
        r["g5_back_to_back"] = ok5
        # gate 8: a captured fused launch replayed three times; the device sequence counter advances on
        # every replay, so the rank barriers never see a stale sequence (tp8_soak.py:351-402)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            plan.fused_tp_launch(*args_k, 8, True, layer["bias"])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            plan.fused_tp_launch(*args_k, 8, True, layer["bias"])
        ok8 = True
        for _ in range(3):
            out_pool.zero_()
            dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            ok8 = ok8 and bool(torch.equal(out_pool.view(torch.int16), ref_symm.view(torch.int16)))
        mk.check_status(mk.scratch(T, dev)["workspace"])
        r["g8_graph_replay"] = ok8
        # gate 6
        r["g6_tail_untouched"] = bool((tail == -7.0).all()) if tail.numel() else True
        # gate 4: fold
        if plan.fold_shared:
            resid = (torch.randn(T, spec.hidden, device=dev) * 0.05).to(torch.bfloat16)
            got0 = plan.fused_tp_launch(*args_k, 8, True, layer["bias"], residual=resid, out_scale=0.0, check=True).clone()
            tmp = plan.pool.output(T)
            tmp.copy_(resid)
            torch.ops.symm_mem.multimem_all_reduce_(tmp, "sum", gname)
            torch.cuda.synchronize()
            r["g4_scale0_is_reduced_residual"] = bool(torch.equal(got0.view(torch.int16), tmp.view(torch.int16)))
            ordinary(resid, 2.5)
            torch.ops.symm_mem.multimem_all_reduce_(out_pool, "sum", gname)
            torch.cuda.synchronize()
            ref_fold = out_pool.clone()
            gotf = plan.fused_tp_launch(*args_k, 8, True, layer["bias"], residual=resid, out_scale=2.5, check=True)
            torch.cuda.synchronize()
            r["g4_fold_bitwise"] = bool(torch.equal(gotf.view(torch.int16), ref_fold.view(torch.int16)))
        # gate 7: oracle on sampled tokens (rank 0 computes every shard on CPU)
        if rank == 0 and args.model == "qwen" and T <= 16384:
            from oracle import cpu_oracle as O
            toks = np.sort(np.random.RandomState(1).choice(T, 16, replace=False)).astype(np.int32)
            ids, w, _ = O.route(batch["logits"], mode=0)
            q, s = O.quant_act(batch["hs"])
            tot = torch.zeros(len(toks), spec.hidden)
            for rr in range(world):
                sh = synth.make_layer(spec, seed=0, device=dev, inter_slice=(rr * n, (rr + 1) * n), with_shared=False, chunk=8)
                tot += O.moe_path(toks, q, s, ids, w, sh["w13"], sh["w13_scale"], sh["w2"], sh["w2_scale"]).float()
                del sh
            m = O.parity_metrics(ref_symm.float().cpu()[torch.from_numpy(toks).long()], tot)
            r["g7_oracle"] = m
            r["g7_ok"] = bool(m["rel_l2"] < 5e-3 and m["cos"] >= 0.9995)
        flags = [v for k, v in r.items() if isinstance(v, bool)]
        ok = all(flags)
        t = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        r["all_ranks_ok"] = bool(t.item() == 1.0)
        all_ok = all_ok and r["all_ranks_ok"]
        results[T] = r
        if rank == 0:
            print(f"T={T} C={nchunk} ncomm={plan.ncomm}: {json.dumps(r)}", flush=True)
    if rank == 0:
        os.makedirs(os.path.dirname(args.out), exist_ok=True)
        json.dump({"world": world, "variant": variant, "results": results, "ok": all_ok}, open(args.out, "w"), indent=1)
        print("MULTI-GPU GATES:", "PASS" if all_ok else "FAIL", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if all_ok else 1)


if __name__ == "__main__":
    main()
