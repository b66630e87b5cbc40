"""Host logic of the fused tensor-parallel plan on CPU: chunk-table / ncomm overrides and the
rank-uniform vote over two gloo ranks (a rank that cannot run fused vetoes it for everyone)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from unimonomoe_b200 import tp_fused


def test_chunk_table_and_ncomm_overrides(monkeypatch):
    monkeypatch.delenv("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS", raising=False)
    monkeypatch.delenv("VLLM_PREFILL_MONOKERNEL_TP_NCOMM", raising=False)
    assert tp_fused.env_chunk_table(tp_fused.FUSED_CHUNKS_BY_TOKENS) == {8192: 4, 16384: 8}
    assert tp_fused.env_ncomm(14) == 14
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS", "2")
    assert tp_fused.env_chunk_table(tp_fused.FUSED_CHUNKS_BY_TOKENS) == {8192: 2, 16384: 2}
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS", "4096:2,8192:8")
    assert tp_fused.env_chunk_table(tp_fused.FUSED_CHUNKS_BY_TOKENS) == {4096: 2, 8192: 8}
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS", "8192:0")
    with pytest.raises(ValueError):
        tp_fused.env_chunk_table(tp_fused.FUSED_CHUNKS_BY_TOKENS)
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_NCOMM", "20")
    assert tp_fused.env_ncomm(14) == 20
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_NCOMM", "0")
    with pytest.raises(ValueError):
        tp_fused.env_ncomm(14)
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_NCOMM", "20")
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS", "4096:2,8192:8,16384:8")
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_TP_FOLD_SHARED", "0")
    pol = tp_fused.ReducePolicy.from_env(max_tokens=8192)
    assert dict(pol.chunks_by_tokens) == {4096: 2, 8192: 8} and pol.ncomm == 20 and pol.fold is False
    assert pol.chunks_for(8192) == 8 and pol.chunks_for(1000) == 0 and pol.max_chunks == 8


def test_local_capability_names_the_first_missing_requirement():
    pol = tp_fused.ReducePolicy()
    assert tp_fused.probe_capability(None, pol, enabled=False) == (False, False, "the in-kernel reduce is switched off")

    class FakeKernel:
        def __init__(self, **caps):
            self.caps = dict(usable=True, tp_has_devseq=1, tp_max_c=16, grid_size=148, has_tp_residual=True)
            self.caps.update(caps)

        def tp_caps(self):
            return dict(self.caps)

    if not torch.cuda.is_available():
        assert "CUDA" in tp_fused.probe_capability(FakeKernel(), pol).why
        return
    assert tp_fused.probe_capability(FakeKernel(), pol) == (True, True, "")
    assert "chunks" in tp_fused.probe_capability(FakeKernel(tp_max_c=4), pol).why
    assert "launch counter" in tp_fused.probe_capability(FakeKernel(tp_has_devseq=0), pol).why
    assert tp_fused.probe_capability(FakeKernel(has_tp_residual=False), pol) == (True, False, "")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, answers, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = []
    for case in answers:
        ok, fold = case[rank]

        def cap(plan, ok=ok, fold=fold):
            return tp_fused.Capability(ok, fold, "" if ok else f"rank {rank} cannot")

        plan = tp_fused.FusedTPPlan(None, dist.group.WORLD, hidden=2048, max_tokens=16384, capability=cap,
                                    build_pool=False)
        out.append((plan.usable, plan.fold_shared, plan.reason, plan.chunks_for(8192), plan.chunks_for(1000),
                    plan.rank, plan.world))
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def test_vote_is_rank_uniform_over_two_gloo_ranks():
    # per case: (rank 0 answer, rank 1 answer), each (can run fused, can fold the residual)
    cases = [((True, True), (True, True)), ((True, True), (False, True)), ((True, True), (True, False))]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, cases, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(2):
        all_yes, one_no, no_fold = res[r]
        assert all_yes[0] is True and all_yes[1] is True and all_yes[3] == 4 and all_yes[4] == 0
        assert all_yes[5] == r and all_yes[6] == 2
        assert one_no[0] is False            # one rank's "no" disables the fused path on BOTH ranks
        assert no_fold[0] is True and no_fold[1] is False   # fused, but nobody folds the residual
    assert "cannot" in res[1][1][2] and "peer" in res[0][1][2]


def test_plan_without_process_group_is_unusable():
    plan = tp_fused.FusedTPPlan(None, None, hidden=2048, max_tokens=16384)
    assert not plan.usable and "not initialized" in plan.reason
    assert plan.fused_tp_launch(torch.zeros(8192, 2048), None, None, None, None, None) is None
