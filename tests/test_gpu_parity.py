"""Parity of the CUDA kernel with the CPU oracle, through the C-ABI, on a B200.

Bars: expert ids, per-expert counts/offsets and the sort permutation bit-exact; bf16 output
max|err| <= 2e-2 * rms(ref) and cosine >= 0.9995 against the path-faithful oracle."""
import ctypes
import os

import numpy as np
import pytest
import torch

from unimonomoe_b200 import synth

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def gu():
    from tests import gpu_util
    return gpu_util


@pytest.fixture(scope="module")
def qwen_full(built_libs):
    from tests.gpu_util import DEV
    return synth.make_layer(synth.QWEN, seed=0, device=DEV, with_shared=False)


def tp_shard(full, rank, world, I=512):
    lo, hi = rank * I // world, (rank + 1) * I // world
    nb = I // 128
    dev = full["w13"].device
    rows = torch.cat([torch.arange(lo, hi), torch.arange(I + lo, I + hi)]).to(dev)
    srows = torch.cat([torch.arange(lo // 128, hi // 128), torch.arange(nb + lo // 128, nb + hi // 128)]).to(dev)
    return {"w13": full["w13"].view(torch.uint8)[:, rows].contiguous().view(torch.float8_e4m3fn),
            "w13_scale": full["w13_scale"][:, srows].contiguous(),
            "w2": full["w2"].view(torch.uint8)[:, :, lo:hi].contiguous().view(torch.float8_e4m3fn),
            "w2_scale": full["w2_scale"][:, :, lo // 128:hi // 128].contiguous(), "bias": None,
            "router_w": full["router_w"]}


def ep_shard(full, rank, world):
    n = 256 // world
    sl = slice(rank * n, (rank + 1) * n)
    return {k: (full[k][sl].contiguous() if k in ("w13", "w13_scale", "w2", "w2_scale") else full[k]) for k in full}


@pytest.mark.parametrize("T", [1, 7, 256, 1000, 8192, 16384, 30720])   # 30720: the loader's cap
def test_qwen_single_gpu_parity(gu, oracle, qwen_full, T):
    mk = gu.kernel("qwen_w1")
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=0, device=gu.DEV)
    res = gu.launch(mk, qwen_full, batch)
    ids, w, _ = gu.check_routing(oracle, res, batch, 0, None, 256)
    q, s = gu.check_act_quant(oracle, res, batch)
    assert torch.isfinite(res["out"].float()).all()  # NaN-poisoned output fully overwritten
    # every token up to the benchmark size (the oracle is OpenMP C: seconds); 512 sampled tokens beyond it
    gu.check_output(oracle, res["out"], gu.sample_tokens(T, T if T <= 16384 else 512), q, s, ids, w, qwen_full)


@pytest.mark.parametrize("T", [7, 1000, 16384])
def test_two_cta_pair_build_matches(gu, oracle, qwen_full, T):
    """The build that runs pairs of tiles on clusters of two CTAs (tcgen05 cta_group::2, M = 256, each
    CTA loading half of every weight stage) passes the same bit-exact routing checks and produces the same
    output bytes as the one-CTA build: the arithmetic per row is identical, only the schedule differs."""
    mk2 = gu.kernel("qwen_w1_pair")
    assert mk2._int_symbol("cta_pair") == 1
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=5, device=gu.DEV)
    res2 = gu.launch(mk2, qwen_full, batch)
    gu.check_routing(oracle, res2, batch, 0, None, 256, rows_per_unit=256)
    assert torch.isfinite(res2["out"].float()).all()
    res1 = gu.launch(gu.kernel("qwen_w1"), qwen_full, batch)
    assert torch.equal(res1["out"].view(torch.int16), res2["out"].view(torch.int16))


def test_run_to_run_bitwise_and_token_permutation(gu, oracle, qwen_full):
    """Full-size property checks: two launches agree bit for bit, and permuting the tokens
    permutes the output rows bit for bit (a row's arithmetic does not depend on its tile)."""
    mk = gu.kernel("qwen_w1")
    T = 16384
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=1, device=gu.DEV)
    a = gu.launch(mk, qwen_full, batch)
    out_a = a["out"].clone()
    b = gu.launch(mk, qwen_full, batch)
    assert torch.equal(out_a.view(torch.int16), b["out"].view(torch.int16))
    assert (a["sorted"] == b["sorted"]).all()
    srt = np.sort(a["sorted"])
    assert (srt == np.arange(T * 8)).all() and a["counts"].sum() == T * 8
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(5)).to(gu.DEV)
    pb = {"hs": batch["hs"][perm].contiguous(), "logits": batch["logits"][perm].contiguous()}
    c = gu.launch(mk, qwen_full, pb)
    assert torch.equal(c["out"].view(torch.int16), out_a[perm].view(torch.int16))


def test_ragged_and_degenerate_routing(gu, oracle, qwen_full):
    mk = gu.kernel("qwen_w1")
    # skewed logits: ragged per-expert counts
    batch = synth.make_batch(synth.QWEN, qwen_full, 3000, seed=2, device=gu.DEV, skew=1.0)
    res = gu.launch(mk, qwen_full, batch)
    ids, w, _ = gu.check_routing(oracle, res, batch, 0, None, 256)
    q, s = gu.check_act_quant(oracle, res, batch)
    assert res["counts"].max() > 4 * res["counts"].mean()
    gu.check_output(oracle, res["out"], gu.sample_tokens(3000, 32, 1), q, s, ids, w, qwen_full)
    # every token to the same eight experts: 248 empty experts, eight with T rows each
    T = 1100
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=3, device=gu.DEV)
    batch["logits"][:, [3, 40, 77, 100, 129, 200, 254, 255]] += 50.0
    res = gu.launch(mk, qwen_full, batch)
    ids, w, _ = gu.check_routing(oracle, res, batch, 0, None, 256)
    assert (res["counts"] > 0).sum() == 8 and res["total_tiles"] == 8 * 9
    gu.check_output(oracle, res["out"], gu.sample_tokens(T, 24, 2), *gu.check_act_quant(oracle, res, batch), ids, w, qwen_full)
    # all-zero activations and constant logits: scales take the amax -> 1 branch, ties go to low ids
    batch = {"hs": torch.zeros(130, 2048, dtype=torch.bfloat16, device=gu.DEV),
             "logits": torch.zeros(130, 256, device=gu.DEV)}
    res = gu.launch(mk, qwen_full, batch)
    gu.check_routing(oracle, res, batch, 0, None, 256)
    gu.check_act_quant(oracle, res, batch)
    assert (res["ids"] == np.arange(8)[None]).all() and (res["out"].float() == 0).all()


def test_golden_routing_through_the_kernel(gu, oracle, qwen_full, built_libs):
    g = np.load(os.path.join(G, "routing.npz"))
    logits = torch.from_numpy(g["logits"]).to(gu.DEV)
    T = logits.shape[0]
    hs = torch.randn(T, 2048, device=gu.DEV).to(torch.bfloat16)
    res = gu.launch(gu.kernel("qwen_w1"), qwen_full, {"hs": hs, "logits": logits})
    rows = np.setdiff1d(np.arange(T), g["tie_rows"])
    assert (res["ids"][rows] == g["softmax_ids"][rows]).all()
    assert np.allclose(res["weights"][rows], g["softmax_w"][rows], rtol=1e-5, atol=1e-8)
    assert res["ids"][0].tolist() == list(range(8)) and res["ids"][1][:2].tolist() == [10, 200]


def test_tensor_parallel_shards_sum_to_full(gu, oracle, qwen_full):
    """Each TP=4 rank's kernel run in sequence on one GPU (validation/ep4_acc.py:5-9 does the
    same for EP); the partial outputs must add up to the unsharded layer."""
    T = 2048
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=4, device=gu.DEV)
    mk = gu.kernel("qwen_tp4")
    toks = gu.sample_tokens(T, 32, 3)
    total = torch.zeros(T, 2048, device=gu.DEV)
    ref_total = torch.zeros(len(toks), 2048)
    for r in range(4):
        sh = tp_shard(qwen_full, r, 4)
        res = gu.launch(mk, sh, batch)
        ids, w, _ = gu.check_routing(oracle, res, batch, 0, None, 256)
        q, s = gu.check_act_quant(oracle, res, batch)
        gu.check_output(oracle, res["out"], toks, q, s, ids, w, sh)
        total += res["out"].float()
        ref_total += oracle.moe_path(toks, q, s, ids, w, sh["w13"], sh["w13_scale"], sh["w2"], sh["w2_scale"]).float()
    gu.assert_close(oracle, total.cpu()[torch.from_numpy(toks).long()], ref_total, steps=4)
    full = gu.launch(gu.kernel("qwen_w1"), qwen_full, batch)
    m2 = oracle.parity_metrics(total.cpu(), full["out"].float().cpu())
    assert m2["cos"] > 0.999, m2


def test_expert_parallel_ranks_in_sequence(gu, oracle, qwen_full):
    """The reference's EP gates G1-G7 and G9 (validation/ep4_acc.py:338-391) with four ranks run in
    sequence on one GPU."""
    T = 2048
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=5, device=gu.DEV, skew=1.0)
    mk = gu.kernel("qwen_ep4")
    outs, tis, tws = [], [], []
    q = s = None
    for r in range(4):
        emap = synth.expert_map(synth.QWEN, r, 4, device=gu.DEV)
        sh = ep_shard(qwen_full, r, 4)
        res = gu.launch(mk, sh, batch, expert_map=emap)                       # G1: rc == 0, status ok
        ids, w, gids = gu.check_routing(oracle, res, batch, 0, None, 64, expert_map=emap)
        q, s = gu.check_act_quant(oracle, res, batch)
        assert res["ids"].min() >= -1 and res["ids"].max() < 64              # G2
        assert torch.isfinite(res["out"].float()).all()                      # G6: poison fully overwritten
        gu.check_output(oracle, res["out"], gu.sample_tokens(T, 16, r), q, s, ids, w, sh)
        outs.append(res["out"].float()); tis.append(res["ids"]); tws.append(res["weights"])
    owners = sum((t >= 0).astype(np.int32) for t in tis)
    assert (owners == 1).all()                                               # G3
    gti = np.full((T, 8), -1, np.int64)
    for r in range(4):
        gti = np.where(tis[r] >= 0, tis[r] + 64 * r, gti)
    ref_ids = torch.topk(batch["logits"], 8, dim=1).indices.cpu().numpy()
    assert (np.sort(gti, 1) == np.sort(ref_ids, 1)).all()                    # G4
    for r in range(1, 4):
        assert (tws[0].view(np.uint32) == tws[r].view(np.uint32)).all()      # G5
    summed = torch.stack(outs).sum(0)
    full = gu.launch(gu.kernel("qwen_w1"), qwen_full, batch)                 # G9: the full-width control
    assert (np.sort(full["ids"], 1) == np.sort(gti, 1)).all()
    assert (full["weights"].view(np.uint32) == tws[0].view(np.uint32)).all()
    # the four partial outputs are each rounded to bf16 before they are added, the control is rounded
    # once: the two agree to a few bf16 ulps, which is a looser bound than the one against the oracle
    m = oracle.parity_metrics(summed.cpu(), full["out"].float().cpu())
    assert m["rel_l2"] < 5e-3 and m["cos"] >= 0.99999, m
    toks = gu.sample_tokens(T, 24, 9)
    ref = oracle.moe_path(toks, q, s, full["ids"], full["weights"], qwen_full["w13"], qwen_full["w13_scale"],
                          qwen_full["w2"], qwen_full["w2_scale"])
    mp = oracle.parity_metrics(summed.cpu()[torch.from_numpy(toks).long()], ref.float())
    assert mp["rel_l2"] < 5e-3 and mp["cos"] >= gu.MIN_COS, mp  # four bf16 roundings instead of one: no max-abs bound
    # G7, against the fp64 tier
    ref64 = oracle.moe_fp64(batch["hs"].cpu()[torch.from_numpy(toks).long()], full["ids"][toks], full["weights"][toks],
                            qwen_full["w13"].cpu(), qwen_full["w13_scale"].cpu(), qwen_full["w2"].cpu(),
                            qwen_full["w2_scale"].cpu())
    rl2, cs = oracle.rel_cos(summed.cpu()[torch.from_numpy(toks).long()], ref64)
    assert rl2 < 6e-2 and cs > 0.998, (rl2, cs)


def _qwen_ranks_in_sequence(gu, oracle, qwen_full, split, T, skew):
    """All four ranks of a tensor- or expert-parallel split of the Qwen layer, one after the other on one GPU:
    routing bit-exact on every rank, rank 0 compared with the oracle on EVERY token at T = 8192 (256 sampled
    tokens otherwise), and the sum of the four partial outputs compared with the sum of the oracle's."""
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=4, device=gu.DEV, skew=skew)
    mk = gu.kernel(f"qwen_{split}4")
    toks = gu.sample_tokens(T, 256, 3)
    total = torch.zeros(len(toks), 2048)
    ref_total = torch.zeros(len(toks), 2048)
    for r in range(4):
        if split == "tp":
            sh, emap, n_local = tp_shard(qwen_full, r, 4), None, 256
        else:
            sh, emap, n_local = ep_shard(qwen_full, r, 4), synth.expert_map(synth.QWEN, r, 4, device=gu.DEV), 64
        res = gu.launch(mk, sh, batch, expert_map=emap)
        ids, w, _ = gu.check_routing(oracle, res, batch, 0, None, n_local, expert_map=emap)
        q, s = gu.check_act_quant(oracle, res, batch)
        assert torch.isfinite(res["out"].float()).all()
        mine = gu.sample_tokens(T, T, 0) if (r == 0 and T <= 8192) else toks
        gu.check_output(oracle, res["out"], mine, q, s, ids, w, sh)
        total += res["out"].float().cpu()[torch.from_numpy(toks).long()]
        ref_total += oracle.moe_path(toks, q, s, ids, w, sh["w13"], sh["w13_scale"], sh["w2"], sh["w2_scale"]).float()
        del sh
    gu.assert_close(oracle, total, ref_total, steps=4)


@pytest.mark.parametrize("T", [8192, 16384])
def test_tensor_parallel_4_at_prefill_sizes(gu, oracle, qwen_full, T):
    _qwen_ranks_in_sequence(gu, oracle, qwen_full, "tp", T, skew=0.0)


@pytest.mark.parametrize("T", [8192, 16384])
def test_expert_parallel_4_ragged_at_prefill_sizes(gu, oracle, qwen_full, T):
    """Router logits skewed by a per-expert offset ~N(0,1): ragged expert counts, ragged tile schedule."""
    _qwen_ranks_in_sequence(gu, oracle, qwen_full, "ep", T, skew=1.0)


@pytest.mark.parametrize("T", [8192, 16384])
def test_deepseek_tp8_ranks_in_sequence_at_prefill_sizes(gu, oracle, T):
    """The DeepSeek-V3-like layer under TP = 8 with the eight ranks' kernels run one after the other on one GPU:
    grouped sigmoid routing bit-exact on every rank, rank 0 compared with the oracle on every token at 8192
    (64 sampled tokens otherwise), the sum of the eight partial outputs compared with the sum of the oracle's."""
    spec, mk = synth.DEEPSEEK, gu.kernel("ds_tp8")
    toks = gu.sample_tokens(T, 64, 5)
    total = torch.zeros(len(toks), spec.hidden)
    ref_total = torch.zeros(len(toks), spec.hidden)
    batch = None
    for r in range(8):
        sh = synth.make_layer(spec, seed=0, device=gu.DEV, inter_slice=(256 * r, 256 * (r + 1)), with_shared=False, chunk=8)
        if batch is None:
            batch = synth.make_batch(spec, sh, T, seed=0, device=gu.DEV)
        res = gu.launch(mk, sh, batch)
        ids, w, _ = gu.check_routing(oracle, res, batch, 2, sh["bias"], 256)
        q, s = gu.check_act_quant(oracle, res, batch)
        assert torch.isfinite(res["out"].float()).all()
        mine = gu.sample_tokens(T, T, 0) if (r == 0 and T <= 8192) else toks
        gu.check_output(oracle, res["out"], mine, q, s, ids, w, sh)
        total += res["out"].float().cpu()[torch.from_numpy(toks).long()]
        ref_total += oracle.moe_path(toks, q, s, ids, w, sh["w13"], sh["w13_scale"], sh["w2"], sh["w2_scale"]).float()
        del sh, res
    gu.assert_close(oracle, total, ref_total, steps=8)
    torch.cuda.empty_cache()


def test_plain_sigmoid_router_build(gu, oracle, qwen_full):
    """ROUTER_MODE 1 (sigmoid + per-expert bias, no groups; kernel/qwen_tp/src/prefill_mono_final_nb.cu:134-150,
    1068-1076): ids, weights, counts and the permutation bit-exact against the oracle, the oracle cross-checked
    against a torch statement of the rule (selection on sigmoid + bias, weights from the unbiased sigmoid,
    renormalised), and the output within the layer's tolerance. The golden routing logits go through it too."""
    mk = gu.kernel("qwen_sig_w1")
    assert mk.geometry()["router_mode"] == 1
    g = np.load(os.path.join(G, "routing.npz"))
    bias = torch.from_numpy(g["bias"]).to(gu.DEV)
    layer = dict(qwen_full, bias=bias)
    for T, logits in ((96, torch.from_numpy(g["logits"]).to(gu.DEV)), (3000, None)):
        if logits is None:
            batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=8, device=gu.DEV)
        else:
            batch = {"hs": torch.randn(T, 2048, device=gu.DEV).to(torch.bfloat16), "logits": logits}
        res = gu.launch(mk, layer, batch)
        ids, w, _ = gu.check_routing(oracle, res, batch, 1, bias, 256)
        q, s = gu.check_act_quant(oracle, res, batch)
        gu.check_output(oracle, res["out"], gu.sample_tokens(T, 96), q, s, ids, w, layer)
        # torch statement of the rule, fp32; rows with exact ties are left to the tie rule
        sg = torch.sigmoid(batch["logits"].float())
        sel = sg + bias
        top = torch.topk(sel, 9, dim=1)
        clear = ((top.values[:, :8] - top.values[:, 1:9]) > 1e-6).all(1).cpu().numpy()
        tw = sg.gather(1, top.indices[:, :8])
        tw = tw / tw.sum(1, keepdim=True).clamp(min=1e-30)
        assert (ids[clear] == top.indices[:, :8].cpu().numpy()[clear]).all()
        assert np.allclose(w[clear], tw.cpu().numpy()[clear], rtol=1e-5, atol=1e-7)
        assert clear.sum() >= T - 4


@pytest.mark.parametrize("T", [256, 4096])
def test_deepseek_tp8_shard_grouped_router(gu, oracle, T):
    """DeepSeek-V3 geometry, one rank of TP=8 (H=7168, 256 of 2048 intermediate columns),
    group-limited sigmoid router with bias."""
    layer = synth.make_layer(synth.DEEPSEEK, seed=0, device=gu.DEV, inter_slice=(256, 512), with_shared=False, chunk=8)
    batch = synth.make_batch(synth.DEEPSEEK, layer, T, seed=0, device=gu.DEV)
    res = gu.launch(gu.kernel("ds_tp8"), layer, batch)
    ids, w, _ = gu.check_routing(oracle, res, batch, 2, layer["bias"], 256)
    q, s = gu.check_act_quant(oracle, res, batch)
    assert torch.isfinite(res["out"].float()).all()
    gu.check_output(oracle, res["out"], gu.sample_tokens(T, 12), q, s, ids, w, layer)
    if T == 256:
        g = np.load(os.path.join(G, "routing.npz"))
        lg = torch.from_numpy(g["logits"]).to(gu.DEV)
        gl = dict(layer, bias=torch.from_numpy(g["bias"]).to(gu.DEV))
        hs = torch.randn(lg.shape[0], 7168, device=gu.DEV).to(torch.bfloat16)
        r2 = gu.launch(gu.kernel("ds_tp8"), gl, {"hs": hs, "logits": lg})
        rows = np.setdiff1d(np.arange(lg.shape[0]), g["tie_rows"])
        assert (np.sort(r2["ids"], 1)[rows] == g["grouped_ids_sorted_fp32"][rows]).all()
    # the router linear inside the launch, K = 7168: logits close to an fp64 linear, routing bit-exact on the
    # kernel's own logits, output identical to the logits-in entry fed with them
    mk = gu.kernel("ds_tp8")
    from unimonomoe_b200.loader import prepare_router_weight
    rw16 = prepare_router_weight(layer["router_w"].to(torch.bfloat16))
    out = torch.full((T, 7168), float("nan"), dtype=torch.bfloat16, device=gu.DEV)
    sc = mk.scratch(T, gu.DEV)
    mk.prefill_impl(batch["hs"], None, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], 8, True,
                    layer["bias"], out, check=True, router_weight=rw16)
    lk = sc["logits"].clone()
    ids_k, w_k = sc["topk_ids"].cpu().numpy(), sc["topk_weights"].cpu().numpy()
    ref64 = batch["hs"].double() @ rw16.double().t()
    assert float((lk.double() - ref64).abs().max()) <= 1e-4
    ids2, w2, _ = oracle.route(lk, mode=2, bias=layer["bias"])
    assert (ids_k == ids2).all() and (w_k.view(np.uint32) == w2.view(np.uint32)).all()
    r3 = gu.launch(mk, layer, {"hs": batch["hs"], "logits": lk}, poison=False)
    assert torch.equal(r3["out"].view(torch.int16), out.view(torch.int16))


@pytest.mark.parametrize("variant,width", [("ds_tp2", 1024), ("ds_w1", 2048)])
def test_deepseek_wide_shards_run_in_chunks(gu, oracle, variant, width):
    """DeepSeek-V3 geometry at 1/2 and full expert width: the intermediate (1024 / 2048 columns) exceeds
    what shared memory holds as one e4m3 tile, so every tile is processed in chunks of 512 columns, each
    chunk leaving its own bf16 partial row. Routing stays bit-exact; the output meets the same bounds
    against the oracle, which rounds per chunk in the same way."""
    mk = gu.kernel(variant)
    assert mk._int_symbol("partial_chunks") == width // 512
    layer = synth.make_layer(synth.DEEPSEEK, seed=0, device=gu.DEV, inter_slice=(0, width), with_shared=False, chunk=8)
    for T in (96, 1000):
        batch = synth.make_batch(synth.DEEPSEEK, layer, T, seed=1, device=gu.DEV)
        res = gu.launch(mk, layer, batch)
        ids, w, _ = gu.check_routing(oracle, res, batch, 2, layer["bias"], 256, rows_per_unit=None)
        q, s = gu.check_act_quant(oracle, res, batch)
        assert torch.isfinite(res["out"].float()).all()
        toks = gu.sample_tokens(T, 6)
        gu.check_output(oracle, res["out"], toks, q, s, ids, w, layer)
        # and against the computation that knows nothing of chunks: one bf16 partial row per slot
        # (chunk_cols = the whole width), then the reference's fp64 dequantised layer with its own bounds
        got = res["out"].float().cpu()[torch.from_numpy(toks).long()]
        whole = oracle.moe_path(toks, q, s, ids, w, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"],
                                chunk_cols=width)
        # one bf16 rounding per chunk against one per slot: a different rounding scheme, so single steps are common
        gu.assert_close(oracle, got, whole.float(), steps=width // 512 + 1, rare=None)
        ref64 = oracle.moe_fp64(batch["hs"].cpu()[torch.from_numpy(toks).long()], ids[toks], w[toks], layer["w13"].cpu(),
                                layer["w13_scale"].cpu(), layer["w2"].cpu(), layer["w2_scale"].cpu())
        rl2, cs = oracle.rel_cos(got, ref64)
        assert rl2 < 6e-2 and cs > 0.998, (rl2, cs)
    del layer
    torch.cuda.empty_cache()


def test_folded_residual_and_output_scale(gu, oracle, qwen_full):
    """The reference's fold gates (validation/tp8_fold_gate.py:332-409) on one GPU through the
    _tp2 entry with the collective switched off: a null residual with scale 1 is bitwise inert,
    scale 0 returns the residual, and out = bf16(2.5 * routed + residual)."""
    mk = gu.kernel("qwen_w1")
    T = 512
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=6, device=gu.DEV)
    base = gu.launch(mk, qwen_full, batch)
    resid = (torch.randn(T, 2048, device=gu.DEV) * 0.1).to(torch.bfloat16)
    sc = mk.scratch(T, gu.DEV)
    vp = ctypes.c_void_p

    def tp2(residual, scale):
        out = torch.full((T, 2048), float("nan"), dtype=torch.bfloat16, device=gu.DEV)
        rc = mk.lib.launch_prefill_moe_wgmma_q1_tp2(
            vp(batch["logits"].data_ptr()), T, 128, vp(sc["workspace"].data_ptr()), ctypes.c_size_t(sc["workspace"].numel()),
            vp(batch["hs"].data_ptr()), vp(sc["act_fp8"].data_ptr()), vp(sc["act_scales"].data_ptr()),
            vp(qwen_full["w13"].data_ptr()), vp(qwen_full["w13_scale"].data_ptr()), vp(qwen_full["w2"].data_ptr()),
            vp(qwen_full["w2_scale"].data_ptr()), vp(sc["partial"].data_ptr()), vp(sc["topk_ids"].data_ptr()),
            vp(sc["topk_weights"].data_ptr()), vp(sc["sorted_ids"].data_ptr()), vp(out.data_ptr()), vp(0),
            vp(0), vp(0), 0, 1, 1, 0, ctypes.c_uint(0), vp(0),
            vp(0 if residual is None else residual.data_ptr()), ctypes.c_float(scale),
            vp(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        mk.check_status(sc["workspace"])
        return out

    assert torch.equal(tp2(None, 1.0).view(torch.int16), base["out"].view(torch.int16))
    assert torch.equal(tp2(resid, 0.0).view(torch.int16), resid.view(torch.int16))
    folded = tp2(resid, 2.5)
    q, s = gu.check_act_quant(oracle, base, batch)
    toks = gu.sample_tokens(T, 24, 4)
    gu.check_output(oracle, folded, toks, q, s, base["ids"], base["weights"], qwen_full, out_scale=2.5,
                    residual=resid.cpu())


def test_bounded_wait_reports_instead_of_hanging(gu, qwen_full):
    """A rank barrier that no peer ever answers: the fused tensor-parallel epilogue is launched with
    world = 2 while rank 1 does not exist (its barrier window is plain local memory that nothing
    writes). The wait gives up after the time limit, the status word says which wait, and the
    context stays usable: the next ordinary launch succeeds."""
    mk = gu.kernel("qwen_w1")
    T = 256
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=7, device=gu.DEV)
    sc = mk.scratch(T, gu.DEV)
    out = torch.zeros(T, 2048, dtype=torch.bfloat16, device=gu.DEV)
    ncomm, nchunk, world = 4, 2, 2
    pads = torch.zeros(world, mk.tp_pad_words(nchunk, ncomm, world), dtype=torch.int32, device=gu.DEV)
    pad_ptrs = torch.tensor([pads[0].data_ptr(), pads[1].data_ptr()], dtype=torch.int64, device=gu.DEV)
    seqctr = torch.zeros(1, dtype=torch.int32, device=gu.DEV)
    mk.set_wait_timeout_us(200_000)
    try:
        with pytest.raises(RuntimeError, match="rank barrier timed out"):
            # the "multicast" pointer is never dereferenced: the barrier in front of it fails first
            mk.prefill_out(batch["hs"], batch["logits"], qwen_full["w13"], qwen_full["w13_scale"], qwen_full["w2"],
                           qwen_full["w2_scale"], out, tp_mc_ptr=out.data_ptr(), tp_pads_ptr=pad_ptrs.data_ptr(),
                           tp_seqctr_ptr=seqctr.data_ptr(), tp_rank=0, tp_world=world, tp_nchunk=nchunk,
                           tp_ncomm=ncomm, check=True)
    finally:
        mk.set_wait_timeout_us(2_000_000)
    assert int(seqctr.item()) == 1
    res = gu.launch(mk, qwen_full, batch)
    assert torch.isfinite(res["out"].float()).all()


def test_cuda_graph_capture_and_replay(gu, qwen_full):
    """The launch is capturable (no allocation, no host synchronisation inside it): a captured launch
    replayed three times, with fresh inputs copied into the captured buffers before each replay,
    reproduces eager launches bit for bit (after validation/tp8_soak.py:351-402)."""
    mk = gu.kernel("qwen_w1")
    T = 1536
    batches = [synth.make_batch(synth.QWEN, qwen_full, T, seed=20 + i, device=gu.DEV) for i in range(3)]
    eager = []
    for b in batches:
        eager.append(gu.launch(mk, qwen_full, b, poison=False)["out"].clone())
    hs = batches[0]["hs"].clone()
    lg = batches[0]["logits"].clone()
    out = torch.empty(T, 2048, dtype=torch.bfloat16, device=gu.DEV)
    sc = mk.scratch(T, gu.DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # warm-up on the capture stream, as torch asks
        mk.prefill_impl(hs, lg, qwen_full["w13"], qwen_full["w13_scale"], qwen_full["w2"], qwen_full["w2_scale"], 8, True,
                        None, out, scratch=sc)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        mk.prefill_impl(hs, lg, qwen_full["w13"], qwen_full["w13_scale"], qwen_full["w2"], qwen_full["w2_scale"], 8, True,
                        None, out, scratch=sc)
    for i, b in enumerate(batches):
        hs.copy_(b["hs"])
        lg.copy_(b["logits"])
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        mk.check_status(sc["workspace"])
        assert torch.equal(out.view(torch.int16), eager[i].view(torch.int16)), i


def _fp64_topk_margin(scores64, k=8):
    """Gap between the k-th and (k+1)-th largest selection score of every token, in fp64."""
    top = torch.topk(scores64, k + 1, dim=1).values
    return (top[:, k - 1] - top[:, k])


@pytest.mark.parametrize("T", [1, 1000, 16384, 30720])   # 30720: two token tiles per CTA in the router phase
def test_router_linear_inside_the_launch(gu, oracle, qwen_full, T):
    """The _gemv entry computes logits = x * W_r^T (bf16 operands, fp32 accumulation on the tensor cores)
    for the tokens each CTA routes and routes on them in the same launch. Its accumulation order inside
    one instruction is the hardware's, so the logits are compared with an fp64 linear within a tolerance,
    and routing is pinned in two steps: (1) ids, weights, counts and the permutation are bit-exact against
    the oracle fed with the logits the kernel itself produced; (2) every token whose expert set differs
    from an fp64 route sits at a decision margin below 1e-5 (the rule of research_archive/ds3_acc.py:440-458).
    The output then has to equal, bit for bit, a logits-in launch on those same logits."""
    mk = gu.kernel("qwen_w1")
    assert mk.has_gemv
    from unimonomoe_b200.loader import prepare_router_weight
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=3, device=gu.DEV)
    rw16 = prepare_router_weight(qwen_full["router_w"].to(torch.bfloat16))
    out = torch.full((T, 2048), float("nan"), dtype=torch.bfloat16, device=gu.DEV)
    sc = mk.scratch(T, gu.DEV)
    sc.pop("logits", None)
    mk.prefill_impl(batch["hs"], None, qwen_full["w13"], qwen_full["w13_scale"], qwen_full["w2"], qwen_full["w2_scale"],
                    8, True, None, out, check=True, router_weight=rw16)
    lk = sc["logits"].clone()
    ids_k, w_k, srt_k = sc["topk_ids"].cpu().numpy(), sc["topk_weights"].cpu().numpy(), sc["sorted_ids"].cpu().numpy()
    wv = mk.workspace_view(sc["workspace"])
    # logits against fp64
    ref64 = batch["hs"].double() @ rw16.double().t()
    err = float((lk.double() - ref64).abs().max())
    assert err <= 4e-5, err   # measured 1.2e-5 at |logit| up to 5.4: the accumulator keeps a little less than fp32
    # (1) routing of the kernel's own logits, bit-exact
    ids, w, _ = oracle.route(lk, mode=0)
    assert (ids_k == ids).all() and (w_k.view(np.uint32) == w.view(np.uint32)).all()
    cnt, off, srt = oracle.sort_slots(ids, 256)
    assert (wv["expert_counts"].numpy()[:256] == cnt).all() and (srt_k[:len(srt)] == srt).all()
    # (2) disagreements with an fp64 route only at sub-epsilon margins
    ids64 = torch.topk(ref64, 8, dim=1).indices.sort(1).values.cpu().numpy()
    differ = (np.sort(ids_k, 1) != ids64).any(1)
    if differ.any():
        # the reference's bound is 1e-5 on sigmoid scores in [0, 1]; softmax selection compares raw logits of
        # magnitude ~5, and two logits that are each off by `err` can swap only when they are closer than 2*err
        marg = _fp64_topk_margin(ref64).cpu().numpy()
        assert float(marg[differ].max()) <= 2 * err, (int(differ.sum()), float(marg[differ].max()), err)
    assert differ.sum() <= max(2, T // 2000)
    # same output as the logits-in entry on those logits
    b2 = {"hs": batch["hs"], "logits": lk}
    res = gu.launch(mk, qwen_full, b2, poison=False)
    assert torch.equal(res["out"].view(torch.int16), out.view(torch.int16))


def test_tiny_batches_repeated(gu, qwen_full):
    """At one or a few tokens almost every CTA has no tile and runs straight through the expert phase:
    the hand-back of registers between producer and epilogue warps must not depend on who asks first.
    150 launches each of 1 and 7 tokens, through both entries, with a host-side deadline instead of a
    blocking synchronise so that a stall fails the test."""
    import time
    mk = gu.kernel("qwen_w1")
    from unimonomoe_b200.loader import prepare_router_weight
    rw16 = prepare_router_weight(qwen_full["router_w"].to(torch.bfloat16))
    for T in (1, 7):
        batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=11, device=gu.DEV)
        out = torch.empty(T, 2048, dtype=torch.bfloat16, device=gu.DEV)
        first = None
        for i in range(150):
            ev = torch.cuda.Event()
            mk.prefill_impl(batch["hs"], batch["logits"], qwen_full["w13"], qwen_full["w13_scale"], qwen_full["w2"],
                            qwen_full["w2_scale"], 8, True, None, out, router_weight=rw16 if i % 2 else None)
            ev.record()
            t0 = time.time()
            while not ev.query():
                assert time.time() - t0 < 10.0, f"launch {i} at T={T} did not finish within 10 s"
                time.sleep(0.001)
            if i % 2 == 0:
                if first is None:
                    first = out.clone()
                assert torch.equal(out.view(torch.int16), first.view(torch.int16))
        mk.check_status(mk.scratch(T, gu.DEV)["workspace"])


def test_descriptors_are_made_once_per_weight_tensor(gu, qwen_full):
    """Plan / run split: the TMA descriptors of a layer's weights are encoded at the first launch (or by
    prefill_wgmma_plan_prepare) and found again by every later one; a second layer adds its own two."""
    mk = gu.kernel("qwen_w1")
    lib = mk.lib
    lib.prefill_wgmma_plan_prepare.restype = ctypes.c_int

    def stats():
        h, m = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        lib.prefill_wgmma_plan_stats(ctypes.byref(h), ctypes.byref(m))
        return h.value, m.value

    lib.prefill_wgmma_plan_reset()
    h0, m0 = stats()
    assert lib.prefill_wgmma_plan_prepare(ctypes.c_void_p(qwen_full["w13"].data_ptr()),
                                          ctypes.c_void_p(qwen_full["w2"].data_ptr())) == 0
    h1, m1 = stats()
    assert m1 - m0 == 2 and h1 == h0
    batch = synth.make_batch(synth.QWEN, qwen_full, 300, seed=31, device=gu.DEV)
    first = gu.launch(mk, qwen_full, batch)["out"].clone()
    for _ in range(5):
        again = gu.launch(mk, qwen_full, batch)["out"]
        assert torch.equal(first.view(torch.int16), again.view(torch.int16))
    h2, m2 = stats()
    assert m2 == m1 and h2 - h1 == 12          # six launches, two look-ups each, nothing encoded again
    other = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in qwen_full.items()}
    gu.launch(mk, other, batch)
    assert stats()[1] == m2 + 2


def test_captured_graph_survives_other_batch_sizes(gu, qwen_full):
    """A captured launch holds the addresses of its scratch. Launches of five other sizes through the same
    MonoKernel, one of them larger than anything seen before (which makes the scratch arena grow), must
    leave that memory alone: the replay afterwards still reproduces the eager result bit for bit."""
    from unimonomoe_b200 import MonoKernel, variant_path
    mk = MonoKernel(variant_path("qwen_w1"))          # a fresh object: its arena starts empty
    T = 640
    batch = synth.make_batch(synth.QWEN, qwen_full, T, seed=41, device=gu.DEV)
    w = (qwen_full["w13"], qwen_full["w13_scale"], qwen_full["w2"], qwen_full["w2_scale"])
    eager = torch.empty(T, 2048, dtype=torch.bfloat16, device=gu.DEV)
    mk.prefill_impl(batch["hs"], batch["logits"], *w, 8, True, None, eager, check=True)
    out = torch.empty(T, 2048, dtype=torch.bfloat16, device=gu.DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        mk.prefill_impl(batch["hs"], batch["logits"], *w, 8, True, None, out)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        mk.prefill_impl(batch["hs"], batch["logits"], *w, 8, True, None, out)
    for other in (100, 200, 333, 512, 2000):       # 2000 > 640: a larger arena is added, the old one is kept
        b2 = synth.make_batch(synth.QWEN, qwen_full, other, seed=other, device=gu.DEV)
        o2 = torch.empty(other, 2048, dtype=torch.bfloat16, device=gu.DEV)
        mk.prefill_impl(b2["hs"], b2["logits"], *w, 8, True, None, o2, check=True)
        junk = torch.full((other * 8, 2048), float("nan"), dtype=torch.bfloat16, device=gu.DEV)   # churn the allocator
        del junk
    assert len(mk._retired) == 1
    out.fill_(float("nan"))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), eager.view(torch.int16))


@pytest.mark.parametrize("rank", [0, 5])
def test_deepseek_expert_parallel_8_rank_in_sequence(gu, oracle, rank):
    """DeepSeek-V3 geometry under EP = 8: 32 local experts at the full intermediate width of 2048 columns (the
    configuration in which the reference ran out of shared memory, research_archive/reports/
    ds3_ep_monokernel_result.md:118-153), here processed in four chunks of 512. One rank at a time on one GPU:
    grouped sigmoid routing with the global-to-local map bit-exact, output against the oracle."""
    spec, mk = synth.DEEPSEEK, gu.kernel("ds_ep8")
    geo = mk.geometry()
    assert geo["num_experts_local"] == 32 and geo["n_half"] == 2048 and mk._int_symbol("partial_chunks") == 4
    layer = synth.make_layer(spec, seed=0, device=gu.DEV, expert_slice=(32 * rank, 32 * rank + 32), with_shared=False, chunk=8)
    emap = synth.expert_map(spec, rank, 8, device=gu.DEV)
    for T in (200, 4096):
        batch = synth.make_batch(spec, layer, T, seed=2, device=gu.DEV)
        res = gu.launch(mk, layer, batch, expert_map=emap)
        ids, w, gids = gu.check_routing(oracle, res, batch, 2, layer["bias"], 32, expert_map=emap, rows_per_unit=None)
        q, s = gu.check_act_quant(oracle, res, batch)
        assert res["ids"].min() >= -1 and res["ids"].max() < 32
        owned = (res["ids"] >= 0).sum()
        assert 0 < owned < T * 8
        assert torch.isfinite(res["out"].float()).all()
        gu.check_output(oracle, res["out"], gu.sample_tokens(T, 24, rank), q, s, ids, w, layer)
    del layer
    torch.cuda.empty_cache()


def _shared_reference(oracle, toks, q, s, ids, w, layer, sh, hs, out_scale=1.0, part=(0, 1), residual=None):
    """What the launch with the shared expert inside must produce, from the oracle's bf16 partial rows:
    bf16(out_scale * sum_k routed_row_k + shared_row (+ residual)), all sums in fp32. The shared expert is
    evaluated as one more expert every listed token goes to, weighted by sigmoid(x . g) (or 1 without a gate)."""
    n = len(toks)
    _, part_r, *_ = oracle.moe_path(toks, q, s, ids, w, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"],
                                    want_dumps=True)
    k = ids.shape[1]
    owned = torch.from_numpy((ids[toks] >= 0).astype(np.float32))                      # rows of experts held elsewhere do not exist
    routed = (part_r.float().view(n, k, -1, part_r.shape[-1]).sum(2) * owned[:, :, None]).sum(1)
    T = ids.shape[0]
    if sh["gate"] is not None:
        gw = torch.sigmoid(hs.double().cpu() @ sh["gate"].double().cpu()).float().numpy().reshape(T, 1)
    else:
        gw = np.ones((T, 1), np.float32)
    _, part_s, *_ = oracle.moe_path(toks, q, s, np.zeros((T, 1), np.int32), gw, sh["w13"][None], sh["w13_scale"][None],
                                    sh["w2"][None], sh["w2_scale"][None], want_dumps=True)
    shared = part_s.float().view(n, -1, part_s.shape[-1]).sum(1)
    mine = torch.from_numpy(((toks // 128) % part[1] == part[0]).astype(np.float32))[:, None]
    base = shared * mine
    if residual is not None:
        base = base + residual.float().cpu()[torch.from_numpy(toks).long()]
    return (routed * out_scale + base).to(torch.bfloat16).float()


@pytest.mark.parametrize("T", [200, 3000])
def test_gated_shared_expert_inside_the_launch(gu, oracle, T):
    """The sigmoid-gated shared expert of the Qwen-like layer computed by the same launch as the routed experts
    (as dense tiles appended to the tile schedule): routing stays bit-exact, and the output equals
    bf16(routed + sigmoid(x . g) * shared(x)) built from the oracle's partial rows. A launch without the shared
    expert afterwards is bitwise what it was before."""
    from unimonomoe_b200.loader import prepare_shared_expert
    mk = gu.kernel("qwen_w1")
    assert mk.has_shared
    layer = synth.make_layer(synth.QWEN, seed=0, device=gu.DEV, with_shared=True)
    shd = layer["shared"]
    sh = prepare_shared_expert(shd["w13"], shd["w13_scale"], shd["w2"], shd["w2_scale"], shd["gate"])
    batch = synth.make_batch(synth.QWEN, layer, T, seed=12, device=gu.DEV)
    before = gu.launch(mk, layer, batch)
    out = torch.full((T, 2048), float("nan"), dtype=torch.bfloat16, device=gu.DEV)
    sc = mk.prefill_impl(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], 8,
                         True, None, out, check=True, shared=sh)
    assert torch.isfinite(out.float()).all()
    ids, w, _ = oracle.route(batch["logits"], mode=0)
    assert (sc["topk_ids"].cpu().numpy() == ids).all()
    q, s = oracle.quant_act(batch["hs"])
    toks = gu.sample_tokens(T, 160, 6)
    ref = _shared_reference(oracle, toks, q, s, ids, w, layer, sh, batch["hs"])
    gu.assert_close(oracle, out.float().cpu()[torch.from_numpy(toks).long()], ref, steps=2)
    # the shared half is really there: without it the result is far away
    m = oracle.parity_metrics(before["out"].float().cpu()[torch.from_numpy(toks).long()], ref)
    assert m["rel_l2"] > 0.05, m
    after = gu.launch(mk, layer, batch)
    assert torch.equal(after["out"].view(torch.int16), before["out"].view(torch.int16))


def test_shared_expert_with_scale_residual_and_token_split(gu, oracle):
    """DeepSeek-like shard (ungated shared expert, routed_scaling_factor 2.5 on the routed half, a residual) and
    the token split used by expert-parallel ranks: a launch with (part, parts) = (1, 4) adds the shared expert
    only for the 128-token tiles j with j % 4 == 1."""
    from unimonomoe_b200.loader import prepare_shared_expert
    spec, mk = synth.DEEPSEEK, gu.kernel("ds_tp8")
    layer = synth.make_layer(spec, seed=0, device=gu.DEV, inter_slice=(0, 256), with_shared=False, chunk=8)
    g = torch.Generator(device=gu.DEV).manual_seed(77)
    sw13, sw13s = synth.quantize_block_fp8((torch.randn(512, 7168, device=gu.DEV, generator=g) * 0.02).to(torch.bfloat16))
    sw2, sw2s = synth.quantize_block_fp8((torch.randn(7168, 256, device=gu.DEV, generator=g) * 0.02).to(torch.bfloat16))
    sh = prepare_shared_expert(sw13, sw13s, sw2, sw2s, None)
    T = 900
    batch = synth.make_batch(spec, layer, T, seed=3, device=gu.DEV)
    resid = (torch.randn(T, 7168, device=gu.DEV, generator=g) * 0.05).to(torch.bfloat16)
    ids, w, _ = oracle.route(batch["logits"], mode=2, bias=layer["bias"])
    q, s = oracle.quant_act(batch["hs"])
    toks = gu.sample_tokens(T, 48, 8)
    for part in ((0, 1), (1, 4)):
        out = torch.full((T, 7168), float("nan"), dtype=torch.bfloat16, device=gu.DEV)
        mk.prefill_impl(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], 8,
                        True, layer["bias"], out, residual=resid, out_scale=2.5, check=True, shared=sh, shared_part=part)
        assert torch.isfinite(out.float()).all()
        ref = _shared_reference(oracle, toks, q, s, ids, w, layer, sh, batch["hs"], out_scale=2.5, part=part, residual=resid)
        gu.assert_close(oracle, out.float().cpu()[torch.from_numpy(toks).long()], ref, steps=2)
    del layer
    torch.cuda.empty_cache()
