"""Shared helpers of the GPU parity tests: launch through the C-ABI, compare with the oracle."""
import numpy as np
import torch

from unimonomoe_b200 import MonoKernel, synth, variant_path

DEV = "cuda:0"
# acceptance bounds of the output comparison against the path-faithful oracle
MAX_ABS_OVER_RMS = 2e-2
MIN_COS = 0.9995

_KERNELS = {}


def kernel(variant: str) -> MonoKernel:
    if variant not in _KERNELS:
        _KERNELS[variant] = MonoKernel(variant_path(variant))
    return _KERNELS[variant]


def launch(mk, layer, batch, expert_map=None, poison=True):
    """One launch through the ctypes C-ABI; returns host copies of everything it wrote."""
    T = batch["hs"].shape[0]
    H = layer["w2"].shape[1]
    out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    sc = mk.scratch(T, DEV)
    if poison:
        sc["partial"].fill_(float("nan"))
        sc["sorted_ids"].fill_(-7)
    mk.prefill_impl(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"],
                    8, True, layer.get("bias"), out, expert_map=expert_map, check=True)
    wv = mk.workspace_view(sc["workspace"])
    return {
        "out": out, "ids": sc["topk_ids"].cpu().numpy(), "weights": sc["topk_weights"].cpu().numpy(),
        "sorted": sc["sorted_ids"].cpu().numpy(), "act_q": sc["act_fp8"].cpu().numpy(),
        "act_s": sc["act_scales"].cpu().numpy(), "counts": wv["expert_counts"].numpy(),
        "offsets": wv["expert_offsets"].numpy(), "total_tiles": wv["total_tiles"],
    }


def check_routing(O, res, batch, mode, bias, n_local, expert_map=None, rows_per_unit=128):
    """Expert ids, weights, counts, offsets and the sort permutation must be bit-exact."""
    ids, w, gids = O.route(batch["logits"], mode=mode, bias=bias, expert_map=expert_map)
    assert (res["ids"] == ids).all(), f"{int((res['ids'] != ids).any(1).sum())} tokens routed differently"
    assert (res["weights"].view(np.uint32) == w.view(np.uint32)).all()
    cnt, off, srt = O.sort_slots(ids, n_local)
    assert (res["counts"][:n_local] == cnt).all()
    assert (res["offsets"][:n_local + 1] == off).all()
    assert (res["sorted"][:len(srt)] == srt).all()
    # scheduling units: tiles of 128 sorted rows, or pairs of them in the two-CTA build
    if rows_per_unit is not None:   # builds that process a tile in chunks count (tile, chunk) units instead
        assert res["total_tiles"] == int(((cnt + rows_per_unit - 1) // rows_per_unit).sum())
    return ids, w, gids


def check_act_quant(O, res, batch):
    q, s = O.quant_act(batch["hs"])
    assert (res["act_q"] == q).all()
    assert (res["act_s"].view(np.uint32) == s.view(np.uint32)).all()
    return q, s


def sample_tokens(T, n, seed=0):
    if T <= n:
        return np.arange(T, dtype=np.int32)
    return np.sort(np.random.RandomState(seed).choice(T, n, replace=False)).astype(np.int32)


def bf16_spacing(x: torch.Tensor) -> torch.Tensor:
    """Distance between neighbouring bf16 values at the magnitude of x (fp32 tensor)."""
    mag = x.abs().clamp(min=2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(mag)) - 7.0)


def assert_close(O, got, ref, steps: float = 2.0, rare: float = 1e-4):
    """The acceptance rule of `check_output` for two fp32 tensors; `steps` bf16 steps are allowed where the
    spacing exceeds 2e-2 rms (sums of several bf16 outputs can differ by one step per summand), and at most the
    fraction `rare` of the elements may be of that kind (None: any number, for comparisons between two different
    rounding schemes)."""
    m = O.parity_metrics(got, ref)
    err = (got - ref).abs()
    beyond = err > MAX_ABS_OVER_RMS * m["rms_ref"]
    m["beyond_2e-2_rms"] = int(beyond.sum())
    if beyond.any():
        assert bool((err[beyond] <= bf16_spacing(ref[beyond]) * steps * 1.0001).all()), m
        if rare is not None:
            assert m["beyond_2e-2_rms"] <= max(1, int(ref.numel() * rare)), m
    assert m["cos"] >= MIN_COS, m
    return m


def check_output(O, out, toks, q, s, ids, w, layer, **kw):
    """bf16 output against the path-faithful oracle: cosine >= 0.9995 and every element within
    max(2e-2 * rms(ref), two bf16 steps of the reference value).

    The second term matters only when many elements are compared. The partial rows and the output are bf16: at
    |value| above 3 rms neighbouring bf16 values are more than 2e-2 * rms apart, so there the smallest
    difference two correct implementations can show (the kernel's tensor-core summation order against the
    oracle's, meeting a rounding boundary in a partial row, in the final rounding, or in both) already exceeds
    the first term. Such elements must be within two steps, and they must be rare (below one in 10 000)."""
    ref = O.moe_path(toks, q, s, ids, w, layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"], **kw).float()
    got = out.float().cpu()[torch.from_numpy(toks).long()]
    assert torch.isfinite(got).all()
    return assert_close(O, got, ref, steps=2.0)
