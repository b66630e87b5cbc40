"""Seeded synthetic MoE layers and prefill batches with the shapes, sizes and value
distributions of the reference's measurements (real checkpoints are not available):
weights ~N(0, 0.02) in bf16 quantised to e4m3 with one fp32 scale per [128,128] block
(amax/448, clamped at 1e-12), as validation/tp8_fuse_ab.py:243-258 does; hidden states bf16
~N(0,1); router weight fp32 ~N(0, 0.02). Shards of tensor/expert-parallel ranks are cut
from one global layer so that every rank agrees on it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class LayerSpec:
    name: str
    hidden: int            # H = K
    inter: int             # routed expert intermediate width I
    experts: int = 256
    top_k: int = 8
    router_mode: int = 0   # 0 softmax, 2 grouped sigmoid + bias
    n_group: int = 8
    topk_group: int = 4
    shared_inter: int = 0
    shared_gate: bool = False
    routed_scaling: float = 1.0


QWEN = LayerSpec("qwen3.5-35b-a3b-like", hidden=2048, inter=512, router_mode=0, shared_inter=512, shared_gate=True)
DEEPSEEK = LayerSpec("deepseek-v3-like", hidden=7168, inter=2048, router_mode=2, shared_inter=2048,
                     routed_scaling=2.5)


def quantize_block_fp8(w: torch.Tensor):
    """[..., R, C] (R, C multiples of 128) -> (e4m3 [..., R, C], fp32 scales [..., R/128, C/128])."""
    *lead, R, C = w.shape
    f = w.float().reshape(*lead, R // 128, 128, C // 128, 128)
    sc = (f.abs().amax(dim=(-3, -1)) / 448.0).clamp(min=1e-12).to(torch.float32)
    q = (f / sc[..., :, None, :, None]).clamp(-448, 448).reshape(*lead, R, C).to(torch.float8_e4m3fn)
    return q.contiguous(), sc.contiguous()


def _gen(shape, gen, device, std):
    return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def make_layer(spec: LayerSpec, seed: int = 0, device="cpu", inter_slice=None, expert_slice=None,
               chunk: int = 16, with_shared: bool = True) -> dict:
    """Build the layer (or one rank's shard of it).

    inter_slice=(lo, hi) keeps rows [lo,hi) of gate and of up and columns [lo,hi) of down
    (tensor parallel); expert_slice=(lo, hi) keeps those experts (expert parallel). Experts
    are generated one chunk at a time from per-chunk seeds, so a shard equals the same
    slice of the full layer.
    """
    E, H, I = spec.experts, spec.hidden, spec.inter
    lo, hi = inter_slice or (0, I)
    e_lo, e_hi = expert_slice or (0, E)
    dev = torch.device(device)
    w13, w13s, w2, w2s = [], [], [], []
    for c0 in range(0, E, chunk):
        c1 = min(E, c0 + chunk)
        if c1 <= e_lo or c0 >= e_hi:
            continue
        g = torch.Generator(device=dev).manual_seed(seed * 1000003 + 17 * c0 + 1)
        gu = _gen((c1 - c0, 2 * I, H), g, dev, 0.02)
        dn = _gen((c1 - c0, H, I), g, dev, 0.02)
        q13, s13 = quantize_block_fp8(gu)
        q2, s2 = quantize_block_fp8(dn)
        del gu, dn
        a, b = max(c0, e_lo) - c0, min(c1, e_hi) - c0
        nb = I // 128
        rows = torch.cat([torch.arange(lo, hi), torch.arange(I + lo, I + hi)]).to(dev)
        srows = torch.cat([torch.arange(lo // 128, hi // 128), torch.arange(nb + lo // 128, nb + hi // 128)]).to(dev)
        w13.append(q13[a:b].view(torch.uint8)[:, rows].contiguous())
        w13s.append(s13[a:b][:, srows].contiguous())
        w2.append(q2[a:b].view(torch.uint8)[:, :, lo:hi].contiguous())
        w2s.append(s2[a:b][:, :, lo // 128: hi // 128].contiguous())
        del q13, s13, q2, s2
    g = torch.Generator(device=dev).manual_seed(seed * 1000003 + 999983)
    layer = {
        "spec": spec,
        "w13": torch.cat(w13).view(torch.float8_e4m3fn),
        "w13_scale": torch.cat(w13s),
        "w2": torch.cat(w2).view(torch.float8_e4m3fn),
        "w2_scale": torch.cat(w2s),
        "router_w": torch.randn(E, H, generator=g, device=dev, dtype=torch.float32) * 0.02,
        "bias": None,
        "shared": None,
    }
    if spec.router_mode != 0:
        # e_score_correction_bias: small per-expert offsets
        layer["bias"] = torch.randn(E, generator=g, device=dev, dtype=torch.float32) * 0.01
    if with_shared and spec.shared_inter:
        Is = spec.shared_inter
        s13q, s13s = quantize_block_fp8(_gen((2 * Is, H), g, dev, 0.02))
        s2q, s2s = quantize_block_fp8(_gen((H, Is), g, dev, 0.02))
        layer["shared"] = {
            "w13": s13q, "w13_scale": s13s, "w2": s2q, "w2_scale": s2s,
            "gate": (torch.randn(1, H, generator=g, device=dev, dtype=torch.float32) * 0.02) if spec.shared_gate else None,
        }
    return layer


def make_batch(spec: LayerSpec, layer: dict, T: int, seed: int = 0, device="cpu", skew: float = 0.0,
               act_std: float = 1.0) -> dict:
    """Hidden states bf16 ~N(0, act_std) and the router logits the model would hand over:
    bf16 linear then float for the softmax geometry (research_archive/superseded/acc_final.py:212),
    fp32 linear for the sigmoid geometry (research_archive/ds3_acc.py:412). skew > 0 adds a
    per-expert N(0, skew) logit offset so per-expert token counts become ragged."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed * 7919 + 12345 + T)
    hs = (torch.randn(T, spec.hidden, generator=g, device=dev, dtype=torch.float32) * act_std).to(torch.bfloat16)
    rw = layer["router_w"].to(dev)
    if spec.router_mode == 0:
        logits = torch.nn.functional.linear(hs, rw.to(torch.bfloat16)).float()
    else:
        logits = torch.nn.functional.linear(hs.float(), rw)
    if skew > 0:
        logits = logits + torch.randn(spec.experts, generator=g, device=dev, dtype=torch.float32) * skew
    return {"hs": hs.contiguous(), "logits": logits.contiguous()}


def expert_map(spec: LayerSpec, rank: int, world: int, device="cpu") -> torch.Tensor:
    """int32 [E]: local slot of each global expert on this rank, -1 elsewhere
    (validation/ep4_acc.py:226-233)."""
    n = spec.experts // world
    m = torch.full((spec.experts,), -1, dtype=torch.int32, device=device)
    m[rank * n:(rank + 1) * n] = torch.arange(n, dtype=torch.int32, device=device)
    return m


def routed_flops(spec: LayerSpec, T: int) -> float:
    """Algorithmic FLOPs of the routed experts of one layer: T * top_k * 6 * H * I."""
    return float(T) * spec.top_k * 6.0 * spec.hidden * spec.inter
