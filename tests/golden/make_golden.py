"""Generate the golden vectors under tests/golden/ by EXECUTING the reference's own torch
routines on CPU. Run in the build container only (it reads the reference checkout); the
committed .npz files are what the tests use.

    python tests/golden/make_golden.py [/path/to/reference]

The reference's gate scripts cannot be imported (their top level opens a GPU, a compiled
kernel and a model checkpoint), so the function definitions are lifted out of the source
text with ``ast`` and executed unchanged with the module constants they expect:

* ``route_ref``  research_archive/ds3_acc.py:242-273   grouped sigmoid router (torch)
* ``dequant``, ``oracle``, ``rel_cos``, ``build_map``  research_archive/ds3_acc.py:276-329
  (identical arithmetic to validation/ep4_acc.py:183-233) the fp64 dequantised MoE
* softmax routing reference: ``torch.topk(logits, TOP_K)`` as validation/ep4_acc.py:355 states it
* weight fixture recipe of validation/tp8_fuse_ab.py:243-258 (restated in unimonomoe_b200/synth.py)
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 and __name__ == "__main__" else None
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from unimonomoe_b200 import synth  # noqa: E402


def lift(path, names, env):
    """exec the named top-level function definitions of a source file inside env."""
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, path, "exec"), env)
    missing = [n for n in names if n not in env]
    assert not missing, missing
    return env


def routing_golden():
    E, TOP_K, N_GROUP, TOPK_GROUP, T = 256, 8, 8, 4, 96
    env = dict(torch=torch, DEV="cpu", E=E, TOP_K=TOP_K, N_GROUP=N_GROUP, TOPK_GROUP=TOPK_GROUP)
    lift(os.path.join(REF, "research_archive/ds3_acc.py"), ["route_ref"], env)
    g = torch.Generator().manual_seed(20240607)
    logits = torch.randn(T, E, generator=g) * 1.5
    bias = torch.randn(E, generator=g) * 0.05
    # rows with exact ties and with a dominated group, which the tie rule must resolve
    logits[0, :] = 0.25
    logits[1, 10] = logits[1, 200] = 9.0
    logits[2, 32:64] = -30.0
    ids32, w32, gm32, em32 = env["route_ref"](logits, bias, torch.float32)
    ids64, w64, gm64, em64 = env["route_ref"](logits, bias, torch.float64)
    soft = torch.topk(logits, TOP_K, dim=1)
    sw = torch.softmax(logits, dim=1).gather(1, soft.indices)
    sw = sw / sw.sum(1, keepdim=True).clamp(min=1e-30)
    np.savez_compressed(
        os.path.join(HERE, "routing.npz"),
        logits=logits.numpy(), bias=bias.numpy(),
        grouped_ids_sorted_fp32=ids32.numpy().astype(np.int32), grouped_w_sorted_fp32=w32.numpy(),
        grouped_ids_sorted_fp64=ids64.numpy().astype(np.int32),
        group_margin_fp64=gm64.numpy(), expert_margin_fp64=em64.numpy(),
        softmax_ids=soft.indices.numpy().astype(np.int32), softmax_w=sw.numpy(),
        tie_rows=np.array([0, 1], dtype=np.int32),
    )
    print("routing.npz written; fp32/fp64 grouped disagreement tokens:", int((ids32 != ids64).any(1).sum()))


def moe_golden():
    spec = synth.LayerSpec("golden-tiny", hidden=128, inter=128, experts=8, top_k=2)
    layer = synth.make_layer(spec, seed=7, chunk=8, with_shared=False)
    T = 24
    g = torch.Generator().manual_seed(99)
    hs = torch.randn(T, spec.hidden, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, spec.experts, generator=g)
    top = torch.topk(logits, spec.top_k, dim=1)
    tw = torch.softmax(logits, 1).gather(1, top.indices)
    tw = (tw / tw.sum(1, keepdim=True)).float()
    env = dict(torch=torch, DEV="cpu", E=spec.experts, TOP_K=spec.top_k, H_DIM=spec.hidden, K_DIM=spec.hidden,
               N_HALF=spec.inter, N_UP=2 * spec.inter, E_LOCAL=spec.experts // 2)
    lift(os.path.join(REF, "research_archive/ds3_acc.py"), ["dequant", "oracle", "rel_cos", "build_map"], env)
    L = dict(w13=layer["w13"], w13s=layer["w13_scale"], w2=layer["w2"], w2s=layer["w2_scale"])
    ref = env["oracle"](hs, L, top.indices, tw)
    # the same layer split over two expert-parallel ranks, partial sums per rank
    maps = [env["build_map"](r) for r in range(2)]
    parts = []
    for r in range(2):
        lid = maps[r].long()[top.indices]
        gid = torch.where(lid >= 0, top.indices, torch.full_like(top.indices, -1))
        parts.append(env["oracle"](hs, L, gid, tw))
    np.savez_compressed(
        os.path.join(HERE, "moe_tiny.npz"),
        hs_bf16=hs.view(torch.int16).numpy(), logits=logits.numpy(),
        ids=top.indices.numpy().astype(np.int32), weights=tw.numpy(),
        w13=layer["w13"].view(torch.uint8).numpy(), w13_scale=layer["w13_scale"].numpy(),
        w2=layer["w2"].view(torch.uint8).numpy(), w2_scale=layer["w2_scale"].numpy(),
        ref_fp64=ref.numpy(), ref_ep_part0=parts[0].numpy(), ref_ep_part1=parts[1].numpy(),
        ep_map0=maps[0].numpy(), ep_map1=maps[1].numpy(),
    )
    print("moe_tiny.npz written; |ref| rms", float(ref.pow(2).mean().sqrt()),
          "EP parts sum error", float((parts[0] + parts[1] - ref).abs().max()))


SLAB_SPEC = dict(hidden=2048, inter=512, experts=4, top_k=2)   # the Qwen layer's slab counts: 16 K slabs up, 4 down
SLAB_SEED, SLAB_TOKENS = 11, 48


def slab_case():
    """Inputs of the slab-count golden case, rebuilt from seeds (the 12 MB of weights are not stored)."""
    spec = synth.LayerSpec("golden-slabs", **SLAB_SPEC)
    layer = synth.make_layer(spec, seed=SLAB_SEED, chunk=4, with_shared=False)
    g = torch.Generator().manual_seed(1234)
    hs = torch.randn(SLAB_TOKENS, spec.hidden, generator=g).to(torch.bfloat16)
    logits = torch.randn(SLAB_TOKENS, spec.experts, generator=g)
    top = torch.topk(logits, spec.top_k, dim=1)
    tw = torch.softmax(logits, 1).gather(1, top.indices)
    tw = (tw / tw.sum(1, keepdim=True)).float()
    return spec, layer, hs, top.indices, tw


def moe_slab_golden():
    """The reference's fp64 oracle on a case with the real layer's slab counts (K = 2048, I = 512), so that the
    path-faithful tier can be held to the accuracy band the reference publishes for its kernel."""
    spec, layer, hs, ids, tw = slab_case()
    env = dict(torch=torch, DEV="cpu", E=spec.experts, TOP_K=spec.top_k, H_DIM=spec.hidden, K_DIM=spec.hidden,
               N_HALF=spec.inter, N_UP=2 * spec.inter, E_LOCAL=spec.experts)
    lift(os.path.join(REF, "research_archive/ds3_acc.py"), ["dequant", "oracle", "rel_cos"], env)
    L = dict(w13=layer["w13"], w13s=layer["w13_scale"], w2=layer["w2"], w2s=layer["w2_scale"])
    ref = env["oracle"](hs, L, ids, tw)
    digest = int(layer["w13"].view(torch.uint8).long().sum() * 31 + layer["w2"].view(torch.uint8).long().sum())
    np.savez_compressed(os.path.join(HERE, "moe_slabs.npz"), ref_fp64=ref.numpy(), ids=ids.numpy().astype(np.int32),
                        weights=tw.numpy(), hs_bf16=hs.view(torch.int16).numpy(), weight_digest=np.int64(digest),
                        w13_scale=layer["w13_scale"].numpy(), w2_scale=layer["w2_scale"].numpy())
    print("moe_slabs.npz written; |ref| rms", float(ref.pow(2).mean().sqrt()))


def e4m3_golden():
    codes = torch.arange(256, dtype=torch.uint8)
    dec = codes.view(torch.float8_e4m3fn).float()
    g = torch.Generator().manual_seed(5)
    x = torch.cat([torch.randn(4000, generator=g) * s for s in (300.0, 20.0, 1.0, 0.05, 0.004)]
                  + [torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 0.0146, 0.015625])])
    enc = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    np.savez_compressed(os.path.join(HERE, "e4m3.npz"), decode=dec.numpy(), x=x.numpy(), encode=enc.numpy())
    print("e4m3.npz written")


if __name__ == "__main__":
    if REF is None:
        raise SystemExit("usage: make_golden.py <path of a checkout of the reference repository>")
    routing_golden()
    moe_golden()
    moe_slab_golden()
    e4m3_golden()
