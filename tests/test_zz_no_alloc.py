"""The allocation-free entry point, launch_prefill_moe_noalloc, against the ordinary one.

It exists for hosts that cannot get device memory at call time (an engine that has given all of
HBM to its KV-cache pool, or a caller that cannot afford the device-wide synchronisation inside
cudaMalloc): the kernel's scratch sits in a fixed array inside the library, so the batch is capped.
Two calls in a row must both reproduce the ordinary entry point's output (the array keeps the first
call's contents), and a batch beyond the cap must be refused with -130 before anything is launched.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes

import pytest
import torch

from unimonomoe_b200 import MonoKernel, synth, variant_path

pytestmark = pytest.mark.gpu


def test_noalloc_entry_matches_ordinary_entry_twice_in_a_row():
    dev = "cuda:0"
    mk = MonoKernel(variant_path("qwen_w1"))
    lib = mk.lib
    lib.launch_prefill_moe_noalloc.restype = ctypes.c_int
    cap = int(lib.prefill_wgmma_noalloc_max_tokens())
    assert cap >= 64
    layer = synth.make_layer(synth.QWEN, seed=3, device=dev, with_shared=False)
    vp = ctypes.c_void_p

    def noalloc(batch, out):
        return lib.launch_prefill_moe_noalloc(
            vp(batch["logits"].data_ptr()), batch["hs"].shape[0], vp(batch["hs"].data_ptr()),
            vp(layer["w13"].data_ptr()), vp(layer["w13_scale"].data_ptr()), vp(layer["w2"].data_ptr()),
            vp(layer["w2_scale"].data_ptr()), vp(out.data_ptr()), vp(0), vp(0),
            vp(torch.cuda.current_stream().cuda_stream))

    for call, T in enumerate((cap, 77)):          # two calls in a row, the second on a smaller batch
        batch = synth.make_batch(synth.QWEN, layer, T, seed=10 + call, device=dev)
        ref = mk.prefill(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"],
                         layer["w2_scale"], check=True)
        out = torch.full((T, 2048), float("nan"), dtype=torch.bfloat16, device=dev)
        assert noalloc(batch, out) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        # same kernel, same inputs: the tolerance of the parity tests (max|err| <= 2e-2 rms, cos >= 0.9995)
        # is met with room to spare -- the outputs are in fact identical bit for bit
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    # beyond the cap: refused before any launch, output untouched
    T = cap + 1
    batch = synth.make_batch(synth.QWEN, layer, T, seed=12, device=dev)
    out = torch.full((T, 2048), 5.0, dtype=torch.bfloat16, device=dev)
    assert noalloc(batch, out) == -130
    torch.cuda.synchronize()
    assert (out == 5.0).all()


def _noalloc_call(mk, layer, batch, out, bias=None, emap=None):
    vp = ctypes.c_void_p
    mk.lib.launch_prefill_moe_noalloc.restype = ctypes.c_int
    return mk.lib.launch_prefill_moe_noalloc(
        vp(batch["logits"].data_ptr()), batch["hs"].shape[0], vp(batch["hs"].data_ptr()),
        vp(layer["w13"].data_ptr()), vp(layer["w13_scale"].data_ptr()), vp(layer["w2"].data_ptr()),
        vp(layer["w2_scale"].data_ptr()), vp(out.data_ptr()), vp(0 if bias is None else bias.data_ptr()),
        vp(0 if emap is None else emap.data_ptr()), vp(torch.cuda.current_stream().cuda_stream))


def _noalloc_status(mk):
    """The status words of the last allocation-free launch, through the accessor made for that purpose."""
    words = torch.zeros(4, dtype=torch.int32).pin_memory()
    mk.lib.prefill_wgmma_noalloc_status.restype = ctypes.c_int
    rc = mk.lib.prefill_wgmma_noalloc_status(ctypes.c_void_p(words.data_ptr()),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, words.tolist()


@pytest.mark.parametrize("variant", ["qwen_ep4", "ds_tp8"])
def test_noalloc_entry_on_other_builds_allocates_nothing_and_reports_status(variant):
    """An expert-parallel build (with its expert map) and the H = 7168 build at its cap of 64 tokens: same output
    bytes as the ordinary entry, the free device memory unchanged across the call, and the status words of the
    launch readable although its workspace is inside the library."""
    dev = "cuda:0"
    mk = MonoKernel(variant_path(variant))
    cap = int(mk.lib.prefill_wgmma_noalloc_max_tokens())
    if variant == "qwen_ep4":
        spec, kw, emap = synth.QWEN, {"expert_slice": (64, 128)}, synth.expert_map(synth.QWEN, 1, 4, device=dev)
        assert cap == 256
    else:
        spec, kw, emap = synth.DEEPSEEK, {"inter_slice": (0, 256), "chunk": 8}, None
        assert cap == 64
    layer = synth.make_layer(spec, seed=3, device=dev, with_shared=False, **kw)
    batch = synth.make_batch(spec, layer, cap, seed=21, device=dev)
    ref = mk.prefill(batch["hs"], batch["logits"], layer["w13"], layer["w13_scale"], layer["w2"], layer["w2_scale"],
                     e_score_correction_bias=layer["bias"], expert_map=emap, check=True)
    out = torch.full((cap, spec.hidden), float("nan"), dtype=torch.bfloat16, device=dev)
    assert _noalloc_call(mk, layer, batch, out, layer["bias"], emap) == 0      # first call: resolves the array's address
    torch.cuda.synchronize()
    out.fill_(float("nan"))
    free_before = torch.cuda.mem_get_info()[0]
    stats_before = torch.cuda.memory_stats()["allocation.all.current"]
    assert _noalloc_call(mk, layer, batch, out, layer["bias"], emap) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_stats()["allocation.all.current"] == stats_before
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    rc, words = _noalloc_status(mk)
    assert rc == 0 and words[0] == 0 and words[1] == 0, (rc, words)
