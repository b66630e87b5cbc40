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
