"""C-ABI surface and host logic, CPU only: the libraries load without a GPU driver, export
every symbol include/prefill_mono.h declares, report the geometry they were built for, and
decline bad calls with the reference's return codes before any CUDA call."""
import ctypes
import os
import re

import pytest
import torch

from unimonomoe_b200 import MonoKernel, build, loader, synth, variant_path

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "prefill_mono.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:launch_prefill_moe_wgmma|prefill_wgmma)\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(built_libs):
    names = declared_symbols()
    assert len(names) >= 40
    for variant, path in built_libs.items():
        lib = ctypes.CDLL(path)
        missing = [n for n in names if not hasattr(lib, n)]
        assert not missing, (variant, missing)


@pytest.mark.parametrize("variant", list(build.VARIANTS))
def test_geometry_readback(built_libs, variant):
    g = build.VARIANTS[variant]
    geo = MonoKernel(built_libs[variant]).geometry()
    assert geo["k_dim"] == g["K"] and geo["h_dim"] == g["H"]
    assert geo["n_half"] == g["N_HALF"] and geo["n_up"] == 2 * g["N_HALF"]
    assert geo["num_experts"] == 256 and geo["num_experts_local"] == g["E_LOCAL"]
    assert geo["ep_capable"] == int(g["E_LOCAL"] != 256)
    assert geo["router_mode"] == g["MODE"] and geo["top_k"] == 8 and geo["fused_renorm"] == 1
    assert geo["grid_size"] == 148 and geo["block_m"] == 128 and geo["arch"] == 100
    assert geo["shm_total"] <= 227 * 1024
    assert geo["a_stages"] >= 2 and geo["up_pipe"] >= 2
    assert geo["workspace_bytes"] >= 148 * 256 * 4


def _args(n_tokens=16, ws_bytes=None, null=None, extra=()):
    """Argument list with small dummy host buffers: every call below must be declined before
    the library touches CUDA, so the pointers are never dereferenced."""
    buf = (ctypes.c_char * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    a = [p, ctypes.c_int(n_tokens), ctypes.c_int(128), p, ctypes.c_size_t(1 << 20 if ws_bytes is None else ws_bytes)]
    a += [p] * 12
    if null is not None:
        a[null] = ctypes.c_void_p(0)
    return a + list(extra) + [ctypes.c_void_p(0)], buf


def test_pre_launch_return_codes(built_libs):
    lib = MonoKernel(built_libs["qwen_w1"]).lib
    a, keep = _args(ws_bytes=16)
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -100
    a, keep = _args(null=3)
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -100
    a, keep = _args(n_tokens=0)
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -101
    a, keep = _args(n_tokens=80000)
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -102
    for idx in (0, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16):
        a, keep = _args(null=idx)
        assert lib.launch_prefill_moe_wgmma_q1(*a) == -104, idx
    # fused tensor-parallel argument checks
    vp, ci = ctypes.c_void_p, ctypes.c_int
    buf = (ctypes.c_char * 64)()
    p = ctypes.cast(buf, vp)

    def tp(nchunk, ncomm, rank, world, pads=p, n_tokens=16):
        a, k = _args(n_tokens=n_tokens, extra=[vp(0), p, pads, ci(rank), ci(world), ci(nchunk), ci(ncomm),
                                               ctypes.c_uint(0), vp(0)])
        return lib.launch_prefill_moe_wgmma_q1_tp(*a)

    assert tp(0, 4, 0, 2) == -110
    assert tp(17, 4, 0, 2) == -110
    assert tp(4, 148, 0, 2) == -111
    assert tp(4, 4, 2, 2) == -112
    assert tp(4, 4, 0, 2, pads=vp(0)) == -113
    assert tp(3, 4, 0, 2, n_tokens=1) == -114  # 1*2048 elements do not split into 3 chunks of whole 16-byte units
    # a map handed to a build without expert parallelism
    a, keep = _args(extra=[vp(0), p])
    assert lib.launch_prefill_moe_wgmma_q1_ep(*a) == -121
    # the entry with the router linear inside: weight and logits buffer are both required, and the
    # remaining arguments are checked like those of the other entries
    lib.prefill_wgmma_has_router_gemv.restype = ctypes.c_int
    assert lib.prefill_wgmma_has_router_gemv() == 1
    tail = [vp(0), vp(0), vp(0), ci(0), ci(1), ci(1), ci(0), ctypes.c_uint(0), vp(0), vp(0), ctypes.c_float(1.0), vp(0)]

    def gemv(rw, lg, **kw):
        a, k = _args(extra=tail, **kw)
        return lib.launch_prefill_moe_wgmma_q1_gemv(rw, lg, *a[1:])

    assert gemv(vp(0), p) == -105
    assert gemv(p, vp(0)) == -105
    assert gemv(p, p, n_tokens=0) == -101
    assert gemv(p, p, ws_bytes=16) == -100


def test_expert_parallel_build_declines_without_map(built_libs):
    lib = MonoKernel(built_libs["qwen_ep4"]).lib
    a, keep = _args()
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -120          # the pre-existing ABI forwards a null map
    a, keep = _args(extra=[ctypes.c_void_p(0), ctypes.c_void_p(0)])
    assert lib.launch_prefill_moe_wgmma_q1_ep(*a) == -120
    # order of the checks as in the reference (kernel/qwen_ep/src/prefill_mono_final_nb.cu:1650-1660): the
    # workspace first, then the map against the build, then the token count
    a, keep = _args(ws_bytes=16)
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -100
    a, keep = _args(n_tokens=0)
    assert lib.launch_prefill_moe_wgmma_q1(*a) == -120


def test_plan_symbols_without_a_device(built_libs):
    """The plan step needs a driver to encode descriptors; without one it must fail with a code, not crash,
    and the look-up statistics must be readable."""
    lib = MonoKernel(built_libs["qwen_w1"]).lib
    lib.prefill_wgmma_plan_prepare.restype = ctypes.c_int
    assert lib.prefill_wgmma_plan_prepare(ctypes.c_void_p(0), ctypes.c_void_p(0)) == -104
    hits, misses = ctypes.c_ulonglong(7), ctypes.c_ulonglong(7)
    lib.prefill_wgmma_plan_stats(ctypes.byref(hits), ctypes.byref(misses))
    assert hits.value == 0
    lib.prefill_wgmma_plan_reset()


def test_pad_words_and_caps(built_libs):
    mk = MonoKernel(built_libs["ds_tp8"])
    assert mk.tp_pad_words(8, 14, 8) == (8 * 14 + 1) * 8
    caps = mk.tp_caps()
    assert caps["usable"] and caps["has_tp_residual"] and caps["tp_max_c"] == 16 and caps["tp_mm"] == 8
    assert caps["tp_has_devseq"] == 1 and caps["tp_seq_bytes"] == 4


def test_loader_refuses_unset_binary(monkeypatch):
    monkeypatch.delenv("VLLM_PREFILL_MONOKERNEL_SO", raising=False)
    loader._reset_prefill_monokernel()
    with pytest.raises(RuntimeError, match="VLLM_PREFILL_MONOKERNEL_SO is not set"):
        loader.prefill_monokernel_geometry()
    monkeypatch.setenv("VLLM_PREFILL_MONOKERNEL_SO", variant_path("qwen_tp4"))
    loader._reset_prefill_monokernel()
    assert loader.prefill_monokernel_geometry()["n_half"] == 128
    loader._reset_prefill_monokernel()


def test_validate_checks_every_compiled_dimension(built_libs):
    mk = MonoKernel(built_libs["qwen_tp4"])
    x = torch.zeros(4, 2048, dtype=torch.bfloat16)
    w13 = torch.zeros(256, 256, 2048, dtype=torch.uint8)
    w2 = torch.zeros(256, 2048, 128, dtype=torch.uint8)
    assert mk.validate(x, w13, w2, 8, None) is None
    with pytest.raises(RuntimeError, match=r"N_UP\): compiled 256, got 512"):
        mk.validate(x, torch.zeros(256, 512, 2048, dtype=torch.uint8), w2, 8, None)
    with pytest.raises(RuntimeError, match=r"N_HALF\): compiled 128, got 256"):
        mk.validate(x, w13, torch.zeros(256, 2048, 256, dtype=torch.uint8), 8, None)
    with pytest.raises(RuntimeError, match=r"K_DIM\): compiled 2048, got 1024"):
        mk.validate(torch.zeros(4, 1024, dtype=torch.bfloat16), w13, w2, 8, None)
    with pytest.raises(RuntimeError, match=r"E_LOCAL\): compiled 256, got 64"):
        mk.validate(x, w13[:64], w2[:64], 8, None)
    with pytest.raises(RuntimeError, match=r"TOP_K\): compiled 8, got 4"):
        mk.validate(x, w13, w2, 4, None)
    with pytest.raises(RuntimeError, match="softmax"):
        mk.validate(x, w13, w2, 8, torch.zeros(256))
    with pytest.raises(RuntimeError, match="not an expert-parallel build"):
        mk.validate(x, w13, w2, 8, None, torch.zeros(256, dtype=torch.int32))
    ds = MonoKernel(built_libs["ds_tp8"])
    xd = torch.zeros(4, 7168, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="sigmoid"):
        ds.validate(xd, torch.zeros(256, 512, 7168, dtype=torch.uint8), torch.zeros(256, 7168, 256, dtype=torch.uint8), 8, None)
    ep = MonoKernel(built_libs["qwen_ep4"])
    w13e = torch.zeros(64, 1024, 2048, dtype=torch.uint8)
    w2e = torch.zeros(64, 2048, 512, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="no expert_map given"):
        ep.validate(x, w13e, w2e, 8, None)
    with pytest.raises(RuntimeError, match="int32"):
        ep.validate(x, w13e, w2e, 8, None, torch.zeros(256, dtype=torch.int64))
    assert ep.validate(x, w13e, w2e, 8, None, synth.expert_map(synth.QWEN, 1, 4)) is None


def test_no_cpu_fallback(built_libs):
    mk = MonoKernel(built_libs["qwen_tp4"])
    x = torch.zeros(4, 2048, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        mk.prefill(x, torch.zeros(4, 256), torch.zeros(256, 256, 2048, dtype=torch.uint8), torch.zeros(256, 2, 16),
                   torch.zeros(256, 2048, 128, dtype=torch.uint8), torch.zeros(256, 16, 1))


def test_synthetic_shards_are_slices_of_one_layer():
    spec = synth.LayerSpec("t", hidden=256, inter=256, experts=8, top_k=2)
    full = synth.make_layer(spec, seed=3, chunk=4, with_shared=False)
    tp1 = synth.make_layer(spec, seed=3, chunk=4, with_shared=False, inter_slice=(128, 256))
    assert torch.equal(tp1["w13"].view(torch.uint8)[:, :128], full["w13"].view(torch.uint8)[:, 128:256])
    assert torch.equal(tp1["w13"].view(torch.uint8)[:, 128:], full["w13"].view(torch.uint8)[:, 384:512])
    assert torch.equal(tp1["w2"].view(torch.uint8), full["w2"].view(torch.uint8)[:, :, 128:256])
    assert torch.equal(tp1["w13_scale"], full["w13_scale"][:, [1, 3]])
    assert torch.equal(tp1["w2_scale"], full["w2_scale"][:, :, 1:2])
    ep1 = synth.make_layer(spec, seed=3, chunk=4, with_shared=False, expert_slice=(2, 6))
    assert torch.equal(ep1["w13"].view(torch.uint8), full["w13"].view(torch.uint8)[2:6])
    m = synth.expert_map(spec, 1, 2)
    assert m.tolist() == [-1, -1, -1, -1, 0, 1, 2, 3]


def test_router_weight_preparation():
    """The in-kernel router takes the gate weight in bf16: a weight that is bf16-representable converts
    exactly (the checkpoints' case), anything else is refused instead of silently changing the logits."""
    from unimonomoe_b200.loader import prepare_router_weight
    w = (torch.randn(256, 64) * 0.02).to(torch.bfloat16)
    out = prepare_router_weight(w.float())
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and torch.equal(out, w)
    assert prepare_router_weight(w) is not None
    with pytest.raises(ValueError):
        prepare_router_weight(torch.randn(256, 64) * 0.02)


def test_token_cap_is_enforced_before_any_cuda_call(built_libs, monkeypatch):
    """More tokens than the cap (30720, the reference's MOE_MONOKERNEL_PREFILL_MAX_TOKENS) are refused by
    the host module; the library's own bound on the tile list (-102) sits above it."""
    mk = MonoKernel(built_libs["qwen_w1"])
    assert loader.MOE_MONOKERNEL_PREFILL_MAX_TOKENS == 30720
    assert (30720 * 8 // 128 + 256) <= mk.geometry()["max_tiles"]
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)

    class FakeCuda(torch.Tensor):
        is_cuda = True

    x = torch.empty(30721, 2048, dtype=torch.bfloat16).as_subclass(FakeCuda)
    with pytest.raises(RuntimeError, match="refuses 30721 tokens"):
        mk.prefill_impl(x, None, None, None, torch.empty(256, 2048, 512), None, 8, True, None, None)


def test_scratch_arena_grows_and_never_frees(built_libs):
    """The scratch of a launch comes from one grow-only arena per device: smaller batches are views of it, a
    larger batch adds a larger arena, and the outgrown one stays alive (a captured graph may hold its addresses)."""
    mk = MonoKernel(built_libs["qwen_tp4"])
    a = mk.scratch(100, "cpu")
    b = mk.scratch(50, "cpu")
    assert a["workspace"].data_ptr() == b["workspace"].data_ptr()
    assert a["act_fp8"].data_ptr() == b["act_fp8"].data_ptr() and b["act_fp8"].shape == (50, 2048)
    assert b["partial"].shape == (50 * 9, 2048) and b["sorted_ids"].shape == (400,)   # top_k rows + one shared-expert row
    assert mk.scratch(50, "cpu") is b                      # the views of a size are made once
    old_ptr = a["partial"].data_ptr()
    for m in (60, 70, 80, 90, 100, 30):                    # more sizes than any small cache would hold
        assert mk.scratch(m, "cpu")["partial"].data_ptr() == old_ptr
    c = mk.scratch(200, "cpu")
    assert c["partial"].data_ptr() != old_ptr and c["partial"].shape == (1800, 2048)
    assert len(mk._retired) == 1 and mk._retired[0]["buffers"]["partial"].data_ptr() == old_ptr
    assert mk.scratch(100, "cpu")["partial"].data_ptr() == c["partial"].data_ptr()   # later calls use the larger arena
    assert a["partial"].data_ptr() == old_ptr              # what was handed out earlier is still the same memory


def test_shared_expert_entry_declines_bad_arguments(built_libs):
    """launch_prefill_moe_wgmma_q1_shared: a missing shared-expert tensor, a gate without its scratch and an
    impossible token split are refused with -109 before any CUDA call; the two-CTA build refuses with -108."""
    vp, ci = ctypes.c_void_p, ctypes.c_int
    buf = (ctypes.c_char * 64)()
    p = ctypes.cast(buf, vp)
    tail = [vp(0), vp(0), vp(0), ci(0), ci(1), ci(1), ci(0), ctypes.c_uint(0), vp(0), vp(0), ctypes.c_float(1.0), vp(0)]

    def call(lib, up=p, ups=p, dn=p, dns=p, gate=vp(0), gsc=vp(0), part=0, parts=1, **kw):
        a, keep = _args(extra=tail + [up, ups, dn, dns, gate, gsc, ci(part), ci(parts)], **kw)
        lib.launch_prefill_moe_wgmma_q1_shared.restype = ctypes.c_int
        return lib.launch_prefill_moe_wgmma_q1_shared(*a)

    lib = MonoKernel(built_libs["qwen_w1"]).lib
    lib.prefill_wgmma_has_shared_expert.restype = ctypes.c_int
    assert lib.prefill_wgmma_has_shared_expert() == 1
    assert call(lib, up=vp(0)) == -109
    assert call(lib, dns=vp(0)) == -109
    assert call(lib, gate=p, gsc=vp(0)) == -109
    assert call(lib, part=4, parts=4) == -109 and call(lib, parts=0) == -109
    assert call(lib, ws_bytes=16) == -100 and call(lib, n_tokens=0) == -101
    pair = MonoKernel(built_libs["qwen_w1_pair"]).lib
    pair.prefill_wgmma_has_shared_expert.restype = ctypes.c_int
    assert pair.prefill_wgmma_has_shared_expert() == 0
    assert call(pair) == -108


def _reference_checkout():
    """A checkout of the reference repository, when one is at hand: $REFERENCE_CHECKOUT, or a directory named
    `reference` beside this repository. Only CPU tests in the build container use it."""
    cand = os.environ.get("REFERENCE_CHECKOUT") or os.path.join(os.path.dirname(ROOT), "reference")
    return cand if os.path.isfile(os.path.join(cand, "validation", "geo_readback.py")) else None


@pytest.mark.skipif(_reference_checkout() is None, reason="no checkout of the reference at hand")
def test_the_references_own_readback_script_accepts_every_binary(built_libs):
    """validation/geo_readback.py of the reference, unmodified, run against each binary built here: every
    accessor it asks for is present and reports this build's geometry, and both expert-parallel entry points exist."""
    import subprocess
    import sys
    script = os.path.join(_reference_checkout(), "validation", "geo_readback.py")
    for variant, path in built_libs.items():
        r = subprocess.run([sys.executable, script, path], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, (variant, r.stderr[-500:])
        assert "ABSENT" not in r.stdout, (variant, r.stdout)
        got = dict(line.split()[:2] for line in r.stdout.splitlines()[1:] if len(line.split()) >= 2)
        g = build.VARIANTS[variant]
        assert int(got["k_dim"]) == g["K"] and int(got["h_dim"]) == g["H"] and int(got["n_half"]) == g["N_HALF"]
        assert int(got["num_experts_local"]) == g["E_LOCAL"] and int(got["router_mode"]) == g["MODE"]
        assert int(got["grid_size"]) == 148 and int(got["tp_has_residual"]) == 1 and int(got["tp_has_devseq"]) == 1
        assert got["q1_ep"] == "present" and got["q1_ep2"] == "present"
        assert int(got["workspace_bytes"]) == MonoKernel(path).geometry()["workspace_bytes"]
