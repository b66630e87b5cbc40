"""The vLLM glue on CPU: load-time eligibility against real binaries' compiled geometry (tensors on the meta
device, so no weights are materialised), the expert-map proof, and the reduce-once bookkeeping with a fake plan."""
import types

import pytest
import torch

from unimonomoe_b200 import MonoKernel, synth, vllm_plugin as vp


def _layer(n_local=256, n_up=1024, k=2048, h=2048, n_half=512, n_global=256, top_k=8, scoring="softmax", bias=None,
           emap=None):
    m = lambda *s: torch.empty(*s, dtype=torch.uint8, device="meta")  # noqa: E731
    f = lambda *s: torch.empty(*s, dtype=torch.float32, device="meta")  # noqa: E731
    return types.SimpleNamespace(
        w13_weight=m(n_local, n_up, k), w2_weight=m(n_local, h, n_half),
        w13_weight_scale_inv=f(n_local, n_up // 128, k // 128), w2_weight_scale_inv=f(n_local, h // 128, n_half // 128),
        top_k=top_k, global_num_experts=n_global, scoring_func=scoring, e_score_correction_bias=bias, expert_map=emap,
        renormalize=True)


def test_eligibility_follows_the_compiled_geometry(built_libs, monkeypatch):
    monkeypatch.delenv(vp.ENV_ENABLE, raising=False)
    mk = MonoKernel(built_libs["qwen_w1"])
    assert vp.check_layer(mk, _layer()).ok
    e = vp.check_layer(mk, _layer(n_half=256, n_up=512))
    assert not e.ok and any("n_half: binary 512, layer 256" in r for r in e.reasons) and any("n_up" in r for r in e.reasons)
    assert not vp.check_layer(mk, _layer(top_k=4)).ok
    assert not vp.check_layer(mk, _layer(scoring="sigmoid", bias=torch.zeros(256))).ok
    assert "cannot apply" in " ".join(vp.check_layer(mk, _layer(bias=torch.zeros(256))).reasons)
    assert not vp.check_layer(mk, _layer(), block_quant=False).ok
    assert not vp.check_layer(mk, _layer(), raw_block_fp8_backend=False).ok
    bad_scales = _layer()
    bad_scales.w13_weight_scale_inv = torch.empty(256, 1024, device="meta")
    assert "w13 scales" in " ".join(vp.check_layer(mk, bad_scales).reasons)
    monkeypatch.setenv(vp.ENV_ENABLE, "0")
    assert vp.check_layer(mk, _layer()).reasons == [f"{vp.ENV_ENABLE}=0"]
    monkeypatch.delenv(vp.ENV_ENABLE)
    ds = MonoKernel(built_libs["ds_tp8"])
    ok = vp.check_layer(ds, _layer(n_up=512, k=7168, h=7168, n_half=256, scoring="sigmoid", bias=torch.ones(256)))
    assert ok.ok and ok.bias is not None and not ok.expert_parallel
    assert not vp.check_layer(ds, _layer(n_up=512, k=7168, h=7168, n_half=256, scoring="sigmoid")).ok   # no bias
    assert not vp.check_layer(ds, _layer(n_up=512, k=7168, h=7168, n_half=256, scoring="softmax")).ok


def test_expert_map_has_to_be_proven(built_libs):
    ep = MonoKernel(built_libs["qwen_ep4"])
    good = synth.expert_map(synth.QWEN, 2, 4)
    e = vp.check_layer(ep, _layer(n_local=64, emap=good))
    assert e.ok and e.expert_parallel
    mask = (good >= 0).to(torch.int32)                      # a 0/1 ownership mask: same dtype, same length
    assert "not a global-to-local map" in " ".join(vp.check_layer(ep, _layer(n_local=64, emap=mask)).reasons)
    assert "int32" in " ".join(vp.check_layer(ep, _layer(n_local=64, emap=good.long())).reasons)
    assert "no expert_map" in " ".join(vp.check_layer(ep, _layer(n_local=64)).reasons)
    dup = good.clone()
    dup[dup == 5] = 6
    assert vp.check_expert_map(dup, 256, 64) is not None
    assert vp.check_expert_map(good[:128], 256, 64) is not None
    # the two ways build and weights can disagree about expert parallelism
    assert "every expert" in " ".join(vp.check_layer(ep, _layer(emap=good)).reasons)
    full = MonoKernel(built_libs["qwen_w1"])
    assert "not an expert-parallel build" in " ".join(vp.check_layer(full, _layer(n_local=64, emap=good)).reasons)


class _FakePlan:
    def __init__(self, usable=True, fold=True):
        self.usable, self.fold_shared, self.slots, self.calls = usable, fold, set(), 0

    def output_is_fused(self, t):
        return id(t) in self.slots

    def fused_tp_launch(self, *a, **kw):
        self.calls += 1
        return None


def _glue(built_libs, plan):
    g = vp.MonokernelGlue(MonoKernel(built_libs["qwen_w1"]), _layer())
    g.plan, g.tp_size = plan, 4
    return g


def test_reduce_once_bookkeeping(built_libs):
    reduces = []

    def all_reduce(t):
        reduces.append(t)
        return t * 4          # four ranks holding the same partial sum

    routed, shared = torch.ones(3, 4), torch.full((3, 4), 0.5)
    # 1. the output came out of the in-kernel reduce with the shared half folded in: nothing left to do
    plan = _FakePlan()
    g = _glue(built_libs, plan)
    plan.slots.add(id(routed))
    s, r = g.finish(routed, shared, True, 2.5, all_reduce)
    assert s is None and r is routed and not reduces
    # 2. the same output although no shared half was offered cannot happen: refuse to continue
    with pytest.raises(RuntimeError):
        g.finish(routed, shared, False, 2.5, all_reduce)
    # 3. the ordinary launch at a size the in-kernel reduce declines: scale, add the shared half, ONE reduce
    plan.slots.clear()
    s, r = g.finish(routed, shared, True, 2.5, all_reduce)
    assert s is None and len(reduces) == 1 and torch.equal(r, (routed * 2.5 + shared) * 4)
    # 4. no fold agreed: the routed half is reduced alone, the shared half goes back to the caller
    reduces.clear()
    g = _glue(built_libs, _FakePlan(fold=False))
    s, r = g.finish(routed, shared, False, 2.5, all_reduce)
    assert s is shared and len(reduces) == 1 and torch.equal(r, routed * 4)
    # 5. the plan is not usable: this path promises nothing, the caller reduces as always
    reduces.clear()
    g = _glue(built_libs, _FakePlan(usable=False))
    assert not g.output_is_reduced() and not g.folds_shared_output()
    s, r = g.finish(routed, shared, False, 2.5, all_reduce)
    assert s is shared and r is routed and not reduces


def test_calls_decline_or_fall_back_without_raising(built_libs):
    g = vp.MonokernelGlue(MonoKernel(built_libs["qwen_w1"]), _layer())
    assert g.eligibility.ok and not g.fused_tp_eligible() and g.plan is None
    layer = _layer()
    x = torch.zeros(8, 2048, dtype=torch.bfloat16)
    # on a machine without CUDA the launch raises; the ordinary launch turns that into "declined"
    if not torch.cuda.is_available():
        assert g.try_moe_monokernel(layer, x, torch.zeros(8, 256)) is None
    big = torch.empty(40000, 2048, dtype=torch.bfloat16, device="meta")
    assert g.try_moe_monokernel(layer, big, None) is None          # above the token cap
    bad = vp.MonokernelGlue(MonoKernel(built_libs["qwen_w1"]), _layer(top_k=4))
    assert bad.try_moe_monokernel(layer, x, torch.zeros(8, 256)) is None
    # with the fold agreed, a call that has no shared half to offer must not enter the in-kernel reduce
    plan = _FakePlan()
    g.plan, g.tp_size = plan, 4
    if not torch.cuda.is_available():
        assert g.try_moe_monokernel(layer, x, torch.zeros(8, 256), residual=None) is None
        assert plan.calls == 0
        g.try_moe_monokernel(layer, x, torch.zeros(8, 256), residual=torch.zeros(8, 2048, dtype=torch.bfloat16))
        assert plan.calls == 1


def test_install_needs_a_binary(monkeypatch):
    monkeypatch.delenv("VLLM_PREFILL_MONOKERNEL_SO", raising=False)
    with pytest.raises(RuntimeError, match="no kernel binary"):
        vp.install()


def test_install_attaches_the_hooks_to_the_installed_vllm(built_libs):
    """With vLLM importable, install() gives its Fp8MoEMethod the three names the reference's runner looks up;
    a quant method whose layer was never checked declines."""
    pytest.importorskip("vllm")
    try:
        from vllm.model_executor.layers.quantization.fp8 import Fp8MoEMethod
    except Exception as exc:
        pytest.skip(f"this vLLM has no Fp8MoEMethod: {exc}")
    before = Fp8MoEMethod.process_weights_after_loading
    try:
        assert vp.install(built_libs["qwen_w1"]) is True
        for name in ("try_moe_monokernel", "monokernel_output_is_reduced", "monokernel_folds_shared_output"):
            assert callable(getattr(Fp8MoEMethod, name))
        assert Fp8MoEMethod.process_weights_after_loading is not before
        bare = object.__new__(Fp8MoEMethod)
        assert bare.try_moe_monokernel(None, None, None) is None
        assert bare.monokernel_output_is_reduced() is False and bare.monokernel_folds_shared_output() is False
    finally:
        Fp8MoEMethod.process_weights_after_loading = before
        for name in ("try_moe_monokernel", "monokernel_output_is_reduced", "monokernel_folds_shared_output"):
            if name in Fp8MoEMethod.__dict__:
                delattr(Fp8MoEMethod, name)
