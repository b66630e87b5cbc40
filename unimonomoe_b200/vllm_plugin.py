"""Glue between a vLLM FP8 fused-MoE layer and the prefill kernel: the part of the reference that lives in
vLLM's quant method and MoE runner, as a module that can be installed into a stock vLLM instead of a patch.

What the reference does there, restated here:

* at weight-load time, decide once whether this layer may use the kernel: the compiled geometry of the
  loaded binary must equal the layer's in every dimension, the router rule must be the binary's, and under
  expert parallelism the layer's `expert_map` must be proven to be a global-to-local map of exactly the
  experts whose weights are resident (quantization/fp8.py:755-966);
* per call, offer the batch to the kernel before the router runs (the kernel routes itself), decline above
  the token cap, fall back on a launch error for the ordinary launch but never for the launch whose reduce
  runs inside the kernel (quantization/fp8.py:1090-1176);
* reduce-once bookkeeping: an output that came back from the in-kernel reduce is already summed over the
  tensor-parallel group and, when the shared expert's output was folded in, already contains it; anything else
  still needs `routed * scale + shared` and one all-reduce (fused_moe/runner/moe_runner.py:832-1008).

`MonokernelGlue` works on duck-typed objects (a layer with `w13_weight`, `w2_weight`, their scales, `top_k`,
`global_num_experts`, `expert_map`, `scoring_func`, `e_score_correction_bias`), so it is testable without
vLLM. `install()` attaches it to vLLM's `Fp8MoEMethod` when vLLM is importable.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from . import tp_fused
from .loader import MOE_MONOKERNEL_PREFILL_MAX_TOKENS, MonoKernel

logger = logging.getLogger("unimonomoe_b200.vllm")
ENV_ENABLE = "VLLM_USE_MOE_MONOKERNEL"          # default on; "0" forces vLLM's own fused-MoE path
ENV_FUSE_TP = "VLLM_PREFILL_MONOKERNEL_TP_FUSE"  # default on; "0" keeps the all-reduce outside the kernel


def _env_on(name: str) -> bool:
    return os.environ.get(name, "1").strip().lower() not in ("0", "false", "no", "off")


@dataclass
class Eligibility:
    """Outcome of the load-time check. `reasons` is empty exactly when `ok`."""
    ok: bool
    reasons: list = field(default_factory=list)
    expert_parallel: bool = False
    bias: Optional[torch.Tensor] = None


def _scale_of(layer, which: str, scale_name: str):
    return getattr(layer, f"{which}_{scale_name}")


def check_expert_map(emap, n_global: int, n_local: int) -> Optional[str]:
    """None when `emap` is a global-to-local map for exactly `n_local` resident experts (-1 elsewhere, local
    slots 0..n_local-1), otherwise what is wrong with it. A 0/1 ownership mask has the same dtype and length;
    read as a map it would send every owned token to local slot 1, hence the proof."""
    if emap is None:
        return "the layer has no expert_map"
    if emap.dtype != torch.int32:
        return f"expert_map is {emap.dtype}, the kernel reads int32"
    if emap.numel() != n_global:
        return f"expert_map has {emap.numel()} entries for {n_global} experts"
    owned = emap[emap >= 0]
    if owned.numel() != n_local or (owned.numel() and int(owned.max()) != n_local - 1):
        return (f"expert_map is not a global-to-local map: {owned.numel()} owned entries, largest "
                f"{int(owned.max()) if owned.numel() else None}; expected {n_local} and {n_local - 1}")
    if torch.unique(owned).numel() != n_local:
        return "expert_map assigns a local slot twice"
    return None


def check_layer(kernel: MonoKernel, layer, *, block_quant: bool = True, raw_block_fp8_backend: bool = True,
                scale_name: str = "weight_scale_inv") -> Eligibility:
    """The load-time decision for one layer. Nothing is launched."""
    reasons = []
    if not _env_on(ENV_ENABLE):
        reasons.append(f"{ENV_ENABLE}=0")
    if not block_quant:
        reasons.append("weights are not block-quantised FP8")
    if not raw_block_fp8_backend:
        reasons.append("the selected fused-MoE backend repacks the weights; the kernel reads the checkpoint layout")
    if int(getattr(layer, "top_k", 1)) <= 1:
        reasons.append("top_k <= 1")
    if reasons:
        return Eligibility(False, reasons)
    geo = kernel.geometry()
    n_global = int(getattr(layer, "global_num_experts", 0))
    n_local = int(layer.w13_weight.size(0))
    layer_dims = {
        "num_experts": n_global, "num_experts_local": n_local, "top_k": int(layer.top_k),
        "k_dim": int(layer.w13_weight.size(2)), "n_up": int(layer.w13_weight.size(1)),
        "n_half": int(layer.w2_weight.size(2)), "h_dim": int(layer.w2_weight.size(1)),
    }
    compiled = dict(geo)
    if compiled.get("num_experts_local") is None:      # a binary without the symbol indexes by the global count
        compiled["num_experts_local"] = compiled.get("num_experts")
    for name, have in layer_dims.items():
        want = compiled.get(name)
        if want is not None and want != have:
            reasons.append(f"{name}: binary {want}, layer {have}")
    for which, blk in (("w13", (layer_dims["n_up"], layer_dims["k_dim"])), ("w2", (layer_dims["h_dim"], layer_dims["n_half"]))):
        sc = getattr(layer, f"{which}_{scale_name}", None)
        if sc is None or tuple(sc.shape) != (n_local, blk[0] // 128, blk[1] // 128):
            reasons.append(f"{which} scales are not one fp32 per [128,128] block")
    ep_needed = n_local != n_global
    if ep_needed and not geo.get("ep_capable"):
        reasons.append(f"weights hold {n_local} of {n_global} experts but the binary is not an expert-parallel build")
    elif geo.get("ep_capable") and not ep_needed:
        reasons.append("the binary is an expert-parallel build but the weights hold every expert")
    elif ep_needed:
        why = check_expert_map(getattr(layer, "expert_map", None), n_global, n_local)
        if why:
            reasons.append(why)
    mode = geo.get("router_mode")
    scoring = getattr(layer, "scoring_func", "softmax")
    bias = getattr(layer, "e_score_correction_bias", None)
    bias = getattr(bias, "data", bias)
    if mode == 0 and scoring != "softmax":
        reasons.append(f"the binary routes with softmax, the layer with {scoring}")
    if mode in (1, 2) and scoring != "sigmoid":
        reasons.append(f"the binary routes with sigmoid + bias, the layer with {scoring}")
    if mode in (1, 2) and bias is None:
        reasons.append("the binary routes with sigmoid + bias but the layer has no e_score_correction_bias")
    if mode == 0 and bias is not None:
        reasons.append("the binary routes with softmax and cannot apply an e_score_correction_bias")
    return Eligibility(not reasons, reasons, ep_needed, None if reasons else bias)


class MonokernelGlue:
    """One layer's decision and call path.

    tp_group / tp_size       the tensor-parallel process group (None / 1 without tensor parallelism)
    skip_final_all_reduce    the model reduces the MoE output itself later: never reduce here
    overlaps_shared_experts  vLLM's modular kernel runs the shared experts inside itself: decline everything
    max_tokens, num_ubatches sizes of the symmetric pool (the engine's max_num_batched_tokens and micro-batches)
    """

    def __init__(self, kernel: MonoKernel, layer, *, scale_name: str = "weight_scale_inv", tp_group=None,
                 tp_size: int = 1, skip_final_all_reduce: bool = False, overlaps_shared_experts: bool = False,
                 hidden_dim: Optional[int] = None, max_tokens: int = 0, num_ubatches: int = 1,
                 block_quant: bool = True, raw_block_fp8_backend: bool = True,
                 ubatch_id: Callable[[], int] = lambda: 0):
        self.kernel, self.scale_name = kernel, scale_name
        self.tp_group, self.tp_size = tp_group, int(tp_size)
        self.skip_final_all_reduce = bool(skip_final_all_reduce)
        self.overlaps_shared_experts = bool(overlaps_shared_experts)
        self.ubatch_id = ubatch_id
        self.eligibility = check_layer(kernel, layer, block_quant=block_quant,
                                       raw_block_fp8_backend=raw_block_fp8_backend, scale_name=scale_name)
        if self.eligibility.ok:
            logger.info("MoE prefill kernel enabled for this layer (expert parallel: %s)", self.eligibility.expert_parallel)
        else:
            logger.info("MoE prefill kernel declined: %s", "; ".join(self.eligibility.reasons))
        self.plan = None
        if self.fused_tp_eligible():
            # here, at weight load, in ordinary eager code on every rank: the plan votes and rendezvouses
            self.plan = tp_fused.fused_tp_plan(kernel, tp_group, hidden_dim or int(layer.w2_weight.size(1)),
                                               int(max_tokens), int(num_ubatches), enabled=_env_on(ENV_FUSE_TP))

    # ---- predicates the runner reads (identical on every rank: configuration and agreed capability only)
    def fused_tp_eligible(self) -> bool:
        return (self.eligibility.ok and not self.overlaps_shared_experts and self.tp_size >= 2
                and not self.skip_final_all_reduce and not self.eligibility.expert_parallel)

    def output_is_reduced(self) -> bool:
        """Whether outputs of this path are handed back summed over the tensor-parallel group. Independent of
        the token count on purpose (a traced caller specialises the branch once): for sizes the in-kernel reduce
        declines, `finish` performs the reduce instead."""
        return bool(self.plan is not None and self.plan.usable)

    def folds_shared_output(self) -> bool:
        return bool(self.plan is not None and self.plan.usable and self.plan.fold_shared)

    # ---- the call
    def try_moe_monokernel(self, layer, x, router_logits, residual=None, out_scale: float = 1.0):
        """The layer's routed output for this batch, or None to leave it to vLLM's own path."""
        if not self.eligibility.ok or self.overlaps_shared_experts:
            return None
        if x.size(0) > MOE_MONOKERNEL_PREFILL_MAX_TOKENS:
            return None
        w13s, w2s = _scale_of(layer, "w13", self.scale_name), _scale_of(layer, "w2", self.scale_name)
        if self.output_is_reduced():
            fold = self.plan.fold_shared
            if not (fold and residual is None):     # with the fold on, entering without the shared half would bring back the second reduce
                out = self.plan.fused_tp_launch(x, router_logits, layer.w13_weight, w13s, layer.w2_weight, w2s,
                                                layer.top_k, getattr(layer, "renormalize", True), self.eligibility.bias,
                                                residual=residual if fold else None,
                                                out_scale=float(out_scale) if fold else 1.0, slot=int(self.ubatch_id()))
                if out is not None:
                    return out      # no try/except around this launch: the peers are already in the collective
        try:
            return self.kernel.prefill(x, router_logits, layer.w13_weight, w13s, layer.w2_weight, w2s, layer.top_k,
                                       getattr(layer, "renormalize", True), self.eligibility.bias,
                                       layer.expert_map if self.eligibility.expert_parallel else None)
        except RuntimeError as exc:
            logger.warning("MoE prefill kernel failed (%s); using the ordinary fused-MoE path", exc)
            return None

    # ---- reduce-once bookkeeping
    def finish(self, routed_out, shared_out, residual_was_offered: bool, routed_scaling_factor: float,
               all_reduce: Callable[[torch.Tensor], torch.Tensor]):
        """Bring what `try_moe_monokernel` returned to the state `output_is_reduced()` promises, reducing at most
        once. Returns (shared_out still to be added by the caller or None, routed_out).

        * the output is a pool slot (address test): it is reduced, and folded if a residual was offered;
          a pool slot without the shared half although the fold is on cannot be produced and raises;
        * otherwise, when this path promises reduced outputs: combine `routed * scale + shared` first when the
          fold is on (both halves are still partial sums), then one all-reduce;
        * otherwise nothing happens here: the caller reduces as it always did."""
        if not self.output_is_reduced():
            return shared_out, routed_out
        was_fused = self.plan.output_is_fused(routed_out)
        fold = self.folds_shared_output()
        if was_fused:
            if fold and not residual_was_offered:
                raise RuntimeError("the in-kernel reduce ran without the shared expert's output although folding is on")
            return (None if fold else shared_out), routed_out
        if fold and shared_out is not None:
            if routed_scaling_factor != 1.0:
                routed_out = routed_out * routed_scaling_factor
            routed_out = routed_out + shared_out
            shared_out = None
        return shared_out, all_reduce(routed_out)


def install(kernel_path: Optional[str] = None) -> bool:
    """Attach the glue to vLLM's FP8 MoE quant method: `try_moe_monokernel`, `monokernel_output_is_reduced` and
    `monokernel_folds_shared_output`, the three names the reference's runner looks up
    (fused_moe/runner/moe_runner.py:853-870). The layer is checked after its weights are loaded. Returns False
    when vLLM (or its Fp8MoEMethod) is not importable; raises when no kernel binary is named."""
    path = kernel_path or os.environ.get("VLLM_PREFILL_MONOKERNEL_SO")
    if not path:
        raise RuntimeError("no kernel binary named: pass kernel_path or set VLLM_PREFILL_MONOKERNEL_SO")
    try:
        from vllm.model_executor.layers.quantization.fp8 import Fp8MoEMethod
    except Exception as exc:   # vLLM absent or of an incompatible layout
        logger.info("vLLM's Fp8MoEMethod is not importable (%s): nothing installed", exc)
        return False
    kernel = MonoKernel(path)
    loaded = Fp8MoEMethod.process_weights_after_loading

    def process_weights_after_loading(self, layer):
        loaded(self, layer)
        moe = getattr(self, "moe", None)
        self._monokernel_glue = MonokernelGlue(
            kernel, layer, scale_name=getattr(self, "weight_scale_name", "weight_scale_inv"),
            tp_group=getattr(moe, "tp_group", None), tp_size=int(getattr(moe, "tp_size", 1) or 1),
            skip_final_all_reduce=bool(getattr(moe, "skip_final_all_reduce", False)),
            overlaps_shared_experts=bool(getattr(self, "mk_can_overlap_shared_experts", False)),
            hidden_dim=getattr(moe, "hidden_dim", None),
            max_tokens=int(getattr(self, "_mk_max_num_batched_tokens", 0) or 0),
            num_ubatches=int(getattr(self, "_mk_num_ubatches", 1) or 1),
            block_quant=bool(getattr(self, "block_quant", False)))

    def try_moe_monokernel(self, layer, x, router_logits, residual=None, out_scale=1.0):
        glue = getattr(self, "_monokernel_glue", None)
        return None if glue is None else glue.try_moe_monokernel(layer, x, router_logits, residual, out_scale)

    Fp8MoEMethod.process_weights_after_loading = process_weights_after_loading
    Fp8MoEMethod.try_moe_monokernel = try_moe_monokernel
    Fp8MoEMethod.monokernel_output_is_reduced = lambda self: bool(
        getattr(self, "_monokernel_glue", None) and self._monokernel_glue.output_is_reduced())
    Fp8MoEMethod.monokernel_folds_shared_output = lambda self: bool(
        getattr(self, "_monokernel_glue", None) and self._monokernel_glue.folds_shared_output())
    return True
