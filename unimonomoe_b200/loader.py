"""Host side of the FP8 MoE prefill kernel: load the C-ABI library with ctypes, read its
compiled geometry back, validate a call against it, own the scratch buffers, launch.

Mirrors the reference's loader and launcher (vllm_integration/vllm/_custom_ops.py:4242-4994):
same function names, argument meaning and error behaviour, so a maintainer can swap the
module in behind ``Fp8MoEMethod.try_moe_monokernel``. Differences, all deliberate:

* several binaries can be loaded in one process (one ``MonoKernel`` per .so); the
  module-level functions act on the binary named by ``VLLM_PREFILL_MONOKERNEL_SO`` exactly
  as the reference does, and refuse to guess when it is unset (_custom_ops.py:4259-4272);
* scratch buffers come from one grow-only arena per device instead of being allocated on every
  call (_custom_ops.py:4645-4652), and the per-slot partial buffer is bf16, the size the kernel
  really touches;
* every device-side wait of the kernel is bounded; ``check_status`` reads the status word.

There is no CPU or library fallback: without CUDA and the compiled extension every launch
raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

MOE_MONOKERNEL_PREFILL_MAX_TOKENS = 30720  # _custom_ops.py:4247

_GEOMETRY_SYMBOLS = (
    "num_experts", "num_experts_local", "ep_capable", "top_k", "k_dim", "h_dim", "n_up", "n_half",
    "router_mode", "max_tiles", "grid_size", "fused_renorm", "block_m", "n_group", "topk_group",
    "up_pipe", "dn_pipe", "a_stages", "shm_total", "arch", "block_threads", "stable_sort",
)
_TP_CAP_SYMBOLS = ("tp_max_c", "tp_has_residual", "tp_align", "tp_mm", "tp_has_devseq", "tp_seq_bytes", "grid_size")

STATUS_CODES = {
    0: "ok", 1: "grid barrier timed out", 2: "pipeline barrier timed out", 3: "chunk-ready wait timed out",
    4: "rank barrier timed out", 5: "done-flag wait timed out", 6: "device index out of bounds",
}


def variant_path(variant: str) -> str:
    """Path of the in-tree binary built for a named geometry (see unimonomoe_b200/build.py)."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", f"libprefill_mono_{variant}.so")


def prepare_router_weight(weight: torch.Tensor) -> torch.Tensor:
    """The gate weight [E, K] as the in-kernel router wants it: contiguous bfloat16. Done once when the
    layer is loaded, never per call. The checkpoints of both model families store the gate in bf16 and
    the fp32 router linear of the DeepSeek harness upcasts it (validation/ds3_acc.py:412), so the
    conversion is exact; a weight that does not survive the round trip is refused, because the kernel
    would then route on different logits than the caller's own linear."""
    w16 = weight.to(torch.bfloat16).contiguous()
    if weight.dtype != torch.bfloat16 and not torch.equal(w16.to(weight.dtype), weight):
        raise ValueError("router weight is not exactly representable in bfloat16; keep the router linear outside "
                         "the kernel and pass logits")
    return w16


def prepare_shared_expert(w13, w13_scale, w2, w2_scale, gate=None) -> dict:
    """The shared expert as the launch wants it, converted once at load time: block-FP8 weights in the layout
    of one routed expert (w13 [2*I, K] gate rows then up rows, w2 [H, I], one fp32 scale per [128,128] block)
    and, for a gated shared expert, the gate vector as contiguous bfloat16 [K]."""
    sh = {"w13": w13.contiguous().view(torch.uint8), "w13_scale": w13_scale.float().contiguous(),
          "w2": w2.contiguous().view(torch.uint8), "w2_scale": w2_scale.float().contiguous(), "gate": None}
    if gate is not None:
        sh["gate"] = gate.reshape(-1).to(torch.bfloat16).contiguous()
    return sh


class MonoKernel:
    """One loaded ``libprefill_mono_*.so``."""

    def __init__(self, so_path: str):
        if not so_path:
            raise RuntimeError(
                "no monokernel binary selected; the compiled geometry of the kernel has to be the "
                "caller's explicit choice (set VLLM_PREFILL_MONOKERNEL_SO)")
        if not os.path.exists(so_path):
            raise RuntimeError(f"monokernel binary {so_path} does not exist; build it with "
                               "`python -m unimonomoe_b200.build`")
        self.path = so_path
        lib = ctypes.CDLL(so_path)
        self.lib = lib
        lib.launch_prefill_moe_wgmma_q1.restype = ctypes.c_int
        lib.prefill_wgmma_workspace_bytes.restype = ctypes.c_size_t
        self.has_router = self._bind("launch_prefill_moe_wgmma_q1_router")
        self.has_tp = self._bind("launch_prefill_moe_wgmma_q1_tp")
        self.has_tp2 = self._bind("launch_prefill_moe_wgmma_q1_tp2")
        self.has_ep = self._bind("launch_prefill_moe_wgmma_q1_ep")
        self.has_gemv = self._bind("launch_prefill_moe_wgmma_q1_gemv") and bool(self._int_symbol("has_router_gemv"))
        self.has_shared = self._bind("launch_prefill_moe_wgmma_q1_shared") and bool(self._int_symbol("has_shared_expert"))
        self._caps = {}
        for name in _TP_CAP_SYMBOLS:
            self._caps[name] = self._int_symbol(name)
        try:
            fn = lib.prefill_wgmma_tp_pad_words
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
            self._pad_words_fn = fn
        except AttributeError:
            self._pad_words_fn = None
        self._geo = None
        self._scratch = {}    # device -> arena
        self._retired = []    # outgrown arenas, kept alive for captured graphs
        try:
            lib.prefill_wgmma_set_wait_timeout_us.argtypes = [ctypes.c_ulonglong]
            lib.prefill_wgmma_set_wait_timeout_us.restype = None
            lib.prefill_wgmma_set_debug.argtypes = [ctypes.c_void_p] * 3
            lib.prefill_wgmma_set_debug.restype = None
        except AttributeError:
            pass

    # ------------------------------------------------------------------ symbols
    def _bind(self, name: str) -> bool:
        try:
            getattr(self.lib, name).restype = ctypes.c_int
            return True
        except AttributeError:
            return False

    def _int_symbol(self, name: str):
        try:
            fn = getattr(self.lib, "prefill_wgmma_" + name)
        except AttributeError:
            return None
        fn.restype = ctypes.c_int
        return int(fn())

    def geometry(self) -> dict:
        """Compiled geometry; symbols the binary lacks come back None (_custom_ops.py:4443-4458)."""
        if self._geo is None:
            geo = {n: self._int_symbol(n) for n in _GEOMETRY_SYMBOLS}
            geo["has_router_entry"] = self.has_router
            geo["workspace_bytes"] = int(self.lib.prefill_wgmma_workspace_bytes())
            self._geo = geo
        return dict(self._geo)

    def tp_caps(self) -> dict:
        """Fused tensor-parallel capability (_custom_ops.py:4352-4376)."""
        caps = dict(self._caps)
        caps["has_tp"] = self.has_tp
        caps["has_tp2_entry"] = self.has_tp2
        caps["has_tp_residual"] = bool(self.has_tp2 and caps.get("tp_has_residual"))
        caps["usable"] = bool(self.has_tp and self._pad_words_fn is not None and caps.get("tp_max_c")
                              and caps.get("tp_align") and caps.get("grid_size"))
        return caps

    def tp_pad_words(self, nchunk: int, ncomm: int, world: int) -> int:
        if self._pad_words_fn is None:
            raise RuntimeError("loaded monokernel .so does not export prefill_wgmma_tp_pad_words, "
                               "so it cannot drive the fused TP path")
        return int(self._pad_words_fn(int(nchunk), int(ncomm), int(world)))

    def set_wait_timeout_us(self, us: int) -> None:
        self.lib.prefill_wgmma_set_wait_timeout_us(ctypes.c_ulonglong(int(us)))

    def set_debug(self, acc=None, inter=None, inter_scale=None) -> None:
        f = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731
        self.lib.prefill_wgmma_set_debug(f(acc), f(inter), f(inter_scale))

    # ------------------------------------------------------------------ validation
    def validate(self, activations_in, expert_weights_up, expert_weights_down, top_k, e_score_correction_bias,
                 expert_map=None):
        """Compare the compiled geometry of this binary with the tensors of a call and return the router
        bias to pass (fp32, contiguous) or None. Any disagreement raises RuntimeError before anything is
        launched: a binary run on weights of another shape would index out of its tiles. A dimension the
        binary does not export (None) is not checked. Plays the role of _custom_ops.py:4461-4565."""
        geo = self.geometry()
        experts_got = int(expert_weights_up.size(0))
        local = geo["num_experts_local"] if geo["num_experts_local"] is not None else geo["num_experts"]
        # (what, compiled value, value of this call)
        dims = [
            ("up-projection rows 2*I (N_UP)", geo["n_up"], int(expert_weights_up.size(1))),
            ("intermediate width I (N_HALF)", geo["n_half"], int(expert_weights_down.size(2))),
            ("hidden size of the activations (K_DIM)", geo["k_dim"], int(activations_in.size(1))),
            ("output width (H_DIM)", geo["h_dim"], int(expert_weights_down.size(1))),
            ("experts whose weights are passed (E_LOCAL)", local, experts_got),
            ("experts per token (TOP_K)", geo["top_k"], int(top_k)),
        ]
        if expert_map is None:
            dims.append(("experts the router scores (E), no expert_map given", geo["num_experts"], experts_got))
        else:
            if not geo["ep_capable"]:
                raise RuntimeError("expert_map given, but this binary is not an expert-parallel build: it would "
                                   "index the weights with global expert ids")
            if expert_map.dtype != torch.int32:
                raise RuntimeError(f"expert_map has dtype {expert_map.dtype}; the kernel reads int32")
            dims.append(("entries of expert_map (E)", geo["num_experts"], int(expert_map.numel())))
        wrong = [f"{what}: compiled {want}, got {got}" for what, want, got in dims if want is not None and want != got]
        if wrong:
            raise RuntimeError(f"{os.path.basename(self.path)} does not fit this call: " + "; ".join(wrong))

        mode = geo["router_mode"]
        if e_score_correction_bias is None:
            if mode not in (None, 0):
                raise RuntimeError(f"this binary routes with sigmoid + bias (ROUTER_MODE {mode}) and needs an "
                                   "e_score_correction_bias")
            return None
        if mode == 0:
            raise RuntimeError("this binary routes with softmax (ROUTER_MODE 0) and has no use for an "
                               "e_score_correction_bias")
        if not self.has_router:
            raise RuntimeError("this binary lacks launch_prefill_moe_wgmma_q1_router, the entry that takes the bias")
        return e_score_correction_bias.float().contiguous()

    # ------------------------------------------------------------------ scratch
    def _allocate_scratch(self, tokens: int, device) -> dict:
        geo = self.geometry()
        K, H, k = geo["k_dim"], geo["h_dim"], geo["top_k"]
        chunks = self._int_symbol("partial_chunks") or 1
        return {
            "workspace": torch.zeros(geo["workspace_bytes"], dtype=torch.uint8, device=device),
            "act_fp8": torch.empty(tokens, K, dtype=torch.uint8, device=device),
            "act_scales": torch.empty(tokens, K // 128, dtype=torch.float32, device=device),
            "topk_ids": torch.empty(tokens, k, dtype=torch.int32, device=device),
            "topk_weights": torch.empty(tokens, k, dtype=torch.float32, device=device),
            "sorted_ids": torch.empty(tokens * k, dtype=torch.int32, device=device),
            # top_k rows per token for the routed experts plus one for a shared expert computed in the launch
            "partial": torch.empty(tokens * (k + 1) * chunks, H, dtype=torch.bfloat16, device=device),
            "shared_gate": torch.empty(tokens, dtype=torch.float32, device=device),
        }

    def scratch(self, M: int, device) -> dict:
        """The scratch buffers of a launch for M tokens on `device` (the reference allocates them on
        every call, _custom_ops.py:4645-4652).

        One arena per device, sized for the largest batch seen so far; a call for fewer tokens gets
        views of its first rows, so a new prefill length costs no allocation. Nothing is ever handed back
        to the allocator while this object lives: when a larger batch arrives a larger arena is added
        and the old one is kept, because a captured CUDA graph may still hold its addresses. While the
        current stream is capturing, a batch that does not fit gets fresh buffers that are not cached, so
        that the capture's own memory pool owns them. All launches through one MonoKernel share the arena
        and its workspace: use one MonoKernel per stream, or order the launches."""
        M = int(M)
        dev = torch.device(device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        arena = self._scratch.get(dev)
        if arena is None or arena["tokens"] < M:
            if dev.type == "cuda" and torch.cuda.is_current_stream_capturing():
                return self._allocate_scratch(M, dev)
            if arena is not None:
                self._retired.append(arena)
            arena = {"tokens": M, "buffers": self._allocate_scratch(M, dev), "views": {}}
            self._scratch[dev] = arena
        sc = arena["views"].get(M)
        if sc is None:
            buf, k = arena["buffers"], self.geometry()["top_k"]
            chunks = self._int_symbol("partial_chunks") or 1
            sc = {"workspace": buf["workspace"], "act_fp8": buf["act_fp8"][:M], "act_scales": buf["act_scales"][:M],
                  "topk_ids": buf["topk_ids"][:M], "topk_weights": buf["topk_weights"][:M],
                  "sorted_ids": buf["sorted_ids"][:M * k], "partial": buf["partial"][:M * (k + 1) * chunks],
                  "shared_gate": buf["shared_gate"][:M]}
            arena["views"][M] = sc
        return sc

    def check_status(self, workspace: torch.Tensor) -> None:
        """Synchronise and raise if the last launch on this workspace reported a bounded-wait error."""
        off = self._int_symbol("status_offset")
        torch.cuda.synchronize(workspace.device)
        words = workspace[off:off + 16].cpu().view(torch.int32).tolist()
        st = words[0] & 0xFFFFFFFF
        if st != 0:
            code, site, block = st >> 24, (st >> 16) & 0xFF, st & 0xFFFF
            raise RuntimeError(f"monokernel device status: {STATUS_CODES.get(code, code)} "
                               f"(code {code}, site {site}, block {block}, aux {words[2]}, {words[3]})")

    def workspace_view(self, workspace: torch.Tensor) -> dict:
        """Decoded read-back of the counters the kernel leaves in the workspace."""
        E = self.geometry()["num_experts"]
        w = workspace.cpu()
        g = lambda name, n, dt: w[self._int_symbol(name):self._int_symbol(name) + n * dt.itemsize].view(dt)  # noqa: E731
        return {
            "expert_counts": g("counts_offset", E, torch.int32).clone(),
            "expert_offsets": g("offsets_offset", E + 1, torch.int32).clone(),
            "total_tiles": int(g("total_tiles_offset", 1, torch.int32)[0]),
            "phase_ns": g("phase_ns_offset", 8, torch.int64).clone(),
        }

    # ------------------------------------------------------------------ launch
    def prefill_impl(self, activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                     expert_scales_down, top_k, renormalize, e_score_correction_bias, out, tp=None, residual=None,
                     out_scale=1.0, expert_map=None, scratch=None, check=False, router_weight=None, shared=None,
                     shared_part=(0, 1)) -> dict:
        """Launch the kernel into ``out`` (_custom_ops.py:4568-4762). Returns the scratch dict
        (topk_ids, topk_weights, sorted_ids, workspace, ...) the launch wrote.

        With ``router_weight`` (the gate weight [E, K] in bf16, see `prepare_router_weight`) the router
        linear runs inside the launch; ``router_logits`` is then ignored and may be None, and the logits
        the kernel routed on are left in ``scratch["logits"]``.

        With ``shared`` (see `prepare_shared_expert`) the gated shared expert is computed in the same launch:
        out = bf16(out_scale * routed + shared (+ residual)). ``shared_part = (r, n)`` restricts it to the
        128-token tiles j with j % n == r, so that expert-parallel ranks split the tokens between them."""
        if not torch.cuda.is_available() or not activations_in.is_cuda:
            raise RuntimeError("the FP8 MoE prefill kernel needs a CUDA device; there is no CPU path")
        M, K = activations_in.shape
        H = expert_weights_down.size(1)
        top_k = int(top_k)
        device = activations_in.device
        if M > MOE_MONOKERNEL_PREFILL_MAX_TOKENS:
            raise RuntimeError(f"monokernel refuses {M} tokens (cap {MOE_MONOKERNEL_PREFILL_MAX_TOKENS})")

        act = activations_in.contiguous()
        if act.dtype != torch.bfloat16:
            raise RuntimeError(f"monokernel activations must be bfloat16, got {act.dtype}")
        rw = None
        if router_weight is not None:
            if not self.has_gemv:
                raise RuntimeError("loaded monokernel .so has no launch_prefill_moe_wgmma_q1_gemv")
            rw = router_weight
            E = self.geometry()["num_experts"]
            if rw.dtype != torch.bfloat16 or tuple(rw.shape) != (E, K) or not rw.is_contiguous() or rw.device != device:
                raise RuntimeError(f"in-kernel router needs a contiguous bfloat16 [{E}, {K}] gate weight on {device}, got "
                                   f"{tuple(rw.shape)} {rw.dtype} on {rw.device}; convert once with prepare_router_weight")
            logits = None
        else:
            logits = router_logits.float().contiguous()
        w_up = expert_weights_up.contiguous().view(torch.uint8)
        w_down = expert_weights_down.contiguous().view(torch.uint8)
        s_up = expert_scales_up.float().contiguous()
        s_down = expert_scales_down.float().contiguous()

        emap = None
        if expert_map is not None:
            # The reference refuses the fused collective together with an expert_map (an EP rank's output is
            # reduced by the caller, _custom_ops.py:4626-4633). Here the in-kernel reduce also serves expert
            # parallelism: the partial sums of EP ranks are reduced exactly like those of TP ranks.
            if tp is not None and not hasattr(self.lib, "launch_prefill_moe_wgmma_q1_ep2"):
                raise RuntimeError("the fused collective and an expert_map need launch_prefill_moe_wgmma_q1_ep2")
            emap = expert_map.to(torch.int32).contiguous()
        bias = self.validate(activations_in, expert_weights_up, expert_weights_down, top_k,
                             e_score_correction_bias, emap)
        if out.shape != (M, H) or out.dtype != torch.bfloat16:
            raise RuntimeError(f"monokernel destination must be [{M}, {H}] bfloat16, got {tuple(out.shape)} {out.dtype}")
        if not out.is_contiguous():
            raise RuntimeError("monokernel destination must be contiguous")

        if shared is not None:
            if not self.has_shared:
                raise RuntimeError("loaded monokernel .so has no launch_prefill_moe_wgmma_q1_shared")
            if router_weight is not None:
                raise RuntimeError("the shared expert and the in-kernel router linear have separate entry points; "
                                   "pass logits when a shared expert is given")
            n_half = expert_weights_down.size(2)
            want = {"w13": (2 * n_half, K), "w13_scale": (2 * n_half // 128, K // 128), "w2": (H, n_half),
                    "w2_scale": (H // 128, n_half // 128)}
            for name, shape in want.items():
                if tuple(shared[name].shape) != shape or shared[name].device != device or not shared[name].is_contiguous():
                    raise RuntimeError(f"shared expert {name} must be contiguous {shape} on {device}, got "
                                       f"{tuple(shared[name].shape)} on {shared[name].device}")
            g = shared.get("gate")
            if g is not None and (g.dtype != torch.bfloat16 or tuple(g.shape) != (K,) or not g.is_contiguous()):
                raise RuntimeError(f"shared expert gate must be contiguous bfloat16 [{K}]; use prepare_shared_expert")
        resid_ptr = 0
        if residual is not None:
            if residual.shape != (M, H) or residual.dtype != torch.bfloat16:
                raise RuntimeError(f"monokernel folded residual must be [{M}, {H}] bfloat16, got "
                                   f"{tuple(residual.shape)} {residual.dtype}")
            if not residual.is_contiguous():
                raise RuntimeError("monokernel folded residual must be contiguous")
            if tp is None and shared is None:
                raise RuntimeError("a folded residual is only carried by the fused collective; without a TP "
                                   "configuration there is nothing to fold it into")
            resid_ptr = residual.data_ptr()
        fold = resid_ptr != 0 or float(out_scale) != 1.0
        if fold and tp is None and shared is None:
            raise RuntimeError("an output scale is only applied by the fused collective or together with a shared "
                               "expert; scale the result yourself")
        if fold and not self.has_tp2:
            raise RuntimeError("loaded monokernel .so has no launch_prefill_moe_wgmma_q1_tp2, so it cannot fold a "
                               "residual or apply an output scale")
        if not renormalize and self.geometry()["fused_renorm"]:
            raise RuntimeError("monokernel .so is a FUSED_RENORM build but renormalize=False was requested; the "
                               "in-kernel normalization cannot be undone")

        sc = scratch if scratch is not None else self.scratch(M, device)
        vp = ctypes.c_void_p
        if rw is not None:
            if "logits" not in sc:
                sc["logits"] = torch.empty(M, rw.size(0), dtype=torch.float32, device=device)
            head = [vp(rw.data_ptr()), vp(sc["logits"].data_ptr())]
        else:
            head = [vp(logits.data_ptr())]
        args = head + [
            ctypes.c_int(M), ctypes.c_int(128),
            vp(sc["workspace"].data_ptr()), ctypes.c_size_t(sc["workspace"].numel()),
            vp(act.data_ptr()), vp(sc["act_fp8"].data_ptr()), vp(sc["act_scales"].data_ptr()),
            vp(w_up.data_ptr()), vp(s_up.data_ptr()), vp(w_down.data_ptr()), vp(s_down.data_ptr()),
            vp(sc["partial"].data_ptr()), vp(sc["topk_ids"].data_ptr()), vp(sc["topk_weights"].data_ptr()),
            vp(sc["sorted_ids"].data_ptr()), vp(out.data_ptr()),
        ]
        bias_arg = vp(bias.data_ptr() if bias is not None else 0)
        if shared is not None:
            mc, pads, seqctr, rank, world, nchunk, ncomm = tp[:7] if tp is not None else (0, 0, 0, 0, 1, 1, 0)
            entry = self.lib.launch_prefill_moe_wgmma_q1_shared
            g = shared.get("gate")
            args += [bias_arg, vp(int(mc)), vp(int(pads)), ctypes.c_int(int(rank)), ctypes.c_int(int(world)),
                     ctypes.c_int(int(nchunk)), ctypes.c_int(int(ncomm)), ctypes.c_uint(0), vp(int(seqctr)),
                     vp(int(resid_ptr)), ctypes.c_float(float(out_scale)), vp(emap.data_ptr() if emap is not None else 0),
                     vp(shared["w13"].data_ptr()), vp(shared["w13_scale"].data_ptr()), vp(shared["w2"].data_ptr()),
                     vp(shared["w2_scale"].data_ptr()), vp(g.data_ptr() if g is not None else 0),
                     vp(sc["shared_gate"].data_ptr()), ctypes.c_int(int(shared_part[0])), ctypes.c_int(int(shared_part[1]))]
        elif rw is not None:
            # one entry point carries every option: absent ones are passed as null / neutral values
            mc, pads, seqctr, rank, world, nchunk, ncomm = tp[:7] if tp is not None else (0, 0, 0, 0, 1, 1, 0)
            entry = self.lib.launch_prefill_moe_wgmma_q1_gemv
            args += [bias_arg, vp(int(mc)), vp(int(pads)), ctypes.c_int(int(rank)), ctypes.c_int(int(world)),
                     ctypes.c_int(int(nchunk)), ctypes.c_int(int(ncomm)), ctypes.c_uint(0), vp(int(seqctr)),
                     vp(int(resid_ptr)), ctypes.c_float(float(out_scale)), vp(emap.data_ptr() if emap is not None else 0)]
        elif tp is not None:
            mc, pads, seqctr, rank, world, nchunk, ncomm = tp[:7]
            peers = int(tp[7]) if len(tp) > 7 else 0
            args += [bias_arg, vp(int(mc)), vp(int(pads)), ctypes.c_int(int(rank)), ctypes.c_int(int(world)),
                     ctypes.c_int(int(nchunk)), ctypes.c_int(int(ncomm)), ctypes.c_uint(0), vp(int(seqctr))]
            if peers and self._bind("launch_prefill_moe_wgmma_q1_ep3"):
                # the table of every rank's output window: two ranks then reduce by direct peer loads
                entry = self.lib.launch_prefill_moe_wgmma_q1_ep3
                args += [vp(int(resid_ptr)), ctypes.c_float(float(out_scale)), vp(emap.data_ptr() if emap is not None else 0),
                         vp(peers)]
            elif emap is not None:
                entry = self.lib.launch_prefill_moe_wgmma_q1_ep2
                entry.restype = ctypes.c_int
                args += [vp(int(resid_ptr)), ctypes.c_float(float(out_scale)), vp(emap.data_ptr())]
            elif fold:
                entry = self.lib.launch_prefill_moe_wgmma_q1_tp2
                args += [vp(int(resid_ptr)), ctypes.c_float(float(out_scale))]
            else:
                entry = self.lib.launch_prefill_moe_wgmma_q1_tp
        elif emap is not None:
            if not self.has_ep:
                raise RuntimeError("loaded monokernel .so has no launch_prefill_moe_wgmma_q1_ep")
            entry = self.lib.launch_prefill_moe_wgmma_q1_ep
            args += [bias_arg, vp(emap.data_ptr())]
        elif bias is not None:
            entry = self.lib.launch_prefill_moe_wgmma_q1_router
            args += [bias_arg]
        else:
            entry = self.lib.launch_prefill_moe_wgmma_q1
        args.append(vp(torch.cuda.current_stream(device).cuda_stream))
        rc = entry(*args)
        if rc != 0:
            raise RuntimeError(f"launch_prefill_moe_wgmma_q1 failed: rc={rc}")
        # keep the converted inputs alive until the stream has consumed them
        sc["_keepalive"] = (act, logits, rw, w_up, w_down, s_up, s_down, bias, emap, shared)
        if check:
            self.check_status(sc["workspace"])
        return sc

    def prefill(self, activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                expert_scales_down, top_k=8, renormalize=True, e_score_correction_bias=None, expert_map=None,
                check=False, router_weight=None, shared=None, shared_part=(0, 1), out_scale=1.0) -> torch.Tensor:
        """Allocating variant (_custom_ops.py:4820-4858). Under EP the result is this rank's partial sum.
        ``shared`` adds the shared expert inside the launch (``out_scale`` then scales the routed half)."""
        M, H = activations_in.size(0), expert_weights_down.size(1)
        out = torch.empty(M, H, dtype=torch.bfloat16, device=activations_in.device)
        self.prefill_impl(activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                          expert_scales_down, top_k, renormalize, e_score_correction_bias, out, None, None, out_scale,
                          expert_map, check=check, router_weight=router_weight, shared=shared, shared_part=shared_part)
        return out

    def prefill_out(self, activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                    expert_scales_down, out, top_k=8, renormalize=True, e_score_correction_bias=None, tp_mc_ptr=0,
                    tp_pads_ptr=0, tp_seqctr_ptr=0, tp_rank=0, tp_world=1, tp_nchunk=0, tp_ncomm=0, tp_residual=None,
                    tp_out_scale=1.0, check=False, expert_map=None, router_weight=None, shared=None,
                    shared_part=(0, 1), tp_peers_ptr=0) -> None:
        """Write into a caller-supplied destination (_custom_ops.py:4861-4924). tp_ncomm > 0 selects the
        fused collective, in which case ``out`` must be the symmetric window tp_mc_ptr aliases."""
        tp = None
        if tp_ncomm > 0:
            if not (tp_mc_ptr and tp_pads_ptr):
                raise RuntimeError("fused TP launch requires both a multicast pointer and a barrier pad pointer")
            tp = (tp_mc_ptr, tp_pads_ptr, tp_seqctr_ptr, tp_rank, tp_world, tp_nchunk, tp_ncomm, tp_peers_ptr)
        self.prefill_impl(activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                          expert_scales_down, top_k, renormalize, e_score_correction_bias, out, tp, tp_residual,
                          tp_out_scale, expert_map, check=check, router_weight=router_weight, shared=shared,
                          shared_part=shared_part)


# ---------------------------------------------------------------------- module-level mirror
_prefill_monokernel_lib: Optional[MonoKernel] = None


def _load_prefill_monokernel() -> MonoKernel:
    """The binary named by VLLM_PREFILL_MONOKERNEL_SO; refuses an unset variable
    (_custom_ops.py:4253-4288)."""
    global _prefill_monokernel_lib
    if _prefill_monokernel_lib is None:
        path = os.environ.get("VLLM_PREFILL_MONOKERNEL_SO")
        if not path:
            raise RuntimeError("VLLM_PREFILL_MONOKERNEL_SO is not set, so no monokernel binary has been selected; "
                               "the compiled geometry of the kernel has to be the caller's explicit choice")
        _prefill_monokernel_lib = MonoKernel(path)
    return _prefill_monokernel_lib


def _reset_prefill_monokernel() -> None:
    global _prefill_monokernel_lib
    _prefill_monokernel_lib = None


def prefill_monokernel_geometry() -> dict:
    return _load_prefill_monokernel().geometry()


def prefill_monokernel_tp_caps() -> dict:
    return _load_prefill_monokernel().tp_caps()


def prefill_monokernel_tp_pad_words(nchunk: int, ncomm: int, world: int) -> int:
    return _load_prefill_monokernel().tp_pad_words(nchunk, ncomm, world)


def monokernel_validate(activations_in, expert_weights_up, expert_weights_down, top_k, e_score_correction_bias,
                        expert_map=None):
    return _load_prefill_monokernel().validate(activations_in, expert_weights_up, expert_weights_down, top_k,
                                               e_score_correction_bias, expert_map)


def moe_monokernel_prefill(activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                           expert_scales_down, top_k: int = 8, renormalize: bool = True,
                           e_score_correction_bias=None, expert_map=None) -> torch.Tensor:
    return _load_prefill_monokernel().prefill(activations_in, router_logits, expert_weights_up, expert_scales_up,
                                              expert_weights_down, expert_scales_down, top_k, renormalize,
                                              e_score_correction_bias, expert_map)


def moe_monokernel_prefill_out(activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
                               expert_scales_down, out, top_k: int = 8, renormalize: bool = True,
                               e_score_correction_bias=None, tp_mc_ptr: int = 0, tp_pads_ptr: int = 0,
                               tp_seqctr_ptr: int = 0, tp_rank: int = 0, tp_world: int = 1, tp_nchunk: int = 0,
                               tp_ncomm: int = 0, tp_residual=None, tp_out_scale: float = 1.0) -> None:
    _load_prefill_monokernel().prefill_out(activations_in, router_logits, expert_weights_up, expert_scales_up,
                                           expert_weights_down, expert_scales_down, out, top_k, renormalize,
                                           e_score_correction_bias, tp_mc_ptr, tp_pads_ptr, tp_seqctr_ptr, tp_rank,
                                           tp_world, tp_nchunk, tp_ncomm, tp_residual, tp_out_scale)


def _register_ops() -> None:
    """torch custom ops with fake implementations, as the reference registers them
    (_custom_ops.py:4953-4994): the functional op returns a fresh tensor, the ``_out`` op
    declares that it mutates ``out`` so repeated calls on one buffer stay ordered."""
    try:
        @torch.library.custom_op("unimonomoe::moe_monokernel_prefill", mutates_args=())
        def _op(activations_in: torch.Tensor, router_logits: torch.Tensor, expert_weights_up: torch.Tensor,
                expert_scales_up: torch.Tensor, expert_weights_down: torch.Tensor, expert_scales_down: torch.Tensor,
                top_k: int = 8, renormalize: bool = True, e_score_correction_bias: Optional[torch.Tensor] = None,
                expert_map: Optional[torch.Tensor] = None) -> torch.Tensor:
            return moe_monokernel_prefill(activations_in, router_logits, expert_weights_up, expert_scales_up,
                                          expert_weights_down, expert_scales_down, top_k, renormalize,
                                          e_score_correction_bias, expert_map)

        @_op.register_fake
        def _(activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
              expert_scales_down, top_k=8, renormalize=True, e_score_correction_bias=None, expert_map=None):
            return torch.empty((activations_in.size(0), expert_weights_down.size(1)), dtype=torch.bfloat16,
                               device=activations_in.device)

        @torch.library.custom_op("unimonomoe::moe_monokernel_prefill_out", mutates_args=("out",))
        def _op_out(activations_in: torch.Tensor, router_logits: torch.Tensor, expert_weights_up: torch.Tensor,
                    expert_scales_up: torch.Tensor, expert_weights_down: torch.Tensor,
                    expert_scales_down: torch.Tensor, out: torch.Tensor, top_k: int = 8, renormalize: bool = True,
                    e_score_correction_bias: Optional[torch.Tensor] = None, tp_mc_ptr: int = 0, tp_pads_ptr: int = 0,
                    tp_seqctr_ptr: int = 0, tp_rank: int = 0, tp_world: int = 1, tp_nchunk: int = 0,
                    tp_ncomm: int = 0, tp_residual: Optional[torch.Tensor] = None,
                    tp_out_scale: float = 1.0) -> None:
            moe_monokernel_prefill_out(activations_in, router_logits, expert_weights_up, expert_scales_up,
                                       expert_weights_down, expert_scales_down, out, top_k, renormalize,
                                       e_score_correction_bias, tp_mc_ptr, tp_pads_ptr, tp_seqctr_ptr, tp_rank,
                                       tp_world, tp_nchunk, tp_ncomm, tp_residual, tp_out_scale)

        @_op_out.register_fake
        def _(activations_in, router_logits, expert_weights_up, expert_scales_up, expert_weights_down,
              expert_scales_down, out, top_k=8, renormalize=True, e_score_correction_bias=None, tp_mc_ptr=0,
              tp_pads_ptr=0, tp_seqctr_ptr=0, tp_rank=0, tp_world=1, tp_nchunk=0, tp_ncomm=0, tp_residual=None,
              tp_out_scale=1.0):
            return None
    except Exception:  # already registered in this process
        pass


_register_ops()
