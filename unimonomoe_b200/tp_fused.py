"""Host side of the fused tensor-parallel epilogue: the persistent symmetric output pool and
the rank-uniform plan that decides, once, whether a process may use it.

Mirrors the reference's `fused_moe/symm_output_pool.py` (pool) and `fused_moe/monokernel_tp.py`
(plan, chunk table, vote, launch). The kernel's last `ncomm` CTAs reduce finished chunks of the
output through the NVLS multicast alias of a symmetric buffer while the other CTAs still sum;
the host's job is to own that buffer (one maximum-size allocation per slot, always used from
offset 0), the separate symmetric barrier window, the device sequence counter, and to make
sure EVERY rank takes the same decision: a rank that enters the fused kernel while a peer does
not would wait at the first rank barrier (here: until the bounded wait gives up and reports).

Nothing here runs on the per-call path except `fused_tp_launch`, which allocates nothing and
performs no collective.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .loader import MonoKernel

# Token counts at which the fused epilogue is used, and the number of chunks the reduce is
# released in (monokernel_tp.py:79-82). Anything absent takes the ordinary path.
FUSED_CHUNKS_BY_TOKENS = {8192: 4, 16384: 8}
# CTAs that stop summing and communicate (monokernel_tp.py:87).
FUSED_NCOMM = 14


def env_chunk_table(default: dict) -> dict:
    """VLLM_PREFILL_MONOKERNEL_TP_CHUNKS: unset keeps the table, a bare integer applies to every
    listed size, "T:C,T:C" replaces it; a malformed value raises (monokernel_tp.py:90-117)."""
    raw = os.environ.get("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS", "").strip()
    if not raw:
        return dict(default)
    if ":" not in raw:
        c = int(raw)
        if c < 1:
            raise ValueError("VLLM_PREFILL_MONOKERNEL_TP_CHUNKS must be >= 1")
        return {t: c for t in default}
    out = {}
    for item in raw.split(","):
        t, c = item.split(":")
        out[int(t)] = int(c)
    if not out or any(c < 1 for c in out.values()):
        raise ValueError(f"VLLM_PREFILL_MONOKERNEL_TP_CHUNKS {raw!r} is not a usable T:C list")
    return out


def env_ncomm(default: int) -> int:
    raw = os.environ.get("VLLM_PREFILL_MONOKERNEL_TP_NCOMM", "").strip()
    if not raw:
        return default
    n = int(raw)
    if n < 1:
        raise ValueError("VLLM_PREFILL_MONOKERNEL_TP_NCOMM must be >= 1")
    return n


class SymmOutputPool:
    """Persistent symmetric output buffers, the barrier window and the sequence counter
    (symm_output_pool.py:102-149). Construct once, on every rank of the group, never per call."""

    def __init__(self, group, max_tokens: int, hidden: int, pad_words: int, nslots: int = 1, device=None):
        import torch.distributed._symmetric_memory as sm

        self.group_name = group if isinstance(group, str) else group.group_name
        self.max_tokens, self.hidden, self.nslots = int(max_tokens), int(hidden), int(nslots)
        self.device = device if device is not None else torch.cuda.current_device()
        n = self.max_tokens * self.hidden
        self._bufs, self._handles, self._mc, self._base = [], [], [], []
        for _ in range(self.nslots):
            b = sm.empty(n, device=self.device, dtype=torch.bfloat16)
            h = sm.rendezvous(b, self.group_name)
            mc = int(h.multicast_ptr)
            if not mc:
                raise RuntimeError("symmetric allocation has no multicast pointer; the fused reduce needs one")
            self._bufs.append(b)
            self._handles.append(h)
            self._mc.append(mc)
            self._base.append(int(b.data_ptr()))
        # The barrier window is its own symmetric allocation, not a handle's signal pad
        # (kernel/qwen_tp/src/prefill_mono_final_nb.cu:1540-1542).
        self.pad_words = int(pad_words)
        self._flags = sm.empty(self.pad_words, device=self.device, dtype=torch.int32)
        self._flags_handle = sm.rendezvous(self._flags, self.group_name)
        self._flags.zero_()
        self.pads_ptr = int(self._flags_handle.buffer_ptrs_dev)
        # Rank-local launch counter, zeroed once, never in the workspace (which every launch clears).
        self._seqctr = torch.zeros(1, device=self.device, dtype=torch.int32)
        self.seqctr_ptr = int(self._seqctr.data_ptr())
        self._views = {}
        self._fingerprint = (tuple(self._base), tuple(self._mc), self.pads_ptr, self.seqctr_ptr)
        torch.cuda.synchronize(self.device)

    def output(self, num_tokens: int, slot: int = 0) -> torch.Tensor:
        """The [num_tokens, hidden] view a launch writes: offset 0 of the slot, always."""
        key = (slot, num_tokens)
        v = self._views.get(key)
        if v is None:
            if num_tokens > self.max_tokens:
                raise ValueError(f"{num_tokens} tokens exceeds pool max {self.max_tokens}")
            v = self._bufs[slot][: num_tokens * self.hidden].view(num_tokens, self.hidden)
            self._views[key] = v
        return v

    def mc_ptr(self, slot: int = 0) -> int:
        return self._mc[slot]

    def base_ptr(self, slot: int = 0) -> int:
        return self._base[slot]

    def slot_buffer(self, slot: int = 0) -> torch.Tensor:
        return self._bufs[slot]

    def assert_stable(self) -> None:
        now = (tuple(int(b.data_ptr()) for b in self._bufs), tuple(int(h.multicast_ptr) for h in self._handles),
               int(self._flags_handle.buffer_ptrs_dev), int(self._seqctr.data_ptr()))
        if now != self._fingerprint:
            raise RuntimeError(f"pool pointers moved: {self._fingerprint} -> {now}")

    def describe(self) -> str:
        return (f"slots={self.nslots} max_tokens={self.max_tokens} hidden={self.hidden} pad_words={self.pad_words} "
                f"base0=0x{self._base[0]:x} mc0=0x{self._mc[0]:x} base0%512={self._base[0] % 512} "
                f"mc0%512={self._mc[0] % 512}")


class FusedTPPlan:
    """The agreed fused-path decision of this process plus the buffers it needs
    (monokernel_tp.py:148-323). `group` is the tensor-parallel process group.

    The vote is one MIN all-reduce of two integers (can this rank run fused / can it fold a
    residual); only if every rank says yes is the pool rendezvoused, so the rendezvous cannot
    meet a missing peer. `capability` lets a test inject the local answer."""

    def __init__(self, kernel: Optional[MonoKernel], group, hidden: int, max_tokens: int, nslots: int = 1,
                 enabled: bool = True, capability=None, build_pool: bool = True):
        import torch.distributed as dist

        self.kernel = kernel
        self.usable, self.fold_shared, self.reason, self.pool = False, False, "", None
        self.ncomm = env_ncomm(FUSED_NCOMM)
        self.hidden, self.max_tokens, self.nslots = int(hidden), int(max_tokens), max(1, int(nslots))
        self.rank, self.world = 0, 1
        self.chunks_by_tokens = {}
        self._caps = {}
        self._local_fold = False
        if not dist.is_available() or not dist.is_initialized():
            self.reason = "torch.distributed not initialized"
            return
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world < 2:
            self.reason = f"tp_size={self.world}"
            return
        self.chunks_by_tokens = {t: c for t, c in env_chunk_table(FUSED_CHUNKS_BY_TOKENS).items()
                                 if t <= self.max_tokens}
        local_ok, local_reason = capability(self) if capability is not None else self._local_capability(enabled)
        if not self._vote(local_ok):
            self.reason = local_reason if not local_ok else "a peer rank could not run fused"
            return
        if build_pool and not self._build_pool():
            return
        self.usable = True

    def _local_capability(self, enabled: bool):
        if not enabled:
            return False, "fused TP epilogue not enabled"
        if not torch.cuda.is_available():
            return False, "not CUDA"
        if not self.chunks_by_tokens:
            return False, f"no fused size fits max tokens {self.max_tokens}"
        if self.kernel is None:
            return False, "no monokernel binary loaded"
        caps = self.kernel.tp_caps()
        if not caps.get("usable"):
            return False, f"monokernel .so is not fused-TP capable: {caps}"
        if not caps.get("tp_has_devseq"):
            return False, "monokernel .so has no device sequence counter"
        want = max(self.chunks_by_tokens.values())
        if int(caps["tp_max_c"]) < want:
            return False, f"binary tp_max_c={caps['tp_max_c']} below required chunks={want}"
        if self.ncomm >= int(caps["grid_size"]):
            return False, f"ncomm={self.ncomm} not below grid_size={caps['grid_size']}"
        self._caps = caps
        self._local_fold = bool(caps.get("has_tp_residual"))
        return True, ""

    def _vote(self, local_ok: bool) -> bool:
        import torch.distributed as dist
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else "cpu"
        v = torch.tensor([1 if local_ok else 0, 1 if self._local_fold else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MIN, group=self.group)
        agreed = v.tolist()
        if int(agreed[0]) != 1:
            return False
        self.fold_shared = bool(int(agreed[1]))
        return True

    def _build_pool(self) -> bool:
        if torch.cuda.is_current_stream_capturing():
            self.reason = "the pool cannot be created during CUDA graph capture"
            return False
        caps = self._caps
        pad_words = self.kernel.tp_pad_words(int(caps["tp_max_c"]), int(caps["grid_size"]) - 1, self.world)
        try:
            self.pool = SymmOutputPool(self.group, self.max_tokens, self.hidden, pad_words, nslots=self.nslots)
        except Exception as e:  # a pool failure is a capability answer, the ordinary path remains
            self.reason = f"pool failed: {e}"
            return False
        return True

    def chunks_for(self, num_tokens: int) -> int:
        return self.chunks_by_tokens.get(int(num_tokens), 0)

    def output_is_fused(self, t: torch.Tensor) -> bool:
        """True when `t` is a pool view, i.e. already reduced across ranks (monokernel_tp.py:379-394)."""
        if self.pool is None or t is None:
            return False
        p = int(t.data_ptr())
        return any(p == self.pool.base_ptr(s) for s in range(self.pool.nslots))

    def fused_tp_launch(self, x, router_logits, w13, w13_scale, w2, w2_scale, top_k=8, renormalize=True,
                        e_score_correction_bias=None, residual=None, out_scale=1.0, slot=0, check=False,
                        expert_map=None):
        """Launch with the in-kernel reduce when this token count is in the table; returns the pool
        view holding the REDUCED output, or None when the ordinary path must be taken
        (monokernel_tp.py:421-514). Deliberately no try/except: after the vote there is no fallback."""
        if not self.usable:
            return None
        T = x.size(0)
        nchunk = self.chunks_for(T)
        if nchunk == 0:
            return None
        if (residual is not None or float(out_scale) != 1.0) and not self.fold_shared:
            return None
        out = self.pool.output(T, slot)
        self.pool.assert_stable()
        self.kernel.prefill_out(x, router_logits, w13, w13_scale, w2, w2_scale, out, top_k, renormalize,
                                e_score_correction_bias, tp_mc_ptr=self.pool.mc_ptr(slot),
                                tp_pads_ptr=self.pool.pads_ptr, tp_seqctr_ptr=self.pool.seqctr_ptr,
                                tp_rank=self.rank, tp_world=self.world, tp_nchunk=nchunk, tp_ncomm=self.ncomm,
                                tp_residual=residual, tp_out_scale=out_scale, check=check, expert_map=expert_map)
        return out
