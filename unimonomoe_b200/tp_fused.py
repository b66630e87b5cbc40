"""Host side of the all-reduce that runs inside the prefill kernel.

When the kernel is given a multicast window it turns its last `ncomm` CTAs into communication
CTAs: they reduce finished column chunks of the [T, H] bf16 output across the ranks through
NVLS (`multimem.ld_reduce` / `multimem.st`) while the other CTAs are still summing partial rows.
That makes the launch itself a collective, so three things have to be settled on the host,
once, before any launch:

* where the output lives: symmetric memory that every rank maps (`SymmOutputPool`), one
  maximum-size window per slot, always used from offset 0, plus a window of barrier words and a
  launch counter on the device;
* whether this process may use the path at all: a launch whose peer never launches would sit in
  the kernel's rank barrier until its bounded wait gives up, so "can I" is answered by every rank
  and combined with a MIN all-reduce (`FusedTPPlan`); after a yes there is no local fallback;
* for which token counts, in how many chunks and with how many communication CTAs
  (`ReducePolicy`, overridable through the environment variables the reference reads).

The public names follow the reference's modules so that its runner glue finds them
(fused_moe/symm_output_pool.py: SymmOutputPool and its accessors; fused_moe/monokernel_tp.py:
the plan, `fused_tp_plan`, `reset_fused_tp_plan`, `output_is_fused`, `fused_tp_launch`, and the
VLLM_PREFILL_MONOKERNEL_TP_* variables). Unlike the reference the same reduce also serves
expert-parallel ranks (pass `expert_map`), the kernel's waits are bounded, and the pool is
sized from the kernel's own `tp_pad_words` accessor.

Nothing here allocates or communicates on the per-call path.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, Mapping, NamedTuple, Optional

import torch

from .loader import MonoKernel

ENV_CHUNKS = "VLLM_PREFILL_MONOKERNEL_TP_CHUNKS"
ENV_NCOMM = "VLLM_PREFILL_MONOKERNEL_TP_NCOMM"
ENV_FOLD = "VLLM_PREFILL_MONOKERNEL_TP_FOLD_SHARED"

# Exact token counts that take the in-kernel reduce, and the chunks it is released in
# (the reference's table, monokernel_tp.py:79-82: sizes it measured as wins). Other sizes take the
# ordinary path.
FUSED_CHUNKS_BY_TOKENS = {8192: 4, 16384: 8}
# Communication CTAs. The reference settled on 14 of its 132 (monokernel_tp.py:87).
FUSED_NCOMM = 14
# Group size at which the kernel reduces by direct peer loads instead of the multicast alias: with two ranks the
# switch would fetch this rank's own copy over NVLink as well, one and a half times the traffic for the same bits.
# From three ranks on the in-switch reduction moves less than peer loads would.
PEER_REDUCE_WORLD = 2


def _positive_int(text: str, what: str) -> int:
    value = int(text)
    if value < 1:
        raise ValueError(f"{what} must be a positive integer, got {text!r}")
    return value


def env_chunk_table(default: Mapping[int, int]) -> dict:
    """The chunk table after VLLM_PREFILL_MONOKERNEL_TP_CHUNKS: empty keeps `default`; one integer
    sets that chunk count for every size of `default`; `T:C[,T:C...]` replaces the table. A value
    that does not parse, or a chunk count below one, raises ValueError."""
    text = os.environ.get(ENV_CHUNKS, "").strip()
    if not text:
        return dict(default)
    if ":" in text:
        table = {}
        for pair in text.split(","):
            tokens, _, chunks = pair.partition(":")
            table[_positive_int(tokens, ENV_CHUNKS)] = _positive_int(chunks, ENV_CHUNKS)
        return table
    chunks = _positive_int(text, ENV_CHUNKS)
    return dict.fromkeys(default, chunks)


def env_ncomm(default: int) -> int:
    text = os.environ.get(ENV_NCOMM, "").strip()
    return _positive_int(text, ENV_NCOMM) if text else int(default)


def env_fold_shared() -> bool:
    """VLLM_PREFILL_MONOKERNEL_TP_FOLD_SHARED: fold `out_scale * routed + residual` into the reduce
    (default on; "0", "false", "no", "off" or empty switch it off)."""
    return os.environ.get(ENV_FOLD, "1").strip().lower() not in ("", "0", "false", "no", "off")


@dataclass(frozen=True)
class ReducePolicy:
    """For which token counts the reduce runs inside the kernel and how it is shaped."""
    chunks_by_tokens: Mapping[int, int] = field(default_factory=lambda: dict(FUSED_CHUNKS_BY_TOKENS))
    ncomm: int = FUSED_NCOMM
    fold: bool = True

    @classmethod
    def from_env(cls, max_tokens: Optional[int] = None) -> "ReducePolicy":
        table = env_chunk_table(FUSED_CHUNKS_BY_TOKENS)
        if max_tokens is not None:
            table = {t: c for t, c in table.items() if t <= max_tokens}
        return cls(table, env_ncomm(FUSED_NCOMM), env_fold_shared())

    def chunks_for(self, num_tokens: int) -> int:
        return int(self.chunks_by_tokens.get(int(num_tokens), 0))

    @property
    def max_chunks(self) -> int:
        return max(self.chunks_by_tokens.values(), default=0)


class Capability(NamedTuple):
    """One rank's answer to "can you run the in-kernel reduce", before the ranks compare notes."""
    ok: bool
    fold: bool = False
    why: str = ""


# ---------------------------------------------------------------------------------- the pool
class _Window:
    """One symmetric allocation: the same size on every rank, rendezvoused over the group."""

    def __init__(self, numel: int, dtype, device, group_name: str):
        import torch.distributed._symmetric_memory as symm

        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.tensor, group_name)

    @property
    def local(self) -> int:
        return int(self.tensor.data_ptr())

    @property
    def multicast(self) -> int:
        return int(self.handle.multicast_ptr)

    @property
    def peer_table(self) -> int:
        """Device address of the array of every rank's address of this window."""
        return int(self.handle.buffer_ptrs_dev)


class SymmOutputPool:
    """The symmetric memory one process group needs for the in-kernel reduce, for its lifetime.

    * `nslots` output windows of `max_tokens * hidden` bf16. A launch for T tokens writes rows
      [0, T) of a slot: the kernel addresses the multicast alias with the same offsets as the
      local buffer, so a view at any other offset would reduce the wrong bytes on the peers.
    * one window of `pad_words` 32-bit barrier words (the kernel's `tp_pad_words(C, ncomm, world)`
      for the largest C and ncomm it accepts), zeroed once. It is a separate window, not the
      signal pad torch attaches to a handle (kernel/qwen_tp/src/prefill_mono_final_nb.cu:1540-1542).
    * one 32-bit launch counter in ordinary device memory, zeroed once. The kernel increments it,
      so replays of a captured graph see fresh sequence numbers; it must not live in the workspace,
      which every launch clears.

    Construct on every rank of the group at the same point of the program (the rendezvous is a
    collective), never per call and never during stream capture. Mirrors the surface of
    fused_moe/symm_output_pool.py:78-199.
    """

    def __init__(self, group, max_tokens: int, hidden: int, pad_words: int, nslots: int = 1, device=None):
        self.group_name = group if isinstance(group, str) else group.group_name
        self.max_tokens, self.hidden, self.nslots = int(max_tokens), int(hidden), int(nslots)
        self.pad_words = int(pad_words)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        if min(self.max_tokens, self.hidden, self.nslots, self.pad_words) < 1:
            raise ValueError("pool dimensions must be positive")
        self._outputs = [_Window(self.max_tokens * self.hidden, torch.bfloat16, self.device, self.group_name)
                         for _ in range(self.nslots)]
        missing = [i for i, w in enumerate(self._outputs) if not w.multicast]
        if missing:
            raise RuntimeError(f"no multicast address for output slot(s) {missing}: the in-kernel reduce needs NVLS")
        self._signals = _Window(self.pad_words, torch.int32, self.device, self.group_name)
        self._signals.tensor.zero_()
        self._launches = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self._pinned = self._addresses()

    # ---- what a launch needs
    @property
    def pads_ptr(self) -> int:
        return self._signals.peer_table

    @property
    def seqctr_ptr(self) -> int:
        return int(self._launches.data_ptr())

    def mc_ptr(self, slot: int = 0) -> int:
        return self._outputs[slot].multicast

    def base_ptr(self, slot: int = 0) -> int:
        return self._outputs[slot].local

    def peers_ptr(self, slot: int = 0) -> int:
        """Device address of the array of every rank's address of this slot (for the two-rank peer-load reduce)."""
        return self._outputs[slot].peer_table

    def slot_buffer(self, slot: int = 0) -> torch.Tensor:
        return self._outputs[slot].tensor

    def output(self, num_tokens: int, slot: int = 0) -> torch.Tensor:
        """Rows [0, num_tokens) of a slot as a [num_tokens, hidden] tensor (no allocation)."""
        if not 0 < int(num_tokens) <= self.max_tokens:
            raise ValueError(f"{num_tokens} tokens do not fit a pool sized for {self.max_tokens}")
        return self._outputs[slot].tensor.narrow(0, 0, int(num_tokens) * self.hidden).view(int(num_tokens), self.hidden)

    def owns(self, t: Optional[torch.Tensor]) -> bool:
        """True when `t` starts at the base of one of the slots, i.e. holds an already reduced output."""
        return t is not None and any(int(t.data_ptr()) == w.local for w in self._outputs)

    def bytes_per_slot(self) -> int:
        return self.max_tokens * self.hidden * 2

    # ---- integrity
    def _addresses(self) -> tuple:
        return (tuple((w.local, w.multicast, w.peer_table) for w in self._outputs), self._signals.peer_table,
                self.seqctr_ptr)

    def assert_stable(self) -> None:
        """A captured graph holds these addresses; raise if any of them has changed since construction."""
        now = self._addresses()
        if now != self._pinned:
            raise RuntimeError(f"symmetric pool addresses changed since construction: {self._pinned} -> {now}")

    def describe(self) -> str:
        first = self._outputs[0]
        return (f"{self.nslots} slot(s) x {self.bytes_per_slot() >> 20} MiB ({self.max_tokens} tokens x {self.hidden}), "
                f"{self.pad_words} barrier words, local 0x{first.local:x} (mod 512 = {first.local % 512}), "
                f"multicast 0x{first.multicast:x} (mod 512 = {first.multicast % 512})")


# ---------------------------------------------------------------------------------- the plan
def probe_capability(kernel: Optional[MonoKernel], policy: ReducePolicy, enabled: bool = True) -> Capability:
    """This rank's own answer (no communication). The first failing requirement names itself."""
    caps = kernel.tp_caps() if kernel is not None else {}
    requirements = (
        (enabled, "the in-kernel reduce is switched off"),
        (torch.cuda.is_available(), "no CUDA device"),
        (policy.max_chunks > 0, "no token count of the policy fits the configured maximum"),
        (kernel is not None, "no kernel binary loaded"),
        (bool(caps.get("usable")), f"the binary lacks the fused entry point or its accessors: {caps}"),
        (bool(caps.get("tp_has_devseq")), "the binary has no device-side launch counter"),
        (int(caps.get("tp_max_c") or 0) >= policy.max_chunks,
         f"the policy asks for {policy.max_chunks} chunks, the binary allows {caps.get('tp_max_c')}"),
        (policy.ncomm < int(caps.get("grid_size") or 0),
         f"{policy.ncomm} communication CTAs leave no CTA of {caps.get('grid_size')} to compute"),
    )
    for satisfied, why in requirements:
        if not satisfied:
            return Capability(False, False, why)
    return Capability(True, policy.fold and bool(caps.get("has_tp_residual")), "")


def agree(group, flags) -> list:
    """Element-wise minimum of integer flags over the group: a 1 survives only if every rank said 1."""
    import torch.distributed as dist

    on_gpu = dist.get_backend(group) == "nccl"
    t = torch.tensor([int(bool(f)) for f in flags], dtype=torch.int32,
                     device=torch.device("cuda", torch.cuda.current_device()) if on_gpu else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return [bool(v) for v in t.tolist()]


class FusedTPPlan:
    """The group's decision about the in-kernel reduce, plus the pool when the answer is yes.

    group       the tensor- (or expert-) parallel process group
    capability  optional replacement for `probe_capability`, called as capability(plan) and returning a
                `Capability`; lets a test play a rank that cannot
    build_pool  False: decide only (CPU tests)

    `usable` is identical on every rank. `reason` says why not, from this rank's point of view.
    Mirrors the role of `_FusedTPPlan` (monokernel_tp.py:140-330).
    """

    def __init__(self, kernel: Optional[MonoKernel], group, hidden: int, max_tokens: int, nslots: int = 1,
                 enabled: bool = True, capability: Optional[Callable[["FusedTPPlan"], Capability]] = None,
                 build_pool: bool = True, policy: Optional[ReducePolicy] = None):
        import torch.distributed as dist

        self.kernel, self.group, self.pool = kernel, group, None
        self.hidden, self.max_tokens, self.nslots = int(hidden), int(max_tokens), max(1, int(nslots))
        self.policy = policy if policy is not None else ReducePolicy.from_env(self.max_tokens)
        self.chunks_by_tokens = dict(self.policy.chunks_by_tokens)   # callers may add measured sizes
        self.ncomm = self.policy.ncomm
        self.usable = self.fold_shared = False
        self.rank, self.world, self.reason = 0, 1, ""
        if not (dist.is_available() and dist.is_initialized()):
            self.reason = "torch.distributed is not initialized"
            return
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world < 2:   # comes from the configuration, identical everywhere: may skip the vote
            self.reason = f"a group of {self.world} has nothing to reduce"
            return
        mine = capability(self) if capability is not None else probe_capability(kernel, self.policy, enabled)
        everyone_ok, everyone_folds = agree(group, (mine.ok, mine.fold))
        if not everyone_ok:
            self.reason = mine.why if not mine.ok else "a peer rank cannot run the in-kernel reduce"
            return
        self.fold_shared = everyone_folds
        if build_pool:
            failure = self._make_pool()
            # the rendezvous inside is a collective: it fails everywhere or nowhere, but a later local step
            # might not, so the outcome is agreed as well
            if not agree(group, (failure is None,))[0]:
                self.pool = None
                self.reason = failure or "a peer rank could not create the symmetric pool"
                return
        self.usable = True

    def _make_pool(self) -> Optional[str]:
        if torch.cuda.is_current_stream_capturing():
            return "the symmetric pool cannot be created during stream capture"
        caps = self.kernel.tp_caps()
        # sized for the largest chunk count and communication-CTA count the binary accepts, so the
        # policy can change without a new rendezvous
        words = self.kernel.tp_pad_words(int(caps["tp_max_c"]), int(caps["grid_size"]) - 1, self.world)
        try:
            self.pool = SymmOutputPool(self.group, self.max_tokens, self.hidden, words, nslots=self.nslots)
        except Exception as exc:
            return f"symmetric pool: {exc}"
        return None

    def chunks_for(self, num_tokens: int) -> int:
        return int(self.chunks_by_tokens.get(int(num_tokens), 0))

    def output_is_fused(self, t: Optional[torch.Tensor]) -> bool:
        """Whether `t` is a pool slot, hence already summed over the group: answered from the address,
        which a captured graph replays unchanged (monokernel_tp.py:379-394)."""
        return self.pool is not None and self.pool.owns(t)

    def fused_tp_launch(self, x, router_logits, w13, w13_scale, w2, w2_scale, top_k=8, renormalize=True,
                        e_score_correction_bias=None, residual=None, out_scale=1.0, slot=0, check=False,
                        expert_map=None):
        """Launch with the reduce inside the kernel and return the pool view that will hold the REDUCED
        output; None when this call has to take the ordinary path (a rank-uniform outcome: it depends on
        the agreed plan, the token count and the fold request only). A failure after that point raises:
        the peers are already inside the collective (monokernel_tp.py:421-514)."""
        if not self.usable:
            return None
        tokens = int(x.size(0))
        nchunk = self.chunks_for(tokens)
        wants_fold = residual is not None or float(out_scale) != 1.0
        if nchunk == 0 or (wants_fold and not self.fold_shared):
            return None
        out = self.pool.output(tokens, slot)
        self.pool.assert_stable()
        self.kernel.prefill_out(x, router_logits, w13, w13_scale, w2, w2_scale, out, top_k, renormalize,
                                e_score_correction_bias, tp_mc_ptr=self.pool.mc_ptr(slot),
                                tp_pads_ptr=self.pool.pads_ptr, tp_seqctr_ptr=self.pool.seqctr_ptr,
                                tp_rank=self.rank, tp_world=self.world, tp_nchunk=nchunk, tp_ncomm=self.ncomm,
                                tp_residual=residual, tp_out_scale=out_scale, check=check, expert_map=expert_map,
                                tp_peers_ptr=self.pool.peers_ptr(slot) if self.world == PEER_REDUCE_WORLD else 0)
        return out


# ---------------------------------------------------------------------------------- process-wide plan
_plan: Optional[FusedTPPlan] = None


def fused_tp_plan(kernel: MonoKernel, group, hidden: int, max_tokens: int, nslots: int = 1,
                  enabled: bool = True) -> FusedTPPlan:
    """The process's one plan, created at first use (monokernel_tp.py:362-368). Call it at the same point
    on every rank: creation votes and rendezvouses."""
    global _plan
    if _plan is None:
        _plan = FusedTPPlan(kernel, group, hidden, max_tokens, nslots, enabled)
    return _plan


def reset_fused_tp_plan() -> None:
    """Forget the process-wide plan and release its pool (tests that build several configurations)."""
    global _plan
    _plan = None


def output_is_fused(t: Optional[torch.Tensor]) -> bool:
    """Module-level form of `FusedTPPlan.output_is_fused` for the process-wide plan."""
    return _plan is not None and _plan.usable and _plan.output_is_fused(t)
