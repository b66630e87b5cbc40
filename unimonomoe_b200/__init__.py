"""B200-native (sm_100a) single-launch FP8 MoE prefill layer behind the reference's
loader / C-ABI surface. See loader.py for the host API and csrc/ for the kernel."""
from .loader import (MOE_MONOKERNEL_PREFILL_MAX_TOKENS, MonoKernel, moe_monokernel_prefill,  # noqa: F401
                     moe_monokernel_prefill_out, monokernel_validate, prefill_monokernel_geometry,
                     prefill_monokernel_tp_caps, prefill_monokernel_tp_pad_words, variant_path)
