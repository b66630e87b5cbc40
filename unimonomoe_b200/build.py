"""Compile the kernel once per geometry into unimonomoe_b200/lib/libprefill_mono_<variant>.so.

The geometry of a binary is fixed at compile time and read back through its
``prefill_wgmma_*`` accessors, as in the reference (kernel/build.sh:1-42, one variant per
binary); here the variants share one source and differ by -D macros.

    python -m unimonomoe_b200.build            # every variant
    python -m unimonomoe_b200.build qwen_w1    # one
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")

QWEN = dict(K=2048, H=2048, MODE=0)
DS = dict(K=7168, H=7168, MODE=2)

# name -> geometry. N_HALF is this rank's slice of the expert intermediate width,
# E_LOCAL the experts whose weights this rank holds.
VARIANTS = {
    "qwen_w1": dict(QWEN, N_HALF=512, E_LOCAL=256),   # Qwen3.5-35B-A3B-like, one GPU
    # the same geometry with the plain sigmoid + bias router (ROUTER_MODE 1 of the reference,
    # kernel/qwen_tp/src/prefill_mono_final_nb.cu:134-150): no expert groups
    "qwen_sig_w1": dict(QWEN, N_HALF=512, E_LOCAL=256, MODE=1),
    "qwen_tp2": dict(QWEN, N_HALF=256, E_LOCAL=256),
    "qwen_tp4": dict(QWEN, N_HALF=128, E_LOCAL=256),
    "qwen_ep2": dict(QWEN, N_HALF=512, E_LOCAL=128),
    "qwen_ep4": dict(QWEN, N_HALF=512, E_LOCAL=64),
    "qwen_ep8": dict(QWEN, N_HALF=512, E_LOCAL=32),
    "ds_tp8": dict(DS, N_HALF=256, E_LOCAL=256),      # DeepSeek-V3-like, 1/8 width shard
    "ds_tp4": dict(DS, N_HALF=512, E_LOCAL=256),
    "ds_tp2": dict(DS, N_HALF=1024, E_LOCAL=256),     # intermediate processed in 2 chunks of 512 columns
    "ds_w1": dict(DS, N_HALF=2048, E_LOCAL=256),      # full width on one GPU: 4 chunks
    # DeepSeek-V3 expert parallel over 8 ranks: 32 local experts at full width. The reference stopped here
    # because the [128, 2048] e4m3 intermediate does not fit in shared memory
    # (research_archive/reports/ds3_ep_monokernel_result.md:118-153); processed in 4 chunks of 512 columns
    "ds_ep8": dict(DS, N_HALF=2048, E_LOCAL=32),
    # tiles scheduled as pairs on clusters of two CTAs (tcgen05 cta_group::2); measured equal in speed to
    # qwen_w1 at 16384 tokens (fewer L2 weight bytes per SM, but 11 % more padded rows), so not the default
    "qwen_w1_pair": dict(QWEN, N_HALF=512, E_LOCAL=256, PAIR=1),
}

# development variants (not built by default): the stall-counter build and the builds that leave a piece of the
# expert phase out (wrong results by design; their run-time differences split the phase)
DEV_VARIANTS = {
    "qwen_w1_prof": dict(QWEN, N_HALF=512, E_LOCAL=256, PROFILE=1),
    "qwen_w1_trace": dict(QWEN, N_HALF=512, E_LOCAL=256, PROFILE=1, DEFS=("MONO_TRACE",)),
    **{f"qwen_w1_abl{m}": dict(QWEN, N_HALF=512, E_LOCAL=256, ABLATE=m) for m in (1, 4, 7, 15, 23, 31, 39, 71, 199, 256)},
}

SOURCES = ["mono_kernel.cu", "ptx_sm100.cuh", "pair_sm100.cuh", "bounded_wait.cuh", "route_math.cuh"]


def lib_path(variant: str) -> str:
    return os.path.join(LIBDIR, f"libprefill_mono_{variant}.so")


def _stale(out: str) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(os.path.join(CSRC, s)) > t for s in SOURCES) or os.path.getmtime(__file__) > t


def build_variant(variant: str, force: bool = False, verbose: bool = False) -> str:
    g = VARIANTS.get(variant) or DEV_VARIANTS[variant]
    out = lib_path(variant)
    os.makedirs(LIBDIR, exist_ok=True)
    if not force and not _stale(out):
        return out
    cmd = [
        os.environ.get("NVCC", "nvcc"), "-O3", "-std=c++17",
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--expt-relaxed-constexpr",
        "-Xptxas", "-v", "-shared", "-Xcompiler", "-fPIC",
        f"-DMONO_K_DIM={g['K']}", f"-DMONO_H_DIM={g['H']}", f"-DMONO_N_HALF={g['N_HALF']}",
        f"-DMONO_E_LOCAL={g['E_LOCAL']}", f"-DMONO_ROUTER_MODE={g['MODE']}", f"-DMONO_EPI_WGS={g.get('EPI_WGS', 2)}", f"-DMONO_NSPLIT={g.get('NSPLIT', 1)}",
        *(["-DMONO_PROFILE"] if g.get("PROFILE") else []), f"-DMONO_ABLATE={g.get('ABLATE', 0)}",
        f"-DMONO_PAIR={g.get('PAIR', 0)}", *[f"-D{d}" for d in g.get("DEFS", ())],
        os.path.join(CSRC, "mono_kernel.cu"), "-o", out,
    ]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = r.stdout + r.stderr
    with open(out + ".log", "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {variant}:\n{log}")
    if verbose:
        for line in log.splitlines():
            if "registers" in line or "spill" in line:
                print(f"[{variant}] {line.strip()}")
    return out


def build_microbench() -> str:
    """The hardware micro-benchmarks of csrc/sm100_microbench.cu as an executable (development tool)."""
    os.makedirs(LIBDIR, exist_ok=True)
    out = os.path.join(LIBDIR, "sm100_microbench")
    cmd = [os.environ.get("NVCC", "nvcc"), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-I", CSRC, os.path.join(CSRC, "sm100_microbench.cu"), "-o", out]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for the micro-benchmarks:\n" + r.stdout + r.stderr)
    return out


def build_all(names=None, force: bool = False, verbose: bool = False) -> dict:
    names = list(names or VARIANTS)
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as ex:
        outs = list(ex.map(lambda n: build_variant(n, force, verbose), names))
    return dict(zip(names, outs))


if __name__ == "__main__":
    sel = [a for a in sys.argv[1:] if not a.startswith("-")]
    if "microbench" in sel:
        print("microbench ->", build_microbench())
        sel.remove("microbench")
        if not sel:
            sys.exit(0)
    res = build_all(sel or None, force="--force" in sys.argv, verbose=True)
    for k, v in res.items():
        print(k, "->", v)
