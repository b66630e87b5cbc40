"""CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Python face of ``moe_oracle.c`` (routing, stable sort, activation quantisation and the
path-faithful expert computation) plus the reference's fp64 dequantised MoE in torch.
Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg may import this
module; the product package never does.

Parity pin: see ``tests/golden/`` -- vectors produced by executing the reference's own
torch routines (research_archive/ds3_acc.py:242-313, validation/ep4_acc.py:183-217) on CPU.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile moe_oracle.c into oracle/liboracle.so (gcc, a few seconds)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "moe_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        L.oracle_e4m3_decode.restype = ctypes.c_float
        L.oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
        L.oracle_e4m3_encode.restype = ctypes.c_uint8
        L.oracle_e4m3_encode.argtypes = [ctypes.c_float]
        L.oracle_det_expf.restype = ctypes.c_float
        L.oracle_det_expf.argtypes = [ctypes.c_float]
        L.oracle_float_to_bf16.restype = ctypes.c_uint16
        L.oracle_float_to_bf16.argtypes = [ctypes.c_float]
        L.oracle_num_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _np(t, dtype):
    """torch tensor / ndarray -> contiguous ndarray of dtype (bit views for bf16 / fp8)."""
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        elif t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        t = t.numpy()
    a = np.ascontiguousarray(t)
    if dtype == np.uint16 and a.dtype == np.int16:
        a = a.view(np.uint16)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


def e4m3_decode_table() -> np.ndarray:
    L = lib()
    return np.array([L.oracle_e4m3_decode(i) for i in range(256)], dtype=np.float32)


def route(logits, top_k=8, mode=0, bias=None, n_group=8, topk_group=4, expert_map=None):
    """Returns (ids [T,k] int32 -- local ids when expert_map is given, weights [T,k] fp32,
    global ids [T,k] int32). Restates kernel/qwen_tp/src/prefill_mono_final_nb.cu:1025-1185."""
    lg = _np(logits, np.float32)
    T, E = lg.shape
    b = None if bias is None else _np(bias, np.float32)
    m = None if expert_map is None else _np(expert_map, np.int32)
    ids = np.empty((T, top_k), np.int32)
    gids = np.empty((T, top_k), np.int32)
    w = np.empty((T, top_k), np.float32)
    lib().oracle_route(_p(lg), T, E, top_k, mode, _p(b), n_group, topk_group, _p(m), _p(ids), _p(w), _p(gids))
    return ids, w, gids


def sort_slots(ids, n_local):
    """Stable counting sort of flat slot indices by local expert id.
    Returns (counts [n_local], offsets [n_local+1], sorted [n_owned])."""
    ids = _np(ids, np.int32)
    T, k = ids.shape
    counts = np.zeros(n_local, np.int32)
    offsets = np.zeros(n_local + 1, np.int32)
    srt = np.full(T * k, -1, np.int32)
    lib().oracle_sort(_p(ids), T, k, n_local, _p(counts), _p(offsets), _p(srt))
    return counts, offsets, srt[: int(offsets[-1])]


def quant_act(act_bf16):
    """bf16 [T,K] -> (e4m3 bytes [T,K] uint8, scales [T,K/128] fp32)."""
    a = _np(act_bf16, np.uint16)
    T, K = a.shape
    q = np.empty((T, K), np.uint8)
    s = np.empty((T, K // 128), np.float32)
    lib().oracle_quant_act(_p(a), T, K, _p(q), _p(s))
    return q, s


def moe_path(tokens, act_q, act_scale, ids, weights, w13, w13_scale, w2, w2_scale, out_scale=1.0,
             residual=None, want_dumps=False, chunk_cols=512):
    """Path-faithful expert computation for the listed tokens. Returns out [n_sel,H] as a
    bf16 torch tensor, and with want_dumps also (partial bf16 [n_sel*k*nch,H], acc fp32
    [n_sel*k, 2*n_half], inter uint8 [n_sel*k, n_half], iscale fp32 [n_sel*k, n_half/128]).
    An intermediate wider than chunk_cols columns yields one bf16 partial row per chunk (nch of them),
    as the kernel processes it."""
    tokens = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
    act_q = _np(act_q, np.uint8)
    act_scale = _np(act_scale, np.float32)
    ids = _np(ids, np.int32)
    weights = _np(weights, np.float32)
    w13 = _np(w13, np.uint8)
    w2 = _np(w2, np.uint8)
    w13_scale = _np(w13_scale, np.float32)
    w2_scale = _np(w2_scale, np.float32)
    n_local, n_up, K = w13.shape
    _, H, n_half = w2.shape
    assert n_up == 2 * n_half
    top_k = ids.shape[1]
    n_sel = len(tokens)
    res = None if residual is None else _np(residual, np.uint16)
    out = np.empty((n_sel, H), np.uint16)
    part = acc = inter = isc = None
    if want_dumps:
        nch = max(1, n_half // chunk_cols) if n_half > chunk_cols else 1
        part = np.empty((n_sel * top_k * nch, H), np.uint16)
        acc = np.empty((n_sel * top_k, n_up), np.float32)
        inter = np.empty((n_sel * top_k, n_half), np.uint8)
        isc = np.empty((n_sel * top_k, n_half // 128), np.float32)
    lib().oracle_moe_path(_p(tokens), n_sel, top_k, K, H, n_half, n_local, _p(act_q), _p(act_scale), _p(ids),
                          _p(weights), _p(w13), _p(w13_scale), _p(w2), _p(w2_scale), ctypes.c_float(out_scale),
                          _p(res), _p(out), _p(part), _p(acc), _p(inter), _p(isc), int(chunk_cols))
    out_t = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)
    if want_dumps:
        return out_t, torch.from_numpy(part.view(np.int16)).view(torch.bfloat16), acc, inter, isc
    return out_t


# ---------------------------------------------------------------------------- fp64 tier
def dequant_block(w_fp8: torch.Tensor, scale: torch.Tensor, dtype=torch.float64) -> torch.Tensor:
    """Block-FP8 [rows, cols] with one scale per [128,128] block -> dense matrix
    (validation/ep4_acc.py:183-186)."""
    rows, cols = w_fp8.shape
    s = scale.to(dtype).repeat_interleave(128, 0).repeat_interleave(128, 1)[:rows, :cols]
    return w_fp8.to(dtype) * s


def moe_fp64(hs, ids, weights, w13, w13_scale, w2, w2_scale, dtype=torch.float64):
    """The routed MoE layer on dequantised weights and unquantised activations, on the given
    routing (validation/ep4_acc.py:189-217). ids are local; negative ids are skipped."""
    T = hs.shape[0]
    n_local, n_up, K = w13.shape
    n_half = n_up // 2
    H = w2.shape[1]
    h = hs.to(dtype)
    ids = torch.as_tensor(ids).long()
    tw = torch.as_tensor(weights).to(dtype)
    out = torch.zeros(T, H, dtype=dtype)
    for e in torch.unique(ids).tolist():
        if e < 0:
            continue
        sel = ids == e
        rows = sel.any(1).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        x = h[rows]
        y = x @ dequant_block(w13[e], w13_scale[e], dtype).T
        gate, up = y[:, :n_half], y[:, n_half:]
        act = (gate * torch.sigmoid(gate)) * up
        z = act @ dequant_block(w2[e], w2_scale[e], dtype).T
        w = torch.where(sel[rows], tw[rows], torch.zeros((), dtype=dtype)).sum(1, keepdim=True)
        out[rows] += z * w
    return out


def shared_expert_fp(hs, sh, dtype=torch.float64):
    """Gated shared expert: sigmoid(x . g) * down(SiLU(gate x) * up x) on dequantised block-FP8
    weights (upstream vLLM qwen2_moe.py; the reference pins only how its output is folded)."""
    x = hs.to(dtype)
    w13 = dequant_block(sh["w13"], sh["w13_scale"], dtype)
    w2 = dequant_block(sh["w2"], sh["w2_scale"], dtype)
    n_half = w13.shape[0] // 2
    y = x @ w13.T
    act = torch.nn.functional.silu(y[:, :n_half]) * y[:, n_half:]
    z = act @ w2.T
    if sh.get("gate") is not None:
        z = torch.sigmoid(x @ sh["gate"].to(dtype).T) * z
    return z


def rel_cos(a, b):
    """rel-L2 and cosine from fp64 dot products (validation/ep4_acc.py:220-223)."""
    a = torch.as_tensor(a).to(torch.float64).flatten()
    b = torch.as_tensor(b).to(torch.float64).flatten()
    return float((a - b).norm() / b.norm()), float(torch.dot(a, b) / (a.norm() * b.norm()))


def parity_metrics(out, ref):
    """The acceptance numbers: max|err| / rms(ref), cosine, rel-L2."""
    o = torch.as_tensor(out).to(torch.float64)
    r = torch.as_tensor(ref).to(torch.float64)
    rms = float(r.pow(2).mean().sqrt())
    mae = float((o - r).abs().max())
    rl2, cs = rel_cos(o, r)
    return {"max_abs_over_rms": mae / max(rms, 1e-300), "cos": cs, "rel_l2": rl2, "rms_ref": rms}
