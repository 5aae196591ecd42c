"""Python faces of the CUDA kernels in this folder.

Every function takes CUDA tensors, checks dtypes, shapes and contiguity, and launches on the
current stream.  There is no CPU path and no library stand-in: a tensor that is not on a CUDA
device, or a library that cannot be built, raises.  bfloat16 matrix products go to cuBLAS through
``torch.mm`` where the reference's engine uses a library product (lily/layers/quantization/
base.py:69-72); float32 products use this folder's own FFMA kernel so that no reduced-precision
matrix mode can slip in.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Callable, Optional, Sequence, Tuple

import torch

from lily_b200.csrc import build as _build

_F32, _BF16 = 0, 1
_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "lily_embed": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "lily_logit_transform": [_vp, _sz, _f, _f, _vp],
    "lily_scatter_tokens": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_add_rmsnorm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i, _i, _sz, _vp],
    "lily_silu_mul": [_vp, _vp, _i, _i, _i, _i, _i, _i, _sz, _i, _f, _f, _vp],
    "lily_gemm_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp],
    "lily_qk_norm_rope_write": [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                _i, _i, _i, _i, _i, _sz, _i, _i, _f, _vp, _i, _vp],
    "lily_skinny_gemm": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lily_skinny_swiglu": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _f, _vp],
    "lily_cast": [_vp, _i, _vp, _i, _sz, _vp],
    "lily_gemm_fp32": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "lily_attention_prefill_simt": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _f, _i, _i, _i, _i, _vp],
    "lily_attention_decode_simt": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _f, _i, _i, _i, _i, _vp],
    "lily_attention_combine": [_vp, _vp, _i, _i, _i, _i, _i, _vp],
    "lily_attention_prefill_mma": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i, _i, _vp],
    "lily_attention_prefill_tc": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _f, _i, _vp],
    "lily_attention_decode_mma": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _f, _i, _i, _i, _vp],
    "lily_attention_decode_mma_fused": [_vp, _i, _sz, _i, _vp, _vp, _i, _f, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _vp, _vp,
                                        _i, _i, _i, _i, _i, _i, _i, _f, _i, _f, _vp],
    "lily_sigmoid_gate": [_vp, _i, _vp, _i, _i, _sz, _sz, _vp],
    "lily_normed_mean": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _sz, _vp, _i, _i, _f, _f, _vp],
    "lily_causal_conv_silu": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _vp],
    "lily_causal_conv": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _vp],
    "lily_add_normed_rmsnorm": [_vp, _vp, _i, _i, _sz, _vp, _f, _f, _vp, _i, _vp, _i, _vp, _i, _i, _f, _i, _i, _vp],
    "lily_head_mix": [_vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "lily_delta_rule": [_vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _i, _vp],
    "lily_selective_scan": [_vp, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp],
    "lily_selective_combine": [_vp, _sz, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp],
    "lily_activation": [_vp, _i, _i, _sz, _vp, _i, _sz, _i, _vp],
    "lily_diff_prepare": [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp],
    "lily_diff_combine": [_vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _f, _f, _f, _i, _vp],
    "lily_ssd_scan": [_vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp,
                      _i, _vp, _vp, _i, _vp],
    "lily_ssd_combine": [_vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "lily_gated_group_rmsnorm": [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "lily_latent_attention_prefill_mma": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
    "lily_latent_attention_decode_mma": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
    "lily_add_rmsnorm_multi": [_vp, _vp, _i, _i, _sz, _vp, _i, _i, _sz, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _vp],
    "lily_gemm_fp32_heads": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _sz, _sz, _sz, _vp],
    "lily_token_shift_mix": [_vp, _i, _i, _vp, _i, _vp, _sz, _sz, _vp, _vp, _vp, _vp, _i, _vp],
    "lily_wkv_decay": [_vp, _i, _i, _vp, _vp, _i, _vp, _vp],
    "lily_wkv_scan": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "lily_wkv_combine": [_vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "lily_group_rmsnorm_gate": [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "lily_latent_prepare": [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _vp,
                            _i, _i, _vp],
    "lily_latent_query": [_vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp],
    "lily_head_gate": [_vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _vp],
    "lily_moe_route": [_vp, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _i, _vp],
    "lily_moe_align": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp],
    "lily_moe_gemm": [_i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _f, _f, _i, _vp],
    "lily_moe_combine": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp],
    "lily_moe_gather": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _i, _vp],
    "lily_moe_activation": [_vp, _i, _i, _vp, _f, _f, _i, _vp],
    "lily_moe_combine_rows": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp],
    "lily_argmax": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_apply_penalties": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_top_logprobs": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_sample": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
}

_lib = None


class KernelError(RuntimeError):
    pass


def library():
    """Loads (building first if needed) the kernel library and declares its entry points."""
    global _lib
    if _lib is None:
        lib = _build.load()
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i
        lib.lily_attention_prefill_simt_rows.restype = _i
        lib.lily_argmax_chunks.argtypes = [_i, _i]
        lib.lily_argmax_chunks.restype = _i
        lib.lily_skinny_gemm_max_rows.restype = _i
        lib.lily_skinny_gemm_splits.argtypes = [_i, _i, _i]
        lib.lily_skinny_gemm_splits.restype = _i
        lib.lily_skinny_swiglu_need.argtypes = [_i, _i, _i, _i, ctypes.POINTER(_sz), ctypes.POINTER(_i)]
        lib.lily_skinny_swiglu_need.restype = _i
        lib.lily_attention_prefill_mma_rows.restype = _i
        lib.lily_attention_prefill_tc_rows.restype = _i
        lib.lily_attention_prefill_tc_takes.argtypes = [_i, _i]
        lib.lily_attention_prefill_tc_takes.restype = _i
        lib.lily_attention_mma_supports.argtypes = [_i]
        lib.lily_attention_mma_supports.restype = _i
        lib.lily_top_logprobs_cap.restype = _i
        lib.lily_attention_decode_scratch_floats.argtypes = [_i, _i, _i, _i]
        lib.lily_attention_decode_scratch_floats.restype = _sz
        lib.lily_normed_mean_max.restype = _i
        lib.lily_wkv_max_head_dim.restype = _i
        lib.lily_latent_attention_mma_takes.argtypes = [_i, _i]
        lib.lily_latent_attention_mma_takes.restype = _i
        lib.lily_latent_attention_mma_tile_tokens.argtypes = [_i]
        lib.lily_latent_attention_mma_tile_tokens.restype = _i
        lib.lily_latent_attention_status.restype = _i
        lib.lily_moe_tile_rows.restype = _i
        lib.lily_delta_rule_max_head_dim.restype = _i
        lib.lily_selective_scan_max_state.restype = _i
        _lib = lib
    return _lib


launches = {"count": 0}          # kernels of this package launched so far (bench.py reports the difference)


def _call(name: str, *args) -> None:
    lib = library()
    launches["count"] += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.lily_last_error().decode(errors='replace')}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _dev(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("lily_b200 kernels run on a CUDA device only; got a tensor on " + str(t.device))
        if not t.is_contiguous():
            raise KernelError(f"kernels take contiguous tensors (shape {tuple(t.shape)}, strides {t.stride()})")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _i32(t: Optional[torch.Tensor], name: str):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    return _p(t)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle.  The step launches a few hundred kernels from Python, so the two
    C calls are used directly where this torch has them (the public route builds a Stream object a call)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------ elementwise

def embed(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
          future: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """Rows of ``table`` [vocab, hidden] at ``ids`` [tokens], times ``scale``, as float32 (the residual
    stream).  With ``future`` (int32, one entry per request slot) an id ``-(slot + 1)`` stands for the
    token that ``scatter_tokens`` stored for that slot."""
    _dev(table, ids, out, future)
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _call("lily_embed", _p(table), _dt(table), _i32(ids, "ids"), _i32(future, "future") if future is not None else None,
          _p(out), n, hidden, vocab, float(scale), _stream())
    return out


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """In place on float32 ``logits``: times ``scale``, then ``softcap * tanh(. / softcap)`` when a cap is given."""
    _dev(logits)
    if logits.dtype != torch.float32:
        raise KernelError("logit_transform takes float32 logits")
    _call("lily_logit_transform", _p(logits), logits.numel(), float(scale), float(softcap or 0.0), _stream())
    return logits


def scatter_tokens(tokens: torch.Tensor, logit_rows: torch.Tensor, token_req: torch.Tensor, slots: torch.Tensor,
                   future: torch.Tensor) -> None:
    """``future[slots[token_req[logit_rows[i]]]] = tokens[i]``: each sampled token goes to the entry
    of its request's slot, where the next step's ``embed`` finds it."""
    _dev(tokens, logit_rows, token_req, slots, future)
    n = tokens.numel()
    if logit_rows.numel() < n:
        raise KernelError(f"scatter_tokens: {n} tokens for {logit_rows.numel()} logit rows")
    _call("lily_scatter_tokens", _i32(tokens, "tokens"), _i32(logit_rows, "logit_rows"), _i32(token_req, "token_req"),
          _i32(slots, "slots"), _i32(future, "future"), n, future.numel(), _stream())


def _summed(t: torch.Tensor, rows: int, cols: int, what: str):
    """(splits, stride) of a kernel input that is either [rows, cols] in the activation dtype or
    float32 partial sums [splits, rows, cols] of a split-k product."""
    if t.dim() == 3:
        if t.dtype != torch.float32 or tuple(t.shape[1:]) != (rows, cols):
            raise KernelError(f"{what}: partial sums must be float32 [splits, {rows}, {cols}], got {t.dtype} {tuple(t.shape)}")
        return t.shape[0], rows * cols
    if tuple(t.shape) != (rows, cols):
        raise KernelError(f"{what}: expected [{rows}, {cols}], got {tuple(t.shape)}")
    return 1, 0


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, write_residual: bool = True,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``resid += delta`` (float32, in place when ``write_residual``), then RMSNorm with ``weight``.
    ``delta`` is [tokens, hidden] in the activation dtype or float32 partial sums [splits, tokens,
    hidden].  With ``rows`` only those rows are normalised (and the residual is left as it is)."""
    _dev(resid, delta, weight, rows, out)
    if resid.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    hidden = resid.shape[-1]
    m = resid.shape[0] if rows is None else rows.numel()
    if rows is not None:
        write_residual = False
    if out is None:
        out = torch.empty((m, hidden), dtype=out_dtype, device=resid.device)
    splits, stride = (1, 0) if delta is None else _summed(delta, resid.shape[0], hidden, "add_rmsnorm delta")
    if delta is not None and delta.dtype not in (out.dtype, torch.float32):
        raise KernelError(f"delta {delta.dtype} does not match out {out.dtype}")
    if weight.numel() != hidden:
        raise KernelError(f"norm gain has {weight.numel()} entries, rows have {hidden}")
    _call("lily_add_rmsnorm", _p(resid), _p(delta), _p(weight), _p(out), _i32(rows, "rows"), m, hidden, float(eps),
          int(write_residual), _dt(out), _dt(weight), _dt(delta) if delta is not None else _dt(out), splits, stride,
          _stream())
    return out


def add_rmsnorm_multi(resid: torch.Tensor, deltas: Sequence[torch.Tensor], gains: Sequence[torch.Tensor], eps: float,
                      out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None,
                      write_residual: bool = True) -> Tuple[torch.Tensor, ...]:
    """``resid += sum(deltas) + bias`` (float32, in place), then one RMSNorm of the new rows per entry of ``gains``
    (float32 vectors; none, one or two), all from the same root mean square.  ``deltas`` holds up to two tensors, each
    [tokens, hidden] in the activation dtype or float32 partial sums; ``bias`` is a float32 vector [hidden] added to
    every row.  Returns the normed activations, one tensor per gain."""
    deltas = [d for d in deltas if d is not None]
    if len(deltas) > 2 or len(gains) > 2:
        raise KernelError("add_rmsnorm_multi takes up to two deltas and up to two gains")
    _dev(resid, bias, *deltas, *gains)
    if resid.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    rows, hidden = resid.shape
    for g in gains:
        if g.dtype != torch.float32 or g.numel() != hidden:
            raise KernelError("add_rmsnorm_multi: gains are float32 vectors of the row's length")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != hidden):
        raise KernelError("add_rmsnorm_multi: the bias is a float32 vector of the row's length")
    outs = [torch.empty((rows, hidden), dtype=out_dtype, device=resid.device) for _ in gains]
    desc = []
    for d in deltas:
        splits, stride = _summed(d, rows, hidden, "add_rmsnorm_multi delta")
        if d.dtype not in (out_dtype, torch.float32):
            raise KernelError(f"delta {d.dtype} does not match out {out_dtype}")
        desc += [_p(d), _dt(d), splits, stride]
    desc += [None, _F32, 1, 0] * (2 - len(deltas))
    act = _BF16 if out_dtype == torch.bfloat16 else _F32
    _call("lily_add_rmsnorm_multi", _p(resid), *desc, _p(bias), _p(gains[0]) if gains else None,
          _p(gains[1]) if len(gains) > 1 else None, _p(outs[0]) if gains else None, _p(outs[1]) if len(gains) > 1 else None,
          rows, hidden, float(eps), int(write_residual), act, _stream())
    return tuple(outs)


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}
# the gate/up forms of the stand-alone kernel: the two above, and "swish_clamped": g' sigmoid(alpha g') (u' + 1) with
# g' = min(g, limit) and u' = clamp(u, -limit, limit)
GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def silu_mul(gate_up: torch.Tensor, out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
             block: Optional[int] = None, activation: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """``act(gate) * up`` of ``gate_up`` [tokens, 2I] = [all gate | all up], or, with ``block``,
    alternating runs of ``block`` gate and ``block`` up columns; ``activation`` is "silu" or "gelu_tanh"
    (0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))).  ``gate_up`` may be float32 partial
    sums [splits, tokens, 2I], in which case ``out_dtype`` says what to write."""
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"no gate activation {activation!r}; have {sorted(GATE_ACTIVATIONS)}")
    _dev(gate_up, out)
    n, two_i = gate_up.shape[-2:]
    splits, stride = _summed(gate_up, n, two_i, "silu_mul")
    if out is None:
        out = torch.empty((n, two_i // 2), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    _call("lily_silu_mul", _p(gate_up), _p(out), n, two_i // 2, int(block or two_i // 2), _dt(out), _dt(gate_up), splits,
          stride, GATE_ACTIVATIONS[activation], float(limit), float(alpha), _stream())
    return out


def qk_norm_rope_write(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
                       eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                       positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                       kv_layer: torch.Tensor, nq: int, nkv: int, d: int, rotary_dim: int, page_size: int,
                       write_kv: bool = True, q_out: Optional[torch.Tensor] = None, dv: Optional[int] = None,
                       v_norm: bool = False, v_keep: Optional[torch.Tensor] = None, v_blend: Optional[float] = None) -> torch.Tensor:
    """Per-head RMSNorm of q and k (when gains are given), rotation by the tables, q to ``q_out``
    [tokens, nq * d], k and v into the token's place in its page of ``kv_layer``.  ``qkv`` is
    [tokens, (nq + nkv) d + nkv dv] in the cache's dtype or float32 partial sums [splits, tokens, ...]; value
    heads have ``dv`` features (default d; see ``cache_layer_fits`` for the page layout).
    ``v_norm``: each value head is divided by its root mean square (``eps``, no gain) before it is cached.
    ``v_keep`` float32 [tokens, nkv * dv]: without ``v_blend`` the (normed) values are also left there; with it they
    are read from there and the cached value is ``(1 - v_blend) v + v_blend v_keep``."""
    _dev(qkv, q_gain, k_gain, cos, sin, positions, token_req, block_table, kv_layer, q_out)
    n = qkv.shape[-2]
    dv = int(dv or d)
    splits, stride = _summed(qkv, n, (nq + nkv) * d + nkv * dv, "qk_norm_rope_write qkv")
    if qkv.dtype not in (kv_layer.dtype, torch.float32):
        raise KernelError(f"cache dtype {kv_layer.dtype} differs from activations {qkv.dtype}")
    cache_layer_fits(kv_layer, nkv, page_size, d, dv)
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[-1] != rotary_dim // 2):
        raise KernelError("rotation tables must be float32 [positions, rotary_dim / 2]")
    if q_gain is not None and q_gain.dtype != k_gain.dtype:
        raise KernelError("q and k gains must share a dtype")
    if v_keep is not None and (v_keep.dtype != torch.float32 or tuple(v_keep.shape) != (n, nkv * dv) or not v_keep.is_cuda
                               or not v_keep.is_contiguous() or not write_kv):
        raise KernelError("qk_norm_rope_write: kept values are float32 [tokens, nkv * dv] of a layer that writes its cache")
    if v_blend is not None and v_keep is None:
        raise KernelError("qk_norm_rope_write: a blend needs the kept values")
    if q_out is None:
        q_out = torch.empty((n, nq * d), dtype=kv_layer.dtype, device=qkv.device)
    _call("lily_qk_norm_rope_write", _p(qkv), _p(q_gain), _p(k_gain), float(eps), _p(cos), _p(sin),
          _i32(positions, "positions"), _i32(token_req, "token_req"), _i32(block_table, "block_table"),
          block_table.shape[-1], _p(kv_layer), _p(q_out), n, nq, nkv, d, rotary_dim, page_size, int(write_kv),
          _dt(kv_layer), _dt(q_gain) if q_gain is not None else _F32, _dt(qkv), splits, stride, dv,
          int(bool(v_norm)), float(v_blend or 0.0), _p(v_keep), 0 if v_keep is None else (1 if v_blend is None else 2), _stream())
    return q_out


def cache_layer_fits(kv_layer: torch.Tensor, nkv: int, page_size: int, d: int, dv: int) -> None:
    """A cache layer is [pages, 2, kv_heads, page_size, d] when keys and values have one head size, else
    [pages, kv_heads * page_size * (d + dv)]: a page's keys [kv_heads, page_size, d], then its values
    [kv_heads, page_size, dv] (the first form is the second with dv == d)."""
    want = (2, nkv, page_size, d) if dv == d else (nkv * page_size * (d + dv),)
    if tuple(kv_layer.shape[1:]) != want:
        raise KernelError(f"cache layer shape {tuple(kv_layer.shape)} does not fit kv_heads={nkv} page={page_size} "
                          f"d={d} dv={dv}")


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _dev(x)
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _call("lily_cast", _p(x), _dt(x), _p(out), _dt(out), x.numel(), _stream())
    return out


# ------------------------------------------------------------------------------ matrix products

def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] . weight [N, K]^T (+ bias)``.  float32: this package's FFMA kernel.
    bfloat16: cuBLAS with float32 accumulation; ``out_dtype=float32`` keeps the accumulator's
    precision (used for the logits)."""
    _dev(x, weight, bias)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or weight.dtype != x.dtype:
        raise KernelError(f"linear: x {tuple(x.shape)} {x.dtype} against weight {tuple(weight.shape)} {weight.dtype}")
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        if bias is not None and bias.dtype != torch.float32:
            raise KernelError("float32 linear takes a float32 bias")
        _call("lily_gemm_fp32", _p(x), _p(weight), _p(bias), _p(out), m, n, k, k, n, _stream())
        return out
    if _OWN_PLAIN_GEMM and out_dtype is None and m >= TC_MIN_ROWS and gemm_tc_takes(x, weight):
        return gemm_tc(x, weight, bias.to(x.dtype) if bias is not None else None)
    if out_dtype == torch.float32:
        out = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            out += bias.float()
        return out
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, weight.t())
    return torch.mm(x, weight.t())


TC_MIN_ROWS = 65          # products of more rows than this go to the tcgen05 kernel when it takes the shape


def gate_up_fused_pays(rows: int, fused_rows: int) -> bool:
    """Whether the tcgen05 gate/up product with the SiLU*mul epilogue is the faster way for ``rows`` tokens and a
    fused matrix of ``fused_rows`` rows (gate and up together), against the library product followed by the SiLU*mul
    kernel.  It is, except for 129 to 256 tokens where its 256-wide tiles fill the last round of block pairs badly
    (Qwen3-8B, 96 tiles on 74 pairs: 56 against 47 us at 192 tokens, 57 against 54 at 256; equal from 65 to 128 and
    from 384 on, where the epilogue saves the [tokens, 2 I] intermediate)."""
    if rows < TC_MIN_ROWS:
        return False
    if 128 < rows <= 256:
        tiles, pairs = -(-fused_rows // 256), max(1, sm_count() // 2)
        return -(-tiles // pairs) * pairs < 1.3 * tiles
    return True
# LILY_B200_PLAIN_GEMM=tcgen05 sends the plain bfloat16 products of 65 rows and more (QKV, output, down in prefill) to
# this package's tcgen05 kernel too instead of the library, which is 8 to 10 % faster on them and therefore the default.
_OWN_PLAIN_GEMM = os.environ.get("LILY_B200_PLAIN_GEMM", "") == "tcgen05"


def gemm_tc_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
            silu_mul_block: bool = False, activation: str = "silu", plain_activation: Optional[str] = None,
            limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """``x [M, K] . weight [N, K]^T`` in bfloat16 on the tcgen05 tensor cores (TMA-fed, accumulator
    in tensor memory).  With ``silu_mul_block`` the rows of ``weight`` alternate between 128 gate
    rows and the 128 up rows of the same outputs and the result is ``act(gate) * up`` [M, N / 2]
    (``activation``: "silu", "gelu_tanh", or "swish_clamped" with its ``limit`` and ``alpha``).  ``plain_activation`` ("silu", "gelu_tanh", "relu2"): the plain product
    with that activation on every output, applied to the float32 sums in the epilogue."""
    _dev(x, weight, bias)
    m, k = x.shape
    n = weight.shape[0]
    if not gemm_tc_takes(x, weight) or weight.shape[1] != k:
        raise KernelError(f"gemm_tc: x {tuple(x.shape)} {x.dtype} against weight {tuple(weight.shape)} {weight.dtype}")
    out = torch.empty((m, n // 2 if silu_mul_block else n), dtype=torch.bfloat16, device=x.device)
    _call("lily_gemm_tc", _p(x), _p(weight), _p(out), _p(bias), m, n, k, k, out.shape[1],
          (6 if activation == "swish_clamped" else 1 + ACTIVATIONS[activation]) if silu_mul_block
          else (3 + PLAIN_ACTIVATIONS[plain_activation] if plain_activation else 0), float(limit), float(alpha), _stream())
    return out


def gemm_tc_status() -> int:
    """0, or a code from the first bounded wait that gave up in a tcgen05 kernel (synchronises)."""
    return int(library().lily_gemm_tc_status())


def linear_split(x: torch.Tensor, weight: torch.Tensor, splits: Optional[int] = None) -> Optional[torch.Tensor]:
    """``x [M, K] . weight [N, K]^T`` for a few tokens (decode) by this package's weight-streaming
    kernel, as float32 partial sums ``[splits, M, N]`` over slices of K that the consuming kernel
    (``add_rmsnorm``, ``silu_mul``, ``qk_norm_rope_write``) adds up.  Without ``splits`` the kernel's
    own rule decides, and None comes back for shapes it leaves to the library product (wide
    outputs, more than 16 tokens) or cannot take (K not a multiple of 64, not bfloat16); the caller
    then uses ``linear``.  With ``splits`` given the kernel runs whenever it can (up to 64 tokens)."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return None
    m, k = x.shape
    n = weight.shape[0]
    lib = library()
    if m > lib.lily_skinny_gemm_max_rows() or m < 1 or weight.shape[1] != k or k % 64:
        return None
    if splits is None:
        splits = int(lib.lily_skinny_gemm_splits(m, n, k))
    if splits < 1:
        return None
    _dev(x, weight)
    parts = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
    _call("lily_skinny_gemm", _p(x), _p(weight), _p(parts), m, n, k, splits, _stream())
    return parts


def linear_auto(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The product in whichever form is fastest for the shape: float32 partial sums from
    ``linear_split`` for a few tokens, else ``linear``'s [M, N].  For producers whose consumer is
    one of the kernels that take either form."""
    if bias is None:
        parts = linear_split(x, weight)
        if parts is not None:
            return parts
    return linear(x, weight, bias)


def swiglu_skinny_need(tokens: int, intermediate: int, hidden: int, dtype: torch.dtype,
                       block: Optional[int] = None, whenever_possible: bool = False) -> Optional[Tuple[int, int]]:
    """(float32 of scratch, int32 counters) that ``swiglu_skinny`` wants for this shape, or None when it does not
    take it (more than 8 tokens, not bfloat16, K not a multiple of 64) or, unless ``whenever_possible``, when the
    library product followed by SiLU*mul is the faster pair for it (several tokens of a very wide input): the caller
    then forms the product and SiLU*mul separately.  ``LILY_B200_SWIGLU=library`` always answers None."""
    if dtype != torch.bfloat16 or _LIBRARY_SWIGLU:
        return None
    floats, counters = _sz(0), _i(0)
    verdict = library().lily_skinny_swiglu_need(int(tokens), int(intermediate), int(hidden), int(block or intermediate),
                                                ctypes.byref(floats), ctypes.byref(counters))
    if verdict == 0 or (verdict == 2 and not whenever_possible):
        return None
    return int(floats.value), int(counters.value)


_LIBRARY_SWIGLU = os.environ.get("LILY_B200_SWIGLU", "") == "library"


def swiglu_skinny(x: torch.Tensor, gate_up: torch.Tensor, block: Optional[int], scratch: torch.Tensor,
                  counters: torch.Tensor, out: Optional[torch.Tensor] = None, activation: str = "silu",
                  limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """``act(x . gate^T) * (x . up^T)`` [tokens, I] for up to 8 tokens in one kernel that streams the fused
    gate/up matrix [2 I, K] once (rows in alternating runs of ``block`` gate and up rows; None: all gate, then all
    up).  ``scratch`` (float32) and ``counters`` (int32, zero before the first call; the kernel leaves them zero)
    are sized by ``swiglu_skinny_need``."""
    _dev(x, gate_up, scratch, counters, out)
    m, k = x.shape
    inter = gate_up.shape[0] // 2
    need = swiglu_skinny_need(m, inter, k, x.dtype, block, whenever_possible=True)
    if need is None or gate_up.dtype != torch.bfloat16 or gate_up.shape[1] != k:
        raise KernelError(f"swiglu_skinny: x {tuple(x.shape)} {x.dtype} against {tuple(gate_up.shape)} {gate_up.dtype}")
    if scratch.dtype != torch.float32 or scratch.numel() < need[0] or counters.dtype != torch.int32 or counters.numel() < need[1]:
        raise KernelError(f"swiglu_skinny: {need[0]} float32 of scratch and {need[1]} int32 counters needed")
    if out is None:
        out = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    _call("lily_skinny_swiglu", _p(x), _p(gate_up), _p(out), _p(scratch), _p(counters), m, inter, k, int(block or inter),
          GATE_ACTIVATIONS[activation], float(limit), float(alpha), _stream())
    return out


def logits(x: torch.Tensor, head: torch.Tensor) -> torch.Tensor:
    """``x [rows, hidden] . head [vocab, hidden]^T`` as float32 [rows, vocab]: for a few rows the head is
    streamed once by this package's kernel when one slice of K serves, else a product that keeps the
    accumulator's precision (lily/layers/vocab_embedding.py:89-96 casts a model-dtype product)."""
    parts = linear_split(x, head)
    if parts is not None and parts.shape[0] == 1:
        return parts[0]
    return linear(x, head, out_dtype=torch.float32)


def gate_up_interleave(dtype: torch.dtype, intermediate: int) -> Optional[int]:
    """How a fused gate/up matrix should be laid out for these kernels: None for all gate rows, then all up
    rows; a number for alternating runs of that many gate rows and the up rows of the same outputs (what the
    tcgen05 product's SiLU*mul epilogue wants: both halves of 128 outputs inside one 256-row tile)."""
    return 128 if dtype == torch.bfloat16 and intermediate % 128 == 0 else None


# ------------------------------------------------------------------------------ attention

def uses_tensor_cores(dtype: torch.dtype, d: int) -> bool:
    """Whether attention of this precision and head size runs on the mma.sync kernels
    (bfloat16, head sizes 64, 128, 192, 256); everything else runs on the CUDA-core kernels."""
    return dtype == torch.bfloat16 and bool(library().lily_attention_mma_supports(int(d)))


# A step with fewer new tokens than this in its prompt portions runs them through the mma.sync kernel
# (tiles of 64 rows); from here on the tcgen05 kernel's tiles of 128 rows are worth filling.
TC_ATTENTION_MIN_TOKENS = 128


def uses_tcgen05_attention(dtype: torch.dtype, d: int, page_size: int, new_tokens: int) -> bool:
    """Whether prefill attention of this precision, head size, page size and number of new tokens
    runs on the tcgen05 kernel (bfloat16, head size 128 or 64, pages of a multiple of 64 positions; scores scaled
    or soft-capped)."""
    return (dtype == torch.bfloat16 and new_tokens >= TC_ATTENTION_MIN_TOKENS
            and bool(library().lily_attention_prefill_tc_takes(int(d), int(page_size))))


_SIMT_LATENT = os.environ.get("LILY_B200_LATENT_ATTENTION", "") == "simt"


def latent_tensor_cores(dtype: torch.dtype, d: int, dv: Optional[int], nkv: int = 1, softcap: Optional[float] = None) -> bool:
    """Whether attention whose values are columns of the key rows runs on the tensor-core kernel for cached latents
    (bfloat16, one shared row a position, rows of whole 16-byte pieces, an even value width of up to 512, plain scores)."""
    return (dtype == torch.bfloat16 and nkv == 1 and not softcap and dv is not None and not _SIMT_LATENT
            and bool(library().lily_latent_attention_mma_takes(int(d), int(dv))))


def latent_attention_status() -> int:
    """0, or 1 + the block of the first bounded wait for a key tile that gave up in the tensor-core kernel for cached
    latents (synchronises; the word is cleared when read)."""
    return int(library().lily_latent_attention_status())


def prefill_tile_rows(dtype: torch.dtype = torch.float32, d: int = 0, page_size: int = 0, new_tokens: int = 0,
                      softcap: Optional[float] = None, dv: Optional[int] = None, values_in_keys: bool = False,
                      heads: int = 0, keep_first: int = 0, sink: bool = False, all_values: bool = False) -> int:
    """New tokens per tile of the prefill kernel that will take this precision, head size (``dv`` for the values
    where it differs), page size, number of new tokens and kind of scores and mask."""
    lib = library()
    if values_in_keys and heads and latent_tensor_cores(dtype, d, dv, softcap=softcap):
        return int(lib.lily_latent_attention_mma_tile_tokens(int(heads)))
    if (sink or all_values) and sink_on_tensor_cores(dtype, d, dv, values_in_keys, softcap):
        return int(lib.lily_attention_prefill_mma_rows())
    if sink or all_values:
        return int(lib.lily_attention_prefill_simt_rows())
    same = (dv is None or dv == d) and not values_in_keys and not sink and not all_values      # those run on CUDA cores
    if same and uses_tcgen05_attention(dtype, d, page_size, new_tokens):
        return int(lib.lily_attention_prefill_tc_rows())
    return int(lib.lily_attention_prefill_mma_rows() if same and uses_tensor_cores(dtype, d) else lib.lily_attention_prefill_simt_rows())


def attention_tc_status() -> int:
    """0, or a code from the first bounded wait that gave up in the tcgen05 attention kernel (synchronises)."""
    return int(library().lily_attention_tc_status())


def attention_prefill(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                      prefix_lens: torch.Tensor, tile_req: torch.Tensor, tile_start: torch.Tensor, out: torch.Tensor,
                      nq: int, nkv: int, d: int, page_size: int, scale: float, window: Optional[int] = None,
                      tile_rows: Optional[int] = None, heads_per_block: int = 0, softcap: Optional[float] = None,
                      dv: Optional[int] = None, values_in_keys: bool = False, keep_first: int = 0,
                      sink: bool = False, all_values: bool = False) -> None:
    """Causal attention of each request's new tokens over its cached prefix and themselves.
    ``sink``: the softmax's denominator holds one more unit (a key of score 0 that has no value).  ``all_values``: every
    query head's weights meet the values of all kv heads, ``out`` is float32 [tokens, nq * nkv * dv] (``head_mix``
    follows).  Both run on the CUDA-core kernel.  ``softcap``: scores
    become softcap * tanh(score * scale / softcap) before the softmax; ``keep_first``: beside a window, keys at
    positions below this stay visible; ``dv``: the
    value head size where it differs from d (CUDA-core kernels; ``out`` is then [tokens, nq * dv]).
    ``values_in_keys``: the values are the first ``dv`` columns of the key rows and a page holds keys only (CUDA-core kernels).
    ``q`` and ``out`` are [tokens, nq * d] indexed by ``cu_seqlens``; tiles list (request, offset)
    in steps of ``tile_rows`` (default: ``prefill_tile_rows(q.dtype, d)``), which also names the
    kernel: the tcgen05 kernel takes tiles of its own size, the others theirs.  ``heads_per_block``
    (tcgen05 only) 1 or 2 picks between its one-head and its two-head form; 0 lets the launcher choose."""
    _dev(q, kv_layer, block_table, cu_seqlens, prefix_lens, tile_req, tile_start, out)
    planes = all_values and out.dim() == 3            # one launch of the mma.sync kernel a kv head (``all_values_sums``)
    if q.dtype != kv_layer.dtype or out.dtype != (torch.float32 if all_values and not planes else q.dtype):
        raise KernelError("attention: q, cache and out must share a dtype (sums over all kv heads' values on CUDA cores are float32)")
    if (sink or all_values) and sink_on_tensor_cores(q.dtype, d, dv, values_in_keys, softcap) and (planes or not all_values):
        if (tile_rows or 0) not in (0, int(library().lily_attention_prefill_mma_rows())):
            raise KernelError(f"attention_prefill: the sink runs in tiles of {library().lily_attention_prefill_mma_rows()} rows")
        if planes and tuple(out.shape) != (nkv, q.shape[0], nq * d):
            raise KernelError(f"attention_prefill: planes of sums are [{nkv}, tokens, nq * d]")
        for shift in range(nkv if planes else 1):
            _call("lily_attention_prefill_mma", _p(q), _p(kv_layer), out[shift].data_ptr() if planes else _p(out),
                  _i32(block_table, "block_table"), block_table.shape[-1], _i32(cu_seqlens, "cu_seqlens"),
                  _i32(prefix_lens, "prefix_lens"), _i32(tile_req, "tile_req"), _i32(tile_start, "tile_start"), tile_req.numel(),
                  nq, nkv, d, page_size, int(window or 0), float(scale), float(softcap or 0.0),
                  int(keep_first or 0) if window else 0, int(bool(sink)), shift, _stream())
        return
    if planes:
        # the CUDA-core kernel, one launch a kv head with the value heads shifted
        if tuple(out.shape) != (nkv, q.shape[0], nq * int(dv or d)) or values_in_keys:
            raise KernelError(f"attention_prefill: planes of sums are [{nkv}, tokens, nq * dv]")
        if (tile_rows or 0) not in (0, int(library().lily_attention_prefill_simt_rows())):
            raise KernelError("attention_prefill: planes on the CUDA-core kernel come in its own tiles")
        for shift in range(nkv):
            _call("lily_attention_prefill_simt", _p(q), _p(kv_layer), out[shift].data_ptr(), _i32(block_table, "block_table"),
                  block_table.shape[-1], _i32(cu_seqlens, "cu_seqlens"), _i32(prefix_lens, "prefix_lens"), _i32(tile_req, "tile_req"),
                  _i32(tile_start, "tile_start"), tile_req.numel(), nq, nkv, d, page_size, int(window or 0), float(scale), _dt(q),
                  float(softcap or 0.0), int(dv or d), int(keep_first or 0) if window else 0, 1 if sink else 0, shift, _stream())
        return
    common = (_p(q), _p(kv_layer), _p(out), _i32(block_table, "block_table"), block_table.shape[-1],
              _i32(cu_seqlens, "cu_seqlens"), _i32(prefix_lens, "prefix_lens"), _i32(tile_req, "tile_req"),
              _i32(tile_start, "tile_start"), tile_req.numel(), nq, nkv, d, page_size, int(window or 0), float(scale))
    lib = library()
    dv = int(dv or d)
    cap = float(softcap or 0.0)
    if (values_in_keys and latent_tensor_cores(q.dtype, d, dv, nkv, softcap)
            and tile_rows == int(lib.lily_latent_attention_mma_tile_tokens(int(nq)))):
        _call("lily_latent_attention_prefill_mma", _p(q), _p(kv_layer), _p(out), _i32(block_table, "block_table"),
              block_table.shape[-1], _i32(cu_seqlens, "cu_seqlens"), _i32(prefix_lens, "prefix_lens"),
              _i32(tile_req, "tile_req"), _i32(tile_start, "tile_start"), tile_req.numel(), int(tile_rows), nq, d, dv,
              page_size, int(window or 0), float(scale), _stream())
        return
    keep_first = int(keep_first or 0) if window else 0
    flags = _attention_flags(sink, all_values, values_in_keys, nkv, dv, out, q.shape[0] * nq)
    tensor_cores = dv == d and not values_in_keys and not flags and uses_tensor_cores(q.dtype, d)
    base_rows = int(lib.lily_attention_prefill_mma_rows() if tensor_cores else lib.lily_attention_prefill_simt_rows())
    if tile_rows is not None and tile_rows != base_rows:
        if not (tile_rows == int(lib.lily_attention_prefill_tc_rows()) and q.dtype == torch.bfloat16 and dv == d and not flags
                and lib.lily_attention_prefill_tc_takes(int(d), int(page_size))):
            raise KernelError(f"attention_prefill: no kernel with tiles of {tile_rows} rows for {q.dtype}, head size {d}, "
                              f"page size {page_size}")
        if not (q.is_contiguous() and out.is_contiguous() and kv_layer.is_contiguous()):
            raise KernelError("attention_prefill: the tcgen05 kernel takes contiguous q, out and cache")
        _call("lily_attention_prefill_tc", *common, q.shape[0], kv_layer.shape[0], int(heads_per_block), cap, keep_first, _stream())
    elif tensor_cores:
        _call("lily_attention_prefill_mma", *common, cap, keep_first, 0, 0, _stream())
    else:
        _call("lily_attention_prefill_simt", *common, _dt(q), cap, -dv if values_in_keys else dv, keep_first, flags, 0, _stream())


_MERGED_SHIFTS = os.environ.get("LILY_B200_MERGED_SHIFTS", "1") != "0"
ALL_VALUES_COLUMNS = 512       # value columns a query row of the CUDA-core kernels gathers in one launch
_SIMT_SINK = os.environ.get("LILY_B200_SINK_ATTENTION", "") == "simt"


def sink_on_tensor_cores(dtype: torch.dtype, d: int, dv: Optional[int] = None, values_in_keys: bool = False,
                         softcap: Optional[float] = None) -> bool:
    """Whether attention with a sink (and, in one launch a kv head, with the values of all kv heads) runs on the mma.sync
    kernels: bfloat16, keys and values of one head size that those kernels take; else the CUDA-core kernels."""
    return (not _SIMT_SINK and not values_in_keys and int(dv or d) == d and uses_tensor_cores(dtype, d))


def all_values_decode_rows(dtype: torch.dtype, requests: int, nkv: int, d: int, dv: Optional[int] = None) -> int:
    """The rows to plan the decode attention over the values of all kv heads for (``plan_decode_attention``): on the
    mma.sync kernels a step of single tokens runs every shift of the value heads in one launch, ``nkv`` rows a request."""
    return requests * nkv if sink_on_tensor_cores(dtype, d, dv) and _MERGED_SHIFTS else requests


def all_values_in_planes(dtype: torch.dtype, nkv: int, d: int, dv: Optional[int] = None) -> bool:
    """Whether attention over the values of all kv heads runs as one launch a kv head (``all_values_sums`` then gives
    planes): on the mma.sync kernels, and on the CUDA-core kernels when a row of ``nkv * dv`` columns would pass 512."""
    return sink_on_tensor_cores(dtype, d, dv) or nkv * int(dv or d) > ALL_VALUES_COLUMNS


def all_values_sums(dtype: torch.dtype, tokens: int, nq: int, nkv: int, d: int, dv: Optional[int], device) -> torch.Tensor:
    """The tensor that ``attention_prefill`` / ``attention_decode`` with ``all_values`` fill and ``head_mix`` reads.  On
    the CUDA-core kernels float32 [tokens, nq * nkv * dv]: a query head's row holds its weights' sums over every kv
    head's values.  On the mma.sync kernels, and on the CUDA-core kernels when such a row would pass their 512 columns,
    ``nkv`` planes [nkv, tokens, nq * dv] in ``dtype``: plane s holds, for a query head of kv head g, the sums over the
    values of kv head (g + s) % nkv (one launch a plane)."""
    dv = int(dv or d)
    if all_values_in_planes(dtype, nkv, d, dv):
        return torch.empty((nkv, tokens, nq * dv), dtype=dtype, device=device)
    return torch.empty((tokens, nq * nkv * dv), dtype=torch.float32, device=device)


def _attention_flags(sink: bool, all_values: bool, values_in_keys: bool, nkv: int, dv: int, out: torch.Tensor, rows: int) -> int:
    """The CUDA-core attention kernels' option bits: 1 the sink, 2 values of all kv heads, 4 float32 outputs."""
    if all_values:
        if values_in_keys:
            raise KernelError("attention: values that are columns of the key rows belong to one shared head")
        if out.dim() == 2 and (out.dtype != torch.float32 or out.numel() != rows * nkv * dv):
            raise KernelError(f"attention: sums over all kv heads' values are float32 [rows, nq * {nkv} * {dv}]")
    return (1 if sink else 0) | (6 if all_values else 0)


def decode_clusters(d: int, splits: int, group: int) -> int:
    """How many (request, kv head) pairs the tensor-core decode attention can merge inside clusters of
    ``splits`` blocks at once (0: it would use scratch and the combine kernel)."""
    return int(library().lily_attention_decode_mma_clusters(int(d), int(splits), int(group)))


def decode_scratch_floats(requests: int, nq: int, d: int, splits: int) -> int:
    return int(library().lily_attention_decode_scratch_floats(requests, nq, d, splits))


def attention_decode(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                     out: torch.Tensor, scratch: Optional[torch.Tensor], splits: int, nq: int, nkv: int, d: int,
                     page_size: int, scale: float, window: Optional[int] = None, stages: int = 0,
                     softcap: Optional[float] = None, dv: Optional[int] = None, values_in_keys: bool = False,
                     keep_first: int = 0, sink: bool = False, all_values: bool = False) -> None:
    """``sink`` and ``all_values`` as in ``attention_prefill`` (CUDA-core kernel; the scratch then holds nkv * dv columns a head).
    One query token per request (rows of ``q`` [requests, nq * d]) over ``seq_lens`` cached
    positions (the last ``window`` of them and the first ``keep_first``, where given), keys cut into ``splits`` ranges merged through ``scratch`` (float32).  ``stages`` (tensor-core
    kernel only): the key/value tiles a block holds, 0 for the default (``DecodePlan.stages``)."""
    _dev(q, kv_layer, block_table, seq_lens, out, scratch)
    requests = q.shape[0]
    planes = all_values and out.dim() == 3
    if q.dtype != kv_layer.dtype or out.dtype != (torch.float32 if all_values and not planes else q.dtype):
        raise KernelError("attention: q, cache and out must share a dtype (sums over all kv heads' values on CUDA cores are float32)")
    dv = int(dv or d)
    cap = float(softcap or 0.0)
    flags = _attention_flags(sink, all_values, values_in_keys, nkv, dv, out, requests * nq)
    on_tc = bool(flags) and sink_on_tensor_cores(q.dtype, d, dv, values_in_keys, softcap) and (planes or not all_values)
    if planes and values_in_keys:
        raise KernelError("attention_decode: values that are columns of the key rows belong to one shared head")
    # a step in which every request brings one token: all planes in one launch of the mma.sync kernel (block x works for
    # request x % requests with the value heads shifted by x // requests), so a kv head's keys are fetched while they are in L2
    merged = planes and on_tc and out.shape[1] == requests and nkv > 1 and _MERGED_SHIFTS
    need = decode_scratch_floats(requests * nkv if merged else requests, nq, dv if planes else (nkv * dv if all_values else dv), splits)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: scratch of {need} float32 needed")
    common = (_p(q), _p(kv_layer), _p(out), _i32(block_table, "block_table"), block_table.shape[-1],
              _i32(seq_lens, "seq_lens"), _p(scratch), requests, splits, nq, nkv, d, page_size, int(window or 0),
              float(scale))
    if values_in_keys and latent_tensor_cores(q.dtype, d, dv, nkv, softcap) and not stages:
        _call("lily_latent_attention_decode_mma", _p(q), _p(kv_layer), _p(out), _i32(block_table, "block_table"),
              block_table.shape[-1], _i32(seq_lens, "seq_lens"), _p(scratch), requests, splits, nq, d, dv, page_size,
              int(window or 0), float(scale), _stream())
        if splits > 1:
            _call("lily_attention_combine", _p(scratch), _p(out), requests, nq, dv, splits, _dt(q), _stream())
    elif on_tc:
        for shift in ([-1] if merged else range(nkv if planes else 1)):
            _call("lily_attention_decode_mma", _p(q), _p(kv_layer), out[shift].data_ptr() if planes and not merged else _p(out),
                  _i32(block_table, "block_table"), block_table.shape[-1], _i32(seq_lens, "seq_lens"), _p(scratch), requests, splits,
                  nq, nkv, d, page_size, int(window or 0), float(scale), int(stages), cap, int(keep_first or 0) if window else 0,
                  int(bool(sink)), shift, _stream())
            rows = requests * nkv if merged else requests
            if splits > 1 and (stages or rows * nkv * -(-(nq // nkv) // 16) > decode_clusters(d, splits, nq // nkv)):
                launches["count"] += 1
    elif dv == d and not values_in_keys and not flags and uses_tensor_cores(q.dtype, d):
        _call("lily_attention_decode_mma", *common, int(stages), cap, int(keep_first or 0) if window else 0, 0, 0, _stream())   # merges the splits itself (cluster, or combine behind)
        if splits > 1 and (stages or requests * nkv * -(-(nq // nkv) // 16) > decode_clusters(d, splits, nq // nkv)):
            launches["count"] += 1                                   # the combine kernel, launched inside
    else:
        if stages:
            raise KernelError(f"attention_decode: {stages} stages are the tensor-core kernel's; {q.dtype}, head size {d} runs on CUDA cores")
        for shift in range(nkv if planes else 1):
            _call("lily_attention_decode_simt", _p(q), _p(kv_layer), out[shift].data_ptr() if planes else _p(out),
                  _i32(block_table, "block_table"), block_table.shape[-1], _i32(seq_lens, "seq_lens"), _p(scratch), requests, splits,
                  nq, nkv, d, page_size, int(window or 0), float(scale), _dt(q), cap, -dv if values_in_keys else dv,
                  int(keep_first or 0) if window else 0, (1 if sink else 0) if planes else flags, shift, _stream())
            if splits > 1:
                launches["count"] += 1          # the combine kernel, launched inside


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200)."""
    return int(library().lily_sm_count())


def choose_decode_splits(num_decode: int, kv_heads: int, max_seq_len: int, sm_count: int = 148,
                         blocks_per_sm: int = 3, min_keys: int = 256, max_splits: int = 32,
                         clusters: Optional[Callable[[int], int]] = None) -> int:
    """How many ranges the keys of a decode row are cut into.  One block works on one (request, kv
    head, range); the device holds ``sm_count * blocks_per_sm`` blocks at a time.

    ``clusters(s)`` says how many clusters of ``s`` blocks the attention kernel can have resident at
    once (``decode_clusters``): while every (request, kv head) pair gets one, the blocks of a pair
    merge their ranges through distributed shared memory and no combine kernel follows, and the
    most ranges that allow this are the fastest (measured on a B200, head size 128, 8 kv heads:
    batch 1 and 2: 16 ranges; 4: 10; 8: 6; 16: 3; 24: 2; sizes past 8 want a tenth of room to spare:
    24 pairs in clusters of 15, of which exactly 24 fit, took 21 us against 16 us in clusters of 13).
    A cluster has at most 16 blocks, so a few long rows leave most of the device idle (one row of 131,072 keys:
    128 blocks, 168 us, half of the memory's speed); from 16 k keys on, where one wave of ranges of at least 512
    keys through scratch and the combine kernel has a quarter more blocks than the clusters, the wave is taken
    (measured, 8 kv heads, clusters against the wave: one row of 16 k keys 28 / 23 us, of 24 k 38 / 27, of 131 k
    168 / 88; two rows of 16 k 36 / 32; four rows of 16 k 53 / 51, of 8 k 31 / 32; five rows and more fill the
    device with clusters).
    Without clusters (float32, other head sizes, more pairs than clusters of two): the single wave that
    comes closest to filling the device, and when the rows alone overfill it, about four waves
    (batch 64: 4 ranges).  The reference fixes 32 splits with a floor of 64 keys
    (lily/layers/attention/triton_backend.py:21, decode_attention.py:68,172)."""
    if num_decode == 0:
        return 1
    limit = max(1, min(max_splits, max_seq_len // min_keys))
    pairs, held = num_decode * kv_heads, sm_count * blocks_per_sm
    if clusters is not None:
        full = max(1, min(64, max_seq_len // 512, held // pairs))           # ranges that fill the device once
        for s in range(min(limit, 16), 1, -1):
            room = clusters(s)
            if pairs <= (room if s <= 8 else 0.9 * room):
                if full * 4 >= s * 5 and max_seq_len >= 16384:
                    return full
                return s
    one_wave = min(limit, held // pairs)
    if one_wave >= 1 and (pairs * one_wave >= 0.7 * held or one_wave == limit):
        return one_wave
    return max(1, min(limit, -(-4 * held // pairs)))


@dataclass(frozen=True)
class DecodePlan:
    """How the decode attention of a step runs (the same for every layer of a cache group)."""

    splits: int                 # key ranges per (request, kv head)
    fused: bool                 # the attention kernel starts from the qkv product (norm, rotation, cache write inside)
    scratch_floats: int         # float32 scratch the split ranges are merged through (0: merged inside clusters)
    arm: str                    # which rule chose the splits: "cluster", "wave", "single" or "whole rows"
    stages: int = 0             # key/value tiles a block of the tensor-core kernel holds (0: its default)


def whole_rows_pay(pairs: int, sm_count: int = 148) -> bool:
    """Whether ``pairs`` blocks of the tensor-core kernel with three key/value stages, one block for all keys of a
    (request, kv head), beat ranges of two stages: two such blocks fit a SM, and they keep the memory busy once three
    quarters of those places are taken.  A last round that is less than 45 % full costs more than it saves (a block
    alone on its SM takes about 1.2 us a tile of 64 keys whatever the others do), and past three and a half rounds
    the ranges of two stages are as good or better.
    Measured on a B200, head size 128, 8 kv heads of 4 query heads, decode steps of Qwen3-8B sizes with and without
    (same run, ms): context 4,096: 28 rows 6.66 / 6.45, 32 rows 7.02 / 6.72, 64 rows 10.51 / 10.37, 96 rows 14.36 / 14.13,
    128 rows 17.33 / 17.60; context 1,024: 32 rows 4.67 / 4.44, 64 rows 5.85 / 5.58, 128 rows 7.93 / 7.77, 256 rows 11.94 /
    12.22.  The kernel alone, us, against the best plan of two stages: 32 rows of 4,096 keys 82 against 96, of 1,024 keys
    24 against 32, 64 rows of 1,024 keys 48 against 58; 20 rows of 4,096 keys 79 against 61 (too few blocks)."""
    places = 2 * sm_count
    if pairs < 0.75 * places or pairs > 3.5 * places:
        return False
    last = pairs % places
    return last == 0 or last >= 0.45 * places


def plan_decode_attention(dtype: torch.dtype, requests: int, nq: int, nkv: int, d: int, max_seq_len: int,
                          even: bool = False, dv: Optional[int] = None, values_in_keys: bool = False,
                          keep_first: int = 0, fusable: bool = True, cuda_cores: bool = False) -> DecodePlan:
    """The plan for ``requests`` rows that bring one token each, none longer than ``max_seq_len`` positions.
    A step in which every request brings one token may hand the qkv product straight to the attention kernel
    (``fused``): every block then finishes its own queries, which costs less than a kernel of its own while all
    blocks are resident at once (three a SM) and more when they run in several rounds (measured at batch 64:
    2 % of the step).
    ``cuda_cores``: the attention has options only the CUDA-core kernel has (a sink, values of all kv heads; ``dv`` is
    then the width of a head's output row).
    ``fusable`` False: the caller prepares queries and cache itself (something stands between its projection and
    the attention); ``keep_first``: the window keeps the first positions in sight (the caller then prepares queries
    and cache itself as well).
    ``even``: the caller knows that the rows are about equally long (the longest at most an eighth over their
    mean).  Then, and when ``whole_rows_pay``, a block
    takes all keys of its row with three stages; rows of very different lengths keep their ranges, which spread a
    long row over many blocks."""
    if requests == 0:
        return DecodePlan(1, False, 0, "single")
    group = nq // nkv
    dv = int(dv or d)
    tensor_cores = dv == d and not values_in_keys and not cuda_cores and uses_tensor_cores(dtype, d)      # values of another head size run on CUDA cores
    fusable = fusable and not keep_first          # the kernel that takes the projection itself has no kept first positions
    row_blocks = -(-group // 16)                 # the tensor-core kernel takes 16 query heads of a kv head a block
    pairs = requests * nkv * row_blocks
    if even and tensor_cores and d <= 128 and _WHOLE_ROWS and whole_rows_pay(pairs, sm_count()):
        return DecodePlan(1, fusable and pairs <= 2 * sm_count(), 0, "whole rows", 3)
    room = (lambda s: decode_clusters(d, s, group)) if tensor_cores else None
    splits = choose_decode_splits(requests, nkv, max_seq_len, sm_count=sm_count(), clusters=room)
    in_clusters = tensor_cores and splits > 1 and pairs <= decode_clusters(d, splits, group)
    fused = fusable and tensor_cores and pairs * splits <= 3 * sm_count()
    arm = "single" if splits == 1 else ("cluster" if in_clusters else "wave")
    return DecodePlan(splits, fused, decode_scratch_floats(requests, nq, dv, splits), arm)


_WHOLE_ROWS = os.environ.get("LILY_B200_DECODE_WHOLE_ROWS", "1") != "0"



def prefill_tiles(prefix_lens: Sequence[int], new_lens: Sequence[int], first: int, rows: int,
                  device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(request, offset) of each tile of ``rows`` new tokens over the requests from ``first`` on, as two int32
    device tensors, in the order of the keys a tile attends to (the prefill kernels start with the last,
    longest ones)."""
    pairs = [(prefix_lens[r] + s, r, s) for r in range(first, len(new_lens)) for s in range(0, new_lens[r], rows)]
    pairs.sort()
    both = torch.tensor([[r for _, r, _ in pairs], [s for _, _, s in pairs]], dtype=torch.int32).reshape(2, -1)
    both = both.to(device, non_blocking=True)
    return both[0].contiguous(), both[1].contiguous()


def attention_decode_fused(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                           cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kv_layer: torch.Tensor,
                           block_table: torch.Tensor, seq_lens: torch.Tensor, out: torch.Tensor,
                           scratch: Optional[torch.Tensor], splits: int, nq: int, nkv: int, d: int, rotary_dim: int,
                           page_size: int, scale: float, window: Optional[int] = None, write_kv: bool = True,
                           stages: int = 0, softcap: Optional[float] = None) -> None:
    """``qk_norm_rope_write`` and ``attention_decode`` of a step in which every request brings one token, as one
    kernel: ``qkv`` is the projection's result ([requests, (nq + 2 nkv) d] in the cache's dtype, or float32 partial
    sums [splits, requests, ...]); the attention blocks finish their own query heads, and the block whose key range
    holds the new position finishes the key and the value and writes them to the cache before it reads them."""
    _dev(qkv, q_gain, k_gain, cos, sin, kv_layer, block_table, seq_lens, out, scratch)
    requests = qkv.shape[-2]
    planes, stride = _summed(qkv, requests, (nq + 2 * nkv) * d, "attention_decode_fused qkv")
    if not uses_tensor_cores(kv_layer.dtype, d) or out.dtype != kv_layer.dtype or qkv.dtype not in (kv_layer.dtype, torch.float32):
        raise KernelError(f"attention_decode_fused: cache {kv_layer.dtype}, qkv {qkv.dtype}, out {out.dtype}, head size {d}")
    if tuple(kv_layer.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"cache layer shape {tuple(kv_layer.shape)} does not fit kv_heads={nkv} page={page_size} d={d}")
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[-1] != rotary_dim // 2):
        raise KernelError("rotation tables must be float32 [positions, rotary_dim / 2]")
    if q_gain is not None and q_gain.dtype != k_gain.dtype:
        raise KernelError("q and k gains must share a dtype")
    need = decode_scratch_floats(requests, nq, d, splits)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: scratch of {need} float32 needed")
    _call("lily_attention_decode_mma_fused", _p(qkv), planes, stride, _dt(qkv), _p(q_gain), _p(k_gain),
          _dt(q_gain) if q_gain is not None else _F32, float(eps), _p(cos), _p(sin), int(rotary_dim), int(write_kv),
          _p(kv_layer), _p(out), _i32(block_table, "block_table"), block_table.shape[-1], _i32(seq_lens, "seq_lens"),
          _p(scratch), requests, splits, nq, nkv, d, page_size, int(window or 0), float(scale), int(stages),
          float(softcap or 0.0), _stream())
    if splits > 1 and (stages or requests * nkv * -(-(nq // nkv) // 16) > decode_clusters(d, splits, nq // nkv)):
        launches["count"] += 1                                       # the combine kernel, launched inside


# ------------------------------------------------------------------------------ joining sublayers

def _operand(t: torch.Tensor, rows: int, cols: int, what: str):
    """(pointer, dtype code, splits, stride) of an input that is [rows, cols] in float32 or bfloat16, or float32
    partial sums [splits, rows, cols]."""
    splits, stride = _summed(t, rows, cols, what)
    return _p(t), _dt(t), splits, stride


def sigmoid_gate(out: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """In place: ``out *= sigmoid(gate)``.  ``gate`` has ``out``'s shape [tokens, cols] (any of the two dtypes) or is
    float32 partial sums [splits, tokens, cols]."""
    _dev(out, gate)
    n, cols = out.shape
    ptr, dt, splits, stride = _operand(gate, n, cols, "sigmoid_gate")
    _call("lily_sigmoid_gate", _p(out), _dt(out), ptr, dt, splits, stride, out.numel(), _stream())
    return out


def normed_mean(inputs: Sequence[torch.Tensor], gains: Sequence[torch.Tensor], eps: float,
                add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``mean_k(rms(inputs[k]) * gains[k]) (+ add)`` row by row as float32 ``[1, tokens, width]`` (one plane of
    partial sums, which the residual norm takes): rms(v) = v / sqrt(mean(v^2) + eps).  Inputs and ``add`` are
    [tokens, width] or float32 partial sums [splits, tokens, width]; gains are float32 [width]."""
    count = len(inputs)
    lib = library()
    if not 1 <= count <= int(lib.lily_normed_mean_max()) or len(gains) != count:
        raise KernelError(f"normed_mean: {count} inputs with {len(gains)} gains")
    _dev(*inputs, *gains, add)
    n, width = inputs[0].shape[-2:]
    ops_ = [_operand(t, n, width, "normed_mean input") for t in inputs]
    for g in gains:
        if g.dtype != torch.float32 or g.numel() != width:
            raise KernelError("normed_mean: gains are float32 [width]")
    a = _operand(add, n, width, "normed_mean add") if add is not None else (None, _F32, 1, 0)
    out = torch.empty((1, n, width), dtype=torch.float32, device=inputs[0].device)
    ptrs = (ctypes.c_void_p * count)(*[o[0] for o in ops_])
    dts = (ctypes.c_int * count)(*[o[1] for o in ops_])
    sps = (ctypes.c_int * count)(*[o[2] for o in ops_])
    sts = (ctypes.c_size_t * count)(*[o[3] for o in ops_])
    gs = (ctypes.c_void_p * count)(*[g.data_ptr() for g in gains])
    _call("lily_normed_mean", ptrs, dts, sps, sts, gs, count, a[0], a[1], a[2], a[3], _p(out), n, width, float(eps),
          1.0 / count, _stream())
    return out


# ------------------------------------------------------------------------------ state-space mixer

SSM_CHUNK = 64          # new tokens a thread of the convolution kernel walks; a portion is cut at multiples of it


def token_chunks(new_lens: Sequence[int], chunk: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(request, offset) of every run of up to ``chunk`` new tokens of every request, as two int32 device tensors."""
    pairs = [(r, s) for r, n in enumerate(new_lens) for s in range(0, n, chunk)]
    both = torch.tensor([[r for r, _ in pairs], [s for _, s in pairs]], dtype=torch.int32).reshape(2, -1)
    both = both.to(device, non_blocking=True)
    return both[0].contiguous(), both[1].contiguous()


def causal_conv_silu(proj: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     state: torch.Tensor, state_off: int, chunk_req: torch.Tensor, chunk_start: torch.Tensor,
                     cu_seqlens: torch.Tensor, slots: torch.Tensor, chunk: int = SSM_CHUNK) -> torch.Tensor:
    """``silu(bias + causal depthwise convolution)`` over the columns ``[col0, col0 + channels)`` of ``proj``
    [tokens, width], request by request: ``weight`` is float32 [channels, taps] whose last column multiplies the
    current token; the ``taps - 1`` inputs before a portion's first token are read from, and its last ones written
    to, ``state[slot, state_off:]`` (float32, [(taps - 1), channels], oldest first; zero for a new request)."""
    _dev(proj, weight, bias, state, chunk_req, chunk_start, cu_seqlens, slots)
    n, width = proj.shape
    taps = weight.shape[1]
    if weight.dtype != torch.float32 or tuple(weight.shape) != (channels, taps) or state.dtype != torch.float32:
        raise KernelError("causal_conv_silu: float32 weights [channels, taps] and a float32 state")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != channels):
        raise KernelError("causal_conv_silu: the bias is float32 [channels]")
    if state.dim() != 2 or state_off + (taps - 1) * channels > state.shape[1] or col0 + channels > width:
        raise KernelError("causal_conv_silu: columns or state out of range")
    out = torch.empty((n, channels), dtype=proj.dtype, device=proj.device)
    _call("lily_causal_conv_silu", _p(proj), width, int(col0), int(channels), int(taps), _p(weight), _p(bias), _p(state),
          state.shape[1], int(state_off), _p(out), _i32(chunk_req, "chunk_req"), _i32(chunk_start, "chunk_start"),
          chunk_req.numel(), int(chunk), _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"), _dt(proj), _stream())
    return out


def causal_conv(proj: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                state: torch.Tensor, state_off: int, chunk_req: torch.Tensor, chunk_start: torch.Tensor,
                cu_seqlens: torch.Tensor, slots: torch.Tensor, chunk: int = SSM_CHUNK, activation: str = "silu") -> torch.Tensor:
    """``causal_conv_silu`` with the activation named: "silu", or "none" for the convolution alone."""
    if activation not in ("silu", "none"):
        raise KernelError(f"causal_conv: no activation {activation!r}; have 'silu' and 'none'")
    _dev(proj, weight, bias, state, chunk_req, chunk_start, cu_seqlens, slots)
    n, width = proj.shape
    taps = weight.shape[1]
    if state is None and taps > 1:
        raise KernelError("causal_conv: only a single tap carries nothing from step to step")
    if weight.dtype != torch.float32 or tuple(weight.shape) != (channels, taps) or (state is not None and state.dtype != torch.float32):
        raise KernelError("causal_conv: float32 weights [channels, taps] and a float32 state")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != channels):
        raise KernelError("causal_conv: the bias is float32 [channels]")
    if col0 + channels > width or (state is not None and (state.dim() != 2 or state_off + (taps - 1) * channels > state.shape[1])):
        raise KernelError("causal_conv: columns or state out of range")
    out = torch.empty((n, channels), dtype=proj.dtype, device=proj.device)
    _call("lily_causal_conv", _p(proj), width, int(col0), int(channels), int(taps), _p(weight), _p(bias), _p(state),
          state.shape[1] if state is not None else 0, int(state_off), _p(out), _i32(chunk_req, "chunk_req"), _i32(chunk_start, "chunk_start"),
          chunk_req.numel(), int(chunk), _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"), _dt(proj),
          1 if activation == "silu" else 0, _stream())
    return out


SCAN_CHUNK = 128        # tokens a chunk of a long portion (doubled while the chunk states would pass SCAN_WORKSPACE)
SCAN_DIRECT = 192       # portions up to this many tokens run in one piece, from and to the state in the slot
SCAN_WORKSPACE = 1 << 29


@dataclass
class ScanPlan:
    """How the selective scan of a step runs: the requests whose new tokens run in one piece (``direct``), and the
    long portions cut into chunks that run side by side (``scan_plan``).  All lists are int32 on the device."""

    direct: Optional[torch.Tensor]           # request indices, or None when every request runs in one piece
    num_direct: int
    chunk_req: Optional[torch.Tensor] = None
    chunk_start: Optional[torch.Tensor] = None
    chunk_len: Optional[torch.Tensor] = None
    num_chunks: int = 0
    long_req: Optional[torch.Tensor] = None
    long_first: Optional[torch.Tensor] = None
    long_count: Optional[torch.Tensor] = None
    num_long: int = 0
    chunk: int = 0                           # the longest chunk, in tokens


def scan_plan(new_lens: Sequence[int], device, state_floats: int = 0) -> ScanPlan:
    """Cuts the step's portions for the scan.  A portion of up to SCAN_DIRECT tokens (every decoded token) runs in one
    piece; a longer one in chunks of SCAN_CHUNK tokens that run side by side and are joined by ``ssd_combine``
    (``state_floats``: the size of one scan state, which bounds how many chunks the workspace may hold)."""
    longs = [r for r, n in enumerate(new_lens) if n > SCAN_DIRECT]
    if not longs:
        return ScanPlan(None, len(new_lens))
    chunk = SCAN_CHUNK
    while chunk < 1024 and state_floats and sum(-(-new_lens[r] // chunk) for r in longs) * state_floats * 4 > SCAN_WORKSPACE:
        chunk *= 2
    direct = [r for r, n in enumerate(new_lens) if n <= SCAN_DIRECT]
    creq, cstart, clen, lfirst, lcount = [], [], [], [], []
    for r in longs:
        lfirst.append(len(creq))
        for s in range(0, new_lens[r], chunk):
            creq.append(r)
            cstart.append(s)
            clen.append(min(chunk, new_lens[r] - s))
        lcount.append(len(creq) - lfirst[-1])
    flat = direct + creq + cstart + clen + longs + lfirst + lcount
    dev = torch.tensor(flat, dtype=torch.int32).to(device, non_blocking=True)
    sizes = [len(direct)] + [len(creq)] * 3 + [len(longs)] * 3
    parts = torch.split(dev, sizes)
    return ScanPlan(parts[0], len(direct), parts[1], parts[2], parts[3], len(creq), parts[4], parts[5], parts[6], len(longs),
                    chunk)


def ssd_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             d_skip: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, requests: int,
             heads: int, head_dim: int, n_state: int, groups: int, plan: Optional[ScanPlan] = None,
             workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The selective scan of each request's new tokens from its carried state, per head h of group g:
    ``S = exp(-exp(a_log[h]) dt) S + dt B x^T``, ``y = S^T C + d_skip[h] x`` with ``dt = softplus(proj[:, dt_col + h] +
    dt_bias[h])``, x = ``xbc[:, h * head_dim:]``, B and C = ``xbc[:, heads * head_dim + (g | groups + g) * n_state:]``.
    ``state[slot, :heads * head_dim * n_state]`` holds S as [heads, head_dim, n_state] and is updated in place.
    With a ``plan`` (``scan_plan``) long portions run as chunks side by side through ``workspace`` (float32,
    ``scan_workspace_floats``; made here when absent).  Returns y float32 [tokens, heads * head_dim]."""
    _dev(xbc, proj, dt_bias, a_log, d_skip, state, cu_seqlens, slots, workspace)
    n, channels = xbc.shape
    inner = heads * head_dim
    if channels != inner + 2 * groups * n_state or proj.dtype != xbc.dtype or proj.shape[0] != n:
        raise KernelError(f"ssd_scan: xbc {tuple(xbc.shape)} {xbc.dtype} against proj {tuple(proj.shape)} {proj.dtype}")
    for v in (dt_bias, a_log, d_skip):
        if v.dtype != torch.float32 or v.numel() != heads:
            raise KernelError("ssd_scan: dt_bias, a_log and d_skip are float32 [heads]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < inner * n_state or dt_col + heads > proj.shape[1]:
        raise KernelError("ssd_scan: state or dt columns out of range")
    y = torch.empty((n, inner), dtype=torch.float32, device=xbc.device)
    common = (_p(xbc), channels, _p(proj), proj.shape[1], int(dt_col), _p(dt_bias), _p(a_log), _p(d_skip), _p(state),
              state.shape[1], _p(y), _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"))
    sizes = (heads, head_dim, n_state, groups, _dt(xbc))
    if plan is None or plan.direct is None:
        _call("lily_ssd_scan", *common, int(requests), *sizes, None, None, None, 0, None, None, 0, _stream())
        return y
    if plan.num_direct:
        _call("lily_ssd_scan", *common, plan.num_direct, *sizes, _p(plan.direct), None, None, 0, None, None, 0, _stream())
    need = scan_workspace_floats(plan, heads, head_dim, n_state)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=xbc.device)
    if workspace.dtype != torch.float32 or workspace.numel() < need:
        raise KernelError(f"ssd_scan: a float32 workspace of {need} entries needed")
    chunk_state, chunk_decay = workspace, workspace[plan.num_chunks * inner * n_state:]
    items = (_p(plan.chunk_req), _p(plan.chunk_start), _p(plan.chunk_len))
    _call("lily_ssd_scan", *common, plan.num_chunks, *sizes, *items, 1, _p(chunk_state), _p(chunk_decay), plan.chunk, _stream())
    _call("lily_ssd_combine", _p(state), state.shape[1], _i32(slots, "slots"), _p(chunk_state), _p(chunk_decay),
          _p(plan.long_req), _p(plan.long_first), _p(plan.long_count), plan.num_long, heads, head_dim * n_state, _stream())
    _call("lily_ssd_scan", *common, plan.num_chunks, *sizes, *items, 2, _p(chunk_state), _p(chunk_decay), plan.chunk, _stream())
    return y


def scan_workspace_floats(plan: Optional[ScanPlan], heads: int, head_dim: int, n_state: int) -> int:
    """float32 entries ``ssd_scan`` needs for this plan: a state and one decay a head for every chunk."""
    if plan is None or not plan.num_chunks:
        return 0
    return plan.num_chunks * (heads * head_dim * n_state + heads)


def gated_group_rmsnorm(y: torch.Tensor, proj: torch.Tensor, gain: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """``v = y * silu(z)`` with z the first ``y.shape[1]`` columns of ``proj``; each of ``groups`` equal runs of columns
    divided by its own root mean square (eps inside the root), times ``gain`` (float32).  Returns ``proj``'s dtype."""
    _dev(y, proj, gain)
    n, inner = y.shape
    if y.dtype != torch.float32 or gain.dtype != torch.float32 or gain.numel() != inner or proj.shape[0] != n or proj.shape[1] < inner:
        raise KernelError("gated_group_rmsnorm: float32 y [tokens, inner] and gain [inner], proj [tokens, >= inner]")
    out = torch.empty((n, inner), dtype=proj.dtype, device=y.device)
    _call("lily_gated_group_rmsnorm", _p(y), _p(proj), proj.shape[1], _p(gain), _p(out), n, inner, int(groups), float(eps),
          _dt(proj), _stream())
    return out



# ------------------------------------------------------------------------------ per-head products

def head_linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """One product per head: ``x`` [tokens, heads, k] (a view whose last axis is contiguous; the heads may be columns
    of a wider row), ``weight`` [heads, n, k]; returns [heads, tokens, n].  float32: this package's FFMA kernel, a
    head a grid plane; bfloat16: the library's batched product with float32 accumulation (``out_dtype=float32``
    keeps the accumulator's precision)."""
    _dev(weight)
    tokens, heads, k = x.shape
    if not x.is_cuda or x.stride(2) != 1 or weight.shape[0] != heads or weight.shape[2] != k or weight.dtype != x.dtype:
        raise KernelError(f"head_linear: x {tuple(x.shape)} {x.dtype} strides {x.stride()} against weight {tuple(weight.shape)} {weight.dtype}")
    n = weight.shape[1]
    if x.dtype == torch.float32:
        out = torch.empty((heads, tokens, n), dtype=torch.float32, device=x.device)
        _call("lily_gemm_fp32_heads", _p(x), _p(weight), _p(out), tokens, n, k, x.stride(0), n, heads, x.stride(1), n * k,
              tokens * n, _stream())
        return out
    if out_dtype == torch.float32:
        return torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out_dtype=torch.float32)
    return torch.bmm(x.transpose(0, 1), weight.transpose(1, 2))


# ------------------------------------------------------------------------------ linear attention with a data-dependent decay

def token_shift_mix(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, state_off: int, cu_seqlens: torch.Tensor,
                    token_req: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """``out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]`` for each row s of ``mu`` (float32 [streams, width]); ahead of a
    request's first new token stands the input its slot carries (``state`` float32 [slots, row], from column
    ``state_off`` on; zeros for a new request), and the slot then takes the request's last new input.
    Returns [streams, tokens, width] in ``h``'s dtype."""
    _dev(h, mu, state, cu_seqlens, token_req, slots)
    tokens, width = h.shape
    if mu.dtype != torch.float32 or mu.shape[-1] != width or state.dtype != torch.float32:
        raise KernelError("token_shift_mix: mu and the state are float32, mu [streams, width]")
    if state_off + width > state.shape[1]:
        raise KernelError("token_shift_mix: the carried input does not fit the state row")
    streams = mu.shape[0]
    out = torch.empty((streams, tokens, width), dtype=h.dtype, device=h.device)
    _call("lily_token_shift_mix", _p(h), tokens, width, _p(mu), streams, _p(state), state.stride(0), state_off,
          _i32(cu_seqlens, "cu_seqlens"), _i32(token_req, "token_req"), _i32(slots, "slots"), _p(out), _dt(h), _stream())
    return out


def wkv_decay(a: torch.Tensor, w2t: torch.Tensor, w0: torch.Tensor) -> torch.Tensor:
    """The logarithm of the decay, ``-exp(w0 + tanh(a) . w2t)``: ``a`` [tokens, rank], ``w2t`` [rank, columns],
    ``w0`` [columns], all float32; returns float32 [tokens, columns]."""
    _dev(a, w2t, w0)
    if a.dtype != torch.float32 or w2t.dtype != torch.float32 or w0.dtype != torch.float32:
        raise KernelError("wkv_decay works in float32")
    tokens, rank = a.shape
    cols = w2t.shape[1]
    if w2t.shape[0] != rank or w0.numel() != cols:
        raise KernelError(f"wkv_decay: a {tuple(a.shape)}, w2t {tuple(w2t.shape)}, w0 {tuple(w0.shape)}")
    out = torch.empty((tokens, cols), dtype=torch.float32, device=a.device)
    _call("lily_wkv_decay", _p(a), tokens, rank, _p(w2t), _p(w0), cols, _p(out), _stream())
    return out


def wkv_max_head_dim() -> int:
    return int(library().lily_wkv_max_head_dim())


WKV_CHUNK = 64          # tokens a chunk of a long portion
WKV_DIRECT = 128        # portions up to this many tokens run in one piece, from and to the matrices in the slot


@dataclass
class WkvPlan:
    """How a step's recurrence is cut: portions up to ``WKV_DIRECT`` tokens run whole; longer ones as chunks of
    ``WKV_CHUNK`` tokens side by side (each first from zero, then, once ``wkv_combine`` has walked the chunks, from the
    matrices it starts from).  The lists are device int32; ``short_cu`` / ``short_slots`` describe the short portions
    as requests of their own."""

    items: int
    item_req: Optional[torch.Tensor]
    item_start: Optional[torch.Tensor]
    item_len: Optional[torch.Tensor]
    longs: int
    long_req: Optional[torch.Tensor]
    long_first: Optional[torch.Tensor]
    long_count: Optional[torch.Tensor]
    short_reqs: Optional[torch.Tensor]      # requests that run whole (None: all of them)
    shorts: int


def wkv_plan(new_lens: Sequence[int], device) -> Optional[WkvPlan]:
    """None when every portion runs whole."""
    if not new_lens or max(new_lens) <= WKV_DIRECT:
        return None
    item_req, item_start, item_len, long_req, long_first, long_count, short = [], [], [], [], [], [], []
    for r, n in enumerate(new_lens):
        if n <= WKV_DIRECT:
            short.append(r)
            continue
        long_req.append(r)
        long_first.append(len(item_req))
        long_count.append(-(-n // WKV_CHUNK))
        for s0 in range(0, n, WKV_CHUNK):
            item_req.append(r)
            item_start.append(s0)
            item_len.append(min(WKV_CHUNK, n - s0))
    flat = torch.tensor(item_req + item_start + item_len + long_req + long_first + long_count + short, dtype=torch.int32)
    flat = flat.to(device, non_blocking=True)
    a, b = len(item_req), len(long_req)
    parts = torch.split(flat, [a, a, a, b, b, b, len(short)])
    return WkvPlan(a, parts[0], parts[1], parts[2], b, parts[3], parts[4], parts[5], parts[6] if short else None, len(short))


def wkv_workspace_floats(plan: Optional[WkvPlan], heads: int, d: int) -> int:
    return 0 if plan is None else plan.items * heads * (d * d + d)


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_decay: torch.Tensor, u: torch.Tensor,
             state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, requests: int, heads: int,
             d: int, plan: Optional[WkvPlan] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The recurrence, a request's new tokens one after another from and to the head matrices in its slot (the first
    ``heads * d * d`` numbers of the row, [head, key row, value column]):
    ``o_t = (S + diag(u) k_t v_t^T)^T r_t``, then ``S <- diag(exp(log_decay_t)) S + k_t v_t^T``.
    ``r``, ``k``, ``v`` [tokens, heads * d] in the activation dtype (rows of equal stride), ``log_decay`` float32
    [tokens, heads * d], ``u`` float32 [heads, d].  Returns float32 [tokens, heads * d].  With a ``plan`` (``wkv_plan``)
    and its ``workspace`` (float32, ``wkv_workspace_floats``) long portions run as chunks side by side."""
    _dev(log_decay, u, state, cu_seqlens, slots, workspace)
    tokens = r.shape[0]
    stride = r.stride(0)
    for t in (r, k, v):
        if not t.is_cuda or t.dtype != r.dtype or t.stride(1) != 1 or t.stride(0) != stride or t.shape != (tokens, heads * d):
            raise KernelError("wkv_scan: r, k and v are [tokens, heads * d] of one dtype and row stride")
    if log_decay.dtype != torch.float32 or u.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("wkv_scan: decay, bonus and state are float32")
    if state.shape[1] < heads * d * d:
        raise KernelError("wkv_scan: the state row is too short for the head matrices")
    y = torch.empty((tokens, heads * d), dtype=torch.float32, device=r.device)
    common = (_p(r), _p(k), _p(v), stride, _p(log_decay), _p(u), _p(state), state.stride(0), _p(y),
              _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"))
    if plan is None:
        _call("lily_wkv_scan", *common, requests, heads, d, _dt(r), 0, None, None, None, None, None, _stream())
        return y
    need = wkv_workspace_floats(plan, heads, d)
    if workspace is None or workspace.dtype != torch.float32 or workspace.numel() < need:
        raise KernelError(f"wkv_scan: chunks need a float32 workspace of {need}")
    ws_state = workspace
    ws_decay = workspace[plan.items * heads * d * d:]
    chunks = (_p(plan.item_req), _p(plan.item_start), _p(plan.item_len), _p(ws_state), _p(ws_decay))
    _call("lily_wkv_scan", *common, plan.items, heads, d, _dt(r), 1, *chunks, _stream())
    _call("lily_wkv_combine", _p(state), state.stride(0), _i32(slots, "slots"), _p(ws_state), _p(ws_decay), _p(plan.long_req),
          _p(plan.long_first), _p(plan.long_count), plan.longs, heads, d, _stream())
    _call("lily_wkv_scan", *common, plan.items, heads, d, _dt(r), 2, *chunks, _stream())
    if plan.shorts:
        # the short portions of the same step run whole, from and to their slots
        _call("lily_wkv_scan", *common, plan.shorts, heads, d, _dt(r), 3, _p(plan.short_reqs), None, None, None, None, _stream())
    return y


def group_rmsnorm_gate(y: torch.Tensor, gate: torch.Tensor, gain: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """``y / rms(y over the column's group) * gain * silu(gate)``: ``y`` float32 [tokens, inner], ``gate`` [tokens, inner]
    in the activation dtype (its rows may be strided), ``gain`` float32 [inner]; returns the gate's dtype."""
    _dev(y, gain)
    tokens, inner = y.shape
    if y.dtype != torch.float32 or gain.dtype != torch.float32 or gate.shape != y.shape or gate.stride(1) != 1:
        raise KernelError("group_rmsnorm_gate: y and the gain are float32, the gate has y's shape")
    out = torch.empty((tokens, inner), dtype=gate.dtype, device=y.device)
    _call("lily_group_rmsnorm_gate", _p(y), _p(gate), gate.stride(0), _p(gain), _p(out), tokens, inner, groups, float(eps),
          _dt(gate), _stream())
    return out


# ------------------------------------------------------------------------------ attention over a cached latent

def latent_prepare(down: torch.Tensor, q0: int, q_rank: int, kv0: int, rank: int, rot: int, rotary_dim: int,
                   q_gain: torch.Tensor, kv_gain: torch.Tensor, eps: float, cos: Optional[torch.Tensor],
                   sin: Optional[torch.Tensor], positions: torch.Tensor, token_req: torch.Tensor,
                   block_table: torch.Tensor, layer: torch.Tensor, page_size: int, write_kv: bool = True) -> torch.Tensor:
    """From a token's row of the stacked down-projection ``down`` (the cache's dtype or float32): the RMS-normed query
    latent (columns ``q0`` on, ``q_rank`` of them, gain ``q_gain``), returned as [tokens, q_rank] in the cache's
    dtype; and into the token's cache row [rank + rot] of ``layer`` [pages, page_size * (rank + rot)] the RMS-normed
    key/value latent (columns ``kv0`` on, gain ``kv_gain``) followed by the ``rot`` columns after it, the first
    ``rotary_dim`` of them rotated in halves by the position's angles."""
    _dev(down, q_gain, kv_gain, cos, sin, positions, token_req, block_table, layer)
    tokens = down.shape[0]
    if layer.dim() != 2 or layer.shape[1] != page_size * (rank + rot):
        raise KernelError(f"latent_prepare: cache layer {tuple(layer.shape)} does not hold pages of {page_size} rows of {rank + rot}")
    if q_gain.dtype != torch.float32 or kv_gain.dtype != torch.float32:
        raise KernelError("latent_prepare: gains are float32")
    if rotary_dim and (cos is None or cos.dtype != torch.float32 or cos.shape[-1] != rotary_dim // 2):
        raise KernelError("rotation tables must be float32 [positions, rotary_dim / 2]")
    cq = torch.empty((tokens, q_rank), dtype=layer.dtype, device=down.device)
    _call("lily_latent_prepare", _p(down), _dt(down), down.stride(0), q0, q_rank, kv0, rank, rot, rotary_dim, _p(q_gain),
          _p(kv_gain), float(eps), _p(cos), _p(sin), _i32(positions, "positions"), _i32(token_req, "token_req"),
          _i32(block_table, "block_table"), block_table.shape[-1], _p(layer), page_size, int(write_kv), _p(cq), tokens,
          _dt(layer), _stream())
    return cq


def latent_query(qa: torch.Tensor, q: torch.Tensor, heads: int, d: int, rank: int, rot: int, rotary_dim: int,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor) -> torch.Tensor:
    """The queries the attention over the latent takes, [tokens, heads * (rank + rot)] in ``q``'s dtype: for each head
    ``qa[head, token]`` (its unrotated part carried into the latent's space, [heads, tokens, rank], ``q``'s dtype or
    float32) followed by the last ``rot`` columns of the head in ``q`` [tokens, heads * (d + rot)], rotated."""
    _dev(qa, q, cos, sin, positions)
    tokens = q.shape[0]
    if tuple(qa.shape) != (heads, tokens, rank) or q.shape[1] != heads * (d + rot):
        raise KernelError(f"latent_query: qa {tuple(qa.shape)}, q {tuple(q.shape)}")
    out = torch.empty((tokens, heads * (rank + rot)), dtype=q.dtype, device=q.device)
    _call("lily_latent_query", _p(qa), _dt(qa), _p(q), tokens, heads, d, rank, rot, rotary_dim, _p(cos), _p(sin),
          _i32(positions, "positions"), _p(out), _dt(q), _stream())
    return out


def head_gate(ov: torch.Tensor, gate_rows: torch.Tensor, g0: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``out[t, h * dv + j] = ov[h, t, j] * sigmoid(gate_rows[t, g0 + h])``: ``ov`` [heads, tokens, dv]."""
    _dev(ov, gate_rows)
    heads, tokens, dv = ov.shape
    out = torch.empty((tokens, heads * dv), dtype=out_dtype, device=ov.device)
    _call("lily_head_gate", _p(ov), _dt(ov), _p(gate_rows), _dt(gate_rows), gate_rows.stride(0), g0, tokens, heads, dv,
          _p(out), _dt(out), _stream())
    return out


# ------------------------------------------------------------------------------ routed experts

@dataclass
class ExpertRouting:
    """A step's routing for one layer, all on the device: ``chosen`` / ``weights`` [tokens, top]; the pairs (token, choice)
    of experts that have weights grouped by expert (``offsets``, ``order``, ``place``) and the tiles the grouped
    products run over."""

    chosen: torch.Tensor
    weights: torch.Tensor
    offsets: torch.Tensor
    order: torch.Tensor
    place: torch.Tensor
    tile_expert: torch.Tensor
    tile_row: torch.Tensor
    tile_count: torch.Tensor
    max_tiles: int
    top: int


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int, experts: int) -> ExpertRouting:
    """Softmax scores over all router outputs (float32 logits ``router . h``), the ``top`` largest scores + correction
    chosen, their weights the scores themselves over their sum; then the pairs of the first ``experts`` outputs (those
    with weights; the rest stand for the identity) grouped by expert."""
    _dev(h, router, correction)
    tokens, width = h.shape
    outputs = router.shape[0]
    if router.dtype != torch.float32 or correction.dtype != torch.float32 or router.shape[1] != width or correction.numel() != outputs:
        raise KernelError("moe_route: router [outputs, width] and correction [outputs] are float32")
    dev = h.device
    pairs = tokens * top
    tile_rows = int(library().lily_moe_tile_rows())
    max_tiles = -(-pairs // tile_rows) + experts
    ints = torch.empty(3 * pairs + experts + 1 + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
    chosen, order, place, offsets, tile_expert, tile_row, tile_count = torch.split(
        ints, [pairs, pairs, pairs, experts + 1, max_tiles, max_tiles, 1])
    weights = torch.empty((tokens, top), dtype=torch.float32, device=dev)
    _call("lily_moe_route", _p(h), tokens, width, _p(router), _p(correction), outputs, top, _p(chosen), _p(weights), _dt(h),
          _stream())
    _call("lily_moe_align", _p(chosen), pairs, experts, _p(offsets), _p(order), _p(place), _p(tile_expert), _p(tile_row),
          _p(tile_count), max_tiles, _stream())
    return ExpertRouting(chosen.view(tokens, top), weights, offsets, order, place, tile_expert, tile_row, tile_count,
                         max_tiles, top)


_OWN_GROUPED = os.environ.get("LILY_B200_GROUPED_GEMM", "") == "own"


def grouped_library_takes(dtype: torch.dtype, width: int, ff: int) -> bool:
    """Whether the experts' two products go to the library's grouped product (bfloat16 with rows of whole 16-byte
    units); everything else, and float32 always, runs on this package's grouped kernel."""
    return (dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0 and hasattr(torch, "_grouped_mm")
            and not _OWN_GROUPED)


def moe_experts(h: torch.Tensor, routing: ExpertRouting, w_gate_up: torch.Tensor, w_down: torch.Tensor, limit: float,
                alpha: float) -> torch.Tensor:
    """The chosen experts' outputs summed with their weights, float32 [tokens, width].  ``w_gate_up`` [experts, 2 ff,
    width] (an expert's gate rows, then its up rows), ``w_down`` [experts, width, ff].  An expert computes
    ``W_down (g sigmoid(alpha g) (u + 1))`` with ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``; a
    choice beyond the experts that have weights contributes ``h`` itself."""
    _dev(h, w_gate_up, w_down)
    tokens, width = h.shape
    r = routing
    pairs = tokens * r.top
    experts = w_down.shape[0] if w_down.dim() == 3 else 0
    ff = w_down.shape[2] if experts else 0
    if experts and grouped_library_takes(h.dtype, width, ff):
        # bfloat16: the library's grouped product over the rows in grouped order (groups end at offsets[1:])
        ends = r.offsets[1:]
        rows = torch.empty((pairs, width), dtype=h.dtype, device=h.device)
        _call("lily_moe_gather", _p(h), width, _p(r.offsets), experts, _p(r.order), r.top, pairs, _p(rows), _dt(h), _stream())
        gate_up = torch._grouped_mm(rows, w_gate_up.transpose(1, 2), offs=ends)
        act = torch.empty((pairs, ff), dtype=h.dtype, device=h.device)
        _call("lily_moe_activation", _p(gate_up), ff, pairs, _p(act), float(limit), float(alpha), _dt(h), _stream())
        y = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends)
        out = torch.empty((tokens, width), dtype=torch.float32, device=h.device)
        _call("lily_moe_combine_rows", _p(y), _p(h), _p(r.place), _p(r.weights), tokens, r.top, width, _p(out), _dt(h), _stream())
        return out
    y = torch.empty((max(pairs, 1), width), dtype=torch.float32, device=h.device)
    if experts:
        if w_gate_up.dtype != h.dtype or w_down.dtype != h.dtype or tuple(w_gate_up.shape) != (experts, 2 * ff, width):
            raise KernelError(f"moe_experts: weights {tuple(w_gate_up.shape)} / {tuple(w_down.shape)} {w_down.dtype} for inputs {tuple(h.shape)} {h.dtype}")
        act = torch.empty((max(pairs, 1), ff), dtype=h.dtype, device=h.device)
        _call("lily_moe_gemm", 0, _p(h), h.stride(0), _p(w_gate_up), ff, width, _p(r.offsets), _p(r.order), r.top,
              _p(r.tile_expert), _p(r.tile_row), _p(r.tile_count), r.max_tiles, _p(act), float(limit), float(alpha), _dt(h),
              _stream())
        _call("lily_moe_gemm", 1, _p(act), ff, _p(w_down), width, ff, _p(r.offsets), _p(r.order), r.top, _p(r.tile_expert),
              _p(r.tile_row), _p(r.tile_count), r.max_tiles, _p(y), 0.0, 0.0, _dt(h), _stream())
    out = torch.empty((tokens, width), dtype=torch.float32, device=h.device)
    _call("lily_moe_combine", _p(y), _p(h), _p(r.place), _p(r.weights), tokens, r.top, width, _p(out), _dt(h), _stream())
    return out


# ------------------------------------------------------------------------------ sampling

def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(logits, out)
    if logits.dtype != torch.float32:
        raise KernelError("argmax takes float32 logits")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    chunks = int(library().lily_argmax_chunks(rows, vocab))
    pv = pi = None
    if chunks > 1:          # a large vocabulary: many blocks per row, then a merge
        pv = torch.empty((rows * chunks,), dtype=torch.float32, device=logits.device)
        pi = torch.empty((rows * chunks,), dtype=torch.int32, device=logits.device)
        launches["count"] += 1
    _call("lily_argmax", _p(logits), _i32(out, "out"), _p(pv), _p(pi), rows, vocab, _stream())
    return out


def apply_penalties(logits: torch.Tensor, entry_row: torch.Tensor, entry_token: torch.Tensor,
                    entry_count: torch.Tensor, entry_bias: torch.Tensor, repetition: torch.Tensor,
                    frequency: torch.Tensor, presence: torch.Tensor) -> None:
    _dev(logits, entry_row, entry_token, entry_count, entry_bias, repetition, frequency, presence)
    rows, vocab = logits.shape
    _call("lily_apply_penalties", _p(logits), _i32(entry_row, "entry_row"), _i32(entry_token, "entry_token"),
          _i32(entry_count, "entry_count"), _p(entry_bias), _p(repetition), _p(frequency), _p(presence),
          entry_row.numel(), vocab, _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, want_logprob: bool = False):
    """One token per row of float32 ``logits``; per-row parameters are float32 (``top_k`` int32).
    Returns (tokens int32, logprobs float32 or None)."""
    _dev(logits, temperature, top_k, top_p, min_p, uniform)
    rows, vocab = logits.shape
    for t, name in ((temperature, "temperature"), (top_p, "top_p"), (min_p, "min_p"), (uniform, "uniform")):
        if t.dtype != torch.float32 or t.numel() != rows:
            raise KernelError(f"sample: {name} must be float32 [rows]")
    tokens = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    logprob = torch.empty((rows,), dtype=torch.float32, device=logits.device) if want_logprob else None
    _call("lily_sample", _p(logits), _p(temperature), _i32(top_k, "top_k"), _p(top_p), _p(min_p), _p(uniform),
          _p(tokens), _p(logprob), rows, vocab, _stream())
    return tokens, logprob


def top_logprobs_cap() -> int:
    """The most entries a row of ``top_logprobs`` can return."""
    return int(library().lily_top_logprobs_cap())


def top_logprobs(logits: torch.Tensor, k: torch.Tensor):
    """The ``k[r]`` most probable tokens of each row of float32 ``logits`` with their log-probabilities
    (log-softmax of the logits as given).  Returns (tokens int32 [rows, cap], logprobs float32 [rows, cap],
    counts int32 [rows]): row r holds ``counts[r] >= k[r]`` entries in no particular order (ties at the
    k-th value are all kept, up to cap); rows with ``k[r] <= 0`` hold none."""
    _dev(logits, k)
    if logits.dtype != torch.float32:
        raise KernelError("top_logprobs takes float32 logits")
    rows, vocab = logits.shape
    cap = top_logprobs_cap()
    tokens = torch.empty((rows, cap), dtype=torch.int32, device=logits.device)
    logprobs = torch.empty((rows, cap), dtype=torch.float32, device=logits.device)
    counts = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _call("lily_top_logprobs", _p(logits), _i32(k, "k"), _p(tokens), _p(logprobs), _p(counts), rows, vocab, _stream())
    return tokens, logprobs, counts


# ------------------------------------------------------------------------------ norms on both sides of a sublayer, plain feed-forward

PLAIN_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}
# LILY_B200_FUSED_ACTIVATION=0 keeps the plain feed-forward's activation a pass of its own behind the library product
_FUSED_ACTIVATION = os.environ.get("LILY_B200_FUSED_ACTIVATION", "1") != "0"


def add_normed_rmsnorm(resid: torch.Tensor, delta: torch.Tensor, post_gain: torch.Tensor, post_eps: float, mult: float,
                       weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                       rows: Optional[torch.Tensor] = None, write_residual: bool = True,
                       normalise: bool = True) -> Optional[torch.Tensor]:
    """``normalise`` False: ``resid += mult * (delta * post_gain)``, a gain per column without the division.
    ``resid += mult * (delta / rms(delta) * post_gain)`` in float32 (``delta`` [tokens, width] in either dtype, or
    float32 partial sums [splits, tokens, width]), then the new rows divided by their root mean square times ``weight``
    in ``out_dtype`` (None without ``weight``: the add alone).  With ``rows`` only those tokens' outputs are formed and
    the stream is left as it is."""
    _dev(resid, delta, post_gain, weight, rows)
    n, width = resid.shape
    if resid.dtype != torch.float32 or post_gain.dtype != torch.float32 or post_gain.numel() != width:
        raise KernelError("add_normed_rmsnorm: the residual stream and the gain behind the sublayer are float32")
    ptr, dt, splits, stride = _operand(delta, n, width, "add_normed_rmsnorm delta")
    if rows is not None and write_residual:
        raise KernelError("add_normed_rmsnorm: gathered rows are not written back")
    n_out = n if rows is None else rows.numel()
    out = None
    if weight is not None:
        if weight.numel() != width:
            raise KernelError("add_normed_rmsnorm: gain of another width")
        out = torch.empty((n_out, width), dtype=out_dtype, device=resid.device)
    elif rows is not None:
        return None
    _call("lily_add_normed_rmsnorm", _p(resid), ptr, dt, splits, stride, _p(post_gain), float(post_eps), float(mult),
          _p(weight), _dt(weight) if weight is not None else _F32, _p(out), _dt(out) if out is not None else _F32,
          _i32(rows, "rows"), n_out, width, float(eps), int(bool(write_residual)), int(bool(normalise)), _stream())
    return out


def activation(x: torch.Tensor, out_dtype: torch.dtype, activation: str = "relu2") -> torch.Tensor:
    """``act(x)`` elementwise: "relu2" (the square of max(., 0)), "silu" or "gelu_tanh"; ``x`` [tokens, cols] in either
    dtype or float32 partial sums [splits, tokens, cols]."""
    if activation not in PLAIN_ACTIVATIONS:
        raise KernelError(f"no activation {activation!r}; have {sorted(PLAIN_ACTIVATIONS)}")
    _dev(x)
    n, cols = x.shape[-2:]
    ptr, dt, splits, stride = _operand(x, n, cols, "activation")
    out = torch.empty((n, cols), dtype=out_dtype, device=x.device)
    _call("lily_activation", ptr, dt, splits, stride, _p(out), _dt(out), out.numel(), PLAIN_ACTIVATIONS[activation], _stream())
    return out


def linear_activation(x: torch.Tensor, weight: torch.Tensor, activation_name: str = "relu2") -> torch.Tensor:
    """``act(x @ weight.T)`` in ``x``'s dtype: for 65 tokens and more in bfloat16 the tcgen05 product with the activation
    in its epilogue (where ``gate_up_fused_pays``: the [tokens, N] intermediate is never written); else the product
    (whole, or float32 partial sums for a few tokens) with the activation as a pass over it."""
    if activation_name not in PLAIN_ACTIVATIONS:
        raise KernelError(f"no activation {activation_name!r}; have {sorted(PLAIN_ACTIVATIONS)}")
    if _FUSED_ACTIVATION and gate_up_fused_pays(x.shape[0], weight.shape[0]) and gemm_tc_takes(x, weight) and weight.is_contiguous():
        return gemm_tc(x, weight, plain_activation=activation_name)
    return activation(linear_auto(x, weight), x.dtype, activation_name)


# ------------------------------------------------------------------------------ differential attention

def diff_prepare(proj: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                 kv_layer: torch.Tensor, heads: int, nkv: int, d: int, dv: int, maps: int, page_size: int,
                 temp_coef: float, temp_every: int, write_kv: bool = True) -> torch.Tensor:
    """``proj`` [tokens, heads*maps*d | nkv*maps*d | nkv*dv | ...] in the cache's dtype.  Returns the queries
    [tokens, heads*maps * maps*d]: map m of head h as query head h*maps + m whose columns [m d, (m+1) d) hold the map's
    query times ``1 + temp_coef ln(floor((p + 1) / temp_every) + 1)`` and whose other columns are zero; writes each
    token's keys (rows of maps*d) and values to its place in its page (``cache_layer_fits`` with d = maps*d)."""
    _dev(proj, positions, token_req, block_table, kv_layer)
    n, width = proj.shape
    kd = maps * d
    if proj.dtype != kv_layer.dtype:
        raise KernelError(f"cache dtype {kv_layer.dtype} differs from activations {proj.dtype}")
    cache_layer_fits(kv_layer, nkv, page_size, kd, dv)
    q = torch.empty((n, heads * maps * kd), dtype=proj.dtype, device=proj.device)
    _call("lily_diff_prepare", _p(proj), width, _i32(positions, "positions"), _i32(token_req, "token_req"),
          _i32(block_table, "block_table"), block_table.shape[-1], _p(kv_layer), _p(q), n, heads, nkv, d, dv, maps,
          page_size, float(temp_coef), int(temp_every), int(write_kv), _dt(proj), _stream())
    return q


def diff_combine(maps_out: torch.Tensor, proj: torch.Tensor, gate_col: int, heads: int, dv: int, maps: int, lam: float,
                 out_scale: float, eps: float) -> torch.Tensor:
    """``maps_out`` [tokens, heads*maps*dv] (the maps' attention outputs, head by head): per head
    ``o = a_0 - lam a_1``, divided by its root mean square over dv, times ``out_scale``, times
    ``sigmoid(proj[:, gate_col + head])``; returns [tokens, heads*dv]."""
    _dev(maps_out, proj)
    n = maps_out.shape[0]
    if maps_out.dtype != proj.dtype or maps_out.shape[1] != heads * maps * dv:
        raise KernelError("diff_combine: the maps' outputs are [tokens, heads*maps*dv] in the projection's dtype")
    out = torch.empty((n, heads * dv), dtype=maps_out.dtype, device=maps_out.device)
    _call("lily_diff_combine", _p(maps_out), _p(proj), proj.shape[1], int(gate_col), _p(out), n, heads, dv, maps,
          float(lam), float(out_scale), float(eps), _dt(maps_out), _stream())
    return out


# ------------------------------------------------------------------------------ mixed heads, delta rule, selective scan

def head_mix(sums: torch.Tensor, mix: torch.Tensor, nq: int, nkv: int, dv: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``out[t, h] = sum_g mix[h, g] * sums[t, g, kv(h)]``: ``sums`` float32 [tokens, nq * nkv * dv] holds every query
    head's attention weights summed over the values of every kv head (``attention_*`` with ``all_values``), ``mix``
    float32 [nq, nq]; returns [tokens, nq * dv], each head over its own kv head's values with the mixed weights."""
    _dev(sums, mix)
    planes = sums.dim() == 3                   # [nkv, tokens, nq * dv]: plane s of a head of kv head g over kv head (g + s) % nkv
    tokens = sums.shape[-2]
    if mix.dtype != torch.float32 or tuple(mix.shape) != (nq, nq) or \
            (tuple(sums.shape) != (nkv, tokens, nq * dv) if planes else (sums.dtype != torch.float32 or sums.shape[1] != nq * nkv * dv)):
        raise KernelError("head_mix: float32 sums [tokens, nq * nkv * dv] or planes [nkv, tokens, nq * dv], and a float32 matrix [nq, nq]")
    out = torch.empty((tokens, nq * dv), dtype=out_dtype, device=sums.device)
    _call("lily_head_mix", _p(sums), _dt(sums), int(planes), _p(mix), _p(out), tokens, nq, nkv, dv, _dt(out), _stream())
    return out


def delta_rule_max_head_dim() -> int:
    return int(library().lily_delta_rule_max_head_dim())


def delta_rule(qkv: torch.Tensor, proj: torch.Tensor, b_col: int, a_col: int, a_log: torch.Tensor, dt_bias: torch.Tensor,
               state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, requests: int, heads: int, kv_heads: int,
               d: int, dv: int, unit_eps: float, q_scale: float) -> torch.Tensor:
    """The gated delta rule over each request's new tokens, from and to ``state[slot, :heads * dv * d]`` (float32,
    a head's matrix as [dv, d]).  ``qkv`` [tokens, (2 kv_heads) d + heads dv]: q, k, v behind their convolution and
    activation; ``proj`` [tokens, width]: ``heads`` columns from ``b_col`` (the write strength before its sigmoid) and
    from ``a_col`` (the decay's input).  q and k are made unit vectors per head here (``unit_eps`` inside the root; q
    times ``q_scale``); the decay is ``exp(-exp(a_log) softplus(a + dt_bias))``.  Returns float32 [tokens, heads * dv],
    each token read out after its own write."""
    _dev(qkv, proj, a_log, dt_bias, state, cu_seqlens, slots)
    n = qkv.shape[0]
    if qkv.shape[1] != 2 * kv_heads * d + heads * dv or proj.shape[0] != n or qkv.dtype != proj.dtype:
        raise KernelError("delta_rule: qkv is [tokens, 2 kv_heads d + heads dv] in the projection's dtype")
    if max(b_col, a_col) + heads > proj.shape[1] or a_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 \
            or a_log.numel() != heads or dt_bias.numel() != heads or state.dtype != torch.float32 or state.dim() != 2:
        raise KernelError("delta_rule: columns out of range, or decay constants / state not float32")
    y = torch.empty((n, heads * dv), dtype=torch.float32, device=qkv.device)
    _call("lily_delta_rule", _p(qkv), qkv.shape[1], 0, kv_heads * d, 2 * kv_heads * d, _p(proj), proj.shape[1], int(b_col),
          int(a_col), _p(a_log), _p(dt_bias), _p(state), state.shape[1], _p(y), _i32(cu_seqlens, "cu_seqlens"),
          _i32(slots, "slots"), int(requests), n, heads, kv_heads, d, dv, float(unit_eps), float(q_scale), _dt(qkv), _stream())
    return y


def selective_scan_max_state() -> int:
    return int(library().lily_selective_scan_max_state())


def selective_workspace_floats(plan: Optional[ScanPlan], inner: int, n_state: int) -> int:
    """Float32 scratch the chunks of ``plan`` need: a state and a sum of steps a chunk.  0 when the long portions are
    better run in one piece each: the chunked form does the recurrence's work twice, which pays while the blocks of the
    whole portions (16 channels a block) leave most of the device's warp slots empty (measured, 2,048 tokens of one
    request, 16 state entries: 4,096 channels 564 -> 419 us in chunks, 8,192 channels 666 -> 816 us)."""
    if plan is None or not plan.num_chunks:
        return 0
    if plan.num_long * -(-inner // 16) > 2.5 * sm_count():
        return 0
    return plan.num_chunks * inner * (n_state + 1)


def selective_scan(x: torch.Tensor, low: torch.Tensor, b_col: int, step: torch.Tensor, proj: torch.Tensor, z_col: int,
                   a: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
                   requests: int, plan: Optional[ScanPlan] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The selective scan with a state vector per channel over each request's new tokens, from and to
    ``state[slot, :inner * n]`` (float32).  ``x`` [tokens, inner]: the convolved, activated inputs; ``low``
    [tokens, width]: B in the ``n`` columns from ``b_col``, C in the ``n`` after them; ``step`` float32 [tokens, inner]:
    the step projection with its bias, before softplus; the gate z in ``proj[:, z_col:z_col + inner]``; ``a`` float32
    [inner, n] (negative); ``d_skip`` float32 [inner].  Returns ``(S . C + D x) * silu(z)`` in ``x``'s dtype.
    With a ``plan`` (``scan_plan``) that has chunks and a ``workspace`` of ``selective_workspace_floats``, the long
    portions run as chunks side by side (two passes and ``selective_combine`` between them), the others in one piece."""
    _dev(x, low, step, proj, a, d_skip, state, cu_seqlens, slots, workspace)
    tokens, inner = x.shape
    n = a.shape[1]
    if step.dtype != torch.float32 or tuple(step.shape) != (tokens, inner) or a.dtype != torch.float32 or a.shape[0] != inner \
            or d_skip.dtype != torch.float32 or d_skip.numel() != inner or state.dtype != torch.float32 or state.dim() != 2:
        raise KernelError("selective_scan: float32 steps [tokens, inner], A [inner, n], D [inner] and state")
    if low.dtype != x.dtype or proj.dtype != x.dtype or b_col + 2 * n > low.shape[1] or z_col + inner > proj.shape[1]:
        raise KernelError("selective_scan: B, C or gate columns out of range, or dtypes differ")
    out = torch.empty((tokens, inner), dtype=x.dtype, device=x.device)
    common = (_p(x), _p(low), low.shape[1], int(b_col), int(b_col) + n, _p(step), _p(proj), proj.shape[1], int(z_col), _p(a),
              _p(d_skip), _p(state), state.shape[1], _p(out), _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"))
    need = selective_workspace_floats(plan, inner, n)
    if not need:
        _call("lily_selective_scan", *common, int(requests), tokens, inner, n, _dt(x), None, None, None, 0, None, None, _stream())
        return out
    if workspace is None or workspace.dtype != torch.float32 or workspace.numel() < need:
        raise KernelError(f"selective_scan: a float32 workspace of {need} entries needed")
    ws_state = workspace.data_ptr()
    ws_steps = ws_state + 4 * plan.num_chunks * inner * n
    lists = (_i32(plan.chunk_req, "chunk_req"), _i32(plan.chunk_start, "chunk_start"), _i32(plan.chunk_len, "chunk_len"))
    _call("lily_selective_scan", *common, plan.num_chunks, tokens, inner, n, _dt(x), *lists, 1, ws_state, ws_steps, _stream())
    _call("lily_selective_combine", _p(state), state.shape[1], _i32(slots, "slots"), _i32(plan.long_req, "long_req"),
          _i32(plan.long_first, "long_first"), _i32(plan.long_count, "long_count"), plan.num_long, _p(a), ws_state, ws_steps,
          inner, n, _stream())
    _call("lily_selective_scan", *common, plan.num_chunks, tokens, inner, n, _dt(x), *lists, 2, ws_state, ws_steps, _stream())
    if plan.num_direct:
        _call("lily_selective_scan", *common, plan.num_direct, tokens, inner, n, _dt(x), _i32(plan.direct, "direct"), None, None,
              0, None, None, _stream())
    return out
