"""Python face of the CUDA kernels: argument checks, then one launch each.

Tensors are ``torch`` CUDA tensors used as typed device buffers; the launchers
get their pointers and the current stream.  Every function refuses what the
kernel behind it cannot do with a :class:`KernelError` that says why.  Nothing
here runs on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_lib = None
_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
_L = ctypes.c_longlong

_SIGNATURES = {
    "vcb_embedding": [_P, _P, _P, _I, _I, _I, _P],
    "vcb_add_rmsnorm": [_P, _P, _P, _P, _P, _I, _I, _F, _I, _P],
    "vcb_silu_mul": [_P, _P, _I, _I, _I, _P],
    "vcb_add_bias": [_P, _P, _I, _I, _I, _P],
    "vcb_rope_cache_write": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P],
    "vcb_attention_simt": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P],
    "vcb_gemm_f32": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "vcb_attention_decode_mma": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "vcb_attention_prefill_tc": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "vcb_gemm_bf16_tcgen05": [_P, _I, _I, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P],
    "vcb_gemm_bf16_tcgen05_fused": [_P, _I, _I, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _P, _I, _P,
                                    _P, _I, _I, _I, _F, _P, _I, _P, _P, _I, _I, _P],
    "vcb_tile_weights": [_P, _I, _I, _I, _I, _P, _P],
    "vcb_repetition_penalty": [_P, _I, _P, _P, _P, _I, _I, _P],
    "vcb_sample": [_P, _I, _I, _P, _P, _P, _I, _P],
    "vcb_sample_filtered": [_P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P],
    "vcb_random_normal": [_P, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_ulonglong, _F, _F, _I, _P],
    "vcb_attention_simt_planes": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _I, _P],
    "vcb_attention_decode_mma_planes": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _I, _I, _P],
    "vcb_attention_prefill_tc_planes": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P],
    "vcb_embedding_sinusoid": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _P, _I, _P],
    "vcb_token_shift": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "vcb_gated_norm_residual": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _F, _F, _I, _P],
    "vcb_latent_cache_write": [_P, _I, _P, _P, _P, _P, _I, _P, ctypes.c_longlong, _I, _I, _I, _F, _I, _P, _I, _P],
    "vcb_headwise_linear": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "vcb_sigmoid_gate": [_P, _P, _I, _I, _I, _I, _I, _I, _P],
    "vcb_rows_rmsnorm": [_P, _I, _P, _P, _I, _I, _I, _F, _I, _P],
    "vcb_latent_rope_cache_write": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _I, _P, _L, _I, _I, _I, _F, _I, _I, _P, _I, _P],
    "vcb_cast_rows": [_P, _P, _F, _P, _I, _I, _L, _I, _P],
    "vcb_add_rmsnorm_scaled": [_P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _P],
    "vcb_clamped_swish_mul": [_P, _P, _P, _I, _I, _F, _F, _F, _I, _P],
    "vcb_moe_router_biased": [_P, _L, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "vcb_moe_combine_add": [_P, _P, _L, _P, _P, _P, _I, _I, _I, _P, _L, _I, _P],
    "vcb_attention_talking_mma": [_P, _P, _P, _P, _L, _P, _I, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P, _I, _P],
    "vcb_attention_talking": [_P, _P, _P, _P, _L, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P],
    "vcb_attention_decode_mma_shaped_planes": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _I, _F, _P, _I,
                                               _P, _P, _L, _I, _I, _P],
    "vcb_attention_prefill_tc_shaped_planes": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _F, _P, _I, _P, _P, _L, _I, _I, _P],
    "vcb_attention_decode_mma_shaped": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _I, _F, _P, _I,
                                        _P, _P, _L, _I, _P],
    "vcb_attention_prefill_tc_shaped": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _F, _P, _I, _P, _P, _L, _I, _P],
    "vcb_embedding_scaled": [_P, _P, _P, _I, _I, _I, _P, _F, _I, _P],
    "vcb_norm_residual_norm": [_P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _P],
    "vcb_decayed_state_scan": [_P, _P, _P, _P, _L, _L, _L, _L, _P, _P, _F, _F, _I, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _P, _L, _P, _I, _P],
    "vcb_decayed_state_join": [_P, _L, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "vcb_gated_group_norm": [_P, _L, _P, _L, _P, _I, _P, _L, _I, _I, _I, _I, _F, _I, _P],
    "vcb_scaled_sum": [_P, _P, _P, _L, _F, _F, _I, _P],
    "vcb_qk_norm_cache_write": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P],
    "vcb_attention_biased": [_P, _P, _P, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P, _P, _I, _I, _P],
    "vcb_qk_head_rope_cache_write": [_P, _L, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P],
    "vcb_moe_router": [_P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "vcb_moe_router_ruled": [_P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "vcb_stream_norm": [_P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _F, _F, _I, _P],
    "vcb_stream_join": [_P, _L, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P],
    "vcb_causal_conv": [_P, _L, _P, _P, _P, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "vcb_gate_blocks": [_P, _L, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _F, _I, _P],
    "vcb_linear_recurrence": [_P, _P, _L, _P, _L, _P, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _P],
    "vcb_gated_delta_scan": [_P, _P, _P, _L, _L, _L, _P, _L, _P, _L, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _F, _F, _I, _P, _I, _P],
    "vcb_moe_sort": [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P],
    "vcb_moe_expert_gemm": [_P, _L, _P, _P, _L, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _F, _F, _F, _I, _P],
    "vcb_moe_combine": [_P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _P],
}


_pdl = True


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch of this library's kernels on or off (see common.cuh)."""
    global _pdl
    _pdl = bool(on)
    if _lib is not None:
        _lib.vcb_set_pdl(1 if _pdl else 0)


def lib():
    """The kernel library; built and loaded on first use."""
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine runs on an sm_100a GPU only and has no CPU path")
        l = _build.load()
        for name, sig in _SIGNATURES.items():
            fn = getattr(l, name, None)
            if fn is None:
                raise KernelError(f"kernel library lacks {name}; rebuild it (delete csrc/_build)")
            fn.argtypes = sig
            fn.restype = _I
        l.vcb_set_pdl.argtypes = [_I]
        l.vcb_set_pdl.restype = None
        l.vcb_set_pdl(1 if _pdl else 0)
        _lib = l
    return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch (a caller may have switched streams, as a
    graph capture does), so through torch's raw query where it has one: torch.cuda.current_stream() builds a
    Stream object each time, a quarter of the host's time in a step that is launched kernel by kernel."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


_launches = 0


def launch_count() -> int:
    """Launches of this library's own kernels so far (library products are not counted)."""
    return _launches


def add_launches(n: int) -> None:
    """Account for kernels that ran inside a replayed CUDA graph."""
    global _launches
    _launches += n


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code == 10001:
        raise KernelError(f"{what}: the kernel refused its arguments")
    if code == 10002:
        raise KernelError(f"{what}: size not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"storage type {dt} is not supported (float32 or bfloat16)")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    _need(t.is_cuda, f"{name} must live on the GPU")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _need(t.dtype == dtype, f"{name} must be {dtype}, is {t.dtype}")
    return t.data_ptr()


# --------------------------------------------------------------------- ops
def embedding(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor, scale: float = 1.0) -> None:
    """residual[t] = float(table[ids[t]]) * scale; ids int32 [n], residual float32 [n, hidden].  An id outside the
    table leaves a row of zeros and code 12 in the status word."""
    n, hidden = residual.shape
    _need(table.dim() == 2 and table.shape[1] == hidden, "embedding table width differs from the residual's")
    _need(ids.numel() == n, "one id per residual row")
    _check(lib().vcb_embedding_scaled(_dev(table, "table"), _dev(ids, "ids", torch.int32),
                                      _dev(residual, "residual", torch.float32), n, hidden, table.shape[0],
                                      status_tensor(table.device).data_ptr(), float(scale), dtype_code(table.dtype),
                                      _stream()), "embedding")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor,
                out: torch.Tensor, eps: float, row_index: Optional[torch.Tensor] = None, mult: float = 1.0) -> None:
    """out = rmsnorm(residual (+ mult * delta)) * gain; the sum is written back to residual unless rows are gathered."""
    hidden = residual.shape[1]
    n_rows = out.shape[0]
    _need(out.shape[1] == hidden and gain.numel() == hidden, "add_rmsnorm: widths differ")
    if delta is not None:
        _need(delta.shape == residual.shape and delta.dtype == out.dtype, "add_rmsnorm: delta shape or type differs")
    if row_index is None:
        _need(n_rows == residual.shape[0], "add_rmsnorm: one output row per residual row")
    else:
        _need(row_index.numel() == n_rows, "add_rmsnorm: one row index per output row")
    _check(lib().vcb_add_rmsnorm_scaled(_dev(residual, "residual", torch.float32),
                                        None if delta is None else _dev(delta, "delta"),
                                        _dev(gain, "gain", torch.float32), _dev(out, "out"),
                                        None if row_index is None else _dev(row_index, "row_index", torch.int32),
                                        n_rows, hidden, float(eps), float(mult), dtype_code(out.dtype), _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i]."""
    n, inter = out.shape
    _need(gate_up.shape == (n, 2 * inter) and gate_up.dtype == out.dtype, "silu_mul: gate_up must be [n, 2*inter]")
    _check(lib().vcb_silu_mul(_dev(gate_up, "gate_up"), _dev(out, "out"), n, inter,
                              dtype_code(out.dtype), _stream()), "silu_mul")


def cast_rows(x: torch.Tensor, delta: Optional[torch.Tensor], mult: float, out: torch.Tensor) -> None:
    """out = x + mult * delta (float; ``delta`` None: x itself) rounded to out's type; x float32 [n, width] contiguous,
    delta contiguous of out's type, out rows may be strided.  x is left as it is."""
    n, width = x.shape
    _need(out.shape == x.shape and out.stride(1) == 1 and out.is_cuda, "cast_rows: out like x, unit inner stride")
    _need(delta is None or (delta.shape == x.shape and delta.dtype == out.dtype), "cast_rows: delta like x, of out's type")
    _check(lib().vcb_cast_rows(_dev(x, "x", torch.float32), None if delta is None else _dev(delta, "delta"), float(mult),
                               out.data_ptr(), n, width, out.stride(0), dtype_code(out.dtype), _stream()), "cast_rows")


def clamped_swish_mul(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, limit: float, alpha: float,
                      up_shift: float = 1.0) -> None:
    """out[t, i] = g * sigmoid(alpha * g) * (u + up_shift) with g = min(gate_up[t, i] + bias[i], limit) and
    u = clamp(gate_up[t, inter + i] + bias[inter + i], -limit, limit); ``bias`` float32 [2 * inter] or None."""
    n, inter = out.shape
    _need(gate_up.shape == (n, 2 * inter) and gate_up.dtype == out.dtype, "clamped_swish_mul: gate_up must be [n, 2*inter]")
    _need(bias is None or bias.numel() == 2 * inter, "clamped_swish_mul: one bias value per gate and up feature")
    _need(limit > 0, "clamped_swish_mul: limit must be positive")
    _check(lib().vcb_clamped_swish_mul(_dev(gate_up, "gate_up"), None if bias is None else _dev(bias, "bias", torch.float32),
                                       _dev(out, "out"), n, inter, float(limit), float(alpha), float(up_shift),
                                       dtype_code(out.dtype), _stream()), "clamped_swish_mul")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[t, c] += bias[c] in place."""
    rows, cols = x.shape
    _need(bias.numel() == cols, "add_bias: one bias value per column")
    _check(lib().vcb_add_bias(_dev(x, "x"), _dev(bias, "bias", torch.float32), rows, cols,
                              dtype_code(x.dtype), _stream()), "add_bias")


def rope_cache_write(qkv, bias, positions, req_of_token, block_table, denom, q_out, cache, *,
                     num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, pairing: int,
                     page_size: int, write_kv: bool) -> None:
    """Bias, rotation and cache write in one pass over the q/k/v product (see elementwise.cu)."""
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv.shape == (n, width), f"qkv must be [n, {width}], is {tuple(qkv.shape)}")
    _need(q_out.shape == (n, num_heads * head_dim) and q_out.dtype == qkv.dtype, "q_out shape or type")
    _need(head_dim % 2 == 0 and rotary_dim % 2 == 0 and 0 <= rotary_dim <= head_dim, "rotary_dim must be even and <= head_dim")
    _need(cache.dtype == qkv.dtype, "cache and activations must share a storage type")
    if rotary_dim:
        _need(denom is not None and denom.numel() == rotary_dim // 2, "denom must hold rotary_dim/2 values")
    if bias is not None:
        _need(bias.numel() == width, "bias width")
    _check(lib().vcb_rope_cache_write(
        _dev(qkv, "qkv"), None if bias is None else _dev(bias, "bias", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(req_of_token, "req_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        None if denom is None else _dev(denom, "denom", torch.float32), _dev(q_out, "q_out"),
        _dev(cache, "cache"), n, num_heads, num_kv_heads, head_dim, rotary_dim, pairing, page_size,
        1 if write_kv else 0, cache.shape[0], status_tensor(qkv.device).data_ptr(), dtype_code(qkv.dtype), _stream()),
        "rope_cache_write")


SIMT_MAX_HEAD_DIM = 1024


def attention_simt(q, cache, out, positions, req_of_token, block_table, *, num_heads: int,
                   num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, planes: int = 2) -> None:
    """Plain paged attention.  ``planes`` 2: a page holds keys, then values; 1: one plane of rows that serve
    as key and as value (cached latent rows)."""
    n = q.shape[0]
    _need(head_dim <= SIMT_MAX_HEAD_DIM, f"head_dim {head_dim} exceeds {SIMT_MAX_HEAD_DIM}, the largest this attention kernel takes")
    _need(planes in (1, 2), "planes must be 1 or 2")
    _need(q.shape == (n, num_heads * head_dim) and out.shape == q.shape and out.dtype == q.dtype, "q/out shape")
    _need(num_heads % num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads")
    _need(cache.dtype == q.dtype, "cache and q must share a storage type")
    _check(lib().vcb_attention_simt_planes(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(positions, "positions", torch.int32),
        _dev(req_of_token, "req_of_token", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], n, num_heads, num_kv_heads, head_dim, page_size, window, float(scale),
        cache.shape[0], status_tensor(q.device).data_ptr(), planes, dtype_code(q.dtype), _stream()), "attention_simt")


MMA_HEAD_DIMS = (64, 128)
DECODE_KEY_TILE = 64          # keys per tile of the decode kernel
DECODE_MAX_SPLITS = 32


def _epilogue_args(sink, head_gate, n_tokens: int, num_heads: int, what: str) -> None:
    _need(sink is None or (sink.dtype == torch.float32 and sink.numel() == num_heads and sink.is_contiguous()), f"{what}: sink float32 [heads]")
    _need(head_gate is None or (head_gate.dtype == torch.bfloat16 and head_gate.shape == (n_tokens, num_heads) and head_gate.stride(1) == 1),
          f"{what}: head_gate bfloat16 [tokens, heads] with unit inner stride")


def _epilogue_ptrs(sink, head_gate):
    return (None if sink is None else sink.data_ptr(), None if head_gate is None else head_gate.data_ptr(),
            0 if head_gate is None else head_gate.stride(0))


def attention_decode_mma(q, cache, out, q_start, ctx_lens, block_table, req_list, n_list: int, nsplit: int,
                         part_o, part_ml, counters, *, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         window: int, scale: float, split_tiles=None, planes: int = 2, kv_share: int = 1,
                         cap: float = 0.0, bias_t: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
                         head_gate: Optional[torch.Tensor] = None, precise_weights: bool = False) -> None:
    """Split-KV tensor-core attention for requests that bring one token each (bfloat16).  The grid has
    ``nsplit`` columns; without ``split_tiles`` every request's keys are cut into that many equal parts,
    with it (int32 [1] on the device: tiles of DECODE_KEY_TILE keys per split) a request takes as many
    columns as its context needs, so that requests of different lengths keep all CTAs equally busy.
    ``kv_share`` > 1: ``num_kv_heads`` counts groups of query heads of which ``kv_share`` consecutive ones read the
    same head of the cache (decode_head_groups): each group gets CTAs of its own."""
    _need(q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_decode_mma is a bfloat16 kernel")
    _need(head_dim in MMA_HEAD_DIMS and page_size % 8 == 0,
          f"attention_decode_mma takes head sizes {MMA_HEAD_DIMS} and pages of a multiple of 8 slots, got {head_dim} and {page_size}")
    if nsplit > 1:
        need = n_list * num_heads * nsplit
        _need(part_o is not None and part_o.numel() >= need * head_dim and part_ml.numel() >= need * 2
              and counters is not None and counters.numel() >= n_list * num_kv_heads,
              "attention_decode_mma: scratch for the split merge is too small")
    _need(planes in (1, 2), "planes must be 1 or 2")
    _need(kv_share >= 1 and num_kv_heads % kv_share == 0, "attention_decode_mma: kv_share divides num_kv_heads")
    if cap > 0 or bias_t is not None or sink is not None or head_gate is not None or precise_weights:
        # ``precise_weights``: the softmax weights enter the P V product as two bfloat16 terms (16 bits of mantissa)
        # shaped scores: cap * tanh(scale * q.k / cap) + bias_t[head, min(distance, last)]; the epilogue: a sink logit per
        # head in the denominator, the head's output times sigmoid(head_gate[token, head]) (see attention_mma.cu)
        _need(bias_t is None or (bias_t.dim() == 2 and bias_t.shape[0] == num_heads), "attention_decode_mma: bias_t [heads, distances]")
        _epilogue_args(sink, head_gate, q.shape[0], num_heads, "attention_decode_mma")
        _check(lib().vcb_attention_decode_mma_shaped_planes(
            _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(q_start, "q_start", torch.int32),
            _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32),
            block_table.shape[1], None if req_list is None else _dev(req_list, "req_list", torch.int32),
            n_list, nsplit, None if part_o is None else _dev(part_o, "part_o", torch.float32),
            None if part_ml is None else _dev(part_ml, "part_ml", torch.float32),
            None if counters is None else _dev(counters, "counters", torch.int32),
            None if split_tiles is None else _dev(split_tiles, "split_tiles", torch.int32),
            num_heads, num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0],
            status_tensor(q.device).data_ptr(), kv_share, float(cap),
            None if bias_t is None else _dev(bias_t, "bias_t", torch.float32), 0 if bias_t is None else bias_t.shape[1],
            *_epilogue_ptrs(sink, head_gate), 1 if precise_weights else 0, planes, _stream()), "attention_decode_mma")
        return
    _check(lib().vcb_attention_decode_mma_planes(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(q_start, "q_start", torch.int32),
        _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], None if req_list is None else _dev(req_list, "req_list", torch.int32),
        n_list, nsplit, None if part_o is None else _dev(part_o, "part_o", torch.float32),
        None if part_ml is None else _dev(part_ml, "part_ml", torch.float32),
        None if counters is None else _dev(counters, "counters", torch.int32),
        None if split_tiles is None else _dev(split_tiles, "split_tiles", torch.int32),
        num_heads, num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0],
        status_tensor(q.device).data_ptr(), planes, kv_share, _stream()), "attention_decode_mma")


def decode_head_groups(num_heads: int, num_kv_heads: int) -> int:
    """Into how many equal groups of at most 16 the query heads of one kv head are cut for the decode kernel
    (its fragment has 16 rows; a larger group would walk the keys once per 16 heads in one CTA): the smallest
    divisor of the group's size that leaves at most 16 heads, or 1 if there is none below the size itself."""
    g = num_heads // num_kv_heads
    for s in range(1, g):
        if g % s == 0 and g // s <= 16:
            return s
    return 1


TC_ATTENTION_HEAD_DIMS = (64, 128)      # head sizes of the tcgen05 prefill attention kernel
TC_ATTENTION_TILE_ROWS = 128     # packed rows per tile of its work list


def attention_prefill_tc(q, cache, out, q_start, ctx_lens, block_table, tile_req, tile_row0, *,
                         num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                         scale: float, planes: int = 2, cap: float = 0.0, bias_t: Optional[torch.Tensor] = None,
                         sink: Optional[torch.Tensor] = None, head_gate: Optional[torch.Tensor] = None,
                         precise_weights: bool = False) -> None:
    """Attention for portions of any length on tcgen05 tensor cores (scores and output tiles in tensor
    memory); head sizes 64 and 128, bfloat16, pages of a multiple of 8 slots, tiles of 128 packed rows."""
    _need(q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill_tc is a bfloat16 kernel")
    _need(head_dim in TC_ATTENTION_HEAD_DIMS and page_size % 8 == 0,
          f"attention_prefill_tc takes head sizes {TC_ATTENTION_HEAD_DIMS} and pages of a multiple of 8 slots")
    n_tiles = tile_req.numel()
    _need(tile_row0.numel() == n_tiles, "one first row per tile")
    _need(planes in (1, 2), "planes must be 1 or 2")
    if cap > 0 or bias_t is not None or sink is not None or head_gate is not None or precise_weights:
        _need(bias_t is None or (bias_t.dim() == 2 and bias_t.shape[0] == num_heads), "attention_prefill_tc: bias_t [heads, distances]")
        _epilogue_args(sink, head_gate, q.shape[0], num_heads, "attention_prefill_tc")
        _check(lib().vcb_attention_prefill_tc_shaped_planes(
            _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(q_start, "q_start", torch.int32),
            _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32),
            block_table.shape[1], _dev(tile_req, "tile_req", torch.int32), _dev(tile_row0, "tile_row0", torch.int32),
            n_tiles, num_heads, num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0],
            status_tensor(q.device).data_ptr(), float(cap), None if bias_t is None else _dev(bias_t, "bias_t", torch.float32),
            0 if bias_t is None else bias_t.shape[1], *_epilogue_ptrs(sink, head_gate), 1 if precise_weights else 0, planes, _stream()), "attention_prefill_tc")
        return
    _check(lib().vcb_attention_prefill_tc_planes(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(q_start, "q_start", torch.int32),
        _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], _dev(tile_req, "tile_req", torch.int32), _dev(tile_row0, "tile_row0", torch.int32),
        n_tiles, num_heads, num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0],
        status_tensor(q.device).data_ptr(), planes, _stream()), "attention_prefill_tc")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true 32-bit arithmetic; rows may be strided."""
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and out.shape == (m, n), "gemm_f32: shapes do not agree")
    for t, name in ((a, "a"), (w, "w"), (out, "out")):
        _need(t.is_cuda and t.dtype == torch.float32 and t.stride(1) == 1, f"gemm_f32: {name} must be float32 with unit inner stride")
    _check(lib().vcb_gemm_f32(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                              a.stride(0), w.stride(0), out.stride(0), _stream()), "gemm_f32")


_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the device the engine runs on, asked once (148 on a B200): the
    most CTAs of a persistent kernel, and what the parts size their work lists by."""
    global _sm_count
    if _sm_count is None:
        _need(torch.cuda.is_available(), "no CUDA device")
        _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return _sm_count


_status: Optional[torch.Tensor] = None
STATUS_MEANING = {1: "the TMA producer waited too long for a free stage", 2: "the MMA issuer waited too long for a loaded stage",
                  3: "the epilogue waited too long for the accumulator", 4: "the MMA issuer waited too long for a free accumulator",
                  5: "decode attention waited too long for a cache tile", 6: "prefill attention waited too long for a cache tile",
                  8: "a product's merge waited too long for the tile's other segments",
                  9: "tcgen05 prefill attention waited too long on one of its barriers",
                  10: "tcgen05 prefill attention found its shared memory not aligned to 1024 bytes",
                  12: "a token id outside the vocabulary reached the embedding on the device (a sampled id of the step "
                      "before, which the host had not yet seen); its row was left zero",
                  11: "a block table named a page that the cache does not have (a released or missing entry); "
                      "nothing was written through it and attention read page 0 in its place"}


def status_tensor(device) -> torch.Tensor:
    """The device word in which kernels with bounded waits record a wait that ran out."""
    global _status
    if _status is None or _status.device != torch.device(device):
        _status = torch.zeros(1, dtype=torch.int32, device=device)
    return _status


def check_status() -> None:
    """Raise if a kernel noted something in the status word since the last check: a bounded wait that ran
    out, a page or a token id that does not exist (synchronises)."""
    if _status is None:
        return
    code = int(_status.item())
    if code:
        _status.zero_()
        raise KernelError(f"a kernel left status {code}: {STATUS_MEANING.get(code, code)}")


def tcgen05_plan(tokens: int, features: int, k: int):
    """(swapped, bn) for out[tokens, features] = x[tokens, k] @ w[features, k]^T: few tokens put the
    weights on the 128-row side of the tensor-core tile."""
    if tokens <= 128:
        return True, (16 if tokens <= 16 else 32 if tokens <= 32 else 64 if tokens <= 64 else 128)
    return False, 256


GEMM_MAX_TICKETS = 16384


def tile_weights(w: torch.Tensor, gated: int = 0) -> torch.Tensor:
    """The pre-tiled image of a weight matrix for decode products (see gemm_tcgen05.cu): made once,
    kept on the tensor object itself (so it lives and dies with the matrix), and used by ``linear``
    whenever the weights sit on the 128-row side.  The matrix must not change afterwards.
    ``gated`` > 0: w is the [2 * gated, k] gate-and-up matrix of a gated feed-forward and the image
    pairs gate and up rows in every tile, for ``linear_gated``."""
    attr = "_vcb_tiled_gated" if gated else "_vcb_tiled"
    t = getattr(w, attr, None)
    if t is None:
        _need(w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1, "tile_weights: a bfloat16 matrix")
        rows, k = w.shape
        _need(gated == 0 or rows == 2 * gated, "tile_weights: a gated matrix has 2 * gated rows")
        tiles = -(-gated // 64) if gated else -(-rows // 128)
        t = torch.empty(tiles * -(-k // 64) * 16384, dtype=torch.uint8, device=w.device)
        _check(lib().vcb_tile_weights(w.data_ptr(), rows, k, w.stride(0), gated, t.data_ptr(), _stream()), "tile_weights")
        setattr(w, attr, t)
    return t


def drop_tiled_weights(w: torch.Tensor) -> None:
    for attr in ("_vcb_tiled", "_vcb_tiled_gated"):
        if getattr(w, attr, None) is not None:
            setattr(w, attr, None)


def tiled_weights_of(w: torch.Tensor, gated: bool = False) -> Optional[torch.Tensor]:
    return getattr(w, "_vcb_tiled_gated" if gated else "_vcb_tiled", None)


class RowScale:
    """Says that the rows of a product's input still lack the factor of an RMSNorm:
    row t is to be multiplied by rsqrt(sum(sumsq[:parts, t]) / width + eps).  ``sumsq`` holds
    partial sums of squares of the un-normalised row, [parts, tokens] float32."""
    __slots__ = ("sumsq", "parts", "width", "eps")

    def __init__(self, sumsq: torch.Tensor, parts: int, width: int, eps: float):
        self.sumsq, self.parts, self.width, self.eps = sumsq, parts, width, float(eps)


class ResidualNorm:
    """Asks a product to end a residual branch itself: residual (float32 [tokens, features]) += result;
    out = bfloat16(residual * gain), the un-normalised input of the norm that follows; sumsq
    ([sumsq_parts(features), tokens] float32) = partial sums of squares of the new residual rows.
    ``scale()`` is the RowScale the next product needs."""
    __slots__ = ("residual", "gain", "sumsq", "eps")

    def __init__(self, residual: torch.Tensor, gain: torch.Tensor, sumsq: torch.Tensor, eps: float):
        self.residual, self.gain, self.sumsq, self.eps = residual, gain, sumsq, float(eps)

    def scale(self) -> RowScale:
        return RowScale(self.sumsq, sumsq_parts(self.residual.shape[1]), self.residual.shape[1], self.eps)


def sumsq_parts(features: int) -> int:
    """Partial sums a ResidualNorm product leaves per token: one per epilogue warp of every 128-row tile."""
    return 4 * (-(-features // 128))


def gemm_bf16_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan=None, max_ctas: Optional[int] = None,
                      use_tiled: bool = True, x_scale: Optional[RowScale] = None,
                      fuse: Optional[ResidualNorm] = None, gated: bool = False) -> None:
    """out = x @ w^T on tcgen05 tensor cores fed by TMA (see gemm_tcgen05.cu); out bfloat16 or float32.
    When the weights are the 128-row operand and tile_weights(w) has been made, the image is used
    (``use_tiled`` False forces the tensor-map path).  ``x_scale`` and ``fuse`` (up to 128 tokens):
    see RowScale and ResidualNorm.  ``gated``: w is a gate-and-up matrix [2 * inter, k] with a gated
    image (tile_weights(w, inter)) and out [tokens, inter] = silu(x gate^T) * (x up^T)."""
    m, k = x.shape
    n = w.shape[0]
    _need(w.shape[1] == k and out.shape == (m, n // 2 if gated else n), "gemm_bf16_tcgen05: shapes do not agree")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_bf16_tcgen05: operands must be bfloat16")
    _need(out.dtype in (torch.bfloat16, torch.float32) and out.stride(1) == 1 and x.stride(1) == 1 and w.stride(1) == 1,
          "gemm_bf16_tcgen05: unit inner strides, out bfloat16 or float32")
    _need(k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0,
          "gemm_bf16_tcgen05: TMA needs K and the row strides to be multiples of 8 and 16-byte aligned bases")
    swapped, bn = plan or tcgen05_plan(m, n, k)
    sc = (None, 0, 0, 1, 0.0)
    if x_scale is not None:
        _need(swapped and m <= bn <= 128, "gemm_bf16_tcgen05: a row scale needs the few-token form")
        _need(x_scale.sumsq.dtype == torch.float32 and x_scale.sumsq.dim() == 2 and x_scale.sumsq.stride(1) == 1
              and x_scale.sumsq.shape[0] >= x_scale.parts and x_scale.sumsq.shape[1] >= m,
              "gemm_bf16_tcgen05: sums of squares must be float32 [parts, tokens]")
        sc = (x_scale.sumsq.data_ptr(), x_scale.parts, x_scale.sumsq.stride(0), x_scale.width, x_scale.eps)
    fu = (None, 0, None, None, 0)
    if fuse is not None:
        _need(swapped and m <= bn <= 128 and out.dtype == torch.bfloat16,
              "gemm_bf16_tcgen05: a fused residual needs the few-token form and a bfloat16 result")
        r, g, ss = fuse.residual, fuse.gain, fuse.sumsq
        _need(r.dtype == torch.float32 and r.shape == (m, n) and r.stride(1) == 1 and g.dtype == torch.float32
              and g.shape == (n,) and g.is_contiguous(), "gemm_bf16_tcgen05: residual float32 [tokens, features], gain float32 [features]")
        _need(ss.dtype == torch.float32 and ss.dim() == 2 and ss.stride(1) == 1 and ss.shape[0] >= sumsq_parts(n)
              and ss.shape[1] >= m, "gemm_bf16_tcgen05: sums of squares must be float32 [sumsq_parts(features), tokens]")
        fu = (r.data_ptr(), r.stride(0), g.data_ptr(), ss.data_ptr(), ss.stride(0))
    p, q = (w, x) if swapped else (x, w)
    tiled = tiled_weights_of(w, gated) if (swapped and use_tiled) else None
    if gated:
        _need(swapped and m <= bn <= 128 and tiled is not None and out.dtype == torch.bfloat16 and fuse is None,
              "gemm_bf16_tcgen05: the gated form needs few tokens, a gated tile image and a bfloat16 result")
    sms = sm_count()
    if max_ctas is None:
        # What the measurement at load chose for this shape (choose_ctas), else: tiles of 32 and 64 columns
        # run two CTAs of the product on every SM (its ring is then four or five stages deep each).  A stage
        # carries the tokens' operand beside the weights', half as much again at 64 tokens, and one CTA's ring
        # does not hold enough bytes in flight for the memory's rate (measured at 64 tokens, 7B sizes:
        # gate-and-up 49.9 -> 44.6 us, qkv 14.8 -> 12.8; at 128 it is slower).
        max_ctas = _cta_choice.get((n, k, bn, bool(gated), fuse is not None), 2 * sms if bn in (32, 64) else sms)
    partial = scratch("gemm_partial", sms * 2 * 256 * 128, out.device)
    tickets = zeroed_ints("gemm_tickets", GEMM_MAX_TICKETS, out.device)
    _check(lib().vcb_gemm_bf16_tcgen05_fused(p.data_ptr(), p.shape[0], p.stride(0),
                                             None if tiled is None else tiled.data_ptr(),
                                             q.data_ptr(), q.shape[0], q.stride(0), k,
                                             out.data_ptr(), out.stride(0), 1 if out.dtype == torch.float32 else 0,
                                             1 if swapped else 0, bn, min(max_ctas, 2 * sms), partial.data_ptr(),
                                             tickets.data_ptr(), GEMM_MAX_TICKETS, status_tensor(out.device).data_ptr(),
                                             *sc, *fu, n // 2 if gated else 0, _stream()), "gemm_bf16_tcgen05")


TCGEN05_MAX_TOKENS = 128      # up to here the engine's own tcgen05 product may run; above, the library's
_tcgen05_linear = True
# (features, k, token bucket) -> True if the tcgen05 kernel was measured faster than cuBLAS here
_linear_choice = {}


def set_tcgen05_linear(on: bool) -> None:
    """Allow this library's tcgen05 product for bfloat16 products with few tokens (default), or cuBLAS for all."""
    global _tcgen05_linear
    _tcgen05_linear = bool(on)


_linear_tuning = True


def set_linear_tuning(on: bool) -> None:
    """With tuning off nothing is measured at load, so every product with few tokens runs this
    library's tcgen05 kernel (tests use it to pin the path)."""
    global _linear_tuning
    _linear_tuning = bool(on)


def token_bucket(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128


def _tcgen05_ok(x, w, out) -> bool:
    m, k = x.shape
    return (m <= TCGEN05_MAX_TOKENS and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.stride(1) == 1 and x.stride(1) == 1
            and w.stride(1) == 1 and -(-w.shape[0] // 128) <= GEMM_MAX_TICKETS)


def _library_mm(x, w, out) -> None:
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        _need(out.dtype == torch.float32, "linear: out must be bfloat16 or float32")
        try:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        except (TypeError, RuntimeError):
            out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))


TOKEN_BUCKETS = ((16, 8), (32, 32), (64, 64), (128, 128))      # (bucket, token count it is measured at)


def time_in_graph(fn, reps: int = 8) -> float:
    """Microseconds per call of ``fn(i)``: ``reps`` calls are captured into a CUDA graph and the graph
    is replayed, so that the host's launch cost stays out of the figure."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(2):
            fn(i)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                fn(i)
        graph.replay()
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        graph.replay()
        e1.record()
        side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    return e0.elapsed_time(e1) * 1e3 / (2 * reps)


def measure_linear(weights, out_dtype=torch.bfloat16, gated: int = 0):
    """{bucket: (microseconds of this library's tcgen05 product, of the library's)} for one shape of
    weight matrix.  ``weights``: matrices of the same shape (the same projection of several layers),
    used in rotation so that the L2 cache cannot serve them; their tiled images must exist.
    ``gated`` > 0: the matrices are gate-and-up matrices with gated images; this library's side is
    ``linear_gated``, the library's side the product followed by the activation kernel.
    Buckets the tcgen05 kernel cannot take are left out."""
    n, k = weights[0].shape
    dev_ = weights[0].device
    out_times = {}
    for bucket, m in TOKEN_BUCKETS:
        x = torch.randn(m, k, device=dev_).to(torch.bfloat16)
        out = torch.empty(m, n, dtype=out_dtype, device=dev_)
        if not _tcgen05_ok(x, weights[0], out):
            continue
        if gated:
            act = torch.empty(m, gated, dtype=out_dtype, device=dev_)

            def theirs(i):
                _library_mm(x, weights[i % len(weights)], out)
                silu_mul(out, act)
            out_times[bucket] = (time_in_graph(lambda i: gemm_bf16_tcgen05(x, weights[i % len(weights)], act, gated=True)),
                                 time_in_graph(theirs))
        else:
            out_times[bucket] = (time_in_graph(lambda i: gemm_bf16_tcgen05(x, weights[i % len(weights)], out)),
                                 time_in_graph(lambda i: _library_mm(x, weights[i % len(weights)], out)))
    check_status()
    return out_times


def measure_layer(products, hidden: int, fusable_norms: int, dtype=torch.bfloat16) -> dict:
    """{bucket: (microseconds of a layer's products as this library runs them, as the library would)}.
    ``products``: for every product of a layer, in the order they run, (matrices of that product
    across layers, gated, reads a norm's output, ends a residual branch) with tiled images made.  This
    library's side is its tcgen05 product for each, linked as the blocks link them: the rows' factor
    applied by a product that reads a norm's output (RowScale), the addition into the residual stream,
    the next norm's gain and the sums of squares in the epilogue of one that ends a branch
    (ResidualNorm), the activation inside the gated ones.  The library's side is a product each, the
    activation kernel after a gated one and ``fusable_norms`` norm kernels, which the other side does
    not need."""
    dev_ = products[0][0][0].device
    times = {}
    for bucket, m in TOKEN_BUCKETS:
        xs, outs, acts = {}, [], []
        ok = True
        for mats, gated, _, _ in products:
            n, k = mats[0].shape
            if k not in xs:
                xs[k] = torch.randn(m, k, device=dev_).to(dtype)
            outs.append(torch.empty(m, n, dtype=dtype, device=dev_))
            acts.append(torch.empty(m, gated, dtype=dtype, device=dev_) if gated else None)
            ok = ok and _tcgen05_ok(xs[k], mats[0], outs[-1])
        if not ok:
            continue
        res = torch.zeros(m, hidden, device=dev_)
        delta = torch.zeros(m, hidden, dtype=dtype, device=dev_)
        normed = torch.empty(m, hidden, dtype=dtype, device=dev_)
        gain = torch.ones(hidden, device=dev_)
        sumsq = torch.ones(sumsq_parts(hidden), m, device=dev_)
        scale = RowScale(sumsq, sumsq_parts(hidden), hidden, 1e-6)
        ends = ResidualNorm(res, gain, torch.empty(sumsq_parts(hidden), m, device=dev_), 1e-6)

        def ours(i):
            for j, (mats, gated, reads_norm, ends_branch) in enumerate(products):
                w = mats[i % len(mats)]
                gemm_bf16_tcgen05(xs[w.shape[1]], w, acts[j] if gated else outs[j],
                                  x_scale=scale if reads_norm and w.shape[1] == hidden else None,
                                  fuse=ends if ends_branch and w.shape[0] == hidden and not gated else None, gated=bool(gated))

        def theirs(i):
            for j, (mats, gated, _, _) in enumerate(products):
                w = mats[i % len(mats)]
                _library_mm(xs[w.shape[1]], w, outs[j])
                if gated:
                    silu_mul(outs[j], acts[j])
            for _ in range(fusable_norms):
                add_rmsnorm(res, delta, gain, normed, 1e-6)

        times[bucket] = (time_in_graph(ours), time_in_graph(theirs))
    check_status()
    return times


# (features, k, tile columns, gated, ends a residual branch) -> persistent CTAs of the tcgen05 product, where a
# measurement chose them
_cta_choice = {}


def cta_candidates(features: int, k: int, gated: int = 0):
    """Grid sizes worth measuring for a few-token product: one CTA per SM (the next kernel's CTAs then sit
    beside this one's and prefetch), two per SM, and in between the counts that cut every 128-row tile into
    the same number of whole runs of k slabs (no CTA then holds pieces of two tiles, and a count equal to the
    number of tiles needs no merge at all)."""
    sms = sm_count()
    tiles = -(-gated // 64) if gated else -(-features // 128)
    slabs = -(-k // 64)
    out = {sms, 2 * sms}
    for per_tile in range(1, slabs // 4 + 1):
        if slabs % per_tile == 0 and sms * 3 // 4 <= tiles * per_tile <= 2 * sms:
            out.add(tiles * per_tile)
    return sorted(out)


def choose_ctas(weights, bucket: int, tokens: int, gated: int = 0, out_dtype=torch.bfloat16, residual: bool = False) -> int:
    """Measure the tcgen05 product on ``weights`` (matrices of one shape, used in rotation) at every candidate
    grid size, record the fastest for this shape and bucket, and return it.  ``residual``: the product as it
    ends a residual branch (ResidualNorm), whose merge does more than the plain one's."""
    n, k = weights[0].shape
    dev_ = weights[0].device
    x = torch.randn(tokens, k, device=dev_).to(torch.bfloat16)
    out = torch.empty(tokens, gated or n, dtype=out_dtype, device=dev_)
    fuse = ResidualNorm(torch.zeros(tokens, n, device=dev_), torch.ones(n, device=dev_),
                        torch.empty(sumsq_parts(n), tokens, device=dev_), 1e-6) if residual else None
    best, best_t = None, None
    for ctas in cta_candidates(n, k, gated):
        t = time_in_graph(lambda i: gemm_bf16_tcgen05(x, weights[i % len(weights)], out, max_ctas=ctas, gated=bool(gated), fuse=fuse))
        if best_t is None or t < best_t * 0.98:           # a larger grid must win by more than the noise
            best, best_t = ctas, t
    _cta_choice[(n, k, tcgen05_plan(tokens, n, k)[1], bool(gated), residual)] = best
    return best


def choose_linear(features: int, k: int, bucket: int, out_dtype, tcgen05: bool) -> None:
    """Record which product ``linear`` runs for this shape and bucket of token counts."""
    _linear_choice[(features, k, bucket, out_dtype)] = bool(tcgen05)


def forget_choices(features: int, k: int) -> None:
    """Drop what was measured for products of this shape (kernel per bucket, grid per tile width): the defaults
    apply again."""
    for key in [key for key in _linear_choice if key[0] == features and key[1] == k]:
        del _linear_choice[key]
    for key in [key for key in _cta_choice if key[0] == features and key[1] == k]:
        del _cta_choice[key]


def linear_tuning() -> bool:
    return _linear_tuning


_norm_fusion = True


def set_norm_fusion(on: bool) -> None:
    """Allow products to take over the norms around them (default), or run every norm as a kernel."""
    global _norm_fusion
    _norm_fusion = bool(on)


def linear_fuses_norm(tokens: int, w: torch.Tensor, out_dtype=torch.bfloat16) -> bool:
    """True if ``linear`` will run this library's tcgen05 product for ``tokens`` rows against ``w``
    (taken contiguous and 16-byte aligned, as workspace buffers and loaded weights are): only then can
    it apply a RowScale or a ResidualNorm."""
    return (_norm_fusion and _tcgen05_linear and w.dtype == torch.bfloat16 and 0 < tokens <= TCGEN05_MAX_TOKENS
            and w.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and -(-w.shape[0] // 128) <= GEMM_MAX_TICKETS
            and _linear_choice.get((w.shape[0], w.shape[1], token_bucket(tokens), out_dtype), True))


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_scale: Optional[RowScale] = None,
           fuse: Optional[ResidualNorm] = None) -> None:
    """out = x @ w^T.  float32: the engine's own FMA kernel.  bfloat16 with up to TCGEN05_MAX_TOKENS
    rows (decode steps, short portions): the engine's tcgen05 + TMA kernel with the weights on the
    128-row side of the tile, where the measurement at load found it faster than the library (and always
    when nothing was measured); otherwise the library product (cuBLAS through torch.mm, float
    accumulation).  out is bfloat16 or float32.  ``x_scale`` / ``fuse`` may be given only where
    ``linear_fuses_norm`` said yes."""
    if x.dtype == torch.float32:
        _need(x_scale is None and fuse is None, "linear: the float32 product fuses no norm")
        gemm_f32(x, w, out)
        return
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must both be bfloat16")
    if _tcgen05_linear and _tcgen05_ok(x, w, out) and \
            _linear_choice.get((w.shape[0], w.shape[1], token_bucket(x.shape[0]), out.dtype), True):
        gemm_bf16_tcgen05(x, w, out, x_scale=x_scale, fuse=fuse)
        return
    _need(x_scale is None and fuse is None, "linear: the library product fuses no norm; ask linear_fuses_norm first")
    _library_mm(x, w, out)


def linear_gated_fuses(tokens: int, w: torch.Tensor) -> bool:
    """True if ``linear_gated`` will run as one kernel (this library's tcgen05 product on a gated tile image)."""
    return tiled_weights_of(w, gated=True) is not None and _tcgen05_linear and 0 < tokens <= TCGEN05_MAX_TOKENS \
        and _linear_choice.get((w.shape[0], w.shape[1], token_bucket(tokens), torch.bfloat16), True)


def linear_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_scale: Optional[RowScale] = None) -> None:
    """out [tokens, inter] = silu(x gate^T) * (x up^T) for w = [gate; up] ([2 * inter, k]) in one kernel;
    only where ``linear_gated_fuses`` said yes."""
    _need(linear_gated_fuses(x.shape[0], w), "linear_gated: ask linear_gated_fuses first")
    gemm_bf16_tcgen05(x, w, out, x_scale=x_scale, gated=True)


# ------------------------------------------------- residual stream: shift, gates, norms on results
def embedding_sinusoid(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                       residual: torch.Tensor, scale: float) -> None:
    """residual[t, i] = float(table[ids[t], i]) * scale + (sin if i even else cos)(positions[t] * inv_freq[i // 2])."""
    n, hidden = residual.shape
    _need(table.dim() == 2 and table.shape[1] == hidden, "embedding table width differs from the residual's")
    _need(ids.numel() == n and positions.numel() == n, "one id and one position per residual row")
    _need(inv_freq.numel() >= (hidden + 1) // 2, "one frequency per pair of coordinates")
    _check(lib().vcb_embedding_sinusoid(_dev(table, "table"), _dev(ids, "ids", torch.int32),
                                        _dev(positions, "positions", torch.int32), _dev(inv_freq, "inv_freq", torch.float32),
                                        _dev(residual, "residual", torch.float32), n, hidden, table.shape[0], float(scale),
                                        status_tensor(table.device).data_ptr(), dtype_code(table.dtype), _stream()),
           "embedding_sinusoid")


def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, shifted: torch.Tensor,
                plain: Optional[torch.Tensor], q_start, req_of_token, positions, state_slots) -> None:
    """shifted[t] = x[t] + (x[t-1] - x[t]) * mu in the activations' type; x float32 [n, hidden].  The row before
    a request's first row of the step is zero at position 0, else the request's slot of ``state`` (float32
    [slots, hidden]), which then receives the request's last row of this step.  ``plain`` (optional): x in the
    activations' type."""
    n, hidden = x.shape
    _need(shifted.shape == x.shape and (plain is None or (plain.shape == x.shape and plain.dtype == shifted.dtype)),
          "token_shift: outputs must have the input's shape")
    _need(mu.numel() == hidden and state.dim() == 2 and state.shape[1] == hidden, "token_shift: widths differ")
    _check(lib().vcb_token_shift(_dev(x, "x", torch.float32), _dev(mu, "mu", torch.float32), _dev(state, "state", torch.float32),
                                 _dev(shifted, "shifted"), None if plain is None else _dev(plain, "plain"),
                                 _dev(q_start, "q_start", torch.int32), _dev(req_of_token, "req_of_token", torch.int32),
                                 _dev(positions, "positions", torch.int32), _dev(state_slots, "state_slots", torch.int32),
                                 n, hidden, dtype_code(shifted.dtype), _stream()), "token_shift")


def gated_norm_residual(y: torch.Tensor, gate: Optional[torch.Tensor], gate_bias: Optional[torch.Tensor],
                        gain: torch.Tensor, x: torch.Tensor, plain: Optional[torch.Tensor], mult: float, eps: float) -> None:
    """z = y * sigmoid(gate + gate_bias) (no gate: z = y);  x += mult * z / sqrt(mean(z^2) + eps) * gain, in float32
    in place; ``gain``: one number or a vector.  ``plain`` (optional): the new x in the activations' type."""
    n, hidden = x.shape
    _need(y.shape == x.shape and (gate is None or (gate.shape == x.shape and gate.dtype == y.dtype)), "gated_norm_residual: shapes")
    _need(gate_bias is None or gate_bias.numel() == hidden, "gated_norm_residual: one bias value per column")
    _need(gain.numel() in (1, hidden), "gated_norm_residual: gain is one number or one per column")
    _need(plain is None or (plain.shape == x.shape and plain.dtype == y.dtype), "gated_norm_residual: plain output")
    _check(lib().vcb_gated_norm_residual(_dev(y, "y"), None if gate is None else _dev(gate, "gate"),
                                         None if gate_bias is None else _dev(gate_bias, "gate_bias", torch.float32),
                                         _dev(gain, "gain", torch.float32), 0 if gain.numel() == 1 else 1,
                                         _dev(x, "x", torch.float32), None if plain is None else _dev(plain, "plain"),
                                         n, hidden, float(mult), float(eps), dtype_code(y.dtype), _stream()),
           "gated_norm_residual")


def norm_residual_norm(y: torch.Tensor, gain: torch.Tensor, x: torch.Tensor, eps: float,
                       next_gain: Optional[torch.Tensor] = None, next_out: Optional[torch.Tensor] = None,
                       next_eps: float = 0.0) -> None:
    """x += y / sqrt(mean(y^2) + eps) * gain in float32 in place (``gain``: whatever multiplies the normed result per
    coordinate); with ``next_out``: next_out = x / sqrt(mean(x^2) + next_eps) * next_gain in the activations' type, the
    input of the sublayer that follows."""
    n, hidden = x.shape
    _need(y.shape == x.shape and gain.numel() == hidden, "norm_residual_norm: shapes")
    if next_out is not None:
        _need(next_gain is not None and next_gain.numel() == hidden and next_out.shape == x.shape and next_out.dtype == y.dtype,
              "norm_residual_norm: the next norm's gain and output")
    _check(lib().vcb_norm_residual_norm(_dev(y, "y"), _dev(gain, "gain", torch.float32), _dev(x, "x", torch.float32),
                                        None if next_out is None else _dev(next_gain, "next_gain", torch.float32),
                                        None if next_out is None else _dev(next_out, "next_out"), n, hidden, float(eps),
                                        float(next_eps), dtype_code(y.dtype), _stream()), "norm_residual_norm")


# ------------------------------------------------- mixers with a decaying matrix state
def _rows(t: torch.Tensor, name: str, dtype) -> None:
    _need(t.is_cuda and t.dim() == 2 and t.stride(1) == 1 and t.dtype == dtype, f"{name}: rows with unit inner stride of {dtype} on the GPU")


def decayed_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                       q_start: torch.Tensor, state_slots: torch.Tensor, n_reqs: int, *, num_heads: int,
                       decay_pre: Optional[torch.Tensor] = None, decay_bias: Optional[torch.Tensor] = None,
                       decay_const: Optional[torch.Tensor] = None, tau: float = 1.0, q_scale: float = 1.0,
                       silu_inputs: bool = False, pieces: Optional[dict] = None) -> None:
    """Per request and head, over the step's tokens:  S = diag(a_t) S + k_t v_t^T;  out_t = S^T q_t, with S (float32
    [dk, dv]) read from and left in the request's slot of ``state`` [slots, heads, dk, dv].  q, k [n, heads * dk] and
    v [n, heads * dv] are rows (strided views allowed) of the activations' type; out float32 [n, heads * dv].  The decay:
    ``decay_pre`` ([n, heads * dk]) gives a_t = sigmoid(decay_pre + decay_bias)^(1 / tau) per key channel;
    ``decay_const`` (float32 [heads]) one number per head; neither: 1.  ``silu_inputs``: q, k and v pass through
    silu; ``q_scale`` multiplies q.

    ``pieces`` (for steps with long portions): the portions cut into pieces of at most SCAN_PIECE tokens that run side
    by side, then are joined (csrc/recurrent.cu): {"start": int32 [pieces + 1] first rows, "req": int32 [n_reqs + 1] the
    pieces of each request, "slots": int32 [pieces] = 0 .. pieces - 1, "count": pieces, "state": float32 scratch
    [pieces, heads, dk, dv], "qp": float32 scratch [n, heads * dk], "dtot": float32 scratch [pieces, heads, dk]}."""
    n = q.shape[0]
    H = num_heads
    _need(q.shape[1] % H == 0 and v.shape[1] % H == 0, "decayed_state_scan: widths must be multiples of the head count")
    dk, dv = q.shape[1] // H, v.shape[1] // H
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _rows(t, name, q.dtype)
    _need(k.shape == q.shape and v.shape[0] == n, "decayed_state_scan: q, k and v of one step")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv),
          "decayed_state_scan: state float32 [slots, heads, dk, dv]")
    _rows(out, "out", torch.float32)
    _need(out.shape == (n, H * dv), "decayed_state_scan: out [n, heads * dv]")
    if decay_pre is not None:
        _rows(decay_pre, "decay_pre", q.dtype)
        _need(decay_pre.shape == q.shape and decay_const is None and tau > 0, "decayed_state_scan: one decay per key channel")
        _need(decay_bias is None or decay_bias.numel() == H * dk, "decayed_state_scan: decay_bias [heads * dk]")
    if decay_const is not None:
        _need(decay_const.numel() == H, "decayed_state_scan: decay_const [heads]")
    if pieces is not None:
        count = int(pieces["count"])
        ps, qp, dtot = pieces["state"], pieces["qp"], pieces["dtot"]
        _need(ps.dtype == torch.float32 and ps.is_contiguous() and tuple(ps.shape) == (count, H, dk, dv)
              and qp.dtype == torch.float32 and qp.is_contiguous() and tuple(qp.shape) == (n, H * dk)
              and dtot.dtype == torch.float32 and dtot.is_contiguous() and dtot.numel() == count * H * dk,
              "decayed_state_scan: scratch of the pieces")
        _check(lib().vcb_decayed_state_scan(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), None if decay_pre is None else decay_pre.data_ptr(),
            q.stride(0), k.stride(0), v.stride(0), 0 if decay_pre is None else decay_pre.stride(0),
            None if decay_bias is None else _dev(decay_bias, "decay_bias", torch.float32),
            None if decay_const is None else _dev(decay_const, "decay_const", torch.float32),
            1.0 / float(tau), float(q_scale), 1 if silu_inputs else 0, ps.data_ptr(), out.data_ptr(), out.stride(0),
            _dev(pieces["start"], "pieces.start", torch.int32), _dev(pieces["slots"], "pieces.slots", torch.int32), count, H, dk, dv,
            1, qp.data_ptr(), qp.stride(0), dtot.data_ptr(), dtype_code(q.dtype), _stream()), "decayed_state_scan")
        _check(lib().vcb_decayed_state_join(qp.data_ptr(), qp.stride(0), ps.data_ptr(), dtot.data_ptr(), state.data_ptr(),
                                            out.data_ptr(), out.stride(0), pieces["start"].data_ptr(),
                                            _dev(pieces["req"], "pieces.req", torch.int32), _dev(state_slots, "state_slots", torch.int32),
                                            count, n_reqs, H, dk, dv, _stream()), "decayed_state_join")
        add_launches(1)            # the join is two kernels
        return
    _check(lib().vcb_decayed_state_scan(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), None if decay_pre is None else decay_pre.data_ptr(),
        q.stride(0), k.stride(0), v.stride(0), 0 if decay_pre is None else decay_pre.stride(0),
        None if decay_bias is None else _dev(decay_bias, "decay_bias", torch.float32),
        None if decay_const is None else _dev(decay_const, "decay_const", torch.float32),
        1.0 / float(tau), float(q_scale), 1 if silu_inputs else 0, state.data_ptr(), out.data_ptr(), out.stride(0),
        _dev(q_start, "q_start", torch.int32), _dev(state_slots, "state_slots", torch.int32), n_reqs, H, dk, dv,
        0, None, 0, None, dtype_code(q.dtype), _stream()), "decayed_state_scan")


SCAN_PIECE = 128          # tokens of a piece of a long portion (decayed_state_scan with ``pieces``)


def scan_pieces(q_lens):
    """Cuts a step's portions into pieces of at most SCAN_PIECE tokens: (first rows [pieces + 1], pieces of each request
    [n_reqs + 1]) as int32 arrays."""
    import numpy as np
    starts, per_req, row = [0], [0], 0
    for n in q_lens:
        left = int(n)
        while left > 0:
            take = min(SCAN_PIECE, left)
            row += take
            left -= take
            starts.append(row)
        per_req.append(len(starts) - 1)
    return np.asarray(starts, dtype=np.int32), np.asarray(per_req, dtype=np.int32)


def gated_group_norm(o: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor, *, group: int,
                     eps: float, gate_act: str = "sigmoid") -> None:
    """out = o / sqrt(mean over each group of ``group`` channels of o^2 + eps) * weight[channel % len(weight)] * act(gate);
    o float32 [n, C], gate and out rows of the activations' type, act "sigmoid" or "silu"."""
    n, C = o.shape
    _rows(o, "o", torch.float32)
    _rows(out, "out", out.dtype)
    _need(out.shape == o.shape and (C % group == 0) and weight.numel() in (group, C), "gated_group_norm: shapes")
    _need(gate_act in ("sigmoid", "silu"), "gated_group_norm: gate_act is 'sigmoid' or 'silu'")
    if gate is not None:
        _rows(gate, "gate", out.dtype)
        _need(gate.shape == o.shape, "gated_group_norm: gate like o")
    _check(lib().vcb_gated_group_norm(o.data_ptr(), o.stride(0), None if gate is None else gate.data_ptr(),
                                      0 if gate is None else gate.stride(0), _dev(weight, "weight", torch.float32),
                                      weight.numel(), out.data_ptr(), out.stride(0), n, C, group,
                                      1 if gate_act == "silu" else 0, float(eps), dtype_code(out.dtype), _stream()),
           "gated_group_norm")


def scaled_sum(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor, a: float, b: float) -> None:
    """out = a * x + b * y, computed in float and rounded once."""
    _need(x.shape == y.shape == out.shape and x.dtype == y.dtype == out.dtype, "scaled_sum: one shape, one type")
    _check(lib().vcb_scaled_sum(_dev(x, "x"), _dev(y, "y"), _dev(out, "out"), x.numel(), float(a), float(b),
                                dtype_code(x.dtype), _stream()), "scaled_sum")


# ------------------------------------------------- attention with capped scores and a bias by distance
def qk_norm_cache_write(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, wq: Optional[torch.Tensor],
                        wk: Optional[torch.Tensor], q_out: torch.Tensor, cache: torch.Tensor, positions, req_of_token,
                        block_table, *, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, row: int,
                        page_size: int, eps: float, write_kv: bool) -> None:
    """A token's row of ``proj`` holds its query projection at ``q_off`` (heads * head_dim), key projection at ``k_off``
    (kv heads * head_dim) and values at ``v_off`` (kv heads * v_head_dim).  Queries and keys are RMS-normed over the whole
    projection with the gains ``wq`` / ``wk`` (None: left as they are); queries go to ``q_out``, keys and values into
    the token's slot of the cache, whose rows are ``row`` elements wide."""
    n = proj.shape[0]
    _rows(proj, "proj", proj.dtype)
    _need(q_out.shape == (n, num_heads * head_dim) and q_out.dtype == proj.dtype and cache.dtype == proj.dtype, "qk_norm_cache_write: types")
    _need(wq is None or wq.numel() == num_heads * head_dim, "qk_norm_cache_write: one query gain per channel")
    _need(wk is None or wk.numel() == num_kv_heads * head_dim, "qk_norm_cache_write: one key gain per channel")
    _need(cache.is_contiguous() and cache.numel() == cache.shape[0] * 2 * num_kv_heads * page_size * row,
          "qk_norm_cache_write: a cache of key and value planes with rows of `row` elements")
    _check(lib().vcb_qk_norm_cache_write(
        proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, None if wq is None else _dev(wq, "wq", torch.float32),
        None if wk is None else _dev(wk, "wk", torch.float32), _dev(q_out, "q_out"), cache.data_ptr(),
        _dev(positions, "positions", torch.int32), _dev(req_of_token, "req_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], n, num_heads, num_kv_heads, head_dim,
        v_head_dim, row, page_size, cache.shape[0], 1 if write_kv else 0, float(eps), status_tensor(proj.device).data_ptr(),
        dtype_code(proj.dtype), _stream()), "qk_norm_cache_write")


def attention_biased(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], positions,
                     req_of_token, block_table, bias: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int,
                     head_dim: int, v_head_dim: int, row: int, page_size: int, window: int, scale: float, cap: float,
                     sink: Optional[torch.Tensor] = None, gate_per_head: bool = False) -> None:
    """Paged attention with  score = cap * tanh(scale * q.k / cap) + bias[min(distance, len(bias) - 1), head]  (cap <= 0: no
    cap; bias float32 [distances, heads] or None), softmax over the keys the window leaves, values of ``v_head_dim``,
    and out *= sigmoid(gate) when a gate is given ([n, heads * v_head_dim] rows, or with ``gate_per_head`` [n, heads]: one
    number per head).  ``sink`` (float32 [heads]): a logit per head that joins the softmax's denominator once, unscaled,
    and has no value."""
    n = q.shape[0]
    _need(q.shape == (n, num_heads * head_dim) and out.shape == (n, num_heads * v_head_dim) and out.dtype == q.dtype
          and cache.dtype == q.dtype, "attention_biased: shapes or types")
    _need(v_head_dim <= 256 and head_dim <= 1024, "attention_biased: head sizes up to 1024 (keys) and 256 (values)")
    if gate is not None:
        _rows(gate, "gate", q.dtype)
        _need(gate.shape == ((n, num_heads) if gate_per_head else out.shape), "attention_biased: gate like out, or one column per head")
    _need(sink is None or sink.numel() == num_heads, "attention_biased: one sink per head")
    if bias is not None:
        _need(bias.dim() == 2 and bias.shape[1] == num_heads, "attention_biased: bias [distances, heads]")
    _check(lib().vcb_attention_biased(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), None if gate is None else gate.data_ptr(),
        0 if gate is None else gate.stride(0), _dev(positions, "positions", torch.int32),
        _dev(req_of_token, "req_of_token", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        None if bias is None else _dev(bias, "bias", torch.float32), 0 if bias is None else bias.shape[0], n, num_heads,
        num_kv_heads, head_dim, v_head_dim, row, page_size, window, float(scale), float(cap), cache.shape[0],
        status_tensor(q.device).data_ptr(), None if sink is None else _dev(sink, "sink", torch.float32),
        1 if gate_per_head else 0, dtype_code(q.dtype), _stream()), "attention_biased")


def qk_head_rope_cache_write(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, wq: Optional[torch.Tensor],
                             wk: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], q_out: torch.Tensor,
                             cache: torch.Tensor, positions, req_of_token, block_table, *, num_heads: int, num_kv_heads: int,
                             head_dim: int, v_head_dim: int, row: int, page_size: int, eps: float, write_kv: bool) -> None:
    """As qk_norm_cache_write, but queries and keys are RMS-normed head by head over ``head_dim`` with gains ``wq`` / ``wk``
    (float32 [head_dim], shared by the heads; None: not normed) and then rotated on their first 2 * len(inv_freq)
    coordinates (coordinate i pairs with i + len(inv_freq); angle = position * inv_freq[i], float32)."""
    n = proj.shape[0]
    _rows(proj, "proj", proj.dtype)
    _need(q_out.shape == (n, num_heads * head_dim) and q_out.dtype == proj.dtype and cache.dtype == proj.dtype, "qk_head_rope_cache_write: types")
    _need(wq is None or wq.numel() == head_dim, "qk_head_rope_cache_write: one query gain per coordinate of a head")
    _need(wk is None or wk.numel() == head_dim, "qk_head_rope_cache_write: one key gain per coordinate of a head")
    rot = 0 if inv_freq is None else 2 * inv_freq.numel()
    _need(rot <= head_dim, "qk_head_rope_cache_write: more rotated coordinates than a head has")
    _need(cache.is_contiguous() and cache.numel() == cache.shape[0] * 2 * num_kv_heads * page_size * row,
          "qk_head_rope_cache_write: a cache of key and value planes with rows of `row` elements")
    _check(lib().vcb_qk_head_rope_cache_write(
        proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, None if wq is None else _dev(wq, "wq", torch.float32),
        None if wk is None else _dev(wk, "wk", torch.float32), None if inv_freq is None else _dev(inv_freq, "inv_freq", torch.float32),
        rot, _dev(q_out, "q_out"), cache.data_ptr(), _dev(positions, "positions", torch.int32),
        _dev(req_of_token, "req_of_token", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.shape[1], n,
        num_heads, num_kv_heads, head_dim, v_head_dim, row, page_size, cache.shape[0], 1 if write_kv else 0, float(eps),
        status_tensor(proj.device).data_ptr(), dtype_code(proj.dtype), _stream()), "qk_head_rope_cache_write")


# ------------------------------------------------- routed experts
MOE_TILE_ROWS = (16, 64)       # heights of the expert products' tiles: short for steps of few tokens


def moe_tile_rows(n_tokens: int, top: int, n_experts: int) -> int:
    """The tile height for a step: 64 rows once an expert gets that many tokens on average, else 16."""
    return 64 if n_tokens * top >= 64 * n_experts else 16


def moe_max_tiles(n_tokens: int, top: int, n_experts: int, tm: int) -> int:
    """The most tiles a step can have: every expert may end with a tile that is not full."""
    pairs = n_tokens * top
    return min(pairs, pairs // tm + n_experts)


ROUTER_SCORES = {"softmax": 0, "sigmoid": 1}
ROUTER_GROUP_TOP_MAX = 4


def moe_router(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], ids: torch.Tensor,
               weights: torch.Tensor, logits: torch.Tensor, *, score: str = "softmax", groups: int = 1, keep_groups: int = 1,
               group_top: int = 1, normalize: bool = False, sum_eps: float = 0.0, scale: float = 1.0,
               logit_bias: Optional[torch.Tensor] = None) -> None:
    """For every row of h: scores in float32 from the logits w_router h, by softmax over all router outputs or by a
    sigmoid of each (``score``); ids [n, top] = the outputs with the largest score + correction (the lower index wins
    among equals), with ``groups`` > ``keep_groups`` only among the ``keep_groups`` best of ``groups`` equal groups of
    neighbouring outputs (a group's score: the sum of its ``group_top`` largest); weights [n, top] = their plain scores,
    with ``normalize`` divided by (their sum + ``sum_eps``), times ``scale``.  ``logit_bias`` (float32 [router outputs]) joins
    the logits before the scores are made.  Softmax scores of the chosen, normalized, are the softmax over the chosen
    logits alone.  ``logits``: float32 scratch [n, router outputs].  Two kernels (csrc/moe.cu)."""
    _need(score in ROUTER_SCORES, f"moe_router: score is one of {sorted(ROUTER_SCORES)}")
    _need(groups >= 1 and w_router.shape[0] % groups == 0 and 1 <= keep_groups <= groups and 1 <= group_top <= ROUTER_GROUP_TOP_MAX,
          "moe_router: equal groups, some of them kept, a group's score from at most four outputs")
    _need(ids.shape[1] <= w_router.shape[0] // groups * keep_groups, "moe_router: more choices than the kept groups hold")
    n, width = h.shape
    _rows(h, "h", h.dtype)
    top = ids.shape[1]
    _need(w_router.shape[1] == width and ids.shape == (n, top) and weights.shape == (n, top), "moe_router: shapes")
    _need(correction is None or correction.numel() == w_router.shape[0], "moe_router: one correction per router output")
    _need(logit_bias is None or logit_bias.numel() == w_router.shape[0], "moe_router: one bias per router output")
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and logits.numel() >= n * w_router.shape[0], "moe_router: logits scratch")
    _check(lib().vcb_moe_router_biased(h.data_ptr(), h.stride(0), _dev(w_router, "w_router", torch.float32),
                                      None if logit_bias is None else _dev(logit_bias, "logit_bias", torch.float32),
                                      None if correction is None else _dev(correction, "correction", torch.float32),
                                      logits.data_ptr(), _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32), n, width,
                                      w_router.shape[0], top, ROUTER_SCORES[score], groups, keep_groups, group_top,
                                      1 if normalize else 0, float(sum_eps), float(scale), dtype_code(h.dtype), _stream()), "moe_router")
    add_launches(1)                # logits and selection


def moe_sort(ids: torch.Tensor, n_experts: int, tm: int, sorted_token, pos, tile_expert, tile_row0, tile_rows, meta) -> None:
    """Groups the (token, choice) pairs of ``ids`` [n, top] by expert (see moe.cu); outputs >= n_experts get pos -1."""
    n, top = ids.shape
    for t, name in ((sorted_token, "sorted_token"), (pos, "pos"), (tile_expert, "tile_expert"), (tile_row0, "tile_row0"),
                    (tile_rows, "tile_rows"), (meta, "meta")):
        _dev(t, name, torch.int32)
    _need(sorted_token.numel() >= n * top and pos.numel() >= n * top, "moe_sort: a row per pair")
    _need(tile_expert.numel() >= moe_max_tiles(n, top, n_experts, tm), "moe_sort: room for every tile")
    _check(lib().vcb_moe_sort(_dev(ids, "ids", torch.int32), n * top, top, n_experts, tm, sorted_token.data_ptr(), pos.data_ptr(),
                              tile_expert.data_ptr(), tile_row0.data_ptr(), tile_rows.data_ptr(), meta.data_ptr(), _stream()),
           "moe_sort")


def moe_expert_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, sorted_token, tile_expert, tile_row0, tile_rows, meta,
                    max_tiles: int, tm: int, *, gated: bool, limit: float = 0.0, alpha: float = 0.0, up_shift: float = 1.0) -> None:
    """The experts' products over the tiles of moe_sort.  gated: a [n, K] the tokens' rows, w [E, 2 * N, K] gate rows then
    up rows, out [pairs, N] of the activations' type = g * sigmoid(alpha * g) * (u + up_shift) with g = min(gate, limit),
    u = clamp(up, -limit, limit) (limit inf, alpha 1, up_shift 0: silu(gate) * up).  Not gated: a [pairs, K] the sorted
    rows, w [E, N, K], out [pairs, N] float32."""
    _rows(a, "a", a.dtype)
    _need(w.dim() == 3 and w.is_contiguous() and w.dtype == a.dtype and w.shape[2] == a.shape[1], "moe_expert_gemm: w [E, N, K]")
    N = w.shape[1] // 2 if gated else w.shape[1]
    _rows(out, "out", a.dtype if gated else torch.float32)
    _need(out.shape[1] == N and tm in MOE_TILE_ROWS, "moe_expert_gemm: out [pairs, N]")
    _check(lib().vcb_moe_expert_gemm(a.data_ptr(), a.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), N, a.shape[1],
                                     sorted_token.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(), tile_rows.data_ptr(),
                                     meta.data_ptr(), max_tiles, tm, 1 if gated else 0, float(limit), float(alpha), float(up_shift),
                                     dtype_code(a.dtype), _stream()), "moe_expert_gemm")


def moe_combine(y: torch.Tensor, h: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor, out: torch.Tensor,
                add: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k weights[t, k] * (y[pos[t, k]] if pos[t, k] >= 0 else h[t]) (+ add[t]: what every token takes beside
    its choices, rows of out's type); y float32 [pairs, width]."""
    n, width = out.shape
    _rows(h, "h", out.dtype)
    _need(y.dtype == torch.float32 and y.is_contiguous() and y.shape[1] == width and h.shape == out.shape, "moe_combine: shapes")
    if add is not None:
        _rows(add, "add", out.dtype)
        _need(add.shape == out.shape, "moe_combine: add like out")
    _check(lib().vcb_moe_combine_add(y.data_ptr(), h.data_ptr(), h.stride(0), _dev(pos, "pos", torch.int32),
                                     _dev(weights, "weights", torch.float32), _dev(out, "out"), n, width, weights.shape[1],
                                     None if add is None else add.data_ptr(), 0 if add is None else add.stride(0),
                                     dtype_code(out.dtype), _stream()), "moe_combine")


# ------------------------------------------------- a residual stream of several copies, read through a layer norm
STREAMS_MAX = 8


def _streams(x: torch.Tensor, name: str):
    _need(x.dim() == 3 and x.dtype == torch.float32 and x.is_cuda and x.stride(2) == 1 and x.stride(1) == x.shape[2]
          and 1 <= x.shape[0] <= STREAMS_MAX, f"{name}: float32 streams [S <= {STREAMS_MAX}, n, hidden] with contiguous rows")
    return x.shape


def stream_norm(x: torch.Tensor, coef: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], out: torch.Tensor, eps: float,
                row_index: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """out = layer_norm(sum_s coef[s] x[s]) * w + b, times ``out_scale``; mean and variance (the mean of the squared
    deviations) in float32.  x float32 [S, n, hidden]; with ``row_index`` out row o reads row row_index[o]."""
    S, n, hidden = _streams(x, "stream_norm")
    rows = out.shape[0]
    _need(out.shape[1] == hidden and w.numel() == hidden and (b is None or b.numel() == hidden) and coef.numel() == S, "stream_norm: widths")
    _need(rows == n if row_index is None else row_index.numel() == rows, "stream_norm: one output row per row read")
    _check(lib().vcb_stream_norm(x.data_ptr(), x.stride(0), _dev(coef, "coef", torch.float32), _dev(w, "w", torch.float32),
                                 None if b is None else _dev(b, "b", torch.float32), _dev(out, "out"),
                                 None if row_index is None else _dev(row_index, "row_index", torch.int32), rows, S, hidden,
                                 float(eps), float(out_scale), dtype_code(out.dtype), _stream()), "stream_norm")


def stream_join(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, out_coef: torch.Tensor, eps: float = 0.0,
                next_coef: Optional[torch.Tensor] = None, next_w: Optional[torch.Tensor] = None,
                next_b: Optional[torch.Tensor] = None, next_out: Optional[torch.Tensor] = None) -> None:
    """x[t] <- sum_s mix[s, t] x[s] + out_coef[t] y for all streams at once, in float32 in place; with ``next_out``:
    next_out = layer_norm(sum_t next_coef[t] x[t]) * next_w + next_b, the input of the sublayer that follows."""
    S, n, hidden = _streams(x, "stream_join")
    _need(y.shape == (n, hidden) and mix.numel() == S * S and out_coef.numel() == S, "stream_join: shapes")
    if next_out is not None:
        _need(next_coef is not None and next_coef.numel() == S and next_w is not None and next_w.numel() == hidden
              and (next_b is None or next_b.numel() == hidden) and next_out.shape == (n, hidden) and next_out.dtype == y.dtype,
              "stream_join: the next sublayer's coefficients, norm and input")
    _check(lib().vcb_stream_join(x.data_ptr(), x.stride(0), _dev(y, "y"), _dev(mix, "mix", torch.float32),
                                 _dev(out_coef, "out_coef", torch.float32),
                                 None if next_out is None else _dev(next_coef, "next_coef", torch.float32),
                                 None if next_out is None else _dev(next_w, "next_w", torch.float32),
                                 None if next_out is None or next_b is None else _dev(next_b, "next_b", torch.float32),
                                 None if next_out is None else _dev(next_out, "next_out"), n, S, hidden, float(eps),
                                 dtype_code(y.dtype), _stream()), "stream_join")


# ------------------------------------------------- recurrent mixers behind a short convolution
CONV_MAX_TAPS = 8


def causal_conv(x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, out: torch.Tensor, q_start, state_slots, n_reqs: int,
                max_q_len: int, *, pre_bias: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                act: str = "none") -> None:
    """out[t, c] = act(sum_j taps[c, j] * in[t - (J - 1) + j, c] + bias[c]) over each request's tokens, in = x + pre_bias;
    the J - 1 inputs before a request's first token of the step come from its slot of ``state`` (float32
    [slots, >= J - 1 rows, C] as a strided view: rows 0 .. J - 2, oldest first; zero at admission), which then receives the
    step's last J - 1 inputs.  x rows of the activations' type [n, C]; taps float32 [C, J]; out float32 [n, C] rows."""
    n, C = x.shape
    J = taps.shape[1]
    _rows(x, "x", x.dtype)
    _rows(out, "out", torch.float32)
    _need(out.shape == (n, C) and taps.shape[0] == C and 1 <= J <= CONV_MAX_TAPS, f"causal_conv: taps [C, up to {CONV_MAX_TAPS}]")
    _need(act in ("none", "silu"), "causal_conv: act is 'none' or 'silu'")
    _need(state.dtype == torch.float32 and state.dim() == 3 and state.shape[2] == C and state.shape[1] >= J - 1
          and state.stride(2) == 1 and (J == 1 or state.shape[1] == 1 or state.stride(1) == C),
          "causal_conv: state float32 [slots, J - 1, C] with contiguous rows")
    for t, name in ((pre_bias, "pre_bias"), (bias, "bias")):
        _need(t is None or t.numel() == C, f"causal_conv: {name} [C]")
    _check(lib().vcb_causal_conv(x.data_ptr(), x.stride(0), None if pre_bias is None else _dev(pre_bias, "pre_bias", torch.float32),
                                 _dev(taps, "taps", torch.float32), None if bias is None else _dev(bias, "bias", torch.float32),
                                 state.data_ptr(), state.stride(0), out.data_ptr(), out.stride(0),
                                 _dev(q_start, "q_start", torch.int32), _dev(state_slots, "state_slots", torch.int32), n_reqs,
                                 max_q_len, C, J, 1 if act == "silu" else 0, dtype_code(x.dtype), _stream()), "causal_conv")


def gate_blocks(u: torch.Tensor, wa: torch.Tensor, wi: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor, lam: torch.Tensor,
                decay: torch.Tensor, drive: torch.Tensor, c_gate: float) -> None:
    """Per block b of W / B channels:  r = sigmoid(wa[b] u_b + ba), i = sigmoid(wi[b] u_b + bi);
    decay = exp(-c_gate * r * softplus(lam)), drive = sqrt(1 - decay^2) * i * u.  u, decay, drive float32 [n, W]; wa, wi
    [B, W / B, W / B] ([out, in]) of the weights' type; the sums, gates and exponentials float32."""
    n, W = u.shape
    B = wa.shape[0]
    _rows(u, "u", torch.float32)
    _need(wa.dim() == 3 and wa.shape == wi.shape and wa.shape[1] == wa.shape[2] and B * wa.shape[1] == W and wa.dtype == wi.dtype,
          "gate_blocks: square blocks that fill the width")
    _need(decay.shape == u.shape and drive.shape == u.shape and decay.is_contiguous() and drive.is_contiguous()
          and decay.dtype == drive.dtype == torch.float32, "gate_blocks: outputs like u")
    _check(lib().vcb_gate_blocks(u.data_ptr(), u.stride(0), _dev(wa, "wa"), _dev(wi, "wi"), _dev(ba, "ba", torch.float32),
                                 _dev(bi, "bi", torch.float32), _dev(lam, "lam", torch.float32), decay.data_ptr(), drive.data_ptr(),
                                 decay.stride(0), n, W, B, float(c_gate), dtype_code(wa.dtype), _stream()), "gate_blocks")


def linear_recurrence(decay: torch.Tensor, drive: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor],
                      state: torch.Tensor, out: torch.Tensor, q_start, state_slots, n_reqs: int, max_q_len: int = 1) -> None:
    """S_t = decay_t * S_(t-1) + drive_t per channel and request, S read from and left in the request's slot of ``state``
    (float32 [slots, W] as a strided view); out = S_t * gelu_tanh(y_t + y_bias) in the activations' type.  ``max_q_len``:
    the longest portion of the step; long ones are walked in stretches side by side (csrc/gated_recurrence.cu)."""
    n, W = decay.shape
    _need(decay.is_contiguous() and drive.is_contiguous() and drive.shape == decay.shape and decay.dtype == drive.dtype == torch.float32,
          "linear_recurrence: decay and drive float32 [n, W]")
    _rows(y, "y", out.dtype)
    _rows(out, "out", out.dtype)
    _need(y.shape == (n, W) and out.shape == (n, W) and (y_bias is None or y_bias.numel() == W), "linear_recurrence: shapes")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == W and state.stride(1) == 1, "linear_recurrence: state [slots, W]")
    _check(lib().vcb_linear_recurrence(decay.data_ptr(), drive.data_ptr(), decay.stride(0), y.data_ptr(), y.stride(0),
                                       None if y_bias is None else _dev(y_bias, "y_bias", torch.float32), state.data_ptr(),
                                       state.stride(0), out.data_ptr(), out.stride(0), _dev(q_start, "q_start", torch.int32),
                                       _dev(state_slots, "state_slots", torch.int32), n_reqs, int(max_q_len), W, dtype_code(out.dtype),
                                       _stream()), "linear_recurrence")


DELTA_PORTIONS_FROM = 8       # a step whose longest portion has this many tokens prepares the recurrence's inputs in a kernel of its own


def gated_delta_work_row(num_heads: int, num_qk_heads: int, head_dim: int) -> int:
    """Floats of a token's row of prepared inputs: unit q and k per qk head, a decay per head and key channel, beta per
    head, q . k per qk head; rounded up to 16 bytes."""
    return ((2 * num_qk_heads + num_heads) * head_dim + num_heads + num_qk_heads + 3) // 4 * 4


def gated_delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta_pre: torch.Tensor, decay_pre: torch.Tensor,
                     a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, out: torch.Tensor, q_start, state_slots,
                     n_reqs: int, *, num_heads: int, num_qk_heads: int, q_scale: float, unit_eps: float, max_q_len: int = 1,
                     work: Optional[torch.Tensor] = None) -> None:
    """The gated delta rule per request and head over the step's tokens, S (float32 [dk, dv]) read from and left in the
    request's slot of ``state`` [slots, heads, dk, dv]:
        S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  out_t = S^T q_t
    q, k float32 rows [n, qk heads * dk] (made unit vectors per head here: x / sqrt(sum x^2 + unit_eps); q times
    ``q_scale``), head h reading qk head h // (heads / qk heads); v float32 rows [n, heads * dv]; beta = sigmoid(beta_pre
    [n, heads]); g = exp(-exp(a_log[h]) * softplus(decay_pre [n, heads * dk] + dt_bias)); out float32 [n, heads * dv].
    A step whose longest portion ``max_q_len`` reaches DELTA_PORTIONS_FROM tokens runs in two kernels: the unit vectors, decays
    and betas of all tokens at once into ``work`` (float32, n * gated_delta_work_row(...) elements; made here if absent),
    then the walk over the tokens, which needs one round of shuffles per token (csrc/gated_recurrence.cu)."""
    n = q.shape[0]
    H, G = num_heads, num_qk_heads
    _need(H % G == 0 and q.shape[1] % G == 0 and v.shape[1] % H == 0, "gated_delta_scan: head counts")
    dk, dv = q.shape[1] // G, v.shape[1] // H
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (out, "out")):
        _rows(t, name, torch.float32)
    _rows(beta_pre, "beta_pre", beta_pre.dtype)
    _rows(decay_pre, "decay_pre", beta_pre.dtype)
    _need(k.shape == q.shape and v.shape[0] == n and out.shape == (n, H * dv) and beta_pre.shape == (n, H)
          and decay_pre.shape == (n, H * dk), "gated_delta_scan: shapes")
    _need(dk <= 1024, "gated_delta_scan: key heads of up to 1024 channels")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv),
          "gated_delta_scan: state float32 [slots, heads, dk, dv]")
    portions = max_q_len >= DELTA_PORTIONS_FROM
    if portions:
        need = n * gated_delta_work_row(H, G, dk)
        if work is None:
            work = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(work.dtype == torch.float32 and work.is_contiguous() and work.numel() >= need, "gated_delta_scan: work too small")
    _check(lib().vcb_gated_delta_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                                      beta_pre.data_ptr(), beta_pre.stride(0), decay_pre.data_ptr(), decay_pre.stride(0),
                                      _dev(a_log, "a_log", torch.float32), _dev(dt_bias, "dt_bias", torch.float32),
                                      state.data_ptr(), out.data_ptr(), out.stride(0), _dev(q_start, "q_start", torch.int32),
                                      _dev(state_slots, "state_slots", torch.int32), n_reqs, H, G, dk, dv, float(q_scale),
                                      float(unit_eps), dtype_code(beta_pre.dtype), work.data_ptr() if portions else None,
                                      n if portions else 0, _stream()), "gated_delta_scan")


# ------------------------------------------------------------------ latent attention
def latent_cache_write(raw: torch.Tensor, gain: torch.Tensor, positions, req_of_token, block_table, cache: torch.Tensor,
                       *, page_size: int, eps: float) -> None:
    """RMS norm (gain vector, float statistics) of the rows of ``raw`` ([n, rank], rows may be strided) and their
    write into the tokens' slots of a one-plane cache [pages, page_size * rank] (kv_pos layout)."""
    n, rank = raw.shape
    _need(raw.stride(1) == 1 and raw.is_cuda, "latent_cache_write: rows with unit inner stride on the GPU")
    _need(cache.dtype == raw.dtype and cache.is_contiguous() and cache.numel() == cache.shape[0] * page_size * rank,
          "latent_cache_write: a one-plane cache of the activations' type")
    _need(gain.numel() == rank, "latent_cache_write: one gain per latent coordinate")
    _check(lib().vcb_latent_cache_write(raw.data_ptr(), raw.stride(0), _dev(gain, "gain", torch.float32),
                                        _dev(positions, "positions", torch.int32), _dev(req_of_token, "req_of_token", torch.int32),
                                        _dev(block_table, "block_table", torch.int32), block_table.shape[1], cache.data_ptr(),
                                        page_size * rank, n, rank, page_size, float(eps), cache.shape[0],
                                        status_tensor(raw.device).data_ptr(), dtype_code(raw.dtype), _stream()),
           "latent_cache_write")


HEADWISE_LIBRARY_TOKENS = 128      # bfloat16 portions longer than this run the library's batched product


def headwise_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                    gate_per_head: bool = False) -> None:
    """out[t, h, :] = x[t, h, :] @ w[h]^T for every head: x [n, heads * K] (rows may be strided), w [heads, N, K],
    out [n, heads * N]; with ``gate`` ([n, heads * N], or with ``gate_per_head`` [n, heads]: one number per head; rows
    may be strided) out *= sigmoid(gate).  float32 and short bfloat16 steps: this library's kernel; long bfloat16
    portions: the library's batched product, then the gate as a kernel."""
    heads, N, K = w.shape
    n = x.shape[0]
    _need(x.shape == (n, heads * K) and out.shape == (n, heads * N) and x.stride(1) == 1 and out.stride(1) == 1,
          "headwise_linear: x [n, heads * K], out [n, heads * N]")
    _need(w.is_contiguous() and x.dtype == w.dtype == out.dtype, "headwise_linear: one type, contiguous weights")
    if gate is not None:
        _need(gate.shape == ((n, heads) if gate_per_head else out.shape) and gate.stride(1) == 1 and gate.dtype == out.dtype,
              "headwise_linear: gate like out, or one column per head")
    if x.dtype == torch.bfloat16 and n > HEADWISE_LIBRARY_TOKENS:
        xh = x.unflatten(1, (heads, K)).transpose(0, 1)             # [heads, n, K]
        oh = out.unflatten(1, (heads, N)).transpose(0, 1)           # [heads, n, N]
        torch.bmm(xh, w.transpose(1, 2), out=oh)                    # the library writes the strided rows itself
        if gate is not None:
            _check(lib().vcb_sigmoid_gate(out.data_ptr(), gate.data_ptr(), n, heads * N, out.stride(0), gate.stride(0),
                                          N if gate_per_head else 1, dtype_code(out.dtype), _stream()), "sigmoid_gate")
        return
    _check(lib().vcb_headwise_linear(x.data_ptr(), w.data_ptr(), out.data_ptr(), None if gate is None else gate.data_ptr(),
                                     n, heads, N, K, x.stride(0), out.stride(0), 0 if gate is None else gate.stride(0),
                                     1 if gate_per_head else 0, dtype_code(x.dtype), _stream()), "headwise_linear")


def sigmoid_gate(out: torch.Tensor, gate: torch.Tensor) -> None:
    """out *= sigmoid(gate) in place; rows of both may be strided."""
    n, cols = out.shape
    _need(gate.shape == out.shape and gate.dtype == out.dtype and out.stride(1) == 1 and gate.stride(1) == 1, "sigmoid_gate: gate like out")
    _check(lib().vcb_sigmoid_gate(out.data_ptr(), gate.data_ptr(), n, cols, out.stride(0), gate.stride(0), 1,
                                  dtype_code(out.dtype), _stream()), "sigmoid_gate")


def rows_rmsnorm(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * gain for rows of the activations' type (both may be strided), float
    statistics: the norm of a low-rank row between two products."""
    n, width = x.shape
    _need(out.shape == x.shape and out.dtype == x.dtype and x.stride(1) == 1 and out.stride(1) == 1 and x.is_cuda, "rows_rmsnorm: rows of one type")
    _need(gain.numel() == width, "rows_rmsnorm: one gain per coordinate")
    _check(lib().vcb_rows_rmsnorm(x.data_ptr(), x.stride(0), _dev(gain, "gain", torch.float32), out.data_ptr(), out.stride(0), n, width,
                                  float(eps), dtype_code(x.dtype), _stream()), "rows_rmsnorm")


def latent_rope_cache_write(raw: torch.Tensor, gain: torch.Tensor, q: Optional[torch.Tensor], inv_freq: torch.Tensor, positions,
                            req_of_token, block_table, cache: torch.Tensor, *, rank: int, num_heads: int, q_stride: int, q_off: int,
                            pairing: int, page_size: int, eps: float, write_kv: bool = True) -> None:
    """``raw`` [n, rank + rot] (rows may be strided): the latent's columns, RMS-normed with ``gain``, and the ``rot`` =
    2 * len(inv_freq) columns of a key part that all heads share, turned by the token's position (pair j: coordinates
    (2j, 2j + 1) with ``pairing`` 1, (j, j + rot / 2) with 0; angle position * inv_freq[j] in float32), go into the token's
    slot of a one-plane cache [pages, page_size * (rank + rot)] (kv_pos layout).  ``q`` [n, heads * q_stride] is turned in
    place on the ``rot`` columns that start at ``q_off`` inside every head."""
    n = raw.shape[0]
    rot = 2 * inv_freq.numel()
    _need(raw.shape[1] == rank + rot and raw.stride(1) == 1 and raw.is_cuda, "latent_rope_cache_write: raw [n, rank + rot]")
    _need(cache.dtype == raw.dtype and cache.is_contiguous() and cache.numel() == cache.shape[0] * page_size * (rank + rot),
          "latent_rope_cache_write: a one-plane cache of the activations' type with rows of rank + rot")
    _need(gain.numel() == rank, "latent_rope_cache_write: one gain per latent coordinate")
    if q is not None:
        _need(q.dtype == raw.dtype and q.shape == (n, num_heads * q_stride) and q.stride(1) == 1 and q_off + rot <= q_stride,
              "latent_rope_cache_write: q [n, heads * q_stride] with the rotated part inside a head")
    _check(lib().vcb_latent_rope_cache_write(
        raw.data_ptr(), raw.stride(0), _dev(gain, "gain", torch.float32), None if q is None else q.data_ptr(),
        0 if q is None else q.stride(0), num_heads, q_stride, q_off, _dev(inv_freq, "inv_freq", torch.float32), rot, int(pairing),
        _dev(positions, "positions", torch.int32), _dev(req_of_token, "req_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], cache.data_ptr(), page_size * (rank + rot), n, rank,
        page_size, float(eps), cache.shape[0], 1 if write_kv else 0, status_tensor(raw.device).data_ptr(), dtype_code(raw.dtype),
        _stream()), "latent_rope_cache_write")


TALKING_MAX_HEADS = 32
TALKING_MMA_MAX_HEADS = 16         # the tensor-core kernel runs a warp per head
TALKING_MMA_HEAD_DIMS = (64, 128)
TALKING_ITEM_ROWS = 16             # query rows of a work item of the tensor-core kernel
TALKING_KEY_TILE = 32
TALKING_MAX_SPLITS = 32
TALKING_ITEM_INTS = 6
TALKING_MAX_PARTS = 8              # most items a portion's tile is cut into along its keys


def talking_mma_fits(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """True if the tensor-core kernel of attention_talking takes these sizes: its shared memory holds two stages of every
    kv head's key and value tiles and two copies of all heads' raw scores of a tile (the same sum as in
    csrc/attention_talking.cu, vcb_attention_talking_mma_smem)."""
    if head_dim not in TALKING_MMA_HEAD_DIMS or num_heads > TALKING_MMA_MAX_HEADS:
        return False
    smem = 4 * num_kv_heads * TALKING_KEY_TILE * (head_dim + 8) * 2 + 2 * num_heads * TALKING_ITEM_ROWS * TALKING_KEY_TILE * 4 + num_heads * num_heads * 4
    return smem <= 220 * 1024


def attention_talking_mma(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], items: torch.Tensor,
                          n_items: int, q_start, ctx_lens, block_table, mix: torch.Tensor, slope: Optional[torch.Tensor], *,
                          nsplit: int, n_reqs: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                          scale: float, part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                          single_rows: bool = False, merge: Optional[torch.Tensor] = None, n_merge: int = 0) -> None:
    """attention_talking on tensor cores for bfloat16 heads of 64 or 128 (keys and values of one width).  ``items`` int32
    [n_items, 6]: (request, first row within the request's rows of this step, rows (at most 16), first key, end of keys,
    partial slot or -1).  ``nsplit`` > 1: every request brings one row, cut into ``nsplit`` runs of keys whose partial sums
    (slot = request * nsplit + run) a second kernel joins through ``part_o`` / ``part_ml`` (float32 scratch).
    ``single_rows``: every item is one row (a step of single tokens); where its tiles fit, the kernel whose fragment rows
    are the heads of a kv head's group runs instead of the one whose rows are tokens.  ``merge`` int32 [n_merge, 5]: portions
    whose keys were cut into several items (request, first row, rows, first slot, slots); their partial sums, kept for
    all 16 rows of an item (scratch of slots * heads * 16 * (head_dim + 2) floats), are joined by a second kernel."""
    n = q.shape[0]
    _need(q.dtype == torch.bfloat16 and cache.dtype == q.dtype and out.dtype == q.dtype, "attention_talking_mma: bfloat16 only")
    _need(head_dim in TALKING_MMA_HEAD_DIMS and num_heads <= TALKING_MMA_MAX_HEADS, "attention_talking_mma: up to 16 heads of 64 or 128")
    _need(q.shape == (n, num_heads * head_dim) and out.shape == q.shape, "attention_talking_mma: shapes")
    _need(mix.shape == (num_heads, num_heads) and mix.is_contiguous(), "attention_talking_mma: mix [heads, heads]")
    _need(items.dtype == torch.int32 and items.is_contiguous() and items.numel() >= n_items * TALKING_ITEM_INTS, "attention_talking_mma: items")
    if gate is not None:
        _rows(gate, "gate", q.dtype)
        _need(gate.shape == out.shape, "attention_talking_mma: gate like out")
    if nsplit > 1:
        need = n_reqs * nsplit * num_heads
        _need(part_o is not None and part_ml is not None and part_o.numel() >= need * head_dim and part_ml.numel() >= need * 2,
              "attention_talking_mma: scratch for the partial sums")
    if n_merge:
        _need(merge is not None and merge.dtype == torch.int32 and merge.is_contiguous() and merge.numel() >= n_merge * 5 and nsplit == 1
              and part_o is not None and part_ml is not None, "attention_talking_mma: merge entries with their scratch")
    _check(lib().vcb_attention_talking_mma(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), None if gate is None else gate.data_ptr(),
        0 if gate is None else gate.stride(0), items.data_ptr(), n_items, _dev(q_start, "q_start", torch.int32),
        _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(mix, "mix", torch.float32), None if slope is None else _dev(slope, "slope", torch.float32),
        None if part_o is None else part_o.data_ptr(), None if part_ml is None else part_ml.data_ptr(), nsplit, n_reqs, num_heads,
        num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0], status_tensor(q.device).data_ptr(),
        1 if single_rows else 0, merge.data_ptr() if n_merge else None, n_merge, _stream()), "attention_talking_mma")
    if nsplit > 1 or n_merge:
        add_launches(1)


def attention_talking(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], positions,
                      req_of_token, block_table, mix: torch.Tensor, slope: Optional[torch.Tensor], *, num_heads: int,
                      num_kv_heads: int, head_dim: int, v_head_dim: int, row: int, page_size: int, window: int, scale: float) -> None:
    """Paged attention whose heads' scores are mixed before the softmax:  raw_g = scale * q_g . k - slope[g] * distance,
    s_h = sum_g mix[h, g] raw_g, softmax over the keys the window leaves, values of ``v_head_dim``, and out *= sigmoid(gate)
    when a gate is given ([n, heads * v_head_dim] rows).  ``mix`` float32 [heads, heads], ``slope`` float32 [heads] or None.
    The plain kernel: a CTA per token, a warp per head (at most 32 heads)."""
    n = q.shape[0]
    _need(q.shape == (n, num_heads * head_dim) and out.shape == (n, num_heads * v_head_dim) and out.dtype == q.dtype
          and cache.dtype == q.dtype, "attention_talking: shapes or types")
    _need(num_heads <= TALKING_MAX_HEADS, f"attention_talking: at most {TALKING_MAX_HEADS} heads")
    _need(v_head_dim <= 256 and head_dim <= 1024, "attention_talking: head sizes up to 1024 (keys) and 256 (values)")
    _need(mix.shape == (num_heads, num_heads) and mix.is_contiguous(), "attention_talking: mix [heads, heads]")
    _need(slope is None or slope.numel() == num_heads, "attention_talking: one slope per head")
    if gate is not None:
        _rows(gate, "gate", q.dtype)
        _need(gate.shape == out.shape, "attention_talking: gate like out")
    _check(lib().vcb_attention_talking(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), None if gate is None else gate.data_ptr(),
        0 if gate is None else gate.stride(0), _dev(positions, "positions", torch.int32),
        _dev(req_of_token, "req_of_token", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(mix, "mix", torch.float32), None if slope is None else _dev(slope, "slope", torch.float32), n, num_heads, num_kv_heads,
        head_dim, v_head_dim, row, page_size, window, float(scale), cache.shape[0], status_tensor(q.device).data_ptr(),
        dtype_code(q.dtype), _stream()), "attention_talking")


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out.flatten()[i] = mean + std * normal(key, first + i), rounded to out's type: the counter-based
    generator of the random-weights mode (csrc/random_init.cu; weights/random_init.py has it in numpy)."""
    _check(lib().vcb_random_normal(_dev(out, "out"), out.numel(), int(first), int(key) & ((1 << 64) - 1),
                                   float(mean), float(std), dtype_code(out.dtype), _stream()), "random_normal")


def repetition_penalty(logits, ids, row_start, penalty) -> None:
    n, vocab = logits.shape
    _check(lib().vcb_repetition_penalty(_dev(logits, "logits", torch.float32), logits.stride(0),
                                        _dev(ids, "ids", torch.int32), _dev(row_start, "row_start", torch.int32),
                                        _dev(penalty, "penalty", torch.float32), n, vocab, _stream()),
           "repetition_penalty")


def sample(logits, temperature, uniform, out) -> None:
    """out[r] = argmax (temperature <= 0) or an inverse-CDF draw with uniform[r] in id order."""
    n, vocab = logits.shape
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _check(lib().vcb_sample(logits.data_ptr(), logits.stride(0), vocab, _dev(temperature, "temperature", torch.float32),
                            _dev(uniform, "uniform", torch.float32), _dev(out, "out", torch.int32), n, _stream()),
           "sample")


_filter_scratch: Optional[torch.Tensor] = None


def sample_filtered(logits, temperature, uniform, top_p, top_k, out, scratch: Optional[torch.Tensor] = None) -> None:
    """Redraws, in place in ``out``, the rows that have top-k or top-p set (see sampling.cu).
    ``scratch``: float32, at least rows * vocab elements; one is kept and grown here if not given."""
    global _filter_scratch
    n, vocab = logits.shape
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _need(vocab <= 1 << 20, f"top-k/top-p sampling takes vocabularies up to {1 << 20}, got {vocab}")
    if scratch is None:
        if _filter_scratch is None or _filter_scratch.numel() < n * vocab or _filter_scratch.device != logits.device:
            _filter_scratch = torch.empty(n * vocab, dtype=torch.float32, device=logits.device)
        scratch = _filter_scratch
    _need(scratch.numel() >= n * vocab, "sample_filtered: scratch too small")
    _check(lib().vcb_sample_filtered(logits.data_ptr(), logits.stride(0), vocab,
                                     _dev(temperature, "temperature", torch.float32),
                                     _dev(uniform, "uniform", torch.float32), _dev(top_p, "top_p", torch.float32),
                                     _dev(top_k, "top_k", torch.int32), _dev(scratch, "scratch", torch.float32),
                                     _dev(out, "out", torch.int32), n, _stream()), "sample_filtered")


_scratch = {}
_scratch_epoch = 0


def scratch_epoch() -> int:
    """Changes whenever a scratch buffer moves; captured CUDA graphs that used one are stale then."""
    return _scratch_epoch


def zeroed_ints(name: str, numel: int, device) -> torch.Tensor:
    """An int32 device buffer of at least ``numel`` zeros, kept under ``name``.  Kernels that
    count tickets in it leave it zero again."""
    t = _scratch.get(name)
    if t is None or t.numel() < numel or t.device != torch.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"scratch buffer {name!r} must be sized before a CUDA graph is captured")
        t = torch.zeros(max(numel, 1024), dtype=torch.int32, device=device)
        _scratch[name] = t
        global _scratch_epoch
        _scratch_epoch += 1
    return t


def scratch(name: str, numel: int, device) -> torch.Tensor:
    """A float32 device buffer of at least ``numel`` elements, kept under ``name`` and grown
    when needed.  Kernels that merge partial results through global memory use it."""
    t = _scratch.get(name)
    if t is None or t.numel() < numel or t.device != torch.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"scratch buffer {name!r} must be sized before a CUDA graph is captured")
        t = torch.empty(max(numel, 1024), dtype=torch.float32, device=device)
        _scratch[name] = t
        global _scratch_epoch
        _scratch_epoch += 1
    return t
