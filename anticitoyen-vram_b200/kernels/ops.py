"""Python faces of the CUDA kernels (ctypes over the C entry points of ``csrc/``).

Each function takes torch CUDA tensors, checks what the kernel assumes (device,
dtype, contiguity) and launches on the current stream.  There is no other
implementation behind these names: without the compiled library, or without a
CUDA device, the first call raises.
"""

from __future__ import annotations

import ctypes
import functools
import math
from ctypes import c_float, c_int, c_void_p

import torch

from .build import BuildError, library_path

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {
    -2: "unsupported element type",
    -3: "a size is outside what this kernel takes",
    -4: "a pointer or stride is not aligned as this kernel needs",
    -5: "scratch memory is too small",
}


class KernelError(RuntimeError):
    pass


_lib = None
_cudart_err = None


def library() -> ctypes.CDLL:
    """Load (building on first use) the kernel library; raise if it cannot be had."""
    global _lib
    if _lib is None:
        try:
            path = library_path()
        except BuildError as exc:
            raise KernelError(f"the CUDA kernels of acvram_b200 could not be built: {exc}") from exc
        lib = ctypes.CDLL(path)
        _declare(lib)
        _lib = lib
    return _lib


def set_programmatic_launch(classes: int | bool) -> None:
    """Which kernel classes are launched so that they may begin while their predecessor finishes
    (bit set: 1 matrix product, 2 norm, 4 rope/append, 8 decode attention, 16 SwiGLU, 32 the rest;
    True = the default set, False = none)."""
    if classes is True:
        classes = 0x3f
    library().acv_set_pdl(int(classes))


def loaded_library_path() -> str | None:
    return None if _lib is None else _lib._name


def _declare(lib: ctypes.CDLL) -> None:
    P, I, F, LL = c_void_p, c_int, c_float, ctypes.c_longlong
    sig = {
        "acv_embed": [P, P, P, I, I, I, I, P],
        "acv_add_rmsnorm": [P, P, P, P, P, I, I, F, I, P],
        "acv_swiglu": [P, P, I, I, I, P],
        "acv_add_bias": [P, I, P, I, I, I, P],
        "acv_qk_norm_rope_append": [P, I, I, I, I, I, P, P, F, P, I, I, P, P, P, I, P, P, P, I, I, I, I, F, P],
        "acv_attention_generic": [P, I, P, I, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, I, I, I, P, P, P],
        "acv_add_group_rmsnorm": [P, P, F, P, P, P, I, I, I, F, I, I, P],
        "acv_input_conv": [P, P, P, P, P, P, P, I, I, I, I, P, P],
        "acv_add_group_rmsnorm_conv": [P, P, F, P, P, P, P, P, I, I, I, F, I, I, I, P],
        "acv_qkv_prepare": [P, I, I, I, I, I, I, P, P, F, P, I, I, F, I, I, F, P, I, F, P, P, P, I, P, P, P, I, I, I, P],
        "acv_token_shift_multi": [P, P, P, P, P, P, P, I, I, I, I, P],
        "acv_wkv_decay": [P, I, P, P, P, I, I, I, P],
        "acv_wkv": [P, P, P, I, P, P, P, P, P, P, P, I, P, P, I, P, I, I, I, I, I, I, P],
        "acv_add_layernorm": [P, P, F, P, P, P, P, I, I, F, I, I, P],
        "acv_token_shift": [P, P, P, P, P, P, P, I, I, I, P],
        "acv_add_layernorm_shift": [P, P, F, P, P, P, P, P, P, I, I, F, I, I, P],
        "acv_add_row_f32": [P, P, I, I, P],
        "acv_softcap_f32": [P, LL, F, P],
        "acv_causal_conv": [P, I, P, P, P, P, P, P, P, P, I, I, I, I, P, P],
        "acv_block_gates": [P, P, P, P, P, P, F, P, P, I, I, I, P],
        "acv_block_gates_mma": [P, P, P, P, P, P, F, P, P, I, I, I, P],
        "acv_gated_scan": [P, P, P, I, P, P, P, P, P, P, I, P, I, P, I, I, I, I, I, P],
        "acv_retention": [P, P, P, I, P, I, I, P, P, F, P, P, P, P, P, I, P, I, P, I, I, I, I, I, I, I, P],
        "acv_retention_gate": [P, I, P, I, P, I, I, I, I, F, F, I, P, I, I, P],
        "acv_gemm_simt": [P, I, P, I, P, I, I, I, I, I, I, P],
        "acv_gemm_simt_batched": [P, I, LL, P, I, LL, P, I, LL, I, I, I, I, I, I, P],
        "acv_gemm_mma_batched_takes": [P, I, LL, P, I, LL, P, I, LL, I, I],
        "acv_gemm_mma_batched": [P, I, LL, P, I, LL, P, I, LL, I, I, I, I, P],
        "acv_attention_mixed": [P, I, P, I, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, P, F, P, P, I, I, P, I, P],
        "acv_attention_mixed_tc_takes": [I, I, I, I, I],
        "acv_attention_mixed_dec_takes": [I, I, I, I, I],
        "acv_attention_mixed_tc": [P, I, P, I, P, P, P, P, I, P, P, I, P, P, P, I, P, I, I, I, I, I, I, F, I, P, F, P, I, P, I, I, P, I, P, P, P],
        "acv_add_normed_rmsnorm": [P, P, I, P, F, P, F, P, I, I, I, P],
        "acv_cast_rows_f32": [P, I, P, I, I, I, I, P],
        "acv_activation": [P, P, LL, I, F, F, I, P],
        "acv_rmsnorm_rows": [P, I, P, F, P, I, I, I, I, P],
        "acv_latent_prepare": [P, I, P, I, P, I, P, F, P, I, I, P, P, P, I, P, P, I, I, I, I, I, I, I, I, P],
        "acv_attention_latent_tc_takes": [I, I, I],
        "acv_attention_latent_tc": [P, I, P, I, P, P, P, I, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, I, P, P, P],
        "acv_gemm_tc_qkv": [P, I, P, I, P, I, I, I, I, I, I, I, P, LL, P, LL, P, I, I, I, I, I, I, P, P, F, P, I, P, P, P, I, P, P, P, I, I, P],
        "acv_gemm_tc": [P, I, P, I, P, I, I, I, I, I, I, I, I, I, P, LL, P, LL, P, I, I, I, P],
        "acv_gemm_tc_bias": [P, I, P, I, P, I, I, I, I, I, I, I, I, I, P, LL, P, LL, P, I, I, I, P, P],
        "acv_attention_decode": [P, I, P, I, P, P, P, P, I, P, P, I, P, I, I, I, I, I, F, I, I, I, P, P, P, LL, LL, LL, I, I, I, I, P, P, P],
        "acv_attention_tc": [P, I, I, P, I, P, P, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, I, I, P, I, P, P, P],
        "acv_attention_chunk": [P, I, P, I, P, P, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, I, I, I, P],
        "acv_table_update": [P, I, I, P, I, P],
        "acv_embed_scaled": [P, P, P, I, I, I, F, I, P],
        "acv_add_rmsnorm_f32": [P, P, P, P, P, I, I, F, I, P],
        "acv_scale_f32": [P, LL, F, P],
        "acv_heads_norm_append": [P, P, I, P, P, I, I, I, I, I, I, I, P, P, F, P, P, P, I, P, P, P, I, I, I, P],
        "acv_diff_combine": [P, I, I, P, I, I, I, I, F, F, F, I, P],
        "acv_diff_attention_generic": [P, I, P, I, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, I, F, F, F, I, P],
        "acv_moe_route": [P, I, P, P, P, I, I, I, I, I, I, I, P, P, P, I, I, I, F, P],
        "acv_moe_group": [P, I, I, I, I, P, P, P, P, P],
        "acv_moe_gather": [P, I, P, P, I, I, P, P, P, I, I, P],
        "acv_gemm_tc_grouped": [P, I, P, I, P, I, I, I, I, I, P, P, I, I, P, F, F, I, P, I, I, P],
        "acv_moe_gemm_simt": [P, I, P, LL, I, P, I, P, P, P, I, I, I, I, I, F, F, I, I, P],
        "acv_moe_gemm_mma": [P, I, P, LL, I, P, I, P, P, P, I, I, I, I, I, F, F, I, P],
        "acv_moe_combine": [P, I, I, P, I, P, I, P, P, I, I, I, I, P],
        "acv_glu": [P, I, P, I, I, I, I, F, F, I, I, P],
        "acv_gemm_tc_glu": [P, I, P, I, P, I, I, I, I, F, F, I, P, I, I, I, P],
        "acv_argmax": [P, I, I, I, P, P],
        "acv_apply_penalties": [P, I, I, P, P, P, I, P, P, P, P],
        "acv_sample": [P, I, I, I, P, P, P, P, P, P, P, P, P],
        "acv_top_logprobs": [P, I, I, I, I, P, P, P],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    lib.acv_set_pdl.argtypes = [c_int]
    lib.acv_set_pdl.restype = None
    lib.acv_decode_layer.argtypes = [ctypes.POINTER(DecodeLayerArgs), P]
    lib.acv_decode_layer.restype = c_int
    lib.acv_decode_layer_takes.argtypes = [I] * 8
    lib.acv_decode_layer_takes.restype = c_int
    lib.acv_attention_decode_resident.argtypes = [I] * 9
    lib.acv_attention_decode_resident.restype = c_int
    lib.acv_random_normal.argtypes = [P, LL, ctypes.c_ulonglong, F, F, P, P, I, P]
    lib.acv_random_normal.restype = c_int
    lib.acv_random_int.argtypes = [P, LL, ctypes.c_ulonglong, ctypes.c_uint, P]
    lib.acv_random_int.restype = c_int
    lib.acv_gemm_tc_test_fault.argtypes = [c_int, c_int]
    lib.acv_gemm_tc_test_fault.restype = None


class DecodeLayerArgs(ctypes.Structure):
    """The arguments of ``acv_decode_layer`` (csrc/decode_layer.cu, ``DlLayerArgs``), field for field."""
    _P, _I, _F, _LL = c_void_p, c_int, c_float, ctypes.c_longlong
    _fields_ = [
        ("T", _I), ("H", _I), ("I", _I), ("NH", _I), ("NKV", _I), ("D", _I),
        ("eps", _F), ("qk_eps", _F), ("scale", _F),
        ("x", _P), ("delta_in", _P), ("w_norm1", _P), ("w_norm2", _P),
        ("w_qkv", _P), ("w_o", _P), ("w_gu", _P), ("w_down", _P),
        ("q_norm", _P), ("k_norm", _P), ("cos_sin", _P), ("table_rows", _I),
        ("positions", _P), ("seq_of_token", _P), ("kv_len", _P),
        ("block_table", _P), ("bt_stride", _I), ("bt_rows", _P),
        ("k_pages", _P), ("v_pages", _P), ("page_size", _I), ("num_pages", _I),
        ("h", _P), ("qkv", _P), ("attn_out", _P), ("a_out", _P), ("act", _P), ("delta_out", _P),
        ("workspace", _P), ("workspace_floats", _LL), ("counters", _P), ("n_counters", _LL),
        ("part", _P), ("part_floats", _LL), ("att_counters", _P), ("n_att_counters", _LL),
        ("bars", _P), ("status", _P),
        ("sm_count", _I), ("max_kv", _I), ("trace", _P),
    ]


LAUNCHES = 0   # kernels of this package launched so far (library matrix products are not counted)


def _check(code: int, name: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code < 0:
        raise KernelError(f"{name}: {_ERRORS.get(code, f'refused with code {code}')}")
    raise KernelError(f"{name}: CUDA error {code} ({_cuda_error_text(code)})")


def _cuda_error_text(code: int) -> str:
    """The runtime's own words for a cudaError_t, asked of the library that the kernels are linked against."""
    try:
        fn = ctypes.CDLL("libcudart.so.12").cudaGetErrorString
        fn.restype = ctypes.c_char_p
        fn.argtypes = [ctypes.c_int]
        return fn(code).decode()
    except Exception:       # no such library name on this system: the number has to do
        return "see cudaError_t"


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not built (float32 and bfloat16 are)") from None


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("acvram_b200 kernels run on a CUDA device only; got a CPU tensor")


# ----------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]].  table [V, H]; tokens int32 [T]; out [T, H]."""
    _need_cuda(table, tokens, out)
    T, H = out.shape
    _check(library().acv_embed(_p(table), _p(tokens), _p(out), T, H, table.shape[0], dtype_code(table.dtype),
                               _stream()), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (in place, when delta is given); out = rmsnorm(x) * weight.

    With ``rows`` (int32 [R]) only those rows are normed, into out[0..R), and x is
    left as it is.  weight is float32 [H]."""
    _need_cuda(x, out, weight)
    n = out.shape[0] if rows is not None else x.shape[0]
    _check(library().acv_add_rmsnorm(_p(x), _p(delta), _p(weight), _p(out), _p(rows), n, x.shape[-1], eps,
                                     dtype_code(x.dtype), _stream()), "add_rmsnorm")
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[t, n] += bias[n] in place (bias float32 [N]; the sum in float, rounded once to out's type)."""
    _need_cuda(out, bias)
    if bias.dtype != torch.float32 or bias.numel() != out.shape[1] or out.stride(1) != 1:
        raise KernelError("add_bias: a float32 bias of the output's width is wanted")
    _check(library().acv_add_bias(_p(out), out.stride(0), _p(bias), out.shape[0], out.shape[1], dtype_code(out.dtype),
                                  _stream()), "add_bias")
    return out


def table_update(table: torch.Tensor, triples: torch.Tensor, n: int) -> None:
    """table[row, column] = page for the first ``n`` (row, column, page) triples of ``triples`` (int32, on the device)."""
    _need_cuda(table, triples)
    if table.dtype != torch.int32 or triples.dtype != torch.int32 or not table.is_contiguous() or triples.numel() < 3 * n:
        raise KernelError("table_update: a contiguous int32 table and 3 n int32 values are wanted")
    _check(library().acv_table_update(_p(table), table.shape[0], table.shape[1], _p(triples), n, _stream()), "table_update")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:].  gate_up [T, 2I] contiguous."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    _check(library().acv_swiglu(_p(gate_up), _p(out), T, I, dtype_code(out.dtype), _stream()), "swiglu")
    return out


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, t1: torch.Tensor, t2: torch.Tensor) -> torch.Tensor:
    """out (float32 or bfloat16, contiguous) = mean + std * z, z the normal deviates of the Philox stream keyed by
    ``key``; t1, t2: the quantile tables (weights/random_init.py).  Bit-equal to the host's arithmetic."""
    _need_cuda(out, t1, t2)
    if not out.is_contiguous() or t1.numel() != 1024 or t2.numel() != 1025:
        raise KernelError("random_normal: a contiguous output and tables of 1024 and 1025 floats are wanted")
    with torch.cuda.device(out.device):
        _check(library().acv_random_normal(_p(out), out.numel(), key, mean, std, _p(t1), _p(t2), dtype_code(out.dtype),
                                           _stream()), "random_normal")
    return out


def random_int(out: torch.Tensor, key: int, mask: int) -> torch.Tensor:
    """out (int32, contiguous) = words of the Philox stream keyed by ``key``, and-ed with ``mask``."""
    _need_cuda(out)
    with torch.cuda.device(out.device):
        _check(library().acv_random_int(_p(out), out.numel(), key, mask, _stream()), "random_int")
    return out


# ----------------------------------------------------------------------------- attention
def qk_norm_rope_append(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                        cos_sin: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                        block_table: torch.Tensor | None, k_pages: torch.Tensor | None,
                        v_pages: torch.Tensor | None, table_rows: torch.Tensor | None = None, value_dim: int = 0,
                        v_scale: float = 1.0) -> None:
    """Per-head norm, rotation and cache append over the stacked projection qkv [T, (NH+2NKV)*D], in place.

    cos_sin float32 [positions, R] (cos of R/2 angles, then sin); pages [NP, NKV, page, D].  ``table_rows``
    (int32 [requests], optional): the row of ``block_table`` of each request of the batch (default: its index).
    ``value_dim`` > 0: value rows of that size (the row is [NH*D | NKV*D | NKV*value_dim], value pages
    [NP, NKV, page, value_dim]); ``v_scale``: a constant on the values as they enter their pages."""
    _need_cuda(qkv)
    T = qkv.shape[0]
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    rows = cos_sin.shape[0] if cos_sin is not None else 0
    page = k_pages.shape[2] if k_pages is not None else 1
    n_pages = k_pages.shape[0] if k_pages is not None else 0
    bts = block_table.stride(0) if block_table is not None else 0
    _check(library().acv_qk_norm_rope_append(
        _p(qkv), qkv.stride(0), T, num_heads, num_kv_heads, head_dim, _p(q_weight), _p(k_weight), eps, _p(cos_sin),
        rot, rows, _p(positions), _p(seq_of_token), _p(block_table), bts, _p(table_rows), _p(k_pages), _p(v_pages), page, n_pages,
        dtype_code(qkv.dtype), int(value_dim), float(v_scale), _stream()), "qk_norm_rope_append")


def _head_vectors(num_heads: int, *vectors) -> None:
    for v in vectors:
        if v is not None and (v.dtype != torch.float32 or v.numel() != num_heads or not v.is_contiguous() or not v.is_cuda):
            raise KernelError("attention: sinks and slopes are contiguous float32 vectors with one number per query head")


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                      num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      table_rows: torch.Tensor | None = None, value_dim: int = 0, keep_first: int = 0,
                      sinks: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention for every token of the step.  q: rows of num_heads*head_dim (row stride free).
    ``value_dim`` > 0: value rows (and the result's heads) of that size; ``keep_first``: the first keys of a request
    that stay visible behind the window.  ``sinks`` (float32 [num_heads]): exp(sink_h) joins the softmax's denominator
    (a score with no key and no value); ``slopes`` (float32 [num_heads]): slope_h * (i - j) is taken off the score of
    query i and key j."""
    _need_cuda(q, out, k_pages)
    _head_vectors(num_heads, sinks, slopes)
    T = q.shape[0]
    _check(library().acv_attention_generic(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(positions), _p(seq_of_token),
        _p(block_table), block_table.stride(0), _p(table_rows), T, num_heads, num_kv_heads, head_dim, k_pages.shape[2],
        k_pages.shape[0], scale, window, dtype_code(q.dtype), int(value_dim), int(keep_first), _p(sinks), _p(slopes), _stream()),
           "attention_generic")
    return out


# ----------------------------------------------------------------------------- matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T with 32-bit accumulation on the CUDA cores."""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N or a.dtype != w.dtype:
        raise KernelError(f"gemm_simt: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_simt: innermost strides must be 1")
    _check(library().acv_gemm_simt(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), M, N, K,
                                   dtype_code(a.dtype), dtype_code(out.dtype), _stream()), "gemm_simt")
    return out


# ----------------------------------------------------------------------------- tensor-core matrix product (bfloat16)
_gemm_scratch: dict = {}


def _gemm_buffers(device, ws_floats: int, n_counters: int):
    key = str(device)
    have = _gemm_scratch.get(key)
    if have is None or have[0].numel() < ws_floats or have[1].numel() < n_counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("gemm_tc: workspace would grow during a graph capture; run the shape once first")
        old = have or (torch.empty(0), torch.empty(0), None)
        ws = torch.empty(max(ws_floats, 2 * old[0].numel(), 1 << 20), device=device, dtype=torch.float32)
        cnt = torch.zeros(max(n_counters, 2 * old[1].numel(), 4096), device=device, dtype=torch.int32)
        status = old[2] if old[2] is not None else torch.zeros(1, device=device, dtype=torch.int32)
        if key in _gemm_scratch:
            _retired.append(_gemm_scratch[key])
        have = (ws, cnt, status)
        _gemm_scratch[key] = have
    return have


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device; 148, a B200's, where there is no device)."""
    if not torch.cuda.is_available():
        return 148
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


# Split and pipeline depth of the products with few tokens (weight rows on the tensor core's M side), as measured
# on a B200 with layer sizes from 0.6B to 32B models: the first row that fits decides.  Splits of K are the CTAs
# of one cluster (summed through its shared memory).  Columns: tiles per SM from (inclusive) to (exclusive),
# k-blocks of 64 from to, tokens per tile (bn) from to (inclusive), then what to do: splits, stages.
#   many tiles: no split, several CTAs share an SM; few tiles: 2..4 splits fill the SMs
INF = float("inf")
GEMM_FEW_TOKENS_RULES = (
    (2.0,    INF,    0,   INF, 16, 128, 1, 8),
    (1.0,    2.0,    0,   INF, 16, 16,  2, 3),
    (1.0,    2.0,    0,   INF, 32, 128, 1, 4),
    (0.0,    1.0,    0,   16,  16, 128, 1, 8),
    (0.0,    1.0,    128, INF, 16, 32,  4, 8),
    (0.0,    1.0,    128, INF, 64, 128, 4, 6),
    (0.2501, 1.0,    16,  128, 16, 16,  4, 4),
    (0.0,    0.2501, 16,  128, 16, 16,  4, 6),
    (0.0,    0.2196, 16,  128, 32, 32,  4, 6),
    (0.2196, 1.0,    16,  128, 32, 32,  2, 6),
    (0.0,    1.0,    16,  128, 64, 128, 3, 6),
)


# Widths of a tile of the tokens-on-rows form, and what a tile costs beside its width, in columns' worth of time.
# Measured on a B200 (2048 x 4096 x 4096: 61 us in tiles of 256 columns, two rounds of the SMs of which the second is
# three quarters empty; 72 us in tiles of 160, three full rounds): a k-block of a tile costs about as much for the 128
# token rows it loads as for 120 of its columns, so a narrower tile pays only where it saves a whole round (1056 x 5120:
# 69 us at 256, 63 us at 160).  The width is chosen so that rounds x (width + overhead) comes out least.
GEMM_TILE_WIDTHS = (256, 224, 192, 160, 128)
GEMM_TILE_OVERHEAD = 120
# Pairs of CTAs on tiles of 256 tokens by 256 features (cta_group::2): a round of such tiles takes about 0.92 of a round
# of 128 x 256 tiles (measured at 2048 and 8192 tokens with the layer sizes of 8B and 14B models: 4 to 11 % less), and
# there are half as many places for them.
GEMM_PAIR_ROUND = 0.92
GEMM_PAIR = 4               # fifth element of a plan: the flag that asks for the pair kernel


def gemm_tc_plan(M: int, N: int, K: int, sms: int | None = None, bn_multiple: int = 16) -> tuple:
    """(swap, bn, splits, stages[, mode]) for x[M,K] @ w[N,K]^T on a device of ``sms`` multiprocessors.

    Up to 128 tokens the weight rows fill the tensor core's M = 128 and the tokens are the narrow
    side (weights stream once whatever the batch); splits of K are chosen so that the work items fill
    whole waves of the SMs (``GEMM_FEW_TOKENS_RULES``).  Above, tokens are the M side and a tile is 128
    tokens by 128..256 features: the width that needs the least rounds x width (``GEMM_TILE_WIDTHS``;
    ``bn_multiple``: widths that are multiples of this only, for an epilogue that wants whole heads),
    or, where that comes out cheaper, 256 x 256 on a pair of CTAs (``mode`` = ``GEMM_PAIR``)."""
    n_kb = -(-K // 64)
    if M <= 128:
        sms = sms or sm_count()
        bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        tiles = -(-N // 128) * -(-M // bn)
        per_sm = tiles / sms
        for t0, t1, k0, k1, b0, b1, splits, stages in GEMM_FEW_TOKENS_RULES:
            if t0 <= per_sm < t1 and k0 <= n_kb < k1 and b0 <= bn <= b1:
                return 1, bn, splits, stages
        return 1, bn, 1, 8
    if N < 256:
        return 0, (128 if N > 64 else 64), 1, 8
    sms = sms or sm_count()
    best, best_cost = 256, None
    for bn in GEMM_TILE_WIDTHS:
        if bn % bn_multiple:
            continue
        tiles = -(-M // 128) * -(-N // bn)
        cost = -(-tiles // sms) * (bn + GEMM_TILE_OVERHEAD)
        if best_cost is None or cost < 0.97 * best_cost:       # a narrower tile has to win clearly
            best, best_cost = bn, cost
    if sms >= 2 and 256 % bn_multiple == 0:
        pair_tiles = -(-M // 256) * -(-N // 256)
        if -(-pair_tiles // (sms // 2)) * (256 + GEMM_TILE_OVERHEAD) * GEMM_PAIR_ROUND < best_cost:
            return 0, 256, 1, 6, GEMM_PAIR
    return 0, best, 1, 8


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: tuple | None = None,
            swiglu_pairs: bool = False, static_weights: bool = False, bias: torch.Tensor | None = None,
            gate_fn: int = 0, unary: str | None = None) -> torch.Tensor:
    """out[M,N] = x[M,K] @ w[N,K]^T (+ bias) on tcgen05; x, w bfloat16, out bfloat16 or float32; ``bias`` float32 [N],
    added in the epilogue to the float accumulator (before the activation of the paired form).

    ``static_weights``: w was written long before this call (a model's weights), so the kernel may
    read its first tiles while the kernel before it in the stream is still running.

    With ``swiglu_pairs`` the rows of w come in (gate, up) pairs and out is [M, N/2]:
    out[:, i] = silu(x . w[2i]) * (x . w[2i+1]), rounded as the separate kernels round; with ``gate_fn`` 1 the gate
    passes through the tanh form of gelu instead (in float on the accumulators, the product rounded once).
    ``unary`` (not with ``swiglu_pairs``): an activation of ``ACTIVATIONS`` (not the first) on every output."""
    _need_cuda(x, w, out)
    if unary is not None and (swiglu_pairs or ACTIVATIONS.get(unary, 0) == 0):
        raise KernelError(f"gemm_tc: no activation '{unary}' in the epilogue (or asked for beside the paired form)")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc: operands must be bfloat16 and the output bfloat16 or float32")
    n_out = N // 2 if swiglu_pairs else N
    if swiglu_pairs and (N % 2 or out.dtype != torch.bfloat16):
        raise KernelError("gemm_tc: the paired SwiGLU output needs an even number of weight rows and a bfloat16 output")
    if w.shape[1] != K or out.shape != (M, n_out) or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_tc: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    plan = plan or gemm_tc_plan(M, N, K)
    swap, bn, splits = plan[:3]
    stages = plan[3] if len(plan) > 3 else 8
    cluster = plan[4] if len(plan) > 4 else (1 if swap and 1 < splits <= 8 else 0)
    tiles = (-(-N // 128) * -(-M // bn)) if swap else (-(-M // 128) * -(-N // bn))
    ws, cnt, status = _gemm_buffers(x.device, tiles * splits * bn * 128 if splits > 1 else 0, tiles)
    args = (_p(x), x.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), M, N, K,
            1 if out.dtype == torch.float32 else 0,
            (1 | (int(gate_fn) << 4)) if swiglu_pairs else ((ACTIVATIONS[unary] << 4) if unary else 0), swap, bn, splits, _p(ws),
            ws.numel(), _p(cnt),
            cnt.numel(), _p(status), sm_count(x.device), stages, cluster | (2 if static_weights else 0))
    if bias is not None:
        if bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous():
            raise KernelError("gemm_tc: the bias is a contiguous float32 vector with one entry for each row of the weight")
        _check(library().acv_gemm_tc_bias(*args, _p(bias), _stream()), "gemm_tc")
    else:
        _check(library().acv_gemm_tc(*args, _stream()), "gemm_tc")
    return out


def gemm_tc_qkv_takes(x: torch.Tensor, w: torch.Tensor, head_dim: int, cos_sin: torch.Tensor | None,
                      k_pages: torch.Tensor | None) -> bool:
    """Whether the stacked q,k,v projection of x can take its epilogue (norm, rotation, append) with it: bfloat16,
    heads of 64 or 128 rotated as a whole, and either up to 32 tokens with a plan that gives every CTA one tile
    (features on the tensor-memory lanes) or more than 128 tokens (tokens on the lanes, whole heads in a tile)."""
    if k_pages is None or x.dtype != torch.bfloat16 or head_dim not in (64, 128) or not gemm_tc_takes(x, w):
        return False
    if cos_sin is not None and (cos_sin.shape[1] != head_dim or cos_sin.dtype != torch.float32):
        return False
    M, K = x.shape
    N = w.shape[0]
    swap, bn, splits = gemm_tc_plan(M, N, K, bn_multiple=head_dim if M > 128 else 16)[:3]
    if not swap:            # tokens on M (one CTA or a pair to a tile): a thread of the epilogue holds whole heads of one token
        return splits == 1 and bn >= head_dim and bn % head_dim == 0
    tiles = -(-N // 128) * -(-M // bn)
    return bn <= 32 and (1 < splits <= 8 or (splits == 1 and tiles <= sm_count(x.device)))


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None,
                positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                v_pages: torch.Tensor, static_weights: bool = False, table_rows: torch.Tensor | None = None,
                plan: tuple | None = None) -> torch.Tensor:
    """The stacked q,k,v projection out[M, (NH+2NKV)*D] = x @ w^T with the epilogue of ``qk_norm_rope_append``
    inside the product's kernel: the query columns of out hold the normed, rotated queries, keys and values go
    to their pages (the key and value columns of out are not written).  ``gemm_tc_qkv_takes`` says when."""
    _need_cuda(x, w, out, k_pages, v_pages)
    M, K = x.shape
    N = w.shape[0]
    plan = plan or gemm_tc_plan(M, N, K, bn_multiple=head_dim if M > 128 else 16)
    swap, bn, splits, stages = plan[:4]
    cluster = plan[4] if len(plan) > 4 else (1 if swap and 1 < splits <= 8 else 0)
    tiles = (-(-N // 128) * -(-M // bn)) if swap else (-(-M // 128) * -(-N // bn))
    ws, cnt, status = _gemm_buffers(x.device, tiles * splits * bn * 128 if splits > 1 else 0, tiles)
    _check(library().acv_gemm_tc_qkv(
        _p(x), x.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), M, N, K, swap, bn, splits, _p(ws), ws.numel(),
        _p(cnt), cnt.numel(), _p(status), sm_count(x.device), stages, cluster | (2 if static_weights else 0), num_heads,
        num_kv_heads, head_dim, _p(q_weight), _p(k_weight), eps, _p(cos_sin),
        cos_sin.shape[0] if cos_sin is not None else 0, _p(positions), _p(seq_of_token), _p(block_table),
        block_table.stride(0), _p(table_rows), _p(k_pages), _p(v_pages), k_pages.shape[2], k_pages.shape[0], _stream()),
        "gemm_tc_qkv")
    return out


def gemm_tc_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel needs 16-byte aligned rows: K and the row strides multiples of 8."""
    return (x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(1) == 1)


def status_word(device) -> torch.Tensor:
    """The int32 word (on ``device``) into which the tensor-core kernels write a code when one of their bounded
    waits runs out (0 otherwise).  The engine copies it to the host with every step's tokens."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return _gemm_buffers(device, 0, 0)[2]


def reset_after_failure() -> None:
    """After a step whose kernels gave up a wait: the status word back to 0, and the arrival counters of the
    split products and of the split attention back to 0 (a CTA that gave up never arrived at its tile)."""
    for _, cnt, status in _gemm_scratch.values():
        status.zero_()
        cnt.zero_()
    for _, _, cnt in _scratch.values():
        cnt.zero_()
    for buf in _layer_scratch.values():
        buf["bars"].zero_()


def gemm_tc_test_fault(wait_limit: int, skip_k_block: int) -> None:
    """For the test of the bounded waits: the next tensor-core product of this process polls each barrier at most
    ``wait_limit`` times and never loads k-block ``skip_k_block``, so it gives up, frees what it holds, returns,
    and leaves the wait's code in the status word.  Nothing faults, traps or hangs."""
    library().acv_gemm_tc_test_fault(int(wait_limit), int(skip_k_block))


def gemm_status(device=None) -> int:
    """0, or the code a bounded wait inside a tensor-core product left when it ran out (synchronises)."""
    worst = 0
    for key, (_, _, status) in _gemm_scratch.items():
        worst = max(worst, int(status.item()))
    return worst


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = argmax(logits[r]) (lowest index among equals).  logits float32 [R, V]; out int32 [R]."""
    _need_cuda(logits, out)
    R, V = logits.shape
    _check(library().acv_argmax(_p(logits), logits.stride(0), R, V, _p(out), _stream()), "argmax")
    return out


def apply_penalties(logits: torch.Tensor, pen_row: torch.Tensor, pen_token: torch.Tensor, pen_count: torch.Tensor,
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> None:
    _need_cuda(logits, pen_row)
    _check(library().acv_apply_penalties(_p(logits), logits.stride(0), logits.shape[1], _p(pen_row), _p(pen_token),
                                         _p(pen_count), pen_row.numel(), _p(repetition), _p(presence),
                                         _p(frequency), _stream()), "apply_penalties")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seed: torch.Tensor, counter: torch.Tensor, out_token: torch.Tensor,
           out_logprob: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row.  seed, counter: int64 [R] (read as unsigned)."""
    _need_cuda(logits, out_token)
    R, V = logits.shape
    _check(library().acv_sample(_p(logits), logits.stride(0), R, V, _p(temperature), _p(top_k), _p(top_p), _p(min_p),
                                _p(seed), _p(counter), _p(out_token), _p(out_logprob), _stream()), "sample")
    return out_token


def top_logprobs(logits: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids int32 [R, k], log probabilities float32 [R, k]) of each row's k most probable tokens, most probable
    first (equal logits: the lower id first); log probability = logit - logsumexp(row).  1 <= k <= 64; where a row
    has fewer than k entries above -inf the rest is id -1 with -inf."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("top_logprobs: float32 rows wanted")
    R, V = logits.shape
    ids = torch.empty((R, k), device=logits.device, dtype=torch.int32)
    lp = torch.empty((R, k), device=logits.device, dtype=torch.float32)
    _check(library().acv_top_logprobs(_p(logits), logits.stride(0), R, V, k, _p(ids), _p(lp), _stream()), "top_logprobs")
    return ids, lp


# ----------------------------------------------------------------------------- tensor-core attention (bfloat16)
_scratch: dict = {}
_retired: list = []     # outgrown scratch buffers, never freed (graphs captured earlier point into them)


def _decode_scratch(device, floats: int, ml_floats: int, counters: int):
    """Scratch of the split-KV kernel, kept between calls and only ever grown (addresses that a
    captured graph holds stay valid as long as a warm-up call of the same shape came first)."""
    key = str(device)
    have = _scratch.get(key)
    if have is None or have[0].numel() < floats or have[1].numel() < ml_floats or have[2].numel() < counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("attention_decode: scratch would grow during a graph capture; run the shape once first")
        grow = lambda n, old: max(n, 2 * old)
        o = have or (torch.empty(0), torch.empty(0), torch.empty(0))
        have = (torch.empty(grow(floats, o[0].numel()), device=device, dtype=torch.float32),
                torch.empty(grow(ml_floats, o[1].numel()), device=device, dtype=torch.float32),
                torch.zeros(grow(counters, o[2].numel()), device=device, dtype=torch.int32))
        if key in _scratch:
            _retired.append(_scratch[key])   # a captured graph may still hold these addresses: keep them alive
        _scratch[key] = have
    return have


# What the choice of the number of splits reckons with: fitted to a sweep on a B200 over 1 to 64 requests, contexts of
# 1024 to 65536 keys (8 kv-heads of 128, 4 query heads each, pages of 64; launches that overlap as in a step, pages
# that no launch finds in L2) and every way of splitting below.  The reckoned time is within 11 % of the measured one
# (root mean square); the splits chosen took 2.7 % more time over the whole sweep than the best of each case (the rule
# before it, "CTAs for not quite twice the SMs": 9 %, and up to 60 % where clusters of 8 did not fit the device at once).
DECODE_KEY_US = 0.0117           # a CTA alone streams a key and its value in this time (its warps wait for their rings)
DECODE_KEY_US_ALONE = 0.00645    # the same where a CTA has an SM to itself and eight warps
DECODE_STREAM_BYTES_US = 6.45e6  # what all CTAs together stream from memory
DECODE_BOUNDS_NORM = 24.0        # a round takes the p-norm of the two times: with this p, the larger
DECODE_MERGE_US = (6.6, 8.0, 0.45, 8.5, 0.81)   # start to end without splits; merged inside a cluster + per split;
                                                # through scratch memory + per split
DECODE_SPLIT_KEYS = 256          # no split shorter than this
DECODE_CLUSTER_SPLITS = (2, 4, 6, 8)       # 3 and 5 were never better than their even neighbours by more than 2 %
DECODE_SCRATCH_SPLITS = (2, 4, 8, 12, 16, 24, 32)
DECODE_WIDE_CLUSTER_FIT = 0.85   # of the clusters of more than 6 CTAs that the runtime says fit at once, this part did
# Inside a step the kernel's end is what the next kernel waits for, and there shorter CTAs won where the sweep saw a tie
# (8 requests of 2100 keys: 4 splits 3.716 ms a step, 2 splits 3.743, none 3.821).  Among the ways that the reckoning
# puts within this factor of the cheapest, the one with the most splits is taken if it merges in clusters and its CTAs
# all fit the device at once.
DECODE_MORE_SPLITS_WITHIN = 1.05


@functools.lru_cache(maxsize=None)
def decode_resident(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, n_splits: int,
                    pages_of_split: int, cluster_merge: bool, alone: bool = False) -> int:
    """How many CTAs of the split-KV kernel the device holds at once (asked of the runtime: a cluster needs its CTAs
    side by side in one part of the chip).  ``alone``: how many it holds one to an SM; a grid of no more CTAs runs with
    eight warps to a CTA instead of four (0: that form does not fit these sizes)."""
    n = library().acv_attention_decode_resident(num_heads, num_kv_heads, head_dim, page_size, 0, n_splits,
                                                pages_of_split * page_size * n_splits, 1 if cluster_merge else 0,
                                                1 if alone else 0)
    if n < 0:
        raise KernelError(f"attention_decode_resident: {_ERRORS.get(n, f'refused with code {n}')}")
    return n if alone else max(1, n)


def decode_splits_cost(n_dec: int, num_kv_heads: int, max_kv: int, n_splits: int, cluster_merge: bool, resident: int,
                       row_bytes: int, resident_alone: int = 0) -> float:
    """Reckoned microseconds of the split-KV kernel: the CTAs run in rounds of ``resident``; a round takes as long as
    one CTA needs for its keys alone, or as the memory needs for the round's bytes; then the merge.  A grid of up to
    ``resident_alone`` CTAs has an SM for each, eight warps to a CTA, and streams faster."""
    ctas = n_dec * num_kv_heads * n_splits
    keys = -(-max_kv // n_splits)
    alone = keys * (DECODE_KEY_US_ALONE if ctas <= resident_alone else DECODE_KEY_US)
    p = DECODE_BOUNDS_NORM
    round_us = lambda n: (alone ** p + (n * keys * row_bytes / DECODE_STREAM_BYTES_US) ** p) ** (1.0 / p)
    full, rest = divmod(ctas, resident)
    us = full * round_us(resident) + (round_us(rest) if rest else 0.0)
    if n_splits == 1:
        return us + DECODE_MERGE_US[0]
    if cluster_merge:
        return us + DECODE_MERGE_US[1] + DECODE_MERGE_US[2] * n_splits
    return us + DECODE_MERGE_US[3] + DECODE_MERGE_US[4] * n_splits


def decode_ways(n_dec: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, keys: int) -> list:
    """Every way of splitting ``keys`` keys of ``n_dec`` requests that the plan chooses from, as (reckoned microseconds,
    splits, merged inside clusters?, all CTAs fit the device at once?)."""
    row_bytes = 2 * head_dim * 2                       # a key and a value of one kv-head in bfloat16
    ways = []
    for n_splits, cluster in [(1, False)] + [(s, True) for s in DECODE_CLUSTER_SPLITS] + \
                             [(s, False) for s in DECODE_SCRATCH_SPLITS]:
        if n_splits > 1 and keys < n_splits * DECODE_SPLIT_KEYS:
            continue
        if n_dec * num_kv_heads * n_splits > 65535 * 4:
            continue
        pages = -(-(-(-keys // n_splits)) // page_size)
        pages = 1 << max(0, pages - 1).bit_length()
        resident = decode_resident(num_heads, num_kv_heads, head_dim, page_size, n_splits, pages, cluster)
        alone = decode_resident(num_heads, num_kv_heads, head_dim, page_size, n_splits, pages, cluster, True)
        if cluster and n_splits > 6:
            resident = max(n_splits, int(resident * DECODE_WIDE_CLUSTER_FIT))
            alone = min(alone, resident)
        resident = max(resident, alone)
        cost = decode_splits_cost(n_dec, num_kv_heads, keys, n_splits, cluster, resident, row_bytes, alone)
        ways.append((cost, n_splits, cluster, n_dec * num_kv_heads * n_splits <= resident))
    return ways


@functools.lru_cache(maxsize=4096)
def decode_plan(n_dec: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, max_kv: int,
                window: int = 0) -> tuple[int, bool]:
    """(splits of the context, merged inside clusters?) for ``n_dec`` one-token requests with up to ``max_kv`` keys:
    by ``decode_splits_cost`` among no split, up to 8 splits merged inside a cluster and up to 32 merged through
    scratch memory.  A split more pays while it shortens what a CTA streams alone; it stops paying when the CTAs no
    longer fit the device at once or the memory is the limit anyway."""
    keys = min(max_kv, window) if window > 0 else max_kv
    ways = decode_ways(n_dec, num_heads, num_kv_heads, head_dim, page_size, keys)
    cheapest = min(ways)
    near = [w for w in ways if w is cheapest or (w[0] <= DECODE_MORE_SPLITS_WITHIN * cheapest[0] and w[2] and w[3])]
    best = max(near, key=lambda w: w[1])
    return best[1], best[2]


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     dec_tokens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int, kv_len: torch.Tensor,
                     block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                     window: int, n_splits: int, max_kv: int = 0, cluster_merge: bool = True,
                     table_rows: torch.Tensor | None = None, chunk: int = 0, keep_first: int = 0,
                     sinks: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of requests that bring one token each, over their pages, split over the context.
    ``sinks``, ``slopes`` (float32 [heads]): as in ``attention_generic``; the sink joins once, where the splits merge.

    Up to 8 splits are merged inside a thread-block cluster (through its shared memory); more, or
    ``cluster_merge=False``, go through partial results in scratch memory and a last-arriver merge."""
    n_rep = num_heads // num_kv_heads
    _head_vectors(num_heads, sinks, slopes)
    use_cluster = cluster_merge and 1 < n_splits <= 8
    parts = n_dec * num_kv_heads * n_splits if n_splits > 1 and not use_cluster else 0
    acc, ml, cnt = _decode_scratch(q.device, parts * n_rep * head_dim, parts * n_rep * 2, n_dec * num_kv_heads)
    _check(library().acv_attention_decode(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(dec_tokens), _p(dec_seqs), n_dec,
        _p(kv_len), _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads, head_dim,
        k_pages.shape[2], k_pages.shape[0], scale, window, chunk, n_splits, _p(acc), _p(ml), _p(cnt), acc.numel(), ml.numel(), cnt.numel(),
        max_kv or block_table.shape[1] * k_pages.shape[2], 1 if use_cluster else 0,
        1 if out.dtype == torch.float32 else 0, int(keep_first), _p(sinks), _p(slopes), _stream()), "attention_decode")
    return out


def attention_chunk(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor,
                    kv_len: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int, table_rows: torch.Tensor | None = None, max_kv: int = 0,
                    chunk: int = 0) -> torch.Tensor:
    """Causal attention of portions of prompts (tiles of QUERY_TILE query tokens) over their requests' pages."""
    _check(library().acv_attention_chunk(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(tile_seq), _p(tile_q0), n_tiles,
        _p(cu_q), _p(kv_len), _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads, head_dim,
        k_pages.shape[2], k_pages.shape[0], scale, window, chunk, 1 if out.dtype == torch.float32 else 0,
        max_kv or block_table.shape[1] * k_pages.shape[2], _stream()), "attention_chunk")
    return out


def attention_tc(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor, kv_len: torch.Tensor,
                 block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 window: int, table_rows: torch.Tensor | None = None, chunk: int = 0, keep_first: int = 0,
                 sinks: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of portions of prompts on tcgen05 (tiles of QUERY_TILE query tokens, pages by TMA).
    ``sinks``, ``slopes`` (float32 [heads]): as in ``attention_generic``."""
    _head_vectors(num_heads, sinks, slopes)
    _, _, status = _gemm_buffers(q.device, 0, 0)
    _check(library().acv_attention_tc(
        _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(tile_seq), _p(tile_q0),
        n_tiles, _p(cu_q), _p(kv_len), _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads,
        head_dim, k_pages.shape[2], k_pages.shape[0], scale, window, chunk, 1 if out.dtype == torch.float32 else 0, _p(status),
        int(keep_first), _p(sinks), _p(slopes), _stream()), "attention_tc")
    return out


def attention_tc_takes(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, head_dim: int) -> bool:
    page = k_pages.shape[2]
    # (out may be float32 beside bfloat16 queries: the kernels then leave their result unrounded)
    return (head_dim in (64, 128) and page in (8, 16, 32, 64, 128) and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and k_pages.is_contiguous())


def tensor_core_attention_takes(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads // num_kv_heads <= 16


# ----------------------------------------------------------------------------- dispatch by shape
QUERY_TILE = 128   # query tokens per tile of the portion-attention kernels (AT_BM of attention_tc.cu)


def attention_work(q_lens, kv_lens, cu_q) -> tuple[dict, dict]:
    """Work lists of the attention kernels for a step: the requests with one token (decoding) and tiles of
    QUERY_TILE tokens of the requests with more (portions of prompts), late tiles first since they see most keys.
    Returns (int32 arrays that the kernels read on the device, counts and maxima for the launches)."""
    import numpy as np
    ql = np.asarray(q_lens, dtype=np.int32)
    dec = np.nonzero(ql == 1)[0].astype(np.int32)
    tile_seq, tile_q0, tile_keys = [], [], []
    for i in np.nonzero(ql > 1)[0]:
        starts_i = np.arange(0, q_lens[i], QUERY_TILE, dtype=np.int32)
        tile_seq.append(np.full(starts_i.size, i, dtype=np.int32))
        tile_q0.append(starts_i)
        tile_keys.append(int(kv_lens[i]) - int(q_lens[i]) + np.minimum(starts_i + QUERY_TILE, int(q_lens[i])))   # keys a tile's last query sees
    empty = np.zeros(0, np.int32)
    if tile_seq:
        # the tiles with most keys first, over all requests: the hardware hands out CTAs in this order, and the kernel
        # that gives a CTA two tiles pairs the list's front with its back
        order = np.argsort(-np.concatenate(tile_keys), kind="stable")
        tile_seq, tile_q0 = [np.concatenate(tile_seq)[order]], [np.concatenate(tile_q0)[order]]
    arrays = {"dec_tokens": np.asarray(cu_q, dtype=np.int32)[:-1][dec], "dec_seqs": dec,
              "tile_seq": np.concatenate(tile_seq) if tile_seq else empty,
              "tile_q0": np.concatenate(tile_q0) if tile_q0 else empty}
    values = {"n_dec": int(dec.size), "n_tiles": int(sum(t.size for t in tile_seq)),
              "max_dec_kv": max((k for k, q in zip(kv_lens, q_lens) if q == 1), default=0),
              "max_tile_kv": max((k for k, q in zip(kv_lens, q_lens) if q > 1), default=0)}
    return arrays, values


def attention_work_decode(padded: int, max_kv: int) -> tuple[dict, dict]:
    """The same for a batch of ``padded`` requests with one token each, made for contexts up to ``max_kv``."""
    import numpy as np
    ar = np.arange(padded, dtype=np.int32)
    return ({"dec_tokens": ar, "dec_seqs": ar, "tile_seq": np.zeros(0, np.int32), "tile_q0": np.zeros(0, np.int32)},
            {"n_dec": padded, "n_tiles": 0, "max_dec_kv": max_kv, "max_tile_kv": 0})


def attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx,
              block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0, work: dict | None = None, chunk: int = 0, value_dim: int = 0,
              keep_first: int = 0, sinks: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's pages.  A query sees the keys at or before its
    position; with ``window`` > 0 the last ``window`` of them, and with ``keep_first`` > 0 also the first
    ``keep_first`` keys of the request; with ``chunk`` > 0 those of its own chunk of ``chunk``
    positions counted from the request's position 0.  ``value_dim``: the size of a value row where it is not ``head_dim``.
    ``sinks`` (float32 [heads]): exp(sink_h) joins the softmax's denominator; ``slopes`` (float32 [heads]): the score of
    query i and key j loses slope_h (i - j).

    ``qkv`` is the stacked projection after norm and rotation (queries are its first
    num_heads*head_dim columns); ``ctx`` is the step's StepContext; ``work`` the step's work lists
    (``attention_work``; default: ``ctx.work``).  bfloat16 with a head size of 64 or 128 goes to the
    tensor-core kernels, requests with one token to the split-KV kernel and portions to the tiled
    one; everything else to the generic kernel."""
    rows = getattr(ctx, "table_rows", None)
    value_dim = value_dim or head_dim
    keep_first = keep_first if window > 0 else 0
    w = work if work is not None else ctx.work
    generic = value_dim != head_dim or not tensor_core_attention_takes(qkv.dtype, num_heads, num_kv_heads, head_dim)
    # the tensor-core kernels read queries in 16-byte pieces: a view into a wider projection whose rows or start are not
    # aligned so (a mixer beside another one, with sizes that are multiples of nothing) takes the generic kernel
    if not generic and (qkv.stride(0) % 8 or qkv.data_ptr() % 16):
        generic = True
    # kept first keys: the split-KV decode kernel and the tcgen05 portion kernel know them, the mma.sync portion kernel does not
    if not generic and keep_first > 0 and (chunk > 0 or (w["n_tiles"] and not attention_tc_takes(qkv, out, k_pages, head_dim))):
        generic = True
    # sinks and slopes: the generic, the split-KV and the tcgen05 portion kernel know them, the mma.sync portion kernel does not
    if not generic and (sinks is not None or slopes is not None) and (chunk > 0 or (
            w["n_tiles"] and not attention_tc_takes(qkv, out, k_pages, head_dim))):
        generic = True
    if generic:
        if chunk > 0:
            raise KernelError("attention: the chunked mask is built for the tensor-core kernels' sizes only")
        return attention_generic(qkv, out, k_pages, v_pages, ctx.positions, ctx.seq_of_token, block_table, num_heads,
                                 num_kv_heads, head_dim, scale, window, table_rows=rows, value_dim=value_dim,
                                 keep_first=keep_first, sinks=sinks, slopes=slopes)
    if w["n_dec"]:
        kv = min(w["max_dec_kv"], window + keep_first) if window > 0 else w["max_dec_kv"]
        kv = min(kv, chunk) if chunk > 0 else kv
        n_splits, in_clusters = (w["n_splits"], True) if w.get("n_splits") else \
            decode_plan(w["n_dec"], num_heads, num_kv_heads, head_dim, k_pages.shape[2], kv)
        attention_decode(qkv, out, k_pages, v_pages, w["dec_tokens"], w["dec_seqs"], w["n_dec"], ctx.kv_len,
                         block_table, num_heads, num_kv_heads, head_dim, scale, window, n_splits, w["max_dec_kv"],
                         cluster_merge=in_clusters, table_rows=rows, chunk=chunk, keep_first=keep_first, sinks=sinks,
                         slopes=slopes)
    if w["n_tiles"] and attention_tc_takes(qkv, out, k_pages, head_dim):
        attention_tc(qkv, out, k_pages, v_pages, w["tile_seq"], w["tile_q0"], w["n_tiles"], ctx.cu_q, ctx.kv_len,
                     block_table, num_heads, num_kv_heads, head_dim, scale, window, table_rows=rows, chunk=chunk,
                     keep_first=keep_first, sinks=sinks, slopes=slopes)
    elif w["n_tiles"]:
        attention_chunk(qkv, out, k_pages, v_pages, w["tile_seq"], w["tile_q0"], w["n_tiles"], ctx.cu_q, ctx.kv_len,
                        block_table, num_heads, num_kv_heads, head_dim, scale, window, table_rows=rows,
                        max_kv=w.get("max_tile_kv", 0), chunk=chunk)
    return out


# ----------------------------------------------------------------------------- one decoder layer of a decode step
DECODE_LAYER_TOKENS = 16     # DL_BN of decode_layer.cu
DECODE_LAYER_TRACE: torch.Tensor | None = None   # int64 [SMs, 8] on the device: every fused layer leaves its phase stamps there
_layer_scratch: dict = {}


def decode_layer_takes(T: int, H: int, I: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                       window: int) -> bool:
    """Whether the fused decode-layer kernel runs a layer of these sizes for a step of ``T`` one-token requests."""
    return bool(library().acv_decode_layer_takes(T, H, I, num_heads, num_kv_heads, head_dim, page_size, window))


def _layer_buffers(device, H: int, I: int, qkv_width: int, q_width: int):
    """Activations of one layer (16 rows each) and the grid barriers, kept between calls (layers run one after the
    other on one stream, and a captured graph holds the addresses)."""
    key = (str(device), H, I, qkv_width, q_width)
    have = _layer_scratch.get(key)
    if have is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("decode_layer: its buffers would be made during a graph capture; run the shape once first")
        n = DECODE_LAYER_TOKENS
        mk = lambda w: torch.zeros((n, w), device=device, dtype=torch.bfloat16)
        have = {"h": mk(H), "qkv": mk(qkv_width), "attn": mk(q_width), "a": mk(H), "act": mk(I),
                "bars": torch.zeros(8, device=device, dtype=torch.int32)}
        _layer_scratch[key] = have
    return have


def decode_layer(x: torch.Tensor, delta: torch.Tensor | None, delta_out: torch.Tensor, norm1_w: torch.Tensor,
                 norm2_w: torch.Tensor, eps: float, w_qkv: torch.Tensor, w_o: torch.Tensor, w_gate_up_pairs: torch.Tensor,
                 w_down: torch.Tensor, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, qk_eps: float,
                 cos_sin: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 positions: torch.Tensor, seq_of_token: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor,
                 table_rows: torch.Tensor | None, k_pages: torch.Tensor, v_pages: torch.Tensor, max_kv: int,
                 trace: torch.Tensor | None = None) -> torch.Tensor:
    """A whole pre-norm decoder layer for a step of up to 16 one-token requests in one persistent kernel
    (csrc/decode_layer.cu): x += delta; a = attention(norm1(x)); x += a; delta_out = swiglu_mlp(norm2(x)).
    ``x`` [T, H] is updated in place, ``delta_out`` [T, H] receives what the next layer adds; the keys and values of
    the step's tokens go to their pages.  ``w_gate_up_pairs``: rows (gate_i, up_i) interleaved, as the fused SwiGLU
    product takes them.  ``decode_layer_takes`` says for which sizes.  ``trace`` (int64 [SMs, 8], optional): each CTA
    leaves the device-wide nanosecond time at which it began and at which it finished each phase (norm, q/k/v,
    attention, output product, norm, gate/up, down)."""
    _need_cuda(x, delta_out, w_qkv, k_pages)
    T, H = x.shape
    I = w_down.shape[1]
    qkv_width, q_width = w_qkv.shape[0], num_heads * head_dim
    buf = _layer_buffers(x.device, H, I, qkv_width, q_width)
    n_rep = num_heads // num_kv_heads
    sms = sm_count(x.device)
    tiles = [-(-n // 128) for n in (qkv_width, H, 2 * I, H)]
    ws, cnt, status = _gemm_buffers(x.device, max(tiles) * 16 * 16 * 128, sum(tiles))
    part, _, att_cnt = _decode_scratch(x.device, sms * n_rep * (head_dim + 2), 0, DECODE_LAYER_TOKENS * num_kv_heads)
    a = DecodeLayerArgs(
        T=T, H=H, I=I, NH=num_heads, NKV=num_kv_heads, D=head_dim, eps=eps, qk_eps=qk_eps, scale=scale,
        x=_p(x), delta_in=_p(delta), w_norm1=_p(norm1_w), w_norm2=_p(norm2_w), w_qkv=_p(w_qkv), w_o=_p(w_o),
        w_gu=_p(w_gate_up_pairs), w_down=_p(w_down), q_norm=_p(q_norm), k_norm=_p(k_norm), cos_sin=_p(cos_sin),
        table_rows=cos_sin.shape[0] if cos_sin is not None else 0, positions=_p(positions), seq_of_token=_p(seq_of_token),
        kv_len=_p(kv_len), block_table=_p(block_table), bt_stride=block_table.stride(0), bt_rows=_p(table_rows),
        k_pages=_p(k_pages), v_pages=_p(v_pages), page_size=k_pages.shape[2], num_pages=k_pages.shape[0],
        h=_p(buf["h"]), qkv=_p(buf["qkv"]), attn_out=_p(buf["attn"]), a_out=_p(buf["a"]), act=_p(buf["act"]),
        delta_out=_p(delta_out), workspace=_p(ws), workspace_floats=ws.numel(), counters=_p(cnt), n_counters=cnt.numel(),
        part=_p(part), part_floats=part.numel(), att_counters=_p(att_cnt), n_att_counters=att_cnt.numel(),
        bars=_p(buf["bars"]), status=_p(status), sm_count=sms, max_kv=max(1, max_kv),
        trace=_p(trace if trace is not None else DECODE_LAYER_TRACE))
    _check(library().acv_decode_layer(ctypes.byref(a), _stream()), "decode_layer")
    return delta_out


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, static_weights: bool = False,
                bias: torch.Tensor | None = None, unary: str | None = None) -> torch.Tensor:
    """out = x @ w^T (+ bias) in bfloat16 with float accumulation: the tcgen05 kernel, the bias in its epilogue; rows
    that are not 16-byte aligned (K or a stride no multiple of 8) go to the library product, as all do in the
    reference, and a kernel of its own adds the bias.  ``unary`` (a name of ``ACTIVATIONS`` other than the first): that
    activation of every output, in the product's epilogue on the float accumulators (or by a kernel of its own behind
    the library product)."""
    if gemm_tc_takes(x, w):
        return gemm_tc(x, w, out, static_weights=static_weights, bias=bias, unary=unary)
    torch.mm(x, w.t(), out=out)
    if bias is not None:
        add_bias(out, bias)
    return activation(out, out, unary) if unary else out


def linear_bf16_swiglu(x: torch.Tensor, w_pairs: torch.Tensor, out: torch.Tensor,
                       static_weights: bool = False, bias: torch.Tensor | None = None, act: int = 1) -> torch.Tensor:
    """out[M, I] = silu(x @ Wg^T + bg) * (x @ Wu^T + bu) in one kernel; w_pairs [2I, K] holds (gate_i, up_i) in rows
    2i, 2i+1, and ``bias`` (float32 [2I]) their biases in the same order.  ``act``: a code of ``GATED_EPILOGUE_ACTS``
    (1: silu; 2: the tanh form of gelu on the gate)."""
    return gemm_tc(x, w_pairs, out, swiglu_pairs=True, static_weights=static_weights, bias=bias, gate_fn=act - 1)


def linear_bf16_f32out(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, static_weights: bool = False,
                       bias: torch.Tensor | None = None) -> torch.Tensor:
    """out (float32) = x @ w^T (+ bias) from bfloat16 operands, accumulated in float32."""
    if gemm_tc_takes(x, w):
        return gemm_tc(x, w, out, static_weights=static_weights, bias=bias)
    gemm_simt(x, w, out)
    return add_bias(out, bias) if bias is not None else out


# ----------------------------------------------------------------------------- a residual stream kept in float
def embed_scaled(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale, out float32 [T, H] whatever the table's type."""
    _need_cuda(table, tokens, out)
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed_scaled: a contiguous float32 output and a contiguous table are wanted")
    T, H = out.shape
    _check(library().acv_embed_scaled(_p(table), _p(tokens), _p(out), T, H, table.shape[0], scale, dtype_code(table.dtype),
                                      _stream()), "embed_scaled")
    return out


def add_rmsnorm_f32(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                    rows: torch.Tensor | None = None) -> torch.Tensor:
    """The float32 stream x += delta (of out's type; in place, unless ``rows``); out = x / sqrt(mean(x^2) + eps) * weight,
    computed in float32 and rounded once to out's type."""
    _need_cuda(x, out, weight)
    if x.dtype != torch.float32 or (delta is not None and delta.dtype != out.dtype) or not x.is_contiguous() \
            or not out.is_contiguous() or (delta is not None and not delta.is_contiguous()):
        raise KernelError("add_rmsnorm_f32: a contiguous float32 stream and a delta of the output's type are wanted")
    n = out.shape[0] if rows is not None else x.shape[0]
    _check(library().acv_add_rmsnorm_f32(_p(x), _p(delta), _p(weight), _p(out), _p(rows), n, x.shape[-1], eps,
                                         dtype_code(out.dtype), _stream()), "add_rmsnorm_f32")
    return out


def scale_f32(x: torch.Tensor, s: float) -> torch.Tensor:
    """x *= s in place (float32, contiguous)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_f32: a contiguous float32 tensor is wanted")
    _check(library().acv_scale_f32(_p(x), x.numel(), s, _stream()), "scale_f32")
    return x


# ----------------------------------------------------------------------------- differential attention
def heads_norm_append(qkv: torch.Tensor, num_q_vectors: int, num_k_vectors: int, num_kv_heads: int, dim: int, value_dim: int,
                      q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, positions: torch.Tensor,
                      seq_of_token: torch.Tensor, block_table: torch.Tensor | None, k_pages: torch.Tensor | None,
                      v_pages: torch.Tensor | None, table_rows: torch.Tensor | None = None,
                      q_out: torch.Tensor | None = None) -> None:
    """RMS norm of each of the ``num_q_vectors`` query vectors of ``dim`` elements at the head of a row of ``qkv``
    (in place) and, when pages are given, of the ``num_k_vectors`` key vectors behind them (written into the key
    pages, ``num_k_vectors / num_kv_heads`` vectors to a key row) and the copy of the ``num_kv_heads`` value rows of
    ``value_dim`` elements behind those into the value pages.  Without pages the row holds queries only.
    ``q_out`` [T, num_q_vectors * key row]: the normed query vectors go there instead, each as a row as long as a key
    row with the vector at its map's offset and zeros elsewhere (queries for kernels that know one vector per head)."""
    _need_cuda(qkv)
    T = qkv.shape[0]
    keeps = k_pages is not None
    q_width = num_q_vectors * dim
    k = qkv[:, q_width:] if keeps else None
    v = qkv[:, q_width + num_k_vectors * dim:] if keeps else None
    _check(library().acv_heads_norm_append(
        _p(qkv), _p(q_out), q_out.stride(0) if q_out is not None else 0, _p(k), _p(v), qkv.stride(0), T, num_q_vectors, num_k_vectors, num_kv_heads, dim, value_dim,
        _p(q_weight), _p(k_weight), eps, _p(positions), _p(seq_of_token), _p(block_table),
        block_table.stride(0) if block_table is not None else 0, _p(table_rows), _p(k_pages), _p(v_pages),
        k_pages.shape[2] if keeps else 1, k_pages.shape[0] if keeps else 0, dtype_code(qkv.dtype), _stream()),
        "heads_norm_append")


def diff_attention_generic(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                           num_kv_heads: int, dim: int, value_dim: int, scale: float, lam: float, eps: float,
                           out_scale: float, window: int = 0, chunk: int = 0,
                           table_rows: torch.Tensor | None = None) -> torch.Tensor:
    """Differential attention of every token of the step: q rows hold ``num_heads`` pairs of query vectors, key pages
    [pages, kv_heads, page, 2 * dim], value pages [pages, kv_heads, page, value_dim]; out rows ``num_heads * value_dim``."""
    _need_cuda(q, out, k_pages, v_pages)
    _check(library().acv_diff_attention_generic(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(positions), _p(seq_of_token),
        _p(block_table), block_table.stride(0), _p(table_rows), q.shape[0], num_heads, num_kv_heads, dim, value_dim,
        k_pages.shape[2], k_pages.shape[0], scale, window, chunk, lam, eps, out_scale, dtype_code(q.dtype), _stream()),
        "diff_attention_generic")
    return out


def diff_attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx,
                   block_table: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, value_dim: int, scale: float,
                   lam: float, eps: float, out_scale: float, window: int = 0, chunk: int = 0,
                   work: dict | None = None) -> torch.Tensor:
    """Differential attention of every token of the step over its request's pages (queries: the first
    ``num_heads * 2 * dim`` columns of ``qkv``, after their norm); dispatch by shape."""
    rows = getattr(ctx, "table_rows", None)
    return diff_attention_generic(qkv, out, k_pages, v_pages, ctx.positions, ctx.seq_of_token, block_table, num_heads,
                                  num_kv_heads, dim, value_dim, scale, lam, eps, out_scale, window, chunk, table_rows=rows)


def diff_attention_as_heads_takes(dtype: torch.dtype, num_heads: int, num_kv_heads: int, dim: int, value_dim: int) -> bool:
    """Whether the two maps can run as twice as many heads of the tensor-core attention kernels: key rows and value
    rows of one size that those kernels take (each map's query padded with zeros to a key row)."""
    return value_dim == 2 * dim and tensor_core_attention_takes(dtype, 2 * num_heads, num_kv_heads, 2 * dim)


def diff_combine(maps: torch.Tensor, out: torch.Tensor, num_heads: int, value_dim: int, lam: float, eps: float,
                 out_scale: float) -> torch.Tensor:
    """out[t, h] = unit_rms(maps[t, 2h] - lam * maps[t, 2h + 1]) * out_scale over the head's ``value_dim`` values."""
    _need_cuda(maps, out)
    _check(library().acv_diff_combine(_p(maps), maps.stride(0), 1 if maps.dtype == torch.float32 else 0, _p(out), out.stride(0), maps.shape[0], num_heads, value_dim,
                                      lam, eps, out_scale, dtype_code(out.dtype), _stream()), "diff_combine")
    return out


# ----------------------------------------------------------------------------- mixture of experts
MOE_TILE = 64               # rows of a tile of the grouped products (MOE_TILE of csrc/moe.cu)
GLU_SWISH_CLAMPED = 0       # g = min(a, limit), u = clamp(b, +-limit): g * sigmoid(alpha g) * (u + 1)


MOE_TC_TILE = 128           # rows of a tile of the grouped tcgen05 product (GT_BM of csrc/gemm_epilogue.cuh)
MOE_TC_ROWS = 1024          # from this many (token, choice) rows on, aligned bfloat16 steps group for the tcgen05 product,
MOE_TC_ROWS_PER_EXPERT = 32  # if an expert gets this many on average (tiles of 128 rows would else be nearly empty)


def moe_max_tiles(rows: int, experts: int, tile: int = MOE_TILE) -> int:
    """Tiles that ``rows`` (token, choice) rows can need at most, whatever the routing: every expert may leave one
    tile partly filled."""
    return -(-rows // tile) + experts


def moe_route(h: torch.Tensor, w_router: torch.Tensor | None, gate_w: torch.Tensor | None, top: int, softmax: bool, renorm: bool,
              ids: torch.Tensor, weights: torch.Tensor, gate: torch.Tensor | None, logits: torch.Tensor | None = None,
              experts: int | None = None, groups: tuple[int, int] | None = None, renorm_eps: float = 0.0) -> None:
    """Router of a mixture of experts, in 32-bit: ids, weights [T, top] (int32, float32); gate [T] = sigmoid(h . gate_w).
    With ``logits`` (float32 [T, >= experts (+ 1)]: the router's columns, then the gate's) the products were made before
    and only the scores and the choice are made here.  ``groups`` = (count, keep): the experts stand in ``count`` equal
    groups of neighbours, a group is worth its best score, and only experts of the ``keep`` best groups can be chosen.
    ``renorm_eps`` joins the sum that the chosen scores are divided by."""
    _need_cuda(h, ids, weights)
    T, H = h.shape
    n_groups, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
    if logits is not None:
        if logits.dtype != torch.float32 or logits.stride(1) != 1 or experts is None:
            raise KernelError("moe_route: float32 logits and the number of experts are wanted")
        _check(library().acv_moe_route(None, 0, None, None, _p(logits), logits.stride(0), T, H, experts, top, int(softmax),
                                       int(renorm), _p(ids), _p(weights), _p(gate), dtype_code(h.dtype), n_groups, keep, float(renorm_eps),
                                       _stream()), "moe_route")
        return
    if w_router.dtype != torch.float32 or not w_router.is_contiguous() or h.stride(1) != 1:
        raise KernelError("moe_route: a contiguous float32 router matrix is wanted")
    _check(library().acv_moe_route(_p(h), h.stride(0), _p(w_router), _p(gate_w), None, 0, T, H, w_router.shape[0], top,
                                   int(softmax), int(renorm), _p(ids), _p(weights), _p(gate), dtype_code(h.dtype), n_groups, keep,
                                   float(renorm_eps), _stream()), "moe_route")


def moe_group(ids: torch.Tensor, experts: int, grouped: torch.Tensor, place: torch.Tensor, tile_expert: torch.Tensor,
              tile: int = MOE_TILE, tiles_used: torch.Tensor | None = None) -> None:
    """Group the rows (token, choice) by expert: ``grouped`` [tiles * tile] holds the rows expert after expert, each
    expert's padded with -1 to whole tiles; ``place`` [rows] where a row went; ``tile_expert`` [tiles] whose a tile is;
    ``tiles_used`` (one int32, optional): how many tiles hold rows."""
    _need_cuda(ids, grouped, place, tile_expert)
    if grouped.numel() < tile_expert.numel() * tile:
        raise KernelError("moe_group: the grouped list is shorter than its tiles")
    _check(library().acv_moe_group(_p(ids), ids.numel(), experts, tile_expert.numel(), tile, _p(grouped), _p(place),
                                   _p(tile_expert), _p(tiles_used), _stream()), "moe_group")


def moe_gather(h: torch.Tensor, grouped: torch.Tensor, weights: torch.Tensor | None, top: int, out: torch.Tensor,
               scale_out: torch.Tensor | None, tiles_used: torch.Tensor | None, tile: int) -> torch.Tensor:
    """out[r] = h[grouped[r] // top] (zeros where grouped[r] < 0), scale_out[r] = weights[grouped[r]]: the tokens' rows in
    grouped order (bfloat16, rows of 16-byte alignment); rows behind the tiles in use are left as they are."""
    _need_cuda(h, grouped, out)
    if h.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not out.is_contiguous() or h.stride(1) != 1:
        raise KernelError("moe_gather: bfloat16 rows are wanted")
    _check(library().acv_moe_gather(_p(h), h.stride(0), _p(grouped), _p(weights), top, h.shape[1], _p(out), _p(scale_out),
                                    _p(tiles_used), tile, out.shape[0], _stream()), "moe_gather")
    return out


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_expert: torch.Tensor, tiles_used: torch.Tensor,
                    glu: bool = False, row_scale: torch.Tensor | None = None, limit: float = 0.0, alpha: float = 0.0,
                    unary: str | None = None) -> torch.Tensor:
    """The experts' products on tcgen05: x [tiles * 128, K] holds the rows in grouped order, w [E, N, K] the experts'
    matrices; out [rows, N] (bfloat16 or float32), or with ``glu`` [rows, N / 2] bfloat16: w's rows come in (gate, up) pairs
    and go through the clamped gated unit, the accumulators times ``row_scale[row]`` first.  Without ``glu``:
    ``row_scale`` multiplies a row's accumulators, and ``unary`` (a name of ``ACTIVATIONS`` other than the first) is then
    applied to every output, in float."""
    _need_cuda(x, w, out, tile_expert, tiles_used)
    E, N, K = w.shape
    M = x.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or x.shape[1] != K or x.stride(1) != 1 \
            or out.shape != (M, N // 2 if glu else N) or out.stride(1) != 1 or M != tile_expert.numel() * MOE_TC_TILE:
        raise KernelError(f"gemm_tc_grouped: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    if glu and out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_grouped: the gated output is bfloat16")
    bn = 256 if N >= 256 else (128 if N >= 128 else 64)
    _, _, status = _gemm_buffers(x.device, 0, 0)
    _check(library().acv_gemm_tc_grouped(_p(x), x.stride(0), _p(w), K, _p(out), out.stride(0), M, N, K, E, _p(tile_expert),
                                         _p(tiles_used), 1 if out.dtype == torch.float32 else 0,
                                         2 if glu else ((ACTIVATIONS[unary] << 4) if unary else 0),
                                         _p(row_scale), limit, alpha, bn, _p(status), sm_count(x.device), 8, _stream()),
           "gemm_tc_grouped")
    return out


def _moe_which(glu: bool, plain_act: str | None, pairs) -> tuple[int, int]:
    """(which product of the grouped kernels, what travels in their ``pairs`` argument)."""
    if plain_act is None:
        return (0 if glu else 1), int(pairs)
    if glu or plain_act not in ACTIVATIONS or ACTIVATIONS[plain_act] == 0:
        raise KernelError(f"grouped products: no plain activation '{plain_act}' (or asked for beside a gate)")
    return 2, ACTIVATIONS[plain_act]


def moe_gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, grouped: torch.Tensor, tile_expert: torch.Tensor,
                  row_weight: torch.Tensor | None, top: int, glu: bool, limit: float = 0.0, alpha: float = 0.0,
                  pairs: bool = False, plain_act: str | None = None) -> torch.Tensor:
    """The experts' products over the grouped rows on the CUDA cores, 32-bit accumulation.  ``pairs``: with ``glu``, the
    rows of w are (gate, up) pairs instead of all gate rows followed by all up rows.  ``plain_act`` (a name of
    ``ACTIVATIONS``; not with ``glu``): experts without a gate: w [E, N, K], a [T, K] the tokens, out
    [tiles * MOE_TILE, N] of a's type = act(w a).

    ``glu``: w [E, 2N, K] (gate rows, then up rows), a [T, K] the tokens, out [tiles * MOE_TILE, N] of a's type =
    act(weight * gate, weight * up).  Otherwise w [E, N, K], a the grouped rows [tiles * MOE_TILE, K], out float32
    [tiles * MOE_TILE, N] (times the row's weight, when given)."""
    _need_cuda(a, w, out, grouped, tile_expert)
    E, NW, K = w.shape
    N = NW // 2 if glu else NW
    which, pairs = _moe_which(glu, plain_act, pairs)
    if a.shape[1] != K or out.shape[1] != N or a.dtype != w.dtype or not w.is_contiguous() or a.stride(1) != 1 or \
            out.stride(1) != 1 or out.dtype != (a.dtype if which != 1 else torch.float32):
        raise KernelError(f"moe_gemm_simt: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check(library().acv_moe_gemm_simt(_p(a), a.stride(0), _p(w), w.stride(0), w.stride(1), _p(out), out.stride(0),
                                       _p(grouped), _p(tile_expert), _p(row_weight), top, tile_expert.numel(), N, K,
                                       which, limit, alpha, int(pairs), dtype_code(a.dtype), _stream()), "moe_gemm_simt")
    return out


def moe_gemm_mma_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core form of the grouped products wants bfloat16 and rows of 16-byte alignment."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.is_contiguous() and (w.shape[1] * w.shape[2]) % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def moe_gemm_mma(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, grouped: torch.Tensor, tile_expert: torch.Tensor,
                 row_weight: torch.Tensor | None, top: int, glu: bool, limit: float = 0.0, alpha: float = 0.0,
                 pairs: bool = False, plain_act: str | None = None) -> torch.Tensor:
    """``moe_gemm_simt`` on the tensor cores (bfloat16 operands, float accumulators; the same arguments)."""
    _need_cuda(a, w, out, grouped, tile_expert)
    E, NW, K = w.shape
    N = NW // 2 if glu else NW
    which, pairs = _moe_which(glu, plain_act, pairs)
    if a.shape[1] != K or out.shape[1] != N or out.stride(1) != 1 or out.dtype != (torch.bfloat16 if which != 1 else torch.float32):
        raise KernelError(f"moe_gemm_mma: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check(library().acv_moe_gemm_mma(_p(a), a.stride(0), _p(w), w.stride(0), w.stride(1), _p(out), out.stride(0),
                                      _p(grouped), _p(tile_expert), _p(row_weight), top, tile_expert.numel(), N, K,
                                      which, limit, alpha, int(pairs), _stream()), "moe_gemm_mma")
    return out


def moe_experts_up(h: torch.Tensor, gate_up: torch.Tensor, act: torch.Tensor, grouped: torch.Tensor, tile_expert: torch.Tensor,
                   row_weight: torch.Tensor | None, top: int, limit: float, alpha: float, pairs: bool = False,
                   plain_act: str | None = None) -> torch.Tensor:
    """act[grouped row] = gated activation of the row's expert's gate and up products of its token (with ``plain_act``:
    that activation of the expert's one up product); dispatch by shape."""
    glu = plain_act is None
    if moe_gemm_mma_takes(h, gate_up):
        return moe_gemm_mma(h, gate_up, act, grouped, tile_expert, row_weight, top, glu, limit, alpha, pairs, plain_act)
    return moe_gemm_simt(h, gate_up, act, grouped, tile_expert, row_weight, top, glu, limit, alpha, pairs, plain_act)


def moe_experts_down(act: torch.Tensor, down: torch.Tensor, out: torch.Tensor, grouped: torch.Tensor, tile_expert: torch.Tensor,
                     row_weight: torch.Tensor | None, top: int) -> torch.Tensor:
    """out[grouped row] (float32) = the row's expert's down product of its activations; dispatch by shape."""
    if moe_gemm_mma_takes(act, down):
        return moe_gemm_mma(act, down, out, grouped, tile_expert, row_weight, top, False)
    return moe_gemm_simt(act, down, out, grouped, tile_expert, row_weight, top, False)


def moe_combine(d: torch.Tensor, place: torch.Tensor, top: int, shared: torch.Tensor | None, gate: torch.Tensor | None,
                out: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_j d[place[t, j]] (+ gate[t] * shared[t]), summed in float32 in the order of the choices
    (d float32, or bfloat16 beside a bfloat16 output)."""
    _need_cuda(d, place, out)
    T, H = out.shape
    _check(library().acv_moe_combine(_p(d), d.stride(0), dtype_code(d.dtype), _p(place), top, _p(shared), shared.stride(0) if shared is not None else 0,
                                     _p(gate), _p(out), out.stride(0), T, H, dtype_code(out.dtype), _stream()), "moe_combine")
    return out


def glu(gate_up: torch.Tensor, out: torch.Tensor, kind: int, limit: float, alpha: float, pairs: bool = False) -> torch.Tensor:
    """out = act(gate, up) for a gated unit's stacked product [T, 2I]: gate columns then up columns, or with ``pairs``
    (gate, up) column by column.  ``kind``: ``GLU_SWISH_CLAMPED``, or a number of ``ACTIVATIONS`` other than 0:
    out = that activation of gate, times up (computed in float, rounded once)."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    _check(library().acv_glu(_p(gate_up), gate_up.stride(0), _p(out), out.stride(0), T, I, kind, limit, alpha, int(pairs),
                             dtype_code(out.dtype), _stream()), "glu")
    return out


def linear_bf16_glu_takes(x: torch.Tensor, w_pairs: torch.Tensor) -> bool:
    """The product with the clamped gated unit in its epilogue exists with tokens on the tensor core's rows: more than
    128 tokens, rows of 16-byte alignment."""
    return x.dtype == torch.bfloat16 and x.shape[0] > 128 and gemm_tc_takes(x, w_pairs) and w_pairs.shape[0] % 16 == 0


def linear_bf16_glu(x: torch.Tensor, w_pairs: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out[M, I] = g * sigmoid(alpha g) * (u + 1), g = min(x . w[2i], limit), u = clamp(x . w[2i + 1], +-limit), in one
    kernel (the activation is the tcgen05 product's epilogue)."""
    _need_cuda(x, w_pairs, out)
    M, K = x.shape
    N = w_pairs.shape[0]
    if out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(1) != 1 or w_pairs.shape[1] != K:
        raise KernelError(f"linear_bf16_glu: shapes {tuple(x.shape)} x {tuple(w_pairs.shape)} -> {tuple(out.shape)} do not fit")
    plan = gemm_tc_plan(M, N, K)
    if plan[0]:
        raise KernelError("linear_bf16_glu: tokens must lie on the rows (more than 128 of them)")
    bn, stages = plan[1], plan[3] if len(plan) > 3 else 8
    mode = plan[4] if len(plan) > 4 else 0
    _, _, status = _gemm_buffers(x.device, 0, 0)
    _check(library().acv_gemm_tc_glu(_p(x), x.stride(0), _p(w_pairs), w_pairs.stride(0), _p(out), out.stride(0), M, N, K, limit,
                                     alpha, bn, _p(status), sm_count(x.device), stages, mode | 2, _stream()), "gemm_tc_glu")
    return out


# ----------------------------------------------------------------------------- layer norm over a float stream, token shift
def add_layernorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
                  out: torch.Tensor, rows: torch.Tensor | None = None, delta_scale: float = 1.0) -> torch.Tensor:
    """x (float32 [T, H]) += delta_scale * delta in place (without ``rows``); out = (x - mean) / sqrt(var + eps) * w + b
    in float, rounded once to out's type.  With ``rows`` (int32 [R]) only those rows, into out[0..R), x untouched."""
    _need_cuda(x, out, weight)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or (delta is not None and not delta.is_contiguous()):
        raise KernelError("add_layernorm: a contiguous float32 stream and contiguous delta and output are wanted")
    n = out.shape[0] if rows is not None else x.shape[0]
    ddt = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    _check(library().acv_add_layernorm(_p(x), _p(delta), float(delta_scale), _p(weight), _p(bias), _p(out), _p(rows), n,
                                       x.shape[-1], eps, ddt, dtype_code(out.dtype), _stream()), "add_layernorm")
    return out


def token_shift(normed: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor,
                seq_of_token: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = n[t] + (n[t-1] - n[t]) * mu; the row before a request's first token of the step comes from
    ``state[slots[request]]`` (float32 [slots, H]), which then takes the request's last row."""
    _need_cuda(normed, mu, state, out)
    if normed.dtype != torch.float32 or state.dtype != torch.float32 or not normed.is_contiguous() or not state.is_contiguous():
        raise KernelError("token_shift: contiguous float32 rows and state are wanted")
    T, H = normed.shape
    _check(library().acv_token_shift(_p(normed), _p(mu), _p(state), _p(slots), _p(cu_q), _p(seq_of_token), _p(out), T, H,
                                     dtype_code(out.dtype), _stream()), "token_shift")
    return out


def add_layernorm_shift(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None,
                        eps: float, mu: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
                        delta_scale: float = 1.0) -> torch.Tensor:
    """``add_layernorm`` and ``token_shift`` in one launch, for a step in which row t is request t's only token."""
    _need_cuda(x, out, weight, state)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or not state.is_contiguous():
        raise KernelError("add_layernorm_shift: a contiguous float32 stream, state and output are wanted")
    ddt = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    _check(library().acv_add_layernorm_shift(_p(x), _p(delta), float(delta_scale), _p(weight), _p(bias), _p(mu), _p(state),
                                             _p(slots), _p(out), x.shape[0], x.shape[1], eps, ddt, dtype_code(out.dtype),
                                             _stream()), "add_layernorm_shift")
    return out


def add_row_f32(x: torch.Tensor, row: torch.Tensor) -> torch.Tensor:
    """x[t] += row for every row of the float32 stream x."""
    _need_cuda(x, row)
    if x.dtype != torch.float32 or row.dtype != torch.float32 or not x.is_contiguous() or row.numel() != x.shape[1]:
        raise KernelError("add_row_f32: a contiguous float32 stream and a float32 vector of its width are wanted")
    _check(library().acv_add_row_f32(_p(x), _p(row), x.shape[0], x.shape[1], _stream()), "add_row_f32")
    return x


def softcap_f32(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("softcap_f32: a contiguous float32 tensor is wanted")
    _check(library().acv_softcap_f32(_p(x), x.numel(), float(cap), _stream()), "softcap_f32")
    return x


# ----------------------------------------------------------------------------- gated linear recurrence
def causal_conv(x: torch.Tensor, x_bias: torch.Tensor | None, taps: torch.Tensor, conv_bias: torch.Tensor | None,
                state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, seq_of_token: torch.Tensor,
                out: torch.Tensor, taps_t: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, c] = conv_bias[c] + sum_j taps[c, K-1-j] * (x[t-j, c] + x_bias[c]) over each request's tokens; what lies
    before the step comes from ``state`` (float32 [slots, K-1, C], oldest first), which is replaced.  x: [T, C] view
    (row stride free), out float32 [T, C].  ``taps_t``: the taps transposed ([K, C], float32): float inputs with aligned
    rows then take the kernel that gives a thread four neighbouring channels."""
    _need_cuda(x, taps, state, out)
    T, C = out.shape
    K = taps.shape[1]
    if out.dtype != torch.float32 or not out.is_contiguous() or x.stride(1) != 1 or taps.dtype != torch.float32 or not state.is_contiguous():
        raise KernelError("causal_conv: float32 taps, state and output are wanted")
    _check(library().acv_causal_conv(_p(x), x.stride(0), _p(x_bias), _p(taps), _p(conv_bias), _p(state), _p(slots), _p(cu_q),
                                     _p(seq_of_token), _p(out), T, C, K, dtype_code(x.dtype),
                                     _p(taps_t) if taps_t is not None and taps_t.is_contiguous() and taps_t.shape == (K, C) else None,
                                     _stream()), "causal_conv")
    return out


SEGMENT_TOKENS = 64     # tokens of a segment of a long portion in the kernels of the linear recurrences


def segment_work(q_lens, seg_len: int = SEGMENT_TOKENS) -> tuple[dict, dict]:
    """The items of the recurrence kernels for a step: a request that brings more than ``seg_len`` tokens is cut into
    segments of ``seg_len`` that run side by side (the recurrences are linear in their state: a first launch leaves
    what each segment adds, a second one folds what lies before it).  Returns (int32 arrays that the kernels read on the
    device: the request and the segment number of every item; counts for the launches)."""
    import numpy as np
    n = [max(1, -(-int(q) // seg_len)) for q in q_lens]
    seq = np.repeat(np.arange(len(q_lens), dtype=np.int32), n)
    idx = np.concatenate([np.arange(k, dtype=np.int32) for k in n]) if n else np.zeros(0, np.int32)
    return ({"seg_seq": seq, "seg_idx": idx}, {"n_items": int(seq.size), "seg_len": seg_len, "summaries": max(n, default=1) > 1})


def segment_work_decode(padded: int, seg_len: int = SEGMENT_TOKENS) -> tuple[dict, dict]:
    """The same for a batch of ``padded`` requests with one token each."""
    import numpy as np
    return ({"seg_seq": np.arange(padded, dtype=np.int32), "seg_idx": np.zeros(padded, np.int32)},
            {"n_items": padded, "seg_len": seg_len, "summaries": False})


def _segments(work: dict | None, num_seqs: int):
    """(seg_seq, seg_idx, seg_len, n_items, summaries) of a step's work, or one whole item for each request."""
    if work is None:
        return None, None, 1 << 30, num_seqs, False
    return work["seg_seq"], work["seg_idx"], work["seg_len"], work["n_items"], work["summaries"]


def block_gates(u: torch.Tensor, wa_t: torch.Tensor, ba: torch.Tensor | None, wb_t: torch.Tensor, bb: torch.Tensor | None,
                softplus_rate: torch.Tensor, c_r: float, a: torch.Tensor, b: torch.Tensor,
                bf16_weights: tuple | None = None) -> None:
    """What the gated recurrence multiplies and adds at every token: r = sigmoid(A_b u_b + ba), g = sigmoid(B_b u_b + bb)
    per block b of the channels, then a = exp(c_r * r * softplus_rate) and b = sqrt(1 - a^2) * g * u.  wa_t, wb_t float32
    [blocks, in, out]; u, a, b float32 [T, C].  ``bf16_weights`` = (A, B) as bfloat16 [blocks, out, in]: the two products
    run on the tensor cores with u rounded to bfloat16 for them (a bfloat16 run's way with its projections), where the
    blocks' width is a multiple of 16 up to 256; everything behind the products stays float."""
    _need_cuda(u, wa_t, wb_t, a, b)
    T, C = u.shape
    if any(t.dtype != torch.float32 or not t.is_contiguous() for t in (u, wa_t, wb_t, a, b, softplus_rate)):
        raise KernelError("block_gates: contiguous float32 tensors are wanted")
    bw = C // wa_t.shape[0]
    if bf16_weights is not None and bw % 16 == 0 and bw <= 256:
        wa, wb = bf16_weights
        if wa.dtype != torch.bfloat16 or wb.dtype != torch.bfloat16 or not wa.is_contiguous() or not wb.is_contiguous():
            raise KernelError("block_gates: contiguous bfloat16 weights [blocks, out, in] are wanted")
        _check(library().acv_block_gates_mma(_p(u), _p(wa), _p(ba), _p(wb), _p(bb), _p(softplus_rate), float(c_r), _p(a),
                                             _p(b), T, C, wa.shape[0], _stream()), "block_gates")
        return
    _check(library().acv_block_gates(_p(u), _p(wa_t), _p(ba), _p(wb_t), _p(bb), _p(softplus_rate), float(c_r), _p(a), _p(b),
                                     T, C, wa_t.shape[0], _stream()), "block_gates")


def gated_scan(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, y_bias: torch.Tensor | None, state: torch.Tensor,
               slots: torch.Tensor, cu_q: torch.Tensor, num_seqs: int, out: torch.Tensor, work: dict | None = None) -> torch.Tensor:
    """S = a S + b per channel along each request's tokens, S from and back to ``state`` (float32 [slots, C]);
    out[t] = S * gelu_tanh(y[t] + y_bias).  y: a [T, C] view, float32 or of out's type; out: [T, C] of the run's type.
    ``work``: the step's segments (``segment_work``); default: every request's portion is one item."""
    _need_cuda(a, b, y, state, out)
    C = a.shape[1]
    if y.stride(1) != 1 or out.stride(1) != 1 or not state.is_contiguous() or not a.is_contiguous() or not b.is_contiguous():
        raise KernelError("gated_scan: rows of y and out must be dense")
    seg_seq, seg_idx, seg_len, n_items, summaries = _segments(work, num_seqs)
    seg = torch.empty((n_items, 2, C), device=a.device, dtype=torch.float32) if summaries else None
    _check(library().acv_gated_scan(_p(a), _p(b), _p(y), y.stride(0), _p(y_bias), _p(state), _p(slots), _p(cu_q),
                                    _p(seg_seq), _p(seg_idx), seg_len, _p(seg), 1 if summaries else 0, _p(out),
                                    out.stride(0), n_items, C, dtype_code(y.dtype), dtype_code(out.dtype), _stream()),
           "gated_scan")
    return out


# ----------------------------------------------------------------------------- retention
def retention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos_sin: torch.Tensor | None, positions: torch.Tensor,
              decay: torch.Tensor, k_scale: float, state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor,
              num_seqs: int, out: torch.Tensor, num_heads: int, dim: int, value_dim: int,
              work: dict | None = None, silu_inputs: bool = False) -> torch.Tensor:
    """S = decay_h S + k v^T, o = S^T q along each request's tokens, per head; q, k ([T, H*dim]) and v ([T, H*value_dim])
    are views of one projection (same row stride); q and k are rotated by ``cos_sin`` (float32 [positions, rot]) and k
    multiplied by ``k_scale`` in float; state float32 [slots, H, dim, value_dim]; out float32 [T, H*value_dim].
    ``work``: the step's segments (``segment_work``); default: every request's portion is one item.
    ``silu_inputs``: q, k and v pass through silu, in float, before anything else."""
    _need_cuda(q, k, v, state, out)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1:
        raise KernelError("retention: q, k and v must be views of one projection with dense rows")
    if out.dtype != torch.float32 or state.dtype != torch.float32 or not state.is_contiguous() or out.stride(1) != 1:
        raise KernelError("retention: float32 state and output are wanted")
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    rows = cos_sin.shape[0] if cos_sin is not None else 0
    seg_seq, seg_idx, seg_len, n_items, summaries = _segments(work, num_seqs)
    seg = torch.empty((n_items, num_heads, dim, value_dim), device=q.device, dtype=torch.float32) if summaries else None
    _check(library().acv_retention(_p(q), _p(k), _p(v), q.stride(0), _p(cos_sin), rot, rows, _p(positions), _p(decay),
                                   float(k_scale), _p(state), _p(slots), _p(cu_q), _p(seg_seq), _p(seg_idx), seg_len,
                                   _p(seg), 1 if summaries else 0, _p(out), out.stride(0), n_items,
                                   num_heads, dim, value_dim, dtype_code(q.dtype), 1 if silu_inputs else 0, _stream()),
           "retention")
    return out


def retention_gate(o: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, num_heads: int, value_dim: int, eps: float,
                   out_scale: float = 1.0, weight: torch.Tensor | None = None, joint: bool = False,
                   gate_fn: str = "silu") -> torch.Tensor:
    """out = o / sqrt(mean over a head of o^2 + eps) * silu(gate) * out_scale; o float32, gate and out views of the run's type.
    ``joint``: the mean is taken over all heads side by side instead of each head by itself; ``weight`` (float32
    [heads * value_dim]) multiplies the normed values; ``gate_fn`` "sigmoid" instead of "silu"."""
    _need_cuda(o, gate, out)
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != num_heads * value_dim or not weight.is_contiguous()):
        raise KernelError("retention_gate: the weight is a contiguous float32 vector over all heads' values")
    if gate_fn not in ("silu", "sigmoid"):
        raise KernelError(f"retention_gate: no gate function '{gate_fn}'")
    if o.dtype != torch.float32 or gate.dtype != out.dtype or gate.stride(1) != 1 or out.stride(1) != 1 or o.stride(1) != 1:
        raise KernelError("retention_gate: float32 o, and gate and out of one type with dense rows, are wanted")
    _check(library().acv_retention_gate(_p(o), o.stride(0), _p(gate), gate.stride(0), _p(out), out.stride(0), o.shape[0],
                                        num_heads, value_dim, eps, float(out_scale), dtype_code(out.dtype), _p(weight),
                                        1 if joint else 0, 1 if gate_fn == "sigmoid" else 0, _stream()), "retention_gate")
    return out


# ----------------------------------------------------------------------------- scores mixed across heads
def distance_buckets(rows: int, far: float) -> tuple[torch.Tensor, int]:
    """(bucket of each distance below the first one that reads the last row, int32 on the host; that last row).
    A table of ``rows`` rows gives one row to each of the first rows/2 distances and spreads the rest evenly over the
    logarithm of the distance up to ``far``; everything beyond reads the last row.  Computed in double precision."""
    half = rows // 2
    last = rows - 1
    if half <= 0 or far <= half:
        return torch.arange(min(max(half, 1), rows), dtype=torch.int32), last
    out = []
    n = 0
    while True:
        b = n if n < half else min(last, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        if n >= half and b >= last:
            break
        out.append(b)
        n += 1
        if n > (1 << 22):
            raise KernelError("distance_buckets: the table's last row is never reached")
    return torch.tensor(out, dtype=torch.int32), last


MIXED_SPLIT_KEYS = 256      # no share of a one-token request's keys is shorter than this


def attention_mixed_tc_takes(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                             rel_rows: int = 0) -> bool:
    """Whether the tensor-core kernel of the head-mixing attention runs these sizes (bfloat16; head sizes in multiples of
    8, values up to 128; up to 64 heads that split evenly over a cluster's CTAs; everything of a tile in shared memory)."""
    return dtype == torch.bfloat16 and bool(library().acv_attention_mixed_tc_takes(num_heads, num_kv_heads, head_dim,
                                                                                    value_dim, rel_rows))


def attention_mixed(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                    table_rows: torch.Tensor | None = None, value_dim: int = 0, temp: torch.Tensor | None = None,
                    softcap: float = 0.0, rel: torch.Tensor | None = None, bucket_of: torch.Tensor | None = None,
                    last_row: int = 0, talk: torch.Tensor | None = None, ctx=None, work: dict | None = None) -> torch.Tensor:
    """Paged causal attention whose scores pass through more steps before the softmax: times ``temp`` [heads], a soft
    cap, plus ``rel`` [rows, heads] by bucketed distance (``bucket_of`` int32 [distances], larger distances read
    ``last_row``), then mixed across heads by ``talk`` [heads, heads]; each step optional.  Everything after the
    score's product is float32; temp, rel and talk are float32 tensors.

    With the step's context and attention work lists (``ctx``, ``work``) bfloat16 runs take the tensor-core kernel
    (tiles of 16 query tokens with all heads, one launch for portions and one-token requests); float32 runs, and sizes
    that kernel refuses, take the kernel with one block a token."""
    _need_cuda(q, out, k_pages)
    for t in (temp, rel, talk):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError("attention_mixed: temp, rel and talk are contiguous float32 tensors")
    n_dist = bucket_of.numel() if bucket_of is not None else 0
    value_dim = int(value_dim) or head_dim
    rel_rows = rel.shape[0] if rel is not None else 0
    if ctx is not None and work is not None and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and \
            attention_mixed_tc_takes(q.dtype, num_heads, num_kv_heads, head_dim, value_dim, rel_rows):
        # one-token requests: a CTA (or cluster) a request leaves most SMs idle and walks a long context alone, so the
        # keys are shared among several (each at least MIXED_SPLIT_KEYS), as many as bring the launch to about the
        # device's SMs; the partial results meet in a second small launch
        n_dec, n_split, acc, ml = work["n_dec"], 1, None, None
        if n_dec:
            seen = min(work["max_dec_kv"], window) if window > 0 else work["max_dec_kv"]
            if library().acv_attention_mixed_dec_takes(num_heads, num_kv_heads, head_dim, value_dim, rel_rows):
                # a launch of their own, a warp a key/value head; its two buffers of keys and values fill an SM's shared memory
                room = max(1, sm_count(q.device) // n_dec)
            else:
                clusters = 1 if num_heads <= 16 else (2 if num_heads <= 32 else 4)
                room = max(1, sm_count(q.device) // (clusters * (n_dec + 8 * work["n_tiles"])))
            n_split = max(1, min(room, seen // MIXED_SPLIT_KEYS, 16))
            if n_split > 1:
                parts = n_dec * n_split * num_heads
                acc, ml, _ = _decode_scratch(q.device, parts * value_dim, parts * 2, 0)
        _check(library().acv_attention_mixed_tc(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(work["tile_seq"]), _p(work["tile_q0"]),
            work["n_tiles"], _p(work["dec_tokens"]), _p(work["dec_seqs"]), work["n_dec"], _p(ctx.cu_q), _p(ctx.kv_len),
            _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads, head_dim, value_dim,
            k_pages.shape[2], k_pages.shape[0], float(scale), int(window), _p(temp), float(softcap), _p(rel), rel_rows,
            _p(bucket_of), n_dist, int(last_row), _p(talk), n_split, _p(acc), _p(ml), _stream()), "attention_mixed_tc")
        return out
    _check(library().acv_attention_mixed(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(positions), _p(seq_of_token),
        _p(block_table), block_table.stride(0), _p(table_rows), q.shape[0], num_heads, num_kv_heads, head_dim,
        value_dim, k_pages.shape[2], k_pages.shape[0], float(scale), int(window), _p(temp), float(softcap),
        _p(rel), _p(bucket_of), n_dist, int(last_row), _p(talk), dtype_code(q.dtype), _stream()), "attention_mixed")
    return out


# ----------------------------------------------------------------------------- norms on both sides of a part
def add_normed_rmsnorm(x: torch.Tensor, delta: torch.Tensor, weight_b: torch.Tensor, eps_b: float,
                       weight: torch.Tensor | None, eps: float, out: torch.Tensor | None) -> torch.Tensor | None:
    """The float32 stream x += delta / sqrt(mean(delta^2) + eps_b) * weight_b, in place; then, with ``out``,
    out = x / sqrt(mean(x^2) + eps) * weight, rounded once to out's type.  delta: float32 or bfloat16."""
    _need_cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous() or not delta.is_contiguous() or delta.shape != x.shape \
            or (out is not None and (not out.is_contiguous() or out.shape != x.shape)):
        raise KernelError("add_normed_rmsnorm: a contiguous float32 stream, and delta and out of its shape, are wanted")
    dtype = dtype_code(out.dtype) if out is not None else dtype_code(delta.dtype)
    _check(library().acv_add_normed_rmsnorm(_p(x), _p(delta), dtype_code(delta.dtype), _p(weight_b), float(eps_b), _p(weight),
                                            float(eps), _p(out), x.shape[0], x.shape[1], dtype, _stream()),
           "add_normed_rmsnorm")
    return out


def cast_rows_f32(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, :] = x[r, :] rounded to out's type; x float32 [rows, H], out a view [rows, H] with dense rows at any stride."""
    _need_cuda(x, out)
    if x.dtype != torch.float32 or x.shape != out.shape or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("cast_rows_f32: a float32 matrix and a view of its shape with dense rows are wanted")
    _check(library().acv_cast_rows_f32(_p(x), x.stride(0), _p(out), out.stride(0), x.shape[0], x.shape[1],
                                       dtype_code(out.dtype), _stream()), "cast_rows_f32")
    return out


ACTIVATIONS = {"xielu": 0, "gelu_tanh": 1, "silu": 2, "gelu": 3}
# gate activations that the tensor-core product applies in its own epilogue: name -> the epilogue's code
GATED_EPILOGUE_ACTS = {"silu": 1, "gelu_tanh": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str, p0: float = 0.0, p1: float = 0.0) -> torch.Tensor:
    """Elementwise, in float, rounded once.  "xielu": z > 0: p0 z^2 + z/2; z <= 0: p1 (exp(z) - 1 - z) + z/2;
    "gelu_tanh"; "silu"."""
    _need_cuda(x, out)
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: no kind '{kind}'; known: {', '.join(ACTIVATIONS)}")
    if x.dtype != out.dtype or not x.is_contiguous() or not out.is_contiguous() or x.shape != out.shape:
        raise KernelError("activation: contiguous input and output of one type and shape are wanted")
    _check(library().acv_activation(_p(x), _p(out), x.numel(), ACTIVATIONS[kind], float(p0), float(p1), dtype_code(x.dtype),
                                    _stream()), "activation")
    return out


# ----------------------------------------------------------------------------- attention through a kept latent
def gemm_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[:, b, :] = a[:, b, :] @ w[b]^T for every b: a [M, B, K] and out [M, B, N] are views with dense last
    dimension (any row and batch strides), w [B, N, K] contiguous; 32-bit accumulation.  bfloat16 views made of 16-byte
    pieces run on the tensor cores (csrc/gemm_mma_batched.cu), everything else on the CUDA cores."""
    _need_cuda(a, w, out)
    M, B, K = a.shape
    N = w.shape[1]
    if w.shape != (B, N, K) or out.shape != (M, B, N) or a.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous() \
            or a.dtype != w.dtype:
        raise KernelError(f"gemm_batched: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    lib = library()
    if a.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and lib.acv_gemm_mma_batched_takes(
            _p(a), a.stride(0), a.stride(1), _p(w), K, N * K, _p(out), out.stride(0), out.stride(1), N, K):
        _check(lib.acv_gemm_mma_batched(_p(a), a.stride(0), a.stride(1), _p(w), K, N * K, _p(out), out.stride(0),
                                        out.stride(1), M, N, K, B, _stream()), "gemm_mma_batched")
        return out
    _check(library().acv_gemm_simt_batched(_p(a), a.stride(0), a.stride(1), _p(w), K, N * K, _p(out), out.stride(0),
                                           out.stride(1), M, N, K, B, dtype_code(a.dtype), dtype_code(out.dtype), _stream()),
           "gemm_batched")
    return out


def latent_prepare(q: torch.Tensor, q_out: torch.Tensor, kv: torch.Tensor, weight: torch.Tensor, eps: float,
                   cos_sin: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                   block_table: torch.Tensor | None, pages: torch.Tensor | None, num_heads: int, dim: int, rot_dim: int,
                   rank: int, table_rows: torch.Tensor | None = None) -> None:
    """The kept row of every token, [normed latent | rotated shared key part], into its page, and every head's rotated
    query part into ``q_out[:, h, rank:]`` (csrc/latent_attention.cu).  q: [T, heads*(dim+rot_dim)]; q_out:
    [T, heads*(rank+rot_dim)]; kv: [T, rank+rot_dim]; pages [num_pages, 1, page_size, rank+rot_dim] or None."""
    _need_cuda(q, q_out, kv)
    if q.stride(1) != 1 or q_out.stride(1) != 1 or kv.stride(1) != 1 or q.dtype != kv.dtype or q_out.dtype != q.dtype:
        raise KernelError("latent_prepare: q, q_out and kv have dense rows and one type")
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    _check(library().acv_latent_prepare(
        _p(q), q.stride(0), _p(q_out), q_out.stride(0), _p(kv), kv.stride(0), _p(weight), float(eps), _p(cos_sin), rot,
        cos_sin.shape[0] if cos_sin is not None else 0, _p(positions), _p(seq_of_token), _p(block_table),
        block_table.stride(0) if block_table is not None else 0, _p(table_rows), _p(pages),
        pages.shape[2] if pages is not None else 1, pages.shape[0] if pages is not None else 0, q.shape[0], num_heads, dim,
        rot_dim, rank, dtype_code(q.dtype), _stream()), "latent_prepare")


def attention_latent_tc_takes(dtype: torch.dtype, num_heads: int, row: int, rank: int) -> bool:
    """Whether the tensor-core kernel over kept latent rows runs these sizes (bfloat16; rows and latents in multiples of
    8 elements, latents up to 512; a unit's queries and two key tiles in shared memory)."""
    return dtype == torch.bfloat16 and bool(library().acv_attention_latent_tc_takes(num_heads, row, rank))


def attention_latent(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, ctx, block_table: torch.Tensor,
                     num_heads: int, row: int, rank: int, scale: float, window: int = 0,
                     work: dict | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's kept rows: ``q`` [T, heads*row] are the queries that meet
    the rows of ``pages`` [num_pages, 1, page_size, row]; ``out`` [T, heads*rank] gets the weighted sums of the rows'
    first ``rank`` elements.  Causal, with ``window`` > 0 limited to the last ``window`` rows.

    With the step's attention work lists (``work``) bfloat16 runs take the tensor-core kernel (one launch for portions
    and one-token requests; csrc/latent_attention_tc.cu); float32 runs, and sizes that kernel refuses, take the generic
    paged kernel with the pages as keys and as values."""
    _need_cuda(q, out, pages)
    rows = getattr(ctx, "table_rows", None)
    if work is not None and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and pages.is_contiguous() and \
            attention_latent_tc_takes(q.dtype, num_heads, row, rank):
        # a step of one-token requests alone: a CTA a request leaves SMs idle, so the rows of a request are shared among
        # several (each at least MIXED_SPLIT_KEYS), and a second small launch merges their partial results
        n_dec, n_split, acc, ml = work["n_dec"], 1, None, None
        if n_dec and not work["n_tiles"]:
            seen = min(work["max_dec_kv"], window) if window > 0 else work["max_dec_kv"]
            room = max(1, sm_count(q.device) // (n_dec * ((num_heads + 63) // 64)))
            n_split = max(1, min(room, seen // MIXED_SPLIT_KEYS, 16))
            if n_split > 1:
                parts = n_dec * n_split * num_heads
                acc, ml, _ = _decode_scratch(q.device, parts * rank, parts * 2, 0)
        _check(library().acv_attention_latent_tc(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(pages), _p(work["tile_seq"]), _p(work["tile_q0"]),
            work["n_tiles"], _p(work["dec_tokens"]), _p(work["dec_seqs"]), work["n_dec"], _p(ctx.cu_q), _p(ctx.kv_len),
            _p(block_table), block_table.stride(0), _p(rows), num_heads, row, rank, pages.shape[2], pages.shape[0],
            float(scale), int(window), n_split, _p(acc), _p(ml), _stream()), "attention_latent_tc")
        return out
    return attention_generic(q, out, pages, pages, ctx.positions, ctx.seq_of_token, block_table, num_heads, 1, row, scale,
                             window, table_rows=rows, value_dim=rank)


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor | None, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = x / sqrt(mean(x^2) + eps) * weight over each row, in float, rounded once; x and out [rows, H] views with
    dense rows at any stride (a column range of a stacked projection's output)."""
    _need_cuda(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("rmsnorm_rows: input and output views of one shape and type with dense rows are wanted")
    _check(library().acv_rmsnorm_rows(_p(x), x.stride(0), _p(weight), float(eps), _p(out), out.stride(0), x.shape[0],
                                      x.shape[1], dtype_code(x.dtype), _stream()), "rmsnorm_rows")
    return out


# ----------------------------------------------------------------------------- grouped norm, a mixer's input convolution
def add_group_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, groups: int,
                      out: torch.Tensor, rows: torch.Tensor | None = None, delta_scale: float = 1.0) -> torch.Tensor:
    """The float32 stream x += delta_scale * delta (in place, unless ``rows``); out = the RMS norm of x taken over each of
    ``groups`` equal consecutive parts of the row by itself, times weight (float32 [H]); computed in float32 and rounded
    once to out's type."""
    _need_cuda(x, out, weight)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or (delta is not None and not delta.is_contiguous()) \
            or weight.dtype != torch.float32:
        raise KernelError("add_group_rmsnorm: a contiguous float32 stream, contiguous delta and output, float32 weight are wanted")
    n = out.shape[0] if rows is not None else x.shape[0]
    _check(library().acv_add_group_rmsnorm(_p(x), _p(delta), float(delta_scale), _p(weight), _p(out), _p(rows), n, x.shape[-1],
                                           int(groups), eps, dtype_code(delta.dtype) if delta is not None else 0,
                                           dtype_code(out.dtype), _stream()), "add_group_rmsnorm")
    return out


def input_conv(h: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor,
               seq_of_token: torch.Tensor, out: torch.Tensor, taps_t: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = h[t] + sum_j taps[:, j] * h[t - K + 1 + j] along each request's tokens (h float32 [T, C], taps float32
    [C, K]); the rows before the step come from ``state`` (float32 [slots, K-1, C], oldest first), which is replaced.
    ``taps_t``: the taps transposed ([K, C], float32): a thread then takes four neighbouring channels."""
    _need_cuda(h, taps, state, out)
    T, C = h.shape
    K = taps.shape[1]
    if h.dtype != torch.float32 or taps.dtype != torch.float32 or state.dtype != torch.float32 or not h.is_contiguous() \
            or not taps.is_contiguous() or not state.is_contiguous() or not out.is_contiguous() or taps.shape[0] != C:
        raise KernelError("input_conv: contiguous float32 input, taps [C, K] and state are wanted")
    if taps_t is not None and (taps_t.dtype != torch.float32 or not taps_t.is_contiguous() or taps_t.shape != (K, C)):
        taps_t = None
    _check(library().acv_input_conv(_p(h), _p(taps), _p(state), _p(slots), _p(cu_q), _p(seq_of_token), _p(out), T, C, K,
                                    dtype_code(out.dtype), _p(taps_t), _stream()), "input_conv")
    return out


def add_group_rmsnorm_conv(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, groups: int,
                           taps: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
                           delta_scale: float = 1.0) -> torch.Tensor:
    """``add_group_rmsnorm`` and ``input_conv`` in one launch for a step in which row r is request r's one token."""
    _need_cuda(x, out, weight, taps, state)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or (delta is not None and
            (not delta.is_contiguous() or delta.dtype != out.dtype)) or not taps.is_contiguous() or not state.is_contiguous():
        raise KernelError("add_group_rmsnorm_conv: a contiguous float32 stream, and delta and output of one type, are wanted")
    _check(library().acv_add_group_rmsnorm_conv(_p(x), _p(delta), float(delta_scale), _p(weight), _p(taps), _p(state), _p(slots),
                                                _p(out), x.shape[0], x.shape[1], int(groups), eps, taps.shape[1],
                                                dtype_code(out.dtype), dtype_code(out.dtype), _stream()), "add_group_rmsnorm_conv")
    return out


# ----------------------------------------------------------------------------- from a stacked projection to queries and pages
def qkv_prepare(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None,
                positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor | None,
                k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, table_rows: torch.Tensor | None = None,
                temp: tuple[float, int] | None = None, value_norm_eps: float | None = None,
                shared_values: torch.Tensor | None = None, share: str | None = None, share_weight: float = 0.0) -> None:
    """The steps between an attention layer's stacked projection [T, NH*D | NKV*D | NKV*DV] and its attention kernel, for
    layers whose steps span more than a head; each optional, all in float, one rounding (queries in place, keys and values
    into the pages):

    ``q_weight``/``k_weight`` (float32 [NH*D], [NKV*D]): RMS norm over the whole of q and the whole of k; ``cos_sin``: partial
    rotate-half rotation by table; ``temp`` = (coef, every): q *= 1 + coef ln(floor((p + 1) / every) + 1);
    ``value_norm_eps``: every value head to unit RMS; ``share`` "source": the values are left in ``shared_values``
    (float32 [T, NKV*DV]); "mix": v <- (1 - share_weight) v + share_weight * shared_values."""
    _need_cuda(qkv)
    T = qkv.shape[0]
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    rows = cos_sin.shape[0] if cos_sin is not None else 0
    page = k_pages.shape[2] if k_pages is not None else 1
    n_pages = k_pages.shape[0] if k_pages is not None else 0
    bts = block_table.stride(0) if block_table is not None else 0
    mode = {None: 0, "source": 1, "mix": 2}[share]
    if mode and (shared_values is None or shared_values.dtype != torch.float32 or not shared_values.is_contiguous()
                 or shared_values.shape != (T, num_kv_heads * value_dim)):
        raise KernelError("qkv_prepare: shared values are float32 [tokens, kv heads * value dim]")
    if qkv.stride(1) != 1 or qkv.shape[1] < (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim:
        raise KernelError("qkv_prepare: the projection's rows are [q | k | v], dense")
    coef, every = temp if temp else (0.0, 0)
    _check(library().acv_qkv_prepare(
        _p(qkv), qkv.stride(0), T, num_heads, num_kv_heads, head_dim, value_dim, _p(q_weight), _p(k_weight), eps, _p(cos_sin),
        rot, rows, float(coef), int(every), 1 if value_norm_eps is not None else 0, float(value_norm_eps or 0.0),
        _p(shared_values), mode, float(share_weight), _p(positions), _p(seq_of_token), _p(block_table), bts, _p(table_rows),
        _p(k_pages), _p(v_pages), page, n_pages, dtype_code(qkv.dtype), _stream()), "qkv_prepare")


# ----------------------------------------------------------------------------- a recurrence with decays of the token's own
def token_shift_multi(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor,
                      seq_of_token: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[s, t] = h[t] + (h[t-1] - h[t]) * mu[s] along each request's tokens (mu float32 [S, C]); the row before the step
    comes from ``state`` (float32 [slots, C]), which the step's last row replaces.  Mixed in float, rounded once."""
    _need_cuda(h, mu, state, out)
    T, C = h.shape
    S = mu.shape[0]
    if mu.dtype != torch.float32 or state.dtype != torch.float32 or not h.is_contiguous() or not mu.is_contiguous() \
            or not state.is_contiguous() or not out.is_contiguous() or out.shape != (S, T, C) or out.dtype != h.dtype:
        raise KernelError("token_shift_multi: contiguous h [T, C], float32 mu [S, C] and state, out [S, T, C] of h's type are wanted")
    _check(library().acv_token_shift_multi(_p(h), _p(mu), _p(state), _p(slots), _p(cu_q), _p(seq_of_token), _p(out), T, C, S,
                                           dtype_code(h.dtype), _stream()), "token_shift_multi")
    return out


def wkv_decay(a: torch.Tensor, w2_t: torch.Tensor, w0: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, c] = exp(-exp(w0[c] + sum_j w2_t[j, c] tanh(a[t, j]))): all float32; a [T, L], w2_t [L, C], out [T, C]."""
    _need_cuda(a, w2_t, w0, out)
    T, L = a.shape
    C = w2_t.shape[1]
    if any(t.dtype != torch.float32 for t in (a, w2_t, w0, out)) or a.stride(1) != 1 or not w2_t.is_contiguous() \
            or not out.is_contiguous() or w2_t.shape[0] != L or out.shape != (T, C):
        raise KernelError("wkv_decay: float32 a [T, L], w2_t [L, C], w0 [C], out [T, C] are wanted")
    _check(library().acv_wkv_decay(_p(a), a.stride(0), _p(w2_t), _p(w0), _p(out), T, C, L, _stream()), "wkv_decay")
    return out


def wkv(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor, state: torch.Tensor,
        slots: torch.Tensor, cu_q: torch.Tensor, num_seqs: int, out: torch.Tensor, num_heads: int, dim: int, value_dim: int,
        work: dict | None = None) -> torch.Tensor:
    """o_t = (S + diag(u) k_t v_t^T)^T r_t, then S = diag(w_t) S + k_t v_t^T, along each request's tokens, per head.
    r, k ([T, H*dim]) and v ([T, H*value_dim]): one type and row stride; w float32 [T, H*dim] (the decays); u float32
    [H*dim]; state float32 [slots, H, dim, value_dim]; out float32 [T, H*value_dim].  ``work``: the step's segments
    (``segment_work``); default: every request's portion is one item."""
    _need_cuda(r, k, v, w, u, state, out)
    if not (r.stride(0) == k.stride(0) == v.stride(0)) or r.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1 \
            or not (r.dtype == k.dtype == v.dtype):
        raise KernelError("wkv: r, k and v of one type with one row stride and dense rows are wanted")
    if out.dtype != torch.float32 or state.dtype != torch.float32 or not state.is_contiguous() or out.stride(1) != 1 \
            or w.dtype != torch.float32 or not w.is_contiguous() or u.dtype != torch.float32 or not u.is_contiguous():
        raise KernelError("wkv: float32 decays, bonus, state and output are wanted")
    seg_seq, seg_idx, seg_len, n_items, summaries = _segments(work, num_seqs)
    seg = torch.empty((n_items, num_heads, dim, value_dim), device=r.device, dtype=torch.float32) if summaries else None
    seg_decay = torch.empty((n_items, num_heads, dim), device=r.device, dtype=torch.float32) if summaries else None
    _check(library().acv_wkv(_p(r), _p(k), _p(v), r.stride(0), _p(w), _p(u), _p(state), _p(slots), _p(cu_q), _p(seg_seq),
                             _p(seg_idx), seg_len, _p(seg), _p(seg_decay), 1 if summaries else 0, _p(out), out.stride(0),
                             n_items, num_heads, dim, value_dim, dtype_code(r.dtype), _stream()), "wkv")
    return out
