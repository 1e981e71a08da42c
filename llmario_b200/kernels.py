"""Python face of the CUDA kernels: argument checks, pointers, status codes.

Each function launches one hand-written kernel of ``csrc/`` on the current CUDA stream of torch.
There is no other implementation behind these functions: a tensor that is not on a CUDA device,
or a library that cannot be built, is an error.
"""
from __future__ import annotations

import contextlib
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from .csrc.build import load_library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load_library()
        _declare(_lib)
    return _lib


def _signatures():
    """Argument types of every exported entry point, as the C sources declare them (a test
    compares the two): P pointer or stream, I int, L long long, F float."""
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    return {
        "llm_embed": [P, P, I, P, I, I, I, P, P],
        "llm_rms_norm": [P, P, P, I, P, I, I, F, P],
        "llm_patch_tokens": [P, P, P, I, P],
        "llm_silu_mul": [P, P, I, I, I, P],
        "llm_add_bias": [P, I, P, I, I, P],
        "llm_table_update": [P, I, P, I, P],
        "llm_table_update_counted": [P, I, P, P, I, P],
        "llm_zero_slots": [P, L, P, P, I, P],
        "llm_kv_gather": [P, P, L, P, I, I, P, P, L, I, I, I, I, P, I, I, P],
        "llm_gemm_simt": [P, I, P, I, P, I, I, I, I, I, I, I, I, P],
        "llm_qk_norm_rope_store": [P, I, P, P, P, I, L, P, I, P, P, P, P, P, P, F, I, I, I, I, I,
                                   I, F, I, I, I, P],
        "llm_rope_table": [P, P, P, I, I, F, P],
        "llm_attention_generic": [P, P, P, P, I, L, P, I, P, P, I, I, I, I, I, F, I, P, I, P],
        "llm_attention_generic_ext": [P, P, P, P, I, L, P, I, P, P, I, I, I, I, I, F, I, P, I, I, P,
                                      P, L, P, I, I, P],
        "llm_qkv_store": [P, I, P, I, P, I, P, P, P, P, P, P, I, L, P, I, P, P, I, I, I, I, I, I, I,
                          I, F, I, I, P],
        "llm_pool_blocks": [P, P, L, P, I, P, P, L, P, I, P, P, I, I, I, I, I, I, P],
        "llm_causal_conv": [P, I, P, P, P, L, P, P, I, I, I, P, I, I, I, I, P],
        "llm_min_gru": [P, P, P, I, P, P, P, L, P, I, I, P, P, I, I, I, I, P],
        "llm_gated_act_limit": [P, P, P, I, I, I, I, I, F, P],
        "llm_act_rows": [P, P, I, L, I, I, P],
        "llm_dual_norm_mean": [P, P, P, P, P, I, I, F, I, P],
        "llm_sample": [P, L, I, I, P, P, P, P, P, P, P, P, P],
        "llm_gemv_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, P],
        "llm_gemm_tcgen05": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "llm_attention_flash": [P, P, P, P, P, P, L, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P],
        "llm_attention_merge": [P, P, P, P, I, I, I, I, P],
        "llm_attention_merge_clear": [P, P, P, P, I, I, I, I, P, I, P],
        "llm_attention_merge_sink": [P, P, P, P, I, I, I, I, P, I, P, P],
        "llm_attention_tcgen05_sink": [P, P, I, P, P, L, L, P, I, P, I, I, I, I, I, F, I, I, P, P, P],
        "llm_attention_tcgen05_extra": [P, P, I, P, P, L, L, P, I, P, I, I, I, I, I, F, I, I, P, P, P,
                                        P, P],
        "llm_attention_merge_extra": [P, P, P, P, I, I, I, I, P, I, P, P, P, P],
        "llm_attention_extras": [P, P, P, P, P, L, P, I, P, P, I, I, I, I, I, F, I, P, I, P, P, L, P,
                                 I, I, P],
        "llm_attention_decode_fused": [P, I, P, P, P, P, L, I, I, P, P, L, P, I, P, P, I, P, P, P,
                                       F, I, I, I, I, I, F, I, I, P, P],
        "llm_attention_decode": [P, P, P, P, P, P, L, P, I, P, P, P, I, I, I, I, I, F, I, I, P],
        "llm_attention_decode_tma": [P, P, P, P, P, L, I, I, P, I, P, P, P, I, I, I, I, I, F, I,
                                     I, P, P],
        "llm_attention_decode_persistent": [P, P, P, P, L, I, I, P, I, P, P, I, I, I, I, I, F, I, I, I,
                                            P, P],
        "llm_attention_tcgen05": [P, P, I, P, P, L, L, P, I, P, I, I, I, I, I, F, I, I, P, P],
        "llm_attention_tcgen05_x2": [P, P, I, P, P, L, L, P, I, P, I, I, I, I, I, F, I, P, P],
        "llm_apply_penalties": [P, L, I, P, I, P, P, P, P, P, I, P],
        "llm_random_normal": [P, I, L, ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, L,
                              P],
        "llm_cast_rows": [P, L, P, I, L, I, I, P],
        "llm_norm_scale_add": [P, P, P, P, P, I, I, F, I, P],
        "llm_head_gate": [P, I, P, I, I, I, I, I, P],
        "llm_segment_table": [P, I, P, I, P],
        "llm_bias_sigmoid_pow": [P, P, I, I, F, P],
        "llm_linear_recurrence": [P, I, P, I, P, I, P, I, P, I, P, P, F, F, P, L, P, I, P, P, I, I,
                                  I, I, I, I, I, I, P],
        "llm_log_gate_scan": [P, P, I, P, P, F, P, L, P, I, P, P, I, I, I, I, P],
        "llm_memory_out_norm": [P, I, P, I, P, I, P, P, I, I, I, I, I, F, F, P],
        "llm_stream_step": [P, L, I, P, P, P, I, I, P, P, F, P, I, P, I, I, P],
        "llm_stream_fill": [P, L, I, I, I, P],
        "llm_gated_act": [P, P, P, I, I, I, I, I, P],
        "llm_scale_soft_cap": [P, L, F, F, P],
        "llm_latent_store": [P, I, P, P, P, I, P, P, P, I, L, P, I, P, P, I, I, I, I, I, F, I, I, P],
        "llm_latent_query": [P, I, P, I, P, P, I, I, I, I, I, I, I, P],
        "llm_gemm_simt_batched": [P, P, P, I, I, I, I, I, I, I, I, I, L, L, L, P],
        "llm_moe_route": [P, I, I, I, I, I, P, P, P, P],
        "llm_moe_router": [P, I, P, P, P, I, I, I, I, I, I, I, P, P, P, P],
        "llm_moe_align": [P, I, I, I, I, P, P, P],
        "llm_moe_gather": [P, P, P, I, I, I, I, P, I, P],
        "llm_moe_combine": [P, P, P, P, P, I, P, I, I, I, I, I, P, I, P, I, I, P],
        "llm_gemm_tcgen05_grouped": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P, P],
        "llm_gemm_tcgen05_batched": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "llm_moe_gate_up_rows": [P, P, P, P, I, I, I, I, I, I, I, F, P],
        "llm_moe_down_rows": [P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, P, P],
        "llm_causal_conv_silu": [P, I, P, P, P, L, P, P, I, I, I, P, I, I, I, P],
        "llm_gated_group_norm": [P, I, P, I, P, I, P, I, P, I, P, I, I, I, I, I, F, I, P],
        "llm_gated_group_norm_act": [P, I, P, I, P, I, P, I, P, I, P, I, I, I, I, I, F, I, I, P],
        "llm_embed_scaled": [P, P, I, P, I, I, I, P, F, P],
        "llm_qkv_store_mix": [P, I, P, I, P, I, P, P, P, P, P, P, I, L, P, I, P, P, I, I, I, I, I,
                              I, I, I, F, I, I, F, I, P, I, F, P],
        "llm_channel_gate": [P, I, P, I, I, I, I, P],
        "llm_delta_recurrence": [P, I, P, I, P, I, P, I, P, I, P, P, F, I, F, P, L, P, I, P, P, I,
                                 I, I, I, I, I, I, I, P],
        "llm_delta_recurrence_grouped": [P, I, P, I, P, I, P, I, P, I, P, P, F, I, F, P, L, P, I, P,
                                         P, I, I, I, I, I, I, I, I, P, L, P],
        "llm_rate_decay": [P, P, P, I, I, I, P],
        "llm_moe_router_scaled": [P, I, P, P, P, I, I, I, I, I, I, I, P, P, P, F, P],
        "llm_moe_route_scaled": [P, I, I, I, I, I, P, P, P, F, P],
    }


def _declare(l) -> None:
    sigs = _signatures()
    for name, args in sigs.items():
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = c_int


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def _stream() -> int:
    """The CUDA stream that torch regards as current on this process's device.  (The direct
    query takes a fraction of a microsecond where ``torch.cuda.current_stream()`` takes several;
    a step launches a few hundred kernels.)"""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("llmario_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device}")


launches = 0   # kernels of this library launched so far (a claim that bench.py reports)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        return
    if status == -1:
        raise KernelError(f"{what}: size or dtype not supported by this kernel")
    if status == -2:
        raise KernelError(f"{what}: inconsistent arguments")
    raise KernelError(f"{what}: CUDA error {status}")


# ------------------------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          err_flag: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[tokens[t]] * scale as float32; a token outside the table sets ``err_flag``
    (int32 [1]) to 1 + its row and gives a row of zeros."""
    _cuda(tokens, table, out, err_flag)
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous()
    rows = tokens.numel()
    _check(lib().llm_embed_scaled(_ptr(tokens), _ptr(table), _dt(table), _ptr(out), rows,
                                  table.shape[1], table.shape[0], _ptr(err_flag), float(scale),
                                  _stream()), "embed")


def rms_norm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
             rows_index: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows_index[r] or r] * rsqrt(mean(x^2) + eps) * weight, x and weight float32."""
    _cuda(x, weight, out, rows_index)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32
    assert x.is_contiguous() and out.is_contiguous()
    rows, width = out.shape
    assert x.shape[1] == width and weight.numel() == width
    _check(lib().llm_rms_norm(_ptr(x), _ptr(weight), _ptr(out), _dt(out), _ptr(rows_index), rows,
                              width, float(eps), _stream()), "rms_norm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t][j] = silu(gate_up[t][j]) * gate_up[t][ff + j]."""
    _cuda(gate_up, out)
    assert gate_up.dtype == torch.float32 and gate_up.is_contiguous() and out.is_contiguous()
    rows, ff = out.shape
    assert gate_up.shape == (rows, 2 * ff)
    _check(lib().llm_silu_mul(_ptr(gate_up), _ptr(out), _dt(out), rows, ff, _stream()),
           "silu_mul")


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[t][j] += bias[j] (bias float32; the sum is made in 32-bit and rounded once)."""
    _cuda(out, bias)
    rows, width = out.shape
    assert out.is_contiguous() and bias.dtype == torch.float32 and bias.shape == (width,)
    _check(lib().llm_add_bias(_ptr(out), _dt(out), _ptr(bias), rows, width, _stream()), "add_bias")


def table_update(table: torch.Tensor, updates: torch.Tensor, n: int) -> None:
    """table[u[0]][u[1]] = u[2] for the first n int32 triples of ``updates``."""
    _cuda(table, updates)
    assert table.dtype == torch.int32 and updates.dtype == torch.int32
    _check(lib().llm_table_update(_ptr(table), table.stride(0), _ptr(updates), n, _stream()),
           "table_update")


def patch_tokens(tokens: torch.Tensor, source: torch.Tensor, index: torch.Tensor) -> None:
    """tokens[i] = source[index[i]] for every i with index[i] >= 0 (all int32, on the device)."""
    _cuda(tokens, source, index)
    assert tokens.dtype == source.dtype == index.dtype == torch.int32
    assert tokens.numel() == index.numel()
    _check(lib().llm_patch_tokens(_ptr(tokens), _ptr(source), _ptr(index), tokens.numel(),
                                  _stream()), "patch_tokens")


def table_update_counted(table: torch.Tensor, updates: torch.Tensor, count: torch.Tensor,
                         max_n: int) -> None:
    """As :func:`table_update`, the number of triples read from ``count[0]`` on the device."""
    _cuda(table, updates, count)
    assert table.dtype == torch.int32 and updates.dtype == torch.int32
    _check(lib().llm_table_update_counted(_ptr(table), table.stride(0), _ptr(updates),
                                          _ptr(count), max_n, _stream()), "table_update")


def zero_slots(state: torch.Tensor, slots: torch.Tensor, count: torch.Tensor, max_n: int) -> None:
    """state[slots[i]] = 0 for i < count[0] (read on the device; at most ``max_n``)."""
    _cuda(state, slots, count)
    assert state.is_contiguous() and slots.dtype == torch.int32 and count.dtype == torch.int32
    row_bytes = state[0].numel() * state.element_size()
    _check(lib().llm_zero_slots(_ptr(state), row_bytes, _ptr(slots), _ptr(count), max_n,
                                _stream()), "zero_slots")


def kv_gather(k_src: torch.Tensor, v_src: torch.Tensor, src_page_stride: int,
              block_table: torch.Tensor, page_size: int, k_dst: torch.Tensor, v_dst: torch.Tensor,
              dst_page_stride: int, dst_page_size: int, num_kv_heads: int, head_dim: int,
              items: torch.Tensor, n_items: int, total_chunks: int) -> None:
    """Copy requests' keys and values from cache pages of ``page_size`` positions into scratch
    pages of ``dst_page_size`` (a multiple).  ``k_src`` / ``v_src`` / ``k_dst`` / ``v_dst``: the
    K and V planes of page 0 on either side, pages ``*_page_stride`` elements apart.  ``items``:
    int32 octuples (block-table row, first position, chunks, first scratch page, lowest and
    highest position read, chunks of the items before, 0); a chunk is one source page; chunks
    wholly outside [lowest, highest] or whose page the request no longer holds become zeros."""
    _cuda(k_src, v_src, block_table, k_dst, v_dst, items)
    assert k_src.dtype == k_dst.dtype and items.dtype == torch.int32
    _check(lib().llm_kv_gather(_ptr(k_src), _ptr(v_src), src_page_stride, _ptr(block_table),
                               block_table.stride(0), page_size, _ptr(k_dst), _ptr(v_dst),
                               dst_page_stride, dst_page_size, num_kv_heads, head_dim, _dt(k_src),
                               _ptr(items), n_items, total_chunks, _stream()), "kv_gather")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False
              ) -> None:
    """out (=|+=) a @ w.T on the CUDA cores with 32-bit accumulation; a [M,K], w [N,K]."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib().llm_gemm_simt(_ptr(a), _dt(a), _ptr(w), _dt(w), _ptr(out), _dt(out), M, N, K,
                               a.stride(0), w.stride(0), out.stride(0), int(accumulate),
                               _stream()), "gemm_simt")


def qk_norm_rope_store(proj: torch.Tensor, q_out: torch.Tensor,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       page_stride: int, block_table: torch.Tensor, row_slot: torch.Tensor,
                       row_pos: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                       k_norm_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                       attn_factor: float, num_heads: int, num_kv_heads: int, head_dim: int,
                       rot_dim: int, page_size: int, eps: float,
                       cos_sin: Optional[torch.Tensor] = None, clear_proj: bool = False,
                       values_are_keys: bool = False) -> None:
    """Per-head norm, rotation and stores for the rows of ``proj`` (float32,
    [rows, (Hq + 2 Hkv) * hd], or [rows, Hq * hd] when no cache is given).  With
    ``values_are_keys`` the rows hold no values ([rows, (Hq + Hkv) * hd]): every key head is
    stored twice, normed and rotated as the key and as projected as the value."""
    _cuda(proj, q_out, k_cache, v_cache, block_table, row_slot, row_pos, q_norm_w, k_norm_w,
          inv_freq)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1
    rows = proj.shape[0]
    has_kv = 0 if k_cache is None else (2 if values_are_keys else 1)
    use_norm = q_norm_w is not None
    if rot_dim > 0:
        assert inv_freq is not None and inv_freq.dtype == torch.float32
        assert inv_freq.numel() == rot_dim // 2
    _check(lib().llm_qk_norm_rope_store(
        _ptr(proj), proj.stride(0), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _dt(q_out),
        page_stride, _ptr(block_table), block_table.stride(0), _ptr(row_slot), _ptr(row_pos),
        _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq), _ptr(cos_sin), float(attn_factor), rows,
        num_heads,
        num_kv_heads, head_dim, rot_dim, page_size, float(eps), int(has_kv), int(use_norm),
        int(clear_proj), _stream()), "qk_norm_rope_store")


def rope_table(row_pos: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor,
               attn_factor: float) -> None:
    """out[t][i] = attn_factor * (cos, sin)(row_pos[t] * inv_freq[i]), float32 [rows, half, 2]."""
    _cuda(row_pos, inv_freq, out)
    rows, half = out.shape[0], out.shape[1]
    assert out.dtype == torch.float32 and out.is_contiguous() and inv_freq.numel() == half
    _check(lib().llm_rope_table(_ptr(row_pos), _ptr(inv_freq), _ptr(out), rows, half,
                                float(attn_factor), _stream()), "rope_table")


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                      row_slot: torch.Tensor, row_pos: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: Optional[int], sink: Optional[torch.Tensor] = None,
                      value_dim: int = 0) -> None:
    _cuda(q, out, k_cache, v_cache, block_table, row_slot, row_pos, sink)
    assert q.dtype == out.dtype == k_cache.dtype and q.is_contiguous() and out.is_contiguous()
    rows = q.shape[0]
    _check(lib().llm_attention_generic(
        _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _dt(q), page_stride, _ptr(block_table),
        block_table.stride(0), _ptr(row_slot), _ptr(row_pos), rows, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), _ptr(sink), int(value_dim),
        _stream()),
        f"attention (head_dim {head_dim})")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor, status_out: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``logits`` (float32 [rows, vocab]): greedy where temperature <= 0,
    else top-k, top-p, min-p, temperature, softmax and a draw with the row's uniform.
    ``status_out`` (int32 [4]): the kernel also copies the library's status words there (see
    :func:`status_words`), so that they reach the host in the same copy as the tokens."""
    _cuda(logits, temperature, top_k, top_p, min_p, uniform, out, status_out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert uniform.dtype == torch.float64 and top_k.dtype == torch.int32
    rows, vocab = logits.shape
    status = status_words(logits.device) if status_out is not None else None
    _check(lib().llm_sample(_ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature),
                            _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out),
                            _ptr(status), _ptr(status_out), _stream()), "sample")


def apply_penalties(logits: torch.Tensor, triples: torch.Tensor, n: int, repeat: torch.Tensor,
                    freq: torch.Tensor, presence: torch.Tensor,
                    inflight_src: Optional[torch.Tensor] = None,
                    drawn: Optional[torch.Tensor] = None) -> None:
    """For the first n (row, token, count) triples adjust logits[row][token] in place.
    ``inflight_src`` (int32 per row, -1: none) names, by its index in ``drawn``, a token that
    enters the row's window but is still being drawn by the step before: it counts once more."""
    _cuda(logits, triples, repeat, freq, presence, inflight_src, drawn)
    assert (inflight_src is None) == (drawn is None)
    _check(lib().llm_apply_penalties(_ptr(logits), logits.stride(0), logits.shape[1], _ptr(triples),
                                     n, _ptr(repeat), _ptr(freq), _ptr(presence),
                                     _ptr(inflight_src), _ptr(drawn), logits.shape[0], _stream()),
           "apply_penalties")


def mask_code(window: Optional[int] = None, chunk: Optional[int] = None) -> int:
    """The one integer by which the attention kernels are told which earlier keys a query sees:
    0 all of them, ``window`` > 0 the last ``window``, ``-chunk`` the keys of the query's own
    chunk of ``chunk`` positions (chunks counted from position 0 of the sequence)."""
    if window and chunk:
        raise KernelError("a sliding window and a chunked mask exclude each other")
    if (window or 0) < 0 or (chunk or 0) < 0:
        raise KernelError("window and chunk sizes are positive")
    return int(window) if window else (-int(chunk) if chunk else 0)


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x rounded to out's type; both [rows, cols] with unit stride along a row (either
    may be a column slice of a wider matrix); x float32."""
    _cuda(x, out)
    assert x.dtype == torch.float32 and x.shape == out.shape and x.dim() == 2
    assert x.stride(1) == 1 and out.stride(1) == 1
    _check(lib().llm_cast_rows(_ptr(x), x.stride(0), _ptr(out), _dt(out), out.stride(0),
                               x.shape[0], x.shape[1], _stream()), "cast_rows")


def norm_scale_add(y: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor],
                   x: torch.Tensor, eps: float, rounded: Optional[torch.Tensor] = None,
                   clear: bool = False) -> None:
    """x += y * rsqrt(mean(y^2) + eps) * weight (* scale): all float32, row by row.  ``rounded``
    (bfloat16, x's shape) also receives the new x, rounded once.  ``clear``: y holds zeros
    afterwards (a split-K product adds its partial sums into it the next time)."""
    _cuda(y, weight, scale, x, rounded)
    assert rounded is None or (rounded.dtype == torch.bfloat16 and rounded.shape == x.shape
                               and rounded.is_contiguous())
    assert y.dtype == x.dtype == weight.dtype == torch.float32 and y.shape == x.shape
    assert y.is_contiguous() and x.is_contiguous() and weight.numel() == x.shape[1]
    assert scale is None or (scale.dtype == torch.float32 and scale.numel() == x.shape[1])
    _check(lib().llm_norm_scale_add(_ptr(y), _ptr(weight), _ptr(scale), _ptr(x), _ptr(rounded),
                                    x.shape[0],
                                    x.shape[1], float(eps), int(clear), _stream()), "norm_scale_add")


def head_gate(out: torch.Tensor, gate: torch.Tensor, num_heads: int, head_dim: int,
              clear: bool = False) -> None:
    """out[r, h, :] *= sigmoid(gate[r, h]); ``gate`` float32 [rows, heads] (a column slice of a
    wider matrix is fine), zeroed after use with ``clear``."""
    _cuda(out, gate)
    assert gate.dtype == torch.float32 and gate.stride(1) == 1 and out.is_contiguous()
    rows = out.shape[0]
    assert gate.shape == (rows, num_heads) and out.shape[1] == num_heads * head_dim
    _check(lib().llm_head_gate(_ptr(out), _dt(out), _ptr(gate), gate.stride(0), rows, num_heads,
                               head_dim, int(clear), _stream()), "head_gate")


def channel_gate(out: torch.Tensor, gate: torch.Tensor, clear: bool = False) -> None:
    """out[r, c] *= sigmoid(gate[r, c]); ``gate`` float32 of out's shape (a column slice of a
    wider matrix is fine), zeroed after use with ``clear``."""
    _cuda(out, gate)
    assert gate.dtype == torch.float32 and gate.stride(1) == 1 and out.is_contiguous()
    assert gate.shape == out.shape and out.dim() == 2
    _check(lib().llm_channel_gate(_ptr(out), _dt(out), _ptr(gate), gate.stride(0), out.shape[0],
                                  out.shape[1], int(clear), _stream()), "channel_gate")


def segment_table(row_slot: torch.Tensor, seg: torch.Tensor) -> None:
    """seg[s, :2] = (first row, row after the last) of the step's rows whose request slot is s,
    (0, 0) for a slot without rows; seg[i, 2] = the slot of the i-th request that has rows (in
    no particular order; -1 behind the last); int32 [slots, 3], made on the device from
    ``row_slot``."""
    _cuda(row_slot, seg)
    assert row_slot.dtype == torch.int32 and seg.dtype == torch.int32 and seg.is_contiguous()
    assert seg.dim() == 2 and seg.shape[1] == 3
    _check(lib().llm_segment_table(_ptr(row_slot), row_slot.numel(), _ptr(seg), seg.shape[0],
                                   _stream()), "segment_table")


DECAY_VECTOR, DECAY_SIGMOID_POW, DECAY_RATE_STEP, DECAY_SCALAR_INPUT = 0, 1, 2, 3


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d: torch.Tensor,
                      state: torch.Tensor, out: torch.Tensor, row_slot: torch.Tensor,
                      seg: Optional[torch.Tensor], heads: int, groups: int, key_dim: int,
                      value_dim: int, kind: int, q_scale: float = 1.0, exponent: float = 1.0,
                      rate_log: Optional[torch.Tensor] = None,
                      step_bias: Optional[torch.Tensor] = None, n_requests: int = 0,
                      input_weight: Optional[torch.Tensor] = None, ones: bool = False) -> None:
    """Per request and head ``S <- diag(a_t) S + k_t v_t^T``, ``o_t = S^T (q_scale q_t)`` over
    the rows of the step in order.  q, k float32 [rows, groups * key_dim], v and out float32
    [rows, heads * value_dim] (column slices of wider matrices are fine); head h uses group
    ``h // (heads // groups)``.  ``state``: float32 [slots, >= heads * value_dim * key_dim], each
    head's [value_dim, key_dim] block, carried from step to step.  ``kind`` says how the decay
    comes from ``d``: DECAY_VECTOR ``a = d`` and DECAY_SIGMOID_POW ``a = sigmoid(d)^exponent``
    with d [rows, heads * key_dim]; DECAY_RATE_STEP with d [rows, heads]:
    ``step = softplus(d + step_bias[h])``, ``a = exp(-exp(rate_log[h]) step)`` and v is
    multiplied by step; DECAY_SCALAR_INPUT with d and ``input_weight`` [rows, heads] (equal row
    strides): ``a = d`` and v is multiplied by the input weight.  ``ones``: v has
    ``value_dim - 1`` channels per head and the last state column is fed the constant 1 (it then
    holds the decayed sum of the keys, and the last output channel its product with q).
    ``seg``: the table of :func:`segment_table` with ``n_requests`` the
    number of requests that have rows in the step, or None when every row is a request of its
    own."""
    _cuda(q, k, v, d, state, out, row_slot, seg, rate_log, step_bias, input_weight)
    for t in (q, k, v, d, state, out):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    rows = out.shape[0]
    assert state.dim() == 2 and state.shape[1] >= heads * value_dim * key_dim
    if input_weight is not None:
        assert input_weight.dtype == torch.float32 and input_weight.stride(0) == d.stride(0)
    _check(lib().llm_linear_recurrence(
        _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(d), d.stride(0),
        _ptr(input_weight), int(ones), _ptr(rate_log), _ptr(step_bias), float(exponent), float(q_scale), _ptr(state),
        state.stride(0), _ptr(out), out.stride(0), _ptr(seg), _ptr(row_slot), rows,
        int(n_requests), int(seg is None), heads, groups, key_dim, value_dim, kind, _stream()),
        f"linear_recurrence (key_dim {key_dim})")


def bias_sigmoid_pow(z: torch.Tensor, bias: Optional[torch.Tensor], exponent: float) -> None:
    """z = sigmoid(z + bias)^exponent in place (float32 [rows, n], contiguous), in 32-bit through
    ``exp(-exponent * softplus(-(z + bias)))``."""
    _cuda(z, bias)
    assert z.dtype == torch.float32 and z.is_contiguous() and z.dim() == 2
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == z.shape[1])
    _check(lib().llm_bias_sigmoid_pow(_ptr(z), _ptr(bias), z.shape[0], z.shape[1],
                                      float(exponent), _stream()), "bias_sigmoid_pow")


def rate_decay(z: torch.Tensor, rate_log: torch.Tensor, bias: Optional[torch.Tensor],
               per: int) -> None:
    """z = exp(-exp(rate_log[c // per]) * softplus(z + bias[c])) in place for column c (float32
    [rows, n], contiguous): the decay of a recurrence from a projected step size, ``per``
    neighbouring columns sharing a rate."""
    _cuda(z, rate_log, bias)
    assert z.dtype == torch.float32 and z.is_contiguous() and z.dim() == 2
    n = z.shape[1]
    assert rate_log.dtype == torch.float32 and rate_log.numel() * per == n
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == n)
    _check(lib().llm_rate_decay(_ptr(z), _ptr(rate_log), _ptr(bias), z.shape[0], n, int(per),
                                _stream()), "rate_decay")


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d: torch.Tensor,
                     beta: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                     row_slot: torch.Tensor, seg: Optional[torch.Tensor], heads: int, groups: int,
                     key_dim: int, value_dim: int, kind: int, q_scale: float = 1.0,
                     unit_floor: Optional[float] = None,
                     rate_log: Optional[torch.Tensor] = None,
                     step_bias: Optional[torch.Tensor] = None, n_requests: int = 0,
                     work: Optional[torch.Tensor] = None) -> None:
    """The gated delta rule per request and head over the rows of the step in order:
    ``S <- diag(a_t) S``, ``u = sigmoid(beta_t) (v_t - S^T k_t)``, ``S <- S + k_t u^T``,
    ``o_t = S^T q_t``.  Tensors, state and ``seg`` as in :func:`linear_recurrence`; ``beta``
    float32 [rows, heads] (a column slice is fine).  ``kind`` DECAY_VECTOR: ``d``
    [rows, heads * key_dim] is the decay; DECAY_RATE_STEP: ``d`` [rows, heads] and
    ``a = exp(-exp(rate_log[h]) softplus(d + step_bias[h]))`` for every key channel of head h.
    ``unit_floor`` (not None): q and k of every head are first divided by
    ``sqrt(sum of squares + unit_floor)``; q is then multiplied by ``q_scale``.
    ``work`` (float32, at least :func:`delta_work_floats` elements): room for what portions of
    prompts need to go four tokens at a time (68 to 256 key channels, a multiple of four);
    without it, and for single tokens, every row goes token by token.  The two ways differ by
    rounding only."""
    _cuda(q, k, v, d, beta, state, out, row_slot, seg, rate_log, step_bias, work)
    assert work is None or (work.dtype == torch.float32 and work.is_contiguous())
    for t in (q, k, v, d, beta, state, out):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    rows = out.shape[0]
    assert state.dim() == 2 and state.shape[1] >= heads * value_dim * key_dim
    assert kind in (DECAY_VECTOR, DECAY_RATE_STEP)
    _check(lib().llm_delta_recurrence_grouped(
        _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(d), d.stride(0),
        _ptr(beta), beta.stride(0), _ptr(rate_log), _ptr(step_bias), float(q_scale),
        int(unit_floor is not None), float(unit_floor or 0.0), _ptr(state), state.stride(0),
        _ptr(out), out.stride(0), _ptr(seg), _ptr(row_slot), rows, int(n_requests),
        int(seg is None), heads, groups, key_dim, value_dim, kind, _ptr(work),
        work.numel() if work is not None else 0, _stream()),
        f"delta_recurrence (key_dim {key_dim})")
    global launches
    if work is not None and seg is not None and delta_work_floats(rows, heads, key_dim) \
            and work.numel() >= delta_work_floats(rows, heads, key_dim):
        launches += 2      # the groups' preparation and their walk are launches of their own


def delta_work_floats(rows: int, heads: int, key_dim: int) -> int:
    """Elements of the ``work`` buffer with which :func:`delta_recurrence` takes the rows of a
    step four tokens at a time, 0 when it has no such form for this many key channels."""
    if not (64 < key_dim <= 256 and key_dim % 4 == 0):
        return 0
    return rows * heads * (4 * key_dim + 41)


def causal_conv_silu(src: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     history: torch.Tensor, out: torch.Tensor, row_slot: torch.Tensor,
                     seg: Optional[torch.Tensor], activation: bool = True) -> None:
    """out[r, c] = silu(bias[c] + sum_j weight[c, taps-1-j] * input(r - j, c)) over each
    request's own tokens; inputs before the step come from ``history`` (float32
    [slots, >= channels * (taps - 1)], each channel's last taps - 1 inputs, oldest first), which
    is brought up to date afterwards.  src, out float32 [rows, channels] (column slices are
    fine); weight float32 [channels, taps].  ``activation=False``: the sum as it is, no silu."""
    _cuda(src, weight, bias, history, out, row_slot, seg)
    for t in (src, weight, history, out):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    rows, channels = out.shape
    taps = weight.shape[1]
    assert weight.is_contiguous() and weight.shape[0] == channels and src.shape == out.shape
    assert history.shape[1] >= channels * (taps - 1)
    _check(lib().llm_causal_conv(
        _ptr(src), src.stride(0), _ptr(weight), _ptr(bias), _ptr(history), history.stride(0),
        _ptr(row_slot), _ptr(seg), rows, history.shape[0], int(seg is None), _ptr(out),
        out.stride(0), channels, taps, int(activation), _stream()), "causal_conv")
    global launches
    launches += int(taps > 1)      # the history is brought up to date by a launch of its own


def gated_group_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor,
                     out: torch.Tensor, group: int, eps: float, gate_first: bool,
                     skip: Optional[torch.Tensor] = None, skip_input: Optional[torch.Tensor] = None,
                     head: int = 0, gate_activation: str = "silu") -> None:
    """The recurrence's output through its gate and a norm over groups of ``group`` channels:
    ``y = o (+ skip[ch // head] * skip_input)``; with ``gate_first``
    ``out = unit(y * silu(gate)) * weight`` else ``out = unit(y) * weight * silu(gate)``, where
    unit divides each group by its root mean square.  ``weight`` is indexed by the channel
    modulo its length.  o, gate, skip_input float32 [rows, channels] (column slices are fine).
    ``gate_activation="sigmoid"``: ``sigmoid(gate)`` stands where ``silu(gate)`` does."""
    _cuda(o, gate, weight, out, skip, skip_input)
    if gate_activation not in ("silu", "sigmoid"):
        raise KernelError(f"the gate of a group norm is silu or sigmoid, not '{gate_activation}'")
    rows, channels = out.shape
    assert o.dtype == gate.dtype == weight.dtype == torch.float32 and channels % group == 0
    assert o.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1
    assert (skip is None) == (skip_input is None)
    _check(lib().llm_gated_group_norm_act(
        _ptr(o), o.stride(0), _ptr(skip_input), skip_input.stride(0) if skip is not None else 0,
        _ptr(skip), head, _ptr(gate), gate.stride(0), _ptr(weight), weight.numel(), _ptr(out),
        _dt(out), out.stride(0), rows, channels // group, group, float(eps), int(gate_first),
        int(gate_activation == "sigmoid"), _stream()), "gated_group_norm")


def min_gru(z: torch.Tensor, u: torch.Tensor, g: torch.Tensor, z_bias: Optional[torch.Tensor],
            u_bias: Optional[torch.Tensor], state: torch.Tensor, out: torch.Tensor,
            row_slot: torch.Tensor, seg: Optional[torch.Tensor]) -> None:
    """Per request and channel ``S <- (1 - s) S + s c`` over the rows of the step in order, with
    ``s = sigmoid(z + z_bias)`` and the candidate ``c = w + 1/2`` where ``w = u + u_bias >= 0``,
    ``sigmoid(w)`` elsewhere; ``out = S * silu(g)``.  z, u, g: float32 column ranges of one
    matrix (equal row strides); state float32 [slots, >= channels],
    carried from step to step; out [rows, channels].  ``seg``: the table of
    :func:`segment_table`, or None when every row is a request of its own."""
    _cuda(z, u, g, z_bias, u_bias, state, out, row_slot, seg)
    for t in (z, u, g, state):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    rows, width = out.shape
    assert z.shape == u.shape == g.shape == (rows, width) and out.stride(1) == 1
    assert z.stride(0) == u.stride(0) == g.stride(0) and state.shape[1] >= width
    for b in (z_bias, u_bias):
        assert b is None or (b.dtype == torch.float32 and b.numel() == width)
    _check(lib().llm_min_gru(_ptr(z), _ptr(u), _ptr(g), z.stride(0), _ptr(z_bias), _ptr(u_bias),
                             _ptr(state), state.stride(0), _ptr(out), _dt(out), out.stride(0),
                             _ptr(row_slot), _ptr(seg), rows, state.shape[0], int(seg is None),
                             width, _stream()), "min_gru")
    global launches
    launches += 1          # the gates are a launch of their own


NORM_NONE, NORM_PER_HEAD, NORM_WHOLE_ROW = 0, 1, 2


def qkv_store(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
              q_out: torch.Tensor, view, row_slot: torch.Tensor, row_pos: torch.Tensor,
              num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, head_dim: int,
              norm: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
              eps: float, rot_dim: int = 0, cos_sin: Optional[torch.Tensor] = None,
              q_temp: Optional[Tuple[float, int]] = None,
              blend: Optional[Tuple[torch.Tensor, float]] = None) -> None:
    """Norm, rotation and stores for the rows of a step.  q float32 [rows, heads * key_dim],
    k [rows, kv_heads * key_dim], v [rows, kv_heads * value_dim] (column slices are fine; k and
    v None: only the queries).  ``norm``: NORM_NONE, NORM_PER_HEAD (weights [key_dim], shared by
    the heads) or NORM_WHOLE_ROW (weights of the whole q and k rows).  ``rot_dim`` > 0: the
    pairs (2i, 2i + 1) of every q and k head are turned by ``cos_sin`` (float32
    [rows, rot_dim / 2, 2]).  q goes to ``q_out`` [rows, heads * head_dim], k and v into the
    pages of ``view``; ``head_dim`` >= both sizes is the cache's row, padded with zeros.
    ``q_temp = (coef, every)``: the queries of position p are multiplied by
    ``1 + coef ln(floor((p + 1) / every) + 1)``.  ``blend = (v0, lam)``: what is stored as the
    value is ``(1 - lam) v + lam v0`` with v0 float32 of v's shape (a column slice is fine)."""
    _cuda(q, k, v, q_out, q_weight, k_weight, cos_sin, row_slot, row_pos)
    coef, every = q_temp if q_temp is not None else (0.0, 0)
    v0, lam = blend if blend is not None and k is not None else (None, 0.0)
    if v0 is not None:
        _cuda(v0)
        assert v0.dtype == torch.float32 and v0.stride(1) == 1 and v0.shape == v.shape
    rows = q.shape[0]
    has_kv = k is not None
    for t in (q, k, v):
        assert t is None or (t.dtype == torch.float32 and t.stride(1) == 1)
    assert q_out.is_contiguous() and q_out.shape == (rows, num_heads * head_dim)
    assert not has_kv or view.k.dtype == q_out.dtype
    if rot_dim:
        assert cos_sin is not None and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
        assert cos_sin.shape == (rows, rot_dim // 2, 2)
    for w, n in ((q_weight, num_heads), (k_weight, num_kv_heads)):
        if norm != NORM_NONE and w is not None:
            assert w.dtype == torch.float32 and w.is_contiguous()
            assert w.numel() == (key_dim if norm == NORM_PER_HEAD else n * key_dim)
    _check(lib().llm_qkv_store_mix(
        _ptr(q), q.stride(0), _ptr(k), k.stride(0) if has_kv else 0, _ptr(v),
        v.stride(0) if has_kv else 0, _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin), _ptr(q_out),
        _ptr(view.k) if has_kv else None, _ptr(view.v) if has_kv else None, _dt(q_out),
        view.page_stride, _ptr(view.block_table), view.block_table.stride(0), _ptr(row_slot),
        _ptr(row_pos), rows, num_heads, num_kv_heads, key_dim, value_dim, head_dim, rot_dim, norm,
        float(eps), view.page_size, int(has_kv), float(coef), int(every), _ptr(v0),
        v0.stride(0) if v0 is not None else 0, float(lam), _stream()), "qkv_store")


def pool_blocks(view, pooled_view, row_slot: torch.Tensor, row_pos: torch.Tensor, rows: int,
                num_kv_heads: int, head_dim: int, pool: int) -> None:
    """Every row of the step whose position ends a block of ``pool`` tokens writes the block's
    entry of the pooled cache: the means of its cached keys and of its cached values."""
    _cuda(view.k, view.v, pooled_view.k, pooled_view.v, row_slot, row_pos)
    assert view.page_size == pooled_view.page_size and view.k.dtype == pooled_view.k.dtype
    _check(lib().llm_pool_blocks(
        _ptr(view.k), _ptr(view.v), view.page_stride, _ptr(view.block_table),
        view.block_table.stride(0), _ptr(pooled_view.k), _ptr(pooled_view.v),
        pooled_view.page_stride, _ptr(pooled_view.block_table), pooled_view.block_table.stride(0),
        _ptr(row_slot), _ptr(row_pos), _dt(view.k), rows, num_kv_heads, head_dim, view.page_size,
        pool, _stream()), "pool_blocks")


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out.flat[i] = mean + std * z(key, first + i), z a standard normal that is a function of
    the key and the index alone (the same bits as ``weights.random_normal`` gives on a host)."""
    _cuda(out)
    assert out.is_contiguous()
    _check(lib().llm_random_normal(_ptr(out), _dt(out), out.numel(), int(key), float(mean),
                                   float(std), int(first), _stream()), "random_normal")


# ------------------------------------------------------------------------------------------
# dispatch: which kernel serves which dtype and size
# ------------------------------------------------------------------------------------------
GEMV_MAX_ROWS = 8


def _gemv_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and a.shape[0] <= GEMV_MAX_ROWS and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, half: int = 0
              ) -> None:
    """Weight-streaming product for up to 8 rows.  mode 0: out = a w^T; 1: out += a w^T
    (float32); 2: out = silu(a wg^T) * (a wu^T) with w = [wg; wu], ``half`` rows each."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _check(lib().llm_gemv_bf16(_ptr(a), _ptr(w), _ptr(out), _dt(out), M, N, K, a.stride(0),
                               w.stride(0), out.stride(0), mode, half, _stream()), "gemv_bf16")


_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """The device word in which the tensor-core kernels record a wait that gave up."""
    st = _tc_status.get(device)          # (keyed by the device object first: no conversions)
    if st is None:
        key = torch.device(device).index or 0
        if key not in _tc_status:
            _tc_status[key] = torch.zeros(4, dtype=torch.int32, device=device)
        st = _tc_status[device] = _tc_status[key]
    return st


status_words = tc_status       # word 0: a wait that gave up; word 1: 1 + row of a bad token id


def status_message(words) -> Optional[str]:
    """What non-zero status words say, or None when all is well."""
    if words[0]:
        return f"a tcgen05 / TMA kernel gave up waiting on a barrier (role {int(words[0])})"
    if words[1]:
        return f"token id outside the embedding table at row {int(words[1]) - 1} of a step"
    return None


def clear_status(device) -> None:
    st = _tc_status.get(torch.device(device).index or 0)
    if st is not None:
        st.zero_()


def check_tc_status(device) -> None:
    """Raise if a kernel recorded a failure in the status words: a tensor-core kernel that gave
    up waiting, or a token id outside the embedding table (synchronises the device; the words
    are cleared)."""
    st = _tc_status.get(torch.device(device).index or 0)
    if st is not None:
        msg = status_message(st.tolist())
        if msg:
            st.zero_()
            raise KernelError(msg)


def selftest_wait_gives_up(device, limit_cycles: int = 20000) -> None:
    """Launch a one-block kernel that waits on a barrier at which nothing ever arrives, with a
    limit of ``limit_cycles`` clock cycles (microseconds) instead of the two seconds of the real
    kernels.  It gives up, records role 99 in the status words and returns: the way every
    bounded wait of the TMA / tcgen05 kernels ends, made to happen without a fault."""
    l = lib()
    l.llm_selftest_wait_gives_up.argtypes = [c_void_p, c_longlong, c_void_p]
    l.llm_selftest_wait_gives_up.restype = c_int
    _check(l.llm_selftest_wait_gives_up(_ptr(status_words(device)), int(limit_cycles), _stream()),
           "selftest_wait_gives_up")


def token_tile(rows: int) -> int:
    """Tokens per tile of the tensor-core product: the smallest tile that holds the rows, 256
    (the persistent kernel) once there are enough rows to fill the GPU with such tiles."""
    for bn in (16, 32, 64, 128):
        if rows <= bn:
            return bn
    return 256 if rows >= 512 else 128


def _tc_ok(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> bool:
    """Whether the tensor-core product takes these operands: 16-bit, and every row of every
    operand (the output's too: it leaves through a TMA store) starts on a 16-byte boundary."""
    if out is not None and ((out.stride(0) * out.element_size()) % 16 or out.data_ptr() % 16
                            or out.stride(1) != 1):
        return False
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1
            and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def use_cta_pairs(on: bool) -> None:
    """Whether products of many rows run on CTA pairs (tcgen05 cta_group::2; the default) or on
    the one-CTA persistent kernel.  For comparisons."""
    l = lib()
    l.llm_set_pair.argtypes = [c_int]
    l.llm_set_pair.restype = None
    l.llm_set_pair(int(on))


def force_pair_k_ranges(n: int) -> None:
    """Cut K into ``n`` ranges in the CTA-pair product that adds into its output, whatever its
    own cost model would choose; 0 gives the choice back to the model.  For measurements."""
    l = lib()
    l.llm_set_pair_ksplits.argtypes = [c_int]
    l.llm_set_pair_ksplits.restype = None
    l.llm_set_pair_ksplits(int(n))


_dependent_launch = True


def use_dependent_launch(on: bool) -> None:
    """Whether kernels are launched as programmatic dependents of the one before them (the
    default) or wait for its end.  For measurements, and see :func:`plain_stream_order`."""
    global _dependent_launch
    l = lib()
    l.llm_set_pdl.argtypes = [c_int]
    l.llm_set_pdl.restype = None
    l.llm_set_pdl(int(on))
    _dependent_launch = bool(on)


@contextlib.contextmanager
def plain_stream_order():
    """Kernels launched inside start only when the kernel before them has ended, whatever
    :func:`use_dependent_launch` says; the setting is put back afterwards."""
    was = _dependent_launch
    if was:
        use_dependent_launch(False)
    try:
        yield
    finally:
        if was:
            use_dependent_launch(True)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, half: int = 0,
                 bn: Optional[int] = None, splits: int = 1, out_is_zero: bool = False) -> None:
    """Tensor-core product of bfloat16 operands.  mode 0: out = a w^T (bfloat16 or float32);
    1: out += a w^T (float32); 2: out = silu(a wg^T) * (a wu^T), w = [wg; wu] of ``half`` rows
    each; 3: the same with w stored as alternating blocks of 16 gate rows and 16 up rows.
    ``bn``: token tile (16..256); ``splits`` > 1 splits K and adds partial sums with atomics
    (mode 0 then needs ``out`` float32, zeroed here unless ``out_is_zero``)."""
    _cuda(a, w, out)
    T, K = a.shape
    N = w.shape[0]
    assert out.stride(1) == 1
    bn = bn or token_tile(T)
    _check(lib().llm_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(out), _dt(out), T, N, K, a.stride(0),
                                  w.stride(0), out.stride(0), mode, half, bn, splits,
                                  int(out_is_zero), _ptr(tc_status(a.device)), _stream()),
           "gemm_tcgen05")


_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the device in use (148 on a B200; asked once)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device())
                     .multi_processor_count if torch.cuda.is_available() else 148)
    return _sm_count

# Up to this many rows a caller may keep a split-K destination at zero itself (the kernel that
# consumes it clears it) instead of having it cleared before every product.
SPLIT_K_MAX_ROWS = 256


def k_splits(rows: int, out_features: int, in_features: int) -> int:
    """How many ways to split K so that a product with few output tiles still fills the GPU."""
    tiles = -(-out_features // 128) * -(-rows // token_tile(rows))
    if tiles >= 2 * sm_count() - 40:
        return 1
    # two CTAs fit an SM: aim at one full wave of two CTAs per SM, at least 256 of K each
    return max(1, min(16, round(2 * sm_count() / tiles), in_features // 256))


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
           out_is_zero: bool = False) -> None:
    """out (=|+=) a @ w.T with the fastest hand-written kernel that takes these operands:
    tensor cores for bfloat16 (they fetch weights ahead of the kernel before them), the
    CUDA-core kernels for everything else (32-bit operands, unaligned sizes).
    ``out_is_zero``: the caller guarantees that ``out`` holds zeros, so a split-K product need
    not clear it first."""
    if _tc_ok(a, w, out):
        rows, k = a.shape
        n = w.shape[0]
        splits = k_splits(rows, n, k) if out.dtype == torch.float32 else 1
        gemm_tcgen05(a, w, out, 1 if accumulate else 0, splits=splits, out_is_zero=out_is_zero)
    elif _gemv_ok(a, w):
        gemv_bf16(a, w, out, 1 if accumulate else 0)
    else:
        gemm_simt(a, w, out, accumulate)


def gated_interleave_ok(gate: torch.Tensor, up: torch.Tensor) -> bool:
    """Whether the gate and up matrices can be stored interleaved for the tensor-core product."""
    return (gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.is_cuda
            and gate.shape == up.shape and gate.shape[0] % 16 == 0 and gate.shape[1] % 8 == 0)


def gate_up_silu(ctx, h: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor,
                 interleaved: bool = False) -> None:
    """act = silu(h Wg^T) * (h Wu^T) for Wg, Wu stacked in ``w_gate_up`` ([2 ff][hidden]):
    gate rows then up rows, or (``interleaved``) alternating blocks of 16 gate and 16 up rows."""
    rows, ff = act.shape
    if interleaved:
        if not _tc_ok(h, w_gate_up, act):
            raise KernelError("interleaved gate/up weights need the tensor-core product")
        gemm_tcgen05(h, w_gate_up, act, 3, ff)
        return
    if _tc_ok(h, w_gate_up, act):
        gemm_tcgen05(h, w_gate_up, act, 2, ff)
        return
    if _gemv_ok(h, w_gate_up):
        gemv_bf16(h, w_gate_up, act, 2, ff)
        return
    gu = ctx.buffer("ffn.gate_up", (rows, 2 * ff), torch.float32)
    linear(h, w_gate_up, gu)
    silu_mul(gu, act)


FLASH_HEAD_DIMS = (32, 64, 128)
ATTENTION_MAX_HEAD_DIM = 640      # MAX_HD of attention_generic.cu, the kernel of last resort


def attention_refusal(num_heads: int, num_kv_heads: int, head_dim: int) -> Optional[str]:
    """Why no attention kernel of this library takes these sizes, or None when one does (the
    generic kernel takes every head size up to 256 and every group)."""
    if head_dim <= 0 or head_dim > ATTENTION_MAX_HEAD_DIM:
        return (f"head_dim {head_dim}: the attention kernels take head sizes up to "
                f"{ATTENTION_MAX_HEAD_DIM}")
    if num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
        return f"{num_heads} query heads cannot be shared among {num_kv_heads} KV heads"
    return None


def attention_flash(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                    items: Optional[torch.Tensor], n_items: int, rows_per_cta: int,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                    scale: float, window: Optional[int], splits: int = 1,
                    part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                    row_slot: Optional[torch.Tensor] = None,
                    row_pos: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention over the paged cache for ``n_items`` work items (int32 quadruples
    first row, tokens, request slot, first position); without ``items`` every row is an item
    of one token given by ``row_slot`` / ``row_pos``.  With ``splits`` > 1 the result is left
    in ``part_o`` / ``part_ml`` for :func:`attention_merge`."""
    _cuda(q, out, k_cache, v_cache, block_table, items, part_o, part_ml, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    _check(lib().llm_attention_flash(
        _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(k_cache), _ptr(v_cache),
        page_stride, _ptr(block_table), block_table.stride(0), _ptr(items), _ptr(row_slot),
        _ptr(row_pos), n_items, rows_per_cta, num_heads, num_kv_heads, head_dim, page_size,
        float(scale), int(window or 0), splits, _stream()), f"attention_flash (head_dim {head_dim})")


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                     v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                     items: Optional[torch.Tensor], n_items: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: Optional[int], splits: int = 1,
                     part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                     row_slot: Optional[torch.Tensor] = None,
                     row_pos: Optional[torch.Tensor] = None) -> None:
    """Decode form of the tensor-core attention: items of at most eight (token, head of the
    group) pairs, keys on the M side of the tile.  Arguments as :func:`attention_flash`."""
    _cuda(q, out, k_cache, v_cache, block_table, items, part_o, part_ml, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    _check(lib().llm_attention_decode(
        _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(k_cache), _ptr(v_cache),
        page_stride, _ptr(block_table), block_table.stride(0), _ptr(items), _ptr(row_slot),
        _ptr(row_pos), n_items, num_heads, num_kv_heads, head_dim, page_size, float(scale),
        int(window or 0), splits, _stream()), f"attention_decode (head_dim {head_dim})")


def attention_decode_tma(q: torch.Tensor, out: torch.Tensor, storage: torch.Tensor, slot: int,
                         block_table: torch.Tensor, items: Optional[torch.Tensor], n_items: int,
                         num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         scale: float, window: Optional[int], splits: int = 1,
                         part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None,
                         row_slot: Optional[torch.Tensor] = None,
                         row_pos: Optional[torch.Tensor] = None) -> None:
    """As :func:`attention_decode`, with K and V fetched by TMA tile loads from the group's
    whole cache tensor ``storage`` [pages, slots, 2, kv heads, page size, head dim]."""
    _cuda(q, out, storage, block_table, items, part_o, part_ml, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and storage.dtype == torch.bfloat16
    assert storage.is_contiguous() and storage.dim() == 6
    _check(lib().llm_attention_decode_tma(
        _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(storage), storage.shape[0],
        storage.shape[1], slot, _ptr(block_table), block_table.stride(0), _ptr(items),
        _ptr(row_slot), _ptr(row_pos), n_items, num_heads, num_kv_heads, head_dim, page_size,
        float(scale), int(window or 0), splits, _ptr(tc_status(q.device)), _stream()),
        f"attention_decode_tma (head_dim {head_dim})")


def attention_decode_persistent(q: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                                storage: torch.Tensor, slot: int, block_table: torch.Tensor,
                                row_slot: torch.Tensor, row_pos: torch.Tensor, num_heads: int,
                                num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                                window: Optional[int], parts: int, ctas: Optional[int] = None) -> None:
    """Decode attention of one new token per row with the tiles of all (row, KV head) units
    shared evenly by ``ctas`` one-warp CTAs (default: what the GPU holds at once).  Leaves
    ``parts`` parts per (row, head) in ``part_o`` / ``part_ml`` (some marked empty) for
    :func:`attention_merge` with ``splits = parts``."""
    _cuda(q, part_o, part_ml, storage, block_table, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and storage.dtype == torch.bfloat16
    assert storage.is_contiguous() and storage.dim() == 6
    rows = q.shape[0]
    assert part_o.numel() >= rows * num_heads * parts * head_dim
    _check(lib().llm_attention_decode_persistent(
        _ptr(q), _ptr(part_o), _ptr(part_ml), _ptr(storage), storage.shape[0], storage.shape[1],
        slot, _ptr(block_table), block_table.stride(0), _ptr(row_slot), _ptr(row_pos), rows,
        num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0), parts,
        int(ctas or DECODE_TMA_CTAS_PER_SM * sm_count()), _ptr(tc_status(q.device)), _stream()),
        f"attention_decode_persistent (head_dim {head_dim})")


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                      items: torch.Tensor, n_items: int, num_heads: int, num_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: Optional[int],
                      n_pages: int = 0, persistent: bool = True,
                      sink: Optional[torch.Tensor] = None,
                      outside: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> None:
    """Attention of prompt portions on tcgen05: items of at most 128 / (heads per KV head)
    tokens; scores and output accumulate in tensor memory.  ``n_pages``: pages of the cache that
    ``k_cache`` / ``v_cache`` are planes of; given it, pages of 32 positions or more are
    fetched by TMA, and with ``persistent`` and more (item, KV head) pairs than SMs one CTA per
    SM walks its share of the pairs.  ``sink`` (float32 [heads]) joins every row's sum as
    ``exp(sink)``; ``outside``: the two buffers of :func:`attention_outside`, one more part of
    every row's softmax."""
    eo, eml = outside if outside is not None else (None, None)
    _cuda(q, out, k_cache, v_cache, block_table, items, sink, eo, eml)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous()
    _check(lib().llm_attention_tcgen05_extra(
        _ptr(q), _ptr(out), q.shape[0], _ptr(k_cache), _ptr(v_cache), page_stride, int(n_pages),
        _ptr(block_table), block_table.stride(0), _ptr(items), n_items, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), int(persistent),
        _ptr(tc_status(q.device)), _ptr(sink), _ptr(eo), _ptr(eml), _stream()),
        f"attention_tcgen05 (head_dim {head_dim})")


def attention_outside(q: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor, view,
                      row_slot: torch.Tensor, row_pos: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: int,
                      sink: Optional[torch.Tensor] = None, keep_first: int = 0, pool: int = 0,
                      pooled_view=None) -> None:
    """What every row of a step sees outside its window of the last ``window`` keys, as one part
    of its softmax per head: the first ``keep_first`` keys of its sequence that the window has
    passed, the entries of ``pooled_view`` (one per block of ``pool`` positions) whose blocks
    lie wholly behind the window, and ``exp(sink)``.  part_o float32 [rows, heads, head_dim]
    (weighted values, not divided), part_ml float32 [rows, heads, 2] (the maximum as a base-2
    logarithm, the sum of weights): :func:`attention_tcgen05` and :func:`attention_merge` take
    them in.  bfloat16."""
    pk = pv = pt = None
    pstride = ptstride = 0
    if pool:
        pk, pv, pt = pooled_view.k, pooled_view.v, pooled_view.block_table
        pstride, ptstride = pooled_view.page_stride, pt.stride(0)
    _cuda(q, part_o, part_ml, view.k, view.v, view.block_table, row_slot, row_pos, sink, pk, pv, pt)
    assert q.dtype == torch.bfloat16 and view.k.dtype == torch.bfloat16 and q.is_contiguous()
    assert part_o.dtype == part_ml.dtype == torch.float32
    rows = q.shape[0]
    assert part_o.numel() >= rows * num_heads * head_dim and part_ml.numel() >= rows * num_heads * 2
    _check(lib().llm_attention_extras(
        _ptr(q), _ptr(part_o), _ptr(part_ml), _ptr(view.k), _ptr(view.v), view.page_stride,
        _ptr(view.block_table), view.block_table.stride(0), _ptr(row_slot), _ptr(row_pos), rows,
        num_heads, num_kv_heads, head_dim, view.page_size, float(scale), int(window), _ptr(sink),
        int(keep_first), _ptr(pk), _ptr(pv), pstride, _ptr(pt), ptstride, int(pool), _stream()),
        f"attention_outside (head_dim {head_dim})")


def attention_tcgen05_x2(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                         v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                         items: torch.Tensor, n_items: int, num_heads: int, num_kv_heads: int,
                         head_dim: int, page_size: int, scale: float, window: Optional[int],
                         n_pages: int) -> None:
    """As :func:`attention_tcgen05` with two query tiles per CTA: items of at most
    2 * 128 / (heads per KV head) tokens.  Pages of a power of two of at least 32 positions."""
    _cuda(q, out, k_cache, v_cache, block_table, items)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous()
    _check(lib().llm_attention_tcgen05_x2(
        _ptr(q), _ptr(out), q.shape[0], _ptr(k_cache), _ptr(v_cache), page_stride, int(n_pages),
        _ptr(block_table), block_table.stride(0), _ptr(items), n_items, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), _ptr(tc_status(q.device)),
        _stream()), f"attention_tcgen05_x2 (head_dim {head_dim})")


def decode_tma_ok(view, head_dim: int) -> bool:
    st = getattr(view, "storage", None)
    ps = view.page_size
    return (st is not None and st.is_contiguous() and head_dim in (64, 128)
            and ps & (ps - 1) == 0 and st.shape[0] * st.shape[1] * 2 < (1 << 31))


def attention_merge(part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor,
                    rows: Optional[torch.Tensor], n_rows: int, num_heads: int, head_dim: int,
                    splits: int, clear: Optional[torch.Tensor] = None,
                    sink: Optional[torch.Tensor] = None,
                    outside: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> None:
    """Merge the parts of split keys.  ``clear`` (float32 [rows, >= heads * head_dim]): the
    first heads * head_dim values of every merged row of it are zeroed as well.  ``sink`` and
    ``outside`` as in :func:`attention_tcgen05`."""
    eo, eml = outside if outside is not None else (None, None)
    _cuda(part_o, part_ml, out, rows, clear, sink, eo, eml)
    _check(lib().llm_attention_merge_extra(
        _ptr(part_o), _ptr(part_ml), _ptr(out), _ptr(rows), n_rows, num_heads, head_dim, splits,
        _ptr(clear), clear.stride(0) if clear is not None else 0, _ptr(sink), _ptr(eo), _ptr(eml),
        _stream()), "attention_merge")


FUSE_DECODE = "few waves"     # or "always" / "never": for measurements (see fuse_decode)


def fuse_decode(mode: str) -> None:
    """When decode attention runs fused with the rotation and the cache write: "few waves" (the
    default), "always" or "never".  For measurements; sets it for parts driven from Python and
    for the native step driver alike."""
    global FUSE_DECODE
    code = {"few waves": 0, "always": 1, "never": 2}[mode]
    FUSE_DECODE = mode
    l = lib()
    l.llm_set_fuse_decode.argtypes = [c_int]
    l.llm_set_fuse_decode.restype = None
    l.llm_set_fuse_decode(code)


def decode_fusion_ok(ctx, view, num_heads: int, num_kv_heads: int, head_dim: int, rot_dim: int,
                     cos_sin: Optional[torch.Tensor], window: Optional[int] = None) -> bool:
    """Whether the step runs norm, rotation, cache write and attention as one kernel: every
    row a single new token, 16-bit, whole heads rotated by the step's table of cosines and
    sines, a cache the TMA decode kernel takes, and at most two waves of CTAs (every wave pays
    the longer start of the fused kernel; from about four waves on that costs more than the
    separate rotation kernel: Qwen3-8B sizes at batch 64, 5.71 against 5.67 ms a step)."""
    if FUSE_DECODE == "never":
        return False
    ok = (ctx.dtype == torch.bfloat16 and cos_sin is not None and rot_dim == head_dim
          and num_heads // num_kv_heads <= 8 and decode_tma_ok(view, head_dim)
          and all(s.rows == 1 for s in ctx.segments))
    if not ok or FUSE_DECODE == "always":
        return ok
    reach = min(ctx.max_pos + 1, window) if window else ctx.max_pos + 1
    resident = DECODE_TMA_CTAS_PER_SM * sm_count()
    return (ctx.rows * num_kv_heads * decode_splits(ctx.rows, num_kv_heads, reach, resident,
                                                   DECODE_TMA_TILE) <= 2 * resident)


def attention_decode_fused(ctx, proj: torch.Tensor, out: torch.Tensor, view, writes_cache: bool,
                           q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                           cos_sin: torch.Tensor, eps: float, clear: bool, num_heads: int,
                           num_kv_heads: int, head_dim: int, scale: float,
                           window: Optional[int], splits: Optional[int] = None) -> None:
    """A decode step's attention from the output of the q/k/v product ``proj`` (float32
    [rows, (heads + 2 kv heads) * head_dim], or only the queries when another call owns the
    cache): per-head norm, rotation, write of the new key and value, attention over the cache
    and, with split keys, the merge.  With ``clear`` what was consumed of ``proj`` is zeroed."""
    _cuda(proj, out, view.storage, view.block_table, ctx.row_slot, ctx.row_pos, q_norm_w,
          k_norm_w, cos_sin)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and out.dtype == torch.bfloat16
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    rows = ctx.rows
    reach = min(ctx.max_pos + 1, window) if window else ctx.max_pos + 1
    if splits is None:
        splits = decode_splits(rows, num_kv_heads, reach, DECODE_TMA_CTAS_PER_SM * sm_count(),
                               DECODE_TMA_TILE)
    part_o = part_ml = None
    if splits > 1:
        part_o = ctx.buffer("attn.part_o", (rows * num_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.buffer("attn.part_ml", (rows * num_heads * splits * 2,), torch.float32)
    st = view.storage
    _check(lib().llm_attention_decode_fused(
        _ptr(proj), proj.stride(0), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(st), st.shape[0],
        st.shape[1], view.slot, _ptr(view.k if writes_cache else None),
        _ptr(view.v if writes_cache else None), view.page_stride, _ptr(view.block_table),
        view.block_table.stride(0), _ptr(ctx.row_slot), _ptr(ctx.row_pos), rows, _ptr(q_norm_w),
        _ptr(k_norm_w), _ptr(cos_sin), float(eps), int(clear), num_heads, num_kv_heads, head_dim,
        view.page_size, float(scale), int(window or 0), splits, _ptr(tc_status(proj.device)),
        _stream()), f"attention_decode_fused (head_dim {head_dim})")
    if splits > 1:
        attention_merge(part_o, part_ml, out, None, rows, num_heads, head_dim, splits,
                        clear=proj if clear else None)


def decode_splits(n_items: int, num_kv_heads: int, max_len: int, resident: int = 592,
                  tile: int = 32) -> int:
    """Parts into which the keys of a one-token item are cut.  ``resident``: how many CTAs of
    the kernel the GPU holds at once; ``tile``: keys of the kernel's tiles (parts are whole
    tiles).  The cost of a choice is modelled as waves of CTAs times the length of one CTA's
    walk (its keys, in units of 32, plus a fixed start-up worth about 96 keys), plus the merge,
    which grows with the number of parts; measured step times at batch 1, 8 and 64 and contexts
    of 1024 and 4096 keys rank the choices the same way."""
    ctas = max(1, n_items * num_kv_heads)
    tiles = max(1, -(-max_len // tile))
    best, best_cost = 1, None
    for s in range(1, min(32, max(1, max_len // 64)) + 1):
        waves = -(-ctas * s // resident)
        cost = waves * (-(-tiles // s) * (tile // 32) + 3) + 0.1 * s
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


DECODE_TMA_TILE = 32      # keys of a tile of attention_decode_tma.cu
DECODE_TMA_CTAS_PER_SM = 4    # its one-warp CTAs that fit an SM at head size 128
PERSISTENT_ATTENTION_MAX_KEYS = 6144


# ---------------------------------------------------------------------------------------------
# parts that other designs than the first two brought: several residual streams, a matrix memory
# with exponential gates, attention through latents, routed experts, other activations

def log_gate_scan(zi: torch.Tensor, zf: torch.Tensor, bias_i: Optional[torch.Tensor],
                  bias_f: Optional[torch.Tensor], cap: float, m_state: torch.Tensor,
                  out: torch.Tensor, row_slot: torch.Tensor, seg: Optional[torch.Tensor],
                  heads: int, n_requests: int = 0) -> None:
    """The exponential gates of a matrix memory per (row, head), kept in range by a running
    maximum ``m`` that is carried per request in ``m_state`` ([slots, >= heads] float32 view):
    ``i = cap tanh((zi + bias_i) / cap)``, ``f = log sigmoid(cap tanh((zf + bias_f) / cap))``
    (``cap`` 0: no cap), ``m_t = max(f_t + m_(t-1), i_t)``; ``out[row]`` = [exp(f + m_(t-1) -
    m_t) | exp(i - m_t) | m_t], each ``heads`` wide.  zi, zf: float32 [rows, heads] with equal
    row strides."""
    _cuda(zi, zf, bias_i, bias_f, m_state, out, row_slot, seg)
    rows = zi.shape[0]
    assert zi.dtype == zf.dtype == out.dtype == m_state.dtype == torch.float32
    assert zi.stride(0) == zf.stride(0) and zi.stride(1) == 1 and zf.stride(1) == 1
    assert out.shape == (rows, 3 * heads) and out.stride(1) == 1 and m_state.stride(1) == 1
    _check(lib().llm_log_gate_scan(_ptr(zi), _ptr(zf), zi.stride(0), _ptr(bias_i), _ptr(bias_f),
                                   float(cap), _ptr(m_state), m_state.stride(0), _ptr(out),
                                   out.stride(0), _ptr(seg), _ptr(row_slot), rows, int(n_requests),
                                   int(seg is None), heads, _stream()), "log_gate_scan")


def memory_out_norm(o: torch.Tensor, m: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor,
                    out: torch.Tensor, heads: int, value_dim: int, eps: float,
                    floor: float) -> None:
    """``y = o[..., :V] / (max(|o[..., V]|, exp(-m)) + floor)`` per (row, head), then
    ``out = y / rms(y) * weight * sigmoid(gate)``.  o: float32 [rows, heads * (V + 1)]; m: float32
    [rows, heads] (a column slice is fine); gate: float32 [rows, heads * V] (a column slice is
    fine); weight: float32 [heads * V]; out: [rows, heads * V] in the activation type."""
    _cuda(o, m, gate, weight, out)
    rows = out.shape[0]
    assert o.dtype == m.dtype == gate.dtype == weight.dtype == torch.float32
    assert o.shape == (rows, heads * (value_dim + 1)) and o.stride(1) == 1 and m.stride(1) == 1
    assert gate.stride(1) == 1 and out.stride(1) == 1 and weight.numel() == heads * value_dim
    _check(lib().llm_memory_out_norm(_ptr(o), o.stride(0), _ptr(m), m.stride(0), _ptr(gate),
                                     gate.stride(0), _ptr(weight), _ptr(out), _dt(out),
                                     out.stride(0), rows, heads, value_dim, float(eps),
                                     float(floor), _stream()), "memory_out_norm")


STREAM_KEEP_WIDTH = 4096     # widest row of a stream step that does not store its new streams


def stream_step(xs: torch.Tensor, y: Optional[torch.Tensor] = None,
                mix: Optional[torch.Tensor] = None, out_coef: Optional[torch.Tensor] = None,
                clear_y: bool = False, store: bool = True,
                in_coef: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None,
                eps: float = 0.0, out: Optional[torch.Tensor] = None,
                rows_index: Optional[torch.Tensor] = None) -> None:
    """One sublayer boundary of a model with several residual streams ``xs`` (float32
    [S, rows, width]).  With ``y`` (float32 [rows, width]): ``xs[t] <- sum_s mix[s, t] xs[s] +
    out_coef[t] y`` for all t at once (``clear_y`` zeroes what was read of y).  With ``in_coef``:
    ``out = rms_norm(sum_s in_coef[s] xs[s]) * weight`` from the new streams.  ``rows_index``: the
    rows to work on (``out`` has one row per index), else all rows."""
    _cuda(xs, y, mix, out_coef, in_coef, weight, out, rows_index)
    S, rows, width = xs.shape
    assert xs.dtype == torch.float32 and xs.is_contiguous()
    if y is not None:
        assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (rows, width)
        assert mix.dtype == out_coef.dtype == torch.float32 and mix.is_contiguous()
        assert mix.numel() == S * S and out_coef.numel() == S
    n = rows
    if in_coef is not None:
        assert in_coef.dtype == weight.dtype == torch.float32 and in_coef.numel() == S
        assert weight.numel() == width and out.is_contiguous() and out.shape[1] == width
        n = out.shape[0]
    if rows_index is not None:
        assert rows_index.dtype == torch.int32 and rows_index.numel() == n
    _check(lib().llm_stream_step(_ptr(xs), xs.stride(0), S, _ptr(y), _ptr(mix), _ptr(out_coef),
                                 int(clear_y), int(store), _ptr(in_coef), _ptr(weight),
                                 float(eps), _ptr(out), _dt(out) if out is not None else F32,
                                 _ptr(rows_index), n, width, _stream()), "stream_step")


def stream_fill(xs: torch.Tensor) -> None:
    """xs[s] = xs[0] for every other stream s."""
    _cuda(xs)
    S, rows, width = xs.shape
    assert xs.dtype == torch.float32 and xs.is_contiguous()
    _check(lib().llm_stream_fill(_ptr(xs), xs.stride(0), S, rows, width, _stream()),
           "stream_fill")


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}
PLAIN_ACTIVATIONS = {"relu_squared": 3}


def gated_act(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              activation: str, clear: bool = False, limit: float = 0.0) -> None:
    """out[t][j] = act(gate_up[t][j] + bias[j]) * (gate_up[t][ff + j] + bias[ff + j]).
    ``clear``: gate_up is zeroed once read (a buffer that is kept at zero between steps).
    ``clamped_swish`` with ``limit`` L: with g = min(gate, L) and u = clamp(up, -L, L) the result
    is g * sigmoid(1.702 g) * (u + 1)."""
    _cuda(gate_up, bias, out)
    rows, ff = out.shape
    assert gate_up.dtype == torch.float32 and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.shape == (rows, 2 * ff)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * ff)
    _check(lib().llm_gated_act_limit(_ptr(gate_up), _ptr(bias), _ptr(out), _dt(out), rows, ff,
                                     ACTIVATIONS[activation], int(clear), float(limit),
                                     _stream()), "gated_act")


def act_rows(x: torch.Tensor, out: torch.Tensor, activation: str, clear: bool = False) -> None:
    """out = act(x) for an activation without a gate (``relu_squared``: max(x, 0)^2); x float32,
    both contiguous and of one shape.  ``clear``: x is zeroed once read."""
    _cuda(x, out)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert x.shape == out.shape
    _check(lib().llm_act_rows(_ptr(x), _ptr(out), _dt(out), x.numel(),
                              PLAIN_ACTIVATIONS[activation], int(clear), _stream()), "act_rows")


def dual_norm_mean(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor,
                   y: torch.Tensor, eps: float, accumulate: bool = False) -> None:
    """y (=|+=) (unit(a) * wa + unit(b) * wb) / 2 row by row, unit(.) a row over its root mean square
    (eps inside the root); all float32, [rows, width]."""
    _cuda(a, b, wa, wb, y)
    for t in (a, b, wa, wb, y):
        assert t.dtype == torch.float32 and t.is_contiguous()
    rows, width = y.shape
    assert a.shape == b.shape == y.shape and wa.numel() == wb.numel() == width
    _check(lib().llm_dual_norm_mean(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), _ptr(y), rows, width,
                                    float(eps), int(accumulate), _stream()), "dual_norm_mean")


def scale_soft_cap(z: torch.Tensor, scale: float, cap: float) -> None:
    """z <- cap tanh(z scale / cap) in place (``cap`` 0: z <- z scale); float32, contiguous."""
    _cuda(z)
    assert z.dtype == torch.float32 and z.is_contiguous()
    _check(lib().llm_scale_soft_cap(_ptr(z), z.numel(), float(scale), float(cap), _stream()),
           "scale_soft_cap")


def latent_store(proj: torch.Tensor, q_weight: torch.Tensor, c_weight: torch.Tensor,
                 cos_sin: Optional[torch.Tensor], cq_out: torch.Tensor, view,
                 row_slot: torch.Tensor, row_pos: torch.Tensor, q_rank: int, kv_rank: int,
                 rot_dim: int, eps: float, write_cache: bool = True, clear: bool = False) -> None:
    """From proj (float32 [rows, >= q_rank + kv_rank + rot_dim]): the normed query latent into
    ``cq_out`` and the key row [normed latent | rotated key part] into the paged cache ``view``
    (K plane whole, V plane the latent alone).  ``cos_sin``: float32 [rows, pairs, 2]."""
    _cuda(proj, q_weight, c_weight, cos_sin, cq_out, view.k, view.v, row_slot, row_pos)
    rows = cq_out.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and cq_out.is_contiguous()
    assert cq_out.dtype == view.k.dtype and cq_out.shape[1] == q_rank
    half = 0 if cos_sin is None else cos_sin.shape[1]
    _check(lib().llm_latent_store(_ptr(proj), proj.stride(0), _ptr(q_weight), _ptr(c_weight),
                                  _ptr(cos_sin), half, _ptr(cq_out), _ptr(view.k), _ptr(view.v),
                                  _dt(cq_out), view.page_stride, _ptr(view.block_table),
                                  view.block_table.stride(0), _ptr(row_slot), _ptr(row_pos), rows,
                                  view.page_size, q_rank, kv_rank, rot_dim, float(eps),
                                  int(write_cache), int(clear), _stream()), "latent_store")


def latent_query(q: torch.Tensor, cos_sin: Optional[torch.Tensor], q_plain: torch.Tensor,
                 q_full: torch.Tensor, heads: int, dim: int, rot_dim: int, kv_rank: int,
                 clear: bool = False) -> None:
    """From q (float32 [rows, heads * (dim + rot_dim)]): every head's plain part rounded into
    ``q_plain`` [rows, heads * dim], its rotated part into ``q_full`` [rows, heads * (kv_rank +
    rot_dim)] behind the first kv_rank channels."""
    _cuda(q, cos_sin, q_plain, q_full)
    rows = q.shape[0]
    assert q.dtype == torch.float32 and q.stride(1) == 1
    assert q_plain.is_contiguous() and q_full.is_contiguous() and q_plain.dtype == q_full.dtype
    half = 0 if cos_sin is None else cos_sin.shape[1]
    _check(lib().llm_latent_query(_ptr(q), q.stride(0), _ptr(cos_sin), half, _ptr(q_plain),
                                  _ptr(q_full), _dt(q_full), rows, heads, dim, rot_dim, kv_rank,
                                  int(clear), _stream()), "latent_query")


HEAD_LINEAR_SIMT_ROWS = 128     # up to so many rows the per-head maps are one CUDA-core launch


def head_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """A map per head: ``out[r, h, :] = w[h] @ a[r, h, :]``.  a [rows, H, in] and out
    [rows, H, out_features] may be views with a row stride and a head stride (the last dimension dense); w
    [H, out_features, in] contiguous.  Many rows of bfloat16 operands whose rows are whole
    16-byte units go to the tensor-core product head by head; few rows (a launch per head would
    cost more than the arithmetic) and everything else to one batched CUDA-core launch."""
    _cuda(a, w, out)
    rows, H, k = a.shape
    n = w.shape[1]
    assert w.shape == (H, n, k) and w.is_contiguous() and out.shape == (rows, H, n)
    assert a.stride(2) == 1 and out.stride(2) == 1 and a.dtype == w.dtype
    if (rows > HEAD_LINEAR_SIMT_ROWS and a.dtype == torch.bfloat16 and k % 8 == 0
            and a.stride(0) % 8 == 0 and a.stride(1) % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and out.stride(1) >= n):
        # every head's product in one launch of the tensor-core kernel (its one-CTA form:
        # a head's product is small)
        _check(lib().llm_gemm_tcgen05_batched(_ptr(a), _ptr(w), _ptr(out), _dt(out), rows, n, k,
                                              a.stride(0), k, out.stride(0), 128, H, a.stride(1),
                                              out.stride(1), _ptr(tc_status(a.device)),
                                              _stream()), "head_linear")
        return
    _check(lib().llm_gemm_simt_batched(_ptr(a), _ptr(w), _ptr(out), _dt(a), _dt(out), rows, n, k,
                                       a.stride(0), k, out.stride(0), H, a.stride(1), n * k,
                                       out.stride(1), _stream()), "head_linear")


ROUTE_SOFTMAX_CHOSEN, ROUTE_SOFTMAX_ALL, ROUTE_SOFTMAX_ALL_RENORMED = 0, 1, 2
ROUTE_MODES = {"softmax_chosen": ROUTE_SOFTMAX_CHOSEN, "softmax_all": ROUTE_SOFTMAX_ALL,
               "softmax_all_renormed": ROUTE_SOFTMAX_ALL_RENORMED}


def _route_mode(scores: str, correction: Optional[torch.Tensor], experts: int) -> int:
    if scores not in ROUTE_MODES:
        raise KernelError(f"router scores '{scores}' ({', '.join(ROUTE_MODES)})")
    if correction is not None:
        assert scores != "softmax_chosen" and correction.dtype == torch.float32
        assert correction.is_contiguous() and correction.numel() == experts
    return ROUTE_MODES[scores]


def moe_route(z: torch.Tensor, experts: int, top: int, ids: torch.Tensor, wts: torch.Tensor,
              scores: str = "softmax_chosen", correction: Optional[torch.Tensor] = None,
              weight_scale: float = 1.0) -> None:
    """Per row the ``top`` largest of the first ``experts`` logits of z (float32, a column slice
    is fine) into ``ids`` (int32 [rows, top]) and the softmax over the chosen into ``wts``.
    ``scores="softmax_all"``: the scores are the softmax over all ``experts`` logits, the choice
    goes by score + ``correction`` (float32 [experts], optional), and a chosen expert's weight is
    its score, not renormalised.  ``"softmax_all_renormed"``: the same choice; the weights are the
    chosen scores over their sum (+ 1e-20), times ``weight_scale``."""
    _cuda(z, ids, wts, correction)
    mode = _route_mode(scores, correction, experts)
    rows = z.shape[0]
    assert z.dtype == torch.float32 and z.stride(1) == 1 and z.shape[1] >= experts
    assert ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (rows, top)
    assert wts.dtype == torch.float32 and wts.is_contiguous() and wts.shape == (rows, top)
    _check(lib().llm_moe_route_scaled(_ptr(z), z.stride(0), rows, experts, top, mode,
                                      _ptr(correction), _ptr(ids), _ptr(wts),
                                      float(weight_scale), _stream()), "moe_route")


def moe_router(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], experts: int,
               top: int, z: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor,
               scores: str = "softmax_chosen", correction: Optional[torch.Tensor] = None,
               weight_scale: float = 1.0) -> None:
    """Router logits ``z = h w^T + bias`` (w float32 [n_out, width], sums in 32-bit) and, over
    the first ``experts`` of them, the ``top`` largest per row into ``ids`` with the softmax over
    the chosen into ``wts``: the product and :func:`moe_route` in one launch (``scores``,
    ``correction`` and ``weight_scale`` as there)."""
    _cuda(h, w, bias, z, ids, wts, correction)
    mode = _route_mode(scores, correction, experts)
    rows, width = h.shape
    n_out = w.shape[0]
    assert w.dtype == torch.float32 and w.is_contiguous() and w.shape[1] == width
    assert h.is_contiguous() and z.dtype == torch.float32 and z.shape == (rows, n_out)
    assert z.stride(1) == 1 and (bias is None or (bias.dtype == torch.float32 and bias.numel() == n_out))
    assert ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (rows, top)
    assert wts.dtype == torch.float32 and wts.is_contiguous() and wts.shape == (rows, top)
    _check(lib().llm_moe_router_scaled(_ptr(h), _dt(h), _ptr(w), _ptr(bias), _ptr(z),
                                       z.stride(0), rows, width, experts, n_out, top, mode,
                                       _ptr(correction), _ptr(ids), _ptr(wts),
                                       float(weight_scale), _stream()),
           "moe_router")


def moe_gate_up_rows(h: torch.Tensor, gate_up: torch.Tensor, ids: torch.Tensor,
                     act: torch.Tensor, activation: str = "silu", limit: float = 0.0) -> None:
    """act[r, k] = silu(Wg_e h_r) * (Wu_e h_r), e = ids[r, k]; gate_up [E, 2 ff, width].  With
    ``activation="clamped_swish"`` the gated form of that name (see :func:`gated_act`).  A pair
    whose expert is not one of the E with matrices is left out.  ``activation="relu_squared"``:
    experts without a gate, ``gate_up`` [E, ff, width] holds their up matrices and
    act[r, k] = max(Wu_e h_r, 0)^2."""
    _cuda(h, gate_up, ids, act)
    if activation not in ("silu", "clamped_swish", "relu_squared"):
        raise KernelError(f"routed experts have no activation '{activation}'")
    rows, width = h.shape
    top = ids.shape[1]
    ff = gate_up.shape[1] if activation == "relu_squared" else gate_up.shape[1] // 2
    assert h.is_contiguous() and gate_up.is_contiguous() and act.is_contiguous()
    assert h.dtype == gate_up.dtype == act.dtype and act.shape == (rows, top, ff)
    _check(lib().llm_moe_gate_up_rows(_ptr(h), _ptr(gate_up), _ptr(ids), _ptr(act), _dt(h), rows,
                                      width, ff, top, gate_up.shape[0],
                                      {**ACTIVATIONS, **PLAIN_ACTIVATIONS}[activation],
                                      float(limit), _stream()), "moe_gate_up_rows")


def moe_down_rows(act: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor,
                  y: torch.Tensor, accumulate: bool, shared: Optional[torch.Tensor] = None,
                  shared_gate: Optional[torch.Tensor] = None, clear_shared: bool = False,
                  identity_input: Optional[torch.Tensor] = None) -> None:
    """y[r] (+)= sum_k wts[r, k] Wd_e act[r, k] (+ sigmoid(shared_gate[r]) shared[r]);
    down [E, width, ff]; y, shared float32 [rows, width]; shared_gate float32 [rows] (strided).
    ``identity_input`` ([rows, width], act's type): an expert index of E or more is an identity
    expert, whose output is that row."""
    _cuda(act, down, ids, wts, y, shared, shared_gate, identity_input)
    if identity_input is not None:
        assert identity_input.dtype == act.dtype and identity_input.is_contiguous()
    rows, top, ff = act.shape
    width = down.shape[1]
    assert act.is_contiguous() and down.is_contiguous() and act.dtype == down.dtype
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (rows, width)
    if shared is not None:
        assert shared.dtype == torch.float32 and shared.is_contiguous()
        assert shared_gate.dtype == torch.float32 and shared_gate.shape[0] == rows
    _check(lib().llm_moe_down_rows(_ptr(act), _ptr(down), _ptr(ids), _ptr(wts), _ptr(shared),
                                   _ptr(shared_gate),
                                   shared_gate.stride(0) if shared_gate is not None else 0,
                                   _ptr(y), _dt(act), rows, width, ff, top, int(accumulate),
                                   int(clear_shared),
                                   down.shape[0] if identity_input is not None else (1 << 30),
                                   _ptr(identity_input), _stream()), "moe_down_rows")


def moe_grouped_ok(h_dtype: torch.dtype, width: int, ff: int) -> bool:
    """Whether the routed experts of these sizes run as grouped tensor-core products."""
    return h_dtype == torch.bfloat16 and width % 8 == 0 and ff % 16 == 0


def moe_tile(pairs: int, experts: int) -> int:
    """Rows of a tile of the padded buffer: the smallest tile that holds an expert's average share."""
    share = -(-pairs // experts)
    for bn in (16, 32, 64):
        if share <= bn:
            return bn
    return 128


def moe_align(ids: torch.Tensor, experts: int, bn: int, pos: torch.Tensor,
              tile_group: torch.Tensor) -> None:
    """Sort the (row, choice) pairs of ``ids`` by expert: ``pos`` (int32 [pairs]) is each pair's
    row in a buffer in which every expert's rows start a tile of ``bn`` rows, ``tile_group``
    (int32 [tiles], tiles >= pairs / bn + experts) the expert of every tile or -1."""
    _cuda(ids, pos, tile_group)
    assert ids.dtype == pos.dtype == tile_group.dtype == torch.int32
    assert ids.is_contiguous() and pos.numel() == ids.numel()
    assert tile_group.numel() * bn >= ids.numel() + experts * (bn - 1)
    _check(lib().llm_moe_align(_ptr(ids), ids.numel(), experts, bn, tile_group.numel(), _ptr(pos),
                               _ptr(tile_group), _stream()), "moe_align")


def moe_gather(h: torch.Tensor, pos: torch.Tensor, xp: torch.Tensor, top: int,
               ids: Optional[torch.Tensor] = None, experts: int = 0) -> None:
    """xp[pos[i]] = h[i // top] (with ``ids``: only for pairs whose expert is below ``experts``)."""
    _cuda(h, pos, xp, ids)
    assert h.is_contiguous() and xp.is_contiguous() and h.dtype == xp.dtype
    assert h.shape[1] == xp.shape[1] and pos.numel() == h.shape[0] * top
    _check(lib().llm_moe_gather(_ptr(h), _ptr(pos), _ptr(xp), _dt(h), pos.numel(), h.shape[1], top,
                                _ptr(ids), int(experts), _stream()), "moe_gather")


def moe_combine(d: torch.Tensor, pos: torch.Tensor, wts: torch.Tensor, y: torch.Tensor,
                accumulate: bool, shared: Optional[torch.Tensor] = None,
                shared_gate: Optional[torch.Tensor] = None, clear_shared: bool = False,
                ids: Optional[torch.Tensor] = None, experts: int = 0,
                identity_input: Optional[torch.Tensor] = None) -> None:
    """y[r] (+)= sum_k wts[r, k] d[pos[r, k]] (+ sigmoid(shared_gate[r]) shared[r]).  With
    ``ids``: a pair whose expert is ``experts`` or more is an identity expert, whose output is
    the row of ``identity_input`` ([rows, width])."""
    _cuda(d, pos, wts, y, shared, shared_gate, ids, identity_input)
    if ids is not None:
        assert identity_input is not None and identity_input.stride(1) == 1
    rows, top = wts.shape
    width = y.shape[1]
    assert d.dtype == y.dtype == wts.dtype == torch.float32 and d.is_contiguous()
    assert y.is_contiguous() and d.shape[1] == width and pos.numel() == rows * top
    if shared is not None:
        assert shared.dtype == torch.float32 and shared.is_contiguous()
    _check(lib().llm_moe_combine(_ptr(d), _ptr(pos), _ptr(wts), _ptr(shared), _ptr(shared_gate),
                                 shared_gate.stride(0) if shared_gate is not None else 0, _ptr(y),
                                 rows, width, top, int(accumulate), int(clear_shared), _ptr(ids),
                                 int(experts), _ptr(identity_input),
                                 _dt(identity_input) if identity_input is not None else 0,
                                 identity_input.stride(0) if identity_input is not None else 0,
                                 _stream()),
           "moe_combine")


def gemm_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor,
                 bn: int, gated: bool) -> None:
    """The tensor-core product with a matrix per tile of ``bn`` rows of ``a``: tile t uses
    ``w[tile_group[t]]`` (w [groups, N, K] bfloat16; a negative entry leaves the tile out).
    ``gated``: w[g] = [gate; up] and out = silu(a gate^T) * (a up^T) ([rows, N / 2])."""
    _cuda(a, w, out, tile_group)
    T, K = a.shape
    G, N, _ = w.shape
    assert a.dtype == w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    assert out.stride(1) == 1 and tile_group.numel() * bn >= T
    _check(lib().llm_gemm_tcgen05_grouped(_ptr(a), _ptr(w), _ptr(out), _dt(out), T, N, K,
                                          a.stride(0), K, out.stride(0), 2 if gated else 0,
                                          N // 2 if gated else 0, bn, G, _ptr(tile_group),
                                          _ptr(tc_status(a.device)), _stream()), "gemm_grouped")
