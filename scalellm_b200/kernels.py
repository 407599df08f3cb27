"""Operator-level face of the B200 decode path: the reference's `src/kernels` free
functions, same names / argument order / in-place conventions, on torch CUDA tensors.

    llm::kernel::rms_norm, rms_norm_residual     src/kernels/layernorm_kernels.h:6-19
    llm::kernel::apply_rotary_pos_emb            src/kernels/pos_embedding_kernels.h:7-13
    llm::kernel::set_kv_cache                    src/kernels/kv_cache_kernels.h:6-11
    llm::kernel::silu, silu_with_mul             src/kernels/activation_kernels.h:6-14
    llm::paged_kv_varlen_mha                     src/kernels/attention/attn_api.h:12-27
    marlin::awq_repack / gptq_repack / gptq_gemm src/kernels/quantization/marlin.h:17-37
        -> w4a16_prepack_awq / w4a16_prepack_gptq / w4a16_gemm (our own packed layout)

Every call goes through the C ABI of libb200decode.so on the current CUDA stream.
CPU tensors are rejected — there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import NamedTuple, Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import B200Error, check  # noqa: F401

_DT = {torch.bfloat16: _lib.B200_BF16, torch.float16: _lib.B200_FP16, torch.float32: _lib.B200_FP32}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("scalellm_b200 kernels require CUDA tensors (no CPU fallback)")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_i32(*ts: torch.Tensor) -> None:
    for t in ts:
        if t.dtype != torch.int32:
            raise TypeError("index / length tensors must be int32 (reference: torch::kInt)")
        if not t.is_contiguous():
            raise ValueError("index / length tensors must be contiguous")


# ---------------------------------------------------------------------------
# workspace cache (per device).  Allocate BEFORE CUDA-graph capture by calling the
# op once eagerly, exactly like the reference warms its kernels before capture.
# ---------------------------------------------------------------------------
_WS: Dict[Tuple[str, int], torch.Tensor] = {}
_WS_RETIRED: list = []   # outgrown workspaces: a captured CUDA graph may still hold their addresses


def _workspace(kind: str, device: torch.device, nbytes: int, zero: bool = False) -> torch.Tensor:
    """Grow-only: a larger request allocates a new buffer, but the old one is never freed — a
    CUDA graph captured earlier (GraphedStep) has its raw pointer baked in and would otherwise
    replay into memory the caching allocator has handed to someone else."""
    key = (kind, device.index if device.index is not None else torch.cuda.current_device())
    ws = _WS.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _WS_RETIRED.append(ws)
        ws = (torch.zeros if zero else torch.empty)(max(nbytes, 1), dtype=torch.uint8, device=device)
        _WS[key] = ws
    return ws


# ---------------------------------------------------------------------------
# norms
# ---------------------------------------------------------------------------
def rms_norm(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, epsilon: float) -> None:
    _cuda(out, input, weight)
    assert input.is_contiguous() and out.is_contiguous(), "tensors must be contiguous"
    n = input.shape[-1]
    rows = input.numel() // n
    if rows == 0:
        return
    check(_lib.load().b200_rms_norm(_p(out), _p(input), _p(weight), rows, n, epsilon, _dt(input),
                                    _stream()))


def rms_norm_residual(out: torch.Tensor, residual: torch.Tensor, input: torch.Tensor,
                      weight: torch.Tensor, epsilon: float) -> None:
    _cuda(out, residual, input, weight)
    assert input.is_contiguous() and out.is_contiguous() and residual.is_contiguous()
    n = input.shape[-1]
    rows = input.numel() // n
    if rows == 0:
        return
    check(_lib.load().b200_rms_norm_residual(_p(out), _p(residual), _p(input), _p(weight), rows, n,
                                             epsilon, _dt(input), _stream()))


# ---------------------------------------------------------------------------
# rotary embedding / kv cache
# ---------------------------------------------------------------------------
def apply_rotary_pos_emb(querys: torch.Tensor, keys: torch.Tensor, positions: torch.Tensor,
                         cos_sin: torch.Tensor, rotary_dim: int, interleaved: bool) -> None:
    """In place on querys [T,H,D] and keys [T,Hkv,D] (heads dense, token stride free)."""
    _cuda(querys, keys, positions, cos_sin)
    _check_i32(positions)
    assert querys.stride(-1) == 1 and querys.stride(-2) == querys.size(-1)
    assert keys.stride(-1) == 1 and keys.stride(-2) == keys.size(-1)
    assert cos_sin.is_contiguous() and cos_sin.dtype == querys.dtype
    T, H, D = querys.shape[-3], querys.shape[-2], querys.shape[-1]
    check(_lib.load().b200_rope_inplace(_p(querys), _p(keys), _p(positions), _p(cos_sin), T, H,
                                        keys.shape[-2], D, rotary_dim, querys.stride(-3),
                                        keys.stride(-3), int(interleaved), _dt(querys), _stream()))


def set_kv_cache(slot_ids: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                 key_cache: torch.Tensor, value_cache: torch.Tensor) -> None:
    _cuda(slot_ids, keys, values, key_cache, value_cache)
    _check_i32(slot_ids)
    assert keys.stride(-1) == 1 and keys.stride(-2) == keys.size(-1)
    assert values.stride(-1) == 1 and values.stride(-2) == values.size(-1)
    assert key_cache.is_contiguous() and value_cache.is_contiguous()
    T, Hkv, D = keys.shape[-3], keys.shape[-2], keys.shape[-1]
    check(_lib.load().b200_kv_write(_p(slot_ids), _p(keys), _p(values), _p(key_cache),
                                    _p(value_cache), T, Hkv, D, keys.stride(-3), values.stride(-3),
                                    _dt(keys), _stream()))


def get_kv_cache(slot_ids: torch.Tensor, key_cache: torch.Tensor,
                 value_cache: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """KVCache::get_kv_cache (src/memory/kv_cache.cpp:60-98) as a device gather."""
    _cuda(slot_ids, key_cache, value_cache)
    _check_i32(slot_ids)
    T = slot_ids.numel()
    Hkv, D = key_cache.shape[-2], key_cache.shape[-1]
    k = torch.empty((T, Hkv, D), dtype=key_cache.dtype, device=key_cache.device)
    v = torch.empty_like(k)
    check(_lib.load().b200_kv_gather(_p(slot_ids), _p(key_cache), _p(value_cache), _p(k), _p(v), T,
                                     Hkv, D, _dt(key_cache), _stream()))
    return k, v


def rope_and_set_kv_cache(querys: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                          positions: torch.Tensor, cos_sin: torch.Tensor, slot_ids: torch.Tensor,
                          key_cache: torch.Tensor, value_cache: torch.Tensor, rotary_dim: int,
                          interleaved: bool) -> None:
    """Fused apply_rotary_pos_emb + set_kv_cache (bit-identical to the two calls)."""
    _cuda(querys, keys, values, positions, cos_sin, slot_ids, key_cache, value_cache)
    _check_i32(positions, slot_ids)
    assert querys.stride(-1) == 1 and querys.stride(-2) == querys.size(-1)
    assert keys.stride(-1) == 1 and keys.stride(-2) == keys.size(-1)
    assert values.stride(-1) == 1 and values.stride(-2) == values.size(-1)
    assert key_cache.is_contiguous() and value_cache.is_contiguous()
    T, H, D = querys.shape[-3], querys.shape[-2], querys.shape[-1]
    check(_lib.load().b200_rope_kv_write(_p(querys), _p(keys), _p(values), _p(positions),
                                         _p(cos_sin), _p(slot_ids), _p(key_cache), _p(value_cache),
                                         T, H, keys.shape[-2], D, rotary_dim, querys.stride(-3),
                                         keys.stride(-3), values.stride(-3), int(interleaved),
                                         _dt(querys), _stream()))


# ---------------------------------------------------------------------------
# activations
# ---------------------------------------------------------------------------
def silu(input: torch.Tensor) -> torch.Tensor:
    _cuda(input)
    assert input.dim() == 2 and input.stride(1) == 1
    out = torch.empty((input.shape[0], input.shape[1]), dtype=input.dtype, device=input.device)
    check(_lib.load().b200_silu(_p(out), _p(input), input.shape[0], input.shape[1],
                                input.stride(0), _dt(input), _stream()))
    return out


def silu_with_mul(input: torch.Tensor) -> torch.Tensor:
    _cuda(input)
    assert input.dim() == 2 and input.is_contiguous()
    n = input.shape[1] // 2
    out = torch.empty((input.shape[0], n), dtype=input.dtype, device=input.device)
    check(_lib.load().b200_silu_mul(_p(out), _p(input), input.shape[0], n, _dt(input), _stream()))
    return out


# ---------------------------------------------------------------------------
# dense bf16 linear (A8): F::linear -> cuBLASLt of the reference, parallel_linear.cpp:256-263,294-308
# ---------------------------------------------------------------------------
def dense_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Shapes / dtypes the tcgen05 dense kernel takes (rank-invariant: sizes, dtypes and strides of
    freshly allocated activations only)."""
    return (x.is_cuda and _lib.has("b200_dense_gemm")
            and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.dim() >= 2 and x.shape[-1] % 64 == 0 and weight.shape[0] % 8 == 0
            and weight.stride(1) == 1 and weight.stride(0) % 8 == 0)


def dense_gemm(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ W^T (+ bias): A [M, K] bf16 (rows dense in K), W [N, K] bf16 as nn.Linear stores it."""
    _cuda(a, weight, bias)
    assert a.dim() == 2 and a.stride(1) == 1 and weight.dim() == 2 and weight.stride(1) == 1
    M, K = a.shape
    N = weight.shape[0]
    assert weight.shape[1] == K
    if a.stride(0) % 8 or a.data_ptr() % 16:
        a = a.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if M == 0:
        return out
    ws = _workspace("dense", a.device, int(_lib.load().b200_dense_workspace_bytes(M, N, K)))
    check(_lib.load().b200_dense_gemm(_p(out), _p(a), _p(weight), _p(bias), M, N, K, a.stride(0),
                                      weight.stride(0), out.stride(0), _p(ws), ws.numel(), _stream()))
    return out


def dense_gemm_splitk(a: torch.Tensor, weight: torch.Tensor, poison: bool = False) -> "W4Partials":
    """Partials mode of the dense GEMM: fp32 partials [slots, M, N] in the int4 GEMM's stream-K
    format, for the same fused consumers.  M <= 128, N and K multiples of 128."""
    _cuda(a, weight)
    assert a.dim() == 2 and a.dtype == torch.bfloat16 and a.stride(1) == 1
    assert weight.dim() == 2 and weight.dtype == torch.bfloat16 and weight.stride(1) == 1
    M, K = a.shape
    N = weight.shape[0]
    if a.stride(0) % 8 or a.data_ptr() % 16:
        a = a.contiguous()
    slots = int(_lib.load().b200_dense_splitk_splits(M, N, K))
    assert slots > 0, "dense_gemm_splitk: N and K must be multiples of 128"
    partials = torch.empty((slots, M, N), dtype=torch.float32, device=a.device)
    if poison:
        partials.fill_(float("nan"))
    check(_lib.load().b200_dense_gemm_splitk(_p(partials), _p(a), _p(weight), M, N, K, a.stride(0),
                                             weight.stride(0), slots, _stream()))
    return W4Partials(partials, K)


# ---------------------------------------------------------------------------
# sampling tail: logits processors (src/kernels/sampling/sampling_kernels.h:7-29), in place
# ---------------------------------------------------------------------------
def apply_temperature_penalty(logits: torch.Tensor, temperatures: torch.Tensor) -> None:
    _cuda(logits, temperatures)
    assert logits.dim() == 2 and logits.is_contiguous() and temperatures.is_contiguous()
    assert temperatures.dtype == logits.dtype and temperatures.numel() == logits.shape[0]
    check(_lib.load().b200_apply_temperature(_p(logits), _p(temperatures), logits.shape[0], logits.shape[1],
                                             _dt(logits), _stream()))


def apply_repetition_penalty(logits: torch.Tensor, token_ids: torch.Tensor, token_ids_lens: torch.Tensor,
                             penalties: torch.Tensor) -> None:
    _cuda(logits, token_ids, token_ids_lens, penalties)
    assert logits.dim() == 2 and logits.is_contiguous() and token_ids.is_contiguous()
    assert token_ids.dtype == torch.int64 and token_ids_lens.dtype == torch.int32 and penalties.dtype == logits.dtype
    check(_lib.load().b200_apply_repetition_penalty(_p(logits), _p(token_ids), _p(token_ids_lens), _p(penalties),
                                                    logits.shape[0], logits.shape[1], token_ids.shape[1],
                                                    _dt(logits), _stream()))


def apply_frequency_presence_penalty(logits: torch.Tensor, token_ids: torch.Tensor, token_counts: torch.Tensor,
                                     token_ids_lens: torch.Tensor, frequency_penalties: torch.Tensor,
                                     presence_penalties: torch.Tensor) -> None:
    _cuda(logits, token_ids, token_counts, token_ids_lens, frequency_penalties, presence_penalties)
    assert logits.dim() == 2 and logits.is_contiguous() and token_ids.is_contiguous() and token_counts.is_contiguous()
    assert token_ids.dtype == torch.int64 and token_counts.dtype == torch.int32 and token_ids_lens.dtype == torch.int32
    check(_lib.load().b200_apply_frequency_presence_penalty(
        _p(logits), _p(token_ids), _p(token_counts), _p(token_ids_lens), _p(frequency_penalties),
        _p(presence_penalties), logits.shape[0], logits.shape[1], token_ids.shape[1], _dt(logits), _stream()))


def invoke_softmax(logits: torch.Tensor) -> None:
    _cuda(logits)
    assert logits.dim() == 2 and logits.is_contiguous()
    check(_lib.load().b200_softmax(_p(logits), logits.shape[0], logits.shape[1], _dt(logits), _stream()))


def apply_top_k_top_p(logits: torch.Tensor, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor]) -> None:
    """TopKTopPLogitsProcessor::forward (src/sampling/logits_processor.h:243-276) in place, one launch:
    everything outside the top-k / top-p cut of its row becomes -inf.  top_k [batch] int64 (<= 0: off),
    top_p [batch] float32 (>= 1: off); either may be None."""
    _cuda(logits, top_k, top_p)
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float16)
    assert top_k is None or (top_k.dtype == torch.int64 and top_k.is_contiguous() and top_k.numel() == logits.shape[0])
    assert top_p is None or (top_p.dtype == torch.float32 and top_p.is_contiguous() and top_p.numel() == logits.shape[0])
    check(_lib.load().b200_topk_topp_filter(_p(logits), _p(top_k), _p(top_p), logits.shape[0], logits.shape[1],
                                            logits.stride(0), _dt(logits), _stream()))


def _gelu(input: torch.Tensor, act: int, with_mul: bool) -> torch.Tensor:
    _cuda(input)
    assert input.dim() == 2 and input.stride(1) == 1 and (not with_mul or input.is_contiguous())
    n = input.shape[1] // 2 if with_mul else input.shape[1]
    out = torch.empty((input.shape[0], n), dtype=input.dtype, device=input.device)
    check(_lib.load().b200_gelu(_p(out), _p(input), input.shape[0], n, input.stride(0), act,
                                1 if with_mul else 0, _dt(input), _stream()))
    return out


def gelu_new(input: torch.Tensor) -> torch.Tensor:
    """activation_kernels.h:8 (tanh form, tanh.approx)"""
    return _gelu(input, 1, False)


def gelu_fast(input: torch.Tensor) -> torch.Tensor:
    return _gelu(input, 2, False)


def gelu_new_with_mul(input: torch.Tensor) -> torch.Tensor:
    return _gelu(input, 1, True)


def gelu_fast_with_mul(input: torch.Tensor) -> torch.Tensor:
    return _gelu(input, 2, True)


def gemma_rms_norm(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, epsilon: float) -> None:
    """layernorm_kernels.h:11-14: out = (T)(x * rstd * (1 + w))"""
    _cuda(out, input, weight)
    assert input.is_contiguous() and out.is_contiguous()
    n = input.shape[-1]
    check(_lib.load().b200_gemma_rms_norm(_p(out), _p(input), _p(weight), input.numel() // n, n, epsilon,
                                          _dt(input), _stream()))


def layer_norm(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
               bias: Optional[torch.Tensor], epsilon: float) -> None:
    """layernorm_kernels.h:21-25 (bias may be None / undefined)"""
    _cuda(out, input, weight)
    assert input.is_contiguous() and out.is_contiguous()
    n = input.shape[-1]
    check(_lib.load().b200_layer_norm(_p(out), _p(input), _p(weight), None if bias is None else _p(bias),
                                      input.numel() // n, n, epsilon, _dt(input), _stream()))


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act_func(gate) * up on strided views of the fused gate_up output (llama.h:61-64)."""
    _cuda(gate, up)
    assert gate.dim() == 2 and gate.shape == up.shape and gate.stride(1) == 1 and up.stride(1) == 1
    if out is None:
        out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    check(_lib.load().b200_silu_mul_strided(_p(out), _p(gate), _p(up), gate.shape[0], gate.shape[1],
                                            gate.stride(0), up.stride(0), _dt(gate), _stream()))
    return out


# ---------------------------------------------------------------------------
# paged attention
# ---------------------------------------------------------------------------
def paged_attn_workspace_bytes(batch: int, max_q_len: int, max_kv_len: int, n_heads: int,
                               n_kv_heads: int, head_dim: int) -> int:
    return int(_lib.load().b200_paged_attn_workspace_bytes(batch, max_q_len, max_kv_len, n_heads,
                                                           n_kv_heads, head_dim))


def paged_kv_varlen_mha(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                        value_cache: torch.Tensor, q_cu_lens: torch.Tensor,
                        kv_cu_lens: torch.Tensor, block_table: torch.Tensor,
                        block_cu_lens: torch.Tensor, alibi_slopes: Optional[torch.Tensor],
                        block_size: int, max_q_len: int, max_kv_len: int, sm_scale: float,
                        logits_soft_cap: float, sliding_window: int,
                        workspace: Optional[torch.Tensor] = None) -> None:
    _cuda(out, query, key_cache, value_cache, q_cu_lens, kv_cu_lens, block_table, block_cu_lens,
          alibi_slopes)
    _check_i32(q_cu_lens, kv_cu_lens, block_table, block_cu_lens)
    assert query.stride(-1) == 1 and out.stride(-1) == 1
    assert key_cache.stride(-1) == 1 and value_cache.stride(-1) == 1
    assert key_cache.stride() == value_cache.stride() and key_cache.shape == value_cache.shape
    if alibi_slopes is not None:
        assert alibi_slopes.dtype == torch.float32 and alibi_slopes.is_contiguous()
    batch = q_cu_lens.numel() - 1
    H, D = query.shape[-2], query.shape[-1]
    Hkv = key_cache.shape[-2]
    need = paged_attn_workspace_bytes(batch, max_q_len, max_kv_len, H, Hkv, D)
    if workspace is None and need > 0:
        workspace = _workspace("attn", query.device, need)
    check(_lib.load().b200_paged_attn_decode(
        _p(out), _p(query), _p(key_cache), _p(value_cache), _p(q_cu_lens), _p(kv_cu_lens),
        _p(block_table), _p(block_cu_lens), _p(alibi_slopes), batch, H, Hkv, D,
        key_cache.shape[0], query.stride(0), query.stride(1), out.stride(0), out.stride(1),
        key_cache.stride(0), key_cache.stride(1), block_size, max_q_len, max_kv_len, sm_scale,
        logits_soft_cap, sliding_window, _p(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(), _dt(query),
        _stream()))


# ---------------------------------------------------------------------------
# W4A16
# ---------------------------------------------------------------------------
def w4a16_packed_bytes(K: int, N: int, group_size: int) -> int:
    n = int(_lib.load().b200_w4a16_packed_bytes(K, N, group_size))
    if n < 0:
        raise ValueError(f"W4A16 needs K % 128 == 0 and N % 128 == 0, got K={K} N={N}")
    return n


def w4a16_prepack_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                      group_size: int) -> torch.Tensor:
    """AWQ checkpoint tensors -> opaque packed weight (replaces marlin::awq_repack + the
    zero-point / scale permutations of qlinear_awq_marlin_impl.cpp:62-125)."""
    _cuda(qweight, qzeros, scales)
    assert qweight.dtype == torch.int32 and qzeros.dtype == torch.int32
    assert scales.dtype == torch.bfloat16, "W4A16 path computes in bf16"
    assert qweight.is_contiguous() and qzeros.is_contiguous() and scales.is_contiguous()
    K, N = qweight.shape[0], qweight.shape[1] * 8
    packed = torch.empty(w4a16_packed_bytes(K, N, group_size), dtype=torch.uint8,
                         device=qweight.device)
    check(_lib.load().b200_w4a16_prepack_awq(_p(packed), _p(qweight), _p(qzeros), _p(scales), K, N,
                                             group_size, _stream()))
    return packed


def w4a16_prepack_gptq(qweight: torch.Tensor, qzeros: Optional[torch.Tensor], scales: torch.Tensor,
                       group_size: int, zeros_plus_one: bool = True) -> torch.Tensor:
    """GPTQ checkpoint tensors -> packed weight.  qzeros=None means the symmetric zero point 8
    used by the reference's Marlin path (qlinear_gptq_marlin_impl.cpp:18-20)."""
    _cuda(qweight, qzeros, scales)
    assert qweight.dtype == torch.int32 and scales.dtype == torch.bfloat16
    assert qweight.is_contiguous() and scales.is_contiguous()
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    packed = torch.empty(w4a16_packed_bytes(K, N, group_size), dtype=torch.uint8,
                         device=qweight.device)
    check(_lib.load().b200_w4a16_prepack_gptq(_p(packed), _p(qweight), _p(qzeros), _p(scales), K,
                                              N, group_size, int(zeros_plus_one), _stream()))
    return packed


def w4a16_prepack_gptq_actorder(qweight: torch.Tensor, qzeros: Optional[torch.Tensor], scales: torch.Tensor,
                                g_idx: torch.Tensor, group_size: int, zeros_plus_one: bool = True):
    """GPTQ desc_act checkpoint -> (packed weight, perm): rows sorted by quant group
    (perm = argsort(g_idx), qlinear_gptq_marlin_impl.cpp:43-56); the caller gathers the activation
    columns with the same perm (permute_cols) before the GEMM.  Whole K only."""
    _cuda(qweight, qzeros, scales, g_idx)
    assert qweight.dtype == torch.int32 and scales.dtype == torch.bfloat16 and group_size > 0
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    assert g_idx.numel() == K
    perm = torch.argsort(g_idx.to(torch.int64), stable=True).to(torch.int32).contiguous()
    g_sorted = g_idx.to(torch.int32)[perm.long()].contiguous()
    # whole K: every group has exactly group_size rows, so sorted rows fall into aligned blocks
    want = torch.arange(K, device=g_idx.device, dtype=torch.int32) // group_size
    if not torch.equal(g_sorted, want):
        raise ValueError("act-order: g_idx does not cover K with groups of exactly group_size rows "
                         "(a K-sharded act-order weight is not supported)")
    packed = torch.empty(w4a16_packed_bytes(K, N, group_size), dtype=torch.uint8, device=qweight.device)
    check(_lib.load().b200_w4a16_prepack_gptq_actorder(_p(packed), _p(qweight), _p(qzeros), _p(scales),
                                                       _p(perm), _p(g_sorted), K, N, group_size,
                                                       int(zeros_plus_one), _stream()))
    return packed, perm


def permute_cols(x: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    """out[:, j] = x[:, perm[j]] (permute_cols_kernel, marlin/gptq_gemm.cu:66-104)"""
    _cuda(x, perm)
    assert x.dim() == 2 and x.stride(1) == 1 and perm.dtype == torch.int32 and perm.numel() == x.shape[1]
    out = torch.empty((x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    check(_lib.load().b200_permute_cols(_p(out), _p(x), _p(perm), x.shape[0], x.shape[1], x.stride(0),
                                        out.stride(0), _dt(x), _stream()))
    return out


def w4a16_repack_nibbles(qweight: torch.Tensor, method: str, perm: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The operator-level drop-in's repack (marlin::awq_repack / gptq_repack with the reference's
    signature): nibble tiles only, [K/16, N*16/8] int32."""
    _cuda(qweight, perm)
    if method == "awq":
        K, N = qweight.shape[0], qweight.shape[1] * 8
        out = torch.empty((K // 16, N * 2), dtype=torch.int32, device=qweight.device)
        check(_lib.load().b200_w4a16_repack_awq(_p(out), _p(qweight), K, N, _stream()))
    else:
        K, N = qweight.shape[0] * 8, qweight.shape[1]
        out = torch.empty((K // 16, N * 2), dtype=torch.int32, device=qweight.device)
        check(_lib.load().b200_w4a16_repack_gptq(_p(out), _p(qweight), _p(perm), K, N, _stream()))
    return out


def w4a16_assemble_marlin(nibbles: torch.Tensor, scales_marlin: torch.Tensor,
                          zeros_marlin: Optional[torch.Tensor], K: int, N: int, group_size: int) -> torch.Tensor:
    """nibble tiles + Marlin-order scales (+ Marlin-packed zero points; None = symmetric 8) -> tile blobs"""
    _cuda(nibbles, scales_marlin, zeros_marlin)
    packed = torch.empty(w4a16_packed_bytes(K, N, group_size), dtype=torch.uint8, device=nibbles.device)
    check(_lib.load().b200_w4a16_assemble_marlin(_p(packed), _p(nibbles), _p(scales_marlin), _p(zeros_marlin),
                                                 K, N, group_size, _stream()))
    return packed


def w4a16_dequant(packed: torch.Tensor, K: int, N: int, group_size: int) -> torch.Tensor:
    _cuda(packed)
    w = torch.empty((K, N), dtype=torch.bfloat16, device=packed.device)
    check(_lib.load().b200_w4a16_dequant(_p(w), _p(packed), K, N, group_size, _stream()))
    return w


def w4a16_workspace(device: torch.device, M: int, N: int, K: int) -> torch.Tensor:
    need = int(_lib.load().b200_w4a16_workspace_bytes(M, N, K))
    return _workspace("w4a16", device, need, zero=False)


def w4a16_gemm(a: torch.Tensor, packed: torch.Tensor, N: int, group_size: int,
               bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M,N] = A[M,K] @ dequant(packed).  A bf16 with unit inner stride."""
    _cuda(a, packed, bias, out)
    assert a.dim() == 2 and a.dtype == torch.bfloat16 and a.stride(1) == 1
    M, K = a.shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (M, N)
    if workspace is None:
        workspace = w4a16_workspace(a.device, M, N, K)
    check(_lib.load().b200_w4a16_gemm(_p(out), _p(a), _p(packed), _p(bias), M, N, K, a.stride(0),
                                      out.stride(0), group_size, _p(workspace),
                                      workspace.numel(), _stream()))
    return out


def w4a16_splitk_splits(M: int, N: int, K: int) -> int:
    return int(_lib.load().b200_w4a16_splitk_splits(M, N, K))


class W4Partials(NamedTuple):
    """fp32 stream-K partials of a W4A16 GEMM: data [slots, M, N]; K is the GEMM's reduction
    dimension (the consumer recomputes the tile -> contributor-slot partition from (N, K))."""
    data: torch.Tensor
    K: int


def w4a16_gemm_splitk(a: torch.Tensor, packed: torch.Tensor, N: int, group_size: int,
                      poison: bool = False) -> W4Partials:
    """Partials mode: the GEMM writes fp32 partials [slots, M, N] and the consumer
    (rms_norm_residual_splitk, the TP all-reduce, w4a16_reduce_partials) performs the reduction.
    M <= 128."""
    _cuda(a, packed)
    assert a.dim() == 2 and a.dtype == torch.bfloat16 and a.stride(1) == 1
    M, K = a.shape
    slots = w4a16_splitk_splits(M, N, K)
    partials = torch.empty((slots, M, N), dtype=torch.float32, device=a.device)
    if poison:  # tests: slots a tile does not use must never be read
        partials.fill_(float("nan"))
    check(_lib.load().b200_w4a16_gemm_splitk(_p(partials), _p(a), _p(packed), M, N, K, a.stride(0),
                                             group_size, slots, _stream()))
    return W4Partials(partials, K)


def w4a16_reduce_partials(partials: W4Partials, out: Optional[torch.Tensor] = None,
                          bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] (bf16) = bf16(sum over slots of partials) (+ bias)."""
    data = partials.data
    S, M, N = data.shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=data.device)
    _cuda(data, out, bias)
    assert out.dtype == torch.bfloat16 and out.stride(-1) == 1
    check(_lib.load().b200_w4a16_reduce_partials(_p(out), _p(data), S, partials.K, _p(bias), M, N,
                                                 out.stride(0), _stream()))
    return out


def rope_and_set_kv_cache_splitk(partials: W4Partials, n_heads: int, n_kv_heads: int, head_dim: int,
                                 positions: torch.Tensor, cos_sin: torch.Tensor,
                                 slot_ids: torch.Tensor, key_cache: torch.Tensor,
                                 value_cache: torch.Tensor, rotary_dim: int, interleaved: bool,
                                 dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """qkv GEMM partials -> qkv [T, (H + 2 Hkv) D] with q, k rotated, rotated k and v written to
    their cache slots: the GEMM's reduction + RoPE + set_kv_cache in one launch."""
    data = partials.data
    _cuda(data, positions, cos_sin, slot_ids, key_cache, value_cache)
    _check_i32(positions, slot_ids)
    S, T, n = data.shape
    assert n == (n_heads + 2 * n_kv_heads) * head_dim and data.is_contiguous()
    assert key_cache.is_contiguous() and value_cache.is_contiguous()
    qkv = torch.empty((T, n), dtype=dtype, device=data.device)
    check(_lib.load().b200_rope_kv_write_splitk(_p(qkv), _p(data), S, partials.K, _p(positions),
                                                _p(cos_sin), _p(slot_ids), _p(key_cache),
                                                _p(value_cache), T, n_heads, n_kv_heads, head_dim,
                                                rotary_dim, int(interleaved), _dt(qkv), _stream()))
    return qkv


def silu_mul_splitk(partials: W4Partials, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """gate_up GEMM partials [slots, rows, 2*inter] -> silu(gate) * up [rows, inter]."""
    data = partials.data
    _cuda(data)
    S, rows, n2 = data.shape
    assert n2 % 2 == 0 and data.is_contiguous()
    out = torch.empty((rows, n2 // 2), dtype=dtype, device=data.device)
    check(_lib.load().b200_silu_mul_splitk(_p(out), _p(data), S, partials.K, rows, n2 // 2,
                                           _dt(out), _stream()))
    return out


def silu_mul_splitk_available() -> bool:
    return _lib.has("b200_silu_mul_splitk")


def rms_norm_residual_splitk(out: torch.Tensor, residual: torch.Tensor, partials: W4Partials,
                             weight: torch.Tensor, epsilon: float) -> None:
    """residual += T(sum over slots of partials); out = rms_norm(residual) * weight."""
    data = partials.data
    _cuda(out, residual, data, weight)
    assert data.dtype == torch.float32 and data.is_contiguous() and data.dim() == 3
    assert out.is_contiguous() and residual.is_contiguous()
    S, rows, n = data.shape
    if rows == 0:
        return
    check(_lib.load().b200_rms_norm_residual_splitk(_p(out), _p(residual), _p(data), S, partials.K,
                                                    _p(weight), rows, n, epsilon, _dt(out),
                                                    _stream()))


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy sampling: torch.argmax(logits, dim=-1) (first maximal index) in one launch."""
    _cuda(logits)
    assert logits.dim() == 2 and logits.stride(1) == 1
    out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    check(_lib.load().b200_argmax(_p(out), _p(logits), logits.shape[0], logits.shape[1],
                                  logits.stride(0), _dt(logits), _stream()))
    return out


def launch_count() -> int:
    return int(_lib.load().b200_launch_count())


def launch_count_reset() -> None:
    _lib.load().b200_launch_count_reset()


# ---------------------------------------------------------------------------
# residual streams (hyper-connections), offset RMS norm, token shift, gated sublayer results
# (csrc/hyper.cu).  Streams, norm weights, shift vectors, biases and coefficients are fp32.
# ---------------------------------------------------------------------------
def _f32(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError("expected a contiguous float32 tensor")


def embed_streams(table: torch.Tensor, tokens: torch.Tensor, n_streams: int) -> torch.Tensor:
    """X [rows, S, W] fp32 with every stream equal to the token's embedding row."""
    _cuda(table, tokens)
    _check_i32(tokens)
    assert table.dim() == 2 and table.is_contiguous()
    X = torch.empty((tokens.numel(), n_streams, table.shape[1]), dtype=torch.float32, device=table.device)
    check(_lib.load().b200_embed_streams(_p(X), _p(table), _p(tokens), tokens.numel(), table.shape[1],
                                         n_streams, table.shape[0], _dt(table), _stream()))
    return X


def hc_norm(X: torch.Tensor, collapse: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
            offset: float, dtype: torch.dtype, want_fp32: bool = False):
    """Collapse the streams (sum_s collapse[s] X[:, s]) and RMS-normalise with weight (offset + w).
    Returns the rows as `dtype` and, if asked, also in fp32 (for the token shift)."""
    _cuda(X, weight)
    _f32(X, collapse, weight)
    rows, S, W = X.shape
    out = torch.empty((rows, W), dtype=dtype, device=X.device)
    out32 = torch.empty((rows, W), dtype=torch.float32, device=X.device) if want_fp32 else None
    check(_lib.load().b200_hc_norm(_p(out), _p(out32), _p(X), _p(collapse), _p(weight), rows, W, S, eps,
                                   offset, _DT[dtype], _stream()))
    return (out, out32) if want_fp32 else out


def token_shift(n32: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, q_cu: torch.Tensor,
                positions: torch.Tensor, token_seq: torch.Tensor, state_slots: torch.Tensor,
                dtype: torch.dtype) -> torch.Tensor:
    _cuda(n32, mu, state)
    _f32(n32, mu, state)
    _check_i32(q_cu, positions, token_seq, state_slots)
    rows, W = n32.shape
    assert state.dim() == 2 and state.shape[1] == W
    out = torch.empty((rows, W), dtype=dtype, device=n32.device)
    check(_lib.load().b200_token_shift(_p(out), _p(n32), _p(mu), _p(state), _p(q_cu), _p(positions),
                                       _p(token_seq), _p(state_slots), rows, W, _DT[dtype], _stream()))
    return out


def gated_hc_update(X: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor],
                    gate_bias: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                    out_coef: Optional[torch.Tensor]) -> None:
    """In place: X[:, t] <- sum_s mix[s, t] X[:, s] + out_coef[t] * y * sigmoid(gate + gate_bias)."""
    _cuda(X, y, gate)
    _f32(X, gate_bias, mix, out_coef)
    rows, S, W = X.shape
    assert y.shape == (rows, W) and y.stride(1) == 1
    assert gate is None or (gate.shape == (rows, W) and gate.stride(1) == 1 and gate.dtype == y.dtype)
    check(_lib.load().b200_gated_hc_update(_p(X), _p(y), y.stride(0), _p(gate),
                                           gate.stride(0) if gate is not None else 0, _p(gate_bias),
                                           _p(mix), _p(out_coef), rows, W, S, _dt(y), _stream()))


def gated_act(gate_up: torch.Tensor, act: str) -> torch.Tensor:
    """act(gate) * up for a [rows, 2n] matrix [gate | up]; act: "silu" or "gelu_tanh" (tanhf)."""
    _cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.stride(1) == 1 and gate_up.shape[1] % 2 == 0
    n = gate_up.shape[1] // 2
    out = torch.empty((gate_up.shape[0], n), dtype=gate_up.dtype, device=gate_up.device)
    check(_lib.load().b200_gated_act(_p(out), _p(gate_up), gate_up.shape[0], n, gate_up.stride(0),
                                     {"silu": 0, "gelu_tanh": 1}[act], _dt(gate_up), _stream()))
    return out


def heads_to_rows(x: torch.Tensor, gate: Optional[torch.Tensor]) -> torch.Tensor:
    """[H, rows, d] -> [rows, H * d], optionally times sigmoid(gate [rows, H * d])."""
    _cuda(x, gate)
    assert x.dim() == 3 and x.is_contiguous()
    H, rows, d = x.shape
    assert gate is None or (gate.shape == (rows, H * d) and gate.stride(1) == 1 and gate.dtype == x.dtype)
    out = torch.empty((rows, H * d), dtype=x.dtype, device=x.device)
    check(_lib.load().b200_heads_to_rows(_p(out), _p(x), _p(gate), gate.stride(0) if gate is not None else 0,
                                         rows, H, d, _dt(x), _stream()))
    return out


# ---------------------------------------------------------------------------
# latent attention (csrc/latent_attn.cu)
# ---------------------------------------------------------------------------
def latent_prepare(q: torch.Tensor, dkv: torch.Tensor, cache: torch.Tensor, c_norm_weight: torch.Tensor,
                   inv_freq: torch.Tensor, mult: float, positions: torch.Tensor, slots: torch.Tensor,
                   n_heads: int, dim: int, rot_dim: int, rot_dims: int, rank: int, eps: float,
                   half_pairs: bool = False) -> None:
    """In place on q (rotary part of every head) and on the cache rows `slots` (latent + rotary key).
    half_pairs: channel i turns with channel i + rot_dims / 2 instead of its neighbour."""
    _cuda(q, dkv, cache)
    _f32(c_norm_weight, inv_freq)
    _check_i32(positions, slots)
    assert q.dim() == 2 and q.stride(1) == 1 and dkv.dim() == 2 and dkv.stride(1) == 1
    assert cache.dim() == 2 and cache.stride(1) == 1 and cache.shape[1] == rank + rot_dim
    assert q.dtype == dkv.dtype == cache.dtype and inv_freq.numel() == rot_dims // 2
    check(_lib.load().b200_latent_prepare(_p(q), q.stride(0), _p(dkv), dkv.stride(0), _p(cache), cache.stride(0),
                                          _p(c_norm_weight), _p(inv_freq), mult, _p(positions), _p(slots),
                                          q.shape[0], n_heads, dim, rot_dim, rot_dims, rank, eps,
                                          1 if half_pairs else 0, _dt(q), _stream()))


def latent_attn_splits(rows: int, n_heads: int, kv_max: int, dtype: torch.dtype, width: int, rank: int = 0) -> int:
    """How the keys of a row are cut over CTAs.  0: the CUDA-core kernel (fp32 models, rows that are not
    16-byte multiples, B200_LATENT_IMPL=simt).  Otherwise the tensor-core kernel with enough key ranges to
    fill (and not overflow) the two CTAs an SM holds when the step has few rows (decoding), one range otherwise."""
    if dtype != torch.bfloat16 or width % 8 or rank > 512 or os.environ.get("B200_LATENT_IMPL") == "simt":
        return 0
    ctas = rows * ((n_heads + 15) // 16)
    resident = 2 * 148                    # two CTAs of this kernel fit on an SM; stay within one wave of them
    return max(1, min(resident // max(ctas, 1), -(-kv_max // 64), 64))


def latent_attn(q_absorbed: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, q_cu: torch.Tensor,
                kv_cu: torch.Tensor, block_tables: torch.Tensor, cu_block_lens: torch.Tensor,
                token_seq: torch.Tensor, n_heads: int, dim: int, rot_dim: int, rank: int, block_size: int,
                scale: float, kv_max: int = 0, window: int = 0) -> torch.Tensor:
    """q_absorbed [H, rows, rank] (fp32 or q's dtype), q [rows, >= H * (dim + rot_dim)] with the rotary
    parts already rotated; returns the attention-weighted latents [H, rows, rank] in q's dtype.
    kv_max: the longest cached length of the step (a host number; it only steers the key split).
    window > 0: a row sees only the last `window` keys, its own included."""
    _cuda(q_absorbed, q, cache)
    _check_i32(q_cu, kv_cu, block_tables, cu_block_lens, token_seq)
    rows = q.shape[0]
    assert q_absorbed.shape == (n_heads, rows, rank) and q_absorbed.stride(2) == 1
    assert q_absorbed.dtype in (torch.float32, q.dtype) and q.stride(1) == 1 and cache.dtype == q.dtype
    out = torch.empty((n_heads, rows, rank), dtype=q.dtype, device=q.device)
    visible = min(kv_max, window) if window > 0 and kv_max > 0 else kv_max
    splits = latent_attn_splits(rows, n_heads, visible, q.dtype, rank + rot_dim, rank) if cache.stride(0) % 8 == 0 else 0
    ws, ws_bytes = None, 0
    if splits > 1:
        ws_bytes = int(_lib.load().b200_latent_attn_workspace_bytes(rows, n_heads, rank, splits))
        ws = _workspace("latent_attn", q.device, ws_bytes)
    check(_lib.load().b200_latent_attn(_p(out), out.stride(0), out.stride(1), _p(q_absorbed),
                                       q_absorbed.stride(0), q_absorbed.stride(1),
                                       1 if q_absorbed.dtype == torch.float32 else 0, _p(q), q.stride(0),
                                       _p(cache), cache.stride(0), _p(q_cu), _p(kv_cu), _p(block_tables),
                                       _p(cu_block_lens), _p(token_seq), rows, n_heads, dim, rot_dim, rank,
                                       block_size, scale, window, splits, _p(ws), ws_bytes, _dt(q), _stream()))
    return out


# ---------------------------------------------------------------------------
# generalised delta rule (csrc/delta_rule.cu)
# ---------------------------------------------------------------------------
def delta_rule(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_logits: torch.Tensor,
               removal_logits: torch.Tensor, gate_logits: torch.Tensor, decay_bias: torch.Tensor,
               removal_bias: torch.Tensor, norm_weight: torch.Tensor, state: torch.Tensor,
               q_cu: torch.Tensor, positions: torch.Tensor, state_slots: torch.Tensor, n_heads: int,
               head_dim: int, decay_scale: float, key_eps: float, eps: float) -> torch.Tensor:
    """r, k, v, removal and gate logits: column blocks [rows, H * d] of one matrix (same row stride);
    state fp32 [n_slots, H, d, d], updated in place.  Returns [rows, H * d]."""
    _cuda(r, k, v, decay_logits, removal_logits, gate_logits, state)
    _f32(decay_bias, removal_bias, norm_weight, state)
    _check_i32(q_cu, positions, state_slots)
    rows, n = r.shape
    assert n == n_heads * head_dim
    ld = r.stride(0)
    for t in (r, k, v, removal_logits, gate_logits):
        assert t.shape == (rows, n) and t.stride(1) == 1 and t.stride(0) == ld and t.dtype == r.dtype
    assert decay_logits.shape == (rows, n) and decay_logits.stride(1) == 1 and decay_logits.dtype == r.dtype
    assert state.shape[1:] == (n_heads, head_dim, head_dim)
    out = torch.empty((rows, n), dtype=r.dtype, device=r.device)
    check(_lib.load().b200_delta_rule(_p(out), n, _p(r), _p(k), _p(v), _p(decay_logits), _p(removal_logits),
                                      _p(gate_logits), ld, decay_logits.stride(0), _p(decay_bias),
                                      _p(removal_bias), _p(norm_weight), _p(state), _p(q_cu), _p(positions),
                                      _p(state_slots), state_slots.numel(), n_heads, head_dim, decay_scale,
                                      key_eps, eps, _dt(r), _stream()))
    return out


# ---------------------------------------------------------------------------
# mixture of experts (csrc/moe.cu)
# ---------------------------------------------------------------------------
def moe_route(h: torch.Tensor, router_weight: torch.Tensor, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sigmoid router in fp32: (expert ids [rows, top] int32, routing weights [rows, top] fp32)."""
    _cuda(h, router_weight)
    _f32(router_weight)
    rows, W = h.shape
    E = router_weight.shape[0]
    assert h.stride(1) == 1 and router_weight.shape[1] == W
    ids = torch.empty((rows, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((rows, top), dtype=torch.float32, device=h.device)
    check(_lib.load().b200_moe_route(_p(ids), _p(wts), _p(h), h.stride(0), _p(router_weight), rows, W, E, top,
                                     _dt(h), _stream()))
    return ids, wts


def moe_plan(expert_ids: torch.Tensor, n_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(offsets [E + 1], sorted_pair [n], pos_of_pair [n]) of the (token, choice) pairs grouped by expert."""
    _cuda(expert_ids)
    _check_i32(expert_ids)
    n = expert_ids.numel()
    dev = expert_ids.device
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(n, dtype=torch.int32, device=dev)
    pos_of_pair = torch.empty(n, dtype=torch.int32, device=dev)
    check(_lib.load().b200_moe_plan(_p(offsets), _p(sorted_pair), _p(pos_of_pair), _p(expert_ids), n, n_experts,
                                    _stream()))
    return offsets, sorted_pair, pos_of_pair


def grouped_gemm(a: torch.Tensor, weights: torch.Tensor, offsets: torch.Tensor, n_rows: int,
                 sorted_pair: Optional[torch.Tensor] = None, pair_scale: Optional[torch.Tensor] = None,
                 top: int = 1) -> torch.Tensor:
    """C[pos] = A(pos) @ weights[e]^T for the sorted positions pos of every expert e (offsets).
    With sorted_pair, A(pos) = pair_scale[pair] * a[pair // top] (gather form); else A(pos) = a[pos]."""
    _cuda(a, weights)
    _check_i32(offsets)
    E, N, K = weights.shape
    assert weights.is_contiguous() and a.dim() == 2 and a.shape[1] == K and a.stride(1) == 1
    assert a.dtype == weights.dtype and offsets.numel() == E + 1
    if sorted_pair is not None:
        _check_i32(sorted_pair)
        _f32(pair_scale)
    out = torch.empty((n_rows, N), dtype=a.dtype, device=a.device)
    es = a.element_size()
    if n_rows <= _GEMV_ROWS and (K * es) % 16 == 0 and 8 * K * es <= 200 * 1024:
        # decoding: a few rows per expert, the weights are the traffic
        check(_lib.load().b200_grouped_gemv(_p(out), N, _p(a), a.stride(0), _p(sorted_pair), _p(pair_scale), top,
                                            _p(weights), _p(offsets), n_rows, E, N, K, _dt(a), _stream()))
        return out
    if (a.dtype == torch.bfloat16 and K % 8 == 0 and N % 8 == 0 and os.environ.get("B200_MOE_IMPL") != "tile"):
        # prompt-sized: the library's grouped GEMM over the sorted rows (the group ends are offsets[1:])
        if sorted_pair is not None:
            xs = torch.empty((n_rows, K), dtype=a.dtype, device=a.device)
            check(_lib.load().b200_moe_gather(_p(xs), _p(a), a.stride(0), _p(sorted_pair), _p(pair_scale), top,
                                              n_rows, K, _dt(a), _stream()))
        else:
            xs = a if a.is_contiguous() else a.contiguous()
        return torch.nn.functional.grouped_mm(xs, weights.transpose(1, 2), offs=offsets[1:])
    check(_lib.load().b200_grouped_gemm(_p(out), N, _p(a), a.stride(0), _p(sorted_pair), _p(pair_scale), top,
                                        _p(weights), _p(offsets), n_rows, E, N, K, _dt(a), _stream()))
    return out


_GEMV_ROWS = 256   # at most this many (token, choice) rows: the weight-streaming kernel


def moe_combine(y: torch.Tensor, pos_of_pair: torch.Tensor, rows: int, top: int, scale: float = 1.0,
                addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[row] = scale * (sum of the row's `top` expert results in y) (+ addend[row])."""
    _cuda(y, addend)
    _check_i32(pos_of_pair)
    assert y.dim() == 2 and y.stride(1) == 1 and pos_of_pair.numel() == rows * top
    assert addend is None or (addend.shape == (rows, y.shape[1]) and addend.stride(1) == 1 and addend.dtype == y.dtype)
    out = torch.empty((rows, y.shape[1]), dtype=y.dtype, device=y.device)
    check(_lib.load().b200_moe_combine(_p(out), _p(y), y.stride(0), _p(pos_of_pair), rows, y.shape[1], top, scale,
                                       _p(addend), addend.stride(0) if addend is not None else 0, _dt(y), _stream()))
    return out


def moe_table_route(table: torch.Tensor, tokens: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Expert ids [rows, top] int32 read from a table [vocab, top] by token id."""
    _cuda(table, tokens)
    _check_i32(table, tokens)
    assert table.dim() == 2
    ids = torch.empty((tokens.numel(), table.shape[1]), dtype=torch.int32, device=table.device)
    check(_lib.load().b200_moe_table_route(_p(ids), _p(table), _p(tokens), tokens.numel(), table.shape[1],
                                           table.shape[0], n_experts, _stream()))
    return ids


# ---------------------------------------------------------------------------
# post-norm residual with a depth-weighted history, clamped GLU, token-gated projection (csrc/postnorm.cu)
# ---------------------------------------------------------------------------
def bigram_embed(table: torch.Tensor, pair_table: Optional[torch.Tensor], tokens: torch.Tensor,
                 prev_tokens: Optional[torch.Tensor], buckets: int, mul_prev: int, mul_cur: int, scale: float,
                 x_out: Optional[torch.Tensor] = None, want_h: bool = True):
    """x = scale * table[tok] + pair_table[hash(prev, tok)] as fp32 rows (into x_out when given) and, if asked and
    the table is not fp32 itself, the same rows in the table's dtype.  Returns (x, h or None)."""
    _cuda(table, pair_table, tokens, prev_tokens)
    _check_i32(tokens)
    assert table.dim() == 2 and table.is_contiguous()
    assert pair_table is None or (pair_table.is_contiguous() and pair_table.dtype == table.dtype
                                  and pair_table.shape == (buckets + 1, table.shape[1]))
    rows, W = tokens.numel(), table.shape[1]
    x = x_out if x_out is not None else torch.empty((rows, W), dtype=torch.float32, device=table.device)
    _f32(x)
    assert x.shape == (rows, W)
    h = torch.empty((rows, W), dtype=table.dtype, device=table.device) if want_h and table.dtype != torch.float32 else None
    check(_lib.load().b200_bigram_embed(_p(x), _p(h), _p(table), _p(pair_table), _p(tokens), _p(prev_tokens), rows, W,
                                        table.shape[0], buckets, mul_prev, mul_cur, scale, _dt(table), _stream()))
    return x, h


_PLANS: Dict[Tuple[int, int], "C.Array"] = {}


def splitk_plan(N: int, K: int):
    """The dense split-K GEMM's partition of an [N, K] weight as the six integers its fused consumers take."""
    key = (N, K)
    if key not in _PLANS:
        buf = (C.c_int32 * 6)()
        if _lib.load().b200_dense_splitk_plan(N, K, buf) <= 0:
            raise ValueError(f"no split-K partition for a [{N}, {K}] weight")
        _PLANS[key] = buf
    return _PLANS[key]


def splitk_consumers_available() -> bool:
    return _lib.has("b200_dense_gemm_splitk") and _lib.has("b200_dense_splitk_plan")


def postnorm_residual_splitk(x: torch.Tensor, partials: "W4Partials", weight: torch.Tensor, groups: int, mult: float,
                             eps: float, dtype: torch.dtype, hist: Optional[torch.Tensor] = None, n_hist: int = 0,
                             coef: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None):
    """postnorm_residual whose y is the sum of a dense split-K GEMM's partials [slots, rows, W] rounded to `dtype`
    (the GEMM's reduction folded into this launch)."""
    data = partials.data
    _cuda(x, data, weight, hist, coef)
    _f32(x, data, weight, hist, coef)
    S, rows, W = data.shape
    assert x.shape == (rows, W)
    out = x if x_out is None else x_out
    assert hist is None or (hist.dim() == 3 and hist.shape[1:] == (rows, W) and 0 < n_hist <= hist.shape[0]
                            and coef is not None and coef.numel() >= n_hist)
    h = torch.empty((rows, W), dtype=dtype, device=x.device) if dtype != torch.float32 else None
    check(_lib.load().b200_postnorm_residual_splitk(_p(out), _p(h), _p(x), _p(data), S, splitk_plan(W, partials.K),
                                                    _p(weight), rows, W, groups, mult, eps, _p(hist),
                                                    rows * W if hist is not None else 0, n_hist, _p(coef),
                                                    _DT[dtype], _stream()))
    return out, h


def glu_clamped_splitk(partials: "W4Partials", limit: float, slope: float, dtype: torch.dtype) -> torch.Tensor:
    """glu_clamped over the [gate | up] GEMM's split-K partials [slots, rows, 2n]."""
    data = partials.data
    _cuda(data)
    _f32(data)
    S, rows, n2 = data.shape
    out = torch.empty((rows, n2 // 2), dtype=dtype, device=data.device)
    check(_lib.load().b200_glu_clamped_splitk(_p(out), _p(data), S, splitk_plan(n2, partials.K), rows, n2 // 2, limit,
                                              slope, _DT[dtype], _stream()))
    return out


def postnorm_residual(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, groups: int, mult: float, eps: float,
                      hist: Optional[torch.Tensor] = None, n_hist: int = 0, coef: Optional[torch.Tensor] = None,
                      x_out: Optional[torch.Tensor] = None, want_h: bool = True):
    """x_out (default: x, in place) = x + mult * group_rms_norm(y) * weight; with hist [stages, rows, W] the result
    is stored as stage n_hist - 1 and x_out becomes sum_j coef[j] hist[j] over the first n_hist stages.
    Returns (x_out, x_out in y's dtype or None when y is fp32 or it is not asked for)."""
    _cuda(x, y, weight, hist, coef)
    _f32(x, weight, hist, coef)
    rows, W = x.shape
    assert y.shape == (rows, W) and y.stride(1) == 1
    out = x if x_out is None else x_out
    _f32(out)
    assert hist is None or (hist.dim() == 3 and hist.shape[1:] == (rows, W) and 0 < n_hist <= hist.shape[0]
                            and coef is not None and coef.numel() >= n_hist)
    h = torch.empty((rows, W), dtype=y.dtype, device=x.device) if want_h and y.dtype != torch.float32 else None
    check(_lib.load().b200_postnorm_residual(_p(out), _p(h), _p(x), _p(y), y.stride(0), _p(weight), rows, W, groups,
                                             mult, eps, _p(hist), rows * W if hist is not None else 0, n_hist,
                                             _p(coef), _dt(y), _stream()))
    return out, h


def group_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight with one root mean square per group of W / groups channels; x fp32."""
    _cuda(x, weight)
    _f32(x, weight)
    rows, W = x.shape
    out = torch.empty((rows, W), dtype=dtype, device=x.device)
    check(_lib.load().b200_group_rms_norm(_p(out), _p(x), _p(weight), rows, W, groups, eps, _DT[dtype], _stream()))
    return out


def glu_clamped(gate_up: torch.Tensor, limit: float, slope: float) -> torch.Tensor:
    """g sigmoid(slope g) (u + 1) for a [rows, 2n] matrix [gate | up], g = min(gate, limit), u = clamp(up, +-limit)."""
    _cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.stride(1) == 1 and gate_up.shape[1] % 2 == 0
    n = gate_up.shape[1] // 2
    out = torch.empty((gate_up.shape[0], n), dtype=gate_up.dtype, device=gate_up.device)
    check(_lib.load().b200_glu_clamped(_p(out), _p(gate_up), gate_up.shape[0], n, gate_up.stride(0), limit, slope,
                                       _dt(gate_up), _stream()))
    return out


def token_gated_gelu(a: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor) -> torch.Tensor:
    """gelu_tanh(a [rows, n]) * table[tokens, col0 : col0 + n]."""
    _cuda(a, table, tokens)
    _check_i32(tokens)
    assert a.dim() == 2 and a.stride(1) == 1 and table.dim() == 2 and table.stride(1) == 1 and table.dtype == a.dtype
    rows, n = a.shape
    out = torch.empty((rows, n), dtype=a.dtype, device=a.device)
    check(_lib.load().b200_token_gated_gelu(_p(out), _p(a), a.stride(0), _p(table), table.stride(0), col0,
                                            _p(tokens), rows, n, table.shape[0], _dt(a), _stream()))
    return out


# ---------------------------------------------------------------------------
# minimal gated recurrent unit (csrc/mingru.cu)
# ---------------------------------------------------------------------------
def token_side_postnorm(x: torch.Tensor, h: torch.Tensor, gate_w: torch.Tensor, proj_wt: torch.Tensor,
                        table: torch.Tensor, col0: int, tokens: torch.Tensor, weight: torch.Tensor, groups: int,
                        mult: float, eps: float, hist: Optional[torch.Tensor] = None, n_hist: int = 0,
                        coef: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None):
    """postnorm_residual(x, P (gelu_tanh(G h) * table[tokens, col0 : col0 + sd]), ...) in one launch (few rows).
    proj_wt: the projection weight transposed, [sd, W]."""
    _cuda(x, h, gate_w, proj_wt, table, tokens, weight, hist, coef)
    _f32(x, weight, hist, coef)
    _check_i32(tokens)
    rows, W = x.shape
    sd = gate_w.shape[0]
    assert h.shape == (rows, W) and h.is_contiguous() and gate_w.shape == (sd, W) and proj_wt.shape == (sd, W)
    assert gate_w.is_contiguous() and proj_wt.is_contiguous() and table.stride(1) == 1
    assert h.dtype == gate_w.dtype == proj_wt.dtype == table.dtype
    out = x if x_out is None else x_out
    _f32(out)
    assert hist is None or (hist.dim() == 3 and hist.shape[1:] == (rows, W) and 0 < n_hist <= hist.shape[0]
                            and coef is not None and coef.numel() >= n_hist)
    hh = torch.empty((rows, W), dtype=h.dtype, device=x.device) if h.dtype != torch.float32 else None
    check(_lib.load().b200_token_side_postnorm(_p(out), _p(hh), _p(x), _p(h), _p(gate_w), _p(proj_wt), _p(table),
                                               table.stride(0), col0, _p(tokens), table.shape[0], sd, _p(weight),
                                               rows, W, groups, mult, eps, _p(hist),
                                               rows * W if hist is not None else 0, n_hist, _p(coef), _dt(h),
                                               _stream()))
    return out, hh


# portions at least this long are cut into chunks of MINGRU_CHUNK tokens that run side by side
MINGRU_CHUNKED_MIN_ROWS = 128
MINGRU_CHUNK = 64


def mingru_scan(proj: torch.Tensor, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor],
                state: torch.Tensor, q_cu: torch.Tensor, positions: torch.Tensor, state_slots: torch.Tensor,
                n_seq: int, width: int, q_max: int = 0, chunk_len: int = 0) -> torch.Tensor:
    """proj [rows, >= 3 width] = [z | x | g]; returns S_t * silu(g_t) [rows, width]; state fp32 [slots, width].
    q_max (host number: the step's longest portion): long portions run as chunks side by side (chunk_len, default
    MINGRU_CHUNK, forces it)."""
    _cuda(proj, state)
    _f32(z_bias, x_bias, state)
    _check_i32(q_cu, positions, state_slots)
    assert proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= 3 * width and state.shape[1] == width
    out = torch.empty((proj.shape[0], width), dtype=proj.dtype, device=proj.device)
    lib = _lib.load()
    if chunk_len > 0 or q_max >= MINGRU_CHUNKED_MIN_ROWS:
        L = chunk_len or MINGRU_CHUNK
        q_max = q_max or proj.shape[0]
        n = lib.b200_mingru_chunked_workspace_floats(n_seq, width, q_max, L)
        ws = torch.empty(n, dtype=torch.float32, device=proj.device)
        check(lib.b200_mingru_scan_chunked(_p(out), width, _p(proj), proj.stride(0), _p(z_bias), _p(x_bias),
                                           _p(state), _p(q_cu), _p(positions), _p(state_slots), n_seq, width, q_max,
                                           L, _p(ws), n, _dt(proj), _stream()))
        return out
    check(lib.b200_mingru_scan(_p(out), width, _p(proj), proj.stride(0), _p(z_bias), _p(x_bias), _p(state),
                               _p(q_cu), _p(positions), _p(state_slots), n_seq, width, _dt(proj), _stream()))
    return out


# ---------------------------------------------------------------------------
# differential sliding-window attention (csrc/diff_attn.cu)
# ---------------------------------------------------------------------------
def diff_attn_prepare(q_in: torch.Tensor, k_in: Optional[torch.Tensor], v_in: Optional[torch.Tensor],
                      k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], q_norm_w: torch.Tensor,
                      k_norm_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rot_mult: float,
                      rot_dims: int, positions: torch.Tensor, slots: torch.Tensor, H: int, G: int, dim: int,
                      vdim: int, eps: float) -> torch.Tensor:
    """Normalised, rotated queries fp32 [rows, H, 2, dim]; with k_in / v_in (column blocks of the same projection
    matrix as q_in) the normalised, rotated keys and the values go to the cache rows `slots`."""
    _cuda(q_in, k_in, v_in, k_cache, v_cache)
    _f32(q_norm_w, k_norm_w, inv_freq)
    _check_i32(positions, slots)
    rows, ld = q_in.shape[0], q_in.stride(0)
    assert q_in.stride(1) == 1 and q_in.shape[1] == H * 2 * dim
    if k_in is not None:
        assert k_in.stride(0) == ld and v_in.stride(0) == ld and k_in.dtype == v_in.dtype == q_in.dtype
        assert k_cache.dtype == v_cache.dtype == q_in.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[1:] == (G, 2 * dim) and v_cache.shape[1:] == (G, vdim)
    q = torch.empty((rows, H, 2, dim), dtype=torch.float32, device=q_in.device)
    check(_lib.load().b200_diff_attn_prepare(_p(q), _p(q_in), _p(k_in), _p(v_in), ld, _p(k_cache), _p(v_cache),
                                             _p(q_norm_w), _p(k_norm_w), _p(inv_freq), rot_mult, _p(positions),
                                             _p(slots), rows, H, G, dim, vdim, rot_dims, eps, _dt(q_in), _stream()))
    return q


# a step whose longest portion has at least this many tokens runs the tensor-core kernel (bf16, fitting head sizes)
DIFF_ATTN_PREFILL_MIN_ROWS = 4
# single tokens in bf16 with at least this many query heads per key/value head run as tensor-core tiles of heads
DIFF_ATTN_DECODE_TC_MIN_GROUP = 2


def diff_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, gate: Optional[torch.Tensor],
              q_cu: torch.Tensor, kv_cu: torch.Tensor, block_tables: torch.Tensor, cu_block_lens: torch.Tensor,
              token_seq: torch.Tensor, block_size: int, scale: float, window: int, keep_first: int, lam: float,
              out_scale: float, eps: float, n_seq: int = 0, q_max: int = 0, kv_max: int = 0,
              n_splits: int = 0) -> torch.Tensor:
    """[rows, H * vdim] in the cache's dtype: (softmax(s1) V - lam softmax(s2) V), RMS-normalised per head, times
    out_scale and sigmoid(gate [rows, H]).  With n_seq and q_max (the step's sequence count and longest portion,
    host numbers) a step with prompt portions in bf16 runs on the tensor cores where the head sizes allow it;
    single tokens in bf16 with grouped heads run as tensor-core tiles of heads, their keys shared out over several
    CTAs per row when the step has few rows (kv_max: an upper bound of the cached lengths, sizes the split;
    n_splits forces it); fp32 and odd sizes run the CUDA-core kernels."""
    _cuda(q, k_cache, v_cache, gate)
    _f32(q)
    _check_i32(q_cu, kv_cu, block_tables, cu_block_lens, token_seq)
    rows, H, _, dim = q.shape
    G, vdim = v_cache.shape[1], v_cache.shape[2]
    assert gate is None or (gate.shape == (rows, H) and gate.stride(1) == 1 and gate.dtype == k_cache.dtype)
    out = torch.empty((rows, H * vdim), dtype=k_cache.dtype, device=q.device)
    lib = _lib.load()
    impl = os.environ.get("B200_DIFF_ATTN_IMPL")      # "simt": CUDA cores throughout; "simt_decode": for single tokens
    if (n_seq > 0 and q_max >= DIFF_ATTN_PREFILL_MIN_ROWS and impl != "simt"
            and lib.b200_diff_attn_prefill_supported(dim, vdim, _dt(k_cache))):
        check(lib.b200_diff_attn_prefill(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(gate),
                                         gate.stride(0) if gate is not None else 0, _p(q_cu), _p(kv_cu),
                                         _p(block_tables), _p(cu_block_lens), n_seq, q_max, H, G, dim, vdim,
                                         block_size, scale, window, keep_first, lam, out_scale, eps, _dt(k_cache),
                                         _stream()))
        return out
    args = (_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(gate), gate.stride(0) if gate is not None else 0,
            _p(q_cu), _p(kv_cu), _p(block_tables), _p(cu_block_lens), _p(token_seq), rows, H, G, dim, vdim, block_size,
            scale, window, keep_first, lam, out_scale, eps, _dt(k_cache), _stream())
    if (impl not in ("simt", "simt_decode") and H // G >= DIFF_ATTN_DECODE_TC_MIN_GROUP
            and lib.b200_diff_attn_prefill_supported(dim, vdim, _dt(k_cache))):
        if n_splits <= 0:       # only steps with fewer CTAs than SMs are split (measured: a split of 256 CTAs costs more
            # in per-CTA set-up and merging than it gains), to about two CTAs per SM, two 64-key tiles each at least
            visible = min(kv_max, window + keep_first) if window > 0 and kv_max > 0 else kv_max
            tiles = max(1, -(-visible // 64) + (1 if keep_first else 0))
            ctas = rows * G * -(-(H // G) // 16)
            n_splits = max(1, min(296 // ctas, tiles // 2, 64))
        ws = None
        if n_splits > 1:
            ws = torch.empty(rows * H * n_splits * (4 + 2 * vdim), dtype=torch.float32, device=q.device)
        check(lib.b200_diff_attn_decode_tc(*args[:-2], n_splits, _p(ws), ws.numel() if ws is not None else 0,
                                           *args[-2:]))     # the group's heads as the rows of a tensor-core tile
        return out
    check(lib.b200_diff_attn(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(gate),
                             gate.stride(0) if gate is not None else 0, _p(q_cu), _p(kv_cu),
                             _p(block_tables), _p(cu_block_lens), _p(token_seq), rows, H, G, dim, vdim,
                             block_size, scale, window, keep_first, lam, out_scale, eps, _dt(k_cache),
                             _stream()))
    return out


# ---------------------------------------------------------------------------
# norm after the residual sum, logit cap (csrc/postnorm.cu)
# ---------------------------------------------------------------------------
def sumnorm_residual(x: torch.Tensor, y, weight: torch.Tensor, alpha: float, eps: float,
                     dtype: Optional[torch.dtype] = None, x_out: Optional[torch.Tensor] = None):
    """s = alpha x + y ; x_out (default: x, in place) = s / sqrt(mean(s^2) + eps) * weight, weight one number or one
    per channel.  y: the sublayer's result [rows, W], or the split-K partials of the matrix product that makes it
    (their sum is rounded to `dtype` first).  Returns (x_out, x_out as y's type or None when that is fp32)."""
    partials = isinstance(y, W4Partials)
    data = y.data if partials else y
    _cuda(x, data, weight)
    _f32(x, weight)
    rows, W = x.shape
    assert weight.numel() in (1, W)
    out = x if x_out is None else x_out
    _f32(out)
    w_stride = 0 if weight.numel() == 1 and W != 1 else 1
    lib = _lib.load()
    if partials:
        _f32(data)
        assert data.shape[1:] == (rows, W) and dtype is not None
        h = torch.empty((rows, W), dtype=dtype, device=x.device) if dtype != torch.float32 else None
        check(lib.b200_sumnorm_residual_splitk(_p(out), _p(h), _p(x), _p(data), data.shape[0], splitk_plan(W, y.K),
                                               _p(weight), w_stride, rows, W, alpha, eps, _DT[dtype], _stream()))
        return out, h
    assert data.shape == (rows, W) and data.stride(1) == 1
    h = torch.empty((rows, W), dtype=data.dtype, device=x.device) if data.dtype != torch.float32 else None
    check(lib.b200_sumnorm_residual(_p(out), _p(h), _p(x), _p(data), data.stride(0), _p(weight), w_stride, rows, W,
                                    alpha, eps, _dt(data), _stream()))
    return out, h


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """In place: x <- cap * tanh(x / cap)."""
    _cuda(x)
    assert x.is_contiguous()
    check(_lib.load().b200_softcap(_p(x), _p(x), x.numel(), cap, _dt(x), _stream()))
    return x


# ---------------------------------------------------------------------------
# attention with unit queries and keys, a distance bias and a sink (csrc/sink_attn.cu)
# ---------------------------------------------------------------------------
def sink_attn_prepare(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, v_other: Optional[torch.Tensor],
                      lam: float, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                      slots: torch.Tensor, H: int, G: int, dim: int, vdim: int, eps: float, temp_coef: float = 0.0,
                      temp_every: int = 0) -> torch.Tensor:
    """Unit-length queries with their temperature, fp32 [rows, H, dim]; unit-length keys and the values (blended
    with v_other where given: (1 - lam) v + lam v_other) go to the cache rows `slots`.  q_in, k_in, v_in: column
    blocks of one projection matrix."""
    _cuda(q_in, k_in, v_in, v_other, k_cache, v_cache)
    _check_i32(positions, slots)
    rows, ld = q_in.shape[0], q_in.stride(0)
    assert q_in.stride(1) == 1 and q_in.shape[1] == H * dim
    assert k_in.stride(0) == ld and v_in.stride(0) == ld and k_in.dtype == v_in.dtype == q_in.dtype
    assert k_in.stride(1) == 1 and v_in.stride(1) == 1
    assert k_cache.dtype == v_cache.dtype == q_in.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1:] == (G, dim) and v_cache.shape[1:] == (G, vdim)
    assert v_other is None or (v_other.shape == (rows, G * vdim) and v_other.stride(1) == 1 and v_other.dtype == q_in.dtype)
    q = torch.empty((rows, H, dim), dtype=torch.float32, device=q_in.device)
    check(_lib.load().b200_sink_attn_prepare(_p(q), _p(q_in), _p(k_in), _p(v_in), ld, _p(v_other),
                                             v_other.stride(0) if v_other is not None else 0, lam, _p(k_cache),
                                             _p(v_cache), _p(positions), _p(slots), rows, H, G, dim, vdim, eps,
                                             temp_coef, temp_every, _dt(q_in), _stream()))
    return q


# a step whose longest portion has at least this many tokens runs the tensor-core kernel (bf16, fitting head sizes)
SINK_ATTN_PREFILL_MIN_ROWS = 4
# single tokens in bf16 with at least this many query heads per key/value head run as tensor-core tiles of heads
SINK_ATTN_DECODE_TC_MIN_GROUP = 2


def sink_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, r1: Optional[torch.Tensor],
              r2: Optional[torch.Tensor], sink: Optional[torch.Tensor], q_cu: torch.Tensor, kv_cu: torch.Tensor,
              block_tables: torch.Tensor, cu_block_lens: torch.Tensor, token_seq: torch.Tensor, block_size: int,
              scale: float, n_seq: int = 0, q_max: int = 0, kv_max: int = 0, n_splits: int = 0) -> torch.Tensor:
    """[rows, H * vdim] in the cache's dtype: causal softmax attention with the score scale q . k - r1 ln(1 + r2
    (i - j)) and exp(sink) added to the denominator (r1 / r2 / sink fp32 [H] or None).  With n_seq and q_max (the
    step's sequence count and longest portion, host numbers) a step with prompt portions in bf16 runs on the tensor
    cores where the head sizes allow it; single tokens in bf16 with grouped heads run as tensor-core tiles of heads,
    their keys shared out over several CTAs per row when the step has few rows (kv_max: an upper bound of the cached
    lengths, sizes the split; n_splits forces it); fp32 and odd sizes run the CUDA-core kernel."""
    _cuda(q, k_cache, v_cache, r1, r2, sink)
    _f32(q, r1, r2, sink)
    _check_i32(q_cu, kv_cu, block_tables, cu_block_lens, token_seq)
    rows, H, dim = q.shape
    G, vdim = v_cache.shape[1], v_cache.shape[2]
    out = torch.empty((rows, H * vdim), dtype=k_cache.dtype, device=q.device)
    lib = _lib.load()
    impl = os.environ.get("B200_SINK_ATTN_IMPL")      # "simt": CUDA cores throughout; "simt_decode": for single tokens
    if (n_seq > 0 and q_max >= SINK_ATTN_PREFILL_MIN_ROWS and impl != "simt"
            and lib.b200_sink_attn_prefill_supported(dim, vdim, _dt(k_cache))):
        check(lib.b200_sink_attn_prefill(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(r1), _p(r2), _p(sink),
                                         _p(q_cu), _p(kv_cu), _p(block_tables), _p(cu_block_lens), n_seq, q_max, H, G,
                                         dim, vdim, block_size, scale, _dt(k_cache), _stream()))
        return out
    if (impl not in ("simt", "simt_decode") and H // G >= SINK_ATTN_DECODE_TC_MIN_GROUP
            and lib.b200_sink_attn_prefill_supported(dim, vdim, _dt(k_cache))):
        if n_splits <= 0:
            # steps with fewer CTAs than SMs are split to about two CTAs per SM; walks of 32 tiles (2 048 keys) and
            # more are cut in four whatever the step's size (measured: a CTA's walk is bound by its own latency, and
            # four shorter walks per row keep three CTAs resident per SM); never fewer than two 64-key tiles a share
            tiles = max(1, -(-kv_max // 64))
            ctas = rows * G * -(-(H // G) // 16)
            n_splits = max(1, min(max(296 // ctas, 4 if tiles >= 32 else 1), tiles // 2, 64))
        ws = None
        if n_splits > 1:
            ws = torch.empty(rows * H * n_splits * (2 + vdim), dtype=torch.float32, device=q.device)
        check(lib.b200_sink_attn_decode_tc(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(r1), _p(r2), _p(sink),
                                           _p(q_cu), _p(kv_cu), _p(block_tables), _p(cu_block_lens), _p(token_seq),
                                           rows, H, G, dim, vdim, block_size, scale, n_splits, _p(ws),
                                           ws.numel() if ws is not None else 0, _dt(k_cache), _stream()))
        return out
    check(lib.b200_sink_attn(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(r1), _p(r2), _p(sink), _p(q_cu),
                             _p(kv_cu), _p(block_tables), _p(cu_block_lens), _p(token_seq), rows, H, G, dim, vdim,
                             block_size, scale, _dt(k_cache), _stream()))
    return out


# ---------------------------------------------------------------------------
# sigmoid attention inside blocks of positions with a head mix (csrc/sigmoid_attn.cu)
# ---------------------------------------------------------------------------
def sigmoid_attn_prepare(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, q_bias: Optional[torch.Tensor],
                         k_bias: Optional[torch.Tensor], v_bias: Optional[torch.Tensor], k_cache: torch.Tensor,
                         v_cache: torch.Tensor, inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                         slots: torch.Tensor, H: int, G: int, dim: int, vdim: int, rot_dims: int) -> torch.Tensor:
    """Biased, turned queries as fp32 [rows, H, dim]; biased, turned keys and biased values go to the cache rows
    `slots`.  The turn pairs channel t with t + rot_dims / 2 of every head (angle position * inv_freq[t]).
    q_in, k_in, v_in: column blocks of one projection matrix; biases fp32 or None."""
    _cuda(q_in, k_in, v_in, k_cache, v_cache, q_bias, k_bias, v_bias, inv_freq)
    _f32(q_bias, k_bias, v_bias, inv_freq)
    _check_i32(positions, slots)
    rows, ld = q_in.shape[0], q_in.stride(0)
    assert q_in.stride(1) == 1 and q_in.shape[1] == H * dim and k_in.shape[1] == G * dim and v_in.shape[1] == G * vdim
    assert k_in.stride(0) == ld and v_in.stride(0) == ld and k_in.dtype == v_in.dtype == q_in.dtype
    assert k_in.stride(1) == 1 and v_in.stride(1) == 1
    assert k_cache.dtype == v_cache.dtype == q_in.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1:] == (G, dim) and v_cache.shape[1:] == (G, vdim)
    assert rot_dims == 0 or (inv_freq is not None and inv_freq.numel() == rot_dims // 2)
    q = torch.empty((rows, H, dim), dtype=torch.float32, device=q_in.device)
    check(_lib.load().b200_sigmoid_attn_prepare(_p(q), _p(q_in), _p(k_in), _p(v_in), ld, _p(q_bias), _p(k_bias),
                                                _p(v_bias), _p(k_cache), _p(v_cache), _p(inv_freq), _p(positions),
                                                _p(slots), rows, H, G, dim, vdim, rot_dims, _dt(q_in), _stream()))
    return q


# a step whose longest portion has at least this many tokens runs the tensor-core kernel (bf16, fitting sizes)
SIGMOID_ATTN_PREFILL_MIN_ROWS = 4


def sigmoid_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, head_bias: Optional[torch.Tensor],
                 head_mix: Optional[torch.Tensor], q_cu: torch.Tensor, kv_cu: torch.Tensor, block_tables: torch.Tensor,
                 cu_block_lens: torch.Tensor, token_seq: torch.Tensor, block_size: int, scale: float, cap: float,
                 size: int, q_max: int = 1, n_seq: int = 0, kv_max: int = 0, n_splits: int = 0) -> torch.Tensor:
    """[rows, H * vdim] in the cache's dtype: out_h = sum_j a'_hj v_j over the keys j <= i of row i's block of `size`
    positions (size 0: every j <= i), a_hj = sigmoid(cap tanh(scale q_h . k_j / cap) + head_bias[h]) and
    a'_h = sum_g head_mix[h, g] a_g (head_bias fp32 [H], head_mix fp32 [H, H], either None).  q_max: the step's
    longest portion (a host number): CTAs take up to 8 consecutive rows and share their key tiles.  With n_seq (the
    step's sequence count) a step with prompt portions in bf16 runs on the tensor cores where the sizes allow it; fp32,
    single tokens and odd sizes run the CUDA-core kernel.  A step of single tokens with fewer rows than two CTAs per SM
    shares every row's key tiles out over several CTAs (kv_max: an upper bound of the cached lengths, sizes the split;
    n_splits forces it)."""
    _cuda(q, k_cache, v_cache, head_bias, head_mix)
    _f32(q, head_bias, head_mix)
    _check_i32(q_cu, kv_cu, block_tables, cu_block_lens, token_seq)
    rows, H, dim = q.shape
    G, vdim = v_cache.shape[1], v_cache.shape[2]
    assert head_mix is None or head_mix.shape == (H, H)
    out = torch.empty((rows, H * vdim), dtype=k_cache.dtype, device=q.device)
    lib = _lib.load()
    if (n_seq > 0 and q_max >= SIGMOID_ATTN_PREFILL_MIN_ROWS and os.environ.get("B200_SIGMOID_ATTN_IMPL") != "simt"
            and lib.b200_sigmoid_attn_prefill_supported(H, G, dim, vdim, 1 if head_mix is not None else 0,
                                                        _dt(k_cache))):
        check(lib.b200_sigmoid_attn_prefill(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(head_bias),
                                            _p(head_mix), _p(q_cu), _p(kv_cu), _p(block_tables), _p(cu_block_lens),
                                            n_seq, q_max, H, G, dim, vdim, block_size, scale, cap, size,
                                            _dt(k_cache), _stream()))
        return out
    ws = None
    if q_max <= 1:
        if n_splits <= 0:
            visible = min(kv_max, size) if size > 0 else kv_max
            tiles = max(1, -(-visible // 32))
            # about two CTAs per SM (measured: more and shorter walks cost more in their fixed parts than they hide)
            n_splits = max(1, min(296 // max(rows, 1), tiles, 64))
        if n_splits > 1:
            ws = torch.empty(rows * n_splits * H * vdim, dtype=torch.float32, device=q.device)
    else:
        n_splits = 1
    check(lib.b200_sigmoid_attn(_p(out), H * vdim, _p(q), _p(k_cache), _p(v_cache), _p(head_bias),
                                _p(head_mix), _p(q_cu), _p(kv_cu), _p(block_tables), _p(cu_block_lens),
                                _p(token_seq), rows, H, G, dim, vdim, block_size, scale, cap, size,
                                max(1, q_max), n_splits, _p(ws), ws.numel() if ws is not None else 0, _dt(k_cache),
                                _stream()))
    return out


# ---------------------------------------------------------------------------
# gated delta rule with short input filters (csrc/delta_rule.cu)
# ---------------------------------------------------------------------------
def gated_delta_prepare(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, beta_in: torch.Tensor,
                        decay_in: torch.Tensor, q_filter: torch.Tensor, k_filter: torch.Tensor, v_filter: torch.Tensor,
                        a_log: torch.Tensor, dt_bias: torch.Tensor, filter_state: torch.Tensor, q_cu: torch.Tensor,
                        positions: torch.Tensor, token_seq: torch.Tensor, state_slots: torch.Tensor, H: int, G: int,
                        dim: int, vdim: int, unit_eps: float):
    """(q [rows, G, dim], k [rows, G, dim], v [rows, H, vdim], decay [rows, H, dim], beta [rows, H]), all fp32:
    filtered (causal, per channel, `taps` = filter.shape[1] columns, the last one the current token's), silu, q and k
    of unit length per head and q times dim^(-1/2); decay = exp(-exp(a_log[h]) softplus(decay_in + dt_bias)), beta =
    sigmoid(beta_in).  filter_state fp32 [n_slots, taps - 1, 2 G dim + H vdim] gives the inputs before the step and
    takes the step's last ones.  q_in, k_in, v_in, beta_in: column blocks of one matrix."""
    _cuda(q_in, k_in, v_in, beta_in, decay_in, q_filter, k_filter, v_filter, a_log, dt_bias, filter_state)
    _f32(q_filter, k_filter, v_filter, a_log, dt_bias, filter_state)
    _check_i32(q_cu, positions, token_seq, state_slots)
    rows, ld = q_in.shape[0], q_in.stride(0)
    taps = q_filter.shape[1]
    nqk, nv = G * dim, H * vdim
    for t, n in ((q_in, nqk), (k_in, nqk), (v_in, nv), (beta_in, H)):
        assert t.shape == (rows, n) and t.stride(1) == 1 and t.stride(0) == ld and t.dtype == q_in.dtype
    assert decay_in.shape == (rows, H * dim) and decay_in.stride(1) == 1 and decay_in.dtype == q_in.dtype
    assert q_filter.shape == (nqk, taps) and k_filter.shape == (nqk, taps) and v_filter.shape == (nv, taps)
    assert a_log.numel() == H and dt_bias.numel() == H * dim
    assert filter_state.dim() == 3 and filter_state.shape[1:] == (max(taps - 1, 0), 2 * nqk + nv)
    dev = q_in.device
    q = torch.empty((rows, G, dim), dtype=torch.float32, device=dev)
    k = torch.empty((rows, G, dim), dtype=torch.float32, device=dev)
    v = torch.empty((rows, H, vdim), dtype=torch.float32, device=dev)
    decay = torch.empty((rows, H, dim), dtype=torch.float32, device=dev)
    beta = torch.empty((rows, H), dtype=torch.float32, device=dev)
    check(_lib.load().b200_gated_delta_prepare(_p(q), _p(k), _p(v), _p(decay), _p(beta), _p(q_in), _p(k_in), _p(v_in),
                                               _p(beta_in), ld, _p(decay_in), decay_in.stride(0), _p(q_filter),
                                               _p(k_filter), _p(v_filter), _p(a_log), _p(dt_bias), _p(filter_state),
                                               _p(q_cu), _p(positions), _p(token_seq), _p(state_slots), rows,
                                               state_slots.numel(), H, G, dim, vdim, taps, unit_eps, _dt(q_in),
                                               _stream()))
    return q, k, v, decay, beta


# a step whose longest portion has at least this many tokens norms and gates the read-outs in a launch of its own
GATED_DELTA_SPLIT_NORM_MIN_ROWS = 16


def gated_delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor,
                     gate_logits: torch.Tensor, norm_weight: torch.Tensor, state: torch.Tensor, q_cu: torch.Tensor,
                     positions: torch.Tensor, state_slots: torch.Tensor, eps: float, q_max: int = 1) -> torch.Tensor:
    """The recurrence S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per (sequence, head) over
    the step's rows in order, state fp32 [n_slots, H, dim, vdim] updated in place; returns
    o / rms(o) * norm_weight * sigmoid(gate_logits) as [rows, H * vdim] in gate_logits' dtype.  q_max: the step's
    longest portion (a host number): long portions leave the walk with plain read-outs and take norm and gate in a
    token-parallel launch, which spares the walk a barrier and a reduction per token."""
    _cuda(q, k, v, decay, beta, gate_logits, norm_weight, state)
    _f32(q, k, v, decay, beta, norm_weight, state)
    _check_i32(q_cu, positions, state_slots)
    rows, G, dim = q.shape
    H, vdim = v.shape[1], v.shape[2]
    assert k.shape == q.shape and decay.shape == (rows, H, dim) and beta.shape == (rows, H)
    assert gate_logits.shape == (rows, H * vdim) and gate_logits.stride(1) == 1
    assert norm_weight.numel() == vdim and state.shape[1:] == (H, dim, vdim)
    out = torch.empty((rows, H * vdim), dtype=gate_logits.dtype, device=q.device)
    raw = None
    if q_max >= GATED_DELTA_SPLIT_NORM_MIN_ROWS:
        raw = torch.empty((rows, H * vdim), dtype=torch.float32, device=q.device)
    check(_lib.load().b200_gated_delta_scan(_p(out), H * vdim, _p(q), _p(k), _p(v), _p(decay), _p(beta),
                                            _p(gate_logits), gate_logits.stride(0), _p(norm_weight), _p(state),
                                            _p(q_cu), _p(positions), _p(state_slots), state_slots.numel(), H, G, dim,
                                            vdim, eps, _p(raw), rows, _dt(gate_logits), _stream()))
    return out


# ---------------------------------------------------------------------------
# softmax router with group limits and pass-through outputs; branch norms; squared ReLU (csrc/moe.cu, postnorm.cu)
# ---------------------------------------------------------------------------
def moe_route_softmax(h: torch.Tensor, router_weight: torch.Tensor, correction: Optional[torch.Tensor], top: int,
                      n_groups: int = 1, keep_groups: int = 1, weight_eps: float = 0.0,
                      extra_weight: Optional[torch.Tensor] = None):
    """(ids [rows, top] int32, weights [rows, top] fp32, extra [rows] fp32 or None): p = softmax(router_weight h) in
    fp32; the `top` largest p + correction among the outputs of the keep_groups best of n_groups equal runs of
    neighbours (a run's score: its largest p + correction) are chosen; weights are their p over the sum of the chosen
    p (+ weight_eps).  extra = sigmoid(extra_weight . h) when extra_weight (fp32 [W]) is given."""
    _cuda(h, router_weight, correction, extra_weight)
    _f32(router_weight, correction, extra_weight)
    rows, W = h.shape
    E = router_weight.shape[0]
    assert h.stride(1) == 1 and router_weight.shape[1] == W
    assert correction is None or correction.numel() == E
    ids = torch.empty((rows, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((rows, top), dtype=torch.float32, device=h.device)
    extra = torch.empty(rows, dtype=torch.float32, device=h.device) if extra_weight is not None else None
    check(_lib.load().b200_moe_route_softmax(_p(ids), _p(wts), _p(extra), _p(h), h.stride(0), _p(router_weight),
                                             _p(correction), _p(extra_weight), rows, W, E, top, n_groups, keep_groups,
                                             weight_eps, _dt(h), _stream()))
    return ids, wts, extra


def moe_combine_weighted(y: torch.Tensor, pos_of_pair: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                         n_real: int, h: torch.Tensor, addend: Optional[torch.Tensor] = None,
                         addend_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[row] = sum_k weights[row, k] * (ids[row, k] < n_real ? y[pos_of_pair[row, k]] : h[row])
    (+ addend_gate[row] * addend[row])."""
    _cuda(y, h, addend, addend_gate)
    _check_i32(pos_of_pair, ids)
    _f32(weights, addend_gate)
    rows, top = ids.shape
    W = h.shape[1]
    assert y.dim() == 2 and y.stride(1) == 1 and y.shape[1] == W and h.stride(1) == 1 and y.dtype == h.dtype
    assert pos_of_pair.numel() == rows * top and weights.shape == (rows, top) and weights.is_contiguous()
    assert addend is None or (addend.shape == (rows, W) and addend.stride(1) == 1 and addend.dtype == y.dtype)
    out = torch.empty((rows, W), dtype=y.dtype, device=y.device)
    check(_lib.load().b200_moe_combine_weighted(_p(out), _p(y), y.stride(0), _p(pos_of_pair), _p(ids), _p(weights),
                                                n_real, _p(h), h.stride(0), rows, W, top, _p(addend),
                                                addend.stride(0) if addend is not None else 0, _p(addend_gate),
                                                _dt(y), _stream()))
    return out


def branch_norm_residual(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], weight_a: Optional[torch.Tensor],
                         weight_b: Optional[torch.Tensor], weight: torch.Tensor, weight_next: Optional[torch.Tensor],
                         eps: float, x_out: Optional[torch.Tensor] = None, want_h: bool = True):
    """m = (norm(a) weight_a + norm(b) weight_b) / 2 (one branch: norm(a) weight_a; no branch weight: a itself);
    x_out (default: x, in place) = x + norm(m) weight; h = norm(x_out) weight_next, or x_out itself without
    weight_next, in a's dtype.  norm(z) = z / sqrt(mean(z^2) + eps).  Returns (x_out, h or None)."""
    _cuda(x, a, b, weight_a, weight_b, weight, weight_next)
    _f32(x, weight_a, weight_b, weight, weight_next)
    rows, W = x.shape
    assert a.shape == (rows, W) and a.stride(1) == 1
    assert b is None or (b.shape == (rows, W) and b.stride(1) == 1 and b.dtype == a.dtype)
    out = x if x_out is None else x_out
    _f32(out)
    h = torch.empty((rows, W), dtype=a.dtype, device=x.device) if want_h else None
    check(_lib.load().b200_branch_norm_residual(_p(out), _p(h), _p(x), _p(a), a.stride(0), _p(b),
                                                b.stride(0) if b is not None else 0, _p(weight_a), _p(weight_b),
                                                _p(weight), _p(weight_next), rows, W, eps, _dt(a), _stream()))
    return out, h


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2 of a [rows, n] matrix (rows may be strided)."""
    _cuda(x)
    assert x.dim() == 2 and x.stride(1) == 1
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    check(_lib.load().b200_relu_squared(_p(out), _p(x), x.shape[0], x.shape[1], x.stride(0), _dt(x), _stream()))
    return out
