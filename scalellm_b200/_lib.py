"""ctypes binding of libb200decode.so (the C ABI in include/b200_decode.h).

The library must have been built in-tree (``python -c "import __graft_entry__ as g; g.build()"``
or ``make -C scalellm_b200/csrc``).  There is NO fallback: if the shared object
is missing, importing the kernels raises immediately.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200decode.so")

B200_BF16, B200_FP16, B200_FP32 = 0, 1, 2
AR_HANDLE_BYTES = 128


class B200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libb200decode error {code}: {msg}")
        self.code = code


_i64, _i32, _f32, _vp, _int = C.c_int64, C.c_int32, C.c_float, C.c_void_p, C.c_int

# name -> (restype, argtypes).  Kept in lock-step with include/b200_decode.h;
# tests/test_abi.py checks that every B200_API symbol in the header is listed here
# and exported by the shared object.
SIGNATURES = {
    "b200_abi_version": (_int, []),
    "b200_last_error": (C.c_char_p, []),
    "b200_launch_count": (_i64, []),
    "b200_launch_count_reset": (None, []),
    "b200_rms_norm": (_int, [_vp, _vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "b200_rms_norm_residual": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "b200_rope_inplace": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                 _int, _int, _vp]),
    "b200_kv_write": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_rope_kv_write": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                  _i64, _i64, _i64, _i64, _int, _int, _vp]),
    "b200_kv_gather": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_silu": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_silu_mul": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "b200_silu_mul_strided": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_paged_attn_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _i64, _i64]),
    "b200_paged_attn_decode": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,  # ptrs
                                      _i64, _i64, _i64, _i64, _i64,                # batch..n_slots
                                      _i64, _i64, _i64, _i64, _i64, _i64,          # strides
                                      _int, _int, _int, _f32, _f32, _int,          # bs..window
                                      _vp, _i64, _int, _vp]),
    "b200_w4a16_packed_bytes": (_i64, [_i64, _i64, _int]),
    "b200_w4a16_prepack_awq": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "b200_w4a16_prepack_gptq": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "b200_w4a16_dequant": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "b200_w4a16_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b200_w4a16_gemm": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _i64,
                               _vp]),
    "b200_w4a16_splitk_splits": (_int, [_i64, _i64, _i64]),
    "b200_w4a16_gemm_splitk": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _vp]),
    "b200_w4a16_reduce_partials": (_int, [_vp, _vp, _int, _i64, _vp, _i64, _i64, _i64, _vp]),
    "b200_debug_attn_plan": (_int, [_i64, _int, _int, _int, _int, _int, _int, _vp]),
    "b200_debug_w4a16_plan": (_int, [_i64, _i64, _int, _int, _vp, _vp, _vp]),
    "b200_gemma_rms_norm": (_int, [_vp, _vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "b200_layer_norm": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "b200_gelu": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp]),
    "b200_apply_temperature": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "b200_apply_repetition_penalty": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_apply_frequency_presence_penalty": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_softmax": (_int, [_vp, _i64, _i64, _int, _vp]),
    "b200_topk_topp_filter": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_argmax": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_rope_kv_write_splitk": (_int, [_vp, _vp, _int, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                         _i64, _i64, _int, _int, _vp]),
    "b200_silu_mul_splitk": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _int, _vp]),
    "b200_rms_norm_residual_splitk": (_int, [_vp, _vp, _vp, _int, _i64, _vp, _i64, _i64, _f32, _int, _vp]),
    "b200_debug_set_trace": (None, [_vp]),
    "b200_w4a16_prepack_gptq_actorder": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "b200_w4a16_repack_awq": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "b200_w4a16_repack_gptq": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b200_w4a16_assemble_marlin": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "b200_permute_cols": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_dense_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b200_dense_gemm": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200_dense_splitk_splits": (_int, [_i64, _i64, _i64]),
    "b200_dense_gemm_splitk": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_ar_create": (_int, [C.POINTER(_vp), _int, _int, _i64, _vp]),
    "b200_ar_open_peers": (_int, [_vp, _vp]),
    "b200_ar_create_all": (_int, [C.POINTER(_vp), C.POINTER(C.c_int), _int, _i64]),
    "b200_ar_allreduce": (_int, [_vp, _vp, _i64, _int, _vp]),
    "b200_ar_allgather": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b200_ar_allreduce_splitk": (_int, [_vp, _vp, _vp, _int, _i64, _i64, _i64, _int, _vp]),
    "b200_ar_allreduce_splitk_norm": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _vp, _i64, _i64, _f32, _int, _vp]),
    "b200_ar_argmax": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_ar_destroy": (_int, [_vp]),
    # residual streams, latent attention, delta rule, mixture of experts (hyper.cu, latent_attn.cu,
    # delta_rule.cu, moe.cu)
    "b200_embed_streams": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_hc_norm": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _f32, _int, _vp]),
    "b200_token_shift": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "b200_gated_hc_update": (_int, [_vp, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_gated_act": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "b200_heads_to_rows": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_latent_prepare": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _f32, _vp, _vp, _i64, _i64,
                                   _i64, _i64, _i64, _i64, _f32, _int, _int, _vp]),
    "b200_latent_attn": (_int, [_vp, _i64, _i64, _vp, _i64, _i64, _int, _vp, _i64, _vp, _i64, _vp, _vp, _vp,
                                _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _i64, _int, _vp, _i64, _int, _vp]),
    "b200_latent_attn_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "b200_delta_rule": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp,
                               _vp, _vp, _i64, _i64, _i64, _f32, _f32, _f32, _int, _vp]),
    "b200_moe_route": (_int, [_vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_moe_plan": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "b200_grouped_gemm": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64,
                                 _int, _vp]),
    "b200_grouped_gemv": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64,
                                 _int, _vp]),
    "b200_moe_gather": (_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_moe_combine": (_int, [_vp, _vp, _i64, _vp, _i64, _i64, _i64, _f32, _vp, _i64, _int, _vp]),
    "b200_moe_table_route": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    # post-norm residual with depth-weighted history, minimal gated recurrence, differential attention
    # (postnorm.cu, mingru.cu, diff_attn.cu)
    "b200_bigram_embed": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _int, _vp]),
    "b200_postnorm_residual": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _f32, _f32, _vp, _i64, _i64,
                                      _vp, _int, _vp]),
    "b200_dense_splitk_plan": (_int, [_i64, _i64, _vp]),
    "b200_postnorm_residual_splitk": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _f32, _vp, _i64,
                                             _i64, _vp, _int, _vp]),
    "b200_glu_clamped_splitk": (_int, [_vp, _vp, _i64, _vp, _i64, _i64, _f32, _f32, _int, _vp]),
    "b200_group_rms_norm": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp]),
    "b200_glu_clamped": (_int, [_vp, _vp, _i64, _i64, _i64, _f32, _f32, _int, _vp]),
    "b200_token_gated_gelu": (_int, [_vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_token_side_postnorm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64,
                                        _i64, _f32, _f32, _vp, _i64, _i64, _vp, _int, _vp]),
    "b200_mingru_scan": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "b200_mingru_chunked_workspace_floats": (_i64, [_i64, _i64, _i64, _i64]),
    "b200_mingru_scan_chunked": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp,
                                        _i64, _int, _vp]),
    "b200_diff_attn_prepare": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _i64, _i64,
                                      _i64, _i64, _i64, _i64, _f32, _int, _vp]),
    "b200_diff_attn": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                              _i64, _i64, _f32, _i64, _i64, _f32, _f32, _f32, _int, _vp]),
    "b200_diff_attn_prefill_supported": (_int, [_i64, _i64, _int]),
    "b200_diff_attn_decode_tc": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                        _i64, _i64, _i64, _f32, _i64, _i64, _f32, _f32, _f32, _i64, _vp, _i64, _int,
                                        _vp]),
    "b200_diff_attn_prefill": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                      _i64, _i64, _i64, _f32, _i64, _i64, _f32, _f32, _f32, _int, _vp]),
    # norm after the residual sum, logit cap, attention with a distance bias and a sink (postnorm.cu, sink_attn.cu)
    "b200_sumnorm_residual": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _f32, _f32, _int, _vp]),
    "b200_sumnorm_residual_splitk": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _f32, _int,
                                            _vp]),
    "b200_softcap": (_int, [_vp, _vp, _i64, _f32, _int, _vp]),
    "b200_sink_attn_prepare": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _f32, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                      _i64, _i64, _f32, _f32, _i64, _int, _vp]),
    "b200_sink_attn": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                              _i64, _i64, _f32, _int, _vp]),
    "b200_sink_attn_prefill_supported": (_int, [_i64, _i64, _int]),
    "b200_sink_attn_decode_tc": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                        _i64, _i64, _i64, _i64, _f32, _i64, _vp, _i64, _int, _vp]),
    "b200_sink_attn_prefill": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                      _i64, _i64, _i64, _i64, _f32, _int, _vp]),
    # sigmoid attention in blocks of positions with a head mix, gated delta rule with input filters, softmax router
    # with group limits, branch norms (sigmoid_attn.cu, delta_rule.cu, moe.cu, postnorm.cu)
    "b200_sigmoid_attn_prepare": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                         _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_sigmoid_attn": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                 _i64, _i64, _f32, _f32, _i64, _i64, _i64, _vp, _i64, _int, _vp]),
    "b200_sigmoid_attn_prefill_supported": (_int, [_i64, _i64, _i64, _i64, _int, _int]),
    "b200_sigmoid_attn_prefill": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                         _i64, _i64, _i64, _f32, _f32, _i64, _int, _vp]),
    "b200_gated_delta_prepare": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _vp,
                                        _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                        _f32, _int, _vp]),
    "b200_gated_delta_scan": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64,
                                     _i64, _i64, _i64, _i64, _f32, _vp, _i64, _int, _vp]),
    "b200_moe_route_softmax": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                      _f32, _int, _vp]),
    "b200_moe_combine_weighted": (_int, [_vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _i64,
                                         _vp, _int, _vp]),
    "b200_branch_norm_residual": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _f32,
                                         _int, _vp]),
    "b200_relu_squared": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
}

# Which source files a partial library needs for a group of entry points.  The whole library
# (libb200decode.so, every source) serves everything; where it has not been built, `ensure()` compiles
# just the sources a model asks for into a library of its own.
ALL_SOURCES = ("runtime.cu", "elementwise.cu", "sampling.cu", "paged_attn.cu", "prefill_attn.cu", "w4a16.cu",
               "dense.cu", "allreduce.cu", "hyper.cu", "latent_attn.cu", "delta_rule.cu", "moe.cu", "postnorm.cu", "mingru.cu",
               "diff_attn.cu", "sink_attn.cu", "sigmoid_attn.cu")

_lib: Optional[C.CDLL] = None
_lib_sources: frozenset = frozenset()


def _bind(lib: C.CDLL, partial: bool) -> C.CDLL:
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if partial:     # a partial library exports the entry points of its sources only
                continue
            raise
        fn.restype = res
        fn.argtypes = args
    return lib


def has(name: str) -> bool:
    """Whether the loaded library exports an entry point (a partial library may not)."""
    try:
        getattr(load(), name)
        return True
    except AttributeError:
        return False


def load() -> C.CDLL:
    """Load (once) and return the shared library; raises if it was not built."""
    global _lib, _lib_sources
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: the CUDA extension is not built. Build it with "
            "`python -c \"import __graft_entry__ as g; g.build()\"` (needs nvcc), or let a model "
            "build the part it needs (scalellm_b200._lib.ensure). There is no CPU / PyTorch fallback.")
    _lib = _bind(C.CDLL(LIB_PATH), False)
    _lib_sources = frozenset(ALL_SOURCES)
    return _lib


def ensure(sources) -> C.CDLL:
    """Make sure a library with (at least) these csrc sources is loaded.  The whole library is used
    when it exists; otherwise the named sources (plus runtime.cu) are compiled with nvcc for sm_100a
    into scalellm_b200/libb200part-<key>.so — nothing else is built — and that library is loaded."""
    global _lib, _lib_sources
    need = frozenset(sources) | {"runtime.cu"}
    unknown = need - set(ALL_SOURCES)
    if unknown:
        raise ValueError(f"unknown csrc sources {sorted(unknown)}")
    if _lib is not None and need <= _lib_sources:
        return _lib
    if os.path.exists(LIB_PATH) and _lib is None:
        return load()
    need = need | _lib_sources
    srcs = [s for s in ALL_SOURCES if s in need]
    import hashlib
    key = hashlib.sha1(" ".join(srcs).encode()).hexdigest()[:10]
    out = os.path.join(_HERE, f"libb200part-{key}.so")
    csrc = os.path.join(_HERE, "csrc")
    deps = [os.path.join(csrc, s) for s in srcs] + [os.path.join(csrc, "common.cuh"),
                                                    os.path.join(_HERE, "..", "include", "b200_decode.h")]
    import fcntl
    import subprocess
    os.makedirs(os.path.join(csrc, "build"), exist_ok=True)
    with open(os.path.join(csrc, "build", ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not (os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps)):
            jobs = str(max(1, min(8, os.cpu_count() or 1)))
            r = subprocess.run(["make", "-C", csrc, "-j", jobs, "SRCS=" + " ".join(srcs),
                                "OUT=../" + os.path.basename(out)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("nvcc build of " + os.path.basename(out) + " failed:\n" + r.stdout[-3000:]
                                   + "\n" + r.stderr[-3000:])
    _lib = _bind(C.CDLL(out), True)
    _lib_sources = frozenset(srcs)
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise B200Error(rc, load().b200_last_error().decode("utf-8", "replace"))
