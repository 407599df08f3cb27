"""Plugin-level face of the B200 decode path: mirrors of the `src/layers` interfaces the
reference's models are written against, backed by scalellm_b200.kernels.

    InputParameters          src/models/parameters.h:11-56
    KVCache                  src/memory/kv_cache.{h,cpp}
    AttentionHandler         src/layers/attention/handler.h:15-65
    B200AttnHandler          drop-in for ScaleAttnHandler (scale_attn_handler.cpp:24-84)
    Attention                src/layers/attention/attention.cpp:22-46
    RMSNorm                  src/layers/normalization.h:114-139
    RotaryEmbedding          src/layers/pos_embedding.cpp:183-215 (kernel variant)
    QuantArgs                src/layers/quantization/quant_args.h:10-33
    Column/RowParallelQLinear  qlinear_awq_marlin_impl.cpp:129-365, qlinear_gptq_marlin_impl.cpp
    Column/RowParallelLinear   src/layers/linear/parallel_linear.cpp:221-308 (dense bf16 -> cuBLASLt)
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from . import kernels
from .model_parallel import (ParallelArgs, gather_from_model_parallel_region,
                             reduce_from_model_parallel_region, scatter_to_model_parallel_region,
                             shard_range)


# ---------------------------------------------------------------------------
# step metadata + KV cache
# ---------------------------------------------------------------------------
@dataclass
class InputParameters:
    num_sequences: int = 0
    q_cu_seq_lens: Optional[torch.Tensor] = None    # int32 [n_seq+1]
    kv_cu_seq_lens: Optional[torch.Tensor] = None   # int32 [n_seq+1]
    kv_max_seq_len: int = 0
    q_max_seq_len: int = 0
    new_cache_slots: Optional[torch.Tensor] = None  # int32 [n_tokens]
    block_tables: Optional[torch.Tensor] = None     # int32 [n_blocks] first-slot ids (batch.cpp:206-209)
    cu_block_lens: Optional[torch.Tensor] = None    # int32 [n_seq+1]
    # models with per-sequence recurrent state (token shift, delta rule): which packed row belongs to
    # which sequence of the step, and the state slot of every sequence
    token_seq: Optional[torch.Tensor] = None        # int32 [n_tokens]
    state_slots: Optional[torch.Tensor] = None      # int32 [n_seq]
    # models whose embedding reads the token before: that token for every packed row, -1 at a sequence's start
    prev_tokens: Optional[torch.Tensor] = None      # int32 [n_tokens]

    def to(self, device) -> "InputParameters":
        mv = lambda t: None if t is None else t.to(device)
        return InputParameters(self.num_sequences, mv(self.q_cu_seq_lens), mv(self.kv_cu_seq_lens),
                               self.kv_max_seq_len, self.q_max_seq_len, mv(self.new_cache_slots),
                               mv(self.block_tables), mv(self.cu_block_lens), mv(self.token_seq),
                               mv(self.state_slots), mv(self.prev_tokens))


class KVCache:
    """Per-layer K and V tensors [n_blocks*block_size, n_kv_heads, head_dim] (kv_cache.cpp:15-27)."""

    def __init__(self, n_blocks: int, block_size: int, n_kv_heads: int, head_dim: int,
                 dtype: torch.dtype, device, value_dim: Optional[int] = None):
        """value_dim: width of a value head where it differs from the key head's (default: the same)."""
        self._block_size = block_size
        self.key_cache = torch.empty((n_blocks * block_size, n_kv_heads, head_dim), dtype=dtype,
                                     device=device)
        self.value_cache = (torch.empty_like(self.key_cache) if value_dim is None else
                            torch.empty((n_blocks * block_size, n_kv_heads, value_dim), dtype=dtype, device=device))

    def block_size(self) -> int:
        return self._block_size

    def empty(self) -> bool:
        return self.key_cache.numel() == 0

    def get_kv_cache(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.key_cache, self.value_cache

    def set_kv_cache(self, slot_ids: torch.Tensor, keys: torch.Tensor, values: torch.Tensor) -> None:
        kernels.set_kv_cache(slot_ids, keys, values, self.key_cache, self.value_cache)

    def get_kv_by_slots(self, slot_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return kernels.get_kv_cache(slot_ids, self.key_cache, self.value_cache)


# ---------------------------------------------------------------------------
# rotary embedding
# ---------------------------------------------------------------------------
def compute_default_inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    """pos_embedding.cpp:75-81"""
    sl = torch.arange(0, rotary_dim, 2, dtype=torch.float32)
    return 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), sl / rotary_dim)


def apply_llama3_rope_scaling(inv_freq: torch.Tensor, factor: float, low_freq_factor: float,
                              high_freq_factor: float, old_context_len: int) -> torch.Tensor:
    """pos_embedding.cpp:83-109 (vectorised, float32)."""
    f = inv_freq.to(torch.float32)
    wavelen = (2 * math.pi) / f
    low_wl = old_context_len / low_freq_factor
    high_wl = old_context_len / high_freq_factor
    smooth = (old_context_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    mid = (1 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen < high_wl, f, torch.where(wavelen > low_wl, f / factor, mid))
    return out.to(torch.float32)


def apply_yarn_rope_scaling(inv_freq: torch.Tensor, base: float, rotary_dim: int, factor: float,
                            original_len: float, fast: float, slow: float) -> Tuple[torch.Tensor, float]:
    """YaRN: frequencies whose wavelength fits the original context `slow` times or fewer are divided by
    `factor`, those that fit it `fast` times or more are kept, with a linear ramp over the pair index
    in between.  Returns (inv_freq, multiplier of cos and sin = 0.1 ln(factor) + 1).  Evaluated in
    float64 and rounded once to float32."""
    f = inv_freq.to(torch.float64)

    def pair_index(turns: float) -> float:   # the pair that makes `turns` full turns over original_len
        return rotary_dim * math.log(original_len / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_index(fast)), 0)
    hi = min(math.ceil(pair_index(slow)), rotary_dim - 1)
    i = torch.arange(f.numel(), dtype=torch.float64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    out = f / factor * ramp + f * (1.0 - ramp)
    return out.to(torch.float32), 0.1 * math.log(factor) + 1.0


class RotaryEmbedding:
    """RotaryEmbeddingKernel: cos|sin cache in the model dtype, in-place kernel."""

    def __init__(self, rotary_dim: int, max_position_embeddings: int, inv_freq: torch.Tensor,
                 interleaved: bool, dtype: torch.dtype, device):
        self.rotary_dim, self.interleaved = rotary_dim, interleaved
        t = torch.arange(0, max_position_embeddings, dtype=torch.float32)
        freqs = torch.einsum("i,j->ij", t, inv_freq.to(torch.float32).cpu())
        self.cos_sin_cache = torch.cat([freqs.cos(), freqs.sin()], dim=-1).to(dtype).to(device)

    def forward(self, query: torch.Tensor, key: torch.Tensor,
                positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        kernels.apply_rotary_pos_emb(query, key, positions, self.cos_sin_cache, self.rotary_dim,
                                     self.interleaved)
        return query, key

    __call__ = forward


# ---------------------------------------------------------------------------
# attention handler plugin
# ---------------------------------------------------------------------------
class AttentionHandler:
    """handler.h:15-65"""

    def get_estimate_workspace_size(self) -> int:
        return -1

    def set_workspace(self, workspace: torch.Tensor) -> None:
        pass

    def apply_pos_emb(self, query, key, positions):
        raise NotImplementedError

    def batch_decode(self, query, kv_cache: KVCache, input_params: InputParameters,
                     sliding_window: int, output: torch.Tensor) -> None:
        raise NotImplementedError

    def append_kv_cache(self, kv_cache: KVCache, key, value, input_params: InputParameters) -> None:
        raise NotImplementedError


class B200AttnHandler(AttentionHandler):
    """The `--attention_handler=b200` plugin.  Same three calls as ScaleAttnHandler; when the
    caller uses `Attention.forward` the rope + cache write are fused into one launch."""

    def __init__(self, sm_scale: float, logits_soft_cap: float = 0.0,
                 alibi_slopes: Optional[torch.Tensor] = None,
                 pos_emb: Optional[RotaryEmbedding] = None):
        self.sm_scale, self.logits_soft_cap = sm_scale, logits_soft_cap
        self.alibi_slopes, self.pos_emb = alibi_slopes, pos_emb
        self._workspace: Optional[torch.Tensor] = None

    @classmethod
    def create_handler_with_rope(cls, head_dim: int, rotary_dim: int, max_position: int,
                                 inv_freq: torch.Tensor, interleaved: bool, dtype, device,
                                 logits_soft_cap: float = 0.0) -> "B200AttnHandler":
        rope = RotaryEmbedding(rotary_dim, max_position, inv_freq, interleaved, dtype, device)
        return cls(1.0 / math.sqrt(head_dim), logits_soft_cap, None, rope)

    def set_workspace(self, workspace: torch.Tensor) -> None:
        self._workspace = workspace

    def apply_pos_emb(self, query, key, positions):
        if positions is not None and self.pos_emb is not None:
            return self.pos_emb(query, key, positions)
        return query, key

    def append_kv_cache(self, kv_cache, key, value, input_params) -> None:
        if not kv_cache.empty():
            kv_cache.set_kv_cache(input_params.new_cache_slots, key, value)

    def apply_pos_emb_and_append(self, query, key, value, positions, kv_cache: KVCache,
                                 input_params: InputParameters) -> None:
        if self.pos_emb is None or positions is None or kv_cache.empty():
            self.apply_pos_emb(query, key, positions)
            self.append_kv_cache(kv_cache, key, value, input_params)
            return
        kernels.rope_and_set_kv_cache(query, key, value, positions, self.pos_emb.cos_sin_cache,
                                      input_params.new_cache_slots, kv_cache.key_cache,
                                      kv_cache.value_cache, self.pos_emb.rotary_dim,
                                      self.pos_emb.interleaved)

    def batch_decode(self, query, kv_cache, input_params, sliding_window, output) -> None:
        kc, vc = kv_cache.get_kv_cache()
        kernels.paged_kv_varlen_mha(output, query, kc, vc, input_params.q_cu_seq_lens,
                                    input_params.kv_cu_seq_lens, input_params.block_tables,
                                    input_params.cu_block_lens, self.alibi_slopes,
                                    kv_cache.block_size(), input_params.q_max_seq_len,
                                    input_params.kv_max_seq_len, self.sm_scale,
                                    self.logits_soft_cap, sliding_window,
                                    workspace=self._workspace)


class Attention:
    """attention.cpp:22-46"""

    def __init__(self, n_heads: int, n_kv_heads: int, head_dim: int, handler: AttentionHandler,
                 sliding_window: int = -1, fuse_rope_kv: bool = True):
        assert n_heads % n_kv_heads == 0
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.handler, self.sliding_window, self.fuse = handler, sliding_window, fuse_rope_kv

    def forward(self, query, key, value, positions, kv_cache: KVCache,
                input_params: InputParameters) -> torch.Tensor:
        T = query.size(0)
        q = query.view(T, self.n_heads, self.head_dim)
        k = key.view(T, self.n_kv_heads, self.head_dim)
        v = value.view(T, self.n_kv_heads, self.head_dim)
        if self.fuse and isinstance(self.handler, B200AttnHandler):
            self.handler.apply_pos_emb_and_append(q, k, v, positions, kv_cache, input_params)
        else:
            q, k = self.handler.apply_pos_emb(q, k, positions)
            self.handler.append_kv_cache(kv_cache, k, v, input_params)
        out = torch.empty((T, self.n_heads, self.head_dim), dtype=q.dtype, device=q.device)
        self.handler.batch_decode(q, kv_cache, input_params, self.sliding_window, out)
        return out.view(T, -1)

    def supports_partials(self) -> bool:
        h = self.handler
        return (self.fuse and isinstance(h, B200AttnHandler) and h.pos_emb is not None)

    def forward_partials(self, qkv_partials, positions, kv_cache: KVCache,
                         input_params: InputParameters, dtype=torch.bfloat16) -> torch.Tensor:
        """Same as forward, with q | k | v delivered as the qkv GEMM's stream-K partials: their
        reduction, RoPE and the KV-slot write are one launch."""
        h = self.handler
        qkv = kernels.rope_and_set_kv_cache_splitk(
            qkv_partials, self.n_heads, self.n_kv_heads, self.head_dim, positions,
            h.pos_emb.cos_sin_cache, input_params.new_cache_slots, kv_cache.key_cache,
            kv_cache.value_cache, h.pos_emb.rotary_dim, h.pos_emb.interleaved, dtype)
        T = qkv.size(0)
        q = qkv[:, : self.n_heads * self.head_dim].view(T, self.n_heads, self.head_dim)
        out = torch.empty((T, self.n_heads, self.head_dim), dtype=qkv.dtype, device=qkv.device)
        h.batch_decode(q, kv_cache, input_params, self.sliding_window, out)
        return out.view(T, -1)

    __call__ = forward


# ---------------------------------------------------------------------------
# norm
# ---------------------------------------------------------------------------
class RMSNorm:
    def __init__(self, dim: int, eps: float, dtype: torch.dtype, device):
        self.weight = torch.ones(dim, dtype=dtype, device=device)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        kernels.rms_norm(out, x, self.weight, self.eps)
        return out

    def forward_residual(self, x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """residual += x (in place), returns norm(residual): kernel::rms_norm_residual."""
        out = torch.empty_like(x)
        kernels.rms_norm_residual(out, residual, x, self.weight, self.eps)
        return out

    def forward_residual_partials(self, partials, residual: torch.Tensor, pa=None) -> torch.Tensor:
        """Same, with x delivered as the producing GEMM's stream-K partials (kernels.W4Partials):
        the cross-CTA reduction of the GEMM is fused into this kernel.  With a tensor-parallel
        group (pa.world_size > 1) the partials are this rank's share and the TP all-reduce is
        fused in as well."""
        if pa is not None and pa.world_size > 1:
            return pa.process_group.allreduce_partials_norm(partials, residual, self.weight, self.eps)
        out = torch.empty_like(residual)
        kernels.rms_norm_residual_splitk(out, residual, partials, self.weight, self.eps)
        return out

    __call__ = forward


# ---------------------------------------------------------------------------
# linear layers
# ---------------------------------------------------------------------------
@dataclass
class QuantArgs:
    """quant_args.h:10-33"""
    quant_method: str = ""      # "awq" | "gptq" | ""
    bits: int = 0
    group_size: int = 0
    desc_act: bool = False
    is_sym: bool = False
    zero_point: bool = True


_DENSE_PREFILL_ROWS = 256   # above this many rows: dequant + bf16 GEMM (B200_W4_PREFILL_DENSE=0: streaming kernel)


def _check_quant(qa: QuantArgs, in_features: int, out_features: int) -> None:
    # qlinear_awq_marlin_impl.cpp:28-31,150-151
    if qa.bits != 4:
        raise NotImplementedError("B200 W4A16 path supports 4-bit weights only")
    if qa.group_size not in (-1, 32, 64, 128):
        raise NotImplementedError(f"group_size {qa.group_size} not in (-1, 32, 64, 128)")
    if in_features % 128 or out_features % 128:
        raise ValueError("W4A16 needs in_features % 128 == 0 and out_features % 128 == 0 per shard")


class _QLinearBase:
    def __init__(self, in_features: int, out_features: int, bias: bool, qa: QuantArgs,
                 device):
        _check_quant(qa, in_features, out_features)
        self.K, self.N, self.qa, self.device = in_features, out_features, qa, device
        self.packed: Optional[torch.Tensor] = None
        self.perm: Optional[torch.Tensor] = None     # GPTQ act-order: activation column order
        self.bias: Optional[torch.Tensor] = None
        self._has_bias = bias
        self._ckpt: Dict[str, torch.Tensor] = {}

    # weights arrive in checkpoint format; packing is lazy like repack_weight
    # (qlinear_awq_marlin_impl.cpp:99-125,232-235)
    def _set_shard(self, qweight, qzeros, scales, bias=None, g_idx=None) -> None:
        self._ckpt = dict(qweight=qweight.contiguous().to(self.device),
                          qzeros=None if qzeros is None else qzeros.contiguous().to(self.device),
                          scales=scales.contiguous().to(self.device).to(torch.bfloat16),
                          g_idx=None if g_idx is None else g_idx.contiguous().to(self.device))
        self.packed, self.perm = None, None
        if bias is not None:
            self.bias = bias.to(self.device).to(torch.bfloat16)

    def verify_loaded_weights(self) -> None:
        if not self._ckpt and self.packed is None:
            raise RuntimeError("qweight / qzeros / scales not loaded")

    def _ensure_packed(self) -> None:
        if self.packed is not None:
            return
        self.verify_loaded_weights()
        c = self._ckpt
        g = self.qa.group_size
        if self.qa.quant_method == "awq":
            self.packed = kernels.w4a16_prepack_awq(c["qweight"], c["qzeros"], c["scales"], g)
        else:
            qz = None if self.qa.is_sym else c["qzeros"]
            if self.qa.desc_act and c.get("g_idx") is not None:
                # act-order: rows sorted by group at pack time, activation columns gathered with the
                # same perm at run time (qlinear_gptq_marlin_impl.cpp:43-56, gptq_gemm.cu:66-104)
                self.packed, self.perm = kernels.w4a16_prepack_gptq_actorder(
                    c["qweight"], qz, c["scales"], c["g_idx"], g, zeros_plus_one=True)
            else:
                self.packed = kernels.w4a16_prepack_gptq(c["qweight"], qz, c["scales"], g,
                                                         zeros_plus_one=True)
        # The first GEMM follows on the same stream with the programmatic-launch attribute and its
        # weight producer skips griddepcontrol.wait (weights are constants): make the prepack's
        # writes visible first.  One-time, never inside a graph capture (it allocates).
        torch.cuda.current_stream().synchronize()
        self._ckpt = {}

    def _gemm(self, x: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        self._ensure_packed()
        x2 = x.reshape(-1, x.shape[-1])
        if self.perm is not None:
            x2 = kernels.permute_cols(x2, self.perm)
        if x2.shape[0] > _DENSE_PREFILL_ROWS and os.environ.get("B200_W4_PREFILL_DENSE", "1") != "0":
            # Prefill-sized batches are compute bound: the streaming kernel would re-read the int4
            # weights once per 128 rows.  Dequantise once (same bf16 values as the fused kernel,
            # b200_w4a16_dequant) and let the library bf16 GEMM do the rest (a plain library GEMM, like
            # the reference's dense layers; TTFT path: 51.6 -> 31.9 ms p50 on B200).
            w = kernels.w4a16_dequant(self.packed, self.K, self.N, self.qa.group_size)
            out = torch.matmul(x2, w)
            if bias is not None:
                out = out + bias
            return out.view(*x.shape[:-1], self.N)
        out = kernels.w4a16_gemm(x2, self.packed, self.N, self.qa.group_size, bias=bias)
        return out.view(*x.shape[:-1], self.N)


def _shard_qtensors(sd: Dict[str, torch.Tensor], qa: QuantArgs, dim: int, rank: int, world: int,
                    K: int, N: int):
    """Shard checkpoint tensors.  dim=1: column parallel (split N); dim=0: row parallel (split K).
    AWQ: qweight [K, N/8], qzeros [K/g, N/8], scales [K/g, N];
    GPTQ: qweight [K/8, N], qzeros [K/g, N/8], scales [K/g, N]."""
    qw, qz, sc = sd["qweight"], sd.get("qzeros"), sd["scales"]
    if world == 1:
        return qw, qz, sc
    g = K if qa.group_size <= 0 else qa.group_size
    if dim == 1:
        r_n = shard_range(N, rank, world)
        r_n8 = slice(r_n.start // 8, r_n.stop // 8)
        qw_s = qw[:, r_n8] if qa.quant_method == "awq" else qw[:, r_n]
        return qw_s, None if qz is None else qz[:, r_n8], sc[:, r_n]
    r_k = shard_range(K, rank, world)
    assert (K // world) % g == 0, "row-parallel shard must align to quant groups"  # :287
    r_g = slice(r_k.start // g, r_k.stop // g)
    qw_s = qw[r_k, :] if qa.quant_method == "awq" else qw[r_k.start // 8: r_k.stop // 8, :]
    return qw_s, None if qz is None else qz[r_g, :], sc[r_g, :]


class ColumnParallelQLinear(_QLinearBase):
    """Y = X W (+b), W split along N (qlinear_awq_marlin_impl.cpp:129-257)."""

    def __init__(self, in_features: int, out_features: int, bias: bool, gather_output: bool,
                 qa: QuantArgs, pa: ParallelArgs, device):
        assert out_features % pa.world_size == 0
        super().__init__(in_features, out_features // pa.world_size, bias, qa, device)
        self.full_N, self.gather_output, self.pa = out_features, gather_output, pa

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        qw, qz, sc = _shard_qtensors(sd, self.qa, 1, self.pa.rank, self.pa.world_size, self.K,
                                     self.full_N)
        b = sd.get("bias")
        if b is not None:
            b = b[shard_range(self.full_N, self.pa.rank, self.pa.world_size)]
        self._set_shard(qw, qz, sc, b, sd.get("g_idx") if self.qa.desc_act else None)

    def supports_partials(self, n_rows: int) -> bool:
        """Partials output for a fused consumer (rope / silu*mul): the column shard is rank-local,
        so this also holds under tensor parallelism (no gather, no bias)."""
        return (self.bias is None and 0 < n_rows <= 128 and not self.qa.desc_act
                and not (self.pa.world_size > 1 and self.gather_output))

    def forward_partials(self, x: torch.Tensor) -> "kernels.W4Partials":
        self._ensure_packed()
        x2 = x.reshape(-1, x.shape[-1])
        return kernels.w4a16_gemm_splitk(x2, self.packed, self.N, self.qa.group_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = self._gemm(x, self.bias)
        if self.pa.world_size > 1 and self.gather_output:
            out = gather_from_model_parallel_region(out, self.pa)
        return out

    __call__ = forward


class RowParallelQLinear(_QLinearBase):
    """Y = sum_ranks X_r W_r (+b), W split along K (qlinear_awq_marlin_impl.cpp:260-365)."""

    def __init__(self, in_features: int, out_features: int, bias: bool,
                 input_is_parallelized: bool, qa: QuantArgs, pa: ParallelArgs, device):
        assert in_features % pa.world_size == 0
        super().__init__(in_features // pa.world_size, out_features, bias, qa, device)
        self.full_K, self.input_is_parallelized, self.pa = in_features, input_is_parallelized, pa

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        qw, qz, sc = _shard_qtensors(sd, self.qa, 0, self.pa.rank, self.pa.world_size,
                                     self.full_K, self.N)
        g_idx = sd.get("g_idx") if self.qa.desc_act else None
        if g_idx is not None and self.pa.world_size > 1:
            raise NotImplementedError("act-order (desc_act) on a K-sharded (row-parallel, TP > 1) weight: "
                                      "its groups are split across ranks (is_k_full = false)")
        self._set_shard(qw, qz, sc, sd.get("bias"), g_idx)

    def supports_partials(self, n_rows: int) -> bool:
        """Partials output (the GEMM's cross-CTA reduction fused into the consumer norm; under TP
        the all-reduce is fused into the same kernel) — no bias."""
        if self.bias is not None or not 0 < n_rows <= 128 or self.qa.desc_act:
            return False
        if self.pa.world_size == 1:
            return True
        pg = self.pa.process_group
        return (os.environ.get("B200_FUSE_AR_NORM", "1") != "0" and hasattr(pg, "supports_partials_norm")
                and pg.supports_partials_norm(n_rows, self.N, torch.bfloat16))

    def forward_partials(self, x: torch.Tensor) -> "kernels.W4Partials":
        self._ensure_packed()
        x2 = x.reshape(-1, x.shape[-1])
        return kernels.w4a16_gemm_splitk(x2, self.packed, self.N, self.qa.group_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallelized:
            x = scatter_to_model_parallel_region(x, self.pa)
        if self.pa.world_size == 1:
            return self._gemm(x, self.bias)
        x2 = x.reshape(-1, x.shape[-1])
        pg = self.pa.process_group
        if 0 < x2.shape[0] <= 128 and hasattr(pg, "allreduce_partials") and x2.is_cuda:
            # split-K partials go straight into the NVLink all-reduce (no GEMM fix-up pass)
            self._ensure_packed()
            parts = kernels.w4a16_gemm_splitk(x2, self.packed, self.N, self.qa.group_size)
            out = pg.allreduce_partials(parts, x.dtype).view(*x.shape[:-1], self.N)
        else:
            out = self._gemm(x, None)
            out = reduce_from_model_parallel_region(out, self.pa)
        if self.bias is not None:  # bias after the reduction (:360-363)
            out = out + self.bias
        return out

    __call__ = forward


def _dense_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """F::linear of the reference's dense layers (parallel_linear.cpp:258,299): the tcgen05 stream
    kernel of csrc/dense.cu for bf16 on CUDA (B200_DENSE_IMPL=cublas: the library GEMM, for A/B)."""
    if os.environ.get("B200_DENSE_IMPL") != "cublas" and kernels.dense_supported(x, weight):
        x2 = x.reshape(-1, x.shape[-1])
        return kernels.dense_gemm(x2, weight).view(*x.shape[:-1], weight.shape[0])
    return F.linear(x, weight)


def _dense_partials_ok(x_rows: int, weight: torch.Tensor) -> bool:
    return (os.environ.get("B200_DENSE_IMPL") != "cublas" and weight.is_cuda
            and weight.dtype == torch.bfloat16 and 0 < x_rows <= 128
            and weight.shape[0] % 128 == 0 and weight.shape[1] % 128 == 0)


class ColumnParallelLinear:
    """Dense bf16 column-parallel linear (parallel_linear.cpp:221-263): csrc/dense.cu."""

    def __init__(self, in_features: int, out_features: int, gather_output: bool, pa: ParallelArgs,
                 dtype, device):
        assert out_features % pa.world_size == 0
        self.weight = torch.empty((out_features // pa.world_size, in_features), dtype=dtype,
                                  device=device)
        self.full_N, self.gather_output, self.pa = out_features, gather_output, pa

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        w = sd["weight"][shard_range(self.full_N, self.pa.rank, self.pa.world_size)]
        self.weight.copy_(w)

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's column shard of the output (no gather)."""
        return _dense_linear(x, self.weight)

    def supports_partials(self, n_rows: int) -> bool:
        """Partials for a fused consumer (rope / silu*mul), like ColumnParallelQLinear."""
        return _dense_partials_ok(n_rows, self.weight) and not (self.pa.world_size > 1 and self.gather_output)

    def forward_partials(self, x: torch.Tensor) -> "kernels.W4Partials":
        return kernels.dense_gemm_splitk(x.reshape(-1, x.shape[-1]), self.weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = _dense_linear(x, self.weight)
        if self.pa.world_size > 1 and self.gather_output:
            out = gather_from_model_parallel_region(out, self.pa)
        return out

    __call__ = forward


class RowParallelLinear:
    """Dense bf16 row-parallel linear (parallel_linear.cpp:266-308)."""

    def __init__(self, in_features: int, out_features: int, input_is_parallelized: bool,
                 pa: ParallelArgs, dtype, device):
        assert in_features % pa.world_size == 0
        self.weight = torch.empty((out_features, in_features // pa.world_size), dtype=dtype,
                                  device=device)
        self.full_K, self.input_is_parallelized, self.pa = in_features, input_is_parallelized, pa

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        w = sd["weight"][:, shard_range(self.full_K, self.pa.rank, self.pa.world_size)]
        self.weight.copy_(w)

    def supports_partials(self, n_rows: int) -> bool:
        """Partials for the fused residual + RMSNorm consumer (under TP: fused into the all-reduce),
        like RowParallelQLinear."""
        if not _dense_partials_ok(n_rows, self.weight):
            return False
        if self.pa.world_size == 1:
            return True
        pg = self.pa.process_group
        return (os.environ.get("B200_FUSE_AR_NORM", "1") != "0" and hasattr(pg, "supports_partials_norm")
                and pg.supports_partials_norm(n_rows, self.weight.shape[0], torch.bfloat16))

    def forward_partials(self, x: torch.Tensor) -> "kernels.W4Partials":
        return kernels.dense_gemm_splitk(x.reshape(-1, x.shape[-1]), self.weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallelized:
            x = scatter_to_model_parallel_region(x, self.pa)
        out = _dense_linear(x, self.weight)
        return reduce_from_model_parallel_region(out, self.pa)

    __call__ = forward


# ---------------------------------------------------------------------------
# layers of decoders with several fp32 residual streams, latent attention, delta-rule mixers and
# token-choice experts (kernels: csrc/hyper.cu, latent_attn.cu, delta_rule.cu, moe.cu).  The
# reference has no such layers; each class states its arithmetic.  Small vectors (norm weights,
# biases, stream coefficients, router weights) are kept in fp32 whatever the model dtype is.
# ---------------------------------------------------------------------------
class Linear:
    """Unsharded y = x W^T in the model dtype, W [out, in].  bf16 with at most _DENSE_PREFILL_ROWS
    rows: the tcgen05 stream kernel where the library has it and the shape fits; otherwise the
    library GEMM (fp32 weights: true fp32, TF32 is never enabled here)."""

    def __init__(self, weight: torch.Tensor):
        assert weight.dim() == 2
        self.weight = weight.contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[0] <= _DENSE_PREFILL_ROWS:
            return _dense_linear(x, self.weight)
        return F.linear(x, self.weight)

    def supports_partials(self, n_rows: int) -> bool:
        """Whether the product can hand its split-K partials to a fused consumer (decode-sized bf16 steps with the
        stream kernel in the loaded library) instead of reducing them in a launch of its own."""
        return (_dense_partials_ok(n_rows, self.weight) and self.weight.is_contiguous()
                and kernels.splitk_consumers_available())

    def forward_partials(self, x: torch.Tensor) -> "kernels.W4Partials":
        return kernels.dense_gemm_splitk(x, self.weight)

    def forward_fusable(self, x: torch.Tensor):
        """The product, as split-K partials where a fused consumer can take them, else as a tensor."""
        return self.forward_partials(x) if self.supports_partials(x.shape[0]) else self.forward(x)

    __call__ = forward


class LatentKVCache:
    """One row [latent (rank) | rotary key (rot_dim)] per cached token: [n_blocks * block_size, rank + rot_dim]."""

    def __init__(self, n_blocks: int, block_size: int, rank: int, rot_dim: int, dtype: torch.dtype, device):
        self._block_size = block_size
        self.rows = torch.zeros((n_blocks * block_size, rank + rot_dim), dtype=dtype, device=device)

    def block_size(self) -> int:
        return self._block_size


class HyperConnection:
    """Reads a sublayer's input from S residual streams and writes its result back:
        read   u = sum_s a[s] x_s ;  n = u / rms(u) * (offset + w)
        write  x_t <- sum_s M[s, t] x_s + b[t] * y * sigmoid(G n + c)        (G absent: no gate)
    S = 1 with a = b = M = 1 is the ordinary pre-norm residual.  X is fp32 [rows, S, W]."""

    def __init__(self, norm_weight: torch.Tensor, eps: float, norm_offset: float,
                 collapse: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                 out_coef: Optional[torch.Tensor], gate: Optional[Linear], gate_bias: Optional[torch.Tensor],
                 dtype: torch.dtype):
        f = lambda t: None if t is None else t.to(torch.float32).contiguous()
        self.norm_weight, self.eps, self.norm_offset = f(norm_weight), eps, norm_offset
        self.collapse, self.mix, self.out_coef = f(collapse), f(mix), f(out_coef)
        self.gate, self.gate_bias, self.dtype = gate, f(gate_bias), dtype

    def read(self, X: torch.Tensor, want_fp32: bool = False):
        return kernels.hc_norm(X, self.collapse, self.norm_weight, self.eps, self.norm_offset, self.dtype,
                               want_fp32)

    def write(self, X: torch.Tensor, y: torch.Tensor, n: torch.Tensor) -> None:
        g = self.gate(n) if self.gate is not None else None
        kernels.gated_hc_update(X, y, g, self.gate_bias, self.mix, self.out_coef)


class TokenShift:
    """h_t = n_t + (n_{t-1} - n_t) * mu, with the last unshifted row of every sequence kept in a state slot."""

    def __init__(self, mu: torch.Tensor, n_slots: int, dtype: torch.dtype, device):
        self.mu = mu.to(torch.float32).contiguous()
        self.state = torch.zeros((n_slots, mu.numel()), dtype=torch.float32, device=device)
        self.dtype = dtype

    def forward(self, n32: torch.Tensor, positions: torch.Tensor, params: InputParameters) -> torch.Tensor:
        return kernels.token_shift(n32, self.mu, self.state, params.q_cu_seq_lens, positions, params.token_seq,
                                   params.state_slots, self.dtype)

    __call__ = forward


class LatentAttention:
    """Attention with keys and values compressed into one latent per token:
        q = Wq h (per head [dim | rot_dim]) ; [c_raw | kr_raw] = Wdkv h
        c = rmsnorm(c_raw) * wc ; kr = rope(kr_raw), one rotary key part for all heads ; rope(q rotary part)
        k_h = Uk_h c ; v_h = Uv_h c ; s = (q_h[:dim] . k_h + q_h[dim:] . kr) * scale ; causal softmax
        out = Wo (concat_h(sum_j p_j v_hj) (* sigmoid(Wg h) when there is an output gate))
    Only [c | kr] is cached (LatentKVCache).  The key map is folded into the query and the value map is
    applied after the weighted sum of latents, so the attention kernel runs in the latent space.
    window > 0: position i sees only the keys j with i - j < window.  half_pairs: the rotary turn pairs channel t
    with channel t + rot_dims / 2 instead of its neighbour."""

    def __init__(self, w: Dict[str, torch.Tensor], n_heads: int, dim: int, rot_dim: int, vdim: int, rank: int,
                 scale: float, inv_freq: torch.Tensor, rot_mult: float, rot_dims: int, eps: float,
                 dtype: torch.dtype, device, window: int = 0, half_pairs: bool = False, fusable_out: bool = False):
        """fusable_out: hand on the output projection's split-K partials where a fused consumer can take them."""
        self.H, self.dim, self.rd, self.vd, self.rank = n_heads, dim, rot_dim, vdim, rank
        self.window, self.half_pairs, self.fusable_out = window, half_pairs, fusable_out
        self.scale, self.rot_mult, self.rot_dims, self.eps, self.dtype = scale, rot_mult, rot_dims, eps, dtype
        self.inv_freq = inv_freq.to(torch.float32).to(device).contiguous()
        qw = n_heads * (dim + rot_dim)
        parts = [w["q"], w["dkv"]] + ([w["g"]] if "g" in w else [])
        self.has_gate = "g" in w
        self.in_proj = Linear(torch.cat(parts, dim=0))          # one GEMM for everything that reads h
        self.q_end, self.dkv_end = qw, qw + rank + rot_dim
        self.c_norm = w["dkv.norm"].to(torch.float32).contiguous()
        self.uk = w["uk"].reshape(n_heads, dim, rank).contiguous()               # [H, dim, rank]
        self.uv_t = w["uv"].reshape(n_heads, vdim, rank).transpose(1, 2).contiguous()   # [H, rank, vdim]
        self.o_proj = Linear(w["o"])

    def forward(self, h: torch.Tensor, positions: torch.Tensor, cache: LatentKVCache,
                params: InputParameters) -> torch.Tensor:
        T = h.shape[0]
        H, dim, rd, rank = self.H, self.dim, self.rd, self.rank
        proj = self.in_proj(h)
        q, dkv = proj[:, : self.q_end], proj[:, self.q_end: self.dkv_end]
        kernels.latent_prepare(q, dkv, cache.rows, self.c_norm, self.inv_freq, self.rot_mult, positions,
                               params.new_cache_slots, H, dim, rd, self.rot_dims, rank, self.eps, self.half_pairs)
        qu = q.view(T, H, dim + rd)[:, :, :dim].transpose(0, 1)                 # [H, T, dim] (strided view)
        qa = torch.bmm(qu, self.uk)                                             # folded query [H, T, rank]
        lat = kernels.latent_attn(qa, q, cache.rows, params.q_cu_seq_lens, params.kv_cu_seq_lens,
                                  params.block_tables, params.cu_block_lens, params.token_seq, H, dim, rd, rank,
                                  cache.block_size(), self.scale, params.kv_max_seq_len, self.window)
        o = torch.bmm(lat, self.uv_t)                                           # [H, T, vdim]
        o = kernels.heads_to_rows(o, proj[:, self.dkv_end:] if self.has_gate else None)
        return self.o_proj.forward_fusable(o) if self.fusable_out else self.o_proj(o)

    __call__ = forward


class DeltaRuleMixer:
    """Generalised delta rule (csrc/delta_rule.cu): r, k, v, output gate and removal logits are
    projections of h; the decay logits come through a low-rank pair W2 tanh(W1 h).  The recurrent
    state [n_slots, H, d, d] is fp32."""

    def __init__(self, w: Dict[str, torch.Tensor], n_heads: int, head_dim: int, decay_scale: float,
                 key_eps: float, eps: float, n_slots: int, dtype: torch.dtype, device):
        self.H, self.d, self.dtype = n_heads, head_dim, dtype
        self.decay_scale, self.key_eps, self.eps = decay_scale, key_eps, eps
        self.n = n_heads * head_dim
        self.in_proj = Linear(torch.cat([w["r"], w["k"], w["v"], w["g"], w["a"], w["w1"]], dim=0))
        self.w2 = Linear(w["w2"])
        f = lambda t: t.to(torch.float32).contiguous()
        self.w0, self.a0, self.norm_weight = f(w["w0"]), f(w["a.b"]), f(w["norm"])
        self.o_proj = Linear(w["o"])
        self.state = torch.zeros((n_slots, n_heads, head_dim, head_dim), dtype=torch.float32, device=device)

    def forward(self, h: torch.Tensor, positions: torch.Tensor, params: InputParameters) -> torch.Tensor:
        n = self.n
        proj = self.in_proj(h)
        r, k, v, g, a = (proj[:, i * n:(i + 1) * n] for i in range(5))
        wl = self.w2(torch.tanh(proj[:, 5 * n:]))
        o = kernels.delta_rule(r, k, v, wl, a, g, self.w0, self.a0, self.norm_weight, self.state,
                               params.q_cu_seq_lens, positions, params.state_slots, self.H, self.d,
                               self.decay_scale, self.key_eps, self.eps)
        return self.o_proj(o)

    __call__ = forward


class GatedMLP:
    """down(act(gate h) * (up h)); act "silu" or "gelu_tanh".  gate and up share one GEMM.  For decode-sized bf16
    steps the SiLU form takes the split-K partials of that GEMM (its reduction folded into the activation launch)."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act: str):
        self.gate_up, self.down, self.act = Linear(torch.cat([gate, up], dim=0)), Linear(down), act
        self.ff = gate.shape[0]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if (self.act == "silu" and h.dtype == torch.bfloat16 and self.ff % 64 == 0
                and self.gate_up.supports_partials(h.shape[0]) and kernels.silu_mul_splitk_available()):
            return self.down(kernels.silu_mul_splitk(self.gate_up.forward_partials(h), h.dtype))
        return self.down(kernels.gated_act(self.gate_up(h), self.act))

    __call__ = forward


class SparseMoE:
    """Token-choice experts with a sigmoid router: s = sigmoid(Wr h) in fp32, the `top` largest are chosen,
    the routing weight is s (not renormalised) and scales the expert's INPUT:
        out = sum over chosen e of down_e(act(gate_e x) * (up_e x)),  x = s_e * h.
    Expert weights are stacked [E, ...]; pairs are grouped by expert on the device (no host sync)."""

    def __init__(self, router: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                 top: int, act: str):
        self.router = router.to(torch.float32).contiguous()
        self.gate_up = torch.cat([gate, up], dim=1).contiguous()     # [E, 2 ff, W]
        self.down = down.contiguous()                                  # [E, W, ff]
        self.E, self.top, self.act = router.shape[0], top, act

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        rows = h.shape[0]
        ids, wts = kernels.moe_route(h, self.router, self.top)
        offsets, sorted_pair, pos_of_pair = kernels.moe_plan(ids, self.E)
        n = rows * self.top
        gu = kernels.grouped_gemm(h, self.gate_up, offsets, n, sorted_pair, wts.view(-1), self.top)
        y = kernels.grouped_gemm(kernels.gated_act(gu, self.act), self.down, offsets, n)
        return kernels.moe_combine(y, pos_of_pair, rows, self.top)

    __call__ = forward


# ---------------------------------------------------------------------------
# Layers of decoders that normalise each sublayer's result (post-norm on the branch), mix tokens with a
# minimal gated recurrence or with differential sliding-window attention, and add a per-token learned term.
# ---------------------------------------------------------------------------
class PostNormResidual:
    """x <- x + mult * group_rms_norm(y) * w on an fp32 residual x: the sublayer reads x itself and its RESULT y is
    normalised (the row in `groups` equal consecutive parts, each with its own root mean square).  With a history
    [stages, rows, W] the new x becomes stage n_hist - 1 and what the next layer reads is sum_j coef[j] stage_j."""

    def __init__(self, weight: torch.Tensor, groups: int, mult: float, eps: float):
        self.weight = weight.to(torch.float32).contiguous()
        self.groups, self.mult, self.eps = groups, mult, eps

    def forward(self, x: torch.Tensor, y, x_out: Optional[torch.Tensor] = None,
                hist: Optional[torch.Tensor] = None, n_hist: int = 0, coef: Optional[torch.Tensor] = None):
        """y: the sublayer's result, or the split-K partials of the product that makes it (Linear.forward_fusable).
        Returns (new x fp32, the same rows in y's dtype for the next matrix product — x itself in fp32)."""
        if isinstance(y, kernels.W4Partials):
            out, h = kernels.postnorm_residual_splitk(x, y, self.weight, self.groups, self.mult, self.eps,
                                                      torch.bfloat16, hist, n_hist, coef, x_out)
        else:
            out, h = kernels.postnorm_residual(x, y, self.weight, self.groups, self.mult, self.eps, hist, n_hist,
                                               coef, x_out)
        return out, (h if h is not None else out)

    __call__ = forward


class MinGRUMixer:
    """z = sigmoid(Wz h + bz), u = Wx h + bx, c = u + 1/2 (u >= 0) | sigmoid(u); S_t = (1 - z) S_{t-1} + z c per
    channel (fp32, one state row per sequence slot); out = Wo (S_t * silu(Wg h)).  (csrc/mingru.cu)"""

    def __init__(self, w: Dict[str, torch.Tensor], n_slots: int, dtype: torch.dtype, device):
        self.width = w["z"].shape[0]
        self.in_proj = Linear(torch.cat([w["z"], w["x"], w["g"]], dim=0))
        f = lambda t: None if t is None else t.to(torch.float32).contiguous()
        self.z_bias, self.x_bias = f(w.get("z.b")), f(w.get("x.b"))
        self.o_proj = Linear(w["o"])
        self.state = torch.zeros((n_slots, self.width), dtype=torch.float32, device=device)

    def forward(self, h: torch.Tensor, positions: torch.Tensor, params: InputParameters) -> torch.Tensor:
        o = kernels.mingru_scan(self.in_proj(h), self.z_bias, self.x_bias, self.state, params.q_cu_seq_lens,
                                positions, params.state_slots, params.num_sequences, self.width,
                                params.q_max_seq_len)
        return self.o_proj.forward_fusable(o)

    __call__ = forward


class DiffAttention:
    """Differential attention (csrc/diff_attn.cu): per head two query/key maps [dim] over one set of values [vdim],
        o = softmax(s1) V - lam softmax(s2) V,  lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff,
        o <- o / rms(o) * (1 - diff) * sigmoid(Wg h)_head ; out = Wo concat(o)
    with per-map RMS norm (one weight [dim] for queries, one for keys) before the rotary turn, a sliding window of
    `window` keys that also keeps the first `keep_first` tokens visible (window 0: plain causal), and H / G query
    heads per key/value head.  A layer built without its own k / v weights attends over another layer's cache."""

    def __init__(self, w: Dict[str, torch.Tensor], n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 window: int, keep_first: int, diff: float, inv_freq: Optional[torch.Tensor], rot_mult: float,
                 rot_dims: int, eps: float, dtype: torch.dtype, device):
        self.H, self.G, self.dim, self.vd = n_heads, n_kv_heads, dim, vdim
        self.scale, self.window, self.keep_first, self.diff = scale, window, keep_first, diff
        self.rot_mult, self.rot_dims, self.eps, self.dtype = rot_mult, rot_dims, eps, dtype
        self.inv_freq = None if inv_freq is None else inv_freq.to(torch.float32).to(device).contiguous()
        self.own_kv = "k" in w
        parts = [w["q"]] + ([w["k"], w["v"]] if self.own_kv else []) + ([w["g"]] if "g" in w else [])
        self.has_gate = "g" in w
        self.in_proj = Linear(torch.cat(parts, dim=0))          # one GEMM for everything that reads h
        self.q_end = n_heads * 2 * dim
        self.k_end = self.q_end + (n_kv_heads * 2 * dim if self.own_kv else 0)
        self.v_end = self.k_end + (n_kv_heads * vdim if self.own_kv else 0)
        f = lambda t: t.to(torch.float32).contiguous()
        self.q_norm = f(w["q.norm"])
        self.k_norm = f(w["k.norm"]) if self.own_kv else None
        d = lambda a, b: float((w[a].double() * w[b].double()).sum())
        self.lam = math.exp(d("lq1", "lk1")) - math.exp(d("lq2", "lk2")) + diff
        self.o_proj = Linear(w["o"])

    def forward(self, h: torch.Tensor, positions: torch.Tensor, cache: KVCache, params: InputParameters) -> torch.Tensor:
        proj = self.in_proj(h)
        k_in = proj[:, self.q_end: self.k_end] if self.own_kv else None
        v_in = proj[:, self.k_end: self.v_end] if self.own_kv else None
        q = kernels.diff_attn_prepare(proj[:, : self.q_end], k_in, v_in, cache.key_cache if self.own_kv else None,
                                      cache.value_cache if self.own_kv else None, self.q_norm, self.k_norm,
                                      self.inv_freq, self.rot_mult, self.rot_dims, positions, params.new_cache_slots,
                                      self.H, self.G, self.dim, self.vd, self.eps)
        gate = proj[:, self.v_end: self.v_end + self.H] if self.has_gate else None
        o = kernels.diff_attn(q, cache.key_cache, cache.value_cache, gate, params.q_cu_seq_lens, params.kv_cu_seq_lens,
                              params.block_tables, params.cu_block_lens, params.token_seq, cache.block_size(),
                              self.scale, self.window, self.keep_first, self.lam, 1.0 - self.diff, self.eps,
                              params.num_sequences, params.q_max_seq_len, params.kv_max_seq_len)
        return self.o_proj.forward_fusable(o)

    __call__ = forward


class ClampedGLU:
    """down(g * sigmoid(slope * g) * (u + 1)), g = min(gate h, limit), u = clamp(up h, -limit, limit).
    gate and up share one GEMM."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float, slope: float):
        self.gate_up, self.down = Linear(torch.cat([gate, up], dim=0)), Linear(down)
        self.limit, self.slope = limit, slope

    def forward(self, h: torch.Tensor, fusable_out: bool = True):
        """The result, or (fusable_out) the down projection's split-K partials where the post-norm can take them."""
        gu = self.gate_up.forward_fusable(h)
        if isinstance(gu, kernels.W4Partials):
            act = kernels.glu_clamped_splitk(gu, self.limit, self.slope, h.dtype)
        else:
            act = kernels.glu_clamped(gu, self.limit, self.slope)
        return self.down.forward_fusable(act) if fusable_out else self.down(act)

    __call__ = forward


class TokenSideInput:
    """A per-token, per-layer learned vector e = table[token, col0 : col0 + dim] gates a narrow projection of the
    residual: y = P (gelu_tanh(G h) * e), which enters the residual through a PostNormResidual.  Steps of at most
    FUSED_ROWS rows run gate, projection and post-norm as one launch."""

    FUSED_ROWS = 64

    def __init__(self, table: torch.Tensor, col0: int, gate: torch.Tensor, proj: torch.Tensor, norm: PostNormResidual):
        self.table, self.col0, self.norm = table, col0, norm
        self.gate, self.proj = Linear(gate), Linear(proj)
        self.proj_t = proj.t().contiguous()       # [dim, W]: the one-launch form reads it along W

    def forward(self, x: torch.Tensor, h: torch.Tensor, tokens: torch.Tensor, x_out: Optional[torch.Tensor] = None,
                hist: Optional[torch.Tensor] = None, n_hist: int = 0, coef: Optional[torch.Tensor] = None):
        """x: fp32 residual, h: the same rows as the matrix products read them.  Returns (new x, new h)."""
        n = self.norm
        if x.shape[0] <= self.FUSED_ROWS:
            out, hh = kernels.token_side_postnorm(x, h, self.gate.weight, self.proj_t, self.table, self.col0,
                                                  tokens, n.weight, n.groups, n.mult, n.eps, hist, n_hist, coef, x_out)
            return out, (hh if hh is not None else out)
        y = self.proj(kernels.token_gated_gelu(self.gate(h), self.table, self.col0, tokens))
        return n(x, y, x_out=x_out, hist=hist, n_hist=n_hist, coef=coef)

    __call__ = forward


# ---------------------------------------------------------------------------
# Layers of decoders that normalise after the residual sum with one gain per norm, attend with unit-length queries
# and keys under a distance bias and a sink, and choose experts by the token id.
# ---------------------------------------------------------------------------
class SumNormResidual:
    """x <- (alpha x + y) / rms(alpha x + y) * w on an fp32 residual x: the sublayer reads x itself and the norm
    follows the sum.  w: one number for all channels, or one per channel."""

    def __init__(self, weight: torch.Tensor, alpha: float, eps: float):
        self.weight = weight.to(torch.float32).reshape(-1).contiguous()
        self.alpha, self.eps = alpha, eps

    def forward(self, x: torch.Tensor, y, dtype: torch.dtype, x_out: Optional[torch.Tensor] = None):
        """y: the sublayer's result, or the split-K partials of the product that makes it (Linear.forward_fusable).
        Returns (new x fp32, the same rows in `dtype` for the next matrix product — x itself in fp32)."""
        out, h = kernels.sumnorm_residual(x, y, self.weight, self.alpha, self.eps, dtype, x_out)
        return out, (h if h is not None else out)

    __call__ = forward


class SinkAttention:
    """Causal softmax attention (csrc/sink_attn.cu) whose queries and keys are divided by their root mean square per
    head (no weight), with
        a query temperature  q_i *= 1 + temp_coef ln(floor((i + 1) / temp_every) + 1)        (temp_every 0: none)
        a distance bias      s_ij = scale q_i . k_j - r1_h ln(1 + r2_h (i - j))               ("r1", "r2" [H], optional)
        a sink               exp(sink_h) joins the softmax denominator, with no value         ("sink" [H], optional)
    and H / G query heads per key/value head.  With mix_values the layer blends its values with those that another
    layer made of the same tokens, v <- (1 - lam) v + lam v_other, before caching them; `lam` is this layer's
    number.  No rotary turn: positions enter through the temperature and the bias only."""

    def __init__(self, w: Dict[str, torch.Tensor], n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 temp_coef: float, temp_every: int, lam: Optional[float], eps: float, dtype: torch.dtype, device):
        self.H, self.G, self.dim, self.vd = n_heads, n_kv_heads, dim, vdim
        self.scale, self.temp_coef, self.temp_every, self.lam = scale, temp_coef, temp_every, lam
        self.eps, self.dtype = eps, dtype
        self.in_proj = Linear(torch.cat([w["q"], w["k"], w["v"]], dim=0))       # one GEMM for everything that reads h
        self.q_end = n_heads * dim
        self.k_end = self.q_end + n_kv_heads * dim
        self.v_end = self.k_end + n_kv_heads * vdim
        f = lambda name: w[name].to(torch.float32).to(device).contiguous() if name in w else None
        self.r1, self.r2, self.sink = f("r1"), f("r2"), f("sink")
        if (self.r1 is None) != (self.r2 is None):
            raise ValueError("the distance bias takes both r1 and r2")
        self.o_proj = Linear(w["o"])

    def forward(self, h: torch.Tensor, positions: torch.Tensor, cache: KVCache, params: InputParameters,
                v_other: Optional[torch.Tensor] = None):
        """Returns (the mixer's result or its split-K partials, this layer's own unblended values of the step's rows
        [rows, G * vdim]: what a later layer may blend into its own)."""
        proj = self.in_proj(h)
        v_in = proj[:, self.k_end: self.v_end]
        blend = v_other if self.lam is not None else None
        q = kernels.sink_attn_prepare(proj[:, : self.q_end], proj[:, self.q_end: self.k_end], v_in, blend,
                                      self.lam if blend is not None else 0.0, cache.key_cache, cache.value_cache,
                                      positions, params.new_cache_slots, self.H, self.G, self.dim, self.vd, self.eps,
                                      self.temp_coef, self.temp_every)
        o = kernels.sink_attn(q, cache.key_cache, cache.value_cache, self.r1, self.r2, self.sink,
                              params.q_cu_seq_lens, params.kv_cu_seq_lens, params.block_tables, params.cu_block_lens,
                              params.token_seq, cache.block_size(), self.scale, params.num_sequences,
                              params.q_max_seq_len, params.kv_max_seq_len)
        return self.o_proj.forward_fusable(o), v_in

    __call__ = forward


class TableMoE:
    """Experts chosen by the token id: row `tok` of an integer table [vocab, top] names the token's experts, each
    weighted 1 / top:   out = (1 / top) sum_e down_e(act(gate_e h) * (up_e h))  (+ shared(h), an expert that every
    token uses).  Expert weights are stacked [E, ...]; pairs are grouped by expert on the device (no host sync)."""

    def __init__(self, table: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act: str,
                 shared: Optional["GatedMLP"] = None):
        self.table = table.to(torch.int32).contiguous()
        self.gate_up = torch.cat([gate, up], dim=1).contiguous()     # [E, 2 ff, W]
        self.down = down.contiguous()                                  # [E, W, ff]
        self.E, self.top, self.act, self.shared = gate.shape[0], self.table.shape[1], act, shared

    def forward(self, h: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        rows = h.shape[0]
        ids = kernels.moe_table_route(self.table, tokens, self.E)
        offsets, sorted_pair, pos_of_pair = kernels.moe_plan(ids, self.E)
        n = rows * self.top
        gu = kernels.grouped_gemm(h, self.gate_up, offsets, n, sorted_pair, None, self.top)
        y = kernels.grouped_gemm(kernels.gated_act(gu, self.act), self.down, offsets, n)
        return kernels.moe_combine(y, pos_of_pair, rows, self.top, 1.0 / self.top,
                                   self.shared(h) if self.shared is not None else None)

    __call__ = forward


# ---------------------------------------------------------------------------
# Layers of decoders that run two mixers side by side on the same rows (sigmoid attention inside blocks of positions
# with a head mix, and a gated delta rule with short input filters), average their normalised results, and route
# tokens to experts with a softmax router under group limits.
# ---------------------------------------------------------------------------
class BranchNormResidual:
    """x <- x + norm(m) w on an fp32 residual, where m is a sublayer's result, or the average of two results each
    normalised with its own weight first: m = (norm(a) wa + norm(b) wb) / 2.  norm(z) = z / sqrt(mean(z^2) + eps).
    The new residual is handed on under the next sublayer's input norm (next_weight) or as it is."""

    def __init__(self, weight: torch.Tensor, eps: float, weight_a: Optional[torch.Tensor] = None,
                 weight_b: Optional[torch.Tensor] = None):
        f = lambda t: None if t is None else t.to(torch.float32).contiguous()
        self.weight, self.weight_a, self.weight_b, self.eps = f(weight), f(weight_a), f(weight_b), eps

    def forward(self, x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor] = None,
                next_weight: Optional[torch.Tensor] = None, want_h: bool = True):
        """Returns (new x fp32, the rows the next matrix product reads in a's dtype, or None if not wanted)."""
        return kernels.branch_norm_residual(x, a, b, self.weight_a, self.weight_b if b is not None else None,
                                            self.weight, next_weight, self.eps, want_h=want_h)

    __call__ = forward


class SigmoidBlockAttention:
    """Attention whose weights are sigmoids, not a softmax (csrc/sigmoid_attn.cu):
        q, k, v = affine maps of h (biases "q.b", "k.b", "v.b", optional); the first rot_dims channels of every q and
        k head turn with the position (channel t with t + rot_dims / 2, angle p * inv_freq[t]);
        s = cap tanh(scale q . k / cap) (cap 0: none); a_h(i, j) = sigmoid(s + pb_h) for the keys j <= i of i's block
        of `size` positions counted from 0 (size 0: all j <= i); a'_h = sum_g talk[h, g] a_g (no "talk": a' = a);
        out = Wo concat_h(sum_j a'_h(i, j) v_kv(h)(j)),  H / G query heads per key/value head.
    `in_weight` [n_in, W] is everything that reads h, so a caller with other mixers on the same rows can make one
    matrix product of them and hand this mixer its column block (run)."""

    def __init__(self, w: Dict[str, torch.Tensor], n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 cap: float, size: int, inv_freq: Optional[torch.Tensor], rot_dims: int, dtype: torch.dtype, device):
        self.H, self.G, self.dim, self.vd = n_heads, n_kv_heads, dim, vdim
        self.scale, self.cap, self.size, self.rot_dims, self.dtype = scale, cap, size, rot_dims, dtype
        self.inv_freq = None if inv_freq is None else inv_freq.to(torch.float32).to(device).contiguous()
        self.in_weight = torch.cat([w["q"], w["k"], w["v"]], dim=0)
        self.n_in = self.in_weight.shape[0]
        self.q_end = n_heads * dim
        self.k_end = self.q_end + n_kv_heads * dim
        f = lambda name: w[name].to(torch.float32).to(device).contiguous() if name in w else None
        self.q_bias, self.k_bias, self.v_bias = f("q.b"), f("k.b"), f("v.b")
        self.head_bias, self.head_mix = f("pb"), f("talk")
        self.o_proj = Linear(w["o"])
        self._in_proj: Optional[Linear] = None

    def run(self, proj: torch.Tensor, positions: torch.Tensor, cache: KVCache, params: InputParameters) -> torch.Tensor:
        """proj [rows, n_in]: this mixer's column block of the input product (without biases)."""
        q = kernels.sigmoid_attn_prepare(proj[:, : self.q_end], proj[:, self.q_end: self.k_end],
                                         proj[:, self.k_end: self.n_in], self.q_bias, self.k_bias, self.v_bias,
                                         cache.key_cache, cache.value_cache, self.inv_freq, positions,
                                         params.new_cache_slots, self.H, self.G, self.dim, self.vd, self.rot_dims)
        o = kernels.sigmoid_attn(q, cache.key_cache, cache.value_cache, self.head_bias, self.head_mix,
                                 params.q_cu_seq_lens, params.kv_cu_seq_lens, params.block_tables,
                                 params.cu_block_lens, params.token_seq, cache.block_size(), self.scale, self.cap,
                                 self.size, params.q_max_seq_len, params.num_sequences, params.kv_max_seq_len)
        return self.o_proj(o)

    def forward(self, h: torch.Tensor, positions: torch.Tensor, cache: KVCache, params: InputParameters) -> torch.Tensor:
        if self._in_proj is None:
            self._in_proj = Linear(self.in_weight)
        return self.run(self._in_proj(h), positions, cache, params)

    __call__ = forward


class GatedDeltaMixer:
    """Gated delta rule with a decay per key channel and short causal filters on its inputs (csrc/delta_rule.cu):
        q, k [G heads x dim], v [H heads x vdim] = silu(filter(W h)), filters [channels, taps] ("q.conv", ...);
        q, k of unit length per head (unit_eps under the root), q times dim^(-1/2); beta = sigmoid(Wb h) per head;
        decay = exp(-exp(A_log_h) softplus(a2 (a1 h) + dt_bias)) per head and key channel;
        S <- diag(decay) S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q      (S [dim, vdim] per head, fp32)
        out = Wo concat_h(o / rms(o) * norm * sigmoid(g2 (g1 h))),  value head h reads q / k head h / (H / G).
    Per sequence slot the layer keeps S and the last taps - 1 filter inputs, both fp32.  `in_weight` [n_in, W] is
    everything that reads h (see SigmoidBlockAttention)."""

    def __init__(self, w: Dict[str, torch.Tensor], n_heads: int, n_kv_heads: int, dim: int, vdim: int, unit_eps: float,
                 eps: float, n_slots: int, dtype: torch.dtype, device):
        self.H, self.G, self.dim, self.vd = n_heads, n_kv_heads, dim, vdim
        self.unit_eps, self.eps, self.dtype = unit_eps, eps, dtype
        self.nqk, self.nv = n_kv_heads * dim, n_heads * vdim
        self.ra, self.rg = w["a1"].shape[0], w["g1"].shape[0]
        self.in_weight = torch.cat([w["q"], w["k"], w["v"], w["b"], w["a1"], w["g1"]], dim=0)
        self.n_in = self.in_weight.shape[0]
        # the second factors of the decay and gate pairs as ONE product: [a1 h | g1 h] times a block-diagonal weight
        # (the zero blocks add exact zeros), so a step has one small launch instead of two and two copies
        low2 = torch.zeros((n_heads * dim + self.nv, self.ra + self.rg), dtype=w["a2"].dtype, device=w["a2"].device)
        low2[: n_heads * dim, : self.ra] = w["a2"]
        low2[n_heads * dim:, self.ra:] = w["g2"]
        self.low2 = Linear(low2)
        f = lambda t: t.to(torch.float32).to(device).contiguous()
        self.q_filter, self.k_filter, self.v_filter = f(w["q.conv"]), f(w["k.conv"]), f(w["v.conv"])
        self.taps = self.q_filter.shape[1]
        self.a_log, self.dt_bias, self.norm_weight = f(w["A_log"]), f(w["dt_bias"]), f(w["norm"])
        self.o_proj = Linear(w["o"])
        self.state = torch.zeros((n_slots, n_heads, dim, vdim), dtype=torch.float32, device=device)
        self.filter_state = torch.zeros((n_slots, max(self.taps - 1, 0), 2 * self.nqk + self.nv), dtype=torch.float32,
                                        device=device)
        self._in_proj: Optional[Linear] = None

    def run(self, proj: torch.Tensor, positions: torch.Tensor, params: InputParameters) -> torch.Tensor:
        """proj [rows, n_in]: this mixer's column block of the input product."""
        o0 = 2 * self.nqk + self.nv
        low = self.low2(proj[:, o0 + self.H: o0 + self.H + self.ra + self.rg])      # [decay logits | gate logits]
        nd = self.H * self.dim
        q, k, v, decay, beta = kernels.gated_delta_prepare(
            proj[:, : self.nqk], proj[:, self.nqk: 2 * self.nqk], proj[:, 2 * self.nqk: o0], proj[:, o0: o0 + self.H],
            low[:, :nd], self.q_filter, self.k_filter, self.v_filter, self.a_log, self.dt_bias, self.filter_state,
            params.q_cu_seq_lens, positions, params.token_seq, params.state_slots, self.H, self.G, self.dim, self.vd,
            self.unit_eps)
        o = kernels.gated_delta_scan(q, k, v, decay, beta, low[:, nd:], self.norm_weight, self.state,
                                     params.q_cu_seq_lens, positions, params.state_slots, self.eps,
                                     params.q_max_seq_len)
        return self.o_proj(o)

    def forward(self, h: torch.Tensor, positions: torch.Tensor, params: InputParameters) -> torch.Tensor:
        if self._in_proj is None:
            self._in_proj = Linear(self.in_weight)
        return self.run(self._in_proj(h), positions, params)

    __call__ = forward


class ParallelMixer:
    """Two mixers side by side on the same rows: an attention-like one with a paged cache (`left`) and a recurrent one
    with state slots (`right`).  Everything that reads h is ONE matrix product; the results come back as a pair (the
    caller's BranchNormResidual normalises and averages them)."""

    def __init__(self, left, right):
        self.left, self.right = left, right
        self.in_proj = Linear(torch.cat([left.in_weight, right.in_weight], dim=0))

    def forward(self, h: torch.Tensor, positions: torch.Tensor, cache: KVCache, params: InputParameters):
        proj = self.in_proj(h)
        n = self.left.n_in
        return (self.left.run(proj[:, :n], positions, cache, params),
                self.right.run(proj[:, n:], positions, params))

    __call__ = forward


class ReluSquaredMLP:
    """down(max(up h, 0)^2)."""

    def __init__(self, up: torch.Tensor, down: torch.Tensor):
        self.up, self.down = Linear(up), Linear(down)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(kernels.relu_squared(self.up(h)))

    __call__ = forward


class GroupLimitedMoE:
    """Token-choice experts behind a softmax router (csrc/moe.cu):
        p = softmax(R h) in fp32 over n_real + n_pass outputs; choice score c = p + correction; the outputs form
        n_groups equal runs of neighbours, a run scores its largest c, and only outputs of the keep_groups best runs
        can be chosen; the `top` largest c are chosen; weight = p / (sum of the chosen p + weight_eps);
        out = sum over chosen e of weight_e * expert_e(h), where the last n_pass outputs are pass-through experts
        (expert(h) = h, no weights) and a real expert is down(g sigmoid(slope g) (u + 1)), g = min(gate h, limit),
        u = clamp(up h, -limit, limit);  plus sigmoid(w_sg . h) * shared(h) for an expert every token uses.
    Expert weights are stacked [n_real, ...]; pairs are grouped by output on the device (no host sync); the pairs of
    pass-through outputs sort after every real expert's and never enter a matrix product."""

    def __init__(self, router: torch.Tensor, correction: Optional[torch.Tensor], gate: torch.Tensor, up: torch.Tensor,
                 down: torch.Tensor, top: int, n_groups: int, keep_groups: int, limit: float, slope: float,
                 weight_eps: float, shared: Optional["ClampedGLU"] = None, shared_gate: Optional[torch.Tensor] = None):
        f = lambda t: None if t is None else t.to(torch.float32).contiguous()
        self.router, self.correction = f(router), f(correction)
        self.gate_up = torch.cat([gate, up], dim=1).contiguous()     # [n_real, 2 ff, W]
        self.down = down.contiguous()                                  # [n_real, W, ff]
        self.n_out, self.n_real, self.top = router.shape[0], gate.shape[0], top
        self.n_groups, self.keep_groups = n_groups, keep_groups
        self.limit, self.slope, self.weight_eps = limit, slope, weight_eps
        self.shared = shared
        self.shared_gate = None if shared_gate is None else f(shared_gate.reshape(-1))
        if self.n_out < self.n_real or self.n_out % max(n_groups, 1):
            raise ValueError(f"router with {self.n_out} outputs for {self.n_real} experts in {n_groups} groups")

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        rows = h.shape[0]
        ids, wts, sg = kernels.moe_route_softmax(h, self.router, self.correction, self.top, self.n_groups,
                                                 self.keep_groups, self.weight_eps,
                                                 self.shared_gate if self.shared is not None else None)
        offsets, sorted_pair, pos_of_pair = kernels.moe_plan(ids, self.n_out)
        real = offsets[: self.n_real + 1]
        n = rows * self.top
        gu = kernels.grouped_gemm(h, self.gate_up, real, n, sorted_pair, None, self.top)
        y = kernels.grouped_gemm(kernels.glu_clamped(gu, self.limit, self.slope), self.down, real, n)
        shared = self.shared(h, fusable_out=False) if self.shared is not None else None
        return kernels.moe_combine_weighted(y, pos_of_pair, ids, wts, self.n_real, h, shared, sg)

    __call__ = forward
