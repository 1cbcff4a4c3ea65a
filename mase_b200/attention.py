"""Quantized attention block and gated MLP around the MX Linear layers
(chop/nn/quantized/modules/llama/attention.py:130-457, mlp.py:48-77).

The reference's classes subclass the transformers library's LlamaAttention / LlamaMLP of one pinned release; the
classes here carry the same children (`q_proj`, `k_proj`, `v_proj`, `o_proj`; `gate_proj`, `up_proj`, `down_proj`,
plain `nn.Linear` that the quantize pass swaps separately by name), the same `q_config` / `bypass` keys and the same
arithmetic, without the dependency: they are built from the sizes (or from any module that has those children) and
called like the reference's (`hidden_states, position_embeddings, attention_mask, past_key_value, cache_position`).

What runs on this package's kernels: the rotary embedding with quantized tables (`mxq_rope`), the MX quantizers of
queries, probabilities and cached keys / values, the quantizer + fp32 softmax (`mxq_softmax_quant`), and both matrix
products as one batched launch each (`mxq_gemm_dense_batched`: Q K^T over batch x heads with K = head_dim, P V with
K = the key length).  One operand of each product is unquantized in the reference (keys, values), so fp32 tensors go
through the split that keeps fp32-level products; bf16 products are exact.
"""

from __future__ import annotations

import torch
from torch import Tensor, nn

from . import functional as F_mx
from .gemm import batched_product
from .modules import forward_siblings
from .quantizers import mxfp_quantizer, mxint_quantizer


def repeat_kv(x: Tensor, n_rep: int) -> Tensor:
    """[batch, kv_heads, seq, dim] -> [batch, kv_heads * n_rep, seq, dim]."""
    if n_rep == 1:
        return x
    b, h, s, d = x.shape
    return x[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)


class HeadRMSNorm(nn.Module):
    """weight * x / sqrt(mean(x^2) + eps) over the last dimension, evaluated in fp32 and cast back before the weight
    is applied (the RMS norm of the transformers library's Llama / Qwen3 models)."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.variance_epsilon = eps

    def forward(self, x: Tensor) -> Tensor:
        dt = x.dtype
        x = x.to(torch.float32)
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * x.to(dt)


class _AttentionMX(nn.Module):
    _qk_norm = False
    _format = ""  # "mxfp" / "mxint": the operand quantizer of queries, probabilities and cached keys / values

    def __init__(self, config=None, layer_idx: int = 0, q_config: dict | None = None, *, hidden_size: int | None = None,
                 num_heads: int | None = None, num_kv_heads: int | None = None, head_dim: int | None = None,
                 bias: bool = False, attention_dropout: float = 0.0, rms_norm_eps: float = 1e-6, device=None, dtype=None):
        """Either `config` (an object with hidden_size, num_attention_heads, num_key_value_heads and optionally
        head_dim, attention_bias, attention_dropout -- the call the quantize pass makes,
        chop/passes/module/module_modify_helper.py:265-275) or the sizes as keywords."""
        super().__init__()
        if config is not None:
            hidden_size = config.hidden_size
            num_heads = config.num_attention_heads
            num_kv_heads = getattr(config, "num_key_value_heads", None)
            head_dim = getattr(config, "head_dim", None)
            bias = getattr(config, "attention_bias", False)
            attention_dropout = getattr(config, "attention_dropout", 0.0)
            rms_norm_eps = getattr(config, "rms_norm_eps", rms_norm_eps)
        self.config = config
        self.layer_idx = layer_idx
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = head_dim or hidden_size // num_heads
        self.num_key_value_groups = self.num_heads // self.num_kv_heads
        self.scaling = self.head_dim ** -0.5
        self.attention_dropout = attention_dropout
        kw = {"device": device, "dtype": dtype}
        self.q_proj = nn.Linear(hidden_size, self.num_heads * self.head_dim, bias=bias, **kw)
        self.k_proj = nn.Linear(hidden_size, self.num_kv_heads * self.head_dim, bias=bias, **kw)
        self.v_proj = nn.Linear(hidden_size, self.num_kv_heads * self.head_dim, bias=bias, **kw)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, hidden_size, bias=bias, **kw)
        if self._qk_norm:  # the Qwen3 family normalises queries and keys over the head dimension
            self.q_norm = HeadRMSNorm(self.head_dim, rms_norm_eps, **kw)
            self.k_norm = HeadRMSNorm(self.head_dim, rms_norm_eps, **kw)
        q_config = q_config or {}
        self.qk_config = q_config.get("qk_matmul", {})
        self.av_config = q_config.get("av_matmul", {})
        self.rope_config = q_config.get("rope", {})
        self.softmax_config = q_config.get("softmax", {})
        self.kv_cache_config = q_config.get("kv_cache", {})
        self.qk_bypass = self.qk_config.get("bypass", False)
        self.av_bypass = self.av_config.get("bypass", False)
        self.rope_bypass = self.rope_config.get("bypass", False)
        self.softmax_bypass = self.softmax_config.get("bypass", False)
        self.kv_cache_bypass = self.kv_cache_config.get("bypass", False)

    # the operand quantizer of the format: MXFP or MXINT along the last dimension
    def _quantize(self, x: Tensor, cfg: dict) -> Tensor:
        raise NotImplementedError

    def _kv_cache(self, k: Tensor, v: Tensor):
        raise NotImplementedError

    @classmethod
    def from_attention(cls, attention: nn.Module, q_config: dict | None = None):
        """A block with the sizes and weights of `attention`: any module with q/k/v/o_proj Linear children and either a
        `config` (hidden_size, num_attention_heads, num_key_value_heads, head_dim) or `head_dim` of its own."""
        cfg = getattr(attention, "config", None)
        q, k = attention.q_proj, attention.k_proj
        head_dim = getattr(attention, "head_dim", None) or getattr(cfg, "head_dim", None) or \
            cfg.hidden_size // cfg.num_attention_heads
        norm = getattr(attention, "q_norm", None)
        new = cls(None, getattr(attention, "layer_idx", 0), q_config, hidden_size=q.in_features,
                  num_heads=q.out_features // head_dim, num_kv_heads=k.out_features // head_dim, head_dim=head_dim,
                  bias=q.bias is not None, attention_dropout=getattr(attention, "attention_dropout", 0.0),
                  rms_norm_eps=getattr(norm, "variance_epsilon", getattr(norm, "eps", None) or 1e-6),
                  device=q.weight.device, dtype=q.weight.dtype)
        new.load_state_dict(attention.state_dict(), strict=True)
        return new

    def _product(self, a: Tensor, b: Tensor, exact: bool) -> Tensor:
        """a[B, H, M, K] @ b[B, H, N, K]^T in one launch."""
        B, H, M, K = a.shape
        out = batched_product(a.reshape(B * H, M, K), b.reshape(B * H, b.shape[2], K), a.dtype, fp32_exact=exact)
        return out.view(B, H, M, b.shape[2])

    def forward(self, hidden_states: Tensor, position_embeddings, attention_mask: Tensor | None = None,
                past_key_value=None, cache_position=None, **kwargs):
        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, self.head_dim)
        q, k, v = forward_siblings([self.q_proj, self.k_proj, self.v_proj], hidden_states)
        q, k = q.view(hidden_shape), k.view(hidden_shape)
        if self._qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        query, key = q.transpose(1, 2), k.transpose(1, 2)
        value = v.view(hidden_shape).transpose(1, 2)
        cos, sin = position_embeddings
        if not self.rope_bypass:
            query, key = F_mx.rope_minifloat(query, key, cos, sin, self.rope_config)
        else:
            query, key = F_mx._apply_rope(query, key, cos, sin, 1)
        if past_key_value is not None:
            if not self.kv_cache_bypass:
                key, value = self._kv_cache(key, value)
            key, value = past_key_value.update(key, value, self.layer_idx,
                                               {"sin": sin, "cos": cos, "cache_position": cache_position})
        key = repeat_kv(key, self.num_key_value_groups)
        value = repeat_kv(value, self.num_key_value_groups)
        if not self.qk_bypass:
            query = self._quantize(query, self.qk_config)
        # only the quantized operand is known to fit tf32; the other one takes the fp32 split
        weights = self._product(query, key, exact=False)
        dropout = self.training and self.attention_dropout > 0
        # scaling, mask, the softmax with its input quantizer and the quantizer of the probabilities: one kernel
        fused = F_mx.attention_softmax(weights, self.scaling, attention_mask,
                                       None if self.softmax_bypass else "minifloat", self.softmax_config,
                                       None if self.av_bypass or dropout else self._format, self.av_config)
        if fused is not None:
            weights = fused
            if dropout:
                weights = nn.functional.dropout(weights, p=self.attention_dropout, training=True)
                if not self.av_bypass:
                    weights = self._quantize(weights, self.av_config)
        else:
            weights = weights * self.scaling
            if attention_mask is not None:
                weights = weights + attention_mask[:, :, :, : key.shape[-2]]
            if not self.softmax_bypass:
                weights = F_mx.softmax_minifloat(weights, self.softmax_config, dim=-1)
            else:
                weights = torch.softmax(weights.to(torch.float32), dim=-1).to(weights.dtype)
            if dropout:
                weights = nn.functional.dropout(weights, p=self.attention_dropout, training=True)
            if not self.av_bypass:
                weights = self._quantize(weights, self.av_config)
        out = self._product(weights, value.transpose(2, 3).contiguous(), exact=False)  # [B, H, S, D]
        out = out.transpose(1, 2).contiguous().reshape(*input_shape, -1)
        return self.o_proj(out), weights


class AttentionMXFP(_AttentionMX):
    """chop/nn/quantized/modules/llama/attention.py:130-233 (LlamaAttentionMXFP)."""

    _format = "mxfp"

    def _quantize(self, x, cfg):
        return mxfp_quantizer(x, block_size=cfg["data_in_block_size"], element_exp_bits=cfg["data_in_exponent_width"],
                              element_frac_bits=cfg["data_in_frac_width"], block_dim=-1)

    def _kv_cache(self, k, v):
        return F_mx.kv_cache_mxfp(k, v, self.kv_cache_config)


class AttentionMXInt(_AttentionMX):
    """chop/nn/quantized/modules/llama/attention.py:236-331 (LlamaAttentionMXInt)."""

    _format = "mxint"

    def _quantize(self, x, cfg):
        return mxint_quantizer(x, block_size=cfg["data_in_block_size"], element_bits=cfg["data_in_width"], block_dim=-1)

    def _kv_cache(self, k, v):
        return F_mx.kv_cache_mxint(k, v, self.kv_cache_config)


class GatedMLPMX(nn.Module):
    """down(silu(minifloat(gate(x))) * up(x)) (chop/nn/quantized/modules/llama/mlp.py:48-77; the MXFP and MXINT classes
    of the reference are the same code).  `q_config` holds the minifloat format of the SiLU input and `bypass`."""

    def __init__(self, config=None, layer_idx: int | None = None, q_config: dict | None = None, *,
                 hidden_size: int | None = None, intermediate_size: int | None = None, bias: bool = False, device=None,
                 dtype=None):
        super().__init__()
        if config is not None:
            hidden_size, intermediate_size = config.hidden_size, config.intermediate_size
            bias = getattr(config, "mlp_bias", False)
        self.config = config
        kw = {"device": device, "dtype": dtype}
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=bias, **kw)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=bias, **kw)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias, **kw)
        self.layer_idx = layer_idx
        self.q_config = q_config or {}
        self.bypass = self.q_config.get("bypass", False)

    @classmethod
    def from_mlp(cls, mlp: nn.Module, q_config: dict | None = None):
        g = mlp.gate_proj
        new = cls(None, getattr(mlp, "layer_idx", None), q_config, hidden_size=g.in_features,
                  intermediate_size=g.out_features, bias=g.bias is not None, device=g.weight.device, dtype=g.weight.dtype)
        new.load_state_dict(mlp.state_dict(), strict=True)
        return new

    def forward(self, x: Tensor) -> Tensor:
        gate, up = forward_siblings([self.gate_proj, self.up_proj], x)
        if self.bypass:
            return self.down_proj(nn.functional.silu(gate) * up)
        return self.down_proj(F_mx.silu_minifloat(gate, self.q_config) * up)


class Qwen3AttentionMXFP(AttentionMXFP):
    """chop/nn/quantized/modules/qwen3/attention.py:20-120: the same block with RMS norms over the head dimension of
    queries and keys before the rotary embedding (children `q_norm`, `k_norm`)."""

    _qk_norm = True


class Qwen3AttentionMXInt(AttentionMXInt):
    """chop/nn/quantized/modules/qwen3/attention.py:127-227."""

    _qk_norm = True


LlamaAttentionMXFP, LlamaAttentionMXInt = AttentionMXFP, AttentionMXInt
LlamaMLPMXFP = LlamaMLPMXInt = Qwen3MLPMXFP = Qwen3MLPMXInt = GatedMLPMX
