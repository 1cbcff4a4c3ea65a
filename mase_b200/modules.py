"""Quantized Linear modules with MASE's constructor, config keys and state_dict layout.

Counterparts of `LinearMXFP`, `LinearMXInt` and `LinearBlockFP` in
chop/nn/quantized/modules/linear.py (:817-895, :898-972, :199-219) and of `linearBlockFP` in
chop/nn/quantized/functional/linear.py:220-278.  The quantize pass builds them as
`cls(in_features, out_features, bias, device, dtype, config=...)` and then calls
`load_state_dict(old.state_dict(), strict=False)` (chop/passes/module/module_modify_helper.py:103-176),
which is where MX weights are quantized once; activations are quantized on every forward.
"""

from __future__ import annotations

from functools import partial

import torch
from torch import Tensor

from .gemm import (MXOperand, fp4_supported, linear_forward, mma_supported, mx_gated_linear, mx_gemm, mx_linear,
                   pack_mx_operand)
from .quantizers import block_fp_quantizer, mxfp_quantizer, mxint_quantizer


class _LinearBase(torch.nn.Linear):
    """chop/nn/quantized/modules/linear.py:61-83"""

    # dtype of the forward result; None = the input's dtype like the reference.  The row-parallel wrapper asks for
    # float32 partial sums so that the cross-GPU reduction happens before the only rounding to the output dtype.
    output_dtype = None

    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, dtype=None) -> None:
        super().__init__(in_features, out_features, bias, device, dtype)
        self.bypass = False
        self.pruning_masks = None


class LinearMXFP(_LinearBase):
    """Linear whose weight (and optionally bias) is MXFP-quantized at load time and whose input is
    MXFP-quantized along the feature dimension on every forward.  Inference only."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None, config=None):
        super().__init__(in_features, out_features, bias, device, dtype)
        assert config is not None, "config is None!"
        self.config = config
        self.bypass = config.get("bypass", False)
        self.gptq = config.get("gptq", False)
        self.clip_search = config.get("clip_search", False)

    def load_state_dict(self, state_dict, strict=True, assign=False):
        """Load pretrained weights, then quantize them in place (blocks run along in_features)."""
        if "weight_codes" in state_dict:  # written by a layer after drop_dense_weight()
            from . import _lib

            dev = self.weight.device
            codes, scales = state_dict["weight_codes"], state_dict["weight_scales"]
            want = [(self.out_features, self.in_features), (self.out_features, self.in_features // 2)]
            if tuple(codes.shape) not in want or codes.dtype != torch.uint8:
                raise RuntimeError(f"weight_codes of shape {tuple(codes.shape)} do not fit a layer "
                                   f"{self.in_features} -> {self.out_features}")
            if scales.numel() != int(_lib.lib().mxq_mma_scale_bytes(self.out_features, self.in_features)):
                raise RuntimeError(f"weight_scales hold {scales.numel()} bytes, not the scale array of a "
                                   f"[{self.out_features}, {self.in_features}] operand")
            if strict:
                unexpected = [k for k in state_dict if k not in ("weight", "bias", "weight_codes", "weight_scales")]
                if unexpected:
                    raise RuntimeError(f"unexpected keys in state_dict: {unexpected}")
            self._weight_dtype = self.weight.dtype
            self.register_buffer("weight_codes", state_dict["weight_codes"].to(dev), persistent=True)
            self.register_buffer("weight_scales", state_dict["weight_scales"].to(dev), persistent=True)
            self.weight = torch.nn.Parameter(torch.empty(0, dtype=self._weight_dtype, device=dev), requires_grad=False)
            self._dense_dropped = True
            if self.bias is not None and "bias" in state_dict:
                self.bias.data.copy_(state_dict["bias"])
            return torch.nn.modules.module._IncompatibleKeys([], [])
        result = super().load_state_dict(state_dict, strict=strict, assign=assign)
        if self.bypass or self.gptq:
            return result
        cfg = self.config
        self._weight_quantized = True  # from here on `weight` holds MX values: exact on the tf32 tensor cores
        self._pack_weight_for_tensor_cores()  # from the unquantized weight: quantizing twice is not idempotent
        self.weight.data.copy_(
            mxfp_quantizer(
                self.weight.data,
                block_size=cfg["weight_block_size"],
                element_exp_bits=cfg["weight_exponent_width"],
                element_frac_bits=cfg["weight_frac_width"],
                block_dim=1,
            )
        )
        b_block, b_exp, b_frac = cfg.get("bias_block_size"), cfg.get("bias_exponent_width"), cfg.get("bias_frac_width")
        if self.bias is not None and b_block is not None and b_exp is not None:
            self.bias.data.copy_(
                mxfp_quantizer(self.bias.data, block_size=b_block, element_exp_bits=b_exp, element_frac_bits=b_frac,
                               block_dim=0)
            )
        return result

    def _pack_weight_for_tensor_cores(self) -> None:
        """Keep the weight's MXFP codes and scales as block-scaled MMA operands next to the fake-quantized
        `weight` (which stays in the state_dict exactly as the reference stores it).  Only when both the weight
        and the activation format fit the block-scaled MMA; otherwise forward multiplies the fake-quantized
        tensors.  The copy is tied to the parameter's version counter: an in-place update of `weight` after
        loading makes forward fall back to the fake-quantized tensors."""
        cfg = self.config
        self._mx_weight_version = None
        for name in ("_mx_w_codes", "_mx_w_scales"):
            if name in self._buffers:
                del self._buffers[name]
        w = self.weight.data
        x_block, x_exp, x_frac = cfg.get("data_in_block_size"), cfg.get("data_in_exponent_width"), cfg.get("data_in_frac_width")
        if not w.is_cuda or x_block is None or x_exp is None or x_frac is None:
            return
        if not (mma_supported(cfg["weight_exponent_width"], cfg["weight_frac_width"], cfg["weight_block_size"], w.shape[1])
                and mma_supported(x_exp, x_frac, x_block, w.shape[1])):
            return
        # MXFP4 weights stay nibble-packed (0.53 bytes per element with the scales); other formats are E4M3 bytes
        op = pack_mx_operand(w, cfg["weight_exponent_width"], cfg["weight_frac_width"],
                             fp4=fp4_supported(cfg["weight_exponent_width"], cfg["weight_frac_width"], w.shape[1]))
        self.register_buffer("_mx_w_codes", op.codes, persistent=False)
        self.register_buffer("_mx_w_scales", op.scales, persistent=False)
        self._mx_weight_version = self.weight._version
        self._mx_weight_key = (self.weight.data_ptr(), tuple(self.weight.shape), self.weight.dtype)

    def _apply(self, fn, recurse=True):
        """Module.to / .cuda move `weight` and the packed copy together: the copy stays valid when only the device
        (and with it the storage pointer) changed, not when the move also changed the dtype."""
        valid = self._buffers.get("_mx_w_codes") is not None and self._packed_weight() is not None
        dtype = self.weight.dtype
        out = super()._apply(fn, recurse)
        if valid and self.weight.dtype == dtype and self._buffers["_mx_w_codes"].device == self.weight.device:
            self._mx_weight_version = self.weight._version
            self._mx_weight_key = (self.weight.data_ptr(), tuple(self.weight.shape), self.weight.dtype)
        return out

    def __deepcopy__(self, memo):
        """copy.deepcopy: the copy's packed weight belongs to the copy's `weight` (new storage, same values)."""
        import copy

        valid = self._buffers.get("_mx_w_codes") is not None and self._packed_weight() is not None
        new = self.__class__.__new__(self.__class__)
        memo[id(self)] = new
        for k, v in self.__dict__.items():
            if k != "_mx_operand":
                new.__dict__[k] = copy.deepcopy(v, memo)
        if valid:
            new._mx_weight_version = new.weight._version
            new._mx_weight_key = (new.weight.data_ptr(), tuple(new.weight.shape), new.weight.dtype)
        return new

    def _operand(self, codes: Tensor, scales: Tensor) -> MXOperand:
        cached = self.__dict__.get("_mx_operand")
        if cached is not None and cached.codes is codes and cached.scales is scales:
            return cached
        fp4 = codes.shape[1] * 2 == self.in_features and codes.shape[1] != self.in_features
        e5m2 = (self.config.get("weight_exponent_width"), self.config.get("weight_frac_width")) == (5, 2)
        op = MXOperand(codes, scales, codes.shape[0], self.in_features, fp4, e5m2)
        self.__dict__["_mx_operand"] = op
        return op

    def _packed_weight(self) -> MXOperand | None:
        """The tensor-core copy of the weight, or None when there is none or `weight` has changed since it was made.
        The copy is tied to the parameter's version counter, storage pointer and shape; an update that bypasses all
        three (writing through `weight.data` in place) needs a call of `_pack_weight_for_tensor_cores()`."""
        if getattr(self, "_dense_dropped", False):
            return self._operand(self._buffers["weight_codes"], self._buffers["weight_scales"])
        codes = self._buffers.get("_mx_w_codes")
        if codes is None or getattr(self, "_mx_weight_version", None) != self.weight._version:
            return None
        if getattr(self, "_mx_weight_key", None) != (self.weight.data_ptr(), tuple(self.weight.shape), self.weight.dtype):
            return None
        if codes.device != self.weight.device:
            return None
        return self._operand(codes, self._buffers["_mx_w_scales"])

    def drop_dense_weight(self) -> None:
        """Weight-only memory saving (not in the reference, whose state_dict keeps the fake-quantized tensor in the
        original dtype): keep only the tensor-core operands -- one byte per element (half a byte for MXFP4 weights,
        which are stored nibble-packed) plus one scale byte per 32 -- and release the bf16 / fp32 `weight`.  The state_dict then carries `weight_codes` and `weight_scales`
        (which `load_state_dict` accepts) and an empty `weight`; forward needs CUDA inputs of the original dtype."""
        packed = self._packed_weight()
        if packed is None:
            raise RuntimeError("drop_dense_weight: this layer has no tensor-core operands (load a weight on a CUDA "
                               "device with weight and data_in formats that fit the block-scaled MMA first)")
        self._weight_dtype = self.weight.dtype
        for name in ("_mx_w_codes", "_mx_w_scales"):
            self._buffers.pop(name, None)
        self.register_buffer("weight_codes", packed.codes, persistent=True)
        self.register_buffer("weight_scales", packed.scales, persistent=True)
        self.weight = torch.nn.Parameter(torch.empty(0, dtype=self._weight_dtype, device=packed.codes.device),
                                         requires_grad=False)
        self._dense_dropped = True

    @torch.no_grad()
    def forward(self, x: Tensor) -> Tensor:
        if self.bypass:
            return linear_forward(x, self.weight, self.bias, self.output_dtype)
        cfg = self.config
        x_block, x_exp, x_frac = cfg.get("data_in_block_size"), cfg.get("data_in_exponent_width"), cfg.get("data_in_frac_width")
        if getattr(self, "_dense_dropped", False) and not (x.is_cuda and x.dtype == self.weight.dtype):
            raise RuntimeError("this layer keeps only packed weights: inputs must be CUDA tensors of dtype "
                               f"{self.weight.dtype}")
        if x_block is not None and x_exp is not None:
            packed = self._packed_weight()
            if packed is not None and x.is_cuda and x.dtype == self.weight.dtype:
                # activations are quantized straight into tensor-core operands; same codes and scales as
                # mxfp_quantizer, multiplied by tcgen05 block-scaled MMAs
                return mx_linear(x, packed, self.bias, x_exp, x_frac, self.output_dtype)
            x = mxfp_quantizer(x, block_size=x_block, element_exp_bits=x_exp, element_frac_bits=x_frac, block_dim=-1)
        return linear_forward(x, self.weight, self.bias, self.output_dtype)


    # ---- sharing one activation quantization between sibling projections (q/k/v, gate/up) ----------------------
    def _input_format(self):
        cfg = self.config
        return ("mxfp", cfg.get("data_in_block_size"), cfg.get("data_in_exponent_width"), cfg.get("data_in_frac_width"))

    def _uses_packed_path(self, x: Tensor) -> bool:
        _, x_block, x_exp, _ = self._input_format()
        return (not self.bypass and x_block is not None and x_exp is not None and self._packed_weight() is not None
                and x.is_cuda and x.dtype == self.weight.dtype)

    @torch.no_grad()
    def quantize_input(self, x: Tensor):
        """The quantized form of x that `forward_quantized` takes: tensor-core operands when this layer multiplies
        block-scaled codes, else the fake-quantized tensor (or x itself for a layer without input quantization)."""
        _, x_block, x_exp, x_frac = self._input_format()
        if self._uses_packed_path(x):
            x2 = x.reshape(-1, x.shape[-1])
            return pack_mx_operand(x2, x_exp, x_frac), x.shape[:-1]
        if self.bypass or x_block is None or x_exp is None:
            return x, None
        return mxfp_quantizer(x, block_size=x_block, element_exp_bits=x_exp, element_frac_bits=x_frac, block_dim=-1), None

    @torch.no_grad()
    def forward_quantized(self, quantized) -> Tensor:
        """forward(x) for an x that went through `quantize_input` of a layer with the same input format."""
        xq, lead = quantized
        if isinstance(xq, MXOperand):
            out_dtype = self.output_dtype or self.weight.dtype
            return mx_gemm(xq, self._packed_weight(), self.bias, out_dtype, static_b=True).reshape(*lead, self.out_features)
        return linear_forward(xq, self.weight, self.bias, self.output_dtype,
                              fp32_exact=not self.bypass and getattr(self, "_weight_quantized", False))

    @torch.no_grad()
    def forward_gated(self, gate: Tensor, up: Tensor) -> Tensor:
        """forward(silu(gate) * up) -- the down projection of a gated MLP -- without materialising the product: one
        kernel reads gate and up and writes the quantized tensor-core operand.  Falls back to the plain forward where
        the block-scaled path does not apply."""
        _, x_block, x_exp, x_frac = self._input_format()
        if gate.dtype == torch.bfloat16 and self._uses_packed_path(gate) and x_exp <= 4:
            return mx_gated_linear(gate, up, self._packed_weight(), self.bias, x_exp, x_frac, self.output_dtype)
        return self.forward(torch.nn.functional.silu(gate) * up)


class LinearMXInt(_LinearBase):
    """Linear with MXINT weight (quantized at load time) and MXINT activations.  Inference only."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None, config=None):
        super().__init__(in_features, out_features, bias, device, dtype)
        assert config is not None, "config is None!"
        self.config = config
        self.bypass = config.get("bypass", False)
        self.gptq = config.get("gptq", False)
        self.clip_search = config.get("clip_search", False)

    def load_state_dict(self, state_dict, strict=True, assign=False):
        result = super().load_state_dict(state_dict, strict=strict, assign=assign)
        if self.bypass or self.gptq:
            return result
        cfg = self.config
        self._weight_quantized = True  # from here on `weight` holds MX values: exact on the tf32 tensor cores
        self.weight.data.copy_(
            mxint_quantizer(self.weight.data, block_size=cfg["weight_block_size"], element_bits=cfg["weight_width"],
                            block_dim=1, quantile_search=self.clip_search)
        )
        b_block, b_bits = cfg.get("bias_block_size"), cfg.get("bias_width")
        if self.bias is not None and b_block is not None and b_bits is not None:
            self.bias.data.copy_(
                mxint_quantizer(self.bias.data, block_size=b_block, element_bits=b_bits, block_dim=0,
                                quantile_search=self.clip_search)
            )
        return result

    @torch.no_grad()
    def forward(self, x: Tensor) -> Tensor:
        if self.bypass:
            return linear_forward(x, self.weight, self.bias, self.output_dtype)
        cfg = self.config
        x_block, x_bits = cfg.get("data_in_block_size"), cfg.get("data_in_width")
        if x_block is not None and x_bits is not None:
            x = mxint_quantizer(x, block_size=x_block, element_bits=x_bits, block_dim=-1)
            return linear_forward(x, self.weight, self.bias, self.output_dtype,
                                  fp32_exact=getattr(self, "_weight_quantized", False))
        return linear_forward(x, self.weight, self.bias, self.output_dtype)


    def _input_format(self):
        cfg = self.config
        return ("mxint", cfg.get("data_in_block_size"), cfg.get("data_in_width"))

    @torch.no_grad()
    def quantize_input(self, x: Tensor):
        _, x_block, x_bits = self._input_format()
        if self.bypass or x_block is None or x_bits is None:
            return x, None
        return mxint_quantizer(x, block_size=x_block, element_bits=x_bits, block_dim=-1), None

    @torch.no_grad()
    def forward_quantized(self, quantized) -> Tensor:
        return linear_forward(quantized[0], self.weight, self.bias, self.output_dtype,
                              fp32_exact=not self.bypass and getattr(self, "_weight_quantized", False))


def forward_siblings(layers, x: Tensor) -> list[Tensor]:
    """[layer(x) for layer in layers] for projections that read the same input (q/k/v; gate/up), quantizing x once
    when the layers are of one class, share the input format and take the same kind of quantized operand.  The
    reference quantizes x inside every forward (chop/nn/quantized/modules/linear.py:877-890, :956-969); the values
    are the same, only the repeated work is dropped."""
    first = layers[0]
    shareable = all(hasattr(m, "quantize_input") and type(m) is type(first) and not m.bypass
                    and m._input_format() == first._input_format() for m in layers)
    if shareable and isinstance(first, LinearMXFP):
        shareable = len({m._uses_packed_path(x) for m in layers}) == 1
    if not shareable:
        return [m(x) for m in layers]
    q = first.quantize_input(x)
    return [m.forward_quantized(q) for m in layers]


def linearBlockFP(x: Tensor, weight: Tensor, bias: Tensor = None, config: dict = None, out_dtype=None) -> Tensor:
    """Quantize x, weight and bias with block floating point on every call, then multiply
    (chop/nn/quantized/functional/linear.py:220-278)."""
    w_quantizer = partial(
        block_fp_quantizer,
        width=config["weight_width"],
        exponent_width=config["weight_exponent_width"],
        exponent_bias=config["weight_exponent_bias"],
        block_size=config["weight_block_size"],
        skip_first_dim=False,
    )
    x_quantizer = partial(
        block_fp_quantizer,
        width=config["data_in_width"],
        exponent_width=config["data_in_exponent_width"],
        exponent_bias=config["data_in_exponent_bias"],
        block_size=config["data_in_block_size"],
        skip_first_dim=config.get("data_in_skip_first_dim", True),
    )
    b_quantizer = partial(
        block_fp_quantizer,
        width=config["bias_width"],
        exponent_width=config["bias_exponent_width"],
        exponent_bias=config["bias_exponent_bias"],
        block_size=config["bias_block_size"],
        skip_first_dim=False,
    )
    x = x_quantizer(x)
    weight = w_quantizer(weight)
    bias = b_quantizer(bias) if bias is not None else None
    # width counts the sign: up to 12 means at most 11 significant bits, which tf32 multiplies exactly
    return linear_forward(x, weight, bias, out_dtype,
                          fp32_exact=config["weight_width"] <= 12 and config["data_in_width"] <= 12)


class LinearBlockFP(_LinearBase):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None, config=None):
        super().__init__(in_features, out_features, bias, device, dtype)
        assert config is not None, "config is None!"
        self.config = config
        self.bypass = config.get("bypass", False)

    def forward(self, x: Tensor) -> Tensor:
        if self.bypass:
            return linear_forward(x, self.weight, self.bias, self.output_dtype)
        return linearBlockFP(x, self.weight, self.bias, self.config, self.output_dtype)


class _EmbeddingMX(torch.nn.Embedding):
    """Embedding whose weight is MX-quantized along the embedding dimension at forward time
    (chop/nn/quantized/modules/embedding.py:9-71).  The reference quantizes the whole table on every call and then
    looks the rows up; blocks run along a row, so when a row is a whole number of blocks the quantized rows do not
    depend on one another and this class looks up first and quantizes only the rows that were asked for -- the same
    values for a fraction of the work.  Tables whose rows are not whole blocks (flattened blocks straddle rows) and
    lookups with `max_norm` (which rewrites the table) take the reference's order."""

    def __init__(self, num_embeddings, embedding_dim, config=None, **kwargs):
        super().__init__(num_embeddings, embedding_dim, **kwargs)
        self.config = config or {}
        self.bypass = self.config.get("bypass", False)

    def _quantize(self, rows: Tensor) -> Tensor:
        raise NotImplementedError

    @torch.no_grad()
    def forward(self, input: Tensor) -> Tensor:
        if self.bypass:
            return super().forward(input)
        args = (self.padding_idx, self.max_norm, self.norm_type, self.scale_grad_by_freq, self.sparse)
        if self.max_norm is not None or self.embedding_dim % self.config["weight_block_size"]:
            return torch.nn.functional.embedding(input, self._quantize(self.weight), *args)
        rows = torch.nn.functional.embedding(input, self.weight, *args)
        return self._quantize(rows.reshape(-1, self.embedding_dim)).reshape(rows.shape)


class EmbeddingMXFP(_EmbeddingMX):
    def _quantize(self, rows: Tensor) -> Tensor:
        cfg = self.config
        return mxfp_quantizer(rows, block_size=cfg["weight_block_size"], element_exp_bits=cfg["weight_exponent_width"],
                              element_frac_bits=cfg["weight_frac_width"], block_dim=1)


class EmbeddingMXInt(_EmbeddingMX):
    def _quantize(self, rows: Tensor) -> Tensor:
        cfg = self.config
        return mxint_quantizer(rows, block_size=cfg["weight_block_size"], element_bits=cfg["weight_width"], block_dim=1)


class RMSNormMinifloat(torch.nn.Module):
    """RMSNorm with minifloat-quantized input and weight, quantized at forward time: the arithmetic of
    LlamaRMSNormMinifloat (chop/nn/quantized/modules/llama/rms_norm.py:34-84) without the dependency on a
    `transformers` model config.  `RMSNormMinifloat(hidden_size, eps, q_config)`, or `from_config(config, layer_idx,
    q_config)` with the reference's constructor arguments."""

    def __init__(self, hidden_size: int | None = None, eps: float = 1e-6, q_config: dict | None = None, layer_idx=None,
                 device=None, dtype=None, config=None):
        super().__init__()
        if config is not None:  # the call of the quantize pass: (config=..., layer_idx=..., q_config=...)
            hidden_size, eps = config.hidden_size, config.rms_norm_eps
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.variance_epsilon = eps
        self.layer_idx = layer_idx
        self.q_config = q_config or {}
        self.bypass = self.q_config.get("bypass", False)
        self.weight_bypass = self.q_config.get("weight_bypass", False)
        self.data_in_bypass = self.q_config.get("data_in_bypass", False)

    @classmethod
    def from_config(cls, config=None, layer_idx=None, q_config: dict | None = None):
        return cls(config.hidden_size, config.rms_norm_eps, q_config, layer_idx)

    def _meta(self, prefix: str):
        from .quantizers import MinifloatMeta

        q = self.q_config
        return MinifloatMeta(exp_bits=q[prefix + "_exponent_width"], frac_bits=q[prefix + "_frac_width"],
                             is_finite=q.get(prefix + "_is_finite", True), round_mode=q.get(prefix + "_round_mode", "rn"))

    def forward(self, hidden_states: Tensor) -> Tensor:
        from .quantizers import minifloat_quantizer_sim

        input_dtype = hidden_states.dtype
        if not self.bypass and not self.data_in_bypass:
            hidden_states = minifloat_quantizer_sim(hidden_states, self._meta("data_in"))
        hidden_states = hidden_states.to(torch.float32)
        variance = hidden_states.pow(2).mean(-1, keepdim=True)
        hidden_states = hidden_states * torch.rsqrt(variance + self.variance_epsilon)
        weight = self.weight
        if not self.bypass and not self.weight_bypass:
            weight = minifloat_quantizer_sim(self.weight.data, self._meta("weight"))
        return weight * hidden_states.to(input_dtype)


# entries of chop.nn.quantized.modules.quantized_module_map (nn/quantized/modules/__init__.py:241-246)
quantized_module_map = {
    "linear_mxfp": LinearMXFP,
    "linear_mxint": LinearMXInt,
    "linear_block_fp": LinearBlockFP,
}
# entry of chop.nn.quantized.functional.quantized_func_map (nn/quantized/functional/__init__.py:287)
quantized_func_map = {
    "linear_block_fp": linearBlockFP,
}
