"""GPTQ weight optimisation with an MX inner quantizer (chop/passes/module/transforms/gptq/).

Calibration-time pass, not part of the inference path: the weights of every Linear in a decoder layer are quantized
column block by column block, and the quantization error of each block, weighted by the inverse Hessian of the layer's
inputs, is pushed into the columns that are still to come.  What the reference spends its time on runs on this
package's kernels:

* the Hessian 2/n * X^T X and the rank-`block` error updates go through the package's GEMM (fp32 operands split into
  tf32-exact parts, so products keep fp32-level accuracy);
* the inner quantizer, with or without the clipping search, is one kernel launch per column block
  (`mxfp_quantizer_sim` / `mxint_quantizer_sim` on a contiguous [rows, block] slice).

The two Cholesky factorisations per layer stay with `torch.linalg` (a dense solver library call, once per layer).

Same names and arguments as the reference: `GPTQ(layer).add_batch / fasterquant / free` (gptq.py:17-128),
`quantize_tensor` (quantize_dispatch.py:34-82), `find_qlayers` (utils.py:9-20), `run_gptq(network, gptq_config)`
(run.py:21-232) and the per-layer checkpoints of checkpoint.py:9-135.  The one difference in `run_gptq`: calibration
token batches are passed in (`gptq_config["calibration_data"]` or the `dataloader` argument) because downloading a
dataset is outside this package.
"""

from __future__ import annotations

import json
import logging
import math
import os
from pathlib import Path

import torch
from torch import Tensor, nn

from .gemm import linear_forward
from .quantizers import MXFPMeta, MXIntMeta, mxfp_quantizer_sim, mxint_quantizer_sim

logger = logging.getLogger(__name__)


def quantize_tensor(input: Tensor, block_dim: int, fmt: str, config: dict, quantile_search: bool,
                    act_tensor: Tensor | None = None, dtype: torch.dtype | None = None,
                    cali_batch_size: int = 32) -> Tensor:
    """Fake-quantize `input` with the MX format `fmt` ("mxfp" or "mxint") described by a weight config dict
    (quantize_dispatch.py:34-82)."""
    if fmt == "mxfp":
        meta = MXFPMeta(block_size=config["weight_block_size"], scale_exp_bits=8,
                        element_exp_bits=config["weight_exponent_width"], element_frac_bits=config["weight_frac_width"],
                        element_is_finite=True, round_mode="rn")
        return mxfp_quantizer_sim(input, block_dim=block_dim, mxfp_meta=meta, act_tensor=act_tensor, dtype=dtype,
                                  quantile_search=quantile_search, cali_batch_size=cali_batch_size)
    if fmt == "mxint":
        meta = MXIntMeta(block_size=config["weight_block_size"], scale_bits=8, element_bits=config["weight_width"])
        return mxint_quantizer_sim(input, block_dim=block_dim, mxint_meta=meta, act_tensor=act_tensor, dtype=dtype,
                                   quantile_search=quantile_search, cali_batch_size=cali_batch_size)
    raise ValueError(f"Unsupported GPTQ format: {fmt}. Use 'mxfp' or 'mxint'.")


class GPTQ:
    """Hessian accumulation and the block-wise sweep for one Linear (gptq.py:17-128)."""

    def __init__(self, layer: nn.Linear):
        self.layer = layer
        self.dev = layer.weight.device
        if self.dev.type != "cuda":
            raise RuntimeError("GPTQ: the layer must live on a CUDA device (there is no CPU path)")
        self.rows, self.columns = layer.weight.shape
        self.H = torch.zeros((self.columns, self.columns), device=self.dev, dtype=torch.float32)
        self.nsamples = 0

    @torch.no_grad()
    def add_batch(self, inp: Tensor, out: Tensor | None = None) -> None:
        """H <- running mean of 2 * X^T X over the samples seen so far (gptq.py:28-38); a 2-D input is one sample."""
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        batch = inp.shape[0]
        x = inp.reshape(-1, inp.shape[-1])
        self.H *= self.nsamples / (self.nsamples + batch)
        self.nsamples += batch
        xt = (math.sqrt(2 / self.nsamples) * x.float()).t().contiguous()  # [columns, tokens]
        self.H += linear_forward(xt, xt, None, torch.float32)

    @torch.no_grad()
    def fasterquant(self, activation: Tensor | None, fmt: str, weight_config: dict, percdamp: float = 0.01,
                    cali_batch_size: int = 32, layer_name: str | None = None, quant_search: bool = True) -> Tensor:
        """The quantized weight [rows, columns] (gptq.py:40-123).  `activation` [batch, seq, columns] switches the
        inner clipping search to its activation-weighted error."""
        W = self.layer.weight.data.clone()
        H = self.H
        del self.H
        dead = torch.diag(H) == 0
        H[dead, dead] = 1
        W[:, dead] = 0
        idx = torch.arange(self.columns, device=self.dev)
        H[idx, idx] += percdamp * torch.mean(torch.diag(H))
        H = torch.linalg.cholesky(H)
        H = torch.cholesky_inverse(H)
        Hinv = torch.linalg.cholesky(H, upper=True)
        del H
        diag = torch.diag(Hinv).clone()
        # the update multiplies by rows c0:c1 of Hinv right of the block: keep the transpose once so that every step
        # hands the GEMM a [columns - c1, block] weight-like operand
        hinv_t = Hinv.t().contiguous()
        Q = torch.zeros_like(W)
        block = weight_config["weight_block_size"]
        for c0 in range(0, self.columns, block):
            c1 = min(c0 + block, self.columns)
            W1 = W[:, c0:c1].clone()
            act1 = activation[:, :, c0:c1].clone() if activation is not None else None
            Q1 = quantize_tensor(W1, block_dim=1, fmt=fmt, config=weight_config, quantile_search=quant_search,
                                 act_tensor=act1, cali_batch_size=cali_batch_size)
            Q[:, c0:c1] = Q1
            if c1 < self.columns:
                err = (W1 - Q1).float() / diag[c0:c1].unsqueeze(0)
                W[:, c1:] -= linear_forward(err, hinv_t[c1:, c0:c1], None, torch.float32)
        return Q

    def free(self) -> None:
        self.H = None
        torch.cuda.empty_cache()


def find_qlayers(module: nn.Module, layers=(nn.Linear,), name: str = "") -> dict[str, nn.Module]:
    """{dotted name: module} of the sub-modules whose type is one of `layers` (utils.py:9-20)."""
    if type(module) in tuple(layers):
        return {name: module}
    found = {}
    for child_name, child in module.named_children():
        found.update(find_qlayers(child, layers, f"{name}.{child_name}" if name else child_name))
    return found


# ----------------------------------------------------------------------------------------------------------------
# per-layer checkpoints (checkpoint.py:9-135): <dir>/<model_name>_layer_<i>.safetensors + _metadata.json
# ----------------------------------------------------------------------------------------------------------------
def save_layer_checkpoint(model, layer_idx: int, checkpoint_dir, model_name: str = "quantized_model") -> None:
    if checkpoint_dir is None:
        return
    from safetensors.torch import save_file

    path = Path(checkpoint_dir)
    path.mkdir(parents=True, exist_ok=True)
    prefix = f"model.layers.{layer_idx}."
    state = {n[len(prefix):]: p.detach().cpu().contiguous() for n, p in model.named_parameters() if n.startswith(prefix)}
    if not state:
        logger.warning("no parameters found for layer %d", layer_idx)
        return
    target = path / f"{model_name}_layer_{layer_idx}.safetensors"
    tmp = path / f".{model_name}_layer_{layer_idx}.tmp"
    save_file(state, str(tmp))
    os.replace(tmp, target)  # a run that dies while saving leaves no half-written checkpoint to resume from
    meta = {"layer_idx": layer_idx, "total_layers": len(model.model.layers), "checkpoint_file": str(target),
            "model_name": model_name, "num_parameters": len(state), "parameter_names": list(state)}
    with open(path / f"{model_name}_layer_{layer_idx}_metadata.json", "w") as fh:
        json.dump(meta, fh, indent=2)


def detect_quantized_layers(checkpoint_dir, model_name: str = "quantized_model") -> dict[int, str]:
    if checkpoint_dir is None or not os.path.exists(checkpoint_dir):
        return {}
    found = {}
    for f in Path(checkpoint_dir).glob(f"{model_name}_layer_*.safetensors"):
        try:
            found[int(f.stem.split("_layer_")[-1])] = str(f)
        except ValueError:
            continue
    return found


def load_layer_checkpoint(model, layer_idx: int, checkpoint_file: str) -> bool:
    from safetensors.torch import load_file

    if not os.path.exists(checkpoint_file):
        return False
    try:
        state = load_file(checkpoint_file)
    except Exception as exc:  # a damaged file ends the resume at this layer
        logger.error("could not read %s: %s", checkpoint_file, exc)
        return False
    model.load_state_dict({f"model.layers.{layer_idx}.{k}": v for k, v in state.items()}, strict=False)
    return True


def auto_load_quantized_layers(model, checkpoint_dir, model_name: str = "quantized_model") -> int:
    """Loads the consecutive run of saved layers starting at 0; returns the index of the last one (-1: none)."""
    found = detect_quantized_layers(checkpoint_dir, model_name)
    last = -1
    for i in sorted(found):
        if i != last + 1 or not load_layer_checkpoint(model, i, found[i]):
            break
        last = i
    return last


# ----------------------------------------------------------------------------------------------------------------
# orchestration over a decoder-only model (run.py:21-232)
# ----------------------------------------------------------------------------------------------------------------
SEQUENTIAL_GROUPS = (
    ("self_attn.k_proj", "self_attn.v_proj", "self_attn.q_proj"),
    ("self_attn.o_proj",),
    ("mlp.up_proj", "mlp.gate_proj"),
    ("mlp.down_proj",),
)


class _FirstLayerReached(Exception):
    pass


@torch.no_grad()
def run_gptq(network, gptq_config: dict, dataloader=None):
    """GPTQ over every nn.Linear of `network.model.layers`, written back in place (run.py:21-232).

    gptq_config keys as in the reference: device, nsamples, format, weight_config, quantile_search, clip_search_y,
    cali_batch_size, checkpoint_dir, max_layers; plus calibration_data: a list of token-id tensors [1, seqlen]
    (or of (ids, ...) tuples, as the reference's loaders return), also accepted as the `dataloader` argument."""
    dev = torch.device(gptq_config.get("device", "cuda:0"))
    fmt = gptq_config["format"]
    weight_config = gptq_config["weight_config"]
    quantile_search = gptq_config.get("quantile_search", True)
    clip_search_y = gptq_config.get("clip_search_y", False)
    cali_batch_size = gptq_config.get("cali_batch_size", 32)
    checkpoint_dir = gptq_config.get("checkpoint_dir")
    max_layers = gptq_config.get("max_layers")
    data = dataloader if dataloader is not None else gptq_config.get("calibration_data")
    if data is None:
        raise ValueError("run_gptq: pass calibration token batches (gptq_config['calibration_data'] or dataloader=)")
    data = [b[0] if isinstance(b, (tuple, list)) else b for b in data]
    nsamples = min(gptq_config.get("nsamples", len(data)), len(data))
    data = data[:nsamples]

    layers = network.model.layers
    start = 0
    if checkpoint_dir is not None:
        start = auto_load_quantized_layers(network, checkpoint_dir) + 1
        if start == len(layers):
            logger.info("all layers already quantized")
            return network
    use_cache = network.config.use_cache
    network.config.use_cache = False

    # inputs of the first decoder layer, and the keyword arguments every layer is called with
    caught: list[Tensor] = []
    call_kwargs: dict = {}

    def catch(_module, args, kwargs):
        caught.append(args[0] if args else kwargs["hidden_states"])
        call_kwargs.update({k: v for k, v in kwargs.items() if k != "hidden_states"})
        raise _FirstLayerReached

    network.to(dev)
    handle = layers[0].register_forward_pre_hook(catch, with_kwargs=True)
    try:
        for ids in data:
            try:
                network(ids.to(dev))
            except _FirstLayerReached:
                pass
    finally:
        handle.remove()
    inps = [t.detach() for t in caught]

    def run_layer(layer, x):
        out = layer(x, **call_kwargs)
        return out[0] if isinstance(out, (tuple, list)) else out

    # layers loaded from checkpoints still have to produce the inputs of the first layer to be quantized
    for i in range(start):
        inps = [run_layer(layers[i], x) for x in inps]
    end = len(layers) if max_layers is None else min(start + max_layers, len(layers))
    for i in range(start, end):
        layer = layers[i]
        full = find_qlayers(layer, layers=[nn.Linear])
        for names in SEQUENTIAL_GROUPS:
            subset = {n: full[n] for n in names if n in full}
            if not subset:
                continue
            solvers = {n: GPTQ(m) for n, m in subset.items()}
            pre_act: list[Tensor] = []
            hooks = [m.register_forward_hook(lambda _m, inp, _out, n=n: solvers[n].add_batch(inp[0].data))
                     for n, m in subset.items()]
            last = subset[list(subset)[-1]]
            hooks.append(last.register_forward_pre_hook(lambda _m, inp: pre_act.append(inp[0])))
            for x in inps:
                run_layer(layer, x)
            for h in hooks:
                h.remove()
            activation = torch.cat(pre_act, dim=0) if clip_search_y else None
            for n, solver in solvers.items():
                q = solver.fasterquant(activation=activation, fmt=fmt, weight_config=weight_config, percdamp=0.01,
                                       cali_batch_size=cali_batch_size, layer_name=f"layers{i}.{n}",
                                       quant_search=quantile_search)
                assert q.shape == solver.layer.weight.shape
                solver.layer.weight.data.copy_(q)
                solver.free()
        inps = [run_layer(layer, x) for x in inps]  # the next layer calibrates on the quantized layer's outputs
        if checkpoint_dir is not None:
            save_layer_checkpoint(network, i, checkpoint_dir)
    network.config.use_cache = use_cache
    return network
