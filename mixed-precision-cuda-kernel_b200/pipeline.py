"""Model-level steps around the quantized linear: cherry selection, whole-model packing on the
GPU, and the reference's checkpoint format.

Reference: estimate_impact.py:55-89 (running mean of squared gradients per input channel, top
`num_cherries` channels), utils.py:66-101 (`make_quant`, `pack_model`), utils.py:104-149
(`save_quantized` / `from_quantized`: one `torch.save` of the state dict named
`pytorch_model-{w_bits}bit-{group_size}g.bin` beside the configuration) and pack.py:21-27 of the
reference project.  The arithmetic of packing itself is the GPU `pack` of `QuantLinear`
(byte-identical to the reference's); what this module adds is the walking of a module tree, the
selection, and the file layout, so that a checkpoint written by the reference loads here and
vice versa.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch
import torch.nn as nn

from .cherry_linear import QuantLinear as QuantLinearForTraining
from .qlinear import QuantLinear


# ---------------------------------------------------------------------------------- cherry selection
class ImpactAccumulator:
    """Running mean over batches of the squared gradient per input channel
    (estimate_impact.py:66-80): `update(name, grad)` once per batch and weight."""

    def __init__(self):
        self.h: Dict[str, torch.Tensor] = {}
        self.batches: Dict[str, int] = {}

    @torch.no_grad()
    def update(self, name: str, grad: torch.Tensor):
        if grad.ndim < 2:
            return
        h = (grad ** 2).mean(dim=tuple(range(grad.ndim - 1)))
        nb = self.batches.get(name, 0)
        if name not in self.h:
            self.h[name] = torch.zeros(grad.shape[-1], dtype=grad.dtype, device=grad.device)
        else:
            self.h[name] *= nb / (nb + 1)
        self.h[name] += h / (nb + 1)
        self.batches[name] = nb + 1

    def select(self, cherry_fraction: float) -> Dict[str, torch.Tensor]:
        return {k: select_cherries(v, cherry_fraction) for k, v in self.h.items()}


def num_cherries(in_features: int, cherry_fraction: float) -> int:
    return math.ceil(in_features * cherry_fraction) // 8 * 8


@torch.no_grad()
def select_cherries(impact: torch.Tensor, cherry_fraction: float) -> torch.Tensor:
    """Indices of the `num_cherries` channels of largest impact, most important first, int32 on the
    CPU (estimate_impact.py:85-87).  One top-k on whatever device holds the vector; ties are
    broken towards the lower index (the reference's argsort leaves them unspecified)."""
    n = num_cherries(impact.shape[-1], cherry_fraction)
    order = torch.argsort(impact, descending=True, dim=-1, stable=True)[..., :n]
    return order.to(dtype=torch.int32, device="cpu")


# ---------------------------------------------------------------------------------- whole-model packing
def make_quant(module: nn.Module, name: str = "") -> Dict[str, nn.Module]:
    """Replaces every training-side quantized linear below `module` by an (empty) packed
    `QuantLinear` and returns the replaced layers by qualified name (utils.py:66-93)."""
    linears: Dict[str, nn.Module] = {}
    if isinstance(module, QuantLinearForTraining):
        return linears
    for attr, sub in list(module.named_children()):
        if isinstance(sub, QuantLinearForTraining):
            qual = f"{name}.{attr}" if name else attr
            linears[qual] = sub
            new = QuantLinear(sub.w_bits, sub.group_size, sub.quantizer, sub.cherry_fraction, sub.in_features,
                              sub.out_features, sub.bias is not None)
            dev = sub.weight.device
            setattr(module, attr, new.to(dev))
    for attr, child in module.named_children():
        linears.update(make_quant(child, f"{name}.{attr}" if name else attr))
    return linears


def pack_model(model: nn.Module, device=None) -> int:
    """`make_quant` + `QuantLinear.pack` for every quantized linear (utils.py:96-101), each layer
    packed by the GPU kernels; returns the number of layers packed.  Layers living on the CPU are
    packed through `device` (default: the current CUDA device) and their buffers stay there."""
    linears = make_quant(model)
    count = 0
    for qual, mod in model.named_modules():
        if isinstance(mod, QuantLinear) and qual in linears:
            src = linears[qual]
            if not src.weight.is_cuda:
                if not torch.cuda.is_available():
                    raise RuntimeError("pack_model needs a CUDA device (there is no CPU path)")
                mod.to(device or torch.device("cuda"))
            mod.pack(src)
            count += 1
    return count


# ---------------------------------------------------------------------------------- checkpoint format
def checkpoint_name(w_bits: int, group_size: int) -> str:
    return f"pytorch_model-{w_bits}bit-{group_size}g.bin"


def save_quantized(model: nn.Module, save_dir: str, config: dict | None = None) -> str:
    """Writes the state dict the way utils.save_quantized does (utils.py:104-121): CPU tensors, one
    file named after the first quantized linear's bits and group size, plus `config.json`."""
    w_bits = group_size = None
    for m in model.modules():
        if isinstance(m, QuantLinear):
            w_bits, group_size = m.w_bits, m.group_size
            break
    if w_bits is None:
        raise ValueError("the model holds no packed QuantLinear")
    os.makedirs(save_dir, exist_ok=True)
    path = os.path.join(save_dir, checkpoint_name(w_bits, group_size))
    torch.save({k: v.detach().cpu() for k, v in model.state_dict().items()}, path)
    cfg = dict(config or {})
    cfg.update({"w_bits": w_bits, "group_size": group_size})
    with open(os.path.join(save_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return path


def load_quantized_state(load_dir: str):
    """(state dict on the CPU, config dict) of a checkpoint in the reference's layout
    (utils.py:124-149 locates the file from `w_bits` and `group_size` of the configuration)."""
    with open(os.path.join(load_dir, "config.json")) as f:
        cfg = json.load(f)
    path = os.path.join(load_dir, checkpoint_name(cfg["w_bits"], cfg["group_size"]))
    state = torch.load(path, map_location="cpu", weights_only=True)
    return state, cfg


# Names of the quantized projections inside one decoder layer of the reference's LLaMA
# (llama/modeling_llama_quant.py:221-227, 299-308) in the order of CherryDecoder.PROJ.
HF_PROJ = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
           "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}
BUFFERS = ("qweight", "scales", "cherry_weight", "cherry_indices")


def decoder_state_dict(dec) -> Dict[str, torch.Tensor]:
    """State dict of a `CherryDecoder` under the reference model's key names."""
    sd = {"model.embed_tokens.weight": dec.embed, "model.norm.weight": dec.final_norm, "lm_head.weight": dec.lm_head}
    for i, lay in enumerate(dec.layers):
        base = f"model.layers.{i}."
        sd[base + "input_layernorm.weight"] = lay["norm1"]
        sd[base + "post_attention_layernorm.weight"] = lay["norm2"]
        for short, hf in HF_PROJ.items():
            for b in BUFFERS:
                sd[f"{base}{hf}.{b}"] = getattr(lay[short], b)
    return {k: v.detach().cpu() for k, v in sd.items()}


@torch.no_grad()
def load_decoder_state_dict(dec, state: Dict[str, torch.Tensor]):
    """Loads a state dict with the reference model's key names into a `CherryDecoder` of matching
    configuration (buffers are copied to the decoder's device; re-packed copies are rebuilt on use)."""
    def put(dst: torch.Tensor, key: str):
        src = state[key]
        if src.shape != dst.shape or src.dtype != dst.dtype:
            raise ValueError(f"{key}: expected {tuple(dst.shape)} {dst.dtype}, found {tuple(src.shape)} {src.dtype}")
        dst.copy_(src)
    put(dec.embed, "model.embed_tokens.weight")
    put(dec.final_norm, "model.norm.weight")
    put(dec.lm_head, "lm_head.weight")
    for i, lay in enumerate(dec.layers):
        base = f"model.layers.{i}."
        put(lay["norm1"], base + "input_layernorm.weight")
        put(lay["norm2"], base + "post_attention_layernorm.weight")
        for short, hf in HF_PROJ.items():
            ql = lay[short]
            for b in BUFFERS:
                src = state[f"{base}{hf}.{b}"]
                cur = getattr(ql, b)
                if src.shape != cur.shape or src.dtype != cur.dtype:
                    raise ValueError(f"{base}{hf}.{b}: expected {tuple(cur.shape)} {cur.dtype}, found "
                                     f"{tuple(src.shape)} {src.dtype}")
                setattr(ql, b, src.to(cur.device).contiguous())
            ql._drop_copies()
            if dec.dense:
                ql.dense_weight = ql.unpack()
    dec.graph = None
