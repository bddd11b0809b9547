"""Training-side / fake-quant CherryQ linear (reference: llama/cherry_linear.py:12-140).

An nn.Linear whose weight is fake-quantised on the fly: a registered set of input
columns ("cherries") stays in full precision, the remaining columns are compacted,
split into groups and passed through FullSymQuantizer.transform.  `pack()` of the
inference layer reads `weight`, `cherry_indices`, `group_size`, `w_bits` and
`_get_scaling_factors` from this class.  Only the CherryQ 3-/4-bit path of the
reference is kept (5..15-bit and the naive-QAT branches are not).
"""
import math

import torch
import torch.nn as nn

from .quantizer import FullSymQuantizer


class QuantLinear(nn.Linear):
    def __init__(self, *args, bias=False, w_bits=16, weight_layerwise=False, group_size=-1,
                 cherryq=False, cherry_fraction=1 / 256):
        super().__init__(*args, bias=bias)
        self.w_bits = w_bits
        self.weight_layerwise = weight_layerwise
        self.group_size = group_size
        self.cherryq = cherryq
        self.cherry_fraction = cherry_fraction
        if 1 < self.w_bits < 16:
            if self.w_bits > 4:
                raise NotImplementedError("only 2..4-bit FullSymQuantizer layers are supported")
            if self.cherryq:
                self.num_cherries = math.ceil(self.weight.shape[-1] * cherry_fraction) // 8 * 8
                self.register_buffer("cherry_indices", -torch.ones(self.num_cherries, dtype=torch.int32))
                self.cherry_indices_registered = False
            self.quantizer = FullSymQuantizer
            self.dequantized = False

    def register_cherry_indices(self, cherry_indices):
        assert cherry_indices.shape[-1] >= self.cherry_indices.shape[-1], "The passed indices are invalid."
        self.cherry_indices = cherry_indices.to(dtype=torch.int32, device=self.weight.device)
        self.cherry_indices_registered = True

    def _expand_scaling_factors(self, s, weight):
        if s.ndimension() == 0 or s.shape[-1] == 1:
            return s.expand_as(weight)
        return s.repeat_interleave(repeats=self.group_size, dim=-1)[:, :weight.shape[-1]]

    def _get_scaling_factors(self, weight):
        out = []
        for i in range(0, weight.shape[-1], self.group_size):
            out.append(self.quantizer.get_scaling_factor(weight[:, i:i + self.group_size], None, self.w_bits,
                                                         self.weight_layerwise))
        return torch.cat(out, dim=-1)

    def _adjust_weight(self, weight, ste=True):
        assert not self.training or self.cherry_indices_registered, "`cherry_indices` is not registered yet."
        cherry = self.cherry_indices.long()
        quant_idx = torch.ones(weight.shape[1], dtype=torch.bool, device=weight.device).scatter(-1, cherry, 0)
        quant_idx = quant_idx.nonzero().squeeze(1)
        qw = weight.detach().index_select(-1, quant_idx)
        s = self._expand_scaling_factors(self._get_scaling_factors(qw), qw)
        qw = self.quantizer.transform(qw, s, self.w_bits)
        real = weight.detach().clone()
        real[..., quant_idx] = qw
        if ste:
            real = real - weight.detach() + weight
        return real

    @torch.inference_mode()
    def prepare_weight_for_inference(self, weight):
        assert not self.training and not self.dequantized
        assert (self.cherry_indices >= 0).all(), "`cherry_indices` is invalid."
        self.weight.data.copy_(self._adjust_weight(weight, ste=False))
        self.dequantized = True
        return self.weight

    def quant_forward(self, input_):
        weight = self.weight
        if 1 < self.w_bits < 16:
            if not self.cherryq:
                raise NotImplementedError("only the CherryQ path is implemented")
            if self.training:
                weight = self._adjust_weight(weight)
            elif not self.dequantized:
                weight = self.prepare_weight_for_inference(weight)
        out = nn.functional.linear(input_, weight)
        if self.bias is not None:
            out += self.bias
        return out

    def forward(self, x, **kwargs):
        return self.quant_forward(x, **kwargs)
