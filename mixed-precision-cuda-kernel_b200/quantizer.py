"""FullSymQuantizer of the reference (llama/quantizer.py:136-170), forward math only.

Signed codes q in [-2^(b-1), 2^(b-1)-1]; dequantised value (q + 0.5) * s; scale
s = (max|w| + 1e-6) / 2^(b-1).  These are plain torch expressions (they run where
the tensors live); the packed kernels implement the same arithmetic on the GPU.
"""
from collections import namedtuple

import torch

iinfo = namedtuple("iinfo", ["min", "max"])


def get_max_input(input, clip_val, layerwise):
    """llama/quantizer.py:10-34 for the 2-D / 3-D case used by linear weights."""
    if clip_val is not None:
        input = torch.clamp(input, clip_val[0], clip_val[1])
    if layerwise:
        return torch.max(torch.abs(input))
    if input.ndimension() <= 3:
        return torch.max(torch.abs(input), dim=-1, keepdim=True)[0].detach()
    raise ValueError(f"Not implemented for shape: {input.shape}")


class Quantizer:
    pass


class FullSymQuantizer(Quantizer):
    """uniform quantization with full range [-(2 ** (num_bits - 1)), 2 ** (num_bits - 1) - 1]"""

    @staticmethod
    def iinfo(num_bits):
        return iinfo(min=-(2 ** (num_bits - 1)), max=2 ** (num_bits - 1) - 1)

    @staticmethod
    def get_scaling_factor(input, clip_val, num_bits, layerwise):
        return (get_max_input(input, clip_val, layerwise) + 1e-6) / (2 ** (num_bits - 1))

    @staticmethod
    def quantize(input, S, num_bits):
        s = S.expand_as(input)
        qmax = 2 ** (num_bits - 1) - 1e-2
        return torch.round(torch.clamp((input / s).float(), -qmax, qmax) - 0.5).to(torch.int32)

    @staticmethod
    def dequantize(rounded_input, S):
        s = S.expand_as(rounded_input)
        return (rounded_input.to(s.dtype) + 0.5) * s

    @staticmethod
    def transform(input, S, num_bits):
        s = S.expand_as(input)
        qmax = 2 ** (num_bits - 1) - 1e-2
        return (torch.round(torch.clamp(input / s, -qmax, qmax) - 0.5) + 0.5) * s
