"""Torch restatement of the reference's CPU "dequantize-then-matmul" path (TEST / BASELINE
INFRASTRUCTURE ONLY: never imported by the product package).

The reference's packed layer, run with `QuantLinear.dmode(layerwise_dequantize=False)`, unpacks
its buffers to a dense fp16 weight with torch ops and calls F.linear
(llama/qlinear.py:120-162 and :183-195 of the reference project).  The reference is Python and
does not travel to the GPU box, so this file restates those two steps with the same torch
operations on the same tensor shapes; it is what `bench.py` times on the host cores as the CPU
baseline.  Parity status: PINNED - tests/test_oracle_golden.py checks it bit-for-bit against the
fixtures frozen from the reference's own unpack().
"""
import torch


def unpack(qweight, scales, cherry_weight, cherry_indices, bits, group_size, in_features):
    """Dense (out, in) fp16 weight from the four packed buffers (llama/qlinear.py:120-162)."""
    q = qweight.t()                                   # (out, rows)
    s = scales.t()                                    # (out, groups)
    n = q.shape[0]
    if bits == 4:
        sh = torch.arange(0, 8, 4, dtype=torch.uint8)[None, None, :]
        w = torch.bitwise_right_shift(q.unsqueeze(2).expand(-1, -1, 2), sh).to(torch.int8)
        w = torch.bitwise_and(w, 15)
    elif bits == 3:
        t = q.reshape(n, q.shape[1] // 3, 3).to(torch.int32)
        word = t[:, :, 0] | (t[:, :, 1] << 8) | (t[:, :, 2] << 16)
        sh = (3 * torch.arange(8, dtype=torch.int32))[None, None, :]
        w = ((word.unsqueeze(2) >> sh) & 7).to(torch.int8)
    else:
        raise NotImplementedError(bits)
    w = w.reshape(n, -1) + (-(2 ** (bits - 1)))
    sfull = s.repeat_interleave(repeats=group_size, dim=1)[:, :w.shape[1]]
    deq = (w.to(sfull.dtype) + 0.5) * sfull           # FullSymQuantizer.dequantize, llama/quantizer.py:160-163
    dense = torch.zeros(n, in_features, dtype=deq.dtype)
    idx = cherry_indices.long()
    mask = torch.ones(in_features, dtype=torch.bool).scatter(-1, idx, 0)
    dense[..., mask.nonzero().squeeze(1)] = deq
    dense[..., idx] = cherry_weight.t()
    return dense


def forward_dequantize_then_matmul(x, qweight, scales, cherry_weight, cherry_indices, bits, group_size):
    """One call of the reference's CPU path: unpack, then F.linear."""
    dense = unpack(qweight, scales, cherry_weight, cherry_indices, bits, group_size, x.shape[-1])
    return torch.nn.functional.linear(x.to(dense.dtype), dense)
