"""Packed inference CherryQ linear (reference: llama/qlinear.py:13-199).

Same constructor, buffers (`cherry_indices` int16 (C,), `cherry_weight` fp16 (C, N),
`qweight` uint8 (K'/8*bits, N), `scales` fp16 (ceil(K'/G), N), optional `bias`),
`pack()`, `unpack()`, `forward()` and class-level `dmode()` switch as the reference,
so a state dict written by the reference loads into it.  What runs underneath is
different: pack and unpack are GPU kernels, and forward runs on re-packed copies of
the buffers that the module owns (made on first use of the kernel family that needs
them; `release_reference_buffers()` drops the originals afterwards):
  one activation row    row-tile layout, the one-row decode kernel (where the layer fits it)
  2..7 rows             stream layout, the stream matvec
  8 rows or more        the drop-in op's tensor-core GEMM (tile layout, cached by the library)
All of it needs a CUDA device.
"""
import math
from contextlib import contextmanager

import torch
import torch.nn as nn

from . import load_quant_cuda


# No batch beyond this many rows goes to the row-tile decode kernel (four rows per launch, each launch
# reads the weights once); a layer's own limit (RowLayer.preferred_rows) may be lower.  Larger batches
# take the tensor-core GEMM.
ROW_KERNEL_MAX_ROWS = 16


class QuantLinear(nn.Module):
    _layerwise_dequantize = True

    @classmethod
    @contextmanager
    def dmode(cls, layerwise_dequantize=True):
        mode = cls._layerwise_dequantize
        cls._layerwise_dequantize = layerwise_dequantize
        try:
            yield
        finally:
            cls._layerwise_dequantize = mode

    def __init__(self, w_bits, group_size, quantizer, cherry_fraction: float, in_features, out_features,
                 bias=True, **kwargs):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.w_bits = w_bits
        self.group_size = group_size if group_size != -1 else in_features
        self.quantizer = quantizer
        self.cherry_fraction = cherry_fraction
        self.num_cherries = math.ceil(in_features * cherry_fraction) // 8 * 8
        self.num_normal = self.in_features - self.num_cherries
        assert in_features % 8 == 0
        assert out_features % 8 == 0
        self.register_buffer("cherry_indices", torch.zeros(self.num_cherries, dtype=torch.int16))
        self.register_buffer("cherry_weight", torch.zeros((self.num_cherries, out_features), dtype=torch.float16))
        self.register_buffer("qweight", torch.zeros((self.num_normal // 8 * w_bits, out_features), dtype=torch.uint8))
        self.register_buffer("scales", torch.zeros((math.ceil(self.num_normal / self.group_size), out_features),
                                                   dtype=torch.float16))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16))
        else:
            self.bias = None
        self.dequantized = False
        self._prepared = None        # stream layout (PreparedLayer)
        self._row = None             # row-tile layout (RowLayer)
        self._tile = None            # tile layout of the GEMM (TileLayer), only built after a release
        self._row_ok = None          # None = not asked yet
        self._prepared_key = None

    # ------------------------------------------------------------------ pack / unpack
    @torch.inference_mode()
    def pack(self, linear):
        """GPU version of llama/qlinear.py:67-118; `linear` is the training-side layer."""
        qc = load_quant_cuda()
        if linear.bias is not None:
            self.bias = linear.bias.half()
        weight = linear.weight.detach()
        if not weight.is_cuda:
            if not torch.cuda.is_available():
                raise RuntimeError("QuantLinear.pack needs a CUDA device (there is no CPU path)")
            weight = weight.cuda()
        weight = weight.contiguous()
        if weight.dtype not in (torch.float16, torch.float32):
            weight = weight.float()
        idx = linear.cherry_indices.to(device=weight.device, dtype=torch.int32).contiguous()
        gs = linear.group_size if linear.group_size != -1 else self.in_features
        q, s, cw, ci = qc.pack(weight, idx, self.w_bits, gs)
        self.qweight, self.scales, self.cherry_weight, self.cherry_indices = q, s, cw, ci
        self._drop_copies()

    @torch.inference_mode()
    def unpack(self):
        """GPU version of llama/qlinear.py:120-162: dense (out, in) fp16 weight."""
        qc = load_quant_cuda()
        self._require_cuda()
        return qc.unpack_dense(self.qweight, self.scales, self.cherry_weight, self.cherry_indices,
                               self.w_bits, self.in_features, self.group_size)

    # ------------------------------------------------------------------ forward
    def _require_cuda(self):
        if not self.qweight.is_cuda:
            raise RuntimeError("QuantLinear buffers must be on a CUDA device (there is no CPU path)")

    def _buffer_key(self):
        def ver(t):   # tensors made under torch.inference_mode keep no version counter
            return 0 if t.is_inference() else t._version
        bufs = (self.qweight, self.scales, self.cherry_weight, self.cherry_indices)
        return tuple(t.data_ptr() for t in bufs) + tuple(ver(t) for t in bufs)

    def _drop_copies(self):
        self._prepared = None
        self._row = None
        self._tile = None
        self._row_ok = None
        self._prepared_key = None

    def _sync_key(self):
        """Forgets the re-packed copies when the reference buffers were replaced or written to."""
        if self._prepared_key == "released":
            return
        key = self._buffer_key()
        if self._prepared_key != key:
            self._drop_copies()
            self._prepared_key = key

    def _source_buffers(self):
        """The four reference buffers: the module's own, or rebuilt from a copy after a release."""
        if self._prepared_key != "released":
            return self.qweight, self.scales, self.cherry_weight, self.cherry_indices
        src = self._row if self._row is not None else self._prepared
        return src.unprepare()

    def prepared(self):
        """The stream-layout copy of this layer (built on first use)."""
        self._sync_key()
        if self._prepared is None:
            qc = load_quant_cuda()
            self._require_cuda()
            q, s, cw, ci = self._source_buffers()
            self._prepared = qc.PreparedLayer(q, s, cw, ci, self.w_bits, self.in_features, self.group_size)
        return self._prepared

    def row_layer(self):
        """The row-tile copy for the one-row decode kernel, or None where the layer does not fit it."""
        self._sync_key()
        if self._row_ok is None:
            qc = load_quant_cuda()
            self._require_cuda()
            self._row_ok = qc.RowLayer.supported(self.w_bits, self.in_features, self.out_features,
                                                 self.num_cherries, self.group_size)
        if self._row_ok and self._row is None:
            qc = load_quant_cuda()
            q, s, cw, ci = self._source_buffers()
            self._row = qc.RowLayer(q, s, cw, ci, self.w_bits, self.in_features, self.group_size)
        return self._row

    @torch.inference_mode()
    def forward_swiglu(self, gate: torch.Tensor, up: torch.Tensor):
        """This layer applied to silu(gate) * up (the down projection of the reference's LlamaMLP.forward,
        llama/modeling_llama_quant.py): for decode batches the product is formed while the kernel stages its
        input (no separate element-wise kernel, no intermediate tensor), with the same roundings, so the
        result equals forward(silu(gate) * up) bit for bit; other cases compute the product first."""
        rows = gate.numel() // gate.shape[-1]
        row = self.row_layer() if (self._layerwise_dequantize and self.w_bits in (3, 4) and gate.dtype == torch.float16
                                   and rows <= ROW_KERNEL_MAX_ROWS) else None
        if row is None or rows > row.preferred_rows:
            return self(nn.functional.silu(gate.float()).to(gate.dtype) * up)
        g2 = gate.reshape(rows, gate.shape[-1]).contiguous()
        u2 = up.reshape(rows, up.shape[-1]).contiguous()
        out = torch.empty(rows, self.out_features, dtype=torch.float16, device=g2.device)
        row.matvec_swiglu(g2, u2, out)
        out = out.reshape(gate.shape[:-1] + (self.out_features,))
        if self.bias is not None:
            out += self.bias
        return out

    def release_reference_buffers(self):
        """Keeps only the re-packed copies (roughly halves the weight memory);
        `restore_reference_buffers` rebuilds the four buffers bit-exactly."""
        if self.row_layer() is None:
            self.prepared()
        dev = self.qweight.device
        for name in ("qweight", "scales", "cherry_weight", "cherry_indices"):
            setattr(self, name, torch.empty(0, dtype=getattr(self, name).dtype, device=dev))
        self._prepared_key = "released"

    def restore_reference_buffers(self):
        q, s, cw, ci = self._source_buffers()
        self.qweight, self.scales, self.cherry_weight, self.cherry_indices = q, s, cw, ci
        self._prepared_key = self._buffer_key()

    @torch.inference_mode()
    def forward(self, x: torch.Tensor):
        if self._layerwise_dequantize:
            if self.w_bits not in (3, 4):
                raise NotImplementedError(f"{self.w_bits} bit kernel is not implemented yet.")
            out_shape = x.shape[:-1] + (self.out_features,)
            x2 = x.reshape(-1, x.shape[-1])
            if x2.dtype != torch.float16:
                x2 = x2.half()
            x2 = x2.contiguous()
            rows = x2.shape[0]
            row = self.row_layer() if rows <= ROW_KERNEL_MAX_ROWS else None
            if row is not None and rows <= row.preferred_rows:
                out = torch.empty(rows, self.out_features, dtype=torch.float16, device=x2.device)
                row.matvec(x2, out, False)
            elif rows >= 8 and self._prepared_key != "released":
                # more rows: the drop-in op routes them to the tensor-core GEMM (faster from there on)
                qc = load_quant_cuda()
                out = torch.zeros(rows, self.out_features, dtype=torch.float16, device=x2.device)
                if self.w_bits == 4:
                    qc.vecquant4matmul_cherryq(x2, self.qweight, self.cherry_weight, self.cherry_indices,
                                               self.scales, out, self.group_size)
                else:
                    qc.vecquant3matmul_cherryq(x2, self.qweight, self.cherry_weight, self.cherry_indices,
                                               self.scales, out, self.group_size, True)
            elif rows >= 8:
                # released buffers and a large batch: the GEMM on this module's own tile-layout copy
                if self._tile is None:
                    qc = load_quant_cuda()
                    q, s, cw, ci = self._source_buffers()
                    self._tile = qc.TileLayer(q, s, cw, ci, self.w_bits, self.in_features, self.group_size)
                out = torch.empty(rows, self.out_features, dtype=torch.float16, device=x2.device)
                self._tile.gemm(x2, out, False)
            else:
                out = torch.empty(rows, self.out_features, dtype=torch.float16, device=x2.device)
                self.prepared().matvec(x2, out, False)
            out = out.reshape(out_shape).to(x.dtype)
        else:
            if not self.dequantized:
                self.qweight = self.unpack()
                del self.cherry_indices
                del self.cherry_weight
                del self.scales
                self._drop_copies()
                torch.cuda.empty_cache()
                self.dequantized = True
            out = nn.functional.linear(x, self.qweight)
        if self.bias is not None:
            out += self.bias
        return out


def forward_shared_input(layers, x: torch.Tensor):
    """Outputs of several packed layers applied to the same input (q / k / v, gate / up of the
    reference's LLaMA, llama/modeling_llama_quant.py): for decode batches (up to ROW_KERNEL_MAX_ROWS
    rows) and layers that agree in bits, in_features, cherry count and group size this is ONE launch
    of the row-tile kernel per four rows, with the SMs divided among the layers; every other case is
    the layers' own forward, one by one.  The results are bit-identical to the separate calls."""
    layers = list(layers)
    first = layers[0]
    rows = x.numel() // x.shape[-1]
    same = all((l.w_bits, l.in_features, l.num_cherries, l.group_size) ==
               (first.w_bits, first.in_features, first.num_cherries, first.group_size) for l in layers)
    if (rows <= ROW_KERNEL_MAX_ROWS and 1 < len(layers) <= 4 and same and QuantLinear._layerwise_dequantize
            and first.w_bits in (3, 4)):
        rls = [l.row_layer() for l in layers]
        if all(r is not None and rows <= r.preferred_rows for r in rls):
            qc = load_quant_cuda()
            x2 = x.reshape(rows, x.shape[-1])
            if x2.dtype != torch.float16:
                x2 = x2.half()
            x2 = x2.contiguous()
            widths = [l.out_features for l in layers]
            buf = torch.empty(rows, sum(widths), dtype=torch.float16, device=x2.device)
            outs = list(buf.split(widths, dim=1))               # views of one buffer: one row stride
            qc.row_layers_matvec(rls, x2, outs, False)
            res = []
            for l, o in zip(layers, outs):
                o = o.contiguous().reshape(x.shape[:-1] + (l.out_features,)).to(x.dtype)
                if l.bias is not None:
                    o += l.bias
                res.append(o)
            return res
    return [l(x) for l in layers]
