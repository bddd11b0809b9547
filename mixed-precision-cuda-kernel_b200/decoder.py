"""Minimal LLaMA-architecture decode harness around the CherryQ quantized linear.

The reference evaluates its kernels inside a vendored Hugging Face LLaMA
(llama/modeling_llama_quant.py:724-785 decoder layer, :251 MLP, :371-419 attention of the
reference project; protocol of benchmark_perplexity.py:92-113).  This module keeps only what
a decode benchmark needs: RMSNorm fused with the residual add, rotary embeddings (HF "rotate
half" convention) fused with the KV-cache write, SwiGLU (three small CUDA kernels of the
library), an fp16 KV cache, an unquantised fp16 lm_head, greedy sampling, and the seven quantized
projections per layer as `QuantLinear` modules (q, k, v, o, gate, up, down - separate, as in
the reference, each with its own cherry columns).  Weights are random (no checkpoint can be
loaded offline): dense ~ N(0, 0.02), cherry columns ~ N(0, 0.2), packed on the GPU layer by
layer so that the fp16 model never exists in memory.

One decode step (embedding lookup -> layers -> logits -> argmax -> cache / position update)
touches only device tensors, so it is captured once in a CUDA graph and replayed.
Decode attention is a single-query kernel of the library that reads the current position on the
device (so the captured graph serves every step); prefill attention is torch's
scaled_dot_product_attention.  Both are plumbing here, not the measured path.

`tp_group` shards every projection along its output rows over the ranks of a process group
(column parallel: heads for q / k / v, output features for o / gate / up / down) and gathers the
slices with an NCCL all-gather where the next op needs the whole vector (attention output, o,
SwiGLU output, down): four collectives per layer.  Every output element is still computed by
exactly the single-GPU arithmetic, so the tokens are identical for every group size; all ranks
draw the full random weight and pack only their rows.

`dense=True` builds the parity twin: the same packed buffers, every projection computed as
F.linear(x, unpack()) the way the reference's dense mode does (llama/qlinear.py:183-195).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from . import load_quant_cuda
from .qlinear import QuantLinear, forward_shared_input


@dataclass
class DecoderConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    bits: int = 4
    group: int = 128
    cherry_fraction: float = 1 / 256
    max_seq: int = 512
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads


LLAMA2_7B = DecoderConfig()
LLAMA2_13B = DecoderConfig(n_layers=40, hidden=5120, n_heads=40, n_kv_heads=40, ffn=13824, bits=3)
LLAMA2_70B = DecoderConfig(n_layers=80, hidden=8192, n_heads=64, n_kv_heads=8, ffn=28672, bits=3)


def linear_algorithmic_bytes(k: int, n: int, bits: int, group: int, fraction: float, m: int = 1) -> int:
    """Bytes one call of a quantized linear has to move (reference-format sizes)."""
    c = math.ceil(k * fraction) // 8 * 8
    kc = k - c
    return kc // 8 * bits * n + math.ceil(kc / group) * n * 2 + c * n * 2 + c * 2 + m * k * 2 + m * n * 2


class CherryDecoder:
    PROJ = ("q", "k", "v", "o", "gate", "up", "down")

    def __init__(self, cfg: DecoderConfig, device="cuda", seed: int = 0, dense: bool = False,
                 release_reference_buffers: bool = False, tp_group=None, tp_gather: str = "peer", batch: int = 1,
                 attention: str = "auto"):
        if not torch.cuda.is_available():
            raise RuntimeError("CherryDecoder needs a CUDA device (there is no CPU path)")
        if batch < 1:
            raise ValueError("batch must be at least 1")
        self.cfg, self.dev, self.dense = cfg, torch.device(device), dense
        self.batch = batch          # sequences decoded in lockstep (same prompt length, one position counter)
        # decode attention over the KV cache: "own" = this library's kernel (cq_attn_decode); "flash" = the
        # flash_attn package's flash_attn_with_kvcache (a library call, like the lm_head's cuBLAS matmul);
        # "auto" = own, except for grouped-query models with caches of more than 1024 positions where that
        # package imports.  Measured on B200: without grouped queries the own kernel is ahead at every size
        # tried (13B shapes at 2100 positions: 19 us against 22 at batch 1, 91 against 159 at batch 8; 7B at 200
        # positions 9 against 21); with 8 query heads per KV head at 4000 positions its SIMT dot products lose to
        # flash_attn's tensor-core tiles (45 us against 25 at batch 1, 110 against 29 at batch 4).
        if attention not in ("auto", "own", "flash"):
            raise ValueError("attention is 'auto', 'own' or 'flash'")
        self._flash = None
        if attention == "flash" or (attention == "auto" and cfg.max_seq > 1024 and cfg.n_kv_heads < cfg.n_heads):
            try:
                from flash_attn import flash_attn_with_kvcache
                self._flash = flash_attn_with_kvcache
            except Exception:
                if attention == "flash":
                    raise
        self.qc = load_quant_cuda()
        self.group = tp_group
        if tp_group is not None:
            import torch.distributed as dist
            self.tp, self.rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
        else:
            self.tp, self.rank = 1, 0
        # exchange step of the sharded projections: "peer" = this library's peer-memory kernel for
        # slices that fit its landing area (decode batches), NCCL for the rest (prefill); "nccl" = NCCL only
        self.peer = None
        if self.tp > 1 and tp_gather == "peer":
            from .parallel import PeerAllGather
            try:
                self.peer = PeerAllGather(tp_group, self.dev)
            except RuntimeError as e:       # raised on every rank together: all of them take NCCL
                import warnings
                warnings.warn(f"peer-memory exchange unavailable ({e}); the sharded projections use NCCL")
        elif tp_gather not in ("peer", "nccl"):
            raise ValueError("tp_gather is 'peer' or 'nccl'")
        g = torch.Generator(device=self.dev).manual_seed(seed)
        hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        shapes = {"q": (cfg.hidden, h * hd), "k": (cfg.hidden, kv * hd), "v": (cfg.hidden, kv * hd),
                  "o": (h * hd, cfg.hidden), "gate": (cfg.hidden, cfg.ffn), "up": (cfg.hidden, cfg.ffn),
                  "down": (cfg.ffn, cfg.hidden)}
        if h % self.tp or kv % self.tp or any(n % (8 * self.tp) for _, n in shapes.values()):
            raise ValueError(f"{self.tp} ranks do not divide the heads / output features of this configuration")
        self.full_shapes = shapes
        self.shapes = {name: (k, n // self.tp) for name, (k, n) in shapes.items()}    # this rank's shards
        self.h_local, self.kv_local = h // self.tp, kv // self.tp
        self.layers = []
        for _ in range(cfg.n_layers):
            lay = {name: self._make_linear(k, n, g) for name, (k, n) in self.full_shapes.items()}
            lay["norm1"] = torch.ones(cfg.hidden, dtype=torch.float16, device=self.dev)
            lay["norm2"] = torch.ones(cfg.hidden, dtype=torch.float16, device=self.dev)
            if release_reference_buffers and not dense:
                for name in self.PROJ:
                    lay[name].release_reference_buffers()
            self.layers.append(lay)
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, device=self.dev, generator=g) * 0.02).half()
        self.lm_head = (torch.randn(cfg.vocab, cfg.hidden, device=self.dev, generator=g) * 0.02).half()
        self.final_norm = torch.ones(cfg.hidden, dtype=torch.float16, device=self.dev)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=self.dev, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(cfg.max_seq, device=self.dev, dtype=torch.float32), inv)
        self.cos, self.sin = ang.cos(), ang.sin()                      # (max_seq, hd / 2)
        self.k_cache = torch.zeros(cfg.n_layers, batch, cfg.max_seq, self.kv_local, hd, dtype=torch.float16, device=self.dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        # state of the decode loop, all on the device: next token and position of every sequence
        self.tok = torch.zeros(batch, dtype=torch.long, device=self.dev)
        self.pos = torch.zeros(batch, dtype=torch.long, device=self.dev)
        self.pos_host = 0           # the host's copy of `pos`: every step is checked against max_seq before it is launched
        self.graph = None

    # ------------------------------------------------------------------ construction
    def _make_linear(self, k: int, n: int, g: torch.Generator) -> QuantLinear:
        cfg = self.cfg
        w = (torch.randn(n, k, device=self.dev, generator=g) * 0.02).half()
        c = math.ceil(k * cfg.cherry_fraction) // 8 * 8
        idx = torch.randperm(k, device=self.dev, generator=g)[:c].to(torch.int32)
        if c:
            w[:, idx.long()] = (torch.randn(n, c, device=self.dev, generator=g) * 0.2).half()
        if self.tp > 1:            # this rank's output rows of the same full matrix
            n = n // self.tp
            w = w[self.rank * n:(self.rank + 1) * n].contiguous()
        ql = QuantLinear(cfg.bits, cfg.group, None, cfg.cherry_fraction, k, n, bias=False).to(self.dev)
        ql.pack(SimpleNamespace(weight=w, bias=None, cherry_indices=idx, group_size=cfg.group))
        if self.dense:
            ql.dense_weight = ql.unpack()
        return ql

    def quantized_bytes_per_token(self) -> int:
        cfg = self.cfg
        per_layer = sum(linear_algorithmic_bytes(k, n, cfg.bits, cfg.group, cfg.cherry_fraction)
                        for k, n in self.shapes.values())
        return per_layer * cfg.n_layers

    def lm_head_bytes(self) -> int:
        return self.cfg.vocab * self.cfg.hidden * 2

    # ------------------------------------------------------------------ building blocks
    def _lin(self, ql: QuantLinear, x: torch.Tensor) -> torch.Tensor:
        if self.dense:
            return F.linear(x, ql.dense_weight)
        return ql(x)

    def _lins(self, lay, names, x: torch.Tensor):
        """The projections `names` of one layer on the same input: one launch where the kernel allows."""
        if self.dense:
            return [F.linear(x, lay[n].dense_weight) for n in names]
        return forward_shared_input([lay[n] for n in names], x)

    def _lin_gather(self, ql: QuantLinear, x: torch.Tensor) -> torch.Tensor:
        """A sharded projection followed by the exchange of its slices; for decode batches of up to four rows
        both happen in one launch of the row-tile kernel."""
        if self.tp > 1 and self.peer is not None and not self.dense and x.shape[0] <= 4 and x.dtype == torch.float16:
            row = ql.row_layer()
            if row is not None and self.peer.fits(x.shape[0], ql.out_features):
                return self.peer.matvec_gather(row, x.contiguous())
        return self._gather(self._lin(ql, x))

    def _gather(self, x: torch.Tensor) -> torch.Tensor:
        """(t, n_local) slices of all ranks -> (t, tp * n_local), in rank order."""
        if self.tp == 1:
            return x
        import torch.distributed as dist
        t, nl = x.shape
        if self.peer is not None and x.dtype == torch.float16 and self.peer.fits(t, nl):
            return self.peer(x.contiguous())
        out = torch.empty(self.tp, t, nl, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out.view(1, self.tp * nl) if t == 1 else out.permute(1, 0, 2).reshape(t, self.tp * nl)

    def _norm(self, h: torch.Tensor, delta, w: torch.Tensor):
        """(rmsnorm(h + delta) * w, h + delta): the residual add rides in the norm kernel."""
        if delta is None:
            return self.qc.rmsnorm(h, None, w, self.cfg.eps, False)[0], h
        y, hs = self.qc.rmsnorm(h, delta, w, self.cfg.eps, True)
        return y, hs

    def _layer(self, li: int, h: torch.Tensor, delta, pos: torch.Tensor, decode: bool):
        """One decoder layer on the residual stream h with the previous layer's MLP output `delta`
        still to be added; returns (h, delta) in the same form."""
        cfg, lay = self.cfg, self.layers[li]
        t, nh, kv, hd, nb = h.shape[0], self.h_local, self.kv_local, cfg.head_dim, self.batch
        xn, h = self._norm(h, delta, lay["norm1"])
        q, k, v = self._lins(lay, ("q", "k", "v"), xn)
        q, k, v = q.view(t, nh, hd), k.view(t, kv, hd), v.view(t, kv, hd)
        self.qc.rope_cache(q, k, v, self.cos, self.sin, pos, self.k_cache[li], self.v_cache[li])
        if decode:
            if self._flash is not None:
                a = self._flash(q.view(t, 1, nh, hd), self.k_cache[li], self.v_cache[li],
                                cache_seqlens=(pos + 1).to(torch.int32), causal=True).view(t, nh * hd)
            else:
                a = self.qc.attn_decode(q, self.k_cache[li], self.v_cache[li], pos).view(t, nh * hd)
        else:
            ts = t // nb              # tokens per sequence; rows are (sequence, token)
            a = F.scaled_dot_product_attention(q.view(nb, ts, nh, hd).transpose(1, 2), k.view(nb, ts, kv, hd).transpose(1, 2),
                                               v.view(nb, ts, kv, hd).transpose(1, 2), is_causal=True, enable_gqa=(kv != nh))
            a = a.transpose(1, 2).reshape(t, nh * hd)
        xn, h = self._norm(h, self._lin_gather(lay["o"], self._gather(a)), lay["norm2"])
        gate, up = self._lins(lay, ("gate", "up"), xn)
        if self.tp == 1 and not self.dense and t <= 16:
            # one GPU, decode batch: the SwiGLU rides in the down projection's input staging
            return h, lay["down"].forward_swiglu(gate, up)
        act = self.qc.silu_mul(gate, up)
        return h, self._lin_gather(lay["down"], self._gather(act))

    def _logits(self, h: torch.Tensor, delta) -> torch.Tensor:
        return F.linear(self._norm(h, delta, self.final_norm)[0], self.lm_head)

    # ------------------------------------------------------------------ prefill / decode
    @torch.inference_mode()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """Runs the prompts (T,) or (batch, T) through the model, fills the caches, returns the last
        position's logits (batch, vocab)."""
        if tokens.dim() == 1:
            tokens = tokens[None]
        if tokens.shape[0] != self.batch:
            raise ValueError(f"{tokens.shape[0]} prompts for a decoder of batch {self.batch}")
        t = tokens.shape[1]
        if not 0 < t < self.cfg.max_seq:
            raise ValueError(f"a prompt of {t} tokens does not fit max_seq = {self.cfg.max_seq} (one position must stay free)")
        pos = torch.arange(t, device=self.dev).repeat(self.batch)
        h, delta = self.embed[tokens.reshape(-1)], None
        for li in range(self.cfg.n_layers):
            h, delta = self._layer(li, h, delta, pos, decode=False)
        last = torch.arange(self.batch, device=self.dev) * t + (t - 1)
        logits = self._logits(h[last].contiguous(), delta[last].contiguous())
        self._check_exchange()
        self.pos.fill_(t)
        self.pos_host = t
        self.tok.copy_(logits.argmax(-1))
        return logits

    @torch.inference_mode()
    def _step(self) -> torch.Tensor:
        """One greedy decode step on the device-side state; returns the logits (1, vocab)."""
        h, delta = self.embed[self.tok], None
        for li in range(self.cfg.n_layers):
            h, delta = self._layer(li, h, delta, self.pos, decode=True)
        logits = self._logits(h, delta)
        self.tok.copy_(logits.argmax(-1))
        self.pos.add_(1)
        return logits

    @torch.inference_mode()
    def capture(self):
        """Captures one decode step in a CUDA graph (the state tensors are saved and restored)."""
        if self.cfg.max_seq < 4:
            raise ValueError("max_seq must be at least 4")
        # the warm-up and the captured step run at positions 0, 1, 2: always inside the cache, whatever
        # the current position is (state and those cache rows are restored below)
        saved = (self.tok.clone(), self.pos.clone(), self.k_cache[:, :, :3].clone(), self.v_cache[:, :, :3].clone())
        self.pos.zero_()
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):          # warm-up: first-use re-packs and allocations happen here
                self._step()
            s.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=s):
                self.graph_logits = self._step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        for dst, src in zip((self.tok, self.pos, self.k_cache[:, :, :3], self.v_cache[:, :, :3]), saved):
            dst.copy_(src)

    @torch.inference_mode()
    def generate(self, n_tokens: int, use_graph: bool = True) -> torch.Tensor:
        """Greedy continuation after `prefill`: returns the n_tokens generated ids, (n_tokens,) for one
        sequence and (n_tokens, batch) for more (the first one is the prefill's argmax)."""
        if n_tokens < 0 or self.pos_host + n_tokens > self.cfg.max_seq:
            raise ValueError(f"{n_tokens} more tokens after position {self.pos_host} do not fit max_seq = "
                             f"{self.cfg.max_seq}: the KV cache holds max_seq positions")
        out = torch.empty(n_tokens, self.batch, dtype=torch.long, device=self.dev)
        if use_graph and self.graph is None:
            self.capture()
        for i in range(n_tokens):
            out[i:i + 1].copy_(self.tok)
            if use_graph:
                self.graph.replay()
            else:
                self._step()
        self.pos_host += n_tokens
        self._check_exchange()
        return out[:, 0] if self.batch == 1 else out

    def _check_exchange(self):
        """Raises if a peer never delivered a slice (the kernel fills that output with NaN and sets a
        status bit) or a bounded device-side wait of a projection ran out: one host read per call."""
        if self.peer is not None:
            self.peer.check()
        if self.qc.device_timed_out(self.dev.index if self.dev.index is not None else torch.cuda.current_device()):
            raise RuntimeError("a bounded device-side wait of a quantized projection ran out")
