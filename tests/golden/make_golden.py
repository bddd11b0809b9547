"""Generate the golden fixtures in this folder from the REFERENCE project's own code.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/Mixed-precision-CUDA-kernel

It imports the reference's llama/quantizer.py, llama/cherry_linear.py and
llama/qlinear.py unmodified (a stub stands in for the compiled `quant_cuda`
module, which llama/qlinear.py:10 imports at module top but which pack() and
unpack() never call), runs cherry_linear.QuantLinear / qlinear.QuantLinear.pack()
/ .unpack() on seeded inputs and freezes inputs and outputs as .npz files.
The test-suite then checks the numpy oracle and the CUDA kernels against these
files without needing the reference at run time.
"""
import os
import sys
import types

import numpy as np

CASES = [
    # name,                     K,    N,  bits, G,   fraction, dtype, seed
    ("k256_n32_b4_g128_f16",    256,  32, 4,    128, 1 / 16,   "f16", 11),
    ("k256_n32_b3_g128_f16",    256,  32, 3,    128, 1 / 16,   "f16", 12),
    ("k256_n40_b3_g64_f16",     256,  40, 3,    64,  1 / 16,   "f16", 13),
    ("k512_n24_b4_g128_f32",    512,  24, 4,    128, 1 / 32,   "f32", 14),
    ("k640_n8_b3_g64_f32",      640,  8,  3,    64,  1 / 8,    "f32", 15),
    ("k384_n16_b4_g256_f16",    384,  16, 4,    256, 1 / 16,   "f16", 16),
    ("k2048_n16_b4_g128_f16",   2048, 16, 4,    128, 1 / 256,  "f16", 17),
    ("k2048_n16_b3_g128_f16",   2048, 16, 3,    128, 1 / 256,  "f16", 18),
]


def main(ref_root):
    sys.modules["quant_cuda"] = types.ModuleType("quant_cuda")
    sys.path.insert(0, ref_root)
    import torch
    from llama.cherry_linear import QuantLinear as TrainLinear
    from llama.qlinear import QuantLinear as PackedLinear

    here = os.path.dirname(os.path.abspath(__file__))
    for name, k, n, bits, g, frac, dtype, seed in CASES:
        rng = np.random.default_rng(seed)
        w = rng.normal(0.0, 0.02, size=(n, k)).astype(np.float32)
        tl = TrainLinear(k, n, bias=False, w_bits=bits, group_size=g, cherryq=True, cherry_fraction=frac)
        c = tl.num_cherries
        idx = rng.permutation(k)[:c].astype(np.int32)
        w[:, idx] = rng.normal(0.0, 0.2, size=(n, c)).astype(np.float32)
        x = rng.normal(0.0, 1.0, size=(5, k)).astype(np.float16)
        tl.weight.data = torch.from_numpy(w.copy())
        if dtype == "f16":
            tl = tl.half()
        tl.eval()
        tl.register_cherry_indices(torch.from_numpy(idx))
        weight = tl.weight.data.clone()
        pl = PackedLinear(bits, g, tl.quantizer, frac, k, n, bias=False)
        pl.pack(tl)
        dense = pl.unpack()
        fake = tl._adjust_weight(weight, ste=False)
        y = torch.nn.functional.linear(torch.from_numpy(x).float(), dense.float())
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            meta=np.array([k, n, bits, g, c], dtype=np.int64),
            weight=weight.numpy(), cherry_unsorted=idx, x=x,
            qweight=pl.qweight.numpy(), scales=pl.scales.numpy(),
            cherry_weight=pl.cherry_weight.numpy(), cherry_indices=pl.cherry_indices.numpy(),
            dense=dense.numpy(), fake=fake.numpy(), y=y.numpy(),
        )
        print(name, "qweight", tuple(pl.qweight.shape), "scales", tuple(pl.scales.shape))


if __name__ == "__main__":
    main(sys.argv[1])
