"""Column-parallel decode harness on two GPUs: every output element is computed by the single-GPU
arithmetic, so the generated tokens must be identical to the one-GPU run.  Needs two devices."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_two_ranks_generate_the_single_gpu_tokens(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from cherryq_b200 import decoder as D
    cfg = D.DecoderConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1000, bits=4, group=128,
                          cherry_fraction=1 / 32, max_seq=128)
    single = D.CherryDecoder(cfg, seed=5)
    prompt = torch.randint(0, cfg.vocab, (40,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    single.prefill(prompt)
    want = single.generate(12, use_graph=False).cpu()
    out = tmp_path / "tokens.pt"
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_decoder_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", worker, str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stderr[-2000:]
    got = torch.load(out, weights_only=True)
    assert torch.equal(got["eager"], want)
    assert torch.equal(got["graphed"], want)
