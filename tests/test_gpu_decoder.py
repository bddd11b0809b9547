"""The LLaMA-architecture decode harness: every quantized projection through the CUDA kernels
against the same harness with F.linear(x, unpack()) (the reference's dense mode), on a tiny
random model; CUDA-graph replay against eager steps."""
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dec():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cherryq_b200 import decoder
    return decoder


def tiny(dec, bits, kv_heads=4):
    return dec.DecoderConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=kv_heads, ffn=512, vocab=1000, bits=bits,
                             group=128, cherry_fraction=1 / 32, max_seq=128)


@pytest.mark.parametrize("bits,kv", [(4, 4), (3, 2)])
def test_kernel_path_matches_dense_mode(dec, bits, kv):
    cfg = tiny(dec, bits, kv)
    a = dec.CherryDecoder(cfg, seed=5)
    b = dec.CherryDecoder(cfg, seed=5, dense=True)
    for name in a.PROJ:       # same seed -> same packed buffers
        assert torch.equal(a.layers[1][name].qweight, b.layers[1][name].qweight)
    prompt = torch.randint(0, cfg.vocab, (40,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    la, lb = a.prefill(prompt), b.prefill(prompt)            # 40 rows: the GEMM path
    scale = float(lb.float().abs().max())
    assert float((la.float() - lb.float()).abs().max()) <= 2e-2 * scale
    # teacher forcing with the dense twin's tokens: logits of every step stay close
    agree = 0
    for _ in range(24):
        a.tok.copy_(b.tok)
        la, lb = a._step(), b._step()
        assert float((la.float() - lb.float()).abs().max()) <= 2e-2 * scale
        agree += int(torch.equal(a.tok, b.tok))
    assert agree >= 20


def test_graph_replay_equals_eager_steps(dec):
    cfg = tiny(dec, 4)
    prompt = torch.randint(0, cfg.vocab, (33,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    a = dec.CherryDecoder(cfg, seed=7)
    a.prefill(prompt)
    eager = a.generate(20, use_graph=False)
    a.prefill(prompt)
    graphed = a.generate(20, use_graph=True)
    assert torch.equal(eager, graphed)          # deterministic kernels: identical tokens


def test_bytes_accounting(dec):
    cfg = dec.LLAMA2_7B
    per_layer = sum(dec.linear_algorithmic_bytes(k, n, 4, 128, 1 / 256) for k, n in
                    [(4096, 4096)] * 4 + [(4096, 11008)] * 2 + [(11008, 4096)])
    # per-call bytes of the 7B projections incl. batch-1 activations: 4 x 8,765,472 + 2 x 23,543,328 + 23,524,944
    assert per_layer == 4 * 8_765_472 + 2 * 23_543_328 + 23_524_944
    assert abs(per_layer * cfg.n_layers - 3.38e9) < 5e6          # ~3.38 GB of quantized weights per decoded token
