"""Host-side pieces of the decode harness that need no GPU: byte accounting and configurations."""
import pytest

torch = pytest.importorskip("torch")


def test_linear_bytes_match_the_published_per_layer_figures():
    from cherryq_b200 import decoder as D
    # weight-side bytes + batch-1 activations of the LLaMA-7B shapes, 4-bit, group 128, 1/256 cherries
    assert D.linear_algorithmic_bytes(4096, 4096, 4, 128, 1 / 256) == 8_765_472
    assert D.linear_algorithmic_bytes(4096, 11008, 4, 128, 1 / 256) == 23_543_328
    assert D.linear_algorithmic_bytes(11008, 4096, 4, 128, 1 / 256) == 23_524_944
    assert D.linear_algorithmic_bytes(8192, 28672, 3, 128, 1 / 256) == 93_315_136
    assert D.linear_algorithmic_bytes(28672, 8192, 3, 128, 1 / 256) == 93_315_296


def test_architecture_presets():
    from cherryq_b200 import decoder as D
    assert (D.LLAMA2_7B.n_layers, D.LLAMA2_7B.hidden, D.LLAMA2_7B.ffn, D.LLAMA2_7B.head_dim) == (32, 4096, 11008, 128)
    assert (D.LLAMA2_13B.n_layers, D.LLAMA2_13B.hidden, D.LLAMA2_13B.ffn, D.LLAMA2_13B.bits) == (40, 5120, 13824, 3)
    assert (D.LLAMA2_70B.n_layers, D.LLAMA2_70B.n_heads, D.LLAMA2_70B.n_kv_heads, D.LLAMA2_70B.ffn) == (80, 64, 8, 28672)


def test_decoder_refuses_to_run_without_a_gpu():
    from cherryq_b200 import decoder as D
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(RuntimeError):
        D.CherryDecoder(D.DecoderConfig(n_layers=1, hidden=256, n_heads=4, n_kv_heads=4, ffn=512, vocab=100))
