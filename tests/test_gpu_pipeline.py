"""Whole-model packing on the GPU and the checkpoint round trip of the decode harness."""
import numpy as np
import pytest

from oracle import cherryq_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cherryq_b200 import cherry_linear, decoder, pipeline, qlinear
    return cherry_linear, decoder, pipeline, qlinear


def test_pack_model_replaces_and_packs_every_layer_like_the_oracle(mods):
    cherry_linear, decoder, P, qlinear = mods

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = cherry_linear.QuantLinear(256, 64, w_bits=4, group_size=128, cherryq=True, cherry_fraction=1 / 16)
            self.inner = torch.nn.Sequential(
                cherry_linear.QuantLinear(512, 48, w_bits=3, group_size=64, cherryq=True, cherry_fraction=1 / 32),
                torch.nn.ReLU())

    torch.manual_seed(0)
    m = Block().half().cuda()
    acc = P.ImpactAccumulator()
    for name, mod in m.named_modules():
        if isinstance(mod, cherry_linear.QuantLinear):
            acc.update(name, torch.randn(mod.weight.shape, device="cuda"))
    for name, mod in m.named_modules():                  # each layer registers exactly its own number of cherries
        if isinstance(mod, cherry_linear.QuantLinear):
            mod.register_cherry_indices(P.select_cherries(acc.h[name], mod.cherry_fraction))
    originals = {n: (mod.weight.detach().cpu().numpy(), mod.cherry_indices.cpu().numpy()[:mod.num_cherries],
                     mod.w_bits, mod.group_size)
                 for n, mod in m.named_modules() if isinstance(mod, cherry_linear.QuantLinear)}
    assert P.pack_model(m) == 2
    packed = {n: mod for n, mod in m.named_modules() if isinstance(mod, qlinear.QuantLinear)}
    assert set(packed) == set(originals) == {"a", "inner.0"}
    for n, (w, idx, bits, G) in originals.items():
        ref = O.pack(w, idx, bits, G)
        for b in ("qweight", "scales", "cherry_weight", "cherry_indices"):
            assert np.array_equal(getattr(packed[n], b).cpu().numpy().view(np.uint8), ref[b].view(np.uint8)), (n, b)


def test_decoder_checkpoint_round_trip_in_the_reference_layout(mods, tmp_path):
    cherry_linear, D, P, qlinear = mods
    cfg = D.DecoderConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=500, bits=4, group=128,
                          cherry_fraction=1 / 32, max_seq=64)
    a = D.CherryDecoder(cfg, seed=3)
    sd = P.decoder_state_dict(a)
    assert "model.layers.1.self_attn.q_proj.qweight" in sd and "model.layers.0.mlp.down_proj.cherry_indices" in sd
    assert "model.layers.1.post_attention_layernorm.weight" in sd and "lm_head.weight" in sd and "model.norm.weight" in sd
    assert len(sd) == 3 + 2 * (2 + 7 * 4)

    class Holder(torch.nn.Module):          # anything with this state dict saves the same file
        def __init__(self, state, ql):
            super().__init__()
            self.ql = ql
            self._state = state

        def state_dict(self, *a, **k):
            return self._state

    P.save_quantized(Holder(sd, a.layers[0]["q"]), str(tmp_path), {"num_hidden_layers": 2})
    state, conf = P.load_quantized_state(str(tmp_path))
    assert conf["w_bits"] == 4 and conf["group_size"] == 128
    b = D.CherryDecoder(cfg, seed=99)        # different weights, then overwritten from the file
    prompt = torch.randint(0, cfg.vocab, (12,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    # b runs with its own weights first (one-row, batch and prefill paths: every re-packed copy and the
    # drop-in ops' cache are populated), then takes a's weights: nothing of the old copies may survive
    b.prefill(prompt)
    old = b.generate(16, use_graph=False)
    P.load_decoder_state_dict(b, state)
    a.prefill(prompt)
    b.prefill(prompt)
    new_a, new_b = a.generate(16, use_graph=False), b.generate(16, use_graph=False)
    assert torch.equal(new_a, new_b)
    assert not torch.equal(old, new_b)       # the two weight sets really decode differently
    # and once more into a decoder that already captured its decode graph (the loader drops the graph, which
    # holds the old layers' copies)
    c = D.CherryDecoder(cfg, seed=77)
    c.prefill(prompt)
    c.generate(4, use_graph=True)
    P.load_decoder_state_dict(c, state)
    c.prefill(prompt)
    assert torch.equal(c.generate(16, use_graph=True), new_a)


@pytest.mark.parametrize("k,fraction", [(4096, 1 / 256), (11008, 1 / 256), (28672, 1 / 256), (512, 1 / 16)])
def test_select_cherries_on_the_gpu_matches_numpy(mods, k, fraction):
    """Cherry selection on a device-resident impact vector (estimate_impact.py:85-87 of the reference: the
    top of a descending argsort) against numpy's stable argsort, ties included."""
    _, _, P, _ = mods
    rng = np.random.default_rng(k)
    impact = rng.random(k).astype(np.float32)
    impact[rng.integers(0, k, 64)] = impact.max()          # ties at the top: the lower index wins
    got = P.select_cherries(torch.from_numpy(impact).cuda(), fraction)
    n = P.num_cherries(k, fraction)
    want = np.argsort(-impact, kind="stable")[:n]
    assert got.dtype == torch.int32 and got.device.type == "cpu" and got.shape == (n,)
    assert np.array_equal(got.numpy(), want)
    # a batch of vectors (one per layer) in one call
    many = rng.random((5, k)).astype(np.float32)
    gm = P.select_cherries(torch.from_numpy(many).cuda(), fraction).numpy()
    for r in range(5):
        assert np.array_equal(gm[r], np.argsort(-many[r], kind="stable")[:n])
