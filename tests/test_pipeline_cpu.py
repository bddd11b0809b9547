"""Model-level host logic that needs no GPU: cherry selection, the checkpoint file layout."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")


def test_select_cherries_is_the_top_of_a_descending_argsort():
    from cherryq_b200 import pipeline as P
    rng = np.random.default_rng(0)
    impact = rng.random(4096).astype(np.float32)
    got = P.select_cherries(torch.from_numpy(impact), 1 / 256)
    want = np.argsort(-impact, kind="stable")[:16]
    assert got.dtype == torch.int32 and got.device.type == "cpu"
    assert np.array_equal(got.numpy(), want)
    assert P.num_cherries(11008, 1 / 256) == 40 and P.num_cherries(28672, 1 / 256) == 112 and P.num_cherries(100, 1 / 256) == 0


def test_impact_accumulator_is_the_mean_of_squared_gradients():
    from cherryq_b200 import pipeline as P
    rng = np.random.default_rng(1)
    grads = [torch.from_numpy(rng.normal(size=(6, 32)).astype(np.float32)) for _ in range(5)]
    acc = P.ImpactAccumulator()
    for g in grads:
        acc.update("layer", g)
        acc.update("bias", torch.zeros(6))            # 1-D gradients are skipped, as in the reference
    want = torch.stack([(g ** 2).mean(0) for g in grads]).mean(0)
    assert "bias" not in acc.h
    assert torch.allclose(acc.h["layer"], want, rtol=1e-5, atol=1e-7)
    sel = acc.select(1 / 4)
    assert np.array_equal(sel["layer"].numpy(), np.argsort(-want.numpy(), kind="stable")[:8])


def test_checkpoint_layout_round_trip(tmp_path):
    from cherryq_b200 import pipeline as P
    from cherryq_b200.qlinear import QuantLinear

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = QuantLinear(3, 128, None, 1 / 32, 256, 64, bias=False)
            self.norm = torch.nn.LayerNorm(8)

    m = Tiny()
    g = torch.Generator().manual_seed(0)
    m.proj.qweight = torch.randint(0, 256, m.proj.qweight.shape, dtype=torch.uint8, generator=g)
    m.proj.scales = torch.rand(m.proj.scales.shape, generator=g).half()
    path = P.save_quantized(m, str(tmp_path), {"hidden_size": 256})
    assert path.endswith("pytorch_model-3bit-128g.bin")          # utils.save_quantized's file name
    state, cfg = P.load_quantized_state(str(tmp_path))
    assert cfg["w_bits"] == 3 and cfg["group_size"] == 128 and cfg["hidden_size"] == 256
    assert set(state) == set(m.state_dict())
    assert {"proj.qweight", "proj.scales", "proj.cherry_weight", "proj.cherry_indices"} <= set(state)
    for k, v in m.state_dict().items():
        assert torch.equal(state[k], v)
