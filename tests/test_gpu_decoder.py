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


def test_fused_elementwise_ops_match_torch(dec):
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(5, 512, device="cuda", generator=g).half()
    r = torch.randn(5, 512, device="cuda", generator=g).half()
    w = (1 + 0.1 * torch.randn(512, device="cuda", generator=g)).half()
    y, h = qc.rmsnorm(x, r, w, 1e-5, True)
    hs = (x + r)
    ref = (hs.float() * torch.rsqrt(hs.float().pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
    assert torch.equal(h, hs)
    assert float((y.float() - ref.float()).abs().max()) <= 2e-3 * float(ref.float().abs().max())
    y0 = qc.rmsnorm(x, None, w, 1e-5, False)[0]
    ref0 = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
    assert float((y0.float() - ref0.float()).abs().max()) <= 2e-3 * float(ref0.float().abs().max())

    a, b = torch.randn(3, 1000, device="cuda", generator=g).half(), torch.randn(3, 1000, device="cuda", generator=g).half()
    assert float((qc.silu_mul(a, b).float() - (torch.nn.functional.silu(a) * b).float()).abs().max()) <= 4e-3

    T, H, KV, D, S = 6, 4, 2, 64, 32
    q = torch.randn(T, H, D, device="cuda", generator=g).half()
    k = torch.randn(T, KV, D, device="cuda", generator=g).half()
    v = torch.randn(T, KV, D, device="cuda", generator=g).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(S, device="cuda", dtype=torch.float32), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([3, 4, 5, 9, 10, 31], device="cuda")

    def rope(t):
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        t1, t2 = t[..., : D // 2].float(), t[..., D // 2:].float()
        return torch.cat((t1 * c - t2 * s, t2 * c + t1 * s), -1).half()
    rq, rk = rope(q), rope(k)
    kc = torch.zeros(S, KV, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    qc.rope_cache(q, k, v, cos, sin, pos, kc, vc)
    assert float((q.float() - rq.float()).abs().max()) <= 2e-3 and float((k.float() - rk.float()).abs().max()) <= 2e-3
    assert torch.equal(kc[pos], k) and torch.equal(vc[pos], v)
    untouched = torch.ones(S, dtype=torch.bool, device="cuda")
    untouched[pos] = False
    assert not bool(kc[untouched].any()) and not bool(vc[untouched].any())


@pytest.mark.parametrize("H,KV,D,S,P", [(8, 8, 128, 512, 300), (8, 2, 64, 128, 0), (4, 4, 128, 2048, 2047),
                                       (64, 8, 128, 4096, 4000), (8, 8, 128, 4096, 3), (2, 1, 256, 8192, 8191),
                                       (40, 40, 128, 300, 299)])
def test_attention_decode_matches_torch(dec, H, KV, D, S, P):
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    g = torch.Generator(device="cuda").manual_seed(H + P)
    q = torch.randn(1, H, D, device="cuda", generator=g).half()
    kc = torch.randn(S, KV, D, device="cuda", generator=g).half()
    vc = torch.randn(S, KV, D, device="cuda", generator=g).half()
    pos = torch.tensor([P], device="cuda")
    out = qc.attn_decode(q, kc, vc, pos)
    k = kc[:P + 1].float().repeat_interleave(H // KV, dim=1)          # (P+1, H, D)
    v = vc[:P + 1].float().repeat_interleave(H // KV, dim=1)
    w = torch.softmax(torch.einsum("hd,phd->hp", q[0].float(), k) / D ** 0.5, dim=-1)
    ref = torch.einsum("hp,phd->hd", w, v)
    assert float((out[0].float() - ref).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max()))


def test_positions_are_bounded_by_max_seq(dec):
    """The KV cache holds max_seq positions: the host refuses steps beyond it before anything is
    launched, and a full cache is usable up to its last position."""
    cfg = dec.DecoderConfig(n_layers=1, hidden=256, n_heads=4, n_kv_heads=4, ffn=512, vocab=500, bits=4,
                            group=128, cherry_fraction=1 / 32, max_seq=16)
    a = dec.CherryDecoder(cfg, seed=3)
    prompt = torch.randint(0, cfg.vocab, (10,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
    with pytest.raises(ValueError):
        a.prefill(torch.zeros(16, dtype=torch.long, device="cuda"))         # no free position left
    a.prefill(prompt)
    with pytest.raises(ValueError):
        a.generate(7)                                                       # 10 + 7 > 16
    assert a.pos_host == 10 and int(a.pos.item()) == 10                     # nothing ran
    full = a.generate(6)                                                    # positions 10..15: exactly fits
    assert a.pos_host == 16 and int(a.pos.item()) == 16
    with pytest.raises(ValueError):
        a.generate(1)
    # capture at a late position (the graph is built after the prefill of 15 tokens) stays inside the cache
    b = dec.CherryDecoder(cfg, seed=3)
    b.prefill(torch.cat([prompt, full[:5]]))
    last = b.generate(1)
    assert torch.equal(last, full[5:6])                                     # same greedy continuation


def test_device_side_position_guards():
    """Stray positions never reach memory: the rotary kernel skips tokens outside [0, max_seq) and the
    attention kernel attends to at most max_seq positions."""
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    g = torch.Generator(device="cuda").manual_seed(9)
    T, H, KV, D, S = 3, 4, 2, 64, 8
    q = torch.randn(T, H, D, device="cuda", generator=g).half()
    k = torch.randn(T, KV, D, device="cuda", generator=g).half()
    v = torch.randn(T, KV, D, device="cuda", generator=g).half()
    q0, k0 = q.clone(), k.clone()
    ang = torch.outer(torch.arange(S, device="cuda", dtype=torch.float32), torch.ones(D // 2, device="cuda"))
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([2, 8, -1], device="cuda")                           # the last two are outside
    kc = torch.zeros(S, KV, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    qc.rope_cache(q, k, v, cos, sin, pos, kc, vc)
    torch.cuda.synchronize()
    assert torch.equal(q[1:], q0[1:]) and torch.equal(k[1:], k0[1:])        # skipped tokens are left alone
    assert not torch.equal(q[0], q0[0]) and torch.equal(kc[2], k[0]) and torch.equal(vc[2], v[0])
    mask = torch.ones(S, dtype=torch.bool, device="cuda")
    mask[2] = False
    assert not bool(kc[mask].any()) and not bool(vc[mask].any())
    # attention at a position beyond the cache equals attention over the whole cache
    kcr = torch.randn(S, KV, D, device="cuda", generator=g).half()
    vcr = torch.randn(S, KV, D, device="cuda", generator=g).half()
    a = qc.attn_decode(q[:1].contiguous(), kcr, vcr, torch.tensor([S + 5], device="cuda"))
    b = qc.attn_decode(q[:1].contiguous(), kcr, vcr, torch.tensor([S - 1], device="cuda"))
    assert torch.equal(a, b)


@pytest.mark.parametrize("attention", ["own", "flash"])
@pytest.mark.parametrize("bits,kv,batch", [(4, 4, 3), (3, 2, 5)])
def test_batched_decode_matches_single_sequences(dec, bits, kv, batch, attention):
    """`batch` sequences in lockstep (their own KV caches, four activation rows per kernel launch) against
    one decoder per sequence with the same weights, teacher-forced with the batch's tokens."""
    if attention == "flash":
        pytest.importorskip("flash_attn")
    cfg = tiny(dec, bits, kv)
    big = dec.CherryDecoder(cfg, seed=5, batch=batch, attention=attention)
    singles = [dec.CherryDecoder(cfg, seed=5, attention="own") for _ in range(batch)]
    prompts = torch.randint(0, cfg.vocab, (batch, 21), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    lb = big.prefill(prompts)
    scale = float(lb.float().abs().max())
    for i, s in enumerate(singles):
        ls = s.prefill(prompts[i])
        assert float((lb[i].float() - ls[0].float()).abs().max()) <= 5e-3 * scale
    for _ in range(10):
        for i, s in enumerate(singles):
            s.tok.copy_(big.tok[i:i + 1])
        lb = big._step()
        for i, s in enumerate(singles):
            ls = s._step()
            assert float((lb[i].float() - ls[0].float()).abs().max()) <= 5e-3 * scale
    assert int(big.pos[0].item()) == 31 and bool((big.pos == 31).all())
    # graph replay and eager steps agree for a batch too
    big.prefill(prompts)
    eager = big.generate(8, use_graph=False)
    big.prefill(prompts)
    graphed = big.generate(8, use_graph=True)
    assert eager.shape == (8, batch) and torch.equal(eager, graphed)


def test_batched_rope_cache_and_attention_match_torch():
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    g = torch.Generator(device="cuda").manual_seed(21)
    B, H, KV, D, S = 3, 8, 2, 64, 96
    # decode step: one token per sequence, each at its own position
    q = torch.randn(B, H, D, device="cuda", generator=g).half()
    k = torch.randn(B, KV, D, device="cuda", generator=g).half()
    v = torch.randn(B, KV, D, device="cuda", generator=g).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(S, device="cuda", dtype=torch.float32), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([5, 40, 95], device="cuda")

    def rope(t, p):
        c, s = cos[p][:, None, :], sin[p][:, None, :]
        t1, t2 = t[..., : D // 2].float(), t[..., D // 2:].float()
        return torch.cat((t1 * c - t2 * s, t2 * c + t1 * s), -1).half()
    kc = torch.randn(B, S, KV, D, device="cuda", generator=g).half()
    vc = torch.randn(B, S, KV, D, device="cuda", generator=g).half()
    kc0, vc0 = kc.clone(), vc.clone()
    rq, rk = rope(q, pos), rope(k, pos)
    qc.rope_cache(q, k, v, cos, sin, pos, kc, vc)
    assert float((q.float() - rq.float()).abs().max()) <= 2e-3 and float((k.float() - rk.float()).abs().max()) <= 2e-3
    for b in range(B):
        assert torch.equal(kc[b, pos[b]], k[b]) and torch.equal(vc[b, pos[b]], v[b])
        kc0[b, pos[b]], vc0[b, pos[b]] = k[b], v[b]
    assert torch.equal(kc, kc0) and torch.equal(vc, vc0)                 # nothing else was touched
    out = qc.attn_decode(q, kc, vc, pos)
    for b in range(B):
        n = int(pos[b]) + 1
        kk = kc[b, :n].float().repeat_interleave(H // KV, dim=1)
        vv = vc[b, :n].float().repeat_interleave(H // KV, dim=1)
        w = torch.softmax(torch.einsum("hd,phd->hp", q[b].float(), kk) / D ** 0.5, dim=-1)
        ref = torch.einsum("hp,phd->hd", w, vv)
        assert float((out[b].float() - ref).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max()))
    # prefill form: T tokens per sequence, rows ordered (sequence, token)
    T = 4
    q2 = torch.randn(B * T, H, D, device="cuda", generator=g).half()
    k2 = torch.randn(B * T, KV, D, device="cuda", generator=g).half()
    v2 = torch.randn(B * T, KV, D, device="cuda", generator=g).half()
    kc2 = torch.zeros(B, S, KV, D, dtype=torch.float16, device="cuda")
    vc2 = torch.zeros_like(kc2)
    qc.rope_cache(q2, k2, v2, cos, sin, torch.arange(T, device="cuda").repeat(B), kc2, vc2)
    assert torch.equal(kc2[:, :T].reshape(B * T, KV, D), k2) and torch.equal(vc2[:, :T].reshape(B * T, KV, D), v2)
    assert not bool(kc2[:, T:].any())
