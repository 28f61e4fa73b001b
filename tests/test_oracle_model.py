"""CPU tests of the oracle's dense decode step against an independent float64 transformer built from the
same (dequantized) weights: checks RoPE, GQA attention, KV handling, SwiGLU and the residual wiring.
Thresholds follow the reference's own float-vs-quantized tests (cos > 0.999 class, real_llm.rs:10189-10284)."""
import numpy as np
import pytest

import k2t_models as km


def dequant(oracle, m):
    rows = [oracle.ifwht64(oracle.bipolar_dequant_row(m, r) if m.kind == 0 else oracle.nf_dequant_row(m, r)) for r in range(m.rows)]
    return np.stack(rows).astype(np.float64)


def float_model_logits(oracle, spec, tokens):
    c = spec["cfg"]
    h, hd, nq, nkv, inter = c["hidden"], c["head_dim"], c["n_q"], c["n_kv"], c["inter"]
    W = [{k: dequant(oracle, ly[k]) for k in ("qkv", "o", "gate_up", "down")} for ly in spec["layers"]]
    head = dequant(oracle, spec["lm_head"])
    emb = head if spec["embed_bf16"] is None else (spec["embed_bf16"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    rope = spec["rope"].astype(np.float64)
    norm = lambda x, w: x / np.sqrt(np.mean(x * x) + c["eps"]) * w

    def rot(v, pos):
        half = hd // 2
        v = v.reshape(-1, hd).copy()
        x0, x1, co, si = v[:, :half].copy(), v[:, half:].copy(), rope[pos, :half], rope[pos, half:]
        v[:, :half], v[:, half:] = x0 * co - x1 * si, x1 * co + x0 * si
        return v

    K = [[] for _ in W]
    V = [[] for _ in W]
    out = []
    for pos, tok in enumerate(tokens):
        x = emb[tok].copy()
        for l, ly in enumerate(spec["layers"]):
            qkv = W[l]["qkv"] @ norm(x, ly["input_norm"])
            if ly["qkv_bias"] is not None:
                qkv = qkv + ly["qkv_bias"]
            q, k, v = qkv[: nq * hd].reshape(nq, hd), qkv[nq * hd: (nq + nkv) * hd].reshape(nkv, hd), qkv[(nq + nkv) * hd:].reshape(nkv, hd)
            if ly["q_norm"] is not None:
                q = np.stack([norm(r, ly["q_norm"]) for r in q])
                k = np.stack([norm(r, ly["k_norm"]) for r in k])
            q, k = rot(q, pos), rot(k, pos)
            K[l].append(k); V[l].append(v)
            Ks, Vs = np.stack(K[l]), np.stack(V[l])        # [t, nkv, hd]
            att = np.zeros((nq, hd))
            for qh in range(nq):
                kvh = qh // (nq // nkv)
                s = Ks[:, kvh] @ q[qh] / np.sqrt(hd)
                p = np.exp(s - s.max()); p /= p.sum()
                att[qh] = p @ Vs[:, kvh]
            x = x + W[l]["o"] @ att.reshape(-1)
            gu = W[l]["gate_up"] @ norm(x, ly["post_norm"])
            g, u = gu[:inter], gu[inter:]
            x = x + W[l]["down"] @ (g / (1 + np.exp(-g)) * u)
        out.append(head @ norm(x, spec["final_norm"]))
    return np.stack(out)


@pytest.mark.parametrize("mode,kw", [("b6", {}), ("nf4g128", dict(qkv_bias=True, qk_norm=True, tied=False)), ("b5", dict(qkv_bias=True))])
def test_oracle_model_tracks_float_model(oracle, mode, kw):
    spec = km.build(oracle, km.TINY, mode, seed=3, **kw)
    tokens = [5, 17, 300, 42, 7, 199, 63, 250, 11, 90]
    ref = float_model_logits(oracle, spec, tokens)
    m = oracle.Model(spec)
    got = np.stack([m.forward_token(t, threads=2) for t in tokens])
    m.close()
    for t in range(len(tokens)):
        cos = np.dot(got[t], ref[t]) / (np.linalg.norm(got[t]) * np.linalg.norm(ref[t]))
        assert cos > 0.995, (mode, t, cos)
    assert m.h is None


def test_oracle_model_determinism_threads_and_reset(oracle):
    spec = km.build(oracle, km.TINY, "b4", seed=1)
    m = oracle.Model(spec)
    a, la = m.greedy([1, 2, 3, 4], 6, threads=1)
    m.reset()
    b, lb = m.greedy([1, 2, 3, 4], 6, threads=4)
    assert a == b and np.array_equal(la, lb) and m.pos == 10
    e = m.embed(7)
    assert e.shape == (128,) and np.isfinite(e).all()
    m.close()


def test_model_helpers(oracle):
    # exp polynomial close to libm, swiglu definition, rope rotation is norm preserving, argmax takes the first maximum
    x = np.linspace(-20, 20, 401, dtype=np.float32)
    L = oracle.lib()
    oracle.build_rope_table(1, 64, 1e4)   # declares signatures
    approx = np.array([L.k2o_exp_poly(float(v)) for v in x])
    assert np.max(np.abs(approx / np.exp(x.astype(np.float64)) - 1)) < 3e-6
    g, u = x, (x * 0.5 + 1).astype(np.float32)
    assert np.allclose(oracle.swiglu(g, u), g / (1 + np.exp(-g.astype(np.float64))) * u, rtol=1e-5, atol=1e-6)
    rope = oracle.build_rope_table(40, 64, 1e5)
    v = np.random.default_rng(0).standard_normal(3 * 64).astype(np.float32)
    r = oracle.rope_heads(v, 3, 64, rope[17])
    assert np.allclose(np.linalg.norm(r.reshape(3, 64), axis=1), np.linalg.norm(v.reshape(3, 64), axis=1), rtol=1e-5)
    assert np.array_equal(oracle.rope_heads(v, 3, 64, rope[0]), v)       # position 0: cos 1, sin 0
    assert oracle.argmax(np.array([1, 5, 5, 2], np.float32)) == 1
    q, s = oracle.kv_quant_head(v[:64])
    assert np.abs(q).max() == 127 and s > 0


# ----------------------------------------------------------------------------- NF4 Hadamard KV cache (kv_bits = 4)
NF4 = np.array([-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127], np.float32)


def test_nf4_nearest_idx_is_the_nearest_centroid(oracle):
    ys = np.concatenate([np.linspace(-140, 140, 2801, dtype=np.float32), NF4, (NF4[:-1] + NF4[1:]) / 2])
    for y in ys:
        idx = oracle.nf4_nearest_idx(y)
        best = np.abs(NF4 - y).min()
        assert abs(NF4[idx] - y) == best, (y, idx)             # ties at the midpoints may go either way
    assert oracle.nf4_nearest_idx(0.0) == 8 and oracle.nf4_nearest_idx(-0.0) == 8 and oracle.nf4_nearest_idx(-1e-3) == 7


def test_q4_head_quantizer_layout_and_error(oracle):
    from k2t_rng import normal
    for hd in (64, 128):
        x = normal(hd, hd) * np.float32(0.7)
        q4, s16 = oracle.kv_quant_head_q4(x)
        assert q4.size == hd // 2 and s16.size == hd // 64
        rot = oracle.fwht64(x)                                 # block index = group within the head
        for g in range(hd // 64):
            scale = (np.uint32(s16[g]) << 16).view(np.float32)
            blk = rot[g * 64:(g + 1) * 64]
            deq = np.zeros(64, np.float32)
            for h in range(2):
                for i in range(16):
                    b = q4[g * 32 + h * 16 + i]
                    deq[h * 32 + i], deq[h * 32 + 16 + i] = NF4[b & 15] * scale, NF4[b >> 4] * scale
            # every index is the nearest centroid at the stored scale, and the scale is the bf16 least-squares fit
            for j in range(64):
                assert abs(deq[j] - blk[j]) <= np.abs(NF4 * scale - blk[j]).min() + 1e-7
            assert np.linalg.norm(deq - blk) / np.linalg.norm(blk) < 0.12
    z, s = oracle.kv_quant_head_q4(np.zeros(64, np.float32))
    assert s[0] == 0 and (z == 0x88).all()                     # an all-zero group: scale 0, indices 8|8


def test_oracle_q4_cache_tracks_int8_cache_and_byte_count(oracle):
    cfg4 = dict(km.TINY, kv_bits=4)
    spec4, spec8 = km.build(oracle, cfg4, "b5", seed=3), km.build(oracle, km.TINY, "b5", seed=3)
    m4, m8 = oracle.Model(spec4), oracle.Model(spec8)
    for t in [5, 17, 300, 42, 7, 199]:
        a, b = m4.forward_token(t, 2), m8.forward_token(t, 2)
        assert np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)) > 0.985
    k, ks, v, vs = m4.read_kv(1, 1, 3)
    assert k.dtype == np.uint8 and k.size == 32 and ks.size == 1
    m4.close(); m8.close()
    # KV bytes per token of the 135M shape: 12,240 (int8) and 6,120 (NF4), as published with the reference's benchmarks
    c = km.SMOL_135M
    assert 2 * c["layers"] * c["n_kv"] * (c["head_dim"] + 4) == 12240
    assert 2 * c["layers"] * c["n_kv"] * (c["head_dim"] // 2 + 2 * (c["head_dim"] // 64)) == 6120


# ----------------------------------------------------------------------------- sparse-MoE router
@pytest.mark.parametrize("scoring,norm", [(0, True), (0, False), (1, True), (2, True), (2, False)])
def test_moe_router_scoring_modes(oracle, scoring, norm):
    """Routes of the oracle against a direct numpy evaluation of DenseMoeRouter::route_sorted (float64 scores: the expert
    SET and order must agree, the weights to fp32 rounding)."""
    moe = dict(layers=[0], n_experts=8, top_k=3, d_ff=64, bits=4, sgc=1, norm_topk=norm, scoring=scoring, bias=True)
    spec = km.build(oracle, km.MOE_TINY, "b4", seed=5, moe=moe)
    m = oracle.Model(spec)
    m.forward_token(11, 2)
    ids, w = m.last_routes(0)
    assert list(ids) == sorted(ids) and len(ids) == 3
    # recompute from the post-attention hidden state of layer 0: run the attention block by hand
    ly = spec["layers"][0]
    m2 = oracle.Model(spec)
    hidden = m2.embed(11)
    hidden = (hidden + m2.attn_part(0, hidden)).astype(np.float32)
    x = hidden.astype(np.float64)
    xn = x / np.sqrt(np.mean(x * x) + km.MOE_TINY["eps"]) * ly["post_norm"]
    logits = ly["moe"]["router_w"].astype(np.float64) @ xn + ly["moe"]["router_bias"]
    if scoring == 1:
        top = np.argsort(-logits, kind="stable")[:3]
        p = np.exp(logits[top] - logits[top].max()); p /= p.sum()
    else:
        sc = np.exp(logits - logits.max()) / np.exp(logits - logits.max()).sum() if scoring == 0 else 1 / (1 + np.exp(-logits))
        top = np.argsort(-sc, kind="stable")[:3]
        p = sc[top] / (sc[top].sum() if norm else 1.0)
    order = np.argsort(top)
    assert list(ids) == list(top[order])
    assert np.allclose(w, p[order], rtol=1e-4, atol=1e-6)
    m.close(); m2.close()


def test_sliding_window_ring_geometry_and_rollback_guard(oracle):
    """QuantizedKvCache::new_with_opts (real_llm.rs:1235-1257) and can_truncate_kv_to (1806-1821) as restated in the oracle:
    ring rows = sinks + (window - sinks) + 512, sinks capped at window / 2, a window is ignored unless window + 512 < max_seq;
    the reference test's three rollback cases at position 640 (real_llm.rs:10630-10632); while the context is shorter than
    the window the windowed attention agrees with the full one to rounding (it adds one score term per 64-value group)."""
    import k2t_models as km
    cfg = dict(hidden=128, layers=2, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=192, max_seq=1024, eps=1e-5, theta=1e5)
    spec = km.build(oracle, cfg, "b4", seed=5)
    full, win = oracle.Model(spec), oracle.Model(dict(spec, cfg=dict(cfg, kv_bits=4, kv_window=16, kv_sinks=4)))
    try:
        assert win.kv_rows == 4 + 12 + 512 and full.kv_rows == 1024
        assert not full.set_kv_window(8, 600, 4) and full.kv_rows == 1024          # 600 + 512 >= 1024: full context kept
        assert full.set_kv_window(8, 100, 80) and full.kv_rows == 50 + 50 + 512      # sinks capped at window / 2
        assert not full.set_kv_window(8, 0, 0)
        tokens = [(i * 13 + 5) % 192 for i in range(640)]
        for t in tokens:
            win.forward_token(t, threads=2)
        assert win.can_truncate_kv_to(0) and not win.can_truncate_kv_to(8) and win.can_truncate_kv_to(638)
        short = oracle.Model(dict(spec, cfg=dict(cfg, kv_window=64, kv_sinks=4)))
        full.reset()
        for t in tokens[:60]:
            a, b = full.forward_token(t, threads=2), short.forward_token(t, threads=2)
            assert np.max(np.abs(a - b)) <= 1e-5 * max(1.0, float(np.max(np.abs(a))))
        short.close()
    finally:
        full.close(); win.close()


def test_reference_hadamard_q8_kv_attention_accuracy_case(oracle):
    """The reference's own accuracy test for the int8 Hadamard cache, run against this restatement with its generator and
    threshold (test_hadamard_q8_kv_cache_attention_accuracy, src/model/real_llm.rs:10189-10284): 6 query / 2 kv heads, head_dim
    64 and 128, 37 positions with 12x outliers on two channels per head, queries at positions 0, 7, 15, 36 - the attention
    over the quantized cache must keep a cosine above 0.9998 against the unquantized float attention; and the cache costs
    2 * (head_dim + 4) bytes per (layer, kv head, position), the byte identity that test asserts."""
    for hd in (64, 128):
        heads, kv_heads, n_max = 6, 2, 37
        kv_dim = kv_heads * hd
        attn_scale = np.float32(1.0 / np.sqrt(np.float32(hd)))
        assert 2 * 2 * 64 * (2 * hd + 8) == 64 * 2 * 2 * kv_heads * (hd + 4)       # physical_bytes() of 2 layers x 2 kv heads x 64 positions

        def f(i, m):
            base = (np.float32((i * m) % 101) / np.float32(101.0) - np.float32(0.5)) * np.float32(1.6)
            return base * np.float32(12.0) if (i % hd) in (7, hd // 2 + 7) else base

        k_all = np.array([f(i, 19) for i in range(n_max * kv_dim)], np.float32).reshape(n_max, kv_heads, hd)
        v_all = np.array([f(i, 29) for i in range(n_max * kv_dim)], np.float32).reshape(n_max, kv_heads, hd)
        for pos in (0, 7, 15, 36):
            q = np.array([f(i + pos * 13, 37) for i in range(heads * hd)], np.float32).reshape(heads, hd)
            n = pos + 1
            got = oracle.attention_q8(q, k_all[:n].transpose(1, 0, 2), v_all[:n].transpose(1, 0, 2), float(attn_scale))
            want = np.zeros((heads, hd))
            for h in range(heads):
                kvh = h // (heads // kv_heads)
                sc = (k_all[:n, kvh].astype(np.float64) @ q[h].astype(np.float64)) * float(attn_scale)
                e = np.exp(sc - sc.max())
                want[h] = (e / e.sum()) @ v_all[:n, kvh].astype(np.float64)
            a, b = got.astype(np.float64).reshape(-1), want.reshape(-1)
            cos = float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))
            assert cos > 0.99980, (hd, pos, cos)


@pytest.mark.parametrize("gate", [True, False])
def test_shared_expert_adds_its_output_before_the_routed_experts(oracle, gate):
    """SharedMoeExpert::forward_single (sparse_moe.rs:254-314) in the oracle's MoE block against a composition of the oracle's
    own primitives: the shared output (two NF projections around the scalar-exp SwiGLU, times the sigmoid gate) is what the
    block starts from; a model without routed contribution (top-1 expert whose down scales are zero is not constructible
    from files, so the routed part is compared through the model without a shared expert)."""
    moe = dict(layers=[1], n_experts=4, top_k=2, d_ff=64, bits=4, sgc=1, shared=128, shared_gate=gate)
    spec = km.build(oracle, km.MOE_TINY, "b4", seed=23, moe=moe)
    plain = km.build(oracle, km.MOE_TINY, "b4", seed=23, moe=dict(moe, shared=0))
    a, b = oracle.Model(spec), oracle.Model(plain)
    try:
        h = km.MOE_TINY["hidden"]
        hidden = np.random.Generator(np.random.PCG64(3)).standard_normal(h).astype(np.float32)
        with_shared, routed = a.ffn_part(1, hidden), b.ffn_part(1, hidden)
        ly = spec["layers"][1]
        sh = ly["moe"]["shared"]
        x_norm = (hidden * oracle.inv_rms(hidden, km.MOE_TINY["eps"])) * ly["post_norm"]
        act = oracle.act_populate_fwht(x_norm)
        gu = oracle.gemv(sh["gate_up"], act).reshape(-1)
        g, u = gu[:128], gu[128:]
        sw = ((g / (np.float32(1) + np.exp(-g.astype(np.float64)).astype(np.float32))) * u).astype(np.float32)
        out = oracle.gemv(sh["down"], oracle.act_populate_fwht(sw)).reshape(-1)
        if gate:
            z = oracle.dot_f32(sh["gate_w"], x_norm)
            scale = np.float32(1) / (np.float32(1) + np.float32(np.exp(-np.float64(z))))
            out = (out * scale).astype(np.float32)
        # (shared + w0 e0) + w1 e1 against (0 + w0 e0) + w1 e1: equal up to the rounding of the two sums
        assert np.allclose(with_shared - routed, out, rtol=0, atol=4e-6 * max(1.0, float(np.max(np.abs(with_shared)))))
        assert float(np.linalg.norm(out)) > 1e-3          # the shared expert contributes
        # no routed experts at all (expert parallel emulation, rank 1 of 2 holds no routed expert of this token or some): rank 0 carries the shared output
        a.L.k2o_model_set_ep(a.h, 64, 0)                   # 64 ranks, rank 0: at most expert 0 is local
        e, w = a.last_routes(1)
        if 0 not in list(e):
            assert np.array_equal(a.ffn_part(1, hidden), out)
    finally:
        a.close(); b.close()
