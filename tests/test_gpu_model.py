"""GPU parity tests of the whole-token engine (kronos_cuda_engine_*) against the CPU oracle model.

What is exact and what is not:
  * embedding, RMSNorm (sum of squares in the CPU's accumulator order), FWHT + int8 quantization, every
    GEMV, bias, qk-norm, RoPE, the KV cache entries, SwiGLU, argmax, and - for contexts of up to 512
    positions - the attention (scores, exp, the 4-accumulator sum, position-ascending value chains)
    reproduce the CPU arithmetic bit for bit.  So for contexts <= 512 the logits of every token, the KV cache
    and the greedy stream must be identical (np.array_equal);
  * beyond 512 positions the attention runs as a scores and a values kernel in the same order, so everything above
    holds at any length (test_long_context_attention_is_exact, test_greedy_crosses_512_positions);
  * only with the split-KV flag set do long contexts sum in a different order: scores stay exact, the attention
    output agrees to fp32 rounding, logits to the tolerance test_split_kv_attention_on_request states.
"""
import numpy as np
import pytest

import k2t_models as km

pytestmark = pytest.mark.gpu

TOL = 1e-3


@pytest.fixture(scope="module")
def ctx():
    import kronos_2t_b200 as k2
    c = k2.Context(0)
    yield c
    c.close()


def make(ctx, oracle, cfg, mode, **kw):
    import kronos_2t_b200 as k2
    spec = km.build(oracle, cfg, mode, **kw)
    return spec, k2.Engine(ctx, spec), oracle.Model(spec)


def close_logits(got, want):
    return np.max(np.abs(got - want)) <= TOL * max(1.0, float(np.max(np.abs(want))))


VARIANTS = [
    ("b4", {}),
    ("b5", dict(qkv_bias=True)),
    ("b6", dict(qkv_bias=True, qk_norm=True, tied=False)),
    ("nf4g128", dict(qk_norm=True)),
    ("nf4", dict(tied=False)),
    ("nf3g128", {}),
    ("nf5g128", dict(qkv_bias=True)),
    ("e8q2g128", {}),
    ("b4", dict(modes=dict(qkv="b5", o="b5", gate_up="b4", down="b5", head="b4"))),      # the p55454-style mix
]


@pytest.mark.parametrize("mode,kw", VARIANTS)
def test_prompt_logits_and_kv(ctx, oracle, mode, kw):
    spec, eng, ref = make(ctx, oracle, km.TINY, mode, seed=11, **kw)
    try:
        tokens = [5, 17, 300, 42, 7, 199, 63, 250, 11, 90, 3, 3, 18, 77, 123, 9, 311, 64, 128, 255,
                  1, 0, 319, 200, 100, 50, 25, 12, 6, 3, 2, 1, 4, 8, 16, 32, 64, 96, 160, 224]   # crosses a 32-position tile
        want = np.stack([ref.forward_token(t, threads=2) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)
        for t in range(len(tokens)):
            assert np.array_equal(got[t], want[t]), (mode, t, float(np.max(np.abs(got[t] - want[t]))))
        c = spec["cfg"]
        for l in range(c["layers"]):
            for pos in range(len(tokens)):
                for kvh in range(c["n_kv"]):
                    gk, gks, gv, gvs = eng.read_kv(l, kvh, pos)
                    wk, wks, wv, wvs = ref.read_kv(l, kvh, pos)
                    assert np.array_equal(gk, wk) and np.array_equal(gv, wv) and gks == wks and gvs == wvs, (l, pos, kvh)
        assert np.array_equal(eng.read_hidden(), ref.tap_hidden()[-1])      # hidden state before the final norm
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("cfg,mode,kw", [(km.TINY, "b4", {}), (km.TINY, "nf4g128", dict(qkv_bias=True, qk_norm=True)),
                                         (dict(hidden=256, layers=2, n_q=4, n_kv=2, head_dim=128, inter=512, vocab=512, max_seq=80, eps=1e-6, theta=1e6),
                                          "b5", dict(qk_norm=True))])
def test_nf4_kv_cache_logits_and_entries(ctx, oracle, cfg, mode, kw, decode_path):
    """kv_bits = 4: NF4 Hadamard cache (refined bf16 scale per 64 values).  Entries, logits and greedy tokens are identical."""
    cfg = dict(cfg, kv_bits=4)
    spec, eng, ref = make(ctx, oracle, cfg, mode, seed=13, **kw)
    try:
        rng = np.random.Generator(np.random.PCG64(5))
        tokens = [int(t) for t in rng.integers(0, cfg["vocab"], 45)]
        want = np.stack([ref.forward_token(t, threads=2) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)
        assert np.array_equal(got, want)
        for l in range(cfg["layers"]):
            for pos in (0, 1, 31, 44):
                for kvh in range(cfg["n_kv"]):
                    g, w = eng.read_kv(l, kvh, pos), ref.read_kv(l, kvh, pos)
                    assert all(np.array_equal(a, b) for a, b in zip(g, w)), (l, pos, kvh)
        assert eng.kv_bytes(10) == 10 * 2 * cfg["layers"] * cfg["n_kv"] * (cfg["head_dim"] // 2 + 2 * (cfg["head_dim"] // 64))
        ref.reset()
        _greedy_check(eng, ref, tokens[:6], 25)
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("mode,moe,kw", [
    ("nf4g128", dict(layers=[0, 2], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2), dict(qk_norm=True)),        # Qwen3-MoE style: nf3 experts
    ("b5", dict(layers=[1], n_experts=16, top_k=4, d_ff=128, bits=4, sgc=1, norm_topk=False, bias=True), dict(qkv_bias=True)),
    ("nf4", dict(layers=[0, 1, 2], n_experts=6, top_k=6, d_ff=64, bits=5, sgc=2), {}),                          # every expert routed
    ("b4", dict(layers=[2], n_experts=4, top_k=2, d_ff=128, bits=2, sgc=2), {}),                                # E8Q2 experts
    ("nf4g128", dict(layers=[1, 2], n_experts=8, top_k=3, d_ff=64, bits=4, sgc=1, scoring=1), {}),               # top-k softmax router (GptOss)
    ("b5", dict(layers=[0], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=1, scoring=2, bias=True), {}),             # sigmoid router
    ("nf4g128", dict(layers=[0, 2], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2, shared=128), {}),                # shared expert with a sigmoid gate (Qwen2-MoE)
    ("b5", dict(layers=[1], n_experts=8, top_k=3, d_ff=64, bits=4, sgc=1, shared=64, shared_gate=False), dict(qkv_bias=True)),   # ungated shared expert
])
def test_sparse_moe_layers_match_oracle(ctx, oracle, mode, moe, kw):
    """Router (softmax, top-k, renormalisation, expert order), .k2tm expert records, expert SwiGLU and the weighted sum."""
    spec, eng, ref = make(ctx, oracle, km.MOE_TINY, mode, seed=17, moe=moe, **kw)
    try:
        rng = np.random.Generator(np.random.PCG64(9))
        tokens = [int(t) for t in rng.integers(0, km.MOE_TINY["vocab"], 23)]
        want = np.stack([ref.forward_token(t, threads=2) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)
        assert np.array_equal(got, want)
        for l in moe["layers"]:
            ge, gw = eng.read_routes(l)
            we, ww = ref.last_routes(l)
            assert np.array_equal(ge, we) and np.array_equal(gw, ww), (l, ge, we)
            assert len(ge) == min(moe["top_k"], moe["n_experts"]) and list(ge) == sorted(ge)
        assert len(eng.read_routes([l for l in range(3) if l not in moe["layers"]][0])[0]) == 0 if len(moe["layers"]) < 3 else True
        assert np.array_equal(eng.read_hidden(), ref.tap_hidden()[-1])
        ref.reset()
        _greedy_check(eng, ref, tokens[:5], 30)
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("batch", [16, 48, 112])
def test_prompt_batch_size_does_not_change_results(ctx, oracle, monkeypatch, batch):
    """The engine cuts a prompt into batches of KRONOS_CUDA_PROMPT_BATCH tokens (default 256): whatever the size - several batches
    per prompt, a ragged last one, a batch that crosses position 512 where the attention kernels change, token tiles of every
    width in the tensor-core launches - logits of every position and the cache rows equal the oracle's token-by-token run."""
    monkeypatch.setenv("KRONOS_CUDA_PROMPT_BATCH", str(batch))
    rng = np.random.Generator(np.random.PCG64(batch))
    cases = [(km.TINY, "b5", dict(qkv_bias=True), 75), (LONG, "nf4g128", {}, LONG["max_seq"] - 1),
             (km.MOE_TINY, "nf4g128", dict(moe=dict(layers=[0, 2], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2, shared=128)), 75)]
    for cfg, mode, kw, n in cases:
        spec, eng, ref = make(ctx, oracle, cfg, mode, seed=13, **kw)
        try:
            tokens = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
            want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
            got = eng.forward_token_ids(tokens, want_all=True)
            bad = [t for t in range(n) if not np.array_equal(got[t], want[t])]
            assert not bad, (cfg is LONG, mode, bad[:5], len(bad))
            for pos in (0, n // 2, n - 1):
                for kvh in range(cfg["n_kv"]):
                    assert all(np.array_equal(a, b) for a, b in zip(eng.read_kv(cfg["layers"] - 1, kvh, pos), ref.read_kv(cfg["layers"] - 1, kvh, pos)))
        finally:
            eng.close(); ref.close()


def test_host_embeddings_equal_device_lookup(ctx, oracle):
    spec, eng, ref = make(ctx, oracle, km.TINY, "b5", seed=4)
    try:
        tokens = [9, 8, 7, 300, 2]
        emb = np.stack([ref.embed(t) for t in tokens])
        a = eng.forward_tokens(emb, want_all=True)
        b = eng.forward_token_ids(tokens, want_all=True)
        assert np.array_equal(a, b)                         # the device embedding lookup is the CPU's, bit for bit
        last = eng.forward_token_ids(tokens)
        assert np.array_equal(last, b[-1])
        # continuing at pos_start: same as one run
        eng.forward_token_ids(tokens[:3])
        c = eng.forward_token_ids(tokens[3:], pos_start=3, want_all=True)
        assert np.array_equal(c, b[3:])
    finally:
        eng.close(); ref.close()


def test_imported_session_continues_beyond_512_positions(ctx, oracle):
    """A session of 560 positions moved into a fresh engine (kv_import, then save / restore of a prefix snapshot): the rows the
    host wrote are also what the long-context value chains read (their block-transposed copy is rebuilt), so the engine goes
    on exactly as the oracle does."""
    import kronos_2t_b200 as k2
    spec, eng, ref = make(ctx, oracle, LONG4, "b5", seed=31)
    eng2 = k2.Engine(ctx, spec)
    try:
        rng = np.random.Generator(np.random.PCG64(8))
        tokens = [int(t) for t in rng.integers(0, LONG4["vocab"], 580)]
        for t in tokens[:560]:
            ref.forward_token(t, 4)
        blob = ref.kv_export(0, 560)
        eng2.kv_import(blob, 560)                                    # rows from the CPU engine
        want = np.stack([ref.forward_token(t, 4) for t in tokens[560:570]])
        assert np.array_equal(eng2.forward_token_ids(tokens[560:570], pos_start=560, want_all=True), want)
        snap = eng2.save_kv_prefix(570, 570)
        eng.restore_kv_prefix(snap)                                  # and through a prefix snapshot into another engine
        want = np.stack([ref.forward_token(t, 4) for t in tokens[570:580]])
        assert np.array_equal(eng.forward_token_ids(tokens[570:580], pos_start=570, want_all=True), want)
        got = eng.decode_greedy(int(np.argmax(want[-1])), 580, 8)
        tok, out = int(np.argmax(want[-1])), []
        for _ in range(8):
            tok = oracle.argmax(ref.forward_token(tok, 4)); out.append(tok)
        assert list(got) == out
    finally:
        eng.close(); eng2.close(); ref.close()


def _greedy_check(eng, ref, prompt, steps):
    want, want_logits = ref.greedy(prompt, steps, threads=8)
    if len(prompt) > 1:
        eng.forward_token_ids(prompt[:-1])
    got, got_logits = eng.decode_greedy(prompt[-1], len(prompt) - 1, steps + 1, want_logits=True)
    # decode_greedy returns the tokens chosen after each fed token: the first `steps` are the oracle's choices
    assert list(got[:steps]) == want, (list(got[:steps]), want)
    assert np.array_equal(got_logits, want_logits)


@pytest.fixture(params=["fused", "per-operator", "decode-kernel"])
def decode_path(request, monkeypatch):
    """Single-token steps run as a CUDA graph of GEMVs that build their own activations (norm / SwiGLU / embedding
    prologues; the default), as a graph of per-operator kernels (KRONOS_CUDA_FUSED=0 at engine creation), or - greedy
    decoding up to 512 positions, KRONOS_CUDA_MEGA=1 - in the whole-token cooperative kernel."""
    monkeypatch.setenv("KRONOS_CUDA_FUSED", "0" if request.param == "per-operator" else "1")
    monkeypatch.setenv("KRONOS_CUDA_MEGA", "1" if request.param == "decode-kernel" else "0")
    return request.param


@pytest.mark.parametrize("mode,kw", [("b4", {}), ("nf4g128", dict(qkv_bias=True)), ("b6", dict(qk_norm=True, tied=False)),
                                     ("nf3g128", dict(qk_norm=True)), ("b5", dict(modes=dict(gate_up="nf4", down="b6")))])
def test_greedy_matches_oracle_tiny(ctx, oracle, mode, kw, decode_path):
    spec, eng, ref = make(ctx, oracle, km.TINY, mode, seed=21, **kw)
    try:
        _greedy_check(eng, ref, [1, 2, 3, 4], 80)
        ref.reset()
        _greedy_check(eng, ref, [7], 40)                   # the engine restarts at position 0 without a reset call
    finally:
        eng.close(); ref.close()


HD128 = dict(hidden=256, layers=2, n_q=4, n_kv=1, head_dim=128, inter=512, vocab=512, max_seq=80, eps=1e-6, theta=1e6)
GROUP8 = dict(hidden=512, layers=1, n_q=8, n_kv=1, head_dim=64, inter=384, vocab=256, max_seq=300, eps=1e-5, theta=1e4)
LONG = dict(hidden=256, layers=1, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=256, max_seq=1200, eps=1e-5, theta=1e4)
LONG128 = dict(hidden=256, layers=1, n_q=2, n_kv=1, head_dim=128, inter=256, vocab=256, max_seq=800, eps=1e-5, theta=1e4)


@pytest.mark.parametrize("cfg,mode,kw", [(HD128, "b5", dict(qk_norm=True)), (HD128, "nf4g128", dict(qkv_bias=True)),
                                         (GROUP8, "b4", {})])
def test_head_dim_128_and_wide_groups(ctx, oracle, cfg, mode, kw):
    spec, eng, ref = make(ctx, oracle, cfg, mode, seed=5, **kw)
    try:
        n = min(cfg["max_seq"] - 2, 270)                   # GROUP8: crosses the 256-position score tile
        rng = np.random.Generator(np.random.PCG64(1))
        tokens = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)
        assert np.array_equal(got, want)
    finally:
        eng.close(); ref.close()


LONG4 = dict(hidden=256, layers=4, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=256, max_seq=1100, eps=1e-5, theta=1e4)
LONG_G7 = dict(hidden=256, layers=2, n_q=7, n_kv=1, head_dim=128, inter=256, vocab=256, max_seq=900, eps=1e-6, theta=1e6)


@pytest.mark.parametrize("cfg,mode,kv_bits,kw", [(LONG, "b4", 8, {}), (LONG128, "nf4g128", 8, {}), (LONG, "b5", 4, {}), (LONG128, "b4", 4, {}),
                                                 (LONG4, "nf4g128", 8, dict(qk_norm=True)), (LONG_G7, "b5", 8, dict(qkv_bias=True)),
                                                 (LONG4, "b4", 4, {})])
def test_long_context_attention_is_exact(ctx, oracle, cfg, mode, kv_bits, kw):
    """Beyond 512 positions the attention runs as scores / values kernels in the CPU's summation order: logits of every
    position, the attention output and the cache entries stay identical to the oracle (multi-layer models included, where
    a last-bit difference would grow through the int8 activations)."""
    cfg = dict(cfg, kv_bits=kv_bits)
    spec, eng, ref = make(ctx, oracle, cfg, mode, seed=8, **kw)
    try:
        n = cfg["max_seq"] - 1
        rng = np.random.Generator(np.random.PCG64(2))
        tokens = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
        want_attn = ref.tap_attention()
        got = eng.forward_token_ids(tokens, want_all=True)
        bad = [t for t in range(n) if not np.array_equal(got[t], want[t])]
        assert not bad, (bad[:5], len(bad))
        assert np.array_equal(eng.read_attention(), want_attn)
        for pos in (0, 511, 512, n - 1):
            for kvh in range(cfg["n_kv"]):
                for l in (0, cfg["layers"] - 1):
                    assert all(np.array_equal(a, b) for a, b in zip(eng.read_kv(l, kvh, pos), ref.read_kv(l, kvh, pos)))
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("cfg,mode,kv_bits", [(LONG, "b4", 8), (LONG128, "nf4g128", 8), (LONG, "b5", 4), (LONG128, "b4", 4)])
def test_split_kv_attention_on_request(ctx, oracle, cfg, mode, kv_bits):
    """KRONOS_CUDA_ENGINE_SPLIT_KV_ATTENTION: long contexts by the split-KV kernels.  Scores stay exact, partial sums are merged
    in split order: the attention output agrees to fp32 rounding (2e-6 of its largest element); a last-bit difference can
    move one int8 activation by a step, so logits are held to 1e-3 * max(1, max |cpu|) on at least 90 % of the positions
    of a one-layer model and to 1e-2 on all (the tolerance this mode is documented with); cache entries stay identical."""
    cfg = dict(cfg, kv_bits=kv_bits, split_kv_attention=True)
    spec, eng, ref = make(ctx, oracle, cfg, mode, seed=8)
    try:
        n = cfg["max_seq"] - 1
        rng = np.random.Generator(np.random.PCG64(2))
        tokens = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
        want_attn = ref.tap_attention()
        got = eng.forward_token_ids(tokens, want_all=True)
        assert np.array_equal(got[:512], want[:512])       # contexts of 1..512 positions: CPU order
        got_attn = eng.read_attention()
        assert np.max(np.abs(got_attn - want_attn)) <= 2e-6 * float(np.max(np.abs(want_attn)))
        err = np.array([float(np.max(np.abs(got[t] - want[t]))) / max(1.0, float(np.max(np.abs(want[t])))) for t in range(512, n)])
        assert np.mean(err <= TOL) >= 0.9 and err.max() <= 1e-2, (float(np.mean(err <= TOL)), float(err.max()))
        for pos in (0, 511, 512, n - 1):                   # a one-layer model: KV entries never depend on attention
            for kvh in range(cfg["n_kv"]):
                assert all(np.array_equal(a, b) for a, b in zip(eng.read_kv(0, kvh, pos), ref.read_kv(0, kvh, pos)))
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("cfg,mode,kw", [(HD128, "b5", dict(qk_norm=True)), (GROUP8, "nf4g128", dict(qkv_bias=True))])
def test_greedy_head_dim_128_and_wide_groups(ctx, oracle, cfg, mode, kw, decode_path):
    spec, eng, ref = make(ctx, oracle, cfg, mode, seed=6, **kw)
    try:
        _greedy_check(eng, ref, [3, 1, 4, 1, 5, 9, 2, 6], min(cfg["max_seq"] - 10, 262))
    finally:
        eng.close(); ref.close()


def test_greedy_crosses_512_positions(ctx, oracle, decode_path):
    """Up to position 512 the single fused attention kernel decodes, beyond it the scores / values kernels: the token
    streams and the last logits are the oracle's, also for 128 steps that start beyond position 512 on a 4-layer model."""
    if decode_path == "decode-kernel":
        pytest.skip("the whole-token kernel serves contexts up to 512 positions")
    spec, eng, ref = make(ctx, oracle, LONG4, "b4", seed=9)
    try:
        rng = np.random.Generator(np.random.PCG64(3))
        prompt = [int(t) for t in rng.integers(0, LONG4["vocab"], 470)]
        want, want_logits = ref.greedy(prompt, 80 + 128, threads=4)
        eng.forward_token_ids(prompt[:-1])
        a = eng.decode_greedy(prompt[-1], 469, 30)                  # positions 469..498
        b = eng.decode_greedy(int(a[-1]), 499, 50)                  # 499..548: crosses 512
        c, logits = eng.decode_greedy(int(b[-1]), 549, 129, want_logits=True)     # 128 steps that all lie beyond 512
        got = list(a) + list(b) + list(c[:128])
        assert got == want
        assert np.array_equal(logits, want_logits)
    finally:
        eng.close(); ref.close()


_SMOL_WANT = {}


def test_greedy_smollm2_135m_shape_128_steps(ctx, oracle, decode_path):
    """BASELINE configs[0]: the SmolLM2-135M shape (30 layers, hidden 576, 9/3 heads, vocab 49152, tied), b4 planes with b5 for
    qkv / o / down here, int8 KV: a 128-token seeded prompt, then 128 greedy steps - the token stream and the last logits are
    the oracle's.  (Synthetic N(0, 0.02) weights through the oracle's RTN quantizer.)"""
    spec, eng, ref = make(ctx, oracle, km.SMOL_135M, "b4", seed=2, modes=dict(qkv="b5", o="b5", down="b5"))
    try:
        prompt = [int(t) for t in np.random.Generator(np.random.PCG64(128)).integers(0, km.SMOL_135M["vocab"], 128)]
        if "want" not in _SMOL_WANT:                        # the oracle's 256 tokens once for all decode paths
            _SMOL_WANT["want"] = ref.greedy(prompt, 128, threads=16)
        want, want_logits = _SMOL_WANT["want"]
        eng.forward_token_ids(prompt[:-1])
        got, got_logits = eng.decode_greedy(prompt[-1], 127, 129, want_logits=True)
        assert list(got[:128]) == want
        assert np.array_equal(got_logits, want_logits)
        assert eng.kv_bytes(256) == 256 * 2 * 30 * 3 * (64 + 4)
        files = sum(ly[k].file_bytes() for ly in spec["layers"] for k in ("qkv", "o", "gate_up", "down")) + spec["lm_head"].file_bytes()
        assert eng.weight_bytes == files
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("kv_bits", [8, 4])
def test_kv_blob_export_import_and_truncation(ctx, oracle, kv_bits):
    """KV blobs in the reference's position-major format move between the CPU engine and the device: equal bytes for the same
    prompt, a session restored from a CPU blob continues identically, and a truncated context is just an earlier pos_start."""
    cfg = dict(km.TINY, kv_bits=kv_bits)
    spec, eng, ref = make(ctx, oracle, cfg, "b5", seed=23, qkv_bias=True)
    try:
        rng = np.random.Generator(np.random.PCG64(4))
        tokens = [int(t) for t in rng.integers(0, cfg["vocab"], 30)]
        for t in tokens[:20]:
            ref.forward_token(t, 2)
        eng.forward_token_ids(tokens[:20])
        per_pos = 2 * cfg["layers"] * cfg["n_kv"] * ((cfg["head_dim"] + 4) if kv_bits == 8 else (cfg["head_dim"] // 2 + 2))
        assert eng.kv_bytes_per_pos == per_pos
        blob_cpu, blob_gpu = ref.kv_export(0, 20), eng.kv_export(0, 20)
        assert blob_gpu.size == 20 * per_pos and np.array_equal(blob_cpu, blob_gpu)
        assert np.array_equal(eng.kv_export(5, 9), blob_cpu[5 * per_pos:9 * per_pos])
        # a fresh engine restored from the CPU blob continues like the CPU engine
        import kronos_2t_b200 as k2
        eng2 = k2.Engine(ctx, spec)
        try:
            eng2.kv_import(blob_cpu, 20)
            want = np.stack([ref.forward_token(t, 2) for t in tokens[20:]])
            assert np.array_equal(eng2.forward_token_ids(tokens[20:], pos_start=20, want_all=True), want)
            # truncation: go back to position 12 and replay different tokens on both sides
            other = [int(t) for t in rng.integers(0, cfg["vocab"], 6)]
            ref.kv_import(blob_gpu[:12 * per_pos], 12)                 # the CPU engine restored from a device blob
            want = np.stack([ref.forward_token(t, 2) for t in other])
            assert np.array_equal(eng2.forward_token_ids(other, pos_start=12, want_all=True), want)
            with pytest.raises(k2.KronosCudaError, match="shorter"):
                eng2.kv_import(blob_cpu[:100], 20)
            with pytest.raises(k2.KronosCudaError, match="out of bounds"):
                eng2.kv_export(0, cfg["max_seq"] + 1)
        finally:
            eng2.close()
    finally:
        eng.close(); ref.close()


def test_engine_argument_errors(ctx, oracle):
    import kronos_2t_b200 as k2
    spec, eng, ref = make(ctx, oracle, km.TINY, "b4", seed=1)
    try:
        with pytest.raises(k2.KronosCudaError, match="max_seq_len"):
            eng.forward_token_ids([1] * (km.TINY["max_seq"] + 1))
        with pytest.raises(k2.KronosCudaError, match="out of range"):
            eng.forward_token_ids([km.TINY["vocab"]])
        with pytest.raises(k2.KronosCudaError, match="max_seq_len"):
            eng.decode_greedy(1, km.TINY["max_seq"] - 2, 5)
        bad = dict(spec); bad["cfg"] = dict(spec["cfg"], inter=km.TINY["inter"] * 2)
        with pytest.raises(k2.KronosCudaError, match="shape"):
            k2.Engine(ctx, bad)
        # the engine still works after rejected calls
        assert np.array_equal(eng.forward_token_ids([3]), ref.forward_token(3))
    finally:
        eng.close(); ref.close()
