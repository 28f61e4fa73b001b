"""Sliding-window + attention-sink KV ring on the device (QuantizedKvCache::new_with_opts / slot_of_pos /
causal_gqa_group_q4_or_window, src/model/real_llm.rs:1116-1122, 1235-1257, 8794-8988), against the CPU oracle.
The shapes and the 640-token wrap-around case follow the reference's own test
(test_phase2_nf4_untied_embeddings_k2tkronos4_and_q4_sliding_kv_parity, real_llm.rs:10479-10637: window 16, 4 sinks, 640 tokens
through a ring of 528 rows, can_truncate_kv_to(0 / 8 / 638)); where that test asks for a cosine above 0.9999 between batch
prefill and token-by-token decoding, the logits here must be identical to the oracle's at every position."""
import numpy as np
import pytest

import k2t_models as km

pytestmark = pytest.mark.gpu

REF_SHAPE = dict(hidden=256, layers=2, n_q=2, n_kv=1, head_dim=128, inter=512, vocab=192, max_seq=1024, eps=1e-6, theta=1e6)
GQA64 = dict(hidden=256, layers=2, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=256, max_seq=1400, eps=1e-5, theta=1e4)


@pytest.fixture(scope="module")
def ctx():
    import kronos_2t_b200 as k2
    c = k2.Context(0)
    yield c
    c.close()


def make(ctx, oracle, cfg, mode, **kw):
    import kronos_2t_b200 as k2
    spec = km.build(oracle, cfg, mode, seed=31, **kw)
    return spec, k2.Engine(ctx, spec), oracle.Model(spec)


@pytest.mark.parametrize("batch", [48, 112])
def test_ring_wraparound_with_other_prompt_batches(ctx, oracle, monkeypatch, batch):
    """The ring with prompt batches of other sizes than the default (KRONOS_CUDA_PROMPT_BATCH): batches that straddle the
    wrap-around and the end of the sinks give the oracle's logits all the same."""
    monkeypatch.setenv("KRONOS_CUDA_PROMPT_BATCH", str(batch))
    cfg = dict(GQA64, kv_bits=8, kv_window=40, kv_sinks=6)
    spec, eng, ref = make(ctx, oracle, cfg, "b5", tied=False)
    try:
        n = 700
        tokens = [(i * 7 + 3) % cfg["vocab"] for i in range(n)]
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)
        bad = [t for t in range(n) if not np.array_equal(got[t], want[t])]
        assert not bad, (bad[:5], len(bad))
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("cfg,mode,kv_bits,window,sinks,n", [(REF_SHAPE, "b4", 4, 16, 4, 640), (REF_SHAPE, "nf4g128", 8, 16, 4, 640),
                                                            (GQA64, "b5", 8, 600, 9, 1300), (GQA64, "b4", 4, 40, 0, 700)])
def test_ring_wraparound_matches_oracle(ctx, oracle, cfg, mode, kv_bits, window, sinks, n):
    cfg = dict(cfg, kv_bits=kv_bits, kv_window=window, kv_sinks=sinks)
    spec, eng, ref = make(ctx, oracle, cfg, mode, tied=False)
    try:
        assert eng.kv_sliding_window == (window, min(sinks, window // 2))
        assert eng.kv_rows == ref.kv_rows == min(sinks, window // 2) + (window - min(sinks, window // 2)) + 512
        tokens = [(i * 13 + 5) % cfg["vocab"] for i in range(n)]
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)            # batch prefill
        bad = [t for t in range(n) if not np.array_equal(got[t], want[t])]
        assert not bad, (bad[:5], len(bad))
        assert np.array_equal(eng.read_attention(), ref.tap_attention())
        # the ring rows of the last positions hold the oracle's entries
        for pos in (0, 1, n - 2, n - 1):
            for kvh in range(cfg["n_kv"]):
                assert all(np.array_equal(a, b) for a, b in zip(eng.read_kv(1, kvh, pos), ref.read_kv(1, kvh, pos)))
        # rollback guard (can_truncate_kv_to): back to the sinks or by at most the ring's slack
        s, slack = min(sinks, window // 2), 512
        for target in (0, s, s + 1, n - slack - 1, n - slack, n - 2, n):
            assert eng.can_truncate_kv_to(n, target) == ref.can_truncate_kv_to(target), target
        # greedy decoding continues on the ring, token for token
        tok, out = int(np.argmax(want[-1])), []
        steps = 24
        got_tokens, got_logits = eng.decode_greedy(tok, n, steps + 1, want_logits=True)
        logits = None
        for _ in range(steps + 1):
            logits = ref.forward_token(tok, threads=4)
            tok = oracle.argmax(logits)
            out.append(tok)
        assert list(got_tokens) == out and np.array_equal(got_logits, logits)
    finally:
        eng.close(); ref.close()


def test_reference_truncation_cases(ctx, oracle):
    """The three assertions of the reference test: at position 640 with window 16 / 4 sinks, 0 and 638 are reachable, 8 is not."""
    cfg = dict(REF_SHAPE, kv_bits=4, kv_window=16, kv_sinks=4)
    spec, eng, ref = make(ctx, oracle, cfg, "b4")
    try:
        assert eng.can_truncate_kv_to(640, 0) and not eng.can_truncate_kv_to(640, 8) and eng.can_truncate_kv_to(640, 638)
    finally:
        eng.close(); ref.close()


def test_reconfigure_kv_and_blobs_on_the_ring(ctx, oracle):
    """reconfigure_kv switches format and geometry on a live engine (fresh cache, position 0); a window too large for
    max_seq_len is ignored as in the reference; KV blobs of ring positions move between the CPU engine and the device."""
    cfg = dict(GQA64, kv_bits=8)
    spec, eng, ref = make(ctx, oracle, cfg, "b5", qkv_bias=True)
    try:
        tokens = [(i * 7 + 3) % cfg["vocab"] for i in range(620)]
        assert eng.kv_sliding_window is None and eng.kv_rows == cfg["max_seq"]
        eng.reconfigure_kv(4, 64, 8)
        assert ref.set_kv_window(4, 64, 8)
        assert eng.kv_sliding_window == (64, 8) and eng.kv_rows == 8 + 56 + 512
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens])
        got = eng.forward_token_ids(tokens, want_all=True)
        assert np.array_equal(got, want)
        per_pos = eng.kv_bytes_per_pos
        lo, hi = 620 - 56, 620                      # the live ring rows
        blob_gpu, blob_cpu = eng.kv_export(lo, hi), ref.kv_export(lo, hi)
        assert blob_gpu.size == 56 * per_pos and np.array_equal(blob_gpu, blob_cpu)
        assert np.array_equal(eng.kv_export(0, 8), ref.kv_export(0, 8))           # the sinks
        # a window that leaves no room (window + 512 >= max_seq_len) keeps the full context
        eng.reconfigure_kv(8, 1000, 4)
        assert not ref.set_kv_window(8, 1000, 4)
        assert eng.kv_sliding_window is None and eng.kv_rows == cfg["max_seq"]
        want = np.stack([ref.forward_token(t, threads=4) for t in tokens[:40]])
        assert np.array_equal(eng.forward_token_ids(tokens[:40], want_all=True), want)
    finally:
        eng.close(); ref.close()


@pytest.mark.parametrize("kv_bits,window", [(4, 0), (8, 0), (4, 16)])
def test_kv_prefix_snapshot_save_restore(ctx, oracle, kv_bits, window):
    """save_kv_prefix / restore_kv_prefix (real_llm.rs:5876-6155), following the reference test's sequence (10597-10604):
    snapshot after 12 of 24 prompt tokens, run something else, restore, replay the rest - the logits must be the original
    ones.  The device snapshot equals the CPU engine's byte for byte, and each side restores from the other's."""
    cfg = dict(REF_SHAPE, kv_bits=kv_bits, kv_window=window, kv_sinks=4 if window else 0)
    spec, eng, ref = make(ctx, oracle, cfg, "b4")
    try:
        prompt = [(i * 11 + 3) % cfg["vocab"] for i in range(24)]
        want = np.stack([ref.forward_token(t, threads=2) for t in prompt])
        got = eng.forward_token_ids(prompt, want_all=True)
        assert np.array_equal(got, want)
        ref.reset()
        for t in prompt[:12]:
            ref.forward_token(t, threads=2)
        eng.forward_token_ids(prompt[:12])
        snap_cpu, snap_gpu = ref.save_kv_prefix(12), eng.save_kv_prefix(12, 12)
        assert np.array_equal(snap_cpu, snap_gpu)
        rows = eng.kv_rows if window else 12
        per_row = 2 * cfg["layers"] * cfg["n_kv"] * ((cfg["head_dim"] // 2 + 2 * (cfg["head_dim"] // 64)) if kv_bits == 4 else (cfg["head_dim"] + 4))
        assert snap_gpu.size == 32 + rows * per_row
        eng.forward_token_ids([7], pos_start=12)                     # something else at position 12
        eng.restore_kv_prefix(snap_cpu)                                # the CPU engine's snapshot restores on the device
        rest = eng.forward_token_ids(prompt[12:], pos_start=12, want_all=True)
        assert np.array_equal(rest, want[12:])
        ref.forward_token(7, threads=2)
        ref.restore_kv_prefix(snap_gpu, 12)                            # and the device's on the CPU engine
        assert np.array_equal(np.stack([ref.forward_token(t, threads=2) for t in prompt[12:]]), want[12:])
        import kronos_2t_b200 as k2
        with pytest.raises(k2.KronosCudaError, match="not a KV prefix"):
            eng.restore_kv_prefix(np.zeros(64, np.uint8))
    finally:
        eng.close(); ref.close()
