"""The .k2tb dense container (RealLlamaEngine::save_bipolar / load_bipolar, real_llm.rs:3705-4186): host-side writer and
reader of the library, checked byte for byte against an independent parser written here from the format description, and
(GPU) a model loaded from the file against the same model passed in memory and the CPU oracle fed from the file."""
import struct

import numpy as np
import pytest

import k2t_models as km


def parse_independent(raw):
    """Minimal second reader: returns (version, mode_words, [per-layer dict of raw fields], tail dict)."""
    magics = {b"K2TBIPOLAR1\n": 1, b"K2TKRONOS2\n": 2, b"K2TKRONOS3\n": 3, b"K2TKRONOS4\n": 4, b"K2TKRONOS6\n": 6}
    version = next(v for m, v in magics.items() if raw.startswith(m))
    pos = len(next(m for m in magics if raw.startswith(m)))

    def u64():
        nonlocal pos
        v = struct.unpack_from("<Q", raw, pos)[0]; pos += 8
        return v

    def arr(dt):
        nonlocal pos
        n = u64()
        a = np.frombuffer(raw, dt, n, pos).copy(); pos += a.nbytes
        return a

    def blob(n):
        nonlocal pos
        b = raw[pos:pos + n]; pos += n
        return b

    def matrix():
        tag = u64() if version >= 2 else 0
        if tag == 0:
            rows, cols, planes = u64(), u64(), u64()
            return dict(tag=0, rows=rows, cols=cols, bits=planes, a=arr(np.uint8), b=arr(np.uint16))
        rows, cols, bits, sgc = u64(), u64(), u64(), u64()
        cb = np.frombuffer(blob(16), np.int8).copy()
        return dict(tag=2, rows=rows, cols=cols, bits=bits, sgc=sgc, cb=cb, a=arr(np.uint8), b=arr(np.uint8))

    mode = [u64() for _ in range(6)]
    layers = []
    for _ in range(u64()):
        ly = dict(input_norm=arr(np.float32), post_norm=arr(np.float32))
        if version >= 3:
            ly["qkv_bias"] = arr(np.float32)
        if version >= 6:
            ly["q_norm"], ly["k_norm"] = arr(np.float32), arr(np.float32)
        for k in ("qkv", "o", "gate_up", "down"):
            ly[k] = matrix()
        layers.append(ly)
    tail = dict(final_norm=arr(np.float32), lm_head=matrix(), embed_f32=arr(np.float32))
    if version >= 3:
        tail["embed_bf16"] = arr(np.uint16)
    if version >= 4 and u64() == 1:         # flag: an NF4-quantized embedding table follows
        tail["embed_nf4"] = matrix()
    assert pos == len(raw)
    return version, mode, layers, tail


def same_matrix(m, rec):
    if m.kind == 0:
        return rec["tag"] == 0 and (rec["rows"], rec["cols"], rec["bits"]) == (m.rows, m.cols, m.planes) and \
            np.array_equal(rec["a"], m.data) and np.array_equal(rec["b"], m.scales)
    return rec["tag"] == 2 and (rec["rows"], rec["cols"], rec["bits"], rec["sgc"]) == (m.rows, m.cols, m.bits, m.sgc) and \
        np.array_equal(rec["cb"], np.asarray(m.codebook, np.int8)) and np.array_equal(rec["a"], m.pair) and np.array_equal(rec["b"], m.tail)


CASES = [("b4", {}, 1, [0, 4, 0, 0, 0, 0]), ("nf4g128", {}, 2, [5, 4, 2, 0, 0, 0]), ("b5", dict(qkv_bias=True), 3, [0, 5, 0, 0, 0, 0]),
         ("nf3g128", dict(tied=False), 3, [5, 3, 2, 0, 0, 0]), ("b6", dict(qk_norm=True, qkv_bias=True, tied=False), 6, [0, 6, 0, 0, 0, 0]),
         ("nf4g128", dict(tied=False, embed_nf4=True), 4, [5, 4, 2, 0, 0, 0]), ("b5", dict(qk_norm=True, tied=False, embed_nf4=True), 6, [0, 5, 0, 0, 0, 0])]


@pytest.mark.parametrize("mode,kw,version,words", CASES)
def test_k2tb_write_read_round_trip(oracle, tmp_path, mode, kw, version, words):
    import kronos_2t_b200 as k2
    spec = km.build(oracle, km.TINY, mode, seed=31, **kw)
    path = tmp_path / f"kronos-{mode}.k2tb"
    k2.k2tb_save(path, spec, words)
    ver, mw, layers, tail = parse_independent(path.read_bytes())
    assert ver == version and mw == words and len(layers) == km.TINY["layers"]
    for ly, rec in zip(spec["layers"], layers):
        assert np.array_equal(rec["input_norm"], ly["input_norm"]) and np.array_equal(rec["post_norm"], ly["post_norm"])
        if version >= 3:
            assert np.array_equal(rec["qkv_bias"], ly["qkv_bias"] if ly["qkv_bias"] is not None else np.zeros(0, np.float32))
        if version >= 6:
            assert np.array_equal(rec["q_norm"], ly["q_norm"]) and np.array_equal(rec["k_norm"], ly["k_norm"])
        assert all(same_matrix(ly[k], rec[k]) for k in ("qkv", "o", "gate_up", "down"))
    assert np.array_equal(tail["final_norm"], spec["final_norm"]) and same_matrix(spec["lm_head"], tail["lm_head"]) and tail["embed_f32"].size == 0
    if version >= 3:
        want = np.zeros(0, np.uint16) if spec["embed_bf16"] is None else spec["embed_bf16"].reshape(-1)
        assert np.array_equal(tail["embed_bf16"], want)
    # and back through the library's reader
    got, ver2, mw2 = k2.k2tb_load(path, spec["cfg"], spec["rope"])
    assert ver2 == version and mw2 == words
    for a, b in zip(got["layers"], spec["layers"]):
        for k in ("input_norm", "post_norm", "qkv_bias", "q_norm", "k_norm"):
            assert (a[k] is None) == (b[k] is None) and (a[k] is None or np.array_equal(a[k], b[k])), k
        for k in ("qkv", "o", "gate_up", "down"):
            ma, mb = a[k], b[k]
            assert ma.kind == mb.kind and ma.file_bytes() == mb.file_bytes()
            assert np.array_equal(ma.data, mb.data) and np.array_equal(ma.scales, mb.scales) if ma.kind == 0 else \
                np.array_equal(ma.pair, mb.pair) and np.array_equal(ma.tail, mb.tail) and np.array_equal(ma.codebook, mb.codebook)
    assert (got["embed_bf16"] is None) == (spec["embed_bf16"] is None)
    assert ("embed_nf4" in tail) == (spec.get("embed_matrix") is not None) == (got.get("embed_matrix") is not None)
    if "embed_nf4" in tail:
        assert same_matrix(spec["embed_matrix"], tail["embed_nf4"])
        assert np.array_equal(got["embed_matrix"].pair, spec["embed_matrix"].pair) and np.array_equal(got["embed_matrix"].tail, spec["embed_matrix"].tail)
    # the CPU oracle fed from the file reproduces the in-memory model
    a, b = oracle.Model(got), oracle.Model(spec)
    for t in (3, 200, 17):
        assert np.array_equal(a.forward_token(t, 2), b.forward_token(t, 2))
    a.close(); b.close()


def test_k2tb_reader_rejects_malformed_files(oracle, tmp_path):
    import kronos_2t_b200 as k2
    spec = km.build(oracle, km.TINY, "b4", seed=1)
    path = tmp_path / "m.k2tb"
    k2.k2tb_save(path, spec, [0, 4, 0, 0, 0, 0])
    raw = path.read_bytes()
    bad = tmp_path / "bad.k2tb"
    for data, text in ((raw[:len(raw) // 2], "truncated"), (b"K2TWHATEVER\n" + raw[12:], "magic"), (raw + b"\0", "trailing"),
                       (b"K2TKRONOS5\n" + raw[12:], "implausible|truncated|exceeds|tag")):      # a dense body behind the MoE core magic
        bad.write_bytes(data)
        with pytest.raises(k2.KronosCudaError, match=text):
            k2.k2tb_load(bad, spec["cfg"], spec["rope"])
    with pytest.raises(k2.KronosCudaError, match="cannot open"):
        k2.k2tb_load(tmp_path / "missing.k2tb", spec["cfg"], spec["rope"])
    tagged = b"K2TKRONOS2\n" + raw[12:12 + 7 * 8]            # same header, then layer 0 ...
    pos = 12 + 7 * 8
    n = struct.unpack_from("<Q", raw, pos)[0]
    first_layer_norms = raw[pos:pos + 2 * (8 + 4 * n)]
    bad.write_bytes(tagged + first_layer_norms + struct.pack("<Q", 1) + raw[pos + len(first_layer_norms):])   # ... whose first matrix has tag 1
    with pytest.raises(k2.KronosCudaError, match="VQ2"):
        k2.k2tb_load(bad, spec["cfg"], spec["rope"])


@pytest.mark.gpu
@pytest.mark.parametrize("mode,kw,words", [("b4", {}, [0, 4, 0, 0, 0, 0]), ("nf4g128", dict(qk_norm=True, tied=False), [5, 4, 2, 0, 0, 0]),
                                           ("nf4g128", dict(tied=False, embed_nf4=True), [5, 4, 2, 0, 0, 0])])
def test_engine_from_k2tb_file(oracle, tmp_path, mode, kw, words):
    """Oracle and device load the same file: identical logits and greedy tokens."""
    import kronos_2t_b200 as k2
    spec = km.build(oracle, km.TINY, mode, seed=7, **kw)
    path = tmp_path / f"kronos-{mode}.k2tb"
    k2.k2tb_save(path, spec, words)
    loaded, _, _ = k2.k2tb_load(path, spec["cfg"], spec["rope"])
    ctx = k2.Context(0)
    eng, ref = k2.Engine(ctx, loaded), oracle.Model(loaded)
    try:
        tokens = [1, 5, 300, 17, 64, 200, 9]
        want = np.stack([ref.forward_token(t, 2) for t in tokens])
        assert np.array_equal(eng.forward_token_ids(tokens, want_all=True), want)
        nxt, out = int(np.argmax(want[-1])), []
        got = eng.decode_greedy(nxt, len(tokens), 12)
        logits = ref.forward_token(nxt, 2)
        for _ in range(11):
            out.append(oracle.argmax(logits)); logits = ref.forward_token(out[-1], 2)
        assert list(got[:11]) == out
    finally:
        eng.close(); ref.close(); ctx.close()


def test_moe_core_and_expert_shard_readers(oracle, tmp_path):
    """K2TKRONOS5 core + .k2tm shard: the library's readers return what an independent writer (tests/k2t_moe_files.py) put
    in - every vector, matrix, router and expert record, the shard header words, the skipped lookahead projector - and refuse
    malformed files.  No GPU needed."""
    import kronos_2t_b200 as k2
    import k2t_moe_files as mf
    moe = dict(layers=[0, 2], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2, bias=True, shared=128)
    spec = km.build(oracle, km.MOE_TINY, "nf4g128", seed=17, moe=moe, qk_norm=True, qkv_bias=True, tied=False)
    core, shard = str(tmp_path / "core.k2tb"), str(tmp_path / "experts.k2tm")
    words = mf.write_moe_files(core, shard, spec, [6, 4, 3, 2, 0, 0], lookahead_layers=(0,))
    cfg = dict(km.MOE_TINY, moe_top_k=2, moe_norm_topk=True)
    got, hdr, close = k2.moe_load(core, shard, cfg, spec["rope"])
    try:
        assert hdr == words == [2, 8, km.MOE_TINY["hidden"], 64, 2, spec["layers"][0]["moe"]["expert_bytes"], 3]
        for l, (a, b) in enumerate(zip(got["layers"], spec["layers"])):
            for k in ("input_norm", "post_norm", "qkv_bias", "q_norm", "k_norm"):
                assert np.array_equal(a[k], b[k]), (l, k)
            for k in ("qkv", "o"):
                assert np.array_equal(a[k].pair, b[k].pair) and np.array_equal(a[k].codebook, b[k].codebook) and a[k].sgc == b[k].sgc
            if b.get("moe"):
                ma, mb = a["moe"], b["moe"]
                assert np.array_equal(ma["router_w"].reshape(-1), np.asarray(mb["router_w"]).reshape(-1)) and np.array_equal(ma["router_bias"], mb["router_bias"])
                assert np.array_equal(ma["shard"], mb["shard"]) and ma["expert_bytes"] == mb["expert_bytes"]
                assert (ma["n_experts"], ma["d_ff"], ma["bits"], ma["sgc"], ma["top_k"]) == (8, 64, 3, 2, 2)
                sa, sb = ma["shared"], mb["shared"]             # the shared expert: two NF matrices and the gate weight
                assert np.array_equal(sa["gate_up"].pair, sb["gate_up"].pair) and np.array_equal(sa["down"].pair, sb["down"].pair)
                assert (sa["gate_up"].rows, sa["down"].cols) == (256, 128) and np.array_equal(sa["gate_w"], sb["gate_w"])
            else:
                assert np.array_equal(a["gate_up"].pair, b["gate_up"].pair) and np.array_equal(a["down"].pair, b["down"].pair)
        assert np.array_equal(got["final_norm"], spec["final_norm"]) and np.array_equal(got["embed_bf16"], np.asarray(spec["embed_bf16"]).reshape(-1))
        assert np.array_equal(got["lm_head"].pair, spec["lm_head"].pair)
    finally:
        close()
    raw = open(shard, "rb").read()
    bad = str(tmp_path / "bad.k2tm")
    open(bad, "wb").write(raw[:-16384])                                   # a record page missing
    with pytest.raises(k2.KronosCudaError, match="file size"):
        k2.moe_load(core, bad, cfg, spec["rope"])
    open(bad, "wb").write(b"X" + raw[1:])
    with pytest.raises(k2.KronosCudaError, match="magic"):
        k2.moe_load(core, bad, cfg, spec["rope"])
    open(bad, "wb").write(raw[:100])
    with pytest.raises(k2.KronosCudaError, match="16 KiB"):
        k2.moe_load(core, bad, cfg, spec["rope"])
    craw = open(core, "rb").read()
    badc = str(tmp_path / "bad.k2tb")
    open(badc, "wb").write(craw[:len(craw) // 2])
    with pytest.raises(k2.KronosCudaError, match="truncated|exceeds"):
        k2.moe_load(badc, shard, cfg, spec["rope"])
    with pytest.raises(k2.KronosCudaError, match="top_k|K2TKRONOS5|core"):     # a dense container is not a MoE core
        dense = km.build(oracle, km.TINY, "b4", seed=1)
        k2.k2tb_save(str(tmp_path / "dense.k2tb"), dense, [0, 4, 0, 0, 0, 0])
        k2.moe_load(str(tmp_path / "dense.k2tb"), shard, cfg, spec["rope"])


@pytest.mark.gpu
@pytest.mark.parametrize("mode,moe,kw", [
    ("nf4g128", dict(layers=[0, 2], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2), dict(qk_norm=True, tied=False)),     # Qwen3-MoE style
    ("b5", dict(layers=[1], n_experts=16, top_k=4, d_ff=128, bits=4, sgc=1, norm_topk=False, bias=True), dict(qkv_bias=True)),
    ("nf4g128", dict(layers=[0, 1], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2, shared=64), {}),                      # with a gated shared expert
])
def test_moe_engine_from_core_and_shard_files(oracle, tmp_path, mode, moe, kw):
    """load_moe_from_files on the device: a sparse-MoE model written as K2TKRONOS5 core + .k2tm shard, read back through the
    library (the expert records stay in the mapped file until the engine has uploaded them) and run: logits, routes and
    the greedy stream equal the oracle's on the in-memory model."""
    import kronos_2t_b200 as k2
    import k2t_moe_files as mf
    spec = km.build(oracle, km.MOE_TINY, mode, seed=19, moe=moe, **kw)
    core, shard = str(tmp_path / "core.k2tb"), str(tmp_path / "experts.k2tm")
    mf.write_moe_files(core, shard, spec, [6, 4, moe["bits"], moe["sgc"], 0, 0], lookahead_layers=(moe["layers"][0],))
    cfg = dict(km.MOE_TINY, moe_top_k=moe["top_k"], moe_norm_topk=moe.get("norm_topk", True))
    loaded, hdr, close = k2.moe_load(core, shard, cfg, spec["rope"])
    ctx = k2.Context(0)
    try:
        eng = k2.Engine(ctx, loaded)
        close()                                   # the engine owns device copies: the mapping may go
        ref = oracle.Model(spec)
        try:
            rng = np.random.Generator(np.random.PCG64(4))
            tokens = [int(t) for t in rng.integers(0, km.MOE_TINY["vocab"], 21)]
            want = np.stack([ref.forward_token(t, threads=2) for t in tokens])
            assert np.array_equal(eng.forward_token_ids(tokens, want_all=True), want)
            for l in moe["layers"]:
                ge, gw = eng.read_routes(l)
                we, ww = ref.last_routes(l)
                assert np.array_equal(ge, we) and np.array_equal(gw, ww)
            tok, out = int(np.argmax(want[-1])), []
            got = eng.decode_greedy(tok, len(tokens), 20)
            for _ in range(20):
                tok = oracle.argmax(ref.forward_token(tok, threads=2)); out.append(tok)
            assert list(got) == out
        finally:
            eng.close(); ref.close()
    finally:
        ctx.close()
