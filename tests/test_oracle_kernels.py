"""CPU tests of the oracle against independent restatements and the reference's own
cross-implementation equalities (generators and thresholds follow the reference tests cited).
"""
import numpy as np
import pytest

from k2t_rng import normal

M64 = (1 << 64) - 1


# ----------------------------------------------------------------------------- hadamard.rs
def _py_masks(b):
    """Independent big-int SplitMix64 restatement of hadamard.rs:29-44."""
    state = (0x9E3779B97F4A7C15 + b * 0xBF58476D1CE4E5B9) & M64
    out = []
    for _ in range(64):
        state = (state + 0x9E3779B97F4A7C15) & M64
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        z ^= z >> 31
        out.append(0x80000000 if z & 1 else 0)
    return np.array(out, np.uint32)


def _np_fwht(x, block0=0):
    x = np.asarray(x, np.float32).copy().reshape(-1, 64)
    for b in range(x.shape[0]):
        m = _py_masks(block0 + b)
        v = (x[b].view(np.uint32) ^ m).view(np.float32) * np.float32(0.125)
        h = 1
        while h < 64:
            v = v.reshape(-1, 2, h)
            v = np.stack([v[:, 0] + v[:, 1], v[:, 0] - v[:, 1]], axis=1).reshape(-1)
            h *= 2
        x[b] = v
    return x.reshape(-1)


def test_rademacher_masks_match_bigint_generator(oracle):
    for b in (0, 1, 7, 255, 256, 295, 100000):
        assert np.array_equal(oracle.rademacher_masks(b), _py_masks(b))
    # the masks are a fair coin, not a constant
    ones = sum(int((oracle.rademacher_masks(b) != 0).sum()) for b in range(64))
    assert 1800 < ones < 2300


def test_fwht64_orthogonality_and_inverse(oracle):
    # hadamard.rs:300-330 (same generators and thresholds)
    i = np.arange(128, dtype=np.float32)
    x = np.sin(i * np.float32(0.37)).astype(np.float32)
    x[17] = 80.0
    w = np.cos(i * np.float32(0.19)).astype(np.float32)
    w[99] = -25.0
    dot_before = float(np.dot(x.astype(np.float64), w.astype(np.float64)))
    xr, wr = oracle.fwht64(x), oracle.fwht64(w)
    assert np.array_equal(xr, _np_fwht(x))  # second implementation, bit-exact
    assert np.abs(xr).max() < 15.0
    assert abs(float(np.dot(xr.astype(np.float64), wr.astype(np.float64))) - dot_before) < 1e-3
    back = oracle.ifwht64(xr)
    assert np.abs(back - x).max() < 1e-4
    # block index offset = position in the vector
    assert np.array_equal(oracle.fwht64(x[64:], block0=1), xr[64:])


def test_bf16_round_to_nearest_even(oracle):
    assert oracle.f32_to_bf16(1.0) == 0x3F80
    assert oracle.f32_to_bf16(np.float32(1.0) + np.float32(2.0 ** -8)) == 0x3F80  # tie -> even
    assert oracle.f32_to_bf16(np.float32(1.0) + np.float32(3 * 2.0 ** -8)) == 0x3F82  # tie -> even (up)
    assert oracle.f32_to_bf16(np.float32(np.nan)) & 0x7FC0 == 0x7FC0
    for b in (0x0001, 0x3F80, 0xBF80, 0x7F7F):
        assert oracle.f32_to_bf16(oracle.bf16_to_f32(b)) == b


# ----------------------------------------------------------------------------- int8 activations
def _np_quant_blocks(v):
    v = v.reshape(-1, 64)
    q = np.zeros(v.shape, np.int8)
    s = np.zeros(v.shape[0], np.float32)
    m = np.zeros(v.shape[0], np.int32)
    for c in range(v.shape[0]):
        mx = np.float32(np.abs(v[c]).max())
        if mx <= np.finfo(np.float32).eps:
            continue
        inv = np.float32(127.0) / mx
        qi = np.rint(v[c] * inv).astype(np.int32)
        q[c], s[c], m[c] = qi.astype(np.int8), mx / np.float32(127.0), qi.sum()
    return q.reshape(-1), s, m


def test_int8_populate_matches_numpy(oracle):
    # simd_lut.rs:8842-8855: x_i = sin(0.37 i) * 3 with a zero chunk
    x = (np.sin(np.arange(256, dtype=np.float32) * np.float32(0.37)) * np.float32(3.0)).astype(np.float32)
    x[64:128] = 0.0
    a = oracle.act_populate(x)
    q, s, m = _np_quant_blocks(x)
    assert np.array_equal(a.q, q) and np.array_equal(a.scales, s) and np.array_equal(a.sums, m)
    assert a.scales[1] == 0.0 and a.sums[1] == 0 and not a.q[64:128].any()


def test_fused_rmsnorm_fwht_int8_bit_exact(oracle):
    # simd_lut.rs:8857-8905: fused == separate steps, bit for bit
    n = 576
    i = np.arange(n, dtype=np.float32)
    x = (np.sin(i * np.float32(0.113)) * np.float32(2.5)).astype(np.float32)
    x[100] = 40.0
    w = (np.float32(1.0) + np.cos(i * np.float32(0.071)) * np.float32(0.3)).astype(np.float32)
    inv = oracle.inv_rms(x, 1e-5)
    fused = oracle.act_populate_fwht(x, w, inv)
    xn = ((x * inv) * w).astype(np.float32)
    q, s, m = _np_quant_blocks(_np_fwht(xn))
    assert np.array_equal(fused.q[0], q) and np.array_equal(fused.scales[0], s) and np.array_equal(fused.sums[0], m)
    plain = oracle.act_populate_fwht(xn)
    assert np.array_equal(plain.q, fused.q) and np.array_equal(plain.scales, fused.scales)
    # sums really are the sums of q
    assert np.array_equal(fused.sums[0], fused.q[0].reshape(-1, 64).astype(np.int32).sum(1))


def test_inv_rms_close_to_float64(oracle):
    x = normal(3, 2048)
    ref = 1.0 / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5)
    assert abs(float(oracle.inv_rms(x, 1e-5)) - ref) < 1e-5 * ref


# ----------------------------------------------------------------------------- bipolar
@pytest.mark.parametrize("planes", [4, 5, 6])
def test_nibble4_repack_preserves_rows_and_gemv(oracle, planes):
    # simd_lut.rs:8744-8790
    rows, cols = 54, 192
    w = normal(10 + planes, (rows, cols), 0.02)
    m = oracle.bipolar_quantize_rtn(w, planes, threads=2)
    n4 = oracle.nibble4_from_bipolar(m)
    for r in range(rows):
        assert np.array_equal(oracle.bipolar_dequant_row(m, r), oracle.nibble4_dequant_row(n4, r))
        assert oracle.bipolar_unpack_row(m, r).max() < (1 << planes)
    x = normal(77, cols)
    act = oracle.act_populate_fwht(x)
    out, dots = oracle.nibble4_gemv(n4, act, want_dots=True)
    out_def, dots_def = oracle.bipolar_gemv_def(m, act)
    assert np.array_equal(dots[0], dots_def) and np.array_equal(out[0], out_def)
    # against the float weights (rotation preserves inner products): quality check
    ref = w.astype(np.float64) @ x.astype(np.float64)
    cos = np.dot(out[0], ref) / (np.linalg.norm(out[0]) * np.linalg.norm(ref))
    assert cos > (0.995 if planes == 4 else 0.998)
    # integer path vs dequantize-then-float-dot of the same quantized values: cos > 0.9999
    xr = oracle.fwht64(x)
    deq = np.stack([oracle.bipolar_dequant_row(m, r) for r in range(rows)]).astype(np.float64) @ xr.astype(np.float64)
    assert np.dot(out[0], deq) / (np.linalg.norm(out[0]) * np.linalg.norm(deq)) > 0.9999


def test_bipolar_quantizer_reconstruction(oracle):
    w = normal(5, (32, 128), 0.02)
    for planes, tol in ((4, 0.12), (5, 0.06), (6, 0.03)):
        m = oracle.bipolar_quantize_rtn(w, planes)
        deq = np.stack([oracle.ifwht64(oracle.bipolar_dequant_row(m, r)) for r in range(32)])
        rel = np.linalg.norm(deq - w) / np.linalg.norm(w)
        assert rel < tol, (planes, rel)


def test_nibble4_batch_matches_single_and_threads(oracle):
    # simd_lut.rs:8907-8940: rows=54, cols=1536, 15 tokens
    rows, cols, n = 54, 1536, 15
    m = oracle.bipolar_quantize_rtn(normal(21, (rows, cols), 0.02), 5)
    n4 = oracle.nibble4_from_bipolar(m)
    x = normal(22, (n, cols))
    x[3, 128:192] = 0.0  # one skipped chunk
    act = oracle.act_populate_fwht(x)
    batch = oracle.nibble4_gemv(n4, act, threads=3)
    for t in range(n):
        single = oracle.nibble4_gemv(n4, oracle.Act(act.q[t], act.scales[t], act.sums[t]))
        assert np.array_equal(batch[t], single[0])
    assert act.scales[3, 2] == 0.0


def test_nibble4_gate_up_interleave(oracle):
    rows, cols = 256, 128
    m = oracle.bipolar_quantize_rtn(normal(31, (rows, cols), 0.02), 4)
    act = oracle.act_populate_fwht(normal(32, cols))
    plain = oracle.nibble4_gemv(oracle.nibble4_from_bipolar(m), act)[0]
    inter = oracle.nibble4_gemv(oracle.nibble4_from_bipolar(m, True), act)[0]
    half = rows // 2
    for ic in range(half // 64):
        assert np.array_equal(inter[ic * 128: ic * 128 + 64], plain[ic * 64: ic * 64 + 64])
        assert np.array_equal(inter[ic * 128 + 64: ic * 128 + 128], plain[half + ic * 64: half + ic * 64 + 64])


# ----------------------------------------------------------------------------- NF / E8Q2
def test_codebook_constants_and_expand(oracle):
    import ctypes as C
    L = oracle.lib()
    nf4 = np.array((C.c_int8 * 16).in_dll(L, "K2O_NF4_DEFAULT"))
    nf3 = np.array((C.c_int8 * 16).in_dll(L, "K2O_NF3_DEFAULT"))
    nf5 = np.array((C.c_int8 * 16).in_dll(L, "K2O_NF5_DEFAULT_POS"))
    assert nf4.tolist() == [-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127]
    assert nf3.tolist()[:8] == [-127, -79, -45, -14, 14, 45, 79, 127] and not nf3[8:].any()
    assert nf5.tolist() == [3, 8, 13, 19, 24, 30, 36, 42, 49, 56, 64, 72, 82, 93, 107, 127]
    cb32 = oracle.nf_expand_codebook32(5, nf5)
    assert np.array_equal(cb32[16:], nf5) and np.array_equal(cb32[:16], -nf5[::-1])
    assert np.array_equal(oracle.nf_expand_codebook32(4, nf4)[:16], nf4)


def test_e8q2_decode_structure(oracle):
    assert not oracle.e8q2_decode_8d(0, 1).any()  # padding codeword, simd_lut.rs:4434
    seen = set()
    for tpl in range(256):
        for sgn in range(0, 256, 1):
            v = oracle.e8q2_decode_8d(tpl, sgn).astype(np.int32)
            assert np.abs(v).max() <= 96
            assert not (v % 16).any()
            y = v // 16
            even = ((tpl ^ sgn).bit_count() & 1) == 1
            if even:
                assert not (y % 2).any()
            else:
                assert (y % 2).all() and set(np.abs(y).tolist()) <= {1, 3}
                assert y.sum() % 4 == 0  # odd coset points lie on 2*E8
            seen.add(v.tobytes())
    assert len(seen) == 32768 + 4001  # all odd-coset words distinct; even coset has sign bits on zeros


def _nf_ref_dequant(idx, sc, bits, sgc, cb, rows, cols):
    cb32 = np.zeros(32, np.int8)
    if bits == 5:
        cb32[16:] = cb
        cb32[:16] = -cb[::-1]
    else:
        cb32[:16] = cb
    nc = cols // 64
    nsg = -(-nc // sgc)
    sc = sc.reshape(-1, nsg, 16)
    out = np.zeros((rows, cols), np.float32)
    for r in range(rows):
        for c in range(nc):
            d = (np.uint32(sc[r // 16, c // sgc, r % 16]) << 16).view(np.float32) if False else \
                np.array([int(sc[r // 16, c // sgc, r % 16]) << 16], np.uint32).view(np.float32)[0]
            out[r, c * 64:(c + 1) * 64] = cb32[idx[r, c * 64:(c + 1) * 64]].astype(np.float32) * d
    return out


@pytest.mark.parametrize("rows", [71, 128])
@pytest.mark.parametrize("bits", [3, 4, 5])
@pytest.mark.parametrize("sgc", [1, 2])
def test_nf_pack_dequant_gemv(oracle, rows, bits, sgc):
    # simd_lut.rs:9137-9319 (rows 71 has an odd tail stripe; cols=192 leaves a short last group at sgc=2)
    cols = 192
    w = normal(100 + bits * 10 + sgc, (rows, cols), 0.02)
    m, idx, sc = oracle.nf_quantize_rtn(w, bits, sgc, threads=2, return_indices=True)
    assert idx.max() < (1 << bits)
    ref = _nf_ref_dequant(idx, sc, bits, sgc, m.codebook, rows, cols)
    for r in range(rows):
        assert np.array_equal(oracle.nf_dequant_row(m, r), ref[r])
    x = normal(55, (3, cols))
    x[1, 64:128] = 0.0
    act = oracle.act_populate_fwht(x)
    out, dots = oracle.nf_gemv(m, act, want_dots=True, threads=2)
    cb32 = oracle.nf_expand_codebook32(bits, m.codebook).astype(np.int64)
    wi = cb32[idx].reshape(rows, cols // 64, 64)
    for t in range(3):
        want = np.einsum("rci,ci->rc", wi, act.q[t].reshape(-1, 64).astype(np.int64))
        assert np.array_equal(dots[t], want.astype(np.int32))
    # quality vs float weights
    reff = w.astype(np.float64) @ x[0].astype(np.float64)
    cos = np.dot(out[0], reff) / (np.linalg.norm(out[0]) * np.linalg.norm(reff))
    assert cos > {3: 0.96, 4: 0.99, 5: 0.997}[bits]
    # batch == single
    single = oracle.nf_gemv(m, oracle.Act(act.q[1], act.scales[1], act.sums[1]))
    assert np.array_equal(single[0], out[1])


def test_nf_codebook_fit_is_symmetric_and_monotone(oracle):
    w = normal(9, (600, 256), 0.02)
    for bits in (3, 4, 5):
        cb, top = oracle.nf_fit_codebook(w, bits, 2)
        if bits == 5:
            assert (np.diff(cb.astype(int)) > 0).all() and cb[15] == 127 and cb[0] >= 1
        else:
            half = 1 << (bits - 1)
            assert np.array_equal(cb[:half], -cb[half:2 * half][::-1])
            assert (np.diff(cb[:2 * half].astype(int)) > 0).all() and cb[2 * half - 1] == 127
        assert 1.5 < float(top) < 4.0


def test_e8q2_pack_and_gemv(oracle):
    rows, cols, sgc = 71, 128, 2
    rng = np.random.Generator(np.random.PCG64(4))
    tpl = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
    sgn = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
    ns, nsg = (rows + 15) // 16, 1
    sc = rng.integers(0x3800, 0x3C00, ns * nsg * 16).astype(np.uint16)
    m = oracle.e8q2_pack(tpl, sgn, sc, sgc)
    assert m.pair.size == (ns // 2) * (nsg * 64 + 2 * 2 * 256) and m.tail.size == nsg * 32 + 2 * 256
    wi = np.zeros((rows, cols), np.int64)
    for r in range(rows):
        for b in range(cols // 8):
            wi[r, b * 8:(b + 1) * 8] = oracle.e8q2_decode_8d(tpl[r, b], sgn[r, b])
    act = oracle.act_populate_fwht(normal(8, cols))
    out, dots = oracle.nf_gemv(m, act, want_dots=True)
    want = np.einsum("rci,ci->rc", wi.reshape(rows, -1, 64), act.q[0].reshape(-1, 64).astype(np.int64))
    assert np.array_equal(dots[0], want.astype(np.int32))
    d0 = oracle.nf_dequant_row(m, 70)
    s70 = np.array([int(sc[(70 // 16) * nsg * 16 + 70 % 16]) << 16], np.uint32).view(np.float32)[0]
    assert np.array_equal(d0, wi[70].astype(np.float32) * s70)


def test_nf_gate_up_interleave(oracle):
    rows, cols = 256, 128
    m = oracle.nf_quantize_rtn(normal(41, (rows, cols), 0.02), 4, 2)
    act = oracle.act_populate_fwht(normal(42, cols))
    plain = oracle.nf_gemv(m, act)[0]
    inter = oracle.nf_gemv(oracle.nf_gate_up_interleave(m), act)[0]
    half = rows // 2
    for ic in range(half // 64):
        assert np.array_equal(inter[ic * 128: ic * 128 + 64], plain[ic * 64: ic * 64 + 64])
        assert np.array_equal(inter[ic * 128 + 64: ic * 128 + 128], plain[half + ic * 64: half + ic * 64 + 64])


# ----------------------------------------------------------------------------- published sizes
def test_published_byte_counts(oracle):
    L = oracle.lib()

    def bip(rows, cols, planes):
        return L.k2o_bipolar_data_bytes(rows, cols, planes) + 2 * L.k2o_bipolar_scale_count(rows, cols)

    def nf(rows, cols, bits, sgc):
        return L.k2o_nf_pair_stream_bytes(rows, cols, bits, sgc) + L.k2o_nf_tail_stream_bytes(rows, cols, bits, sgc) + 16

    # SmolLM2-135M b4 = 68.1 MiB (reference BENCHMARKS.md:22)
    h, inter, v, layers = 576, 1536, 49152, 30
    total = layers * (bip(960, h, 4) + bip(h, h, 4) + bip(2 * inter, h, 4) + bip(h, inter, 4)) + bip(v, h, 4)
    assert total == 71_442_432 and round(total / 2 ** 20, 1) == 68.1
    # SmolLM2-1.7B nf4g128 = 842 MB (BENCHMARKS.md:101)
    h, inter, layers = 2048, 8192, 24
    total = layers * (nf(3 * h, h, 4, 2) + nf(h, h, 4, 2) + nf(2 * inter, h, 4, 2) + nf(h, inter, 4, 2)) + nf(v, h, 4, 2)
    assert total == 882_378_256 and round(total / 2 ** 20) == 842
    # sweep table: 2048x49152 b4 / nf4g128
    assert bip(49152, 2048, 4) == 53_477_376 and nf(49152, 2048, 4, 2) == 51_904_528
    # Nibble4 records carry the same bytes as the file layout
    assert L.k2o_nibble4_pair_bytes(2048, 2048, 5) == bip(2048, 2048, 5)


@pytest.mark.parametrize("rows", [71, 128])
@pytest.mark.parametrize("bits,sgc", [(3, 1), (3, 2), (4, 1), (4, 2), (5, 1), (5, 2)])
def test_reference_nf_sdot_case_scalar_parity(oracle, rows, bits, sgc):
    """The shapes, generators and tolerance of the reference's NF kernel test (test_nf3_nf4_sdot_neon_scalar_parity_and_quality,
    src/kernels/simd_lut.rs:9137-9319): 256 columns, 71 (odd stripe count) and 128 rows, bits 3 / 4 / 5, scale groups of 1 and 2
    chunks; the oracle's GEMV (NEON semantics: exact int32 chunk dots, fused multiply-add epilogue) against a scalar
    restatement of nf_sdot_stripe_range_scalar_raw (6459-6539: integer dot, (dot * xs) * ws accumulated with separate multiply and
    add) within 1e-4 * max(|y|, 1), for any thread split.  Weights are quantized round-to-nearest (the reference test compiles
    them with a calibration Hessian, which changes the codes, not the kernel arithmetic)."""
    import k2t_refgen as rg
    cols = 256
    w = rg.sample_weights(rows, cols)
    nf, idx, sc = oracle.nf_quantize_rtn(w, bits, sgc, return_indices=True)
    x = rg.sample_x(4242 + bits * 10 + sgc, cols)
    act = oracle.act_populate_fwht(x)
    y, dots = oracle.gemv(nf, act, want_dots=True)
    y, dots = y.reshape(rows), dots.reshape(rows, cols // 64)
    for threads in (2, 3, 5):
        assert np.array_equal(oracle.gemv(nf, act, threads=threads).reshape(rows), y)
    cb = oracle.nf_expand_codebook32(bits, nf.codebook).astype(np.int64)
    q, xs = act.q.reshape(-1).astype(np.int64), act.scales.reshape(-1)
    nsg = (cols // 64 + sgc - 1) // sgc
    want = np.zeros(rows, np.float32)
    for r in range(rows):
        f = np.float32(0.0)
        for c in range(cols // 64):
            dot = int(np.dot(cb[idx[r, c * 64:(c + 1) * 64]], q[c * 64:(c + 1) * 64]))
            assert dot == dots[r, c]
            ws = oracle.bf16_to_f32(sc[((r // 16) * nsg + c // sgc) * 16 + r % 16])
            f = np.float32(f + np.float32(np.float32(np.float32(dot) * xs[c]) * ws))
        want[r] = f
    assert np.all(np.abs(y - want) <= 1e-4 * np.maximum(np.abs(want), 1.0)), float(np.max(np.abs(y - want)))


@pytest.mark.parametrize("rows,cols,sgc", [(37, 128, 1), (64, 192, 2), (96, 576, 2)])
def test_nf4_embedding_table_quantizer(oracle, rows, cols, sgc):
    """NfSdotMatrix::from_bf16_u16_embeddings_nf4 (simd_lut.rs:5230-5495) against a numpy restatement of its per-group steps:
    scale0 = max|v| / 127, indices by the midpoint thresholds, least-squares scale rounded to bf16, indices again; then the
    decoded rows (row dequantization + inverse rotation, embed_token_into 8084-8087) track the bf16 table."""
    rng = np.random.Generator(np.random.PCG64(rows + cols))
    u = (rng.standard_normal((rows, cols)).astype(np.float32) * np.float32(0.05)).view(np.uint32)
    table = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)                    # bf16, round to nearest even
    table[3, :64] = 0                                     # an all-zero scale group: indices 8, scale 0
    to_f32 = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
    m = oracle.nf4_embed_from_bf16(table, sgc, threads=3)
    cb = np.array([-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127], np.float32)
    th = 0.5 * (cb[8:15] + cb[9:16])
    def quant4(v, inv):
        mag = np.searchsorted(th, np.abs(v) * np.float32(inv), side="right")
        return np.where(v >= 0, 8 + mag, 7 - mag)
    worst = 1.0
    for r in range(rows):
        x = oracle.fwht64(to_f32(table[r]))
        want = np.zeros(cols, np.float32)
        for c0 in range(0, cols, sgc * 64):
            g = x[c0:c0 + sgc * 64]
            mx = np.float32(np.max(np.abs(g)))
            if mx <= 1e-12:
                continue
            q = cb[quant4(g, np.float32(127.0) / mx)]
            wq, qq = np.float32(0), np.float32(0)
            for v, qf in zip(g, q):                       # sequential fp32 sums, as the reference loop
                wq = np.float32(wq + v * qf); qq = np.float32(qq + qf * qf)
            delta = oracle.bf16_to_f32(oracle.f32_to_bf16(np.float32(max(wq / qq, 0.0)) if qq > 0 else mx / np.float32(127.0)))
            inv = np.float32(1.0) / delta if delta > 1e-12 else np.float32(0)
            want[c0:c0 + sgc * 64] = cb[quant4(g, inv)] * delta
        got = oracle.nf_dequant_row(m, r)
        assert np.array_equal(got, want), r
        back = oracle.ifwht64(got)
        src = to_f32(table[r])
        if np.linalg.norm(src) > 0:
            worst = min(worst, float(np.dot(back, src) / (np.linalg.norm(back) * np.linalg.norm(src))))
    assert worst > 0.99
