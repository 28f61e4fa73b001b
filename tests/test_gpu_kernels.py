"""GPU parity tests: every kernel is called through the C ABI (host-buffer entry points) and
compared with the CPU oracle on the same seeded inputs.

Bar: bit-exact for the int8 activations, their scales and sums, for the int32 chunk dots, and -
because the kernels keep the reference's ascending-chunk fmaf order - for the fp32 outputs too
(np.array_equal, no tolerance).
"""
import numpy as np
import pytest

from k2t_rng import normal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import kronos_2t_b200 as k2
    c = k2.Context(0)
    yield c
    c.close()


def upload(ctx, m, interleave=False):
    if m.kind == 0:
        return ctx.upload_bipolar(m.rows, m.cols, m.planes, m.data, m.scales, interleave)
    return ctx.upload_nf(m.rows, m.cols, m.bits, m.sgc, m.codebook, m.pair, m.tail, interleave)


def random_bipolar(oracle, seed, rows, cols, planes):
    rng = np.random.Generator(np.random.PCG64(seed))
    u = rng.integers(0, 1 << planes, (rows, cols), dtype=np.uint8)
    sc = rng.integers(0x3800, 0x3C00, (rows, cols // 64)).astype(np.uint16)   # bf16 in [2^-15, 2^-7)
    return oracle.bipolar_from_codes(u, sc, planes)


def random_nf(oracle, seed, rows, cols, bits, sgc, codebook=None):
    rng = np.random.Generator(np.random.PCG64(seed))
    idx = rng.integers(0, 1 << bits, (rows, cols), dtype=np.uint8)
    n_sc = oracle.lib().k2o_nf_scale_count(rows, cols, sgc)
    sc = rng.integers(0x3800, 0x3C00, n_sc).astype(np.uint16)
    if codebook is None:
        codebook = np.array([-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127], np.int8) if bits == 4 \
            else np.array([-127, -79, -45, -14, 14, 45, 79, 127] + [0] * 8, np.int8)
    return oracle.nf_pack(idx, sc, bits, sgc, codebook)


# ----------------------------------------------------------------------------- K1
@pytest.mark.parametrize("cols", [64, 576, 2048, 18944])
def test_fwht_quant_bit_exact(ctx, oracle, cols):
    x = normal(cols, (3, cols))
    x[1, :64] = 0.0                       # a chunk that quantizes to zeros (scale 0, skipped by the GEMV)
    x[2, 5] = 300.0                       # outlier
    want = oracle.act_populate_fwht(x)
    q, s, m = ctx.fwht_quant(x)
    assert np.array_equal(q, want.q) and np.array_equal(s, want.scales) and np.array_equal(m, want.sums)
    assert s[1, 0] == 0.0 and not q[1, :64].any()


def test_fwht_quant_rmsnorm_and_chunk_offset(ctx, oracle):
    cols = 1536
    x = normal(7, (4, cols)) * np.float32(3.0)
    w = (np.float32(1.0) + normal(8, cols) * np.float32(0.2)).astype(np.float32)
    inv = np.array([oracle.inv_rms(x[t], 1e-5) for t in range(4)], np.float32)
    want = oracle.act_populate_fwht(x, w, inv)
    q, s, m = ctx.fwht_quant(x, w, inv)
    assert np.array_equal(q, want.q) and np.array_equal(s, want.scales) and np.array_equal(m, want.sums)
    # a column slice of a tensor-parallel rank uses the global chunk index (and blocks >= 256 use the generator)
    for chunk0 in (5, 300):
        want = oracle.act_populate_fwht(x[0], chunk0=chunk0)
        q, s, m = ctx.fwht_quant(x[0], chunk0=chunk0)
        assert np.array_equal(q, want.q) and np.array_equal(s, want.scales) and np.array_equal(m, want.sums)


# ----------------------------------------------------------------------------- GEMV, quantized weights
def _check_gemv(ctx, oracle, m, x, interleave=False):
    act = oracle.act_populate_fwht(x)
    dm = upload(ctx, m, interleave)
    try:
        out, dots = ctx.gemv(dm, act.q, act.scales, act.sums, want_dots=True)
    finally:
        dm.free()
    if m.kind == 0:
        want, want_dots = oracle.nibble4_gemv(oracle.nibble4_from_bipolar(m, interleave), act, want_dots=True)
    else:
        mm = oracle.nf_gate_up_interleave(m) if interleave else m
        want, want_dots = oracle.nf_gemv(mm, act, want_dots=True)
    assert np.array_equal(dots, want_dots), "int32 chunk dots differ"
    assert np.array_equal(out, want), "fp32 outputs differ"
    return out


@pytest.mark.parametrize("planes", [4, 5, 6])
@pytest.mark.parametrize("rows,cols", [(54, 192), (71, 576), (960, 576), (128, 1536)])
def test_bitplane_gemv_bit_exact(ctx, oracle, planes, rows, cols):
    m = oracle.bipolar_quantize_rtn(normal(rows + planes, (rows, cols), 0.02), planes)
    x = normal(rows * 3 + cols, cols)
    out = _check_gemv(ctx, oracle, m, x)
    ref = np.stack([oracle.ifwht64(oracle.bipolar_dequant_row(m, r)) for r in range(rows)]).astype(np.float64) @ x.astype(np.float64)
    assert np.dot(out[0], ref) / (np.linalg.norm(out[0]) * np.linalg.norm(ref)) > 0.9995


@pytest.mark.parametrize("bits,sgc", [(4, 1), (4, 2), (3, 1), (3, 2)])
@pytest.mark.parametrize("rows,cols", [(71, 192), (128, 576), (1536, 2048)])
def test_nf_gemv_bit_exact(ctx, oracle, bits, sgc, rows, cols):
    m = oracle.nf_quantize_rtn(normal(rows + bits + sgc, (rows, cols), 0.02), bits, sgc)
    _check_gemv(ctx, oracle, m, normal(rows + cols, cols))


@pytest.mark.parametrize("cb", [
    [-120, -90, -70, -50, -33, -20, -9, -1, 3, 14, 29, 47, 60, 80, 101, 127],          # asymmetric, sorted
    [29, -90, -70, 127, -33, -20, -9, -1, 3, 14, -120, 47, 60, 80, 101, -50],          # unsorted: indices re-ranked at upload
    [100, 101, 102, 103, 104, 105, 106, 107, 108, 109, 110, 111, 112, 113, 114, 115],  # two-table decode needs an offset
    [-127, -100, -50, 0, 20, 40, 60, 80, 81, 82, 83, 84, 85, 86, 87, 127],             # lower half spans > 127: general decode
])
@pytest.mark.parametrize("rows,cols", [(96, 256), (1024, 2048)])
def test_nf4_arbitrary_codebooks(ctx, oracle, cb, rows, cols):
    m = random_nf(oracle, 5, rows, cols, 4, 2, np.array(cb, np.int8))
    _check_gemv(ctx, oracle, m, normal(6, (2, cols)))
    _check_gemv(ctx, oracle, m, normal(7, cols))


NF5_POS = [3, 8, 13, 19, 24, 30, 36, 42, 49, 56, 64, 72, 82, 93, 107, 127]      # the reference's default NF5 magnitudes


@pytest.mark.parametrize("cb", [NF5_POS, [1, -2, 5, 9, 17, 21, 33, 40, 41, 59, 70, 77, 90, 100, 120, 127]])
@pytest.mark.parametrize("sgc,rows,cols", [(1, 71, 192), (2, 128, 576), (2, 1536, 2048)])
def test_nf5_gemv_bit_exact(ctx, oracle, cb, sgc, rows, cols):
    """5-bit codebook: index bit 4 picks the sign half of the mirrored 32-entry table (nf_expand_codebook32)."""
    m = random_nf(oracle, rows + sgc, rows, cols, 5, sgc, np.array(cb, np.int8))
    _check_gemv(ctx, oracle, m, normal(rows + cols, cols))
    _check_gemv(ctx, oracle, m, normal(3, (3, cols)))


@pytest.mark.parametrize("sgc,rows,cols", [(2, 71, 128), (2, 256, 1536), (1, 960, 576), (2, 3072, 2048)])
def test_e8q2_gemv_bit_exact(ctx, oracle, sgc, rows, cols):
    """E8 lattice codewords, 2 bits per weight: every (template, sign) byte pair, both cosets."""
    rng = np.random.Generator(np.random.PCG64(rows))
    tpl = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
    sgn = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
    tpl[0, :8], sgn[0, :8] = 0, 1                                   # the padding codeword (decodes to zeros)
    sc = rng.integers(0x3800, 0x3C00, oracle.lib().k2o_nf_scale_count(rows, cols, sgc)).astype(np.uint16)
    m = oracle.e8q2_pack(tpl, sgn, sc, sgc)
    _check_gemv(ctx, oracle, m, normal(rows + 1, cols))
    _check_gemv(ctx, oracle, m, normal(rows + 2, (4, cols)))


@pytest.mark.parametrize("n_tok", [2, 3, 4, 7, 8, 15])
def test_batch_gemv_matches_oracle(ctx, oracle, n_tok):
    # batch forms: same per-(row, token) arithmetic as the single-token kernel
    rows, cols = 54, 1536
    x = normal(n_tok, (n_tok, cols))
    x[n_tok - 1, 128:192] = 0.0
    for m in (oracle.bipolar_quantize_rtn(normal(1, (rows, cols), 0.02), 5),
              oracle.nf_quantize_rtn(normal(2, (rows, cols), 0.02), 4, 2)):
        _check_gemv(ctx, oracle, m, x)


def _wide_matrix(oracle, fmt, rows, cols):
    if fmt.startswith("b"):
        return oracle.bipolar_quantize_rtn(normal(rows + cols, (rows, cols), 0.02), int(fmt[1]))
    if fmt == "e8q2":
        rng = np.random.Generator(np.random.PCG64(rows + cols))
        tpl = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
        sgn = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
        sc = rng.integers(0x3800, 0x3C00, oracle.lib().k2o_nf_scale_count(rows, cols, 2)).astype(np.uint16)
        return oracle.e8q2_pack(tpl, sgn, sc, 2)
    bits, sgc = {"nf3": (3, 1), "nf4": (4, 1), "nf4g128": (4, 2), "nf5g128": (5, 2)}[fmt]
    return oracle.nf_quantize_rtn(normal(rows + cols + bits, (rows, cols), 0.02), bits, sgc)


@pytest.mark.parametrize("fmt", ["b4", "b5", "b6", "nf3", "nf4", "nf4g128", "nf5g128", "e8q2"])
@pytest.mark.parametrize("rows,cols,n_tok", [(54, 192, 16), (71, 1536, 17), (300, 2112, 33), (128, 576, 64), (260, 4160, 100)])
def test_wide_batch_gemm_on_tensor_cores(ctx, oracle, fmt, rows, cols, n_tok):
    """Batches of sixteen tokens and more take the tensor-core kernel (exact int32 chunk dots by tcgen05.mma, the fp32 chains in
    chunk order): outputs equal the oracle's batch form bit for bit - odd row counts, partial token tiles, more than one pass
    of 32 chunks, whole chunks of zero activations for some tokens (their chain steps are skipped)."""
    m = _wide_matrix(oracle, fmt, rows, cols)
    x = normal(n_tok * 7 + rows, (n_tok, cols))
    x[n_tok - 1, 64:128] = 0.0
    x[n_tok // 2, :] = 0.0
    if cols > 1024:
        x[:, 960:1024] = 0.0
    act = oracle.act_populate_fwht(x)
    dm = upload(ctx, m)
    try:
        before = ctx.launch_count
        out = ctx.gemv(dm, act.q, act.scales, act.sums)
        assert ctx.launch_count - before == 1, "one launch for the whole batch"
    finally:
        dm.free()
    want = oracle.nibble4_gemv(oracle.nibble4_from_bipolar(m, False), act) if m.kind == 0 else oracle.nf_gemv(m, act)
    assert np.array_equal(out, want)


@pytest.mark.parametrize("rows", [71, 128])
@pytest.mark.parametrize("bits,sgc", [(3, 1), (3, 2), (4, 1), (4, 2), (5, 1), (5, 2)])
def test_reference_nf_sdot_case(ctx, oracle, rows, bits, sgc):
    """The reference's NF kernel test case (test_nf3_nf4_sdot_neon_scalar_parity_and_quality, src/kernels/simd_lut.rs:9137-9319:
    its LCG weights and activations, 256 columns, 71 / 128 rows, bits 3-5, scale groups of 1 and 2 chunks) and its batch leg
    (15 tokens against the single-token kernel), bit for bit on the device."""
    import k2t_refgen as rg
    m = oracle.nf_quantize_rtn(rg.sample_weights(rows, 256), bits, sgc)
    one = _check_gemv(ctx, oracle, m, rg.sample_x(4242 + bits * 10 + sgc, 256))
    xs = np.stack([rg.sample_x(9000 + t, 256) for t in range(15)])
    batch = _check_gemv(ctx, oracle, m, xs)
    dm = upload(ctx, m)
    try:
        for t in (0, 7, 14):
            act = oracle.act_populate_fwht(xs[t])
            assert np.array_equal(ctx.gemv(dm, act.q, act.scales, act.sums).reshape(-1), batch[t])
    finally:
        dm.free()
    assert one.shape[-1] == rows


def test_gate_up_interleave_upload(ctx, oracle):
    rows, cols = 256, 576
    _check_gemv(ctx, oracle, oracle.bipolar_quantize_rtn(normal(3, (rows, cols), 0.02), 4), normal(4, cols), interleave=True)
    _check_gemv(ctx, oracle, oracle.nf_quantize_rtn(normal(5, (rows, cols), 0.02), 4, 2), normal(6, cols), interleave=True)


def test_linear_end_to_end(ctx, oracle):
    rows, cols = 576, 1536
    m = oracle.bipolar_quantize_rtn(normal(11, (rows, cols), 0.02), 4)
    x = normal(12, (5, cols))
    dm = upload(ctx, m)
    got = ctx.linear(dm, x)
    dm.free()
    want = oracle.nibble4_gemv(oracle.nibble4_from_bipolar(m), oracle.act_populate_fwht(x))
    assert np.array_equal(got, want)


# ----------------------------------------------------------------------------- sweep shapes (random codes)
@pytest.mark.parametrize("fmt,sgc", [("b4", 1), ("b5", 1), ("b6", 1), ("nf4", 2), ("nf4", 1), ("nf3", 2), ("nf5", 2)])
@pytest.mark.parametrize("cols,rows", [(3584, 70), (2560, 130), (18944, 36), (4736, 513)])
def test_wide_ragged_matrices_bit_exact(ctx, oracle, fmt, sgc, cols, rows):
    """Several pass tiles with a ragged last one (56 = 32 + 24 chunks, 40 = 32 + 8, 296 = 9 x 32 + 8, 74 = 64 + 10),
    rows that are no multiple of 4, scale groups of two chunks: 1 and 4 tokens per launch against the oracle."""
    if fmt[0] == "b":
        m = random_bipolar(oracle, rows + cols, rows, cols, int(fmt[1]))
    elif fmt == "nf5":
        m = random_nf(oracle, rows + cols, rows, cols, 5, sgc, np.array(NF5_POS, np.int8))
    else:
        m = random_nf(oracle, rows + cols, rows, cols, int(fmt[2]), sgc)
    x = normal(rows, (4, cols))
    x[2, 64 * 33:64 * 34] = 0.0                      # a zero chunk in the second pass (skipped by the chain)
    act = oracle.act_populate_fwht(x)
    dm = upload(ctx, m)
    try:
        one = ctx.gemv(dm, act.q[0], act.scales[0], act.sums[0])
        four, dots = ctx.gemv(dm, act.q, act.scales, act.sums, want_dots=True)
    finally:
        dm.free()
    want, want_dots = oracle.gemv(m, act, want_dots=True, threads=8)
    assert np.array_equal(dots, want_dots)
    assert np.array_equal(four, want) and np.array_equal(one[0], want[0])


@pytest.mark.parametrize("fmt", ["b4", "b5", "b6", "nf4g128", "nf3g128"])
@pytest.mark.parametrize("cols,rows", [(2048, 2048), (2048, 8192), (8192, 2048), (2048, 49152)])
def test_sweep_shapes_bit_exact(ctx, oracle, fmt, cols, rows):
    if fmt[0] == "b":
        m = random_bipolar(oracle, rows + cols, rows, cols, int(fmt[1]))
    else:
        m = random_nf(oracle, rows + cols, rows, cols, int(fmt[2]), 2)
    x = normal(99, (4, cols))
    act = oracle.act_populate_fwht(x)
    dm = upload(ctx, m)
    try:
        assert dm.file_bytes == m.file_bytes()
        one = ctx.gemv(dm, act.q[0], act.scales[0], act.sums[0])
        four, dots = ctx.gemv(dm, act.q, act.scales, act.sums, want_dots=True)
    finally:
        dm.free()
    want, want_dots = oracle.gemv(m, act, want_dots=True, threads=8)
    assert np.array_equal(dots, want_dots)
    assert np.array_equal(four, want) and np.array_equal(one[0], want[0])
    # size-independent property: column sums of the chunk dots equal the dots of the column-summed codes
    if fmt[0] == "b":
        planes = int(fmt[1])
        u = np.stack([oracle.bipolar_unpack_row(m, r) for r in range(0, rows, max(1, rows // 64))]).astype(np.int64)
        sel = np.arange(0, rows, max(1, rows // 64))
        a = np.einsum("rci,ci->rc", u.reshape(len(sel), -1, 64), act.q[0].reshape(-1, 64).astype(np.int64))
        assert np.array_equal(dots[0][sel], (2 * a - ((1 << planes) - 1) * act.sums[0][None, :]).astype(np.int32))


def test_errors_are_reported_not_swallowed(ctx, oracle):
    import kronos_2t_b200 as k2
    m = oracle.bipolar_quantize_rtn(normal(1, (16, 64), 0.02), 4)
    dm = upload(ctx, m)
    with pytest.raises(k2.KronosCudaError):
        ctx.gemv(dm, np.zeros(64, np.int8), np.zeros(1, np.float32), None)     # bit-planes need xsum
    with pytest.raises(k2.KronosCudaError):
        ctx.upload_bipolar(16, 64, 7, m.data, m.scales)
    dm.free()
    before = ctx.launch_count
    ctx.fwht_quant(normal(2, 64))
    assert ctx.launch_count == before + 1


def test_linear_async_equals_linear(ctx, oracle):
    """Queued host-buffer calls (one wait at the end) give the bits of the synchronous call, in any interleaving of matrices."""
    import torch
    mats = [random_bipolar(oracle, 5, 130, 576, 5), random_nf(oracle, 6, 96, 2560, 4, 2), random_bipolar(oracle, 7, 64, 192, 4)]
    dms = [upload(ctx, m) for m in mats]
    try:
        xs = [torch.from_numpy(normal(10 + i, m.cols).astype(np.float32)).pin_memory() for i, m in enumerate(mats)]
        want = [ctx.linear(dm, x.numpy()) for dm, x in zip(dms, xs)]
        outs = [torch.empty(m.rows, dtype=torch.float32).pin_memory() for m in mats]
        for _ in range(3):
            for dm, x, out in zip(dms, xs, outs):
                ctx.linear_async_ptr(dm, x.data_ptr(), 1, out.data_ptr())
        ctx.synchronize()
        for w, out in zip(want, outs):
            assert np.array_equal(w.reshape(-1), out.numpy())
    finally:
        for dm in dms:
            dm.free()



def test_router_kernel_routes_and_survives_non_finite_inputs(ctx):
    """kronos_cuda_moe_route alone (the router indexes nothing by route id, so hostile inputs cannot fault here): ordinary
    inputs give distinct ascending ids whose renormalised weights sum to 1 and match a numpy softmax / top-k; NaN and Inf
    activations or weights still give ids inside [0, n_experts) - the expert kernels index their tables with them."""
    rng = np.random.Generator(np.random.PCG64(12))
    n_experts, hidden, k = 64, 256, 8
    w = (rng.standard_normal((n_experts, hidden)) * 0.02).astype(np.float32)
    x = rng.standard_normal(hidden).astype(np.float32)
    ids, wt = ctx.moe_route(w, x, k)
    logits = (w.astype(np.float64) @ x.astype(np.float64))
    p = np.exp(logits - logits.max()); p /= p.sum()
    want = np.sort(np.argsort(-p, kind="stable")[:k])
    assert list(ids) == list(want) and np.all(np.diff(ids.astype(np.int64)) > 0)
    assert abs(float(wt.sum()) - 1.0) < 1e-5 and np.allclose(wt, p[want] / p[want].sum(), rtol=1e-4)
    for scoring in (0, 1, 2):
        for poison in ("nan_x", "inf_x", "nan_w", "all_nan"):
            xx, ww = x.copy(), w.copy()
            if poison == "nan_x":
                xx[7] = np.nan
            elif poison == "inf_x":
                xx[3], xx[4] = np.inf, -np.inf
            elif poison == "nan_w":
                ww[5, :] = np.nan
            else:
                xx[:] = np.nan
            ids, wt = ctx.moe_route(ww, xx, k, scoring=scoring)
            assert len(ids) == k and np.all(ids < n_experts), (scoring, poison, ids)
