"""CPU tests of the host-side repack (kronos_cuda_matrix_image) and of the kernels' decode logic.

The decode step of the GEMV kernel (k2t_gemv.cu: decode<FMT>) is re-enacted here word for word
in numpy, including the byte-permute selector tricks, and must reproduce the codes / centroids
the oracle reads out of the reference file formats.  No GPU is needed.
"""
import ctypes as C

import numpy as np
import pytest

import kronos_2t_b200 as k2
from k2t_rng import normal

U32 = np.uint32


def prmt(a, b, sel):
    """PTX prmt.b32 (generic mode): selector nibble = byte index 0..7 (+8: replicate the sign bit)."""
    src = [(a >> (8 * i)) & 0xFF for i in range(4)] + [(b >> (8 * i)) & 0xFF for i in range(4)]
    out = 0
    for i in range(4):
        nib = (sel >> (4 * i)) & 0xF
        v = src[nib & 7]
        if nib & 8:
            v = 0xFF if v & 0x80 else 0
        out |= v << (8 * i)
    return out


def _words(buf):
    return [int(x) for x in np.frombuffer(bytes(buf), dtype="<u4")]


def decode_cell(fmt, ca, cb, cb_words):
    """Returns the 64 weight bytes (unsigned for bit-planes, signed for NF) of one cell (row x chunk),
    given its plane A and plane B bytes, following decode<FMT> of k2t_gemv.cu."""
    a = _words(ca)
    h = _words(cb) if len(cb) else []
    u = [0] * 16
    M = 0xFFFFFFFF
    if fmt in ("bp4", "bp5", "bp6"):
        for i in range(8):
            u[2 * i], u[2 * i + 1] = a[i] & 0x0F0F0F0F, (a[i] >> 4) & 0x0F0F0F0F
        if fmt == "bp5":
            for j in range(8):
                for half in range(2):
                    hv = (h[half] << (4 - j)) & M if j <= 4 else h[half] >> (j - 4)
                    u[8 * half + j] |= hv & 0x10101010
        if fmt == "bp6":
            for v in range(4):
                u[4 * v + 0] |= ((h[v] << 4) & M) & 0x30303030
                u[4 * v + 1] |= ((h[v] << 2) & M) & 0x30303030
                u[4 * v + 2] |= h[v] & 0x30303030
                u[4 * v + 3] |= (h[v] >> 2) & 0x30303030
        dt = np.uint8
    elif fmt == "nf4":
        for i in range(8):
            x = a[i]
            lo3, hb = x & 0x77777777, x & 0x88888888
            hs = (hb << 4) & M
            m0, m1 = prmt(hs, hb, 0xD9C8), prmt(hs, hb, 0xFBEA)
            r_lo, r_hi = prmt(cb_words[0], cb_words[1], lo3), prmt(cb_words[2], cb_words[3], lo3)
            u[2 * i] = (r_lo & ~m0 & M) | (r_hi & m0)
            r_lo, r_hi = prmt(cb_words[0], cb_words[1], lo3 >> 16), prmt(cb_words[2], cb_words[3], lo3 >> 16)
            u[2 * i + 1] = (r_lo & ~m1 & M) | (r_hi & m1)
        dt = np.int8
    elif fmt == "nf3":
        W = a + h
        for i in range(6):
            s = W[i] & 0x77777777
            u[2 * i], u[2 * i + 1] = prmt(cb_words[0], cb_words[1], s), prmt(cb_words[0], cb_words[1], s >> 16)
        for hh in range(2):
            s = (W[3 * hh] >> 3) & 0x11111111
            s |= (W[3 * hh + 1] >> 2) & 0x22222222
            s |= (W[3 * hh + 2] >> 1) & 0x44444444
            u[12 + 2 * hh], u[13 + 2 * hh] = prmt(cb_words[0], cb_words[1], s), prmt(cb_words[0], cb_words[1], s >> 16)
        dt = np.int8
    elif fmt == "nf5":
        sel = lambda lo, hi, m: (lo & ~m & M) | (hi & m)
        for i in range(8):
            x = a[i]
            lo3, hb = x & 0x77777777, x & 0x88888888
            hs = (hb << 4) & M
            m0, m1 = prmt(hs, hb, 0xD9C8), prmt(hs, hb, 0xFBEA)
            hw = h[i // 4]
            for half, (l3, m) in enumerate(((lo3, m0), (lo3 >> 16, m1))):
                j = 2 * (i % 4) + half
                t = (((hw << (4 - j)) & M if j <= 4 else hw >> (j - 4)) & 0x10101010) >> 4
                bmask = (t * 0xFF) & M
                lo16 = sel(prmt(cb_words[0], cb_words[1], l3), prmt(cb_words[2], cb_words[3], l3), m)
                hi16 = sel(prmt(cb_words[4], cb_words[5], l3), prmt(cb_words[6], cb_words[7], l3), m)
                u[2 * i + half] = sel(lo16, hi16, bmask)
        dt = np.int8
    elif fmt == "e8q2":
        spread4 = lambda b: ((((b * 0x00204081) & M) & 0x01010101) * 0xFF) & M
        tab = cb_words                                     # the 28 even-coset template words
        for b in range(8):
            pair = (a[b // 2] >> (16 * (b % 2))) & 0xFFFF
            tpl, sgn = pair & 0xFF, pair >> 8
            tu, tv = tpl & 15, tpl >> 4
            if bin(tpl ^ sgn).count("1") & 1:
                ui = 16 + tu if tu < 12 <= tv else tu
                vi = 16 + tv if tv < 12 <= tu else tv
                mu, mv = tab[ui], tab[vi]
            else:
                mu, mv = (spread4(tu) & 0x20202020) + 0x10101010, (spread4(tv) & 0x20202020) + 0x10101010
            for k, (mag, bits4) in enumerate(((mu, sgn & 15), (mv, sgn >> 4))):
                sm = spread4(bits4)
                pos_b, neg_b = mag & ~sm & M, mag & sm
                u[2 * b + k] = sum((((pos_b >> (8 * q)) & 0xFF) - ((neg_b >> (8 * q)) & 0xFF)) % 256 << (8 * q) for q in range(4))   # __vsub4
        dt = np.int8
    else:
        raise ValueError(fmt)
    return np.array(u, dtype="<u4").view(np.uint8).view(dt)


CELL_BYTES = {"bp4": (16, 16, 0), "bp5": (16, 16, 8), "bp6": (16, 16, 16), "nf4": (16, 16, 0), "nf3": (16, 8, 0), "nf5": (16, 16, 8),
              "e8q2": (16, 0, 0)}
E8Q2_TEMPLATES = [(0, 0, 0, 0), (32, 32, 0, 0), (32, 0, 32, 0), (32, 0, 0, 32), (0, 32, 32, 0), (0, 32, 0, 32), (0, 0, 32, 32), (64, 0, 0, 0),
                  (0, 64, 0, 0), (0, 0, 64, 0), (0, 0, 0, 64), (32, 32, 32, 32), (32, 0, 0, 0), (0, 32, 0, 0), (0, 0, 32, 0), (0, 0, 0, 32),
                  (32, 32, 32, 0), (32, 32, 0, 32), (32, 0, 32, 32), (0, 32, 32, 32), (96, 0, 0, 0), (0, 96, 0, 0), (0, 0, 96, 0), (0, 0, 0, 96),
                  (64, 32, 32, 32), (32, 64, 32, 32), (32, 32, 64, 32), (32, 32, 32, 64)]


def split_image(fmt, image, rows, cols, nsg):
    """-> (plane A bytes [rows, nc, a], plane B bytes [rows, nc, b], scales [rows, nsg]) where A is what
    decode<FMT> sees first (32 B: planes 0+1 for 4-bit formats, 16 B for NF3) and B the rest.

    The image keeps every plane in pass tiles: tile p = chunks 32p.. of all rows (rows padded to 4 with zero cells),
    [row][n_p cells]; the scale plane likewise, 64 bytes x rows_pad per tile, row pitch = the tile's scale groups x 2
    bytes rounded up to 4 (a group that straddles two tiles is stored in both)."""
    nc = cols // 64
    sgc = -(-nc // nsg)
    assert -(-nc // sgc) == nsg
    rows_pad, n_pass = (rows + 3) & ~3, -(-nc // 32)
    off, planes = 0, []
    for cb in CELL_BYTES[fmt]:
        plane = np.zeros((rows, nc, cb), np.uint8)
        for p in range(n_pass):
            n = min(32, nc - 32 * p)
            t0 = off + p * rows_pad * 32 * cb
            tile = image[t0: t0 + rows_pad * n * cb].reshape(rows_pad, n, cb)
            assert not tile[rows:].any()
            plane[:, 32 * p: 32 * p + n] = tile[:rows]
        planes.append(plane)
        off += rows_pad * nc * cb
    scales = np.zeros((rows, nsg), np.uint16)
    seen = np.zeros(nsg, bool)
    for p in range(n_pass):
        n = min(32, nc - 32 * p)
        g_lo, g_hi = (32 * p) // sgc, (32 * p + n - 1) // sgc
        cnt = g_hi - g_lo + 1
        pitch = (cnt * 2 + 3) & ~3
        t0 = off + p * rows_pad * 64
        tile = image[t0: t0 + rows_pad * pitch].reshape(rows_pad, pitch)
        assert not tile[rows:].any() and not tile[:, cnt * 2:].any()
        vals = np.ascontiguousarray(tile[:rows, : cnt * 2]).view("<u2")
        for g in range(g_lo, g_hi + 1):
            if seen[g]:
                assert np.array_equal(scales[:, g], vals[:, g - g_lo])
            scales[:, g] = vals[:, g - g_lo]
            seen[g] = True
    assert seen.all()
    assert image.size == off + n_pass * rows_pad * 64 + 16
    if fmt in ("nf3", "e8q2"):
        return planes[0], planes[1], scales
    return np.concatenate([planes[0], planes[1]], axis=2), planes[2], scales


def image_rows(fmt, image, rows, cols, nsg, cb_words=None):
    """Decodes a whole device image into weight bytes [rows, cols] and bf16 scales [rows, nsg]."""
    pa, pb, scales = split_image(fmt, image, rows, cols, nsg)
    out = np.zeros((rows, cols), np.int16)
    for r in range(rows):
        for c in range(cols // 64):
            out[r, c * 64:(c + 1) * 64] = decode_cell(fmt, pa[r, c], pb[r, c], cb_words)
    return out, scales


@pytest.mark.parametrize("planes", [4, 5, 6])
@pytest.mark.parametrize("rows", [54, 64])
def test_bitplane_image_decodes_to_file_codes(oracle, planes, rows):
    cols = 192
    m = oracle.bipolar_quantize_rtn(normal(planes, (rows, cols), 0.02), planes, threads=2)
    image = k2.matrix_image(k2.bipolar_desc(rows, cols, planes, m.data, m.scales))
    codes, scales = image_rows(f"bp{planes}", image, rows, cols, cols // 64)
    sc_file = m.scales.reshape(-1, cols // 64, 16)
    for r in range(rows):
        assert np.array_equal(codes[r], oracle.bipolar_unpack_row(m, r))
        assert np.array_equal(scales[r], sc_file[r // 16, :, r % 16])


def test_wide_bitplane_image_spans_pass_tiles(oracle):
    """40 chunks = a full pass tile and a ragged one (8 chunks); 22 rows = padding rows in every tile."""
    rows, cols, planes = 22, 2560, 5
    m = oracle.bipolar_quantize_rtn(normal(77, (rows, cols), 0.02), planes, threads=2)
    image = k2.matrix_image(k2.bipolar_desc(rows, cols, planes, m.data, m.scales))
    codes, scales = image_rows("bp5", image, rows, cols, cols // 64)
    sc_file = m.scales.reshape(-1, cols // 64, 16)
    for r in range(rows):
        assert np.array_equal(codes[r], oracle.bipolar_unpack_row(m, r))
        assert np.array_equal(scales[r], sc_file[r // 16, :, r % 16])


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("rows,sgc,cols", [(71, 1, 192), (71, 2, 192), (128, 2, 192), (32, 3, 2560), (32, 2, 2304)])
def test_nf_image_decodes_to_centroids(oracle, bits, rows, sgc, cols):
    m, idx, sc = oracle.nf_quantize_rtn(normal(40 + bits, (rows, cols), 0.02), bits, sgc, threads=2, return_indices=True)
    # an asymmetric codebook exercises the general 16-entry lookup, not just the fitted symmetric one
    cb = m.codebook.copy()
    if bits == 4:
        cb = np.array([-120, -90, -70, -50, -33, -20, -9, -1, 3, 14, 29, 47, 60, 80, 101, 127], np.int8)
    # NF4 indices are re-encoded to the rank of their centroid: the device codebook is the sorted one
    cb_dev = np.sort(cb[:16]) if bits == 4 else cb
    cb_words = _words(cb_dev.tobytes())
    image = k2.matrix_image(k2.nf_desc(rows, cols, bits, sgc, cb, m.pair, m.tail))
    nsg = -(-(cols // 64) // sgc)
    vals, scales = image_rows(f"nf{bits}", image, rows, cols, nsg, cb_words)
    assert np.array_equal(vals[:rows], cb.astype(np.int16)[idx])
    sc_file = sc.reshape(-1, nsg, 16)
    for r in range(rows):
        assert np.array_equal(scales[r], sc_file[r // 16, :, r % 16])


@pytest.mark.parametrize("rows,sgc", [(71, 1), (128, 2)])
def test_nf5_image_decodes_to_centroids(oracle, rows, sgc):
    cols = 192
    rng = np.random.Generator(np.random.PCG64(rows))
    idx = rng.integers(0, 32, (rows, cols), dtype=np.uint8)
    nsg = -(-(cols // 64) // sgc)
    sc = rng.integers(0x3800, 0x3C00, oracle.lib().k2o_nf_scale_count(rows, cols, sgc)).astype(np.uint16)
    cb = np.array([1, -2, 5, 9, 17, 21, 33, 40, 41, 59, 70, 77, 90, 100, 120, 127], np.int8)      # 16 magnitudes, one of them negative
    m = oracle.nf_pack(idx, sc, 5, sgc, cb)
    cb32 = oracle.nf_expand_codebook32(5, cb)                  # [15 - m] = -cb[m], [16 + m] = cb[m]
    image = k2.matrix_image(k2.nf_desc(rows, cols, 5, sgc, cb, m.pair, m.tail))
    vals, scales = image_rows("nf5", image, rows, cols, nsg, _words(cb32.tobytes()))
    assert np.array_equal(vals[:rows], cb32.astype(np.int16)[idx])
    sc_file = sc.reshape(-1, nsg, 16)
    for r in range(rows):
        assert np.array_equal(scales[r], sc_file[r // 16, :, r % 16])


def test_e8q2_image_decodes_to_lattice_points(oracle):
    rows, cols, sgc = 71, 128, 2
    rng = np.random.Generator(np.random.PCG64(3))
    tpl = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
    sgn = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
    tpl[0, 0], sgn[0, 0] = 0, 1                                # the padding codeword
    sc = rng.integers(0x3800, 0x3C00, oracle.lib().k2o_nf_scale_count(rows, cols, sgc)).astype(np.uint16)
    m = oracle.e8q2_pack(tpl, sgn, sc, sgc)
    words = [t[0] | t[1] << 8 | t[2] << 16 | t[3] << 24 for t in E8Q2_TEMPLATES]
    image = k2.matrix_image(k2.nf_desc(rows, cols, 2, sgc, np.zeros(16, np.int8), m.pair, m.tail))
    vals, _ = image_rows("e8q2", image, rows, cols, 1, words)
    for r in range(rows):
        want = np.concatenate([oracle.e8q2_decode_8d(tpl[r, b], sgn[r, b]) for b in range(cols // 8)])
        assert np.array_equal(vals[r], want.astype(np.int16)), r


def nf4_two_table_values(cell, cb_sorted):
    """cell_dot<FMT_NF4>'s decode: centroid = hi[l] + off where index bit 3 is set, off - lo[l] elsewhere,
    each table looked up with one prmt whose selector has bit 3 set for the lanes that must yield 0."""
    cb = cb_sorted.astype(int)
    off_min, off_max = max(cb[7], cb[15] - 127), min(cb[8], cb[0] + 127)
    assert off_min <= off_max
    off = min(max(0, off_min), off_max)
    hi, lo = [int(cb[8 + l] - off) for l in range(8)], [int(off - cb[l]) for l in range(8)]
    assert all(0 <= v <= 127 for v in hi + lo)
    tab = _words(bytes(hi + lo))
    vals = []
    for x in _words(cell):
        y = x ^ 0x88888888
        for sel_hi, sel_lo in ((y, x), (y >> 16, x >> 16)):
            up = np.array([prmt(tab[0], tab[1], sel_hi)], "<u4").view(np.uint8).astype(int)
            dn = np.array([prmt(tab[2], tab[3], sel_lo)], "<u4").view(np.uint8).astype(int)
            vals.extend((up - dn).tolist())
    # every column got exactly one of the two tables; adding the offset restores the centroid
    return np.array(vals) + off


@pytest.mark.parametrize("cb", [
    [-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127],      # reference default
    [29, -90, -70, 127, -33, -20, -9, -1, 3, 14, -120, 47, 60, 80, 101, -50],      # unsorted, asymmetric
    [100, 101, 102, 103, 104, 105, 106, 107, 108, 109, 110, 111, 112, 113, 114, 115],  # needs an offset
])
def test_nf4_two_table_decode(oracle, cb):
    rows, cols = 16, 128
    cb = np.array(cb, np.int8)
    rng = np.random.Generator(np.random.PCG64(11))
    idx = rng.integers(0, 16, (rows, cols), dtype=np.uint8)
    sc = rng.integers(0x3800, 0x3C00, oracle.lib().k2o_nf_scale_count(rows, cols, 1)).astype(np.uint16)
    m = oracle.nf_pack(idx, sc, 4, 1, cb)
    image = k2.matrix_image(k2.nf_desc(rows, cols, 4, 1, cb, m.pair, m.tail))
    pa, _, _ = split_image("nf4", image, rows, cols, 2)
    for r in range(rows):
        for c in range(2):
            got = nf4_two_table_values(pa[r, c], np.sort(cb))
            assert np.array_equal(got, cb.astype(int)[idx[r, c * 64:(c + 1) * 64]])


def test_gate_up_interleave_image(oracle):
    rows, cols = 256, 128
    m = oracle.bipolar_quantize_rtn(normal(3, (rows, cols), 0.02), 4)
    desc = k2.bipolar_desc(rows, cols, 4, m.data, m.scales)
    plain, _ = image_rows("bp4", k2.matrix_image(desc), rows, cols, 2)
    inter, _ = image_rows("bp4", k2.matrix_image(desc, gate_up_interleave=True), rows, cols, 2)
    half = rows // 2
    for ic in range(half // 64):
        assert np.array_equal(inter[ic * 128: ic * 128 + 64], plain[ic * 64: ic * 64 + 64])
        assert np.array_equal(inter[ic * 128 + 64: ic * 128 + 128], plain[half + ic * 64: half + ic * 64 + 64])
    n = oracle.nf_quantize_rtn(normal(4, (rows, cols), 0.02), 4, 2)
    nd = k2.nf_desc(rows, cols, 4, 2, n.codebook, n.pair, n.tail)
    cbw = _words(n.codebook.tobytes())
    cbw = _words(np.sort(n.codebook).tobytes())
    plain, _ = image_rows("nf4", k2.matrix_image(nd), rows, cols, 1, cbw)
    inter, _ = image_rows("nf4", k2.matrix_image(nd, gate_up_interleave=True), rows, cols, 1, cbw)
    assert np.array_equal(inter[64:128], plain[128:192]) and np.array_equal(inter[128:192], plain[64:128])


def test_malformed_descriptors_are_rejected(oracle):
    m = oracle.bipolar_quantize_rtn(normal(1, (16, 64), 0.02), 4)
    L = k2.load_library()
    good = k2.bipolar_desc(16, 64, 4, m.data, m.scales)
    assert L.kronos_cuda_matrix_image(C.byref(good), 0, None, 0) == 2 * 16 * 16 + 16 * 64 + 16
    for kw in ({"cols": 65}, {"bits": 7}, {"rows": 0}, {"kind": 1}, {"len0": 5}):
        bad = k2.bipolar_desc(16, 64, 4, m.data, m.scales)
        for key, val in kw.items():
            setattr(bad, key, val)
        assert L.kronos_cuda_matrix_image(C.byref(bad), 0, None, 0) == 0
    assert L.kronos_cuda_matrix_image(C.byref(good), 1, None, 0) == 0  # interleave needs rows % 128 == 0


def test_library_exports_every_declared_symbol():
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "kronos_cuda_ffi.h")).read()
    names = set(re.findall(r"\b(kronos_cuda_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 12
    L = k2.load_library()
    for n in sorted(names):
        assert hasattr(L, n), n


def test_no_gpu_means_error_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(k2.KronosCudaError):
        k2.Context(0)
