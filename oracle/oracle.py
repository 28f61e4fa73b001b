"""ctypes binding of the CPU oracle (libk2t_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's cpu_baseline / reference legs.  The CUDA backend never imports it.
Parity status of the oracle itself: unpinned (see k2t_oracle.h).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libk2t_oracle.so")


def build(force=False):
    """Compile the oracle with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH)
        for f in ("k2t_oracle.cpp", "k2t_oracle.h", "k2t_model.cpp", "Makefile")
        if os.path.exists(os.path.join(_HERE, f))
    ):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


_sz, _u64, _f32, _i32 = C.c_size_t, C.c_uint64, C.c_float, C.c_int
_p = C.c_void_p


def _declare(L):
    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("k2o_rademacher_masks", None, _u64, _p)
    sig("k2o_fwht64", None, _p, _sz, _u64)
    sig("k2o_ifwht64", None, _p, _sz, _u64)
    sig("k2o_f32_to_bf16", C.c_uint16, _f32)
    sig("k2o_bf16_to_f32", _f32, C.c_uint16)
    sig("k2o_act_populate", None, _p, _sz, _p, _p, _p)
    sig("k2o_act_populate_fwht", None, _p, _sz, _p, _f32, _u64, _p, _p, _p)
    sig("k2o_dot_f32", _f32, _p, _p, _sz)
    sig("k2o_inv_rms", _f32, _p, _sz, _f32)
    sig("k2o_bipolar_data_bytes", _sz, _sz, _sz, _sz)
    sig("k2o_bipolar_scale_count", _sz, _sz, _sz)
    sig("k2o_bipolar_quantize_rtn", None, _p, _sz, _sz, _sz, _sz, _p, _p)
    sig("k2o_bipolar_pack", None, _p, _sz, _sz, _sz, _p)
    sig("k2o_bipolar_unpack_row", None, _p, _sz, _sz, _sz, _sz, _p)
    sig("k2o_bipolar_dequant_row", None, _p, _p, _sz, _sz, _sz, _sz, _p)
    sig("k2o_nibble4_pair_bytes", _sz, _sz, _sz, _sz)
    sig("k2o_nibble4_tail_bytes", _sz, _sz, _sz, _sz)
    sig("k2o_nibble4_from_bipolar", None, _p, _p, _sz, _sz, _sz, _i32, _p, _p)
    sig("k2o_nibble4_dequant_row", None, _p, _p, _sz, _sz, _sz, _sz, _p)
    sig("k2o_nibble4_gemv", None, _p, _p, _sz, _sz, _sz, _p, _p, _p, _sz, _p, _sz, _p, _sz)
    sig("k2o_bipolar_gemv_def", None, _p, _p, _sz, _sz, _sz, _p, _p, _p, _p, _p)
    sig("k2o_nf_expand_codebook32", None, _sz, _p, _p)
    sig("k2o_e8q2_decode_8d", None, C.c_uint8, C.c_uint8, _p)
    sig("k2o_nf_chunk_bytes", _sz, _sz)
    sig("k2o_nf_pair_stream_bytes", _sz, _sz, _sz, _sz, _sz)
    sig("k2o_nf_tail_stream_bytes", _sz, _sz, _sz, _sz, _sz)
    sig("k2o_nf_scale_count", _sz, _sz, _sz, _sz)
    sig("k2o_nf_fit_codebook", _f32, _p, _sz, _sz, _sz, _sz, _p)
    sig("k2o_nf_quantize_rtn", None, _p, _sz, _sz, _sz, _sz, _sz, _p, _p, _p)
    sig("k2o_nf4_embed_from_bf16", None, _p, _sz, _sz, _sz, _sz, _p, _p)
    sig("k2o_nf_pack", None, _p, _p, _sz, _sz, _sz, _sz, _p, _p)
    sig("k2o_e8q2_pack", None, _p, _p, _p, _sz, _sz, _sz, _p, _p)
    sig("k2o_nf_gate_up_interleave", None, _p, _sz, _sz, _sz, _sz, _p)
    sig("k2o_nf_dequant_row", None, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _p)
    sig("k2o_nf_gemv", None, _p, _p, _p, _sz, _sz, _sz, _sz, _p, _p, _sz, _p, _sz, _p, _sz)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# --------------------------------------------------------------------------- hadamard / bf16
def rademacher_masks(block):
    out = np.zeros(64, np.uint32)
    lib().k2o_rademacher_masks(block, _ptr(out))
    return out


def fwht64(x, block0=0):
    y = _c(x, np.float32).copy()
    lib().k2o_fwht64(_ptr(y), y.size, block0)
    return y


def ifwht64(x, block0=0):
    y = _c(x, np.float32).copy()
    lib().k2o_ifwht64(_ptr(y), y.size, block0)
    return y


def f32_to_bf16(v):
    return lib().k2o_f32_to_bf16(float(np.float32(v)))


def bf16_to_f32(b):
    return np.float32(lib().k2o_bf16_to_f32(int(b)))


# --------------------------------------------------------------------------- activations
class Act:
    """Int8ChunkActivation for n_tok tokens: q[n_tok, cols] i8, scales/sums[n_tok, nc]."""

    def __init__(self, q, scales, sums):
        self.q, self.scales, self.sums = q, scales, sums


def act_populate(x):
    x = _c(x, np.float32)
    cols = x.shape[-1]
    q = np.zeros(cols, np.int8)
    s = np.zeros(cols // 64, np.float32)
    m = np.zeros(cols // 64, np.int32)
    lib().k2o_act_populate(_ptr(x), cols, _ptr(q), _ptr(s), _ptr(m))
    return Act(q, s, m)


def act_populate_fwht(x, norm_w=None, inv_rms=1.0, chunk0=0):
    x = _c(x, np.float32)
    if x.ndim == 1:
        x = x[None]
    n, cols = x.shape
    q = np.zeros((n, cols), np.int8)
    s = np.zeros((n, cols // 64), np.float32)
    m = np.zeros((n, cols // 64), np.int32)
    w = None if norm_w is None else _c(norm_w, np.float32)
    inv = np.broadcast_to(np.asarray(inv_rms, np.float32), (n,))
    for t in range(n):
        lib().k2o_act_populate_fwht(_ptr(x[t]), cols, _ptr(w), float(inv[t]), chunk0,
                                    _ptr(q[t]), _ptr(s[t]), _ptr(m[t]))
    return Act(q, s, m)


def dot_f32(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    return np.float32(lib().k2o_dot_f32(_ptr(a), _ptr(b), a.size))


def inv_rms(x, eps):
    x = _c(x, np.float32)
    return np.float32(lib().k2o_inv_rms(_ptr(x), x.size, float(eps)))


# --------------------------------------------------------------------------- bipolar
class Bipolar:
    """FusedBipolarLutMatrix as stored in .k2tb: interleaved planes + stripe-major bf16 scales."""

    kind = 0

    def __init__(self, rows, cols, planes, data, scales):
        self.rows, self.cols, self.planes, self.data, self.scales = rows, cols, planes, data, scales

    def file_bytes(self):
        return self.data.nbytes + self.scales.nbytes


def bipolar_quantize_rtn(w, planes, threads=8):
    w = _c(w, np.float32)
    rows, cols = w.shape
    data = np.zeros(lib().k2o_bipolar_data_bytes(rows, cols, planes), np.uint8)
    sc = np.zeros(lib().k2o_bipolar_scale_count(rows, cols), np.uint16)
    lib().k2o_bipolar_quantize_rtn(_ptr(w), rows, cols, planes, threads, _ptr(data), _ptr(sc))
    return Bipolar(rows, cols, planes, data, sc)


def bipolar_from_codes(u, scales_rc, planes):
    """u[rows, cols] codes, scales_rc[rows, nc] bf16 bits -> Bipolar (file layout)."""
    u = _c(u, np.uint8)
    rows, cols = u.shape
    nc = cols // 64
    data = np.zeros(lib().k2o_bipolar_data_bytes(rows, cols, planes), np.uint8)
    lib().k2o_bipolar_pack(_ptr(u), rows, cols, planes, _ptr(data))
    ns = (rows + 15) // 16
    sc = np.zeros((ns, nc, 16), np.uint16)
    r = np.arange(rows)
    sc[r // 16, :, r % 16] = _c(scales_rc, np.uint16)
    return Bipolar(rows, cols, planes, data, sc.reshape(-1))


def bipolar_unpack_row(m, r):
    out = np.zeros(m.cols, np.uint8)
    lib().k2o_bipolar_unpack_row(_ptr(m.data), m.rows, m.cols, m.planes, r, _ptr(out))
    return out


def bipolar_dequant_row(m, r):
    out = np.zeros(m.cols, np.float32)
    lib().k2o_bipolar_dequant_row(_ptr(m.data), _ptr(m.scales), m.rows, m.cols, m.planes, r, _ptr(out))
    return out


class Nibble4:
    def __init__(self, rows, cols, planes, pair, tail):
        self.rows, self.cols, self.planes, self.pair, self.tail = rows, cols, planes, pair, tail


def nibble4_from_bipolar(m, interleave_gate_up=False):
    pair = np.zeros(lib().k2o_nibble4_pair_bytes(m.rows, m.cols, m.planes), np.uint8)
    tail = np.zeros(max(1, lib().k2o_nibble4_tail_bytes(m.rows, m.cols, m.planes)), np.uint8)
    lib().k2o_nibble4_from_bipolar(_ptr(m.data), _ptr(m.scales), m.rows, m.cols, m.planes,
                                   int(interleave_gate_up), _ptr(pair), _ptr(tail))
    return Nibble4(m.rows, m.cols, m.planes, pair, tail)


def nibble4_dequant_row(n4, r):
    out = np.zeros(n4.cols, np.float32)
    lib().k2o_nibble4_dequant_row(_ptr(n4.pair), _ptr(n4.tail), n4.rows, n4.cols, n4.planes, r, _ptr(out))
    return out


def nibble4_gemv(n4, act, want_dots=False, threads=1):
    q = _c(act.q, np.int8).reshape(-1, n4.cols)
    n = q.shape[0]
    nc = n4.cols // 64
    xs = _c(act.scales, np.float32).reshape(n, nc)
    xm = _c(act.sums, np.int32).reshape(n, nc)
    out = np.zeros((n, n4.rows), np.float32)
    dots = np.zeros((n, n4.rows, nc), np.int32) if want_dots else None
    lib().k2o_nibble4_gemv(_ptr(n4.pair), _ptr(n4.tail), n4.rows, n4.cols, n4.planes, _ptr(q), _ptr(xs),
                           _ptr(xm), n, _ptr(out), n4.rows, _ptr(dots), threads)
    return (out, dots) if want_dots else out


def bipolar_gemv_def(m, act):
    nc = m.cols // 64
    q = _c(act.q, np.int8).reshape(-1)
    xs = _c(act.scales, np.float32).reshape(-1)
    xm = _c(act.sums, np.int32).reshape(-1)
    out = np.zeros(m.rows, np.float32)
    dots = np.zeros((m.rows, nc), np.int32)
    lib().k2o_bipolar_gemv_def(_ptr(m.data), _ptr(m.scales), m.rows, m.cols, m.planes, _ptr(q), _ptr(xs),
                               _ptr(xm), _ptr(out), _ptr(dots))
    return out, dots


# --------------------------------------------------------------------------- NF / E8Q2
class Nf:
    """NfSdotMatrix as stored in .k2tb: pair_stream + tail_stream + 16-byte codebook."""

    kind = 2

    def __init__(self, rows, cols, bits, sgc, codebook, pair, tail):
        self.rows, self.cols, self.bits, self.sgc = rows, cols, bits, sgc
        self.codebook, self.pair, self.tail = codebook, pair, tail

    def file_bytes(self):
        return self.pair.nbytes + self.tail.nbytes + 16


def nf_expand_codebook32(bits, cb):
    cb = _c(cb, np.int8)
    out = np.zeros(32, np.int8)
    lib().k2o_nf_expand_codebook32(bits, _ptr(cb), _ptr(out))
    return out


def e8q2_decode_8d(tpl, sgn):
    out = np.zeros(8, np.int8)
    lib().k2o_e8q2_decode_8d(int(tpl), int(sgn), _ptr(out))
    return out


def nf_fit_codebook(w, bits, sgc):
    w = _c(w, np.float32)
    cb = np.zeros(16, np.int8)
    top = lib().k2o_nf_fit_codebook(_ptr(w), w.shape[0], w.shape[1], bits, sgc, _ptr(cb))
    return cb, np.float32(top)


def _nf_alloc(rows, cols, bits, sgc):
    pair = np.zeros(max(1, lib().k2o_nf_pair_stream_bytes(rows, cols, bits, sgc)), np.uint8)
    tail = np.zeros(max(1, lib().k2o_nf_tail_stream_bytes(rows, cols, bits, sgc)), np.uint8)
    return pair, tail


def nf_pack(idx, scales, bits, sgc, codebook):
    """idx[rows, cols] u8, scales = stripe-major bf16 [stripes*nsg*16]."""
    idx = _c(idx, np.uint8)
    rows, cols = idx.shape
    scales = _c(scales, np.uint16)
    assert scales.size == lib().k2o_nf_scale_count(rows, cols, sgc)
    pair, tail = _nf_alloc(rows, cols, bits, sgc)
    lib().k2o_nf_pack(_ptr(idx), _ptr(scales), rows, cols, bits, sgc, _ptr(pair), _ptr(tail))
    pair = pair[: lib().k2o_nf_pair_stream_bytes(rows, cols, bits, sgc)]
    tail = tail[: lib().k2o_nf_tail_stream_bytes(rows, cols, bits, sgc)]
    return Nf(rows, cols, bits, sgc, _c(codebook, np.int8).copy(), pair, tail)


def nf_quantize_rtn(w, bits, sgc, threads=8, return_indices=False):
    w = _c(w, np.float32)
    rows, cols = w.shape
    cb = np.zeros(16, np.int8)
    idx = np.zeros((rows, cols), np.uint8)
    sc = np.zeros(lib().k2o_nf_scale_count(rows, cols, sgc), np.uint16)
    lib().k2o_nf_quantize_rtn(_ptr(w), rows, cols, bits, sgc, threads, _ptr(cb), _ptr(idx), _ptr(sc))
    m = nf_pack(idx, sc, bits, sgc, cb)
    return (m, idx, sc) if return_indices else m


def nf4_embed_from_bf16(table_bf16, sgc=2, threads=8):
    """NfSdotMatrix::from_bf16_u16_embeddings_nf4: bf16 table [rows, cols] (uint16) -> Nf matrix, default NF4 codebook."""
    t = _c(table_bf16, np.uint16)
    rows, cols = t.shape
    pair, tail = _nf_alloc(rows, cols, 4, sgc)
    lib().k2o_nf4_embed_from_bf16(_ptr(t), rows, cols, sgc, threads, _ptr(pair), _ptr(tail))
    pair = pair[: lib().k2o_nf_pair_stream_bytes(rows, cols, 4, sgc)]
    tail = tail[: lib().k2o_nf_tail_stream_bytes(rows, cols, 4, sgc)]
    cb = np.array([-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127], np.int8)
    return Nf(rows, cols, 4, sgc, cb, pair, tail)


def e8q2_pack(tpl, sgn, scales, sgc):
    tpl, sgn = _c(tpl, np.uint8), _c(sgn, np.uint8)
    rows, cols = tpl.shape[0], tpl.shape[1] * 8
    scales = _c(scales, np.uint16)
    pair, tail = _nf_alloc(rows, cols, 2, sgc)
    lib().k2o_e8q2_pack(_ptr(tpl), _ptr(sgn), _ptr(scales), rows, cols, sgc, _ptr(pair), _ptr(tail))
    pair = pair[: lib().k2o_nf_pair_stream_bytes(rows, cols, 2, sgc)]
    tail = tail[: lib().k2o_nf_tail_stream_bytes(rows, cols, 2, sgc)]
    return Nf(rows, cols, 2, sgc, np.zeros(16, np.int8), pair, tail)


def nf_gate_up_interleave(m):
    out = np.zeros_like(m.pair)
    lib().k2o_nf_gate_up_interleave(_ptr(m.pair), m.rows, m.cols, m.bits, m.sgc, _ptr(out))
    return Nf(m.rows, m.cols, m.bits, m.sgc, m.codebook, out, m.tail)


def nf_dequant_row(m, r):
    out = np.zeros(m.cols, np.float32)
    lib().k2o_nf_dequant_row(_ptr(m.pair), _ptr(m.tail), _ptr(m.codebook), m.rows, m.cols, m.bits, m.sgc, r,
                             _ptr(out))
    return out


def nf_gemv(m, act, want_dots=False, threads=1):
    q = _c(act.q, np.int8).reshape(-1, m.cols)
    n = q.shape[0]
    nc = m.cols // 64
    xs = _c(act.scales, np.float32).reshape(n, nc)
    out = np.zeros((n, m.rows), np.float32)
    dots = np.zeros((n, m.rows, nc), np.int32) if want_dots else None
    lib().k2o_nf_gemv(_ptr(m.pair), _ptr(m.tail), _ptr(m.codebook), m.rows, m.cols, m.bits, m.sgc, _ptr(q),
                      _ptr(xs), n, _ptr(out), m.rows, _ptr(dots), threads)
    return (out, dots) if want_dots else out


def gemv(m, act, want_dots=False, threads=1):
    """Reference CPU GEMV for either matrix kind (bipolar goes through the Nibble4 repack)."""
    if m.kind == 0:
        return nibble4_gemv(nibble4_from_bipolar(m), act, want_dots, threads)
    return nf_gemv(m, act, want_dots, threads)


# --------------------------------------------------------------------------- dense decode model
class MatrixDesc(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("bits", C.c_uint32),
                ("scale_group_chunks", C.c_uint32), ("codebook", C.c_int8 * 16),
                ("data0", C.c_void_p), ("len0", C.c_size_t), ("data1", C.c_void_p), ("len1", C.c_size_t)]


class Config(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("layers", C.c_uint32), ("n_q", C.c_uint32), ("n_kv", C.c_uint32),
                ("head_dim", C.c_uint32), ("inter", C.c_uint32), ("vocab", C.c_uint32), ("max_seq", C.c_uint32),
                ("eps", C.c_float), ("qk_norm_after_rope", C.c_int32), ("kv_bits", C.c_uint32),
                ("o_chunk0", C.c_uint32), ("down_chunk0", C.c_uint32)]


def desc_of(m):
    """MatrixDesc of a Bipolar / Nf object (keeps the arrays alive on the descriptor)."""
    d = MatrixDesc()
    d.rows, d.cols = m.rows, m.cols
    if m.kind == 0:
        d.kind, d.bits, d.scale_group_chunks = 0, m.planes, 1
        a, b = _c(m.data, np.uint8), _c(m.scales, np.uint16)
    else:
        d.kind, d.bits, d.scale_group_chunks = 2, m.bits, m.sgc
        a, b = _c(m.pair, np.uint8), _c(m.tail, np.uint8)
        for i in range(16):
            d.codebook[i] = int(m.codebook[i])
    d.data0, d.len0 = (a.ctypes.data if a.size else None), a.nbytes
    d.data1, d.len1 = (b.ctypes.data if b.size else None), b.nbytes
    d._keep = (a, b)
    return d


_model_declared = False


def _declare_model(L):
    global _model_declared
    if _model_declared:
        return
    D, P = C.POINTER(MatrixDesc), C.c_void_p
    L.k2o_model_new.restype, L.k2o_model_new.argtypes = P, [C.POINTER(Config), P]
    L.k2o_model_free.restype, L.k2o_model_free.argtypes = None, [P]
    L.k2o_model_set_layer.restype, L.k2o_model_set_layer.argtypes = C.c_int, [P, C.c_uint32, P, P, P, P, P, D, D, D, D]
    L.k2o_model_set_head.restype, L.k2o_model_set_head.argtypes = C.c_int, [P, P, D, P]
    L.k2o_model_set_embedding_matrix.restype, L.k2o_model_set_embedding_matrix.argtypes = C.c_int, [P, D]
    L.k2o_model_reset.restype, L.k2o_model_reset.argtypes = None, [P]
    L.k2o_model_pos.restype, L.k2o_model_pos.argtypes = C.c_size_t, [P]
    L.k2o_model_set_pos.restype, L.k2o_model_set_pos.argtypes = None, [P, C.c_size_t]
    L.k2o_model_set_kv_window.restype, L.k2o_model_set_kv_window.argtypes = C.c_int, [P, C.c_uint32, C.c_size_t, C.c_size_t]
    L.k2o_model_kv_rows.restype, L.k2o_model_kv_rows.argtypes = C.c_size_t, [P]
    L.k2o_model_save_kv_prefix.restype, L.k2o_model_save_kv_prefix.argtypes = C.c_size_t, [P, C.c_size_t, P]
    L.k2o_model_restore_kv_prefix.restype, L.k2o_model_restore_kv_prefix.argtypes = C.c_int, [P, P, C.c_size_t, C.c_size_t, C.c_size_t]
    L.k2o_model_can_truncate_kv_to.restype, L.k2o_model_can_truncate_kv_to.argtypes = C.c_int, [P, C.c_size_t]
    L.k2o_model_embed.restype, L.k2o_model_embed.argtypes = None, [P, C.c_uint32, P]
    L.k2o_model_forward_embedding.restype, L.k2o_model_forward_embedding.argtypes = C.c_int, [P, P, P, C.c_size_t]
    L.k2o_model_forward_token.restype, L.k2o_model_forward_token.argtypes = C.c_int, [P, C.c_uint32, P, C.c_size_t]
    L.k2o_model_tap_hidden.restype, L.k2o_model_tap_hidden.argtypes = P, [P]
    L.k2o_model_set_moe.restype = C.c_int
    L.k2o_model_set_moe.argtypes = [P, C.c_uint32, P, P, C.c_uint32, C.c_uint32, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, P, C.c_size_t]
    L.k2o_model_set_moe_shared.restype, L.k2o_model_set_moe_shared.argtypes = C.c_int, [P, C.c_uint32, D, D, P]
    L.k2o_model_last_routes.restype, L.k2o_model_last_routes.argtypes = C.c_uint32, [P, C.c_uint32, P, P]
    L.k2o_model_set_ep.restype, L.k2o_model_set_ep.argtypes = None, [P, C.c_uint32, C.c_uint32]
    L.k2o_nf_expert_layout.restype = C.c_size_t
    L.k2o_nf_expert_layout.argtypes = [C.c_size_t] * 4 + [P] * 4
    L.k2o_model_tap_attention.restype, L.k2o_model_tap_attention.argtypes = P, [P]
    L.k2o_model_read_kv.restype, L.k2o_model_read_kv.argtypes = C.c_int, [P, C.c_uint32, C.c_uint32, C.c_size_t, P, P, P, P]
    for name in ("k2o_model_attn_part", "k2o_model_ffn_part"):
        getattr(L, name).restype, getattr(L, name).argtypes = C.c_int, [P, C.c_uint32, P, P, C.c_size_t]
    L.k2o_model_head_part.restype, L.k2o_model_head_part.argtypes = C.c_int, [P, P, P, C.c_size_t]
    L.k2o_model_advance.restype, L.k2o_model_advance.argtypes = None, [P]
    L.k2o_model_kv_export.restype, L.k2o_model_kv_export.argtypes = C.c_size_t, [P, C.c_size_t, C.c_size_t, P]
    L.k2o_model_kv_import.restype, L.k2o_model_kv_import.argtypes = C.c_int, [P, P, C.c_size_t, C.c_size_t]
    L.k2o_model_read_kv_q4.restype, L.k2o_model_read_kv_q4.argtypes = C.c_int, [P, C.c_uint32, C.c_uint32, C.c_size_t, P, P, P, P]
    L.k2o_kv_quant_head_q4.restype, L.k2o_kv_quant_head_q4.argtypes = None, [P, C.c_size_t, P, P]
    L.k2o_nf4_nearest_idx.restype, L.k2o_nf4_nearest_idx.argtypes = C.c_uint8, [C.c_float]
    L.k2o_argmax.restype, L.k2o_argmax.argtypes = C.c_uint32, [P, C.c_size_t]
    L.k2o_build_rope_table.restype, L.k2o_build_rope_table.argtypes = None, [C.c_size_t, C.c_size_t, C.c_double, P]
    L.k2o_exp_poly.restype, L.k2o_exp_poly.argtypes = C.c_float, [C.c_float]
    L.k2o_swiglu.restype, L.k2o_swiglu.argtypes = None, [P, P, C.c_size_t, P]
    L.k2o_rope_heads.restype, L.k2o_rope_heads.argtypes = None, [P, C.c_size_t, C.c_size_t, P]
    L.k2o_head_rms_norm.restype, L.k2o_head_rms_norm.argtypes = None, [P, C.c_size_t, C.c_size_t, P, C.c_float]
    L.k2o_kv_quant_head.restype, L.k2o_kv_quant_head.argtypes = None, [P, C.c_size_t, P, P]
    _model_declared = True


def build_rope_table(max_seq, head_dim, theta):
    L = lib(); _declare_model(L)
    t = np.zeros((max_seq, head_dim), np.float32)
    L.k2o_build_rope_table(max_seq, head_dim, float(theta), _ptr(t))
    return t


def swiglu(gate, up):
    L = lib(); _declare_model(L)
    g, u = _c(gate, np.float32), _c(up, np.float32)
    out = np.zeros_like(g)
    L.k2o_swiglu(_ptr(g), _ptr(u), g.size, _ptr(out))
    return out


def rope_heads(buf, heads, head_dim, rope_row):
    L = lib(); _declare_model(L)
    b = _c(buf, np.float32).copy()
    r = _c(rope_row, np.float32)
    L.k2o_rope_heads(_ptr(b), heads, head_dim, _ptr(r))
    return b


def head_rms_norm(buf, heads, head_dim, w, eps):
    L = lib(); _declare_model(L)
    b = _c(buf, np.float32).copy()
    ww = _c(w, np.float32)
    L.k2o_head_rms_norm(_ptr(b), heads, head_dim, _ptr(ww), float(eps))
    return b


def nf_expert_layout(d_model, d_ff, bits, sgc):
    """NfExpertByteLayout of a .k2tm record: dict(expert_bytes, gu_off, gu_bytes, dn_off, dn_bytes)."""
    L = lib(); _declare_model(L)
    v = [C.c_size_t() for _ in range(4)]
    total = L.k2o_nf_expert_layout(d_model, d_ff, bits, sgc, *[C.byref(x) for x in v])
    return dict(expert_bytes=total, gu_off=v[0].value, gu_bytes=v[1].value, dn_off=v[2].value, dn_bytes=v[3].value)


def pack_expert_shard(experts, d_model, d_ff, bits, sgc):
    """pack_nf_expert_record (moe_800b.rs:1385-1407) for a list of (gate_up Nf, down Nf): codebooks at 0 / 16, gate_up
    pair_stream at 64, down pair_stream at the next multiple of 64, zero-padded to a 16 KiB multiple per record."""
    lay = nf_expert_layout(d_model, d_ff, bits, sgc)
    shard = np.zeros(len(experts) * lay["expert_bytes"], np.uint8)
    for e, (gu, dn) in enumerate(experts):
        assert gu.tail.size == 0 and dn.tail.size == 0 and gu.pair.size == lay["gu_bytes"] and dn.pair.size == lay["dn_bytes"]
        rec = shard[e * lay["expert_bytes"]:(e + 1) * lay["expert_bytes"]]
        rec[0:16] = np.asarray(gu.codebook, np.int8).view(np.uint8)
        rec[16:32] = np.asarray(dn.codebook, np.int8).view(np.uint8)
        rec[lay["gu_off"]:lay["gu_off"] + lay["gu_bytes"]] = gu.pair
        rec[lay["dn_off"]:lay["dn_off"] + lay["dn_bytes"]] = dn.pair
    return shard, lay


def kv_quant_head_q4(src):
    L = lib(); _declare_model(L)
    x = _c(src, np.float32)
    q4, s16 = np.zeros(x.size // 2, np.uint8), np.zeros(x.size // 64, np.uint16)
    L.k2o_kv_quant_head_q4(_ptr(x), x.size, _ptr(q4), _ptr(s16))
    return q4, s16


def nf4_nearest_idx(y):
    L = lib(); _declare_model(L)
    return int(L.k2o_nf4_nearest_idx(float(y)))


def kv_quant_head(src):
    L = lib(); _declare_model(L)
    s = _c(src, np.float32)
    q = np.zeros(s.size, np.int8)
    sc = np.zeros(1, np.float32)
    L.k2o_kv_quant_head(_ptr(s), s.size, _ptr(q), _ptr(sc))
    return q, sc[0]


def attention_q8(q, k_heads, v_heads, attn_scale):
    """causal_gqa_attention_q8 over keys / values given per kv head as fp32 [n_kv][seq][head_dim]: they are stored through the
    int8 Hadamard quantizer (store_hadamard_q8_head*_raw), then every query head [n_q][head_dim] attends to all of them."""
    L = lib(); _declare_model(L)
    k_heads, v_heads, q = _c(k_heads, np.float32), _c(v_heads, np.float32), _c(q, np.float32)
    n_kv, seq, hd = k_heads.shape
    n_q = q.shape[0]
    kq, vq = np.zeros((n_kv, seq, hd), np.int8), np.zeros((n_kv, seq, hd), np.int8)
    ks, vs = np.zeros((n_kv, seq), np.float32), np.zeros((n_kv, seq), np.float32)
    for h in range(n_kv):
        for t in range(seq):
            kq[h, t], ks[h, t] = kv_quant_head(k_heads[h, t])
            vq[h, t], vs[h, t] = kv_quant_head(v_heads[h, t])
    out = np.zeros((n_q, hd), np.float32)
    L.k2o_attention_q8.restype, L.k2o_attention_q8.argtypes = None, [C.c_size_t] * 4 + [C.c_void_p] * 5 + [C.c_float, C.c_void_p]
    L.k2o_attention_q8(hd, n_q, n_kv, seq, _ptr(kq), _ptr(ks), _ptr(vq), _ptr(vs), _ptr(q), attn_scale, _ptr(out))
    return out


def argmax(v):
    L = lib(); _declare_model(L)
    v = _c(v, np.float32)
    return int(L.k2o_argmax(_ptr(v), v.size))


class Model:
    """Dense Llama/Qwen decode model on the CPU oracle. `spec` is the dict produced by tests/k2t_models.py."""

    def __init__(self, spec):
        L = lib(); _declare_model(L)
        self.L, self.spec = L, spec
        c = spec["cfg"]
        self.cfg = Config(c["hidden"], c["layers"], c["n_q"], c["n_kv"], c["head_dim"], c["inter"], c["vocab"], c["max_seq"],
                          c["eps"], int(c.get("qk_norm_after_rope", 0)), int(c.get("kv_bits", 8)),
                          int(c.get("o_chunk0", 0)), int(c.get("down_chunk0", 0)))
        rope = _c(spec["rope"], np.float32)
        self.h = L.k2o_model_new(C.byref(self.cfg), _ptr(rope))
        assert self.h, "k2o_model_new failed"
        for l, ly in enumerate(spec["layers"]):
            moe = ly.get("moe")
            ds = [desc_of(ly[k]) for k in (("qkv", "o") if moe else ("qkv", "o", "gate_up", "down"))]
            arrs = [None if ly.get(k) is None else _c(ly[k], np.float32) for k in ("input_norm", "post_norm", "qkv_bias", "q_norm", "k_norm")]
            refs = [C.byref(d) for d in ds] + ([None, None] if moe else [])
            rc = L.k2o_model_set_layer(self.h, l, *[_ptr(a) for a in arrs], *refs)
            assert rc == 0, f"set_layer {l} failed"
            if moe:
                rw = _c(moe["router_w"], np.float32)
                rb = None if moe.get("router_bias") is None else _c(moe["router_bias"], np.float32)
                shard = _c(moe["shard"], np.uint8)
                rc = L.k2o_model_set_moe(self.h, l, _ptr(rw), _ptr(rb), moe["n_experts"], moe["top_k"], int(moe["norm_topk"]) | (int(moe.get("scoring", 0)) << 8), moe["d_ff"],
                                         moe["bits"], moe["sgc"], _ptr(shard), moe["expert_bytes"])
                assert rc == 0, f"set_moe {l} failed"
                sh = moe.get("shared")              # dict(gate_up=Nf, down=Nf, gate_w=array or None)
                if sh is not None:
                    dg, dd = desc_of(sh["gate_up"]), desc_of(sh["down"])
                    gw = None if sh.get("gate_w") is None else _c(sh["gate_w"], np.float32)
                    assert L.k2o_model_set_moe_shared(self.h, l, C.byref(dg), C.byref(dd), _ptr(gw)) == 0, f"set_moe_shared {l} failed"
        emb = None if spec.get("embed_bf16") is None else _c(spec["embed_bf16"], np.uint16)
        d = desc_of(spec["lm_head"])
        fn = _c(spec["final_norm"], np.float32)
        assert L.k2o_model_set_head(self.h, _ptr(fn), C.byref(d), _ptr(emb)) == 0
        if spec.get("embed_matrix") is not None:       # the untied table compressed to NF4 (or the whole tied lm_head of a sharded model)
            self._embed_desc = desc_of(spec["embed_matrix"])
            assert L.k2o_model_set_embedding_matrix(self.h, C.byref(self._embed_desc)) == 0
        if int(c.get("kv_window", 0)) > 0:
            self.set_kv_window(int(c.get("kv_bits", 8)), int(c["kv_window"]), int(c.get("kv_sinks", 0)))

    def set_kv_window(self, kv_bits, window, sinks):
        """set_kv_bits + set_kv_sliding_window: rebuilds the cache (position 0); True when the window is active."""
        rc = self.L.k2o_model_set_kv_window(self.h, kv_bits, window, sinks)
        assert rc >= 0
        self.cfg.kv_bits = kv_bits
        return rc == 1

    @property
    def kv_rows(self):
        return self.L.k2o_model_kv_rows(self.h)

    def save_kv_prefix(self, n):
        out = np.zeros(self.L.k2o_model_save_kv_prefix(self.h, n, None), np.uint8)
        self.L.k2o_model_save_kv_prefix(self.h, n, _ptr(out))
        return out

    def restore_kv_prefix(self, blob, total_pos, copy_slots=None):
        b = _c(blob, np.uint8)
        assert self.L.k2o_model_restore_kv_prefix(self.h, _ptr(b), b.size, (1 << 63) if copy_slots is None else copy_slots, total_pos) == 0

    def can_truncate_kv_to(self, target_len):
        return bool(self.L.k2o_model_can_truncate_kv_to(self.h, target_len))

    def close(self):
        if self.h:
            self.L.k2o_model_free(self.h)
            self.h = None

    def reset(self):
        self.L.k2o_model_reset(self.h)

    @property
    def pos(self):
        return self.L.k2o_model_pos(self.h)

    def embed(self, token):
        out = np.zeros(self.cfg.hidden, np.float32)
        self.L.k2o_model_embed(self.h, int(token), _ptr(out))
        return out

    def forward_token(self, token, threads=8):
        logits = np.zeros(self.cfg.vocab, np.float32)
        assert self.L.k2o_model_forward_token(self.h, int(token), _ptr(logits), threads) == 0
        return logits

    def forward_embedding(self, e, threads=8):
        e = _c(e, np.float32)
        logits = np.zeros(self.cfg.vocab, np.float32)
        assert self.L.k2o_model_forward_embedding(self.h, _ptr(e), _ptr(logits), threads) == 0
        return logits

    def tap_hidden(self):
        p = self.L.k2o_model_tap_hidden(self.h)
        n = self.cfg.layers * self.cfg.hidden
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,)).reshape(self.cfg.layers, self.cfg.hidden).copy()

    # ---- pieces of a forward pass (tensor-parallel emulation, see TpModel)
    def attn_part(self, layer, hidden, threads=2):
        out = np.zeros(self.cfg.hidden, np.float32)
        assert self.L.k2o_model_attn_part(self.h, layer, _ptr(_c(hidden, np.float32)), _ptr(out), threads) == 0
        return out

    def ffn_part(self, layer, hidden, threads=2):
        out = np.zeros(self.cfg.hidden, np.float32)
        assert self.L.k2o_model_ffn_part(self.h, layer, _ptr(_c(hidden, np.float32)), _ptr(out), threads) == 0
        return out

    def head_part(self, hidden, threads=2):
        out = np.zeros(self.cfg.vocab, np.float32)
        assert self.L.k2o_model_head_part(self.h, _ptr(_c(hidden, np.float32)), _ptr(out), threads) == 0
        return out

    def advance(self):
        self.L.k2o_model_advance(self.h)

    def kv_export(self, lo, hi):
        n = self.L.k2o_model_kv_export(self.h, lo, hi, None)
        out = np.zeros(n, np.uint8)
        self.L.k2o_model_kv_export(self.h, lo, hi, _ptr(out))
        return out

    def kv_import(self, blob, n):
        b = _c(blob, np.uint8)
        assert self.L.k2o_model_kv_import(self.h, _ptr(b), b.size, n) == 0

    def last_routes(self, layer):
        e, w = np.zeros(32, np.uint32), np.zeros(32, np.float32)
        k = self.L.k2o_model_last_routes(self.h, layer, _ptr(e), _ptr(w))
        return e[:k].copy(), w[:k].copy()

    def tap_attention(self):
        p = self.L.k2o_model_tap_attention(self.h)
        n = self.cfg.n_q * self.cfg.head_dim
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,)).copy()

    def read_kv(self, layer, kv_head, pos):
        hd = self.cfg.head_dim
        if self.cfg.kv_bits == 4:
            k, v = np.zeros(hd // 2, np.uint8), np.zeros(hd // 2, np.uint8)
            ks, vs = np.zeros(hd // 64, np.uint16), np.zeros(hd // 64, np.uint16)
            assert self.L.k2o_model_read_kv_q4(self.h, layer, kv_head, pos, _ptr(k), _ptr(ks), _ptr(v), _ptr(vs)) == 0
            return k, ks, v, vs
        k, v = np.zeros(hd, np.int8), np.zeros(hd, np.int8)
        ks, vs = np.zeros(1, np.float32), np.zeros(1, np.float32)
        assert self.L.k2o_model_read_kv(self.h, layer, kv_head, pos, _ptr(k), _ptr(ks), _ptr(v), _ptr(vs)) == 0
        return k, float(ks[0]), v, float(vs[0])

    def greedy(self, prompt, steps, threads=8):
        """Feeds `prompt` token by token, then decodes `steps` tokens greedily. Returns (tokens, last logits)."""
        logits = None
        for t in prompt:
            logits = self.forward_token(t, threads)
        out = []
        for _ in range(steps):
            nxt = argmax(logits)
            out.append(nxt)
            logits = self.forward_token(nxt, threads)
        return out, logits


class TpModel:
    """Tensor-parallel emulation on the CPU: one rank-local Model per rank (specs from kronos_2t_b200.tp.shard_spec); after
    the attention block and after the MLP the ranks' partial outputs are summed in rank order, ((p0 + p1) + p2) + ..., and
    added to the residual stream; logits are the concatenation of the ranks' lm_head slices.  `embed(token)` must be
    given (the full model's embedding), since a rank only holds a slice of the lm_head."""

    def __init__(self, rank_specs, embed):
        self.ranks = [Model(s) for s in rank_specs]
        self.embed = embed
        self.layers = rank_specs[0]["cfg"]["layers"]

    def close(self):
        for m in self.ranks:
            m.close()

    @staticmethod
    def _sum(parts):
        acc = parts[0].copy()
        for p in parts[1:]:
            acc = (acc + p).astype(np.float32)
        return acc

    def forward_token(self, token, threads=2):
        hidden = np.asarray(self.embed(token), np.float32).copy()
        for l in range(self.layers):
            hidden = (hidden + self._sum([m.attn_part(l, hidden, threads) for m in self.ranks])).astype(np.float32)
            hidden = (hidden + self._sum([m.ffn_part(l, hidden, threads) for m in self.ranks])).astype(np.float32)
        logits = np.concatenate([m.head_part(hidden, threads) for m in self.ranks])
        for m in self.ranks:
            m.advance()
        self.last_hidden = hidden
        return logits


class EpModel:
    """Expert-parallel emulation on the CPU: every rank holds the whole model and runs the dense parts (identically);
    in a sparse-MoE block rank r adds only the routed experts e with e % ep == r, and the ranks' partial sums are added
    in rank order, ((p0 + p1) + p2) + ..., before they join the residual stream."""

    def __init__(self, spec, ep):
        self.ranks = [Model(spec) for _ in range(ep)]
        for r, m in enumerate(self.ranks):
            m.L.k2o_model_set_ep(m.h, ep, r)
        self.layers = spec["cfg"]["layers"]
        self.moe = [bool(ly.get("moe")) for ly in spec["layers"]]

    def close(self):
        for m in self.ranks:
            m.close()

    def forward_token(self, token, threads=2):
        hidden = np.asarray(self.ranks[0].embed(token), np.float32).copy()
        for l in range(self.layers):
            attn = [m.attn_part(l, hidden, threads) for m in self.ranks]          # every rank keeps its own KV cache
            hidden = (hidden + attn[0]).astype(np.float32)
            parts = [m.ffn_part(l, hidden, threads) for m in self.ranks]
            hidden = (hidden + (TpModel._sum(parts) if self.moe[l] else parts[0])).astype(np.float32)
        logits = self.ranks[0].head_part(hidden, threads)
        for m in self.ranks:
            m.advance()
        self.last_hidden = hidden
        return logits

