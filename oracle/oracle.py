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
