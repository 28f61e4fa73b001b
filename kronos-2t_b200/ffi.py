"""ctypes binding of include/kronos_cuda_ffi.h.

Host-buffer methods take numpy arrays; `*_dev` methods take raw device addresses (for example
`torch.Tensor.data_ptr()`), so a harness can keep inputs resident in HBM.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

MATRIX_BIPOLAR = 0
MATRIX_NF = 2
UPLOAD_GATE_UP_INTERLEAVE = 1


class KronosCudaError(RuntimeError):
    pass


def lib_path():
    return os.path.join(_HERE, "lib", "libkronos_cuda.so")


class MatrixDesc(C.Structure):
    _fields_ = [
        ("kind", C.c_uint32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("bits", C.c_uint32),
        ("scale_group_chunks", C.c_uint32), ("codebook", C.c_int8 * 16),
        ("data0", C.c_void_p), ("len0", C.c_size_t), ("data1", C.c_void_p), ("len1", C.c_size_t),
    ]


class EngineConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("struct_size", "hidden_size", "num_layers", "num_attention_heads", "num_key_value_heads",
                                          "head_dim", "intermediate_size", "vocab_size", "max_seq_len")] + \
               [("rms_norm_eps", C.c_float), ("qk_norm_after_rope", C.c_int32), ("kv_bits", C.c_uint32)] + \
               [(n, C.c_uint32) for n in ("moe_num_experts", "moe_top_k", "moe_norm_topk", "moe_d_ff", "moe_bits",
                                          "moe_scale_group_chunks")] + [("moe_expert_bytes", C.c_uint64)] + \
               [(n, C.c_uint32) for n in ("tp_size", "tp_rank", "o_chunk0", "down_chunk0", "vocab_total", "ep_size", "ep_rank",
                                          "kv_window", "kv_sinks", "flags")]

ENGINE_SPLIT_KV_ATTENTION = 1


class LayerDesc(C.Structure):
    _fields_ = [("input_norm", C.c_void_p), ("post_attn_norm", C.c_void_p), ("qkv_bias", C.c_void_p),
                ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("qkv_proj", MatrixDesc), ("o_proj", MatrixDesc), ("gate_up_proj", MatrixDesc), ("down_proj", MatrixDesc),
                ("moe_router_w", C.c_void_p), ("moe_router_bias", C.c_void_p), ("moe_shard", C.c_void_p), ("moe_shard_len", C.c_size_t),
                ("moe_shared_gate_w", C.c_void_p)]


def load_library():
    """Loads libkronos_cuda.so; raises if it has not been built (no fallback exists)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise KronosCudaError(f"{path} is missing: run `python kronos-2t_b200/build.py` (needs nvcc)")
    L = C.CDLL(path)
    vp, sz, i32, u32, u64 = C.c_void_p, C.c_size_t, C.c_int32, C.c_uint32, C.c_uint64

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype, f.argtypes = res, list(args)

    sig("kronos_cuda_context_create", vp, i32)
    sig("kronos_cuda_context_destroy", None, vp)
    sig("kronos_cuda_last_error", C.c_char_p, vp)
    sig("kronos_cuda_synchronize", i32, vp)
    sig("kronos_cuda_launch_count", u64, vp)
    sig("kronos_cuda_set_stream", i32, vp, vp)
    sig("kronos_cuda_matrix_upload", vp, vp, C.POINTER(MatrixDesc), u32)
    sig("kronos_cuda_matrix_clone", vp, vp, vp)
    sig("kronos_cuda_matrix_free", None, vp, vp)
    sig("kronos_cuda_matrix_file_bytes", sz, vp)
    sig("kronos_cuda_matrix_device_bytes", sz, vp)
    sig("kronos_cuda_matrix_image", sz, C.POINTER(MatrixDesc), u32, vp, sz)
    sig("kronos_cuda_fwht_quant", i32, vp, vp, sz, sz, vp, vp, u64, vp, vp, vp)
    sig("kronos_cuda_gemv", i32, vp, vp, vp, vp, vp, sz, vp, sz, vp)
    sig("kronos_cuda_moe_route", i32, vp, vp, vp, vp, u32, u32, u32, i32, u32, vp, vp)
    sig("kronos_cuda_linear", i32, vp, vp, vp, sz, vp)
    sig("kronos_cuda_linear_async", i32, vp, vp, vp, sz, vp)
    sig("kronos_cuda_fwht_quant_dev", i32, vp, vp, sz, sz, vp, vp, u64, vp, vp, vp)
    sig("kronos_cuda_linear_noalloc", i32, vp, vp, vp, sz, vp)
    sig("kronos_cuda_gemv_dev", i32, vp, vp, vp, vp, vp, sz, vp, sz, vp)
    sig("kronos_cuda_engine_create", vp, vp, C.POINTER(EngineConfig), vp, C.POINTER(LayerDesc), sz, vp,
        C.POINTER(MatrixDesc), vp)
    sig("kronos_cuda_engine_destroy", None, vp)
    sig("kronos_cuda_engine_forward_tokens", i32, vp, vp, sz, sz, vp, vp)
    sig("kronos_cuda_engine_forward_token_ids", i32, vp, vp, sz, sz, vp, vp)
    sig("kronos_cuda_engine_decode_greedy", i32, vp, u32, sz, sz, vp, vp)
    sig("kronos_cuda_engine_kv_bytes", sz, vp, sz)
    sig("kronos_cuda_engine_weight_bytes", sz, vp)
    sig("kronos_cuda_engine_read_hidden", i32, vp, vp)
    sig("kronos_cuda_engine_read_attention", i32, vp, vp)
    sig("kronos_cuda_engine_read_routes", sz, vp, u32, vp, vp)
    sig("kronos_cuda_engine_tp_handle", i32, vp, vp)
    sig("kronos_cuda_engine_tp_attach", i32, vp, vp, sz)
    sig("kronos_cuda_engine_set_embedding_matrix", i32, vp, C.POINTER(MatrixDesc))
    sig("kronos_cuda_engine_tp_attach_local", i32, vp, C.POINTER(vp), sz)
    sig("kronos_cuda_engine_kv_prefix_bytes", sz, vp, sz, sz)
    sig("kronos_cuda_engine_save_kv_prefix", C.c_int64, vp, sz, sz, vp, sz)
    sig("kronos_cuda_engine_restore_kv_prefix", i32, vp, vp, sz, sz)
    sig("kronos_cuda_engine_reconfigure_kv", i32, vp, u32, sz, sz)
    sig("kronos_cuda_engine_kv_sliding_window", i32, vp, C.POINTER(sz), C.POINTER(sz))
    sig("kronos_cuda_engine_kv_rows", sz, vp)
    sig("kronos_cuda_engine_can_truncate_kv_to", i32, vp, sz, sz)
    sig("kronos_cuda_engine_kv_bytes_per_pos", sz, vp)
    sig("kronos_cuda_engine_kv_export", C.c_int64, vp, sz, sz, vp, sz)
    sig("kronos_cuda_engine_kv_import", i32, vp, vp, sz, sz)
    sig("kronos_cuda_k2tb_open", vp, C.c_char_p)
    sig("kronos_cuda_k2tb_close", None, vp)
    sig("kronos_cuda_k2tb_last_error", C.c_char_p)
    sig("kronos_cuda_k2tb_info", i32, vp, C.POINTER(u32), C.POINTER(u64 * 6), C.POINTER(sz))
    sig("kronos_cuda_k2tb_layer", i32, vp, sz, C.POINTER(LayerDesc), C.POINTER(sz))
    sig("kronos_cuda_k2tb_head", i32, vp, C.POINTER(vp), C.POINTER(sz), C.POINTER(MatrixDesc), C.POINTER(vp), C.POINTER(sz),
        C.POINTER(vp), C.POINTER(sz))
    sig("kronos_cuda_k2tb_embed_nf4", i32, vp, C.POINTER(MatrixDesc))
    sig("kronos_cuda_k2tb_save", i32, C.c_char_p, C.POINTER(u64 * 6), C.POINTER(LayerDesc), sz, sz, sz, sz, vp,
        C.POINTER(MatrixDesc), vp, sz, C.POINTER(MatrixDesc))
    sig("kronos_cuda_engine_decode_trace", sz, vp, vp, sz)
    sig("kronos_cuda_engine_profile_step", C.c_int64, vp, u32, sz, u32, C.c_char_p, sz)
    sig("kronos_cuda_engine_debug_words", sz, vp, vp, sz)
    sig("kronos_cuda_engine_read_kv_q4", i32, vp, u32, u32, sz, vp, vp, vp, vp)
    sig("kronos_cuda_engine_read_kv", i32, vp, u32, u32, sz, vp, vp, vp, vp)
    _LIB = L
    return L


def bipolar_desc(rows, cols, planes, interleaved, bf16_scales):
    d0, d1 = _np(interleaved, np.uint8), _np(bf16_scales, np.uint16)
    desc = MatrixDesc(kind=MATRIX_BIPOLAR, rows=rows, cols=cols, bits=planes, scale_group_chunks=1,
                      data0=d0.ctypes.data, len0=d0.nbytes, data1=d1.ctypes.data, len1=d1.nbytes)
    desc._keep = (d0, d1)
    return desc


def nf_desc(rows, cols, bits, sgc, codebook, pair_stream, tail_stream):
    d0, d1 = _np(pair_stream, np.uint8), _np(tail_stream, np.uint8)
    desc = MatrixDesc(kind=MATRIX_NF, rows=rows, cols=cols, bits=bits, scale_group_chunks=sgc,
                      data0=d0.ctypes.data if d0.size else None, len0=d0.nbytes,
                      data1=d1.ctypes.data if d1.size else None, len1=d1.nbytes)
    cb = _np(codebook, np.int8)
    for i in range(16):
        desc.codebook[i] = int(cb[i])
    desc._keep = (d0, d1)
    return desc


def matrix_image(desc, gate_up_interleave=False):
    """Host-only: the HBM image (records + scales) of a matrix, as a uint8 array."""
    L = load_library()
    flags = UPLOAD_GATE_UP_INTERLEAVE if gate_up_interleave else 0
    n = L.kronos_cuda_matrix_image(C.byref(desc), flags, None, 0)
    if n == 0:
        raise KronosCudaError("malformed matrix descriptor")
    out = np.zeros(n, np.uint8)
    L.kronos_cuda_matrix_image(C.byref(desc), flags, out.ctypes.data_as(C.c_void_p), n)
    return out


def _np(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Matrix:
    """A quantized matrix resident in HBM (KronosCudaMatrix)."""

    def __init__(self, ctx, handle, rows, cols):
        self.ctx, self.handle, self.rows, self.cols = ctx, handle, rows, cols

    @property
    def file_bytes(self):
        return load_library().kronos_cuda_matrix_file_bytes(self.handle)

    @property
    def device_bytes(self):
        return load_library().kronos_cuda_matrix_device_bytes(self.handle)

    def clone(self):
        h = load_library().kronos_cuda_matrix_clone(self.ctx.handle, self.handle)
        if not h:
            raise KronosCudaError(load_library().kronos_cuda_last_error(self.ctx.handle).decode())
        return Matrix(self.ctx, h, self.rows, self.cols)

    def free(self):
        if self.handle:
            load_library().kronos_cuda_matrix_free(self.ctx.handle, self.handle)
            self.handle = None


class Context:
    """One CUDA device + stream (KronosCudaContext)."""

    def __init__(self, device=0):
        self.L = load_library()
        self.handle = self.L.kronos_cuda_context_create(device)
        if not self.handle:
            raise KronosCudaError(self.L.kronos_cuda_last_error(None).decode())

    def close(self):
        if self.handle:
            self.L.kronos_cuda_context_destroy(self.handle)
            self.handle = None

    def _check(self, rc):
        if rc != 0:
            raise KronosCudaError(self.L.kronos_cuda_last_error(self.handle).decode())

    def synchronize(self):
        self._check(self.L.kronos_cuda_synchronize(self.handle))

    @property
    def launch_count(self):
        return self.L.kronos_cuda_launch_count(self.handle)

    def set_stream(self, cuda_stream):
        self._check(self.L.kronos_cuda_set_stream(self.handle, cuda_stream))

    # ---- matrices
    def upload_bipolar(self, rows, cols, planes, interleaved, bf16_scales, gate_up_interleave=False):
        return self._upload(bipolar_desc(rows, cols, planes, interleaved, bf16_scales), rows, cols, gate_up_interleave)

    def upload_nf(self, rows, cols, bits, sgc, codebook, pair_stream, tail_stream, gate_up_interleave=False):
        return self._upload(nf_desc(rows, cols, bits, sgc, codebook, pair_stream, tail_stream), rows, cols,
                            gate_up_interleave)

    def _upload(self, desc, rows, cols, interleave):
        h = self.L.kronos_cuda_matrix_upload(self.handle, C.byref(desc), UPLOAD_GATE_UP_INTERLEAVE if interleave else 0)
        if not h:
            raise KronosCudaError(self.L.kronos_cuda_last_error(self.handle).decode())
        return Matrix(self, h, rows, cols)

    # ---- host-buffer kernels
    def fwht_quant(self, x, norm_w=None, inv_rms=None, chunk0=0):
        x = _np(x, np.float32)
        if x.ndim == 1:
            x = x[None]
        n, cols = x.shape
        q = np.empty((n, cols), np.int8)
        s = np.empty((n, cols // 64), np.float32)
        m = np.empty((n, cols // 64), np.int32)
        w = None if norm_w is None else _np(norm_w, np.float32)
        inv = None if inv_rms is None else _np(np.broadcast_to(np.asarray(inv_rms, np.float32), (n,)), np.float32)
        self._check(self.L.kronos_cuda_fwht_quant(self.handle, _p(x), n, cols, _p(w), _p(inv), chunk0, _p(q), _p(s), _p(m)))
        return q, s, m

    def gemv(self, mat, xq, xs, xsum=None, want_dots=False):
        xq = _np(xq, np.int8).reshape(-1, mat.cols)
        n, nc = xq.shape[0], mat.cols // 64
        xs = _np(xs, np.float32).reshape(n, nc)
        xm = None if xsum is None else _np(xsum, np.int32).reshape(n, nc)
        out = np.empty((n, mat.rows), np.float32)
        dots = np.empty((n, mat.rows, nc), np.int32) if want_dots else None
        self._check(self.L.kronos_cuda_gemv(self.handle, mat.handle, _p(xq), _p(xs), _p(xm), n, _p(out), mat.rows, _p(dots)))
        return (out, dots) if want_dots else out

    def moe_route(self, router_w, x_norm, top_k, router_bias=None, norm_topk=True, scoring=0):
        """(expert ids ascending, weights) of DenseMoeRouter::route_sorted for one normalised hidden vector."""
        w = _np(router_w, np.float32)
        n_experts, hidden = w.shape
        x = _np(x_norm, np.float32).reshape(hidden)
        b = None if router_bias is None else _np(router_bias, np.float32)
        ids, wt = np.zeros(32, np.uint32), np.zeros(32, np.float32)
        k = self.L.kronos_cuda_moe_route(self.handle, _p(w), _p(b), _p(x), n_experts, hidden, top_k, int(norm_topk), scoring, _p(ids), _p(wt))
        if k < 0:
            self._check(-1)
        return ids[:k].copy(), wt[:k].copy()

    def linear(self, mat, x):
        x = _np(x, np.float32).reshape(-1, mat.cols)
        out = np.empty((x.shape[0], mat.rows), np.float32)
        self._check(self.L.kronos_cuda_linear(self.handle, mat.handle, _p(x), x.shape[0], _p(out)))
        return out

    def linear_ptr(self, mat, x_ptr, n_tok, out_ptr):
        """kronos_cuda_linear on raw host addresses (e.g. pinned torch tensors)."""
        self._check(self.L.kronos_cuda_linear(self.handle, mat.handle, x_ptr, n_tok, out_ptr))

    def linear_async_ptr(self, mat, x_ptr, n_tok, out_ptr):
        """kronos_cuda_linear_async: queued, no wait; call synchronize() before reading the output."""
        self._check(self.L.kronos_cuda_linear_async(self.handle, mat.handle, x_ptr, n_tok, out_ptr))

    # ---- device-buffer kernels
    def fwht_quant_dev(self, d_x, n_tok, cols, d_q, d_scales, d_sums, d_norm_w=None, d_inv_rms=None, chunk0=0):
        self._check(self.L.kronos_cuda_fwht_quant_dev(self.handle, d_x, n_tok, cols, d_norm_w, d_inv_rms, chunk0,
                                                      d_q, d_scales, d_sums))

    def linear_noalloc_dev(self, mat, d_x, n_tok, d_out):
        """kronos_cuda_linear_noalloc: device buffers in and out, static scratch, no synchronization."""
        self._check(self.L.kronos_cuda_linear_noalloc(self.handle, mat.handle, d_x, n_tok, d_out))

    def gemv_dev(self, mat, d_xq, d_xs, d_xsum, n_tok, d_out, out_stride=None, d_dots=None):
        self._check(self.L.kronos_cuda_gemv_dev(self.handle, mat.handle, d_xq, d_xs, d_xsum, n_tok, d_out,
                                                out_stride or mat.rows, d_dots))


def desc_of(m):
    """MatrixDesc of a host matrix object with the fields of the file formats: kind 0 (bit-planes: rows, cols,
    planes, data, scales) or kind 2 (NF: rows, cols, bits, sgc, codebook, pair, tail)."""
    if m.kind == MATRIX_BIPOLAR:
        return bipolar_desc(m.rows, m.cols, m.planes, m.data, m.scales)
    return nf_desc(m.rows, m.cols, m.bits, m.sgc, m.codebook, m.pair, m.tail)


class Engine:
    """Whole-token decode engine (KronosCudaEngine).  `spec`: dict with cfg {hidden, layers, n_q, n_kv, head_dim,
    inter, vocab, max_seq, eps[, qk_norm_after_rope]}, layers [{input_norm, post_norm, qkv_bias, q_norm, k_norm,
    qkv, o, gate_up, down}], final_norm, lm_head, rope [max_seq][head_dim], embed_bf16 (or None = tied)."""

    def __init__(self, ctx, spec):
        self.ctx, self.L = ctx, ctx.L
        c = spec["cfg"]
        self.cfg = EngineConfig(C.sizeof(EngineConfig), c["hidden"], c["layers"], c["n_q"], c["n_kv"], c["head_dim"], c["inter"], c["vocab"],
                                c["max_seq"], c["eps"], int(c.get("qk_norm_after_rope", 0)), int(c.get("kv_bits", 8)))
        self.cfg.kv_window, self.cfg.kv_sinks = int(c.get("kv_window", 0)), int(c.get("kv_sinks", 0))
        self.cfg.flags = ENGINE_SPLIT_KV_ATTENTION if c.get("split_kv_attention") else 0
        if int(c.get("tp_size", 1)) > 1:      # a rank of a tensor-parallel group (spec from kronos_2t_b200.tp.shard_spec)
            self.cfg.tp_size, self.cfg.tp_rank, self.cfg.vocab_total = c["tp_size"], c["tp_rank"], c["vocab_total"]
            self.cfg.o_chunk0, self.cfg.down_chunk0 = c["o_chunk0"], c["down_chunk0"]
        if int(c.get("ep_size", 1)) > 1:      # a rank of an expert-parallel group: the whole spec, experts e % ep_size == ep_rank are used
            self.cfg.ep_size, self.cfg.ep_rank = c["ep_size"], c["ep_rank"]
        moes = [ly["moe"] for ly in spec["layers"] if ly.get("moe")]
        if moes:        # one geometry for every MoE layer of a model (MoeGeometry)
            m0 = moes[0]
            assert all(all(m[k] == m0[k] for k in ("n_experts", "top_k", "norm_topk", "d_ff", "bits", "sgc", "expert_bytes")) for m in moes)
            assert all(m.get("scoring", 0) == m0.get("scoring", 0) for m in moes)
            self.cfg.moe_num_experts, self.cfg.moe_top_k = m0["n_experts"], m0["top_k"]
            self.cfg.moe_norm_topk = int(m0["norm_topk"]) | (int(m0.get("scoring", 0)) << 8)
            self.cfg.moe_d_ff, self.cfg.moe_bits, self.cfg.moe_scale_group_chunks = m0["d_ff"], m0["bits"], m0["sgc"]
            self.cfg.moe_expert_bytes = m0["expert_bytes"]
        keep = []

        def vec(a):
            if a is None:
                return None
            a = _np(a, np.float32)
            keep.append(a)
            return a.ctypes.data

        layers = (LayerDesc * c["layers"])()
        for l, ly in enumerate(spec["layers"]):
            d = layers[l]
            d.input_norm, d.post_attn_norm = vec(ly["input_norm"]), vec(ly["post_norm"])
            d.qkv_bias, d.q_norm, d.k_norm = vec(ly.get("qkv_bias")), vec(ly.get("q_norm")), vec(ly.get("k_norm"))
            moe = ly.get("moe")
            if moe:
                shard = _np(moe["shard"], np.uint8)
                keep.append(shard)
                d.moe_router_w, d.moe_router_bias = vec(moe["router_w"]), vec(moe.get("router_bias"))
                d.moe_shard, d.moe_shard_len = shard.ctypes.data, shard.nbytes
            for name, key in (("qkv_proj", "qkv"), ("o_proj", "o")) + (() if moe else (("gate_up_proj", "gate_up"), ("down_proj", "down"))):
                md = desc_of(ly[key])
                keep.append(md._keep)
                setattr(d, name, md)
            if moe and moe.get("shared") is not None:           # the layer's shared expert rides in the dense FFN fields
                for name, key in (("gate_up_proj", "gate_up"), ("down_proj", "down")):
                    md = desc_of(moe["shared"][key])
                    keep.append(md._keep)
                    setattr(d, name, md)
                d.moe_shared_gate_w = vec(moe["shared"].get("gate_w"))
        head = desc_of(spec["lm_head"])
        rope, fn = _np(spec["rope"], np.float32), _np(spec["final_norm"], np.float32)
        emb = None if spec.get("embed_bf16") is None else _np(spec["embed_bf16"], np.uint16)
        self.handle = self.L.kronos_cuda_engine_create(ctx.handle, C.byref(self.cfg), _p(rope), layers, c["layers"],
                                                       _p(fn), C.byref(head), _p(emb))
        if not self.handle:
            raise KronosCudaError(self.L.kronos_cuda_last_error(ctx.handle).decode())
        self.vocab = self.cfg.vocab_total if self.cfg.tp_size > 1 else self.cfg.vocab_size
        if spec.get("embed_matrix") is not None:
            md = desc_of(spec["embed_matrix"])
            self.ctx._check(self.L.kronos_cuda_engine_set_embedding_matrix(self.handle, C.byref(md)))

    def tp_handle(self):
        """This rank's 64-byte inter-process handle of its exchange buffer."""
        buf = np.zeros(64, np.uint8)
        self.ctx._check(self.L.kronos_cuda_engine_tp_handle(self.handle, _p(buf)))
        return buf.tobytes()

    def tp_attach(self, handles):
        """handles: the tp_handle() bytes of every rank, in rank order.  Barrier across the ranks afterwards."""
        blob = np.frombuffer(b"".join(handles), np.uint8).copy()
        self.ctx._check(self.L.kronos_cuda_engine_tp_attach(self.handle, _p(blob), len(handles)))

    def save_kv_prefix(self, n, cur_pos):
        """KvPrefixSnapshot of the first min(n, cur_pos) positions (the whole ring with a sliding window), as a blob."""
        out = np.empty(self.L.kronos_cuda_engine_kv_prefix_bytes(self.handle, n, cur_pos), np.uint8)
        got = self.L.kronos_cuda_engine_save_kv_prefix(self.handle, n, cur_pos, _p(out), out.size)
        if got < 0:
            raise KronosCudaError(self.L.kronos_cuda_last_error(self.ctx.handle).decode())
        return out[:got]

    def restore_kv_prefix(self, blob, copy_slots=None):
        b = _np(blob, np.uint8)
        self.ctx._check(self.L.kronos_cuda_engine_restore_kv_prefix(self.handle, _p(b), b.size, (1 << 63) if copy_slots is None else copy_slots))

    def reconfigure_kv(self, kv_bits, window=0, sinks=0):
        """set_kv_bits + set_kv_sliding_window: a fresh cache in the given format / geometry (continue at position 0)."""
        self.ctx._check(self.L.kronos_cuda_engine_reconfigure_kv(self.handle, kv_bits, window, sinks))
        self.cfg.kv_bits = kv_bits

    @property
    def kv_sliding_window(self):
        """(window, sinks) of the active ring, or None."""
        w, s = C.c_size_t(0), C.c_size_t(0)
        on = self.L.kronos_cuda_engine_kv_sliding_window(self.handle, C.byref(w), C.byref(s))
        return (w.value, s.value) if on == 1 else None

    @property
    def kv_rows(self):
        return self.L.kronos_cuda_engine_kv_rows(self.handle)

    def can_truncate_kv_to(self, cur_pos, target_len):
        return bool(self.L.kronos_cuda_engine_can_truncate_kv_to(self.handle, cur_pos, target_len))

    def tp_attach_local(self, engines):
        """engines: every rank's Engine (same process), in rank order."""
        arr = (C.c_void_p * len(engines))(*[e.handle for e in engines])
        self.ctx._check(self.L.kronos_cuda_engine_tp_attach_local(self.handle, arr, len(engines)))

    def close(self):
        if self.handle:
            self.L.kronos_cuda_engine_destroy(self.handle)
            self.handle = None

    def forward_tokens(self, embeds, pos_start=0, want_all=False):
        e = _np(embeds, np.float32).reshape(-1, self.cfg.hidden_size)
        n, v = e.shape[0], self.vocab
        last = np.empty(v, np.float32)
        allv = np.empty((n, v), np.float32) if want_all else None
        self.ctx._check(self.L.kronos_cuda_engine_forward_tokens(self.handle, _p(e), n, pos_start, _p(allv), _p(last)))
        return allv if want_all else last

    def forward_token_ids(self, tokens, pos_start=0, want_all=False):
        t = _np(tokens, np.uint32).reshape(-1)
        n, v = t.size, self.vocab
        last = np.empty(v, np.float32)
        allv = np.empty((n, v), np.float32) if want_all else None
        self.ctx._check(self.L.kronos_cuda_engine_forward_token_ids(self.handle, _p(t), n, pos_start, _p(allv), _p(last)))
        return allv if want_all else last

    def decode_greedy(self, first_token, pos_start, n_steps, want_logits=False):
        out = np.empty(n_steps, np.uint32)
        logits = np.empty(self.vocab, np.float32) if want_logits else None
        self.ctx._check(self.L.kronos_cuda_engine_decode_greedy(self.handle, int(first_token), pos_start, n_steps, _p(out),
                                                                _p(logits)))
        return (out, logits) if want_logits else out

    def kv_bytes(self, positions):
        return self.L.kronos_cuda_engine_kv_bytes(self.handle, positions)

    @property
    def weight_bytes(self):
        return self.L.kronos_cuda_engine_weight_bytes(self.handle)

    def read_hidden(self):
        out = np.empty(self.cfg.hidden_size, np.float32)
        self.ctx._check(self.L.kronos_cuda_engine_read_hidden(self.handle, _p(out)))
        return out

    @property
    def kv_bytes_per_pos(self):
        return self.L.kronos_cuda_engine_kv_bytes_per_pos(self.handle)

    def kv_export(self, lo, hi):
        """Positions [lo, hi) as a blob in the reference's position-major format."""
        out = np.empty((hi - lo) * self.kv_bytes_per_pos, np.uint8)
        n = self.L.kronos_cuda_engine_kv_export(self.handle, lo, hi, _p(out), out.size)
        if n < 0:
            raise KronosCudaError(self.L.kronos_cuda_last_error(self.ctx.handle).decode())
        return out[:n]

    def kv_import(self, blob, n):
        b = _np(blob, np.uint8)
        self.ctx._check(self.L.kronos_cuda_engine_kv_import(self.handle, _p(b), b.size, n))

    def read_routes(self, layer):
        e, w = np.zeros(32, np.uint32), np.zeros(32, np.float32)
        k = self.L.kronos_cuda_engine_read_routes(self.handle, layer, _p(e), _p(w))
        return e[:k].copy(), w[:k].copy()

    def read_attention(self):
        out = np.empty(self.cfg.num_attention_heads * self.cfg.head_dim, np.float32)
        self.ctx._check(self.L.kronos_cuda_engine_read_attention(self.handle, _p(out)))
        return out

    def decode_trace(self):
        """Global-timer marks (ns) of the last step of the last whole-token-kernel decode call."""
        buf = np.zeros(4096, np.uint64)
        n = self.L.kronos_cuda_engine_decode_trace(self.handle, _p(buf), buf.size)
        return buf[:n].copy()

    def profile_step(self, token, pos, reps=16):
        """Per-kernel-class timing table (text) of one greedy step at position `pos`, averaged over `reps` replays."""
        buf = C.create_string_buffer(1 << 14)
        n = self.L.kronos_cuda_engine_profile_step(self.handle, int(token), pos, reps, buf, len(buf))
        if n < 0:
            raise KronosCudaError(self.L.kronos_cuda_last_error(self.ctx.handle).decode())
        return buf.value.decode()

    def debug_words(self):
        buf = np.zeros(32, np.uint64)
        n = self.L.kronos_cuda_engine_debug_words(self.handle, _p(buf), buf.size)
        return buf[:n].copy()

    def read_kv(self, layer, kv_head, position):
        """(k_q8, k_scale, v_q8, v_scale) of one cache slot."""
        hd = self.cfg.head_dim
        if self.cfg.kv_bits == 4:
            k, v = np.empty(hd // 2, np.uint8), np.empty(hd // 2, np.uint8)
            ks, vs = np.empty(hd // 64, np.uint16), np.empty(hd // 64, np.uint16)
            self.ctx._check(self.L.kronos_cuda_engine_read_kv_q4(self.handle, layer, kv_head, position, _p(k), _p(ks), _p(v), _p(vs)))
            return k, ks, v, vs
        k, v = np.empty(hd, np.int8), np.empty(hd, np.int8)
        ks, vs = np.empty(1, np.float32), np.empty(1, np.float32)
        self.ctx._check(self.L.kronos_cuda_engine_read_kv(self.handle, layer, kv_head, position, _p(k), _p(ks), _p(v), _p(vs)))
        return k, float(ks[0]), v, float(vs[0])


# ---- .k2tb container (host only)
class _HostMatrix:
    """Matrix read from a container: the fields desc_of (and the CPU oracle) read."""

    def __init__(self, d):
        self.kind, self.rows, self.cols = d.kind, d.rows, d.cols
        a = np.ctypeslib.as_array(C.cast(d.data0, C.POINTER(C.c_uint8)), shape=(d.len0,)).copy() if d.len0 else np.zeros(0, np.uint8)
        b = np.ctypeslib.as_array(C.cast(d.data1, C.POINTER(C.c_uint8)), shape=(d.len1,)).copy() if d.len1 else np.zeros(0, np.uint8)
        if d.kind == MATRIX_BIPOLAR:
            self.planes, self.data, self.scales = d.bits, a, b.view(np.uint16)
        else:
            self.bits, self.sgc, self.pair, self.tail = d.bits, d.scale_group_chunks, a, b
            self.codebook = np.array([d.codebook[i] for i in range(16)], np.int8)

    def file_bytes(self):
        return self.data.nbytes + self.scales.nbytes if self.kind == MATRIX_BIPOLAR else self.pair.nbytes + self.tail.nbytes + 16


def _f32(ptr, n):
    return None if not ptr or n == 0 else np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(n,)).copy()


def k2tb_load(path, cfg, rope):
    """Reads a .k2tb dense container into an engine spec (cfg = shapes from the model's config.json, rope = its rope table).
    Returns (spec, version, mode_words)."""
    L = load_library()
    h = L.kronos_cuda_k2tb_open(os.fsencode(path))
    if not h:
        raise KronosCudaError(L.kronos_cuda_k2tb_last_error().decode())
    try:
        ver, mode, nl = C.c_uint32(), (C.c_uint64 * 6)(), C.c_size_t()
        L.kronos_cuda_k2tb_info(h, C.byref(ver), C.byref(mode), C.byref(nl))
        hd, hid = cfg["head_dim"], cfg["hidden"]
        layers = []
        for l in range(nl.value):
            d, nb = LayerDesc(), C.c_size_t()
            L.kronos_cuda_k2tb_layer(h, l, C.byref(d), C.byref(nb))
            layers.append(dict(input_norm=_f32(d.input_norm, hid), post_norm=_f32(d.post_attn_norm, hid), qkv_bias=_f32(d.qkv_bias, nb.value),
                               q_norm=_f32(d.q_norm, hd), k_norm=_f32(d.k_norm, hd), qkv=_HostMatrix(d.qkv_proj), o=_HostMatrix(d.o_proj),
                               gate_up=_HostMatrix(d.gate_up_proj), down=_HostMatrix(d.down_proj)))
        fn, fnl, emb, embl, ef, efl = C.c_void_p(), C.c_size_t(), C.c_void_p(), C.c_size_t(), C.c_void_p(), C.c_size_t()
        head = MatrixDesc()
        L.kronos_cuda_k2tb_head(h, C.byref(fn), C.byref(fnl), C.byref(head), C.byref(emb), C.byref(embl), C.byref(ef), C.byref(efl))
        embed = None
        if embl.value:
            embed = np.ctypeslib.as_array(C.cast(emb, C.POINTER(C.c_uint16)), shape=(embl.value,)).copy()
        spec = dict(cfg=dict(cfg, layers=nl.value), layers=layers, final_norm=_f32(fn, fnl.value), lm_head=_HostMatrix(head), rope=rope,
                    embed_bf16=embed)
        table = MatrixDesc()
        if L.kronos_cuda_k2tb_embed_nf4(h, C.byref(table)) == 1:      # the untied table as an NF4 matrix: the engine embeds from it
            spec["embed_matrix"] = _HostMatrix(table)
        return spec, ver.value, [int(x) for x in mode]
    finally:
        L.kronos_cuda_k2tb_close(h)


def moe_load(core_path, shard_path, cfg, rope):
    """load_moe_from_files (real_llm.rs:5166-5519): reads a K2TKRONOS5 core and its .k2tm expert shard into an engine spec.
    cfg = shapes and routing from the model's config.json (hidden, heads, ..., plus moe_top_k, moe_norm_topk[, moe_scoring]);
    the shard stays mapped (the spec's `shard` arrays are views into it) until the returned `close()` is called, so build the
    engine first.  Returns (spec, header_words, close)."""
    L = load_library()
    u64, sz, vp = C.c_uint64, C.c_size_t, C.c_void_p
    for name, res, args in (("kronos_cuda_k2tb_moe_info", C.c_int32, [vp, C.POINTER(u64), C.POINTER(u64)]),
                            ("kronos_cuda_k2tb_moe_layer", C.c_int32, [vp, sz, C.POINTER(u64), C.POINTER(u64), C.POINTER(u64)]),
                            ("kronos_cuda_k2tm_open", vp, [C.c_char_p]), ("kronos_cuda_k2tm_close", None, [vp]),
                            ("kronos_cuda_k2tm_info", C.c_int32, [vp, C.POINTER(u64 * 7)]),
                            ("kronos_cuda_k2tm_layer", C.c_int32, [vp, sz, C.POINTER(vp), C.POINTER(sz)])):
        f = getattr(L, name)
        f.restype, f.argtypes = res, args
    h = L.kronos_cuda_k2tb_open(os.fsencode(core_path))
    if not h:
        raise KronosCudaError(L.kronos_cuda_k2tb_last_error().decode())
    tm = L.kronos_cuda_k2tm_open(os.fsencode(shard_path))
    if not tm:
        L.kronos_cuda_k2tb_close(h)
        raise KronosCudaError(L.kronos_cuda_k2tb_last_error().decode())
    try:
        ver, mode, nl = C.c_uint32(), (u64 * 6)(), sz()
        L.kronos_cuda_k2tb_info(h, C.byref(ver), C.byref(mode), C.byref(nl))
        if ver.value != 5:
            raise KronosCudaError("moe_load: the core file is not a K2TKRONOS5 container")
        words = (u64 * 7)()
        L.kronos_cuda_k2tm_info(tm, C.byref(words))
        n_moe_layers, experts, d_model, d_ff, sgc, rec, bits = [int(w) for w in words]
        ebits, esgc = u64(), u64()
        L.kronos_cuda_k2tb_moe_info(h, C.byref(ebits), C.byref(esgc))
        if d_model != cfg["hidden"] or ebits.value != bits or esgc.value != sgc:
            raise KronosCudaError("moe_load: core and expert shard disagree (hidden size, expert bits or scale group)")
        hd, hid = cfg["head_dim"], cfg["hidden"]
        layers = []
        for l in range(nl.value):
            d, nb = LayerDesc(), sz()
            if L.kronos_cuda_k2tb_layer(h, l, C.byref(d), C.byref(nb)) != 0:
                raise KronosCudaError(L.kronos_cuda_k2tb_last_error().decode())
            ly = dict(input_norm=_f32(d.input_norm, hid), post_norm=_f32(d.post_attn_norm, hid), qkv_bias=_f32(d.qkv_bias, nb.value),
                      q_norm=_f32(d.q_norm, hd), k_norm=_f32(d.k_norm, hd), qkv=_HostMatrix(d.qkv_proj), o=_HostMatrix(d.o_proj))
            slot, n_exp, r_hid = u64(), u64(), u64()
            if L.kronos_cuda_k2tb_moe_layer(h, l, C.byref(slot), C.byref(n_exp), C.byref(r_hid)) == 1:
                if n_exp.value != experts or r_hid.value != hid or slot.value >= n_moe_layers:
                    raise KronosCudaError(f"moe_load: layer {l}: router shape or shard slot does not match the expert shard")
                ptr, ln = vp(), sz()
                L.kronos_cuda_k2tm_layer(tm, slot.value, C.byref(ptr), C.byref(ln))
                shard = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(ln.value,))        # a view into the mapping
                ly["gate_up"] = ly["down"] = None
                ly["moe"] = dict(router_w=_f32(d.moe_router_w, experts * hid), router_bias=_f32(d.moe_router_bias, experts), n_experts=experts,
                                 top_k=cfg["moe_top_k"], norm_topk=bool(cfg.get("moe_norm_topk", True)), d_ff=d_ff, bits=bits, sgc=sgc, shard=shard,
                                 expert_bytes=rec, scoring=int(cfg.get("moe_scoring", 0)))
                if d.gate_up_proj.rows:         # the layer's shared expert
                    ly["moe"]["shared"] = dict(gate_up=_HostMatrix(d.gate_up_proj), down=_HostMatrix(d.down_proj), gate_w=_f32(d.moe_shared_gate_w, hid))
            else:
                ly.update(gate_up=_HostMatrix(d.gate_up_proj), down=_HostMatrix(d.down_proj))
            layers.append(ly)
        fn, fnl, emb, embl, ef, efl = vp(), sz(), vp(), sz(), vp(), sz()
        head = MatrixDesc()
        L.kronos_cuda_k2tb_head(h, C.byref(fn), C.byref(fnl), C.byref(head), C.byref(emb), C.byref(embl), C.byref(ef), C.byref(efl))
        embed = np.ctypeslib.as_array(C.cast(emb, C.POINTER(C.c_uint16)), shape=(embl.value,)).copy() if embl.value else None
        spec = dict(cfg=dict(cfg, layers=nl.value), layers=layers, final_norm=_f32(fn, fnl.value), lm_head=_HostMatrix(head), rope=rope, embed_bf16=embed)
        L.kronos_cuda_k2tb_close(h)
        h = None
        return spec, [int(w) for w in words], (lambda: L.kronos_cuda_k2tm_close(tm))
    except Exception:
        L.kronos_cuda_k2tm_close(tm)
        raise
    finally:
        if h:
            L.kronos_cuda_k2tb_close(h)


def k2tb_save(path, spec, mode_words):
    """Writes an engine spec as a .k2tb dense container (version chosen as the reference's save_bipolar does)."""
    L = load_library()
    c = spec["cfg"]
    keep = []

    def vec(a):
        if a is None:
            return None
        a = _np(a, np.float32)
        keep.append(a)
        return a.ctypes.data

    layers = (LayerDesc * len(spec["layers"]))()
    for l, ly in enumerate(spec["layers"]):
        d = layers[l]
        d.input_norm, d.post_attn_norm = vec(ly["input_norm"]), vec(ly["post_norm"])
        d.qkv_bias, d.q_norm, d.k_norm = vec(ly.get("qkv_bias")), vec(ly.get("q_norm")), vec(ly.get("k_norm"))
        for name, key in (("qkv_proj", "qkv"), ("o_proj", "o"), ("gate_up_proj", "gate_up"), ("down_proj", "down")):
            md = desc_of(ly[key])
            keep.append(md._keep)
            setattr(d, name, md)
    head = desc_of(spec["lm_head"])
    fn = _np(spec["final_norm"], np.float32)
    emb = None if spec.get("embed_bf16") is None else _np(spec["embed_bf16"], np.uint16).reshape(-1)
    words = (C.c_uint64 * 6)(*mode_words)
    qkv_rows = (c["n_q"] + 2 * c["n_kv"]) * c["head_dim"]
    table = None if spec.get("embed_matrix") is None else desc_of(spec["embed_matrix"])
    rc = L.kronos_cuda_k2tb_save(os.fsencode(path), C.byref(words), layers, len(spec["layers"]), c["hidden"], qkv_rows, c["head_dim"], _p(fn),
                                 C.byref(head), _p(emb), 0 if emb is None else emb.size, None if table is None else C.byref(table))
    if rc != 0:
        raise KronosCudaError(L.kronos_cuda_k2tb_last_error().decode())
