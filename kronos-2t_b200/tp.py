"""Tensor-parallel sharding of a dense model spec (host logic, numpy only).

The reference runs on one device; its compiled matrices are sliced here IN THEIR FILE FORMATS, so a rank uploads
ordinary FusedBipolar / NF matrices and nothing is re-quantized:

  qkv_proj   column-parallel: the rows of this rank's query heads, key heads and value heads, concatenated [q; k; v]
  o_proj     row-parallel:    the columns (64-column chunks) of this rank's query heads        -> partial output, summed
  gate_up    column-parallel: this rank's gate rows and up rows, concatenated [gate; up]
  down_proj  row-parallel:    the chunks of this rank's MLP columns                            -> partial output, summed
  lm_head    column-parallel: a contiguous block of vocabulary rows                            -> logits slice, gathered

Row slices fall on 16-row stripes (bit-planes) or 32-row stripe pairs (NF); column slices fall on 64-column chunks
(and on whole scale groups for g128 matrices).  The activations of the row-parallel projections keep their GLOBAL chunk
index for the rotation (`o_chunk0`, `down_chunk0` in the rank's cfg), so every rank quantizes exactly the bytes the
single-device engine would.  Partial outputs are summed in rank order, which differs from the single-device fp32 chain
over all chunks only by rounding.
"""
import numpy as np

from .synth import HostMatrix

_NF_CHUNK = {5: 640, 4: 512, 3: 384, 2: 256}


def _check(cond, msg):
    if not cond:
        raise ValueError(msg)


def rows_slice(m, r0, r1):
    """Rows [r0, r1) of a file-format matrix."""
    _check(0 <= r0 < r1 <= m.rows, "row range out of bounds")
    if m.kind == 0:
        _check(r0 % 16 == 0 and (r1 % 16 == 0 or r1 == m.rows), "bit-plane matrices are sliced on 16-row stripes")
        ns = (m.rows + 15) // 16
        data = np.asarray(m.data, np.uint8).reshape(ns, -1)[r0 // 16:(r1 + 15) // 16]
        scales = np.asarray(m.scales, np.uint16).reshape(ns, -1)[r0 // 16:(r1 + 15) // 16]
        return HostMatrix(kind=0, rows=r1 - r0, cols=m.cols, planes=m.planes, data=np.ascontiguousarray(data).reshape(-1),
                          scales=np.ascontiguousarray(scales).reshape(-1))
    _check(m.rows % 32 == 0 and np.asarray(m.tail).size == 0, "NF matrices with an odd stripe count cannot be row-sliced")
    _check(r0 % 32 == 0 and r1 % 32 == 0, "NF matrices are sliced on 32-row stripe pairs")
    pair = np.asarray(m.pair, np.uint8).reshape(m.rows // 32, -1)[r0 // 32:r1 // 32]
    return HostMatrix(kind=2, rows=r1 - r0, cols=m.cols, bits=m.bits, sgc=m.sgc, codebook=np.asarray(m.codebook, np.int8).copy(),
                      pair=np.ascontiguousarray(pair).reshape(-1), tail=np.zeros(0, np.uint8))


def rows_concat(parts):
    """Row concatenation of matrices of one format and width."""
    a = parts[0]
    _check(all(p.kind == a.kind and p.cols == a.cols for p in parts), "rows_concat: mixed formats")
    rows = sum(p.rows for p in parts)
    if a.kind == 0:
        _check(all(p.planes == a.planes for p in parts) and all(p.rows % 16 == 0 for p in parts[:-1]), "rows_concat: stripe alignment")
        return HostMatrix(kind=0, rows=rows, cols=a.cols, planes=a.planes, data=np.concatenate([np.asarray(p.data, np.uint8) for p in parts]),
                          scales=np.concatenate([np.asarray(p.scales, np.uint16) for p in parts]))
    _check(all(p.bits == a.bits and p.sgc == a.sgc and np.array_equal(p.codebook, a.codebook) and np.asarray(p.tail).size == 0 for p in parts),
           "rows_concat: NF parts must share bits, scale groups and codebook")
    return HostMatrix(kind=2, rows=rows, cols=a.cols, bits=a.bits, sgc=a.sgc, codebook=np.asarray(a.codebook, np.int8).copy(),
                      pair=np.concatenate([np.asarray(p.pair, np.uint8) for p in parts]), tail=np.zeros(0, np.uint8))


def cols_slice(m, c0, c1):
    """Chunks [c0, c1) (64 columns each) of a file-format matrix."""
    nc = m.cols // 64
    _check(0 <= c0 < c1 <= nc, "chunk range out of bounds")
    if m.kind == 0:
        ns = (m.rows + 15) // 16
        data = np.asarray(m.data, np.uint8).reshape(ns, m.cols // 8, m.planes * 16)[:, c0 * 8:c1 * 8]
        scales = np.asarray(m.scales, np.uint16).reshape(ns, nc, 16)[:, c0:c1]
        return HostMatrix(kind=0, rows=m.rows, cols=(c1 - c0) * 64, planes=m.planes, data=np.ascontiguousarray(data).reshape(-1),
                          scales=np.ascontiguousarray(scales).reshape(-1))
    sgc, cb = m.sgc, _NF_CHUNK[m.bits]
    _check(m.rows % 32 == 0 and np.asarray(m.tail).size == 0, "NF matrices with an odd stripe count cannot be column-sliced")
    _check(nc % sgc == 0 and c0 % sgc == 0 and c1 % sgc == 0, "NF matrices are column-sliced on whole scale groups")
    group = 64 + sgc * 2 * cb
    pair = np.asarray(m.pair, np.uint8).reshape(m.rows // 32, nc // sgc, group)[:, c0 // sgc:c1 // sgc]
    return HostMatrix(kind=2, rows=m.rows, cols=(c1 - c0) * 64, bits=m.bits, sgc=sgc, codebook=np.asarray(m.codebook, np.int8).copy(),
                      pair=np.ascontiguousarray(pair).reshape(-1), tail=np.zeros(0, np.uint8))


def head_plan(n_q, n_kv, tp, rank):
    """Attention heads of `rank`: (first query head, query heads, first kv head, kv heads).

    tp <= n_kv: every rank takes n_kv / tp kv heads and their query groups.  tp > n_kv (more ranks than kv heads, e.g. the
    28 / 4 heads of Qwen2-7B eight ways): tp / n_kv ranks share one kv head - each keeps its own copy of that head's key /
    value rows and cache - and divide the group's query heads among them as evenly as possible (7 -> 4 + 3), so the
    o_proj columns of a rank are still one contiguous run of chunks."""
    _check(0 <= rank < tp, "rank out of range")
    group = n_q // n_kv
    _check(n_q % n_kv == 0, "query heads must be a multiple of the kv heads")
    if tp <= n_kv:
        _check(n_kv % tp == 0, f"{n_kv} kv heads do not split {tp} ways")
        nkv_l = n_kv // tp
        return rank * nkv_l * group, nkv_l * group, rank * nkv_l, nkv_l
    _check(tp % n_kv == 0, f"{tp} ranks do not divide over {n_kv} kv heads")
    per = tp // n_kv                              # ranks that share a kv head
    _check(group >= per, "more ranks per kv head than query heads in a group")
    kvh, j = rank // per, rank % per
    base, extra = group // per, group % per
    first = j * base + min(j, extra)
    return kvh * group + first, base + (1 if j < extra else 0), kvh, 1


def shard_spec(spec, tp, rank):
    """The rank-local engine spec of `spec` under tp-way tensor parallelism (tp = 1 returns an equivalent spec)."""
    c = spec["cfg"]
    hd, n_q, n_kv, inter, vocab = c["head_dim"], c["n_q"], c["n_kv"], c["inter"], c["vocab"]
    qh0, nq_l, kvh0, nkv_l = head_plan(n_q, n_kv, tp, rank)
    _check(inter % (64 * tp) == 0 and vocab % (32 * tp) == 0, "MLP width / vocabulary do not split on chunk / stripe boundaries")
    inter_l, vocab_l = inter // tp, vocab // tp
    q_dim, kv_dim = n_q * hd, n_kv * hd
    q0, k0, v0 = qh0 * hd, q_dim + kvh0 * hd, q_dim + kv_dim + kvh0 * hd
    qkv_rows = np.concatenate([np.arange(q0, q0 + nq_l * hd), np.arange(k0, k0 + nkv_l * hd), np.arange(v0, v0 + nkv_l * hd)])
    layers = []
    for ly in spec["layers"]:
        _check(not ly.get("moe"), "sparse-MoE layers shard by experts, not by columns")
        layers.append(dict(
            input_norm=ly["input_norm"], post_norm=ly["post_norm"], q_norm=ly.get("q_norm"), k_norm=ly.get("k_norm"),
            qkv_bias=None if ly.get("qkv_bias") is None else np.ascontiguousarray(np.asarray(ly["qkv_bias"], np.float32)[qkv_rows]),
            qkv=rows_concat([rows_slice(ly["qkv"], q0, q0 + nq_l * hd), rows_slice(ly["qkv"], k0, k0 + nkv_l * hd),
                             rows_slice(ly["qkv"], v0, v0 + nkv_l * hd)]),
            o=cols_slice(ly["o"], qh0 * hd // 64, (qh0 + nq_l) * hd // 64),
            gate_up=rows_concat([rows_slice(ly["gate_up"], rank * inter_l, (rank + 1) * inter_l),
                                 rows_slice(ly["gate_up"], inter + rank * inter_l, inter + (rank + 1) * inter_l)]),
            down=cols_slice(ly["down"], rank * inter_l // 64, (rank + 1) * inter_l // 64)))
    cfg = dict(c, n_q=nq_l, n_kv=nkv_l, inter=inter_l, vocab=vocab_l, o_chunk0=qh0 * hd // 64, down_chunk0=rank * inter_l // 64,
               tp_size=tp, tp_rank=rank, vocab_total=vocab)
    out = dict(cfg=cfg, layers=layers, final_norm=spec["final_norm"], lm_head=rows_slice(spec["lm_head"], rank * vocab_l, (rank + 1) * vocab_l),
               rope=spec["rope"], embed_bf16=spec.get("embed_bf16"))
    if spec.get("embed_bf16") is None:
        out["embed_matrix"] = spec["lm_head"]        # tied embeddings: every rank keeps the whole lm_head for the lookup
    return out
