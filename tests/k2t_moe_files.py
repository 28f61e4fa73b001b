"""Writer of the two files of a compiled sparse-MoE model, written here from the reference's readers (the K2TKRONOS5 core of
RealLlamaEngine::load_moe_from_files, src/model/real_llm.rs:5166-5519, and the .k2tm expert shard of K2tmShardHeader,
src/model/moe_800b.rs:790-854) - independent of the library's own reader, which the tests check against it."""
import struct

import numpy as np


def _u64(v):
    return struct.pack("<Q", int(v))


def _f32s(a):
    if a is None:
        return _u64(0)
    a = np.ascontiguousarray(a, np.float32).reshape(-1)
    return _u64(a.size) + a.tobytes()


def _matrix(m):
    if m.kind == 0:
        return (_u64(0) + _u64(m.rows) + _u64(m.cols) + _u64(m.planes) + _u64(m.data.nbytes) + np.ascontiguousarray(m.data, np.uint8).tobytes() +
                _u64(m.scales.size) + np.ascontiguousarray(m.scales, np.uint16).tobytes())
    return (_u64(2) + _u64(m.rows) + _u64(m.cols) + _u64(m.bits) + _u64(m.sgc) + np.ascontiguousarray(m.codebook, np.int8).tobytes() +
            _u64(m.pair.nbytes) + np.ascontiguousarray(m.pair, np.uint8).tobytes() + _u64(m.tail.nbytes) + np.ascontiguousarray(m.tail, np.uint8).tobytes())


def write_moe_files(core_path, shard_path, spec, mode_words, lookahead_layers=()):
    """spec: an engine spec whose MoE layers carry ly["moe"] (tests/k2t_models.build with moe=...).  MoE layers get the shard
    slots 0, 1, ... in layer order.  lookahead_layers: layers that also carry a (dummy) lookahead projector, which readers skip."""
    moes = [ly["moe"] for ly in spec["layers"] if ly.get("moe")]
    m0 = moes[0]
    hidden = spec["cfg"]["hidden"]
    out = [b"K2TKRONOS5\n"] + [_u64(w) for w in mode_words] + [_u64(m0["bits"]), _u64(m0["sgc"]), _u64(len(spec["layers"]))]
    slot = 0
    for l, ly in enumerate(spec["layers"]):
        out += [_f32s(ly["input_norm"]), _f32s(ly["post_norm"]), _f32s(ly.get("qkv_bias")), _f32s(None), _f32s(ly.get("q_norm")), _f32s(ly.get("k_norm")),
                _matrix(ly["qkv"]), _matrix(ly["o"])]
        moe = ly.get("moe")
        if moe:
            out += [_u64(1), _u64(slot), _u64(moe["n_experts"]), _u64(hidden), _f32s(moe["router_w"]), _f32s(moe.get("router_bias"))]
            sh = moe.get("shared")
            if sh is None:
                out += [_u64(0)]
            else:           # shared expert: inter, gate weight (may be empty), gate_up and down as NF matrices (real_llm.rs:5097-5114)
                out += [_u64(1), _u64(sh["down"].cols), _f32s(sh.get("gate_w")), _matrix(sh["gate_up"]), _matrix(sh["down"])]
            if l in lookahead_layers:
                out += [_u64(1), _u64(l + 1), _u64(hidden), _u64(2), _f32s(np.zeros(2 * hidden)), _f32s(np.zeros(2 * hidden))]
            else:
                out += [_u64(0)]
            slot += 1
        else:
            out += [_u64(0), _matrix(ly["gate_up"]), _matrix(ly["down"])]
    out += [_f32s(spec["final_norm"]), _matrix(spec["lm_head"]), _f32s(None)]
    emb = spec.get("embed_bf16")
    out += [_u64(0) if emb is None else _u64(np.asarray(emb).size) + np.ascontiguousarray(emb, np.uint16).tobytes(), _u64(0)]
    with open(core_path, "wb") as f:
        f.write(b"".join(out))
    page = bytearray(16384)
    page[0:12] = b"K2TM800B_V1\0"
    words = [len(moes), m0["n_experts"], hidden, m0["d_ff"], m0["sgc"], m0["expert_bytes"], m0["bits"]]
    page[16:16 + 56] = b"".join(_u64(w) for w in words)
    with open(shard_path, "wb") as f:
        f.write(bytes(page))
        for m in moes:
            f.write(np.ascontiguousarray(m["shard"], np.uint8).tobytes())
    return words
