"""Synthetic matrices in the reference's file formats, built without any quantizer: uniformly random
codes / indices and bf16 scales in [2^-15, 2^-7).  GEMV time does not depend on the code values;
files produced this way are valid inputs for kronos_cuda_matrix_upload (and for the oracle)."""
import numpy as np

NF4_DEFAULT = np.array([-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127], np.int8)
NF3_DEFAULT = np.array([-127, -79, -45, -14, 14, 45, 79, 127, 0, 0, 0, 0, 0, 0, 0, 0], np.int8)
_NF_CHUNK = {5: 640, 4: 512, 3: 384, 2: 256}


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def random_bipolar_bytes(seed, rows, cols, planes):
    """(interleaved planes u8, bf16 scales u16) of a FusedBipolarLutMatrix with random codes."""
    ns, nc = (rows + 15) // 16, cols // 64
    rng = _rng(seed)
    data = rng.integers(0, 256, ns * (cols // 8) * planes * 16, dtype=np.uint8)
    scales = rng.integers(0x3800, 0x3C00, ns * nc * 16, dtype=np.uint16)
    return data, scales


def random_nf_bytes(seed, rows, cols, bits, sgc):
    """(pair_stream, tail_stream) of an NfSdotMatrix with random indices; rows % 32 == 0, (cols/64) % sgc == 0."""
    nc = cols // 64
    assert rows % 32 == 0 and nc % sgc == 0
    nsg, cb = nc // sgc, _NF_CHUNK[bits]
    rng = _rng(seed)
    blk = 64 + sgc * 2 * cb
    stream = rng.integers(0, 256, (rows // 32) * nsg * blk, dtype=np.uint8).reshape(rows // 32, nsg, blk)
    sc = rng.integers(0x3800, 0x3C00, (rows // 32, nsg, 32), dtype=np.uint16)
    stream[:, :, :64] = sc.view(np.uint8).reshape(rows // 32, nsg, 64)
    return stream.reshape(-1), np.zeros(0, np.uint8)


def file_bytes(kind, rows, cols, bits, sgc=1):
    """Bytes of a matrix in the reference file format (the algorithmic weight bytes of one GEMV)."""
    ns, nc = (rows + 15) // 16, cols // 64
    if kind == "bipolar":
        return ns * (cols // 8) * bits * 16 + ns * nc * 16 * 2
    nsg, cb = -(-nc // sgc), _NF_CHUNK[bits]
    return (ns // 2) * (nsg * 64 + nc * 2 * cb) + (ns & 1) * (nsg * 32 + nc * cb) + 16


class HostMatrix:
    """A matrix in the reference file format: the fields kronos_2t_b200.ffi.desc_of (and the oracle) read."""

    def __init__(self, **kw):
        self.__dict__.update(kw)

    def file_bytes(self):
        if self.kind == 0:
            return self.data.nbytes + self.scales.nbytes
        return self.pair.nbytes + self.tail.nbytes + 16


def random_matrix(seed, rows, cols, mode):
    """mode: b4 / b5 / b6 / nf4 / nf4g128 / nf3 / nf3g128."""
    if mode.startswith("b"):
        planes = int(mode[1])
        data, scales = random_bipolar_bytes(seed, rows, cols, planes)
        return HostMatrix(kind=0, rows=rows, cols=cols, planes=planes, data=data, scales=scales)
    bits, sgc = int(mode[2]), 2 if mode.endswith("g128") else 1
    if (cols // 64) % sgc:
        sgc = 1
    pair, tail = random_nf_bytes(seed, rows, cols, bits, sgc)
    return HostMatrix(kind=2, rows=rows, cols=cols, bits=bits, sgc=sgc, codebook=NF4_DEFAULT if bits == 4 else NF3_DEFAULT,
                      pair=pair, tail=tail)


def rope_table(max_seq, head_dim, theta):
    """build_rope_table (src/model/real_llm.rs:9212-9236): rows [cos(hd/2), sin(hd/2)], inv_freq in f64 -> f32."""
    half = head_dim // 2
    inv_freq = (1.0 / np.power(float(theta), (2.0 * np.arange(half)) / head_dim)).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


SMOLLM2_135M = dict(hidden=576, layers=30, n_q=9, n_kv=3, head_dim=64, inter=1536, vocab=49152, max_seq=512, eps=1e-5, theta=1e5)


SMOLLM2_1_7B = dict(hidden=2048, layers=24, n_q=32, n_kv=32, head_dim=64, inter=8192, vocab=49152, max_seq=8192 + 64, eps=1e-5, theta=1.3e5)
QWEN2_7B = dict(hidden=3584, layers=28, n_q=28, n_kv=4, head_dim=128, inter=18944, vocab=152064, max_seq=4096 + 64, eps=1e-6, theta=1e6)
P55454 = dict(qkv="b5", o="b5", gate_up="b4", down="b5", head="b4")     # the reference's mixed-plane tier pQOGDH


def random_bf16(seed, n, lo=0x3800, hi=0x3C00):
    """n bf16 values of random sign with magnitudes in [2^-15, 2^-7)."""
    rng = _rng(seed)
    return (rng.integers(lo, hi, n, dtype=np.uint16) | (rng.integers(0, 2, n, dtype=np.uint16) << 15)).astype(np.uint16)


QWEN3_30B_A3B = dict(hidden=2048, layers=48, n_q=32, n_kv=4, head_dim=128, inter=768, vocab=151936, max_seq=6600 + 64, eps=1e-6, theta=1e6)


def random_moe(seed, hidden, n_experts, top_k, d_ff, bits, sgc, norm_topk=True):
    """One sparse-MoE FFN with random expert codes in the reference's .k2tm record form (nf_expert_byte_layout,
    src/model/moe_800b.rs): codebooks at bytes 0 / 16, the gate_up pair stream at 64, the down pair stream at the next
    multiple of 64, records padded to 16 KiB; router weights N(0, 0.02) (near-uniform routing)."""
    cb = _NF_CHUNK[bits]
    gu_chunks, dn_chunks = hidden // 64, d_ff // 64
    gu_bytes = (2 * d_ff // 32) * (-(-gu_chunks // sgc) * 64 + gu_chunks * 2 * cb)
    dn_bytes = (hidden // 32) * (-(-dn_chunks // sgc) * 64 + dn_chunks * 2 * cb)
    gu_off, dn_off = 64, (64 + gu_bytes + 63) // 64 * 64
    rec = (dn_off + dn_bytes + 16383) // 16384 * 16384
    shard = np.zeros(n_experts * rec, np.uint8)
    book = (NF4_DEFAULT if bits == 4 else NF3_DEFAULT).view(np.uint8)
    for e in range(n_experts):
        r = shard[e * rec:(e + 1) * rec]
        r[0:16] = book
        r[16:32] = book
        r[gu_off:gu_off + gu_bytes] = random_nf_bytes(seed * 1009 + 2 * e, 2 * d_ff, hidden, bits, sgc)[0]
        r[dn_off:dn_off + dn_bytes] = random_nf_bytes(seed * 1009 + 2 * e + 1, hidden, d_ff, bits, sgc)[0]
    router = (_rng(seed * 1009 + 7).standard_normal((n_experts, hidden)) * 0.02).astype(np.float32)
    return dict(router_w=router, router_bias=None, n_experts=n_experts, top_k=top_k, norm_topk=norm_topk, d_ff=d_ff, bits=bits, sgc=sgc,
                shard=shard, expert_bytes=rec, scoring=0)


def random_model(cfg, mode, seed=0, modes=None, qkv_bias=False, untied=False, tp=(1, 0), share_layers=False, moe=None, ep=(1, 0)):
    """Engine spec of a dense Llama-shaped model with random codes (decode time does not depend on the values).

    modes: per-matrix formats {qkv, o, gate_up, down, head} overriding `mode`.  tp = (size, rank): the rank-local
    spec of a tensor-parallel group, generated directly in the rank's shapes (what kronos_2t_b200.tp.shard_spec cuts
    out of a whole model); tensor-parallel specs use an untied embedding table.  share_layers: every layer points at
    layer 0's host arrays (each still becomes its own device copy), which keeps multi-billion-parameter specs quick to make.
    moe: dict(n_experts, top_k, d_ff, bits, sgc) - every layer gets a sparse-MoE FFN (random_moe) instead of the dense MLP;
    ep = (size, rank): expert-parallel rank (the whole spec; the engine keeps the experts e % size == rank)."""
    c = dict(cfg)
    tp_size, tp_rank = tp
    md = dict(qkv=mode, o=mode, gate_up=mode, down=mode, head=mode)
    md.update(modes or {})
    h, hd = c["hidden"], c["head_dim"]
    vocab_total = c["vocab"]
    if tp_size > 1:
        from .tp import head_plan
        assert c["inter"] % (64 * tp_size) == 0 and c["vocab"] % (32 * tp_size) == 0
        qh0, nq_l, _, nkv_l = head_plan(c["n_q"], c["n_kv"], tp_size, tp_rank)      # more ranks than kv heads: the kv head is replicated
        c.update(n_q=nq_l, n_kv=nkv_l, inter=c["inter"] // tp_size, vocab=c["vocab"] // tp_size)
        c.update(tp_size=tp_size, tp_rank=tp_rank, vocab_total=vocab_total, o_chunk0=qh0 * hd // 64,
                 down_chunk0=tp_rank * c["inter"] // 64)
        untied = True
    if ep[0] > 1:
        c.update(ep_size=ep[0], ep_rank=ep[1])
    inter = c["inter"]
    q_dim, kv_dim = c["n_q"] * hd, c["n_kv"] * hd
    layers = []
    for l in range(c["layers"]):
        if share_layers and l > 0:
            layers.append(dict(layers[0]))
            continue
        s = seed * 100003 + 10 * l + 1000003 * tp_rank
        bias = None
        if qkv_bias:
            bias = (_rng(s + 5).standard_normal(q_dim + 2 * kv_dim) * 0.02).astype(np.float32)
        ly = dict(input_norm=np.ones(h, np.float32), post_norm=np.ones(h, np.float32), qkv_bias=bias, q_norm=None, k_norm=None,
                  qkv=random_matrix(s + 1, q_dim + 2 * kv_dim, h, md["qkv"]), o=random_matrix(s + 2, h, q_dim, md["o"]))
        if moe:
            ly["moe"] = random_moe(s + 6, h, moe["n_experts"], moe["top_k"], moe["d_ff"], moe["bits"], moe["sgc"])
        else:
            ly.update(gate_up=random_matrix(s + 3, 2 * inter, h, md["gate_up"]), down=random_matrix(s + 4, h, inter, md["down"]))
        layers.append(ly)
    embed = None
    if untied:       # a 4096-row random block, repeated
        blk = random_bf16(seed * 100003 + 8, min(vocab_total, 4096) * h)
        embed = np.tile(blk, -(-vocab_total // 4096))[:vocab_total * h]
    return dict(cfg=c, layers=layers, final_norm=np.ones(h, np.float32),
                lm_head=random_matrix(seed * 100003 + 7 + 1000003 * tp_rank, c["vocab"], h, md["head"]),
                rope=rope_table(c["max_seq"], hd, c["theta"]), embed_bf16=embed)
