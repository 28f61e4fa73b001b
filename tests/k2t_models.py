"""Synthetic dense Llama/Qwen-shaped models for parity tests and benchmarks: random N(0, 0.02) weights
quantized with the oracle's RTN quantizers, norms near 1, optional qkv bias / qk-norm, tied or bf16
embeddings.  The returned `spec` dict feeds both the CPU oracle model and the CUDA engine."""
import numpy as np

from k2t_rng import normal

TINY = dict(hidden=128, layers=2, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=320, max_seq=96, eps=1e-5, theta=1e5)
SMOL_135M = dict(hidden=576, layers=30, n_q=9, n_kv=3, head_dim=64, inter=1536, vocab=49152, max_seq=512, eps=1e-5, theta=1e5)


def quantize(oracle, w, mode):
    if mode.startswith("b"):
        return oracle.bipolar_quantize_rtn(w, int(mode[1]))
    if mode.startswith("e8q2"):
        # no lattice quantizer here: random E8 codewords with scales that keep the outputs at the size of w @ x
        rows, cols = w.shape
        sgc = 2 if mode.endswith("g128") and (cols // 64) % 2 == 0 else 1
        rng = np.random.Generator(np.random.PCG64(int(abs(float(w[0, 0])) * 1e9) % (1 << 31)))
        tpl = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
        sgn = rng.integers(0, 256, (rows, cols // 8), dtype=np.uint8)
        sc = rng.integers(0x3A00, 0x3A80, oracle.lib().k2o_nf_scale_count(rows, cols, sgc)).astype(np.uint16)    # ~5e-4
        return oracle.e8q2_pack(tpl, sgn, sc, sgc)
    bits = int(mode[2])
    return oracle.nf_quantize_rtn(w, bits, 2 if mode.endswith("g128") else 1)


MOE_TINY = dict(hidden=128, layers=3, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=320, max_seq=96, eps=1e-6, theta=1e6)


def build_moe(oracle, seed, hidden, n_experts, top_k, d_ff, bits, sgc, norm_topk=True, bias=False, scoring=0, shared=0, shared_gate=True):
    """One sparse-MoE FFN: router N(0, 0.02) (near-uniform routing) and NF experts in .k2tm record form."""
    experts = []
    mode = ("e8q2" if bits == 2 else f"nf{bits}") + ("g128" if sgc == 2 else "")     # bits = 2: E8 lattice codewords
    for e in range(n_experts):
        gu = quantize(oracle, normal(seed + 2 * e, (2 * d_ff, hidden), 0.02), mode)
        dn = quantize(oracle, normal(seed + 2 * e + 1, (hidden, d_ff), 0.02), mode)
        assert gu.sgc == sgc and dn.sgc == sgc
        experts.append((gu, dn))
    shard, lay = oracle.pack_expert_shard(experts, hidden, d_ff, bits, sgc)
    sh = None
    if shared:              # shared expert of `shared` intermediate columns (SharedMoeExpert, NF matrices), optional sigmoid gate
        sh = dict(gate_up=quantize(oracle, normal(seed + 5000, (2 * shared, hidden), 0.02), "nf4g128"),
                  down=quantize(oracle, normal(seed + 5001, (hidden, shared), 0.02), "nf4g128"),
                  gate_w=normal(seed + 5002, hidden, 0.3) if shared_gate else None)
    return dict(shared=sh, router_w=normal(seed + 999, (n_experts, hidden), 0.02), router_bias=normal(seed + 998, n_experts, 0.01) if bias else None,
                n_experts=n_experts, top_k=top_k, norm_topk=norm_topk, d_ff=d_ff, bits=bits, sgc=sgc, shard=shard,
                expert_bytes=lay["expert_bytes"], scoring=scoring)


def build(oracle, cfg, mode="b4", seed=0, qkv_bias=False, qk_norm=False, tied=True, head_mode=None, modes=None, moe=None, embed_nf4=False):
    """modes: optional dict {qkv, o, gate_up, down, head} overriding `mode` per matrix (e.g. p55454).
    moe: optional dict(layers=[...], n_experts, top_k, d_ff, bits, sgc[, norm_topk, bias]): those layers get a sparse-MoE FFN."""
    c = dict(cfg)
    h, hd, inter = c["hidden"], c["head_dim"], c["inter"]
    q_dim, kv_dim = c["n_q"] * hd, c["n_kv"] * hd
    modes = modes or {}
    pick = lambda k: modes.get(k, mode)
    s = seed * 1000
    layers = []
    for l in range(c["layers"]):
        ly = dict(
            input_norm=(1.0 + 0.1 * normal(s + 10 * l + 1, h)).astype(np.float32),
            post_norm=(1.0 + 0.1 * normal(s + 10 * l + 2, h)).astype(np.float32),
            qkv_bias=normal(s + 10 * l + 3, q_dim + 2 * kv_dim, 0.02) if qkv_bias else None,
            q_norm=(1.0 + 0.1 * normal(s + 10 * l + 4, hd)).astype(np.float32) if qk_norm else None,
            k_norm=(1.0 + 0.1 * normal(s + 10 * l + 5, hd)).astype(np.float32) if qk_norm else None,
            qkv=quantize(oracle, normal(s + 10 * l + 6, (q_dim + 2 * kv_dim, h), 0.02), pick("qkv")),
            o=quantize(oracle, normal(s + 10 * l + 7, (h, q_dim), 0.02), pick("o")),
            gate_up=quantize(oracle, normal(s + 10 * l + 8, (2 * inter, h), 0.02), pick("gate_up")),
            down=quantize(oracle, normal(s + 10 * l + 9, (h, inter), 0.02), pick("down")),
        )
        if moe and l in moe["layers"]:
            ly["gate_up"] = ly["down"] = None
            ly["moe"] = build_moe(oracle, s + 100 * l + 50, h, moe["n_experts"], moe["top_k"], moe["d_ff"], moe["bits"], moe["sgc"],
                                  moe.get("norm_topk", True), moe.get("bias", False), moe.get("scoring", 0), moe.get("shared", 0),
                                  moe.get("shared_gate", True))
        layers.append(ly)
    head_w = normal(s + 999, (c["vocab"], h), 0.02)
    spec = dict(cfg=c, layers=layers, final_norm=(1.0 + 0.1 * normal(s + 998, h)).astype(np.float32),
                lm_head=quantize(oracle, head_w, head_mode or pick("head")),
                rope=oracle.build_rope_table(c["max_seq"], hd, c["theta"]), embed_bf16=None)
    if not tied:
        e = normal(s + 997, (c["vocab"], h), 0.02)
        spec["embed_bf16"] = (e.view(np.uint32) >> 16).astype(np.uint16)     # truncation is fine for synthetic tables
        if embed_nf4:       # compress_untied_embeddings_nf4 (real_llm.rs:1825-1844): the bf16 rows become an NF4 matrix
            spec["embed_matrix"] = oracle.nf4_embed_from_bf16(spec["embed_bf16"], 2)
            spec["embed_bf16"] = None
    return spec
