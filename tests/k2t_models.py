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


def build(oracle, cfg, mode="b4", seed=0, qkv_bias=False, qk_norm=False, tied=True, head_mode=None, modes=None):
    """modes: optional dict {qkv, o, gate_up, down, head} overriding `mode` per matrix (e.g. p55454)."""
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
        layers.append(ly)
    head_w = normal(s + 999, (c["vocab"], h), 0.02)
    spec = dict(cfg=c, layers=layers, final_norm=(1.0 + 0.1 * normal(s + 998, h)).astype(np.float32),
                lm_head=quantize(oracle, head_w, head_mode or pick("head")),
                rope=oracle.build_rope_table(c["max_seq"], hd, c["theta"]), embed_bf16=None)
    if not tied:
        e = normal(s + 997, (c["vocab"], h), 0.02)
        spec["embed_bf16"] = (e.view(np.uint32) >> 16).astype(np.uint16)     # truncation is fine for synthetic tables
    return spec
