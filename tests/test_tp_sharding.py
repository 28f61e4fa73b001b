"""Tensor-parallel host logic on the CPU: file-format slicing, the rank-order partial-sum semantics (oracle.TpModel), and the
same exchange over a real process group (gloo, world size 2)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import k2t_models as km

TP_CFG = dict(hidden=256, layers=2, n_q=4, n_kv=2, head_dim=64, inter=512, vocab=384, max_seq=64, eps=1e-5, theta=1e5)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dequant_rows(oracle, m):
    return np.stack([oracle.bipolar_dequant_row(m, r) if m.kind == 0 else oracle.nf_dequant_row(m, r) for r in range(m.rows)])


@pytest.mark.parametrize("mode", ["b4", "b6", "nf4g128", "nf3", "nf5g128"])
def test_file_format_slices_select_rows_and_chunks(oracle, mode):
    from kronos_2t_b200 import tp
    from k2t_rng import normal
    m = km.quantize(oracle, normal(5, (192, 512), 0.02), mode)
    full = dequant_rows(oracle, m)                       # rotated domain: a 64-column chunk is self-contained
    assert np.array_equal(dequant_rows(oracle, tp.rows_slice(m, 64, 160)), full[64:160])
    assert np.array_equal(dequant_rows(oracle, tp.cols_slice(m, 2, 6)), full[:, 128:384])
    cat = tp.rows_concat([tp.rows_slice(m, 128, 192), tp.rows_slice(m, 0, 32)])
    assert np.array_equal(dequant_rows(oracle, cat), np.concatenate([full[128:192], full[0:32]]))
    with pytest.raises(ValueError):
        tp.rows_slice(m, 8, 64)
    if mode.endswith("g128"):
        with pytest.raises(ValueError):
            tp.cols_slice(m, 1, 4)                       # not on a scale-group boundary


@pytest.mark.parametrize("mode,kw", [("b5", dict(qkv_bias=True)), ("nf4g128", dict(qk_norm=True, tied=False))])
def test_tp_emulation_matches_the_whole_model(oracle, mode, kw):
    from kronos_2t_b200 import tp
    spec = km.build(oracle, TP_CFG, mode, seed=3, **kw)
    whole = oracle.Model(spec)
    tokens = [5, 17, 300, 42, 7, 199, 63, 250]
    want = np.stack([whole.forward_token(t, 2) for t in tokens])
    embed = lambda t: whole.embed(t)
    one = oracle.TpModel([tp.shard_spec(spec, 1, 0)], embed)
    assert np.array_equal(np.stack([one.forward_token(t) for t in tokens]), want)        # one rank: the same arithmetic, bit for bit
    two = oracle.TpModel([tp.shard_spec(spec, 2, r) for r in range(2)], embed)
    got = np.stack([two.forward_token(t) for t in tokens])
    # two ranks: every row-parallel output is (partial over rank 0's chunks) + (partial over rank 1's chunks) instead of one
    # chain over all chunks: rounding-level differences that the int8 re-quantization of later layers can amplify slightly
    assert np.max(np.abs(got - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))
    cos = [np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)) for a, b in zip(got, want)]
    assert min(cos) > 0.99999
    for m in (one, two):
        m.close()
    whole.close()
    # shapes of a rank
    s0 = tp.shard_spec(spec, 2, 1)
    c = s0["cfg"]
    assert (c["n_q"], c["n_kv"], c["inter"], c["vocab"], c["o_chunk0"], c["down_chunk0"]) == (2, 1, 256, 192, 2, 4)
    assert s0["layers"][0]["qkv"].rows == (2 + 2 * 1) * 64 and s0["layers"][0]["o"].cols == 128 and s0["layers"][0]["down"].cols == 256
    with pytest.raises(ValueError):
        tp.shard_spec(spec, 3, 0)                        # 2 kv heads do not split three ways


def test_more_ranks_than_kv_heads_replicate_the_kv_head(oracle):
    """Eight-way tensor parallelism of a 28 / 4-head model (Qwen2-7B): two ranks share each kv head, keep their own copy of
    its key / value rows and split its seven query heads 4 + 3; the o_proj chunks of the ranks tile the matrix in order.
    On a small model the four-rank emulation (2 kv heads, 2 ranks each) tracks the whole model like the two-rank one."""
    from kronos_2t_b200 import tp
    plan = [tp.head_plan(28, 4, 8, r) for r in range(8)]
    assert [p[1] for p in plan] == [4, 3, 4, 3, 4, 3, 4, 3] and [p[2] for p in plan] == [0, 0, 1, 1, 2, 2, 3, 3] and all(p[3] == 1 for p in plan)
    assert [p[0] for p in plan] == [0, 4, 7, 11, 14, 18, 21, 25]                      # contiguous query heads, in rank order
    assert tp.head_plan(28, 4, 4, 2) == (14, 7, 2, 1) and tp.head_plan(28, 4, 2, 1) == (14, 14, 2, 2)
    cfg = dict(TP_CFG, n_q=6, n_kv=2, hidden=384)                                     # groups of three query heads: 2 + 1 per rank pair
    spec = km.build(oracle, cfg, "b5", seed=3, qkv_bias=True, tied=False)
    whole = oracle.Model(spec)
    tokens = [5, 17, 300, 42, 7, 199, 63, 250]
    want = np.stack([whole.forward_token(t, 2) for t in tokens])
    shards = [tp.shard_spec(spec, 4, r) for r in range(4)]
    assert [s["cfg"]["n_q"] for s in shards] == [2, 1, 2, 1] and all(s["cfg"]["n_kv"] == 1 for s in shards)
    assert [s["cfg"]["o_chunk0"] for s in shards] == [0, 2, 3, 5]
    assert sum(s["layers"][0]["o"].cols for s in shards) == 6 * 64
    four = oracle.TpModel(shards, lambda t: whole.embed(t))
    got = np.stack([four.forward_token(t) for t in tokens])
    assert np.max(np.abs(got - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))
    cos = [np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)) for a, b in zip(got, want)]
    assert min(cos) > 0.99999
    four.close(); whole.close()


WORKER = r'''
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle")); sys.path.insert(0, ROOT)
import numpy as np, torch, torch.distributed as dist
import oracle as o, k2t_models as km
from kronos_2t_b200 import tp
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % os.environ["PORT"], rank=int(os.environ["RANK"]), world_size=2)
rank = dist.get_rank()
cfg = dict(hidden=256, layers=2, n_q=4, n_kv=2, head_dim=64, inter=512, vocab=384, max_seq=64, eps=1e-5, theta=1e5)
spec = km.build(o, cfg, "b5", seed=3, qkv_bias=True)
whole = o.Model(spec)                                    # only for the embedding lookup
local = o.Model(tp.shard_spec(spec, 2, rank))

def all_sum(part):                                       # every rank's partial, summed in rank order on every rank
    parts = [torch.zeros(part.size) for _ in range(2)]
    dist.all_gather(parts, torch.from_numpy(part.copy()))
    acc = parts[0].numpy().copy()
    for p in parts[1:]:
        acc = (acc + p.numpy()).astype(np.float32)
    return acc

out = []
for t in [5, 17, 300, 42, 7]:
    hidden = whole.embed(t)
    for l in range(cfg["layers"]):
        hidden = (hidden + all_sum(local.attn_part(l, hidden))).astype(np.float32)
        hidden = (hidden + all_sum(local.ffn_part(l, hidden))).astype(np.float32)
    sl = torch.from_numpy(local.head_part(hidden))
    parts = [torch.zeros(sl.numel()) for _ in range(2)]
    dist.all_gather(parts, sl)
    out.append(torch.cat(parts).numpy())
    local.advance()
np.save(os.environ["OUT"] + ".%d.npy" % rank, np.stack(out))
dist.destroy_process_group()
'''


def test_two_gloo_ranks_reproduce_the_emulation(oracle, tmp_path):
    from kronos_2t_b200 import tp
    port = str(29000 + os.getpid() % 2000)
    env = dict(os.environ, PORT=port, OUT=str(tmp_path / "logits"))
    procs = [subprocess.Popen([sys.executable, "-c", "ROOT = %r\n" % ROOT + WORKER], env=dict(env, RANK=str(r))) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=240) == 0
    a, b = np.load(str(tmp_path / "logits.0.npy")), np.load(str(tmp_path / "logits.1.npy"))
    assert np.array_equal(a, b)                          # both ranks hold the same logits
    spec = km.build(oracle, TP_CFG, "b5", seed=3, qkv_bias=True)
    whole = oracle.Model(spec)
    emu = oracle.TpModel([tp.shard_spec(spec, 2, r) for r in range(2)], lambda t: whole.embed(t))
    want = np.stack([emu.forward_token(t) for t in [5, 17, 300, 42, 7]])
    assert np.array_equal(a, want)
    emu.close(); whole.close()


@pytest.mark.parametrize("moe,ep", [(dict(layers=[0, 2], n_experts=8, top_k=3, d_ff=64, bits=3, sgc=2), 2),
                                    (dict(layers=[1], n_experts=6, top_k=6, d_ff=64, bits=4, sgc=1, norm_topk=False), 3)])
def test_expert_parallel_emulation_matches_the_whole_model(oracle, moe, ep):
    """Experts e % ep == r on rank r: one rank reproduces the model bit for bit; more ranks differ only by the order of
    the weighted sum (partial sums per rank, added in rank order); routes are the single-device routes on every rank."""
    spec = km.build(oracle, km.MOE_TINY, "b4", seed=21, moe=moe)
    whole = oracle.Model(spec)
    tokens = [5, 17, 300, 42, 7, 199, 63, 250, 11]
    want = np.stack([whole.forward_token(t, 2) for t in tokens])
    one = oracle.EpModel(spec, 1)
    assert np.array_equal(np.stack([one.forward_token(t) for t in tokens]), want)
    many = oracle.EpModel(spec, ep)
    got = np.stack([many.forward_token(t) for t in tokens])
    assert np.max(np.abs(got - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))
    cos = [np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)) for a, b in zip(got, want)]
    assert min(cos) > 0.99999
    for m in (one, many):
        m.close()
    whole.close()


def test_synthetic_moe_records_follow_the_reference_layout(oracle):
    """kronos_2t_b200.synth.random_moe writes .k2tm expert records the oracle parses: record size and offsets equal
    nf_expert_byte_layout, and a model built from them runs (finite logits, top-k routes in ascending expert order)."""
    from kronos_2t_b200 import synth
    for hidden, d_ff, bits, sgc in [(2048, 768, 3, 1), (256, 128, 4, 2), (256, 128, 3, 2)]:
        lay = oracle.nf_expert_layout(hidden, d_ff, bits, sgc)
        m = synth.random_moe(3, hidden, 2, 1, d_ff, bits, sgc)
        assert m["expert_bytes"] == lay["expert_bytes"] and m["shard"].size == 2 * lay["expert_bytes"]
    cfg = dict(hidden=128, layers=2, n_q=4, n_kv=2, head_dim=64, inter=64, vocab=320, max_seq=32, eps=1e-6, theta=1e6)
    spec = synth.random_model(cfg, "nf4g128", seed=2, moe=dict(n_experts=8, top_k=3, d_ff=64, bits=3, sgc=1), ep=(2, 1))
    assert spec["cfg"]["ep_size"] == 2 and spec["cfg"]["ep_rank"] == 1
    ref = oracle.Model(spec)
    logits = ref.forward_token(5)
    ids, w = ref.last_routes(0)
    assert np.isfinite(logits).all() and len(ids) == 3 and list(ids) == sorted(ids) and abs(float(w.sum()) - 1.0) < 1e-5
    ref.close()

