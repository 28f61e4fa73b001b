"""Tensor-parallel engine on two GPUs of one node (skipped where fewer are visible): one child process per rank, the ranks'
exchange-buffer handles swapped over a gloo process group, results compared with the CPU emulation that sums the ranks'
partial outputs in the same (rank) order - so logits and greedy tokens must be identical, bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

import k2t_models as km

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TP_CFG = dict(hidden=256, layers=2, n_q=4, n_kv=2, head_dim=64, inter=512, vocab=384, max_seq=64, eps=1e-5, theta=1e5)
TOKENS = [5, 17, 300, 42, 7, 199, 63, 250, 11]

WORKER = r"""
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle")); sys.path.insert(0, ROOT)
import numpy as np, torch.distributed as dist
import oracle as o, k2t_models as km, kronos_2t_b200 as k2
from kronos_2t_b200 import tp
rank, world = int(os.environ["RANK"]), 2
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % os.environ["PORT"], rank=rank, world_size=world)
cfg = eval(os.environ["CFG"]); mode = os.environ["MODE"]; kw = eval(os.environ["KW"]); tokens = eval(os.environ["TOKENS"])
spec = km.build(o, cfg, mode, seed=3, **kw)
ctx = k2.Context(rank)
eng = k2.Engine(ctx, tp.shard_spec(spec, world, rank))
handles = [None] * world
dist.all_gather_object(handles, eng.tp_handle())
eng.tp_attach(handles)
dist.barrier()
logits = eng.forward_token_ids(tokens, want_all=True)
greedy = eng.decode_greedy(int(np.argmax(logits[-1])), len(tokens), 12)
np.save(os.environ["OUT"] + ".%d.npy" % rank, logits)
np.save(os.environ["OUT"] + ".g%d.npy" % rank, greedy)
dist.barrier()
eng.close(); ctx.close()
dist.destroy_process_group()
"""


def _wait_all(procs, timeout=600):
    """Every child must exit 0; whatever happens, none is left running (a rank whose peer died would otherwise sit in its
    bounded waits for the rest of the session)."""
    try:
        for p in procs:
            assert p.wait(timeout=timeout) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()


def gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode,kw", [("b5", dict(qkv_bias=True)), ("nf4g128", dict(qk_norm=True, tied=False))])
def test_two_rank_engine_matches_rank_order_emulation(oracle, tmp_path, mode, kw):
    from kronos_2t_b200 import tp
    port = str(31000 + os.getpid() % 2000)
    env = dict(os.environ, PORT=port, OUT=str(tmp_path / "tp"), CFG=repr(TP_CFG), MODE=mode, KW=repr(kw), TOKENS=repr(TOKENS))
    procs = [subprocess.Popen([sys.executable, "-c", "ROOT = %r\n" % ROOT + WORKER], env=dict(env, RANK=str(r))) for r in range(2)]
    _wait_all(procs)
    got = [np.load(str(tmp_path / f"tp.{r}.npy")) for r in range(2)]
    greedy = [np.load(str(tmp_path / f"tp.g{r}.npy")) for r in range(2)]
    assert np.array_equal(got[0], got[1]) and np.array_equal(greedy[0], greedy[1])       # every rank ends with the same logits and tokens
    spec = km.build(oracle, TP_CFG, mode, seed=3, **kw)
    whole = oracle.Model(spec)
    emu = oracle.TpModel([tp.shard_spec(spec, 2, r) for r in range(2)], lambda t: whole.embed(t))
    want = np.stack([emu.forward_token(t) for t in TOKENS])
    assert np.array_equal(got[0], want)
    nxt, out = int(np.argmax(want[-1])), []
    for _ in range(12):
        logits = emu.forward_token(nxt); nxt = oracle.argmax(logits); out.append(nxt)
    assert list(greedy[0]) == out
    emu.close(); whole.close()


EP_WORKER = r"""
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle")); sys.path.insert(0, ROOT)
import numpy as np, torch.distributed as dist
import oracle as o, k2t_models as km, kronos_2t_b200 as k2
rank, world = int(os.environ["RANK"]), 2
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % os.environ["PORT"], rank=rank, world_size=world)
moe = eval(os.environ["MOE"]); mode = os.environ["MODE"]; tokens = eval(os.environ["TOKENS"])
spec = km.build(o, km.MOE_TINY, mode, seed=21, moe=moe)
spec["cfg"] = dict(spec["cfg"], ep_size=world, ep_rank=rank)
ctx = k2.Context(rank)
eng = k2.Engine(ctx, spec)
handles = [None] * world
dist.all_gather_object(handles, eng.tp_handle())
eng.tp_attach(handles)
dist.barrier()
logits = eng.forward_token_ids(tokens, want_all=True)
greedy = eng.decode_greedy(int(np.argmax(logits[-1])), len(tokens), 12)
np.save(os.environ["OUT"] + ".%d.npy" % rank, logits)
np.save(os.environ["OUT"] + ".g%d.npy" % rank, greedy)
dist.barrier()
eng.close(); ctx.close()
dist.destroy_process_group()
"""


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode,moe", [("nf4g128", dict(layers=[0, 2], n_experts=8, top_k=3, d_ff=64, bits=3, sgc=2)),
                                      ("b5", dict(layers=[1, 2], n_experts=6, top_k=6, d_ff=64, bits=4, sgc=1, norm_topk=False, bias=True)),
                                      ("nf4g128", dict(layers=[0, 1], n_experts=8, top_k=2, d_ff=64, bits=3, sgc=2, shared=64))])    # rank 0's partial sum carries the shared expert
def test_two_rank_expert_parallel_engine_matches_rank_order_emulation(oracle, tmp_path, mode, moe):
    tokens = [t % km.MOE_TINY["vocab"] for t in TOKENS]
    port = str(33000 + os.getpid() % 2000)
    env = dict(os.environ, PORT=port, OUT=str(tmp_path / "ep"), MODE=mode, MOE=repr(moe), TOKENS=repr(tokens))
    procs = [subprocess.Popen([sys.executable, "-c", "ROOT = %r\n" % ROOT + EP_WORKER], env=dict(env, RANK=str(r))) for r in range(2)]
    _wait_all(procs)
    got = [np.load(str(tmp_path / f"ep.{r}.npy")) for r in range(2)]
    greedy = [np.load(str(tmp_path / f"ep.g{r}.npy")) for r in range(2)]
    assert np.array_equal(got[0], got[1]) and np.array_equal(greedy[0], greedy[1])
    spec = km.build(oracle, km.MOE_TINY, mode, seed=21, moe=moe)
    emu = oracle.EpModel(spec, 2)
    want = np.stack([emu.forward_token(t) for t in tokens])
    assert np.array_equal(got[0], want)
    nxt, out = int(np.argmax(want[-1])), []
    for _ in range(12):
        logits = emu.forward_token(nxt); nxt = oracle.argmax(logits); out.append(nxt)
    assert list(greedy[0]) == out
    emu.close()



def test_absent_peer_is_reported_not_waited_for(oracle, monkeypatch):
    """One GPU is enough: rank 0 of a two-rank group is attached to a rank-1 engine that never runs, so the words rank 0
    polls for are never written.  Its bounded waits run out (a short limit here), the call returns the peer error within
    seconds and the context remembers it: later calls fail at once instead of waiting again."""
    import time
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import tp
    monkeypatch.setenv("KRONOS_CUDA_PEER_WAIT_POLLS", "20000")
    spec = km.build(oracle, TP_CFG, "b5", seed=3, tied=False)
    ctxs = [k2.Context(0), k2.Context(0)]
    engs = [k2.Engine(ctxs[r], tp.shard_spec(spec, 2, r)) for r in range(2)]
    try:
        for e in engs:
            e.tp_attach_local(engs)
        t0 = time.perf_counter()
        with pytest.raises(k2.KronosCudaError, match="peer rank"):
            engs[0].forward_token_ids(TOKENS[:3])
        first = time.perf_counter() - t0
        t0 = time.perf_counter()
        with pytest.raises(k2.KronosCudaError, match="peer rank"):
            engs[0].forward_token_ids(TOKENS[:1])
        again = time.perf_counter() - t0
        assert first < 20.0 and again < 5.0, (first, again)
    finally:
        for e in engs:
            e.close()
        for c in ctxs:
            c.close()
