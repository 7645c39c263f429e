"""CPU tests of the multi-rank (tensor-parallel) path: two gloo ranks each hold their share of the
weights (lighterpp_b200.tp), run the step with one all-reduce after o_proj and one after down_proj,
and must reproduce the single-rank oracle logits; both ranks must end with identical vectors so
the replicated sampler picks the same token without a broadcast."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rmsnorm(x, w):
    ss = np.float32(1.0) / np.sqrt(np.float32(np.mean(x * x, dtype=np.float32)) + np.float32(1e-5))
    return (x * ss * w).astype(np.float32)


def _tp_step(c, W, kc, vc, token, pos, rank, size, allreduce):
    """One decode step on this rank's shard; mirrors src/model.cpp:121-241 with the partition of tp.py."""
    hs = c.head_size
    Hl, KVHl = c.n_heads // size, c.n_kv_heads // size
    gqa = c.n_heads // c.n_kv_heads
    x = W["tok_emb"][token].astype(np.float32).copy()
    for l in range(c.n_layers):
        xb = _rmsnorm(x, W["rms_att"][l])
        q = W["wq"][l] @ xb
        k = W["wk"][l] @ xb
        v = W["wv"][l] @ xb
        for vec in (q, k):
            for i in range(0, vec.size, 2):
                freq = np.float32(1.0) / np.float32(np.power(np.float32(c.rope_base), np.float32((i % hs) / hs)))
                val = np.float32(pos) * freq
                co, si = np.float32(np.cos(val)), np.float32(np.sin(val))
                a, b = vec[i], vec[i + 1]
                vec[i], vec[i + 1] = a * co - b * si, a * si + b * co
        kc[l, :, pos] = k.reshape(KVHl, hs)
        vc[l, :, pos] = v.reshape(KVHl, hs)
        out = np.zeros(Hl * hs, dtype=np.float32)
        for h in range(Hl):
            kv = h // gqa
            s = (kc[l, kv, :pos + 1] @ q[h * hs:(h + 1) * hs]) / np.float32(np.sqrt(hs))
            p = np.exp(s - s.max())
            p /= p.sum()
            out[h * hs:(h + 1) * hs] = p @ vc[l, kv, :pos + 1]
        part = (W["wo"][l] @ out).astype(np.float32)
        if rank == 0:
            part += x  # the residual enters the sum exactly once
        x = allreduce(part)
        xb = _rmsnorm(x, W["rms_ffn"][l])
        g, u = W["w1"][l] @ xb, W["w3"][l] @ xb
        hb = (g / (1.0 + np.exp(-g))) * u
        part = (W["w2"][l] @ hb).astype(np.float32)
        if rank == 0:
            part += x
        x = allreduce(part)
    xf = _rmsnorm(x, W["rms_final"])
    return W.get("w_cls", W["tok_emb"]).astype(np.float32) @ xf


def _worker(rank, size, port, name, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from lighterpp_b200 import synth, tp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    c, dt, tied, seed, T = synth.named(name)
    W = {k: v.astype(np.float32) for k, v in tp.shard_model(c, T, rank, size).items()}
    KVHl = c.n_kv_heads // size
    kc = np.zeros((c.n_layers, KVHl, c.seq_len, c.head_size), np.float32)
    vc = np.zeros_like(kc)

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        dist.all_reduce(t)
        return t.numpy()

    toks = synth.prompt_tokens(c.vocab_size, 4, seed)
    logits = [_tp_step(c, W, kc, vc, int(t), p, rank, size, allreduce) for p, t in enumerate(toks)]
    q.put((rank, np.stack(logits)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name,size", [("tiny-gqa-f16", 2), ("tiny-tp8-f16", 2)])
def test_two_rank_step_matches_oracle(oracle, name, size):
    import torch.multiprocessing as mp
    from lighterpp_b200 import synth
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, size, port, name, q)) for r in range(size)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(size))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c, dt, tied, seed, T = synth.named(name)
    m = oracle.model(c, synth.as_f32(T))
    toks = synth.prompt_tokens(c.vocab_size, 4, seed)
    ref = np.stack([m.step_logits(int(t), p) for p, t in enumerate(toks)])
    for r in range(size):
        assert np.abs(got[r] - ref).max() < 2e-4, np.abs(got[r] - ref).max()
    assert np.array_equal(got[0], got[1])  # replicated tail sees bit-identical inputs on every rank


def test_partition_rules():
    from lighterpp_b200 import synth, tp
    c, dt, tied, seed, T = synth.named("tiny-tp8-f16")
    for size in (1, 2, 4, 8):
        parts = [tp.shard_model(c, T, r, size) for r in range(size)]
        for name in tp.ROW_SLICED:
            assert np.array_equal(np.concatenate([p[name] for p in parts], axis=1), T[name])
        for name in tp.COL_SLICED:
            assert np.array_equal(np.concatenate([p[name] for p in parts], axis=2), T[name])
        assert tp.local_config(c, size)["n_kv_heads"] * size == c.n_kv_heads
    with pytest.raises(ValueError):
        tp.validate(c, 3)
    with pytest.raises(ValueError):
        tp.shard_layer_tensor(c, "wq", T["wq"][0], 2, 2)
