"""Multi-rank host logic on CPU (gloo, world size 2): the (batch, KV-head) units are partitioned with no overlap and
no gap, every rank can compute its shard independently (checked with the CPU oracle standing in for the kernel),
and the optional output gather reassembles the full tensor.  No GPU is touched."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import oracle
    import radiance_kernels_b200 as rk
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, H, Hkv, S, d = 2, 4, 2, 128, 64
    grp = H // Hkv
    rng = np.random.default_rng(7)                      # every rank generates the same global problem
    Q = rng.standard_normal((B, H, S, d), dtype=np.float32)
    K = rng.standard_normal((B, Hkv, S, d), dtype=np.float32)
    V = rng.standard_normal((B, Hkv, S, d), dtype=np.float32)

    def q4(x):
        c, s = oracle.quantize(x.reshape(-1, d))
        return c.reshape(x.shape), s.reshape(x.shape[:-1] + (d // 32,))

    qc, qs = q4(Q); kc, ks = q4(K); vc, vs = q4(V)
    lo, hi = rk.shard_range(B * Hkv, rank, world)       # units = flattened (batch, KV head)
    mine = torch.zeros(B * Hkv, grp, S, d)
    for u in range(lo, hi):
        b, kv = divmod(u, Hkv)
        r = oracle.attn_prefill(qc[b:b + 1, kv * grp:(kv + 1) * grp], kc[b:b + 1, kv:kv + 1], vc[b:b + 1, kv:kv + 1],
                                qs[b:b + 1, kv * grp:(kv + 1) * grp], ks[b:b + 1, kv:kv + 1], vs[b:b + 1, kv:kv + 1],
                                causal=True, softmax_scale=d ** -0.5, block_n=128, nthreads=1)
        mine[u] = torch.from_numpy(r["o_f32"][0])
    counts = torch.zeros(B * Hkv)
    counts[lo:hi] = 1
    dist.all_reduce(counts)                              # each unit owned exactly once
    dist.all_reduce(mine)                                # the optional gather: disjoint slabs, so a sum reassembles
    if rank == 0:
        full = oracle.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, softmax_scale=d ** -0.5, block_n=128, nthreads=1)
        got = mine.view(B, Hkv * grp, S, d).numpy()
        np.save(os.path.join(out_dir, "ok.npy"),
                np.array([float(np.array_equal(counts.numpy(), np.ones(B * Hkv))), float(np.abs(got - full["o_f32"]).max())]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_unit_sharding_and_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ok = np.load(tmp_path / "ok.npy")
    assert ok[0] == 1.0
    assert ok[1] == 0.0
