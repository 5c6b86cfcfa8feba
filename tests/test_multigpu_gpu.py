"""One global batch sharded over 2 GPUs by (batch, KV head) units, as the multi-GPU path is specified: every rank
runs rk_attn_prefill on its contiguous block of units, the optional NCCL gather reassembles O, and the gathered
tensor equals the single-GPU result bit for bit.  Skipped where fewer than two GPUs are visible."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import radiance_kernels_b200 as rk
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    B, H, Hkv, S, d = 2, 8, 4, 512, 128
    grp = H // Hkv
    n_units = B * Hkv
    g = torch.Generator(device=dev).manual_seed(99)              # the same global problem on every rank
    Q = torch.randn(B, H, S, d, generator=g, device=dev)
    K = torch.randn(B, Hkv, S, d, generator=g, device=dev)
    V = torch.randn(B, Hkv, S, d, generator=g, device=dev)
    qc, qs = rk.mx_quantize(Q); kc, ks = rk.mx_quantize(K); vc, vs = rk.mx_quantize(V)
    lo, hi = rk.shard_range(n_units, rank, world)
    # a unit = one KV head with its `grp` query heads; a rank's block of units is a batch of such units
    unit = lambda t, heads: t.reshape(n_units, heads, *t.shape[2:])[lo:hi].contiguous()
    o_mine = rk.attn_prefill(unit(qc, grp), unit(kc, 1), unit(vc, 1), unit(qs, grp), unit(ks, 1), unit(vs, 1), causal=True)
    torch.cuda.synchronize()
    status = rk.last_device_status()
    full = torch.empty(n_units, grp, S, d, dtype=torch.bfloat16, device=dev)
    dist.all_gather_into_tensor(full, o_mine)                    # equal blocks: n_units % world == 0
    if rank == 0:
        whole = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
        torch.cuda.synchronize()
        same = torch.equal(full.view(B, H, S, d), whole)
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(f"{int(same)} {status} {rk.last_device_status()}\n")
    dist.barrier()
    dist.destroy_process_group()


def test_units_sharded_over_two_gpus_and_gathered(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    same, st0, st1 = (int(x) for x in open(tmp_path / "result.txt").read().split())
    assert same == 1 and st0 == 0 and st1 == 0
