"""The N>1 path on CPU: two gloo ranks each take their contiguous run of (batch, head) units,
compute them independently (with the oracle standing in for the kernel), and the gathered result
equals the unsharded computation -- the equivalence the reference checks by splitting the batch
(tests/train/flash_attention/st/test_sharding.py:19-81).  Timing is reduced as max over ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from acctransformer_b200.sharding import max_over_ranks, shard_bnsd, unit_slice
from oracle import attention_ref as ref


def test_unit_slices_partition_the_units():
    for total in (1, 7, 64, 1024):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                a, b = unit_slice(total, r, world)
                seen.extend(range(a, b))
            assert seen == list(range(total))
    with pytest.raises(ValueError):
        unit_slice(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rs = np.random.RandomState(0)
    B, N, S, D = 2, 3, 160, 32
    q, k, v = (torch.tensor(rs.randn(B, N, S, D).astype(np.float16)) for _ in range(3))
    qs, ks, vs = (shard_bnsd(t, rank, world).numpy() for t in (q, k, v))
    o, lse = ref.sa_fwd(qs, ks, vs, causal=True, scale=0.2)
    gathered = [None] * world
    dist.all_gather_object(gathered, (o, lse))
    ms = max_over_ranks(10.0 + rank)
    if rank == 0:
        full_o = np.concatenate([g[0] for g in gathered], axis=1).reshape(B, N, S, D)
        full_l = np.concatenate([g[1] for g in gathered], axis=1).reshape(B, N, S)
        ro, rl = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy(), causal=True, scale=0.2)
        np.save(os.path.join(out_dir, "ok.npy"),
                np.array([np.array_equal(full_o, ro), np.array_equal(full_l, rl), ms == 10.0 + world - 1]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_equivalence(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ok = np.load(os.path.join(str(tmp_path), "ok.npy"))
    assert ok.all(), ok
