"""Host-side multi-GPU logic on CPU: world_size-2 gloo processes check the row partition and the
column split + all-gather assembly against the unsharded oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from reimagined_b200 import sharding


def test_row_range_is_a_partition():
    for total in (0, 1, 5, 64, 4097):
        for world in (1, 2, 3, 8):
            spans = [sharding.row_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.row_range(4, 2, 2)
    with pytest.raises(ValueError):
        sharding.column_range(10, 4, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    P = oracle.port()
    rng = np.random.default_rng(42)          # same data on every rank
    N, K, M = 64, 128, 5
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    words, scale, *_ = P.pack_weights(w)
    full, *_ = P.linear_forward(x, words, scale, N)

    # (a) rows sharded, weights replicated: concatenating the ranks' outputs gives the full result
    lo, hi = sharding.row_range(M, world, rank)
    mine, *_ = P.linear_forward(x[lo:hi], words, scale, N) if hi > lo else (np.zeros((0, N), np.float32),)
    parts = [None] * world                     # ragged slices (5 rows over 2 ranks): gather as objects
    dist.all_gather_object(parts, mine)
    rows_ok = np.array_equal(np.concatenate(parts).view(np.uint32), full.view(np.uint32))

    # (b) columns sharded with the GLOBAL scale, then all-gathered
    shard_words = sharding.column_shard_words(words, N, K, world, rank)
    clo, chi = sharding.column_range(N, world, rank)
    local, *_ = P.linear_forward(x, shard_words, scale, chi - clo)
    gathered = sharding.gather_columns(torch.from_numpy(local), world).numpy()
    cols_ok = np.array_equal(gathered.view(np.uint32), full.view(np.uint32))
    # a shard re-packed on its own would get a different absmean: the global scale matters
    _, local_scale, *_ = P.pack_weights(w[clo:chi])
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(rows_ok)} {int(cols_ok)} {int(local_scale != scale)}")
    dist.destroy_process_group()


def test_two_rank_row_and_column_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        rows_ok, cols_ok, scale_differs = open(tmp_path / f"rank{r}.txt").read().split()
        assert rows_ok == "1" and cols_ok == "1"
