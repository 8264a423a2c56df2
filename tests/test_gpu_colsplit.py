"""Column-split ternary linear over 2 GPUs with an NCCL all-gather (the partition used for the 16384-wide
case).  Needs two visible CUDA devices; on a single-GPU box the test is skipped."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import oracle
    from reimagined_b200.bitlinear import BitLinear
    from reimagined_b200.sharding import ColumnParallelBitLinear
    P = oracle.port()
    rng = np.random.default_rng(9)
    N, K, M = 512, 1024, 4
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    full = BitLinear.from_float(w)
    full.set_exact_linear_mode(True)
    layer = ColumnParallelBitLinear(full, world, rank).to("cuda")
    y = layer.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    want, *_ = P.linear_forward(x, full.packed_weights, full.weight_scale, N)
    ok = np.array_equal(y.view(np.uint32), want.view(np.uint32))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


def test_column_split_all_gather_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(open(tmp_path / f"rank{r}.txt").read() == "1" for r in range(2))
