"""Column-split ternary linear over 2 and 4 GPUs (the partition used for the 16384-wide case): with an NCCL
all-gather, and with the exchange done by the GEMM epilogue's own stores into every GPU's copy of the output.
Needs that many visible CUDA devices; with fewer the case is skipped."""
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
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"     # plain peer mappings: no multicast object is bound
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import oracle
    from oracle import fast
    from reimagined_b200.bitlinear import BitLinear
    from reimagined_b200.sharding import ColumnParallelBitLinear, PeerOutput
    P = oracle.port()
    ok = True
    # a small layer, then the 16384-wide layer the partition exists for (decode row, a 64-row batch on the
    # 2-bit strips and a 128-row batch on the tensor-core GEMM); every output compared bit for bit with the
    # unsharded CPU oracle
    for (N, K, rows) in [(512, 1024, (4,)), (16384, 16384, (1, 64, 128))]:
        rng = np.random.default_rng(9 + N)
        w = rng.standard_normal((N, K), dtype=np.float32)
        w *= np.float32(0.02)
        full = BitLinear.from_float(w)
        del w
        full.set_exact_linear_mode(True)
        t = P.unpack_i8(full.packed_weights, N, K)
        layer = ColumnParallelBitLinear(full, world, rank).to("cuda")
        for M in rows:
            x = rng.standard_normal((M, K), dtype=np.float32)
            y = layer.forward(torch.from_numpy(x).cuda()).cpu().numpy()
            want, *_ = fast.linear_forward(x, t, full.weight_scale)
            ok = ok and y.shape == want.shape and np.array_equal(y.view(np.uint32), want.view(np.uint32))
        # the fused exchange (tensor-core path, M > 64): every rank must end up with the whole output, twice in a
        # row into the same buffer (the second step overwrites the first after a barrier)
        for M in ((130, 77) if N == 512 else (128,)):
            peer = PeerOutput(M, N)
            for rep in range(2):
                x = rng.standard_normal((M, K), dtype=np.float32)
                peer.barrier()                      # everyone has finished reading the previous result
                y = layer.forward_fused(torch.from_numpy(x).cuda(), peer).cpu().numpy()
                want, *_ = fast.linear_forward(x, t, full.weight_scale)
                ok = ok and y.shape == want.shape and np.array_equal(y.view(np.uint32), want.view(np.uint32))
            del peer
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_split_all_gather(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(open(tmp_path / f"rank{r}.txt").read() == "1" for r in range(world))
