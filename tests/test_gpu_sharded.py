"""Row-sharded linear on two GPUs (one process per GPU, NCCL): the gathered result equals the
single-GPU result bit for bit. Skipped on a machine with fewer than two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from jitnn_b200 import Gguf, Tensor, sharded, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    results = {}
    for t, n, k in [("Q4_K", 4096, 4096), ("Q6_K", 1000, 1024), ("Q8_0", 64, 256)]:
        g = torch.Generator().manual_seed(n)
        raw = synth.random_valid_blocks(t, n, k, seed=n).numpy()
        bias = torch.randn(n, generator=g).cuda()
        lin = sharded.ShardedLinear(t, raw, n, k, device=rank, bias=bias)
        whole = Tensor.quantized(t, raw, n, k, device=rank)
        for m in (1, 5):
            x = torch.randn(m, k, generator=g).cuda()
            y = lin(x)
            ref = Gguf.linear(x, whole, bias)
            results["%s_%d" % (t, m)] = bool(torch.equal(y, ref)) and tuple(y.shape) == (m, n)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "ok%d.npy" % rank), np.array([all(results.values())]))
    dist.destroy_process_group()


def test_two_gpu_sharded_linear_is_bitwise_the_single_gpu_linear(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert np.load(os.path.join(str(tmp_path), "ok%d.npy" % rank))[0]
