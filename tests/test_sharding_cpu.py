"""Host logic of the row-sharded linear on CPU: the row partition and the all-gather layout, with two
gloo ranks as child processes (the linear itself is replaced by the oracle: no GPU here)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT
from jitnn_b200 import sharded


def test_row_ranges_cover_without_overlap():
    for n in (1, 7, 8, 23, 4096, 11008, 32000):
        for world in (1, 2, 3, 4, 8):
            ranges = [sharded.row_range(n, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            for a, b in zip(ranges, ranges[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharded.row_range(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n, k, m, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from jitnn_b200 import sharded as sh
    from jitnn_b200 import synth
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    raw = synth.random_valid_blocks("Q4_K", n, k, seed=17).numpy()
    x = np.random.default_rng(5).standard_normal((m, k)).astype(np.float32)
    begin, end = sh.row_range(n, rank, world)
    row_bytes = k // 256 * 144
    local = oracle.linear("Q4_K", raw[begin:end].reshape(-1), x, None, n=end - begin)
    assert raw[begin:end].size == (end - begin) * row_bytes
    y = sh.gather_rows(torch.from_numpy(local), n)
    np.save(os.path.join(out_dir, "y%d.npy" % rank), y.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("n,m", [(24, 1), (24, 3), (23, 2)])
def test_two_rank_gather_equals_the_whole_linear(tmp_path, n, m):
    from jitnn_b200 import synth
    from oracle import oracle
    k, world = 512, 2
    mp.spawn(_worker, args=(world, _free_port(), n, k, m, str(tmp_path)), nprocs=world, join=True)
    raw = synth.random_valid_blocks("Q4_K", n, k, seed=17).numpy()
    x = np.random.default_rng(5).standard_normal((m, k)).astype(np.float32)
    whole = oracle.linear("Q4_K", raw, x, None)
    for rank in range(world):
        got = np.load(os.path.join(str(tmp_path), "y%d.npy" % rank))
        assert got.shape == (m, n)
        assert np.array_equal(got.view(np.uint32), whole.view(np.uint32))
