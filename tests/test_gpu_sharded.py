"""Row-sharded linear on two GPUs (one process per GPU): the gathered result equals the single-GPU result bit for
bit, both with the NCCL all-gather and with the library's own peer-store exchange (also replayed from a CUDA graph).
The row-sharded decoder: logits and greedy tokens of every rank are bitwise those of the unsharded decoder.
Skipped on a machine with fewer than two GPUs."""
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
    import ctypes
    import torch.distributed as dist
    import jitnn_b200
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
        peer = sharded.PeerGather(n, 5, device=rank)
        for m in (1, 5):
            x = torch.randn(m, k, generator=g).cuda()
            y = lin(x)
            ref = Gguf.linear(x, whole, bias)
            results["%s_%d" % (t, m)] = bool(torch.equal(y, ref)) and tuple(y.shape) == (m, n)
            for rep in range(3):  # both y areas of the buffer, and one of them again
                yp = peer.gather(lin.local(x))
                results["%s_%d_peer%d" % (t, m, rep)] = bool(torch.equal(yp, ref)) and tuple(yp.shape) == (m, n)
                yl = peer.linear(lin.weight, x, lin.bias)  # linear and exchange in one call (fused epilogue for Q4_K)
                results["%s_%d_peerlin%d" % (t, m, rep)] = bool(torch.equal(yl, ref)) and tuple(yl.shape) == (m, n)
        peer.close()
    # the exchange inside a captured graph: the sequence numbers live on the device, so replays stay in step
    n, k = 4096, 4096
    raw = synth.random_valid_blocks("Q4_K", n, k, seed=5).numpy()
    lin = sharded.ShardedLinear("Q4_K", raw, n, k, device=rank)
    whole = Tensor.quantized("Q4_K", raw, n, k, device=rank)
    peer = sharded.PeerGather(n, 1, device=rank)
    x = torch.randn(1, k, generator=torch.Generator().manual_seed(9)).cuda()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        views = [peer.gather(lin.local(x)) for _ in range(2)]  # warm-up outside the graph (allocations)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            views = [peer.linear(lin.weight, x) for _ in range(2)]
        ref = Gguf.linear(x, whole, None)
        for rep in range(4):
            for v in views:
                v.zero_()
            stream.synchronize()
            dist.barrier()
            graph.replay()
            stream.synchronize()
            results["graph_%d" % rep] = all(bool(torch.equal(v, ref)) for v in views)
    status = ctypes.c_int(0)
    jitnn_b200.load().jq_device_status(rank, ctypes.byref(status))
    results["status"] = status.value == 0
    dist.barrier()
    peer.close()
    bad = [name for name, ok in results.items() if not ok]
    if bad:
        print("rank", rank, "failed:", bad, flush=True)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "ok%d.npy" % rank), np.array([all(results.values())]))
    dist.destroy_process_group()


def test_two_gpu_sharded_linear_is_bitwise_the_single_gpu_linear(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert np.load(os.path.join(str(tmp_path), "ok%d.npy" % rank))[0]


def _decoder_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import ctypes
    import torch.distributed as dist
    import jitnn_b200
    from jitnn_b200 import LlamaDecoder
    from oracle import llama_oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    L = jitnn_b200.load()
    results = {}
    # grouped-query attention with one key/value head per rank, and mixed formats (Q6_K takes the scatter kernel).
    # With the general kernels (decoder_fused 0) both decoders do the same arithmetic per row: bitwise equal. With the
    # fused kernels the single-token steps sum the norms and the attention in other orders: equal within the decoder
    # tolerance (2e-4 of the largest logit), same token wherever the top-2 margin is decisive.
    for fused in (0, 1):
        L.jq_set_option(b"decoder_fused", fused)
        # the third case is all Q4_K: with the fused kernels both activation images (attention, SwiGLU) are exchanged
        all_q4k = {"wv": "Q4_K", "w2": "Q4_K", "output": "Q4_K"}
        for case, (dim, heads, kv_heads, prompt_len, formats) in enumerate([(512, 4, 2, 21, None), (256, 4, 4, 61, None), (512, 4, 4, 70, all_q4k)]):
            cfg = llama_oracle.Config(layers=2, dim=dim, heads=heads, kv_heads=kv_heads, hidden=2 * dim, vocab=512, max_seq=prompt_len + 16)
            weights = llama_oracle.random_model(cfg, seed=31 + case, formats=formats)
            args = (cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq, cfg.eps, cfg.rope_base)
            whole = LlamaDecoder(*args, device=rank)
            whole.load(weights)
            split = LlamaDecoder(*args, device=rank, sharded=True)
            split.load(weights)
            prompt = np.random.default_rng(5 + case).integers(0, cfg.vocab, prompt_len).astype(np.int32)
            ok = True
            for i in range(0, prompt_len, 8):
                a, na = whole.forward(prompt[i:i + 8], i)
                b, nb = split.forward(prompt[i:i + 8], i)
                ok = ok and np.array_equal(a, b) and np.array_equal(na, nb)  # several tokens per call: general kernels in both
            results["prompt%d_%d" % (case, fused)] = ok
            tok, pos, ok = int(na[-1]), prompt_len, True
            for _ in range(10):  # the second single-token call captures the step, exchanges included, into a CUDA graph
                a, na = whole.forward([tok], pos)
                b, nb = split.forward([tok], pos)
                if fused == 0:
                    ok = ok and np.array_equal(a, b) and int(na[0]) == int(nb[0])
                else:
                    scale = np.abs(a).max()
                    top = np.sort(a[0])[-2:]
                    ok = ok and np.abs(a - b).max() <= 2e-4 * scale and (int(na[0]) == int(nb[0]) or top[1] - top[0] <= 1e-4 * scale)
                tok, pos = int(na[0]), pos + 1
            results["decode%d_%d" % (case, fused)] = ok
            whole.close()
            split.close()
    L.jq_set_option(b"decoder_fused", 1)
    status = ctypes.c_int(0)
    L.jq_device_status(rank, ctypes.byref(status))
    results["status"] = status.value == 0
    bad = [name for name, ok in results.items() if not ok]
    if bad:
        print("rank", rank, "failed:", bad, flush=True)
    np.save(os.path.join(out_dir, "dec%d.npy" % rank), np.array([all(results.values())]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_sharded_decoder_is_bitwise_the_single_gpu_decoder(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_decoder_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert np.load(os.path.join(str(tmp_path), "dec%d.npy" % rank))[0]
