"""A linear split by output rows over the GPUs of one machine, one process per GPU.

Rank g of G holds rows [g*N/G, (g+1)*N/G) of the weight (a byte range of the GGUF tensor: no
requantisation), every rank holds the whole x, each computes its slice y_g [M, N/G] with the ordinary
kernels and an all-gather completes y [M, N] on every rank. The reference never shards a linear; the
collective mirrors its Collective.allGather(rank, input, output) (dist/Collective.java:64-65, NCCL form
dist/NcclOp.java:184-198: FP32 only, output persistent). The per-row arithmetic does not depend on the
shard, so the gathered result is bitwise the single-GPU result.

``torch.distributed`` is the plumbing (process group, NCCL or gloo); the linear itself is
``jq_linear_f32``. The row partition and the gather layout are plain functions so that they can be
tested without a GPU.

Two ways to complete y: ``gather_rows`` (a torch.distributed all-gather: NCCL on GPUs, gloo in the CPU
tests) and ``PeerGather`` (the library's own exchange: every rank stores its slice straight into every
rank's buffer over NVLink as marked 8-byte words and collects the others' words into its y,
``jq_peer_gather``; the process group only carries the 64-byte memory handles at set-up).
"""
import ctypes


def row_range(n, rank, world):
    """Rows [begin, end) of rank `rank`: contiguous, sizes differ by at most one, earlier ranks get the extras."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d of %d" % (rank, world))
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_rows(y_local, n, group=None):
    """All-gathers row slices y_g [M, rows_g] (torch tensors, equal M everywhere) into y [M, N] on every rank.

    Slices of equal width take one all_gather_into_tensor; ragged partitions (N not a multiple of the
    world size) are padded to the widest slice for the collective and trimmed afterwards.
    """
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m = y_local.shape[0]
    widths = [row_range(n, r, world)[1] - row_range(n, r, world)[0] for r in range(world)]
    if len(set(widths)) == 1:
        if m == 1:
            out = torch.empty(1, n, dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(out.view(-1), y_local.contiguous().view(-1), group=group)
            return out
        stacked = torch.empty(world, m, widths[0], dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(stacked.view(-1), y_local.contiguous().view(-1), group=group)
        return stacked.permute(1, 0, 2).reshape(m, n)
    wmax = max(widths)
    padded = torch.zeros(m, wmax, dtype=y_local.dtype, device=y_local.device)
    padded[:, :y_local.shape[1]] = y_local
    stacked = torch.empty(world, m, wmax, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(stacked.view(-1), padded.view(-1), group=group)
    return torch.cat([stacked[r, :, :w] for r, w in enumerate(widths)], dim=1)


class ShardedLinear:
    """y = x W^T (+ b) with W [N, K] split by rows over the ranks of a process group."""

    def __init__(self, dtype, blocks, n, k, device, group=None, bias=None):
        import torch.distributed as dist
        from .ops import Tensor
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.n, self.k = int(n), int(k)
        self.begin, self.end = row_range(self.n, self.rank, self.world)
        self.weight = Tensor.quantized(dtype, blocks, self.n, self.k, device=device, rows=(self.begin, self.end))
        self.bias = None if bias is None else bias[self.begin:self.end].contiguous()

    def local(self, x):
        """This rank's slice y_g [M, rows_g] for a CUDA tensor x [M, K] (no communication)."""
        from .ops import Gguf
        return Gguf.linear(x, self.weight, self.bias)

    def __call__(self, x):
        return gather_rows(self.local(x), self.n, self.group)


class PeerGather:
    """The gathered output y [m_max, n] of one sharded linear on every rank, filled by peer stores.

    Set-up (collective over the group): every rank allocates its buffer (two y areas, used in turn), the
    64-byte CUDA IPC handles travel through ``all_gather_object``, every rank maps the others' buffers.
    ``gather(y_local)`` enqueues the exchange on the current stream and returns this rank's y [m, n] as a
    torch tensor viewing the buffer; it stays valid until the next-but-one gather on this object.
    """

    def __init__(self, n, m_max, device, group=None):
        import torch.distributed as dist
        from . import _lib
        self.lib = _lib.load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n, self.m_max, self.device = int(n), int(m_max), int(device)
        self.begin, self.end = row_range(self.n, self.rank, self.world)
        self.y_bytes = (self.n * self.m_max * 4 + 255) // 256 * 256
        self.area = 3 * self.y_bytes  # y [m_max, n] floats, then the staging words [m_max, n] of 8 bytes that the exchange travels in
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        _lib.check(self.lib.jq_peer_alloc(self.device, 2 * self.area, ctypes.byref(own), handle))
        self.own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.buffers = (ctypes.c_void_p * self.world)()
        self.opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.buffers[r] = self.own
            else:
                p = ctypes.c_void_p()
                _lib.check(self.lib.jq_peer_open(self.device, ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                self.buffers[r] = p.value
                self.opened.append(p.value)
        self.turn = 0
        self.offset = int(self.lib.jq_peer_payload_offset())
        dist.barrier(group=group)

    def gather(self, y_local, stream=None):
        """y_local: CUDA float32 tensor [m, rows of this rank]. Returns y [m, n] (a view of this rank's buffer)."""
        import torch
        from . import _lib
        m = int(y_local.shape[0])
        if m > self.m_max or y_local.shape[1] != self.end - self.begin or y_local.dtype != torch.float32 or not y_local.is_contiguous():
            raise ValueError("PeerGather: slice %s does not fit rows [%d, %d) x at most %d" % (tuple(y_local.shape), self.begin, self.end, self.m_max))
        s = torch.cuda.current_stream(y_local.device).cuda_stream if stream is None else stream
        off = self.turn * self.area
        _lib.check(self.lib.jq_peer_gather(y_local.data_ptr(), m, self.end - self.begin, self.n, self.begin, self.buffers, off, off + self.y_bytes,
                                           self.rank, self.world, s))
        self.turn ^= 1
        return self.view(off, m)

    def linear(self, weight, x, bias=None, stream=None):
        """y = x W^T (+ bias) for this rank's row shard `weight` (a quantised Tensor), completed on every rank: the
        linear and the exchange in one library call (jq_linear_f32_peer). x: CUDA float32 [m, k]."""
        import torch
        from . import _lib
        m = int(x.shape[0])
        if m > self.m_max or x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("PeerGather.linear: x %s, at most %d rows of float32" % (tuple(x.shape), self.m_max))
        s = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
        off = self.turn * self.area
        _lib.check(self.lib.jq_linear_f32_peer(weight._handle(), x.data_ptr(), m, None if bias is None else bias.data_ptr(), self.n, self.begin,
                                               self.buffers, off, off + self.y_bytes, self.rank, self.world, s))
        self.turn ^= 1
        return self.view(off, m)

    def view(self, off, m):
        """This rank's y area at byte offset `off` of the payload as a torch tensor [m, n] (no copy)."""
        import torch

        class _Mem:
            pass
        holder = _Mem()
        holder.__cuda_array_interface__ = {"shape": (m, self.n), "typestr": "<f4", "data": (self.own + self.offset + off, False), "version": 3}
        return torch.as_tensor(holder, device=torch.device("cuda", self.device))

    def close(self):
        """Collective: unmaps the peers' buffers, then frees the own one once every rank has unmapped it."""
        import torch
        import torch.distributed as dist
        if self.own is None:
            return
        torch.cuda.synchronize(self.device)
        for p in self.opened:
            self.lib.jq_peer_close(p)
        self.opened = []
        dist.barrier(group=self.group)
        self.lib.jq_peer_free(self.own)
        self.own = None
