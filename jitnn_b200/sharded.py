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
