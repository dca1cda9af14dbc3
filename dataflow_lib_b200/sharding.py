"""Token sharding for the multi-GPU step: every op on the path is row-independent except two sums over tokens
(the RMSNorm weight gradient and the cross-entropy loss), so ranks take contiguous row blocks, run the ops locally
and exchange one small packed fp32 buffer [loss_sum, valid_rows, dW...] with a single all-reduce."""
import torch
import torch.distributed as dist


def shard_rows(n_rows: int, world: int, rank: int):
    """Contiguous block of rows for `rank`: the first n_rows % world ranks get one extra row. Returns (start, count)."""
    base, extra = divmod(n_rows, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def pack_reduction(loss_sum: torch.Tensor, dW_list):
    """[loss_sum(2) | dW_0 | dW_1 ...] as one fp32 vector on the tensors' device."""
    parts = [loss_sum.float().reshape(-1)] + [d.float().reshape(-1) for d in dW_list]
    return torch.cat(parts)


def unpack_reduction(buf: torch.Tensor, loss_sum: torch.Tensor, dW_list):
    loss_sum.copy_(buf[:loss_sum.numel()].reshape(loss_sum.shape))
    off = loss_sum.numel()
    for d in dW_list:
        d.copy_(buf[off:off + d.numel()].reshape(d.shape).to(d.dtype))
        off += d.numel()


def allreduce_step(loss_sum: torch.Tensor, dW_list, group=None):
    """The step's only collective: sums the per-rank loss sums, valid-row counts and weight gradients in fp32."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    buf = pack_reduction(loss_sum, dW_list)
    dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    unpack_reduction(buf, loss_sum, dW_list)
