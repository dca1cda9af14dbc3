"""Token sharding for the multi-GPU step: every op on the path is row-independent except two sums over tokens
(the RMSNorm weight gradients and the cross-entropy loss), so ranks take contiguous row blocks, run the ops locally
and exchange one small packed fp32 buffer [loss sum, valid rows | dW_0 | dW_1 ...] with a single sum all-reduce.

    shard_rows        which rows a rank owns
    PackedReduction   the packed buffer and its slots: kernels write their fp32 results straight into the slots
                      (submit_softmax_cross_entropy's loss_sum, submit_rms_norm_bwd_w_sums' column_sums), so nothing is packed
                      or unpacked around the collective
    Exchange          the collective itself, through the library's C entry points (include/dataflow_b200_exchange.h: NCCL called
                      from C on a stream of the rank's handle); torch.distributed only carries the 128-byte id to the ranks
    allreduce_packed  the same sum through torch.distributed, for the CPU (gloo) tests of the host-side logic
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import _lib, abi


def shard_rows(n_rows: int, world: int, rank: int):
    """Contiguous block of rows for `rank`: the first n_rows % world ranks get one extra row. Returns (start, count)."""
    base, extra = divmod(n_rows, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


class PackedReduction:
    """[loss sum, valid rows | dW_0 | ... | dW_{n-1}] as one fp32 vector with named views."""

    def __init__(self, dW_sizes, device="cpu"):
        self.sizes = [int(s) for s in dW_sizes]
        self.buffer = torch.zeros(2 + sum(self.sizes), dtype=torch.float32, device=device)
        self.loss = self.buffer[:2]
        self.dW, off = [], 2
        for s in self.sizes:
            self.dW.append(self.buffer[off:off + s])
            off += s

    def __len__(self):
        return self.buffer.numel()


def allreduce_packed(packed: PackedReduction, group=None):
    """The step's collective through torch.distributed (CPU tests with gloo)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed.buffer, op=dist.ReduceOp.SUM, group=group)


class Exchange:
    """dataflow_exchange_* of the C library on a DataflowHandle. With torch.distributed initialised, rank 0's unique id reaches
    the other ranks through one broadcast; a world of one needs neither."""

    def __init__(self, handle, world=None, rank=None, group=None):
        L = _lib.lib
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.handle, self.world, self.rank = handle, world, rank
        self.ex = abi.DataflowExchange()
        ident = None
        if world > 1:
            ident_t = torch.zeros(abi.EXCHANGE_ID_BYTES, dtype=torch.uint8)
            if rank == 0:
                raw = (C.c_uint8 * abi.EXCHANGE_ID_BYTES)()
                if L.dataflow_exchange_unique_id(raw) != 0:
                    raise RuntimeError("dataflow_exchange_unique_id failed (see stderr)")
                ident_t = torch.tensor(list(raw), dtype=torch.uint8)
            on_gpu = dist.get_backend(group) == "nccl"
            ident_t = ident_t.cuda() if on_gpu else ident_t
            dist.broadcast(ident_t, src=0, group=group)
            ident = (C.c_uint8 * abi.EXCHANGE_ID_BYTES)(*ident_t.cpu().tolist())
        if L.dataflow_exchange_init(C.byref(self.ex), C.byref(handle.h), world, rank, ident) != 0:
            raise RuntimeError("dataflow_exchange_init failed (see stderr)")

    def all_reduce(self, stream_id, packed, count=None):
        """In place on `packed` (a PackedReduction, an fp32 CUDA tensor or a device address), on the handle's stream `stream_id`."""
        buf = packed.buffer if isinstance(packed, PackedReduction) else packed
        ptr = buf.data_ptr() if hasattr(buf, "data_ptr") else int(buf)
        n = count if count is not None else buf.numel()
        return _lib.lib.dataflow_exchange_all_reduce_f32(C.byref(self.ex), stream_id, ptr, n)

    def close(self):
        _lib.lib.dataflow_exchange_destroy(C.byref(self.ex))
