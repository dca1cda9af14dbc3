"""World-size-2 test of the token-sharded step on CPU (gloo): ranks take contiguous row blocks, compute their partial
RMSNorm weight gradient and cross-entropy loss sum (here with the CPU oracle standing in for the kernels), and the one
packed all-reduce must reproduce the single-process result. Covers shard_rows edge cases as well."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from dataflow_lib_b200.sharding import PackedReduction, allreduce_packed, shard_rows

ROWS, COLS, VOCAB = 37, 64, 256


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    X, dY = O.fill_normal(O.FP32, (ROWS, COLS), 1), O.fill_normal(O.FP32, (ROWS, COLS), 2)
    rms = (1.0 / np.sqrt((X.astype(np.float64) ** 2).mean(1) + 1e-5)).astype(np.float32)
    logits, labels = O.fill_normal(O.FP32, (ROWS, VOCAB), 3, 0.0, 2.0), O.fill_labels(ROWS, 4, VOCAB)
    labels[5] = VOCAB + 1      # one invalid label
    return X, dY, rms, logits, labels


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    X, dY, rms, logits, labels = _inputs()
    start, count = shard_rows(ROWS, world, rank)
    sl = slice(start, start + count)
    dW = O.rms_norm_bwd_w(O.FP32, O.FP32, rms[sl].copy(), X[sl].copy(), dY[sl].copy(), np.zeros(COLS, np.float32), threads=1)
    _, _, ls = O.softmax_cross_entropy(O.FP32, O.FP32, logits[sl].copy(), labels[sl].copy(), threads=1)
    packed = PackedReduction([COLS])                           # the slots the kernels write on a GPU; the oracle's results stand in here
    packed.loss.copy_(torch.from_numpy(ls.copy()))
    packed.dW[0].copy_(torch.from_numpy(dW.copy()))
    allreduce_packed(packed)
    if rank == 0:
        out.put((packed.loss.numpy().copy(), packed.dW[0].numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_step_matches_single_process():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    loss_sum, dW = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    X, dY, rms, logits, labels = _inputs()
    ref_dW = O.rms_norm_bwd_w(O.FP32, O.FP32, rms, X, dY, np.zeros(COLS, np.float32), threads=1)
    _, _, ref_ls = O.softmax_cross_entropy(O.FP32, O.FP32, logits, labels, threads=1)
    np.testing.assert_allclose(dW, ref_dW, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(loss_sum[0], ref_ls[0], rtol=1e-5)
    assert loss_sum[1] == ref_ls[1] == ROWS - 1


def test_shard_rows_partitions_exactly():
    for n in (0, 1, 7, 8, 37, 131072):
        for world in (1, 2, 3, 8):
            blocks = [shard_rows(n, world, r) for r in range(world)]
            assert sum(c for _, c in blocks) == n
            assert blocks[0][0] == 0 and all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1


def test_packed_reduction_layout():
    p = PackedReduction([4, 6])
    assert len(p) == 12 and p.loss.data_ptr() == p.buffer.data_ptr()
    assert p.dW[0].data_ptr() == p.buffer.data_ptr() + 8 and p.dW[1].data_ptr() == p.buffer.data_ptr() + 8 + 16
    p.dW[1].fill_(3.0)
    assert p.buffer.tolist() == [0.0] * 6 + [3.0] * 6


def test_exchange_of_one_rank_needs_no_collective_library():
    """A world of one: the C exchange (include/dataflow_b200_exchange.h) sets up without NCCL and without a device, and its all-reduce
    is a no-op that succeeds; bad arguments are refused."""
    import ctypes as C
    from dataflow_lib_b200 import _lib, abi
    L = _lib.lib
    h, ex = abi.DataflowHandleStruct(), abi.DataflowExchange()
    assert L.dataflow_exchange_init(C.byref(ex), C.byref(h), 1, 0, None) == 0
    buf = torch.arange(5, dtype=torch.float32)
    assert L.dataflow_exchange_all_reduce_f32(C.byref(ex), 0, buf.data_ptr(), 5) == 0
    assert buf.tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]
    L.dataflow_exchange_destroy(C.byref(ex))
    assert L.dataflow_exchange_init(C.byref(ex), C.byref(h), 2, 2, None) == -1        # rank outside the world
    assert L.dataflow_exchange_init(C.byref(ex), C.byref(h), 2, 0, None) == -1        # several ranks need rank 0's id
    assert L.dataflow_exchange_all_reduce_f32(None, 0, buf.data_ptr(), 5) == -1
