"""The token-sharded step's collective on real GPUs: include/dataflow_b200_exchange.h (NCCL called from C on a stream of each rank's
handle) with rms_norm_bwd_w_sums -- and, in the last step, the one-pass rms_norm_bwd_x_w_sums -- writing the fp32 column sums straight
into the packed buffer. One process per GPU, the communicator
id carried by a gloo process group (any channel will do); needs at least two GPUs, so it is skipped on a single-GPU box. No rank
leaves before all collectives have completed, NVLS off for the test (plain ring / tree paths)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROWS, COLS = 4096, 4096


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    from dataflow_lib_b200 import DataflowHandle
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    from dataflow_lib_b200.sharding import Exchange, PackedReduction
    h = DataflowHandle(device_id=rank, num_streams=2)
    ex = Exchange(h)                                             # rank 0's id reaches the others through the gloo group
    g = torch.Generator(device="cuda").manual_seed(10 + rank)
    X = torch.randn(ROWS, COLS, device="cuda", generator=g).bfloat16()
    dY = torch.randn(ROWS, COLS, device="cuda", generator=g).bfloat16()
    rms = torch.rsqrt(X.float().pow(2).mean(1) + 1e-5)
    packed = PackedReduction([COLS], device="cuda")
    torch.cuda.synchronize()
    BF = int(DT.BF16)
    for step in range(3):                                        # the buffer is overwritten, not accumulated: every step gives the same sums
        packed.loss.copy_(torch.tensor([float(rank + 1), float(ROWS)], device="cuda"))
        torch.cuda.synchronize()
        if step < 2:
            assert h.submit_rms_norm_bwd_w_sums(0, BF, BF, ROWS, COLS, 1e-5, rms, X, dY, packed.dW[0]) == 0
        else:        # the same sums from the op that also does the input gradient (its own summation order over the rows)
            ws, w, dX = torch.zeros(ROWS, device="cuda"), torch.ones(COLS, device="cuda").bfloat16(), torch.zeros_like(X)
            assert h.submit_rms_norm_bwd_x_w(0, BF, BF, ROWS, COLS, 1e-5, ws, rms, w, X, dY, dX, packed.dW[0], sums=True) == 0
        assert h.submit_dependency(1, h.get_stream_state(0)) == 0
        assert ex.all_reduce(1, packed) == 0
        assert h.sync_stream(1) == 0
    local = (dY.float() * X.float() * rms[:, None]).double().sum(0).cpu()
    out.put((rank, packed.buffer.cpu().numpy().copy(), local.numpy()))
    dist.barrier()
    ex.close()
    h.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_sum_their_packed_buffers():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, (buf, local)) for r, buf, local in (q.get(timeout=300) for _ in range(world)))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    total = got[0][1] + got[1][1]
    for r in range(world):
        buf = got[r][0]
        assert buf[0] == 3.0 and buf[1] == 2 * ROWS                       # loss slots: 1 + 2, and the row counts
        np.testing.assert_allclose(buf[2:], total, rtol=2e-5, atol=2e-5 * np.sqrt(2 * ROWS))
    assert np.array_equal(got[0][0], got[1][0])                          # every rank holds the same sums
