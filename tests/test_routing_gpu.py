"""embedding, copy_to_seq_context and select_experts on the GPU against the CPU oracle: all three are bit-exact
(row copies; the router's scores are a fixed sequence of IEEE operations on both sides, so expert ids, weights,
counts and prefix sums must be identical)."""
import numpy as np
import pytest
import torch

import oracle as O
from util import DT_NAME, FWD_DTS, TORCH_OF, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from dataflow_lib_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dt", FWD_DTS, ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("shape", [(1000, 4096), (37, 1000), (5, 33), (1, 8)], ids=str)
def test_embedding(ops, dt, shape):
    T, dim = shape
    vocab = 517
    table = O.fill_normal(dt, (vocab, dim), 1)
    ids = O.fill_labels(T, 2, vocab)
    ids[0], ids[-1] = vocab - 1, 0
    ref = O.embedding(dt, ids, table)
    out = torch.zeros((T, dim), dtype=TORCH_OF[dt], device="cuda")
    ops.embedding(T, dim, torch.from_numpy(ids.astype(np.int32)).cuda(), to_dev(table, dt), out)
    torch.cuda.synchronize()
    assert np.array_equal(to_host(out, dt), ref)


def test_embedding_unaligned_rows(ops):
    """bf16 rows of 6 bytes from a table view that starts 2 bytes into an allocation: the packet size drops to 2 bytes."""
    table = O.fill_normal(O.BF16, (50, 3), 3)
    ids = O.fill_labels(20, 4, 50)
    backing = torch.zeros(50 * 3 + 1, dtype=torch.bfloat16, device="cuda")
    view = backing[1:].view(50, 3)
    view.copy_(to_dev(table, O.BF16))
    out = torch.zeros((20, 3), dtype=torch.bfloat16, device="cuda")
    ops.embedding(20, 3, torch.from_numpy(ids.astype(np.int32)).cuda(), view, out)
    torch.cuda.synchronize()
    assert np.array_equal(to_host(out, O.BF16), O.embedding(O.BF16, ids, table))


@pytest.mark.parametrize("dt", [O.FP32, O.BF16, O.E4M3], ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("kv_dim,misalign", [(1024, 0), (40, 0), (1024, 1), (3, 0)], ids=str)
def test_copy_to_seq_context(ops, dt, kv_dim, misalign):
    """Three sequences of different context sizes in one device buffer; tokens of a batch land at scattered positions.
    misalign = 1 starts every context one element past a 16-byte boundary (the kernel's byte-store path)."""
    es = np.dtype(O.NP_OF[dt]).itemsize
    sizes = [64, 17, 128]
    per_ctx = [30, 17, 43]                                # tokens per sequence (the second one fills its context)
    T = sum(per_ctx)
    rng = np.random.default_rng(5)
    tok_ctx = rng.permutation(np.repeat(np.arange(3), per_ctx))
    pos = np.empty(T, np.int32)
    for c in range(3):                                    # distinct positions per context: the result has no write races
        pos[tok_ctx == c] = rng.permutation(sizes[c])[:per_ctx[c]]
    keys, values = O.fill_normal(dt, (T, kv_dim), 6), O.fill_normal(dt, (T, kv_dim), 7)
    npdt = O.NP_OF[dt]
    host_ctx = [np.full((2 * s, kv_dim), 0, npdt) for s in sizes]
    O.copy_to_seq_context(dt, keys, values, pos, host_ctx, tok_ctx, sizes)

    elems = [2 * s * kv_dim for s in sizes]
    pad = 16 // es
    offs, total = [], misalign
    for n in elems:
        offs.append(total)
        total += (n + pad - 1) // pad * pad
    buf = torch.zeros(total + pad, dtype=torch.uint8 if es == 1 else (torch.int16 if es == 2 else torch.int32), device="cuda")
    assert buf.data_ptr() % 16 == 0
    ptrs = np.array([buf.data_ptr() + offs[c] * es for c in tok_ctx], np.uint64)
    csz = np.array([sizes[c] for c in tok_ctx], np.int32)
    ops.copy_to_seq_context(T * kv_dim, T, kv_dim, to_dev(keys, dt), to_dev(values, dt), torch.from_numpy(pos).cuda(),
                            torch.from_numpy(ptrs.view(np.int64)).cuda(), torch.from_numpy(csz).cuda())
    torch.cuda.synchronize()
    got = buf.cpu().numpy().view(npdt if es != 4 else np.float32)
    for c in range(3):
        g = got[offs[c]:offs[c] + elems[c]].reshape(2 * sizes[c], kv_dim)
        assert np.array_equal(g.view(np.uint8), host_ctx[c].view(np.uint8)), c
    # nothing outside the contexts was written
    mask = np.ones(got.shape, bool)
    for c in range(3):
        mask[offs[c]:offs[c] + elems[c]] = False
    assert not got.view(np.uint8).reshape(-1, es)[mask].any()


@pytest.mark.parametrize("dt", FWD_DTS, ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("shape", [(1000, 64, 8), (37, 8, 2), (4096, 256, 6), (5, 40, 32), (129, 33, 1), (300, 16, 16)], ids=str)
def test_select_experts(ops, dt, shape):
    T, ne, k = shape
    X = O.fill_normal(dt, (T, ne), 11, 0.0, 2.0)           # 16- and 8-bit inputs contain many exact ties
    pre = np.zeros(ne + 1, np.int32)
    pre[:ne] = np.arange(ne) % 3                             # counts accumulate onto what the caller left there
    w_ref, ids_ref, counts_ref, cum_ref, routed_ref = O.select_experts(dt, X, k, counts_in=pre)
    w = torch.zeros((T, k), dtype=TORCH_OF[dt], device="cuda")
    ids = torch.zeros((T, k), dtype=torch.int16, device="cuda")
    counts = torch.from_numpy(pre).cuda()
    cum = torch.full((ne,), -7, dtype=torch.int32, device="cuda")
    routed = torch.full((ne,), -7, dtype=torch.int32, device="cuda")
    ops.select_experts(T, ne, k, to_dev(X, dt), w, ids, counts, cum, routed)
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy().view(np.uint16), ids_ref)
    assert np.array_equal(to_host(w, dt), w_ref)
    assert np.array_equal(counts.cpu().numpy(), counts_ref) and counts_ref[ne] == 0
    assert np.array_equal(cum.cpu().numpy(), cum_ref)
    assert np.array_equal(routed.cpu().numpy(), routed_ref) and not routed_ref.any()
    assert cum_ref[-1] == T * k + int(pre[:ne].sum())


def test_select_experts_through_the_handle():
    from dataflow_lib_b200 import DataflowHandle
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    T, ne, k = 16384, 64, 8
    X = O.fill_normal(O.BF16, (T, ne), 12)
    w_ref, ids_ref, counts_ref, cum_ref, _ = O.select_experts(O.BF16, X, k)
    h = DataflowHandle(device_id=0, num_streams=1)
    w = torch.zeros((T, k), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros((T, k), dtype=torch.int16, device="cuda")
    counts = torch.zeros(ne + 1, dtype=torch.int32, device="cuda")
    cum, routed = torch.zeros(ne, dtype=torch.int32, device="cuda"), torch.ones(ne, dtype=torch.int32, device="cuda")
    for _ in range(2):                                      # twice: the block counter must have been left at zero
        counts.zero_()
        assert h.submit_select_experts(0, DT.BF16, T, ne, k, to_dev(X, O.BF16), w, ids, counts, cum, routed) == 0
        h.sync_stream(0)
        assert np.array_equal(ids.cpu().numpy().view(np.uint16), ids_ref)
        assert np.array_equal(to_host(w, O.BF16), w_ref)
        assert np.array_equal(counts.cpu().numpy(), counts_ref)
        assert np.array_equal(cum.cpu().numpy(), cum_ref)
    tok = torch.from_numpy(O.fill_labels(100, 1, 300).astype(np.int32)).cuda()
    table = to_dev(O.fill_normal(O.BF16, (300, 256), 2), O.BF16)
    out = torch.empty((100, 256), dtype=torch.bfloat16, device="cuda")
    assert h.submit_embedding(0, DT.BF16, 100, 256, tok, table, out) == 0
    h.sync_stream(0)
    assert torch.equal(out, table[tok.long()])
    h.close()


def test_select_experts_rejects_bad_shapes(ops):
    z = torch.zeros(64, dtype=torch.float32, device="cuda")
    zi = torch.zeros(64, dtype=torch.int32, device="cuda")
    zs = torch.zeros(64, dtype=torch.int16, device="cuda")
    for T, ne, k in [(4, 4, 5), (4, 4, 0), (0, 4, 2), (4, 9000, 2), (4, 64, 33)]:
        with pytest.raises(RuntimeError):
            ops.select_experts(T, ne, k, z, z, zs, zi, zi, zi)
