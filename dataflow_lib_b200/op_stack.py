"""A token-sharded training step over a stack of the library's ops, in the data flow of the reference's transformer
blocks (src/dataflow_models/src/dataflow_transformer.c: block forward = RMSNorm -> projections + RoPE -> ... ->
RMSNorm -> SwiGLU FFN with residual; head = RMSNorm -> vocabulary projection -> softmax -> cross entropy), reduced to
the ops this library provides:

    layer l :  h   = rms_norm(x_l, w_l)                      saves weighted sums and rms values
               k   = h[:, :n_kv * head_dim]                  the K view (a copy; nothing consumes it further)
               rope(h as Q, k)                               in place
               x_{l+1} = swiglu_ffn_fp8(h) + x_l             FP8 weights, residual added in the down projection's epilogue
    head    :  h = rms_norm(x_L, w_head);  logits = h @ W_vocab^T (library bf16 GEMM);  fused softmax + cross entropy
    backward:  d h = dlogits @ W_vocab (library GEMM);  rms_norm_bwd_x_w (dx += ..., weight gradient as fp32 column sums, one
               pass over x and d h) for the head, then per layer in reverse: FFN input gradient, rope_bwd_x, rms_norm_bwd_x_w
               accumulating into dx, which carries the residual branch.
    exchange:  [loss sum, valid rows | dW_0 .. dW_L], one packed fp32 buffer that the loss kernel and the weight-gradient kernels
               write directly (sharding.PackedReduction), summed over the ranks by the library's C exchange
               (include/dataflow_b200_exchange.h: NCCL called from C) on a stream of the step's handle.

Attention, the Q/K/V/O projections and the FFN weight gradients are not part of the step: the library has no kernels
for them. The vocabulary projection is the one library GEMM (torch.matmul -> cuBLASLt, as the reference uses cuBLASLt
for it); callers that account time per kernel exclude it.

Every op goes through the C-ABI launchers (ops.py) on stream 0 of the step's own Dataflow_Handle; there is no CPU path.
"""
import torch
import torch.distributed as dist

from . import ops
from .handle import DataflowHandle
from .sharding import Exchange, PackedReduction


_SHARED_HANDLES = {}


def _shared_handle(device_index):
    """One Dataflow_Handle per device for the steps that are not given one, kept until the process exits: the framework's allocators
    remember the stream a pinned buffer or a workspace was last used on and touch that stream again when the buffer is released, so
    a handle whose streams carried framework work must outlive every such buffer."""
    if device_index not in _SHARED_HANDLES:
        _SHARED_HANDLES[device_index] = DataflowHandle(device_id=device_index, num_streams=2, stream_prios=[0, -1], register_ops=False)
        _SHARED_HANDLES[device_index].keep_until_exit = True
    return _SHARED_HANDLES[device_index]


class OpStackStep:
    def __init__(self, tokens, d_model=4096, ffn_dim=14336, n_heads=32, n_kv_heads=8, head_dim=128, vocab=128256, n_layers=4,
                 eps=1e-5, theta=500000.0, device="cuda", handle=None):
        assert n_heads * head_dim == d_model
        self.T, self.d, self.f, self.V, self.L = tokens, d_model, ffn_dim, vocab, n_layers
        self.n_heads, self.n_kv, self.hd, self.eps, self.theta = n_heads, n_kv_heads, head_dim, eps, int(theta)
        self.kv_dim = n_kv_heads * head_dim
        dev, bf = torch.device(device), torch.bfloat16
        T, d, f, V, L = self.T, self.d, self.f, self.V, self.L
        e = lambda *shape, dtype=bf: torch.empty(*shape, dtype=dtype, device=dev)
        self.x = [e(T, d) for _ in range(L + 1)]                 # residual stream: x[0] is the step's input
        self.h, self.k, self.dk = e(T, d), e(T, self.kv_dim), e(T, self.kv_dim)
        self.G, self.U = [e(T, f) for _ in range(L)], [e(T, f) for _ in range(L)]
        self.ws, self.rms = [e(T, dtype=torch.float32) for _ in range(L + 1)], [e(T, dtype=torch.float32) for _ in range(L + 1)]
        self.logits, self.dlogits = e(T, V), e(T, V)
        self.dh, self.dA, self.dx = e(T, d), e(T, d), e(T, d)
        # The step's reductions over tokens live in a packed fp32 buffer that the kernels write directly: [loss sum, valid rows | dW_0 ..
        # dW_L] (dW[l]: gradient of layer l's RMSNorm weight; dW[L]: the head's). Two buffers alternate between steps, so that an
        # exchange running beside the next step is never overwritten by it.
        self.packed = [PackedReduction([d] * (L + 1), device=dev) for _ in range(2)]
        self._parity = 0
        self.pos = torch.arange(T, dtype=torch.int32, device=dev)
        self.labels = torch.zeros(T, dtype=torch.int32, device=dev)
        # weights (set_weights fills them)
        self.w_norm = [e(d) for _ in range(L + 1)]
        u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=dev)
        self.Wg, self.Wu, self.Wd = [u8(f, d) for _ in range(L)], [u8(f, d) for _ in range(L)], [u8(d, f) for _ in range(L)]
        self.sg, self.su = [e(f, dtype=torch.float32) for _ in range(L)], [e(f, dtype=torch.float32) for _ in range(L)]
        self.sd, self.sgu = [e(d, dtype=torch.float32) for _ in range(L)], [e(2 * f, dtype=torch.float32) for _ in range(L)]
        self.WguT, self.WdT = [u8(d, 2 * f) for _ in range(L)], [u8(f, d) for _ in range(L)]
        self.W_vocab = e(V, d)
        self.marks = None                                        # a list while a step is being profiled: (segment name, CUDA event) pairs
        # ops run on stream 0 of the handle, an overlapped exchange on its stream 1 (the caller's handle, else one shared per device)
        self.handle = handle if handle is not None else _shared_handle(dev.index if dev.index is not None else torch.cuda.current_device())
        self.stream = torch.cuda.ExternalStream(self.handle.stream_ptr(0), device=dev)
        self._xstream = torch.cuda.ExternalStream(self.handle.stream_ptr(1), device=dev)
        self._exchange = None                                    # made at the first exchange (needs the process group, if any)
        self._xdone = [None, None]                               # per packed buffer: event after its overlapped exchange
        self.reduced = None                                      # the packed buffer of the last exchanged step (global sums once its exchange is done)
        self.ffn_ws = torch.empty(int(ops._lib_.dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f)), dtype=torch.uint8, device=dev)   # forward and backward

    # ------------------------------------------------------------------ weights
    def set_weights(self, w_norm, ffn, W_vocab):
        """w_norm: L+1 bf16 [d] tensors; ffn: per layer (Wgate_q u8 [f,d], gate_scales [f], Wup_q, up_scales, Wdown_q u8 [d,f],
        down_scales [d]) as produced by quantize_rows_e4m3 on the bf16 weights; W_vocab bf16 [V, d]."""
        for l in range(self.L + 1):
            self.w_norm[l].copy_(w_norm[l])
        for l, (Wg, sg, Wu, su, Wd, sd) in enumerate(ffn):
            self.Wg[l].copy_(Wg); self.sg[l].copy_(sg); self.Wu[l].copy_(Wu); self.su[l].copy_(su); self.Wd[l].copy_(Wd); self.sd[l].copy_(sd)
            self.sgu[l].copy_(torch.cat([sg, su]))
            ops.ffn_fp8_prepare_bwd_weights(self.d, self.f, self.Wg[l], self.Wu[l], self.Wd[l], self.WguT[l], self.WdT[l])
        self.W_vocab.copy_(W_vocab)

    def random_weights(self, seed=0):
        """Random-init weights of the stack's shapes (identical on every rank for the same seed)."""
        g = torch.Generator(device=self.h.device).manual_seed(seed)
        rn = lambda *shape, std: (torch.randn(*shape, generator=g, device=self.h.device, dtype=torch.float32) * std)
        w_norm = [(1.0 + rn(self.d, std=0.02)).bfloat16() for _ in range(self.L + 1)]
        ffn = []
        for _ in range(self.L):
            row = []
            for shape in ((self.f, self.d), (self.f, self.d), (self.d, self.f)):
                W = rn(*shape, std=0.02).bfloat16()
                Q = torch.empty(shape, dtype=torch.uint8, device=W.device)
                s = torch.empty(shape[0], dtype=torch.float32, device=W.device)
                ops.quantize_rows_e4m3(shape[0], shape[1], W, Q, s)
                row += [Q, s]
            ffn.append(tuple(row))
        self.set_weights(w_norm, ffn, rn(self.V, self.d, std=0.02).bfloat16())

    # the current step's slots of the packed buffer
    @property
    def loss_sum(self):
        return self.packed[self._parity].loss

    @property
    def dW(self):
        return self.packed[self._parity].dW

    def _mark(self, name):
        """Segment boundary: when `marks` is a list, records an event that closes segment `name` on the current stream."""
        if self.marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(self.stream)
            self.marks.append((name, ev))

    def segment_ms(self):
        """Milliseconds per segment name summed over the events recorded since `marks` was set (call after a synchronize)."""
        out = {}
        for (_, e0), (name, e1) in zip(self.marks[:-1], self.marks[1:]):
            if name != "start":
                out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out

    # ------------------------------------------------------------------ the step
    def forward(self):
        T, d, f = self.T, self.d, self.f
        self._mark("start")
        for l in range(self.L):
            ops.rms_norm(T, d, self.eps, self.w_norm[l], self.x[l], self.h, self.ws[l], self.rms[l])
            self.k.copy_(self.h[:, :self.kv_dim])
            ops.rope(T * d, d, self.hd, self.n_kv, self.theta, self.pos, self.h, self.k)
            self._mark("rms_norm + rope")
            ops.swiglu_ffn_fp8(T, d, f, self.h, self.Wg[l], self.sg[l], self.Wu[l], self.su[l], self.Wd[l], self.sd[l], self.x[l + 1],
                               self.G[l], self.U[l], residual=self.x[l], workspace=self.ffn_ws)
            self._mark("swiglu_ffn_fp8")
        L = self.L
        ops.rms_norm(T, d, self.eps, self.w_norm[L], self.x[L], self.h, self.ws[L], self.rms[L])
        self._mark("rms_norm + rope")
        torch.matmul(self.h, self.W_vocab.t(), out=self.logits)
        self._mark("vocabulary GEMMs (library)")
        if self._xdone[self._parity] is not None:                 # this buffer's previous exchange (two steps ago) has long finished
            self.stream.wait_event(self._xdone[self._parity])
            self._xdone[self._parity] = None
        ops.softmax_cross_entropy(T, self.V, self.logits, self.labels, self.dlogits, None, self.loss_sum)
        self._mark("softmax_cross_entropy")

    def backward(self):
        T, d, f, L = self.T, self.d, self.f, self.L
        torch.matmul(self.dlogits, self.W_vocab, out=self.dh)
        self._mark("vocabulary GEMMs (library)")
        self.dx.zero_()
        ops.rms_norm_bwd_x_w(T, d, self.eps, self.ws[L], self.rms[L], self.w_norm[L], self.x[L], self.dh, self.dx, self.dW[L], sums=True)
        self.dk.zero_()                                           # nothing consumes K in this stack: its upstream gradient is zero
        self._mark("rms_norm_bwd + rope_bwd")
        for l in reversed(range(L)):
            ops.swiglu_ffn_fp8_bwd(T, d, f, self.dx, self.G[l], self.U[l], self.WdT[l], self.sd[l], self.WguT[l], self.sgu[l], self.dA,
                                   workspace=self.ffn_ws)
            self._mark("swiglu_ffn_fp8_bwd")
            ops.rope_bwd_x(T * d, d, self.hd, self.n_kv, self.theta, self.pos, self.dA, self.dk)
            ops.rms_norm_bwd_x_w(T, d, self.eps, self.ws[l], self.rms[l], self.w_norm[l], self.x[l], self.dA, self.dx, self.dW[l], sums=True)
            self._mark("rms_norm_bwd + rope_bwd")

    def _the_exchange(self, group):
        if self._exchange is None:
            self._exchange = Exchange(self.handle, group=group)
        return self._exchange

    def exchange(self, group=None):
        """The step's collective on the compute stream: afterwards `loss_sum` and `dW` hold the sums over all ranks."""
        packed = self.packed[self._parity]
        if self._the_exchange(group).all_reduce(0, packed) != 0:
            raise RuntimeError("exchange failed (see stderr)")
        self.reduced = packed.buffer
        self._mark("exchange")

    def exchange_overlapped(self, group=None):
        """The same all-reduce on the handle's second stream, behind a dependency on the compute stream, so that the next step's
        kernels run while this rank waits for the slowest one. `reduced` is this step's packed buffer; it holds the global sums once
        wait_exchange (or the exchange after next, which reuses the buffer) has ordered the compute stream after it."""
        packed = self.packed[self._parity]
        h = self.handle
        if h.submit_dependency(1, h.get_stream_state(0)) != 0 or self._the_exchange(group).all_reduce(1, packed) != 0:
            raise RuntimeError("exchange failed (see stderr)")
        done = torch.cuda.Event()
        done.record(self._xstream)
        self._xdone[self._parity] = done
        self.reduced = packed.buffer
        self._mark("exchange")

    def wait_exchange(self):
        """Orders the compute stream after every overlapped exchange issued so far (no host synchronisation)."""
        for i, ev in enumerate(self._xdone):
            if ev is not None:
                self.stream.wait_event(ev)
                self._xdone[i] = None

    def step(self, group=None, overlap=False):
        """One training step on the handle's compute stream (`self.stream`); the caller's current stream is not involved."""
        self._parity ^= 1
        self.stream.wait_stream(torch.cuda.current_stream())      # inputs the caller prepared on its own stream
        with torch.cuda.stream(self.stream):
            self.forward()
            self.backward()
            if overlap:
                self.exchange_overlapped(group)
            else:
                self.exchange(group)

    def close(self):
        """Leaves the communicator of the exchange. The handle stays (see _shared_handle); a caller's own handle is the caller's to close."""
        if self._exchange is not None:
            self._exchange.close()
            self._exchange = None

    # launches of this library's kernels in one step (for accounting): per layer fwd rms 1 + rope 1 + ffn 5 (2 row passes, 3 GEMMs),
    # bwd ffn 4 + rope 1 + norm bwd_x_w 2 (one pass + final sum); head rms 1 + softmax/CE 2 (rows + loss sum) + norm bwd_x_w 2
    def library_launches_per_step(self):
        return self.L * (1 + 1 + 5 + 4 + 1 + 2) + (1 + 2 + 2)
