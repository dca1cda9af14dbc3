"""Launches the REFERENCE's own kernels on the GPU: oracle/_ref/cuda_kernels.cubin is als244/dataflow_lib's
src/ops/nvidia/cuda_kernels.cu compiled unchanged for sm_100a (oracle/Makefile). Test infrastructure only.

Launch geometry follows the reference's *_config.c (grid = SM count or rows, 1024 threads), with the one
correction needed to run rms_norm_bwd_x at all: its dynamic shared memory is sized for what the kernel
actually indexes (n_cols + 2*max_rows floats; src/ops/nvidia/norm/rms_norm_bwd_x.cu:188-197) instead of the
n_cols + max_rows floats of src/ops/nvidia/norm/rms_norm_config.c:135. cross_entropy_loss is not launched:
as written it only touches row 0 (loss/cross_entropy.cu:40)."""
import ctypes as C
import os

import torch

CUBIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "cuda_kernels.cubin")


def available():
    if not os.path.exists(CUBIN) or not torch.cuda.is_available():
        return False
    try:
        from cuda.bindings import driver  # noqa: F401
        return True
    except Exception:
        return False


class RefKernels:
    def __init__(self):
        from cuda.bindings import driver as drv
        self.drv = drv
        torch.cuda.init()
        torch.zeros(1, device="cuda")                     # makes the primary context current
        err, self.module = drv.cuModuleLoad(CUBIN.encode())
        assert err == drv.CUresult.CUDA_SUCCESS, err
        self.sms = torch.cuda.get_device_properties(0).multi_processor_count
        self._fn = {}

    def fn(self, name, max_dyn_smem=0):
        if name not in self._fn:
            err, f = self.drv.cuModuleGetFunction(self.module, name.encode())
            assert err == self.drv.CUresult.CUDA_SUCCESS, (name, err)
            self._fn[name] = f
        f = self._fn[name]
        if max_dyn_smem > 48 * 1024:
            (err,) = self.drv.cuFuncSetAttribute(f, self.drv.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, max_dyn_smem)
            assert err == self.drv.CUresult.CUDA_SUCCESS, err
        return f

    def launch(self, name, grid, block, smem, args, types):
        stream = torch.cuda.current_stream().cuda_stream
        f = self.fn(name, smem)
        (err,) = self.drv.cuLaunchKernel(f, grid, 1, 1, block, 1, 1, smem, stream, (tuple(args), tuple(types)), 0)
        assert err == self.drv.CUresult.CUDA_SUCCESS, (name, err)

    # ---- ops (tensors are torch CUDA tensors; dtype names as in the reference's symbol names) ----
    def rms_norm(self, name_dt, elt, n_rows, n_cols, eps, w, X, out, ws, rms):
        self.launch(f"rms_norm_{name_dt}_kernel", self.sms, 1024, 2 * elt * n_cols,
                    [n_rows, n_cols, eps, w.data_ptr(), X.data_ptr(), out.data_ptr(), ws.data_ptr(), rms.data_ptr()],
                    [C.c_int, C.c_int, C.c_float] + [C.c_void_p] * 5)

    def rms_norm_bwd_x(self, name_dts, n_rows, n_cols, eps, ws, rms, w, X, dY, dX):
        grid = self.sms
        max_rows = -(-n_rows // grid)
        self.launch(f"rms_norm_bwd_x_{name_dts}_kernel", grid, 1024, 4 * (n_cols + 2 * max_rows),
                    [n_rows, n_cols, eps, ws.data_ptr(), rms.data_ptr(), w.data_ptr(), X.data_ptr(), dY.data_ptr(), dX.data_ptr()],
                    [C.c_int, C.c_int, C.c_float] + [C.c_void_p] * 6)

    def rms_norm_bwd_w(self, name_dts, n_rows, n_cols, eps, rms, X, dY, dW):
        grid = self.sms
        max_rows = -(-n_rows // grid)
        self.launch(f"rms_norm_bwd_w_{name_dts}_kernel", grid, 1024, 4 * (n_cols + max_rows),
                    [n_rows, n_cols, eps, rms.data_ptr(), X.data_ptr(), dY.data_ptr(), dW.data_ptr()],
                    [C.c_int, C.c_int, C.c_float] + [C.c_void_p] * 4)

    def rope(self, name_dt, N, model_dim, head_dim, num_kv_heads, theta, pos, Xq, Xk, bwd=False):
        sym = f"rope_bwd_x_{name_dt}_kernel" if bwd else f"rope_{name_dt}_kernel"
        self.launch(sym, -(-(N // 2) // 1024), 1024, 0,
                    [N, model_dim, head_dim, num_kv_heads, theta, pos.data_ptr(), Xq.data_ptr(), Xk.data_ptr()],
                    [C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 3)

    def swiglu(self, name_dt, rows, cols, x1, x3, out):
        self.launch(f"swiglu_{name_dt}_kernel", rows, 1024, 0, [rows, cols, x1.data_ptr(), x3.data_ptr(), out.data_ptr()],
                    [C.c_int, C.c_int] + [C.c_void_p] * 3)

    def swiglu_bwd_x(self, name_dts, rows, cols, x1, x3, dY, d1, d3):
        self.launch(f"swiglu_bwd_x_{name_dts}_kernel", rows, 1024, 0,
                    [rows, cols, x1.data_ptr(), x3.data_ptr(), dY.data_ptr(), d1.data_ptr(), d3.data_ptr()],
                    [C.c_int, C.c_int] + [C.c_void_p] * 5)

    def softmax(self, name_dts, rows, cols, X, out):
        self.launch(f"softmax_{name_dts}_kernel", rows, 1024, 0, [rows, cols, X.data_ptr(), out.data_ptr()],
                    [C.c_int, C.c_int] + [C.c_void_p] * 2)

    def softmax_fp32_out(self, name_dt, rows, cols, X, out, arg_maxs):
        """softmax_<fp16|bf16>_fp32_kernel (src/ops/nvidia/loss/softmax.cu:965-1249): fp32 probabilities + the index of each row's maximum."""
        self.launch(f"softmax_{name_dt}_fp32_kernel", rows, 1024, 0, [rows, cols, X.data_ptr(), out.data_ptr(), arg_maxs.data_ptr()],
                    [C.c_int, C.c_int] + [C.c_void_p] * 3)

    def copy_to_seq_context(self, name_dt, total_tokens, kv_dim, keys, values, seq_positions, seq_context_ptrs, seq_context_sizes):
        """copy_to_seq_context_<dt>_kernel (src/ops/nvidia/attention/copy_to_seq_context.cu), launch geometry of attn_misc_config.c:56-79."""
        N = total_tokens * kv_dim
        self.launch(f"copy_to_seq_context_{name_dt}_kernel", -(-N // 1024), 1024, 0,
                    [N, total_tokens, kv_dim, keys.data_ptr(), values.data_ptr(), seq_positions.data_ptr(), seq_context_ptrs.data_ptr(),
                     seq_context_sizes.data_ptr()], [C.c_uint64, C.c_int, C.c_int] + [C.c_void_p] * 5)

    def select_experts(self, name_dt, total_tokens, n_experts, top_k, X, weights, chosen, counts, cumsum, routed, blocks=64, threads=128):
        """select_experts_<dt>_kernel (src/ops/nvidia/moe/select_experts.cu). The reference has no launch configuration for it; this one keeps
        the conditions its code needs: blocks <= total_tokens (a block without rows returns before it reports completion, and block 0 waits for
        every block, :18-20,198-202), n_experts a multiple of 32 (full-mask shuffles in the prefix sum, :217-231), and dynamic shared memory for
        its four arrays (:44-56)."""
        assert blocks <= total_tokens and n_experts % 32 == 0 and threads % 32 == 0 and (threads // 32 * top_k) % 2 == 0
        warps = threads // 32
        smem = 4 * warps * 32 + 4 * warps * top_k + 2 * warps * top_k + 4 * n_experts
        self.launch(f"select_experts_{name_dt}_kernel", blocks, threads, smem,
                    [total_tokens, n_experts, top_k, X.data_ptr(), weights.data_ptr(), chosen.data_ptr(), counts.data_ptr(), cumsum.data_ptr(),
                     routed.data_ptr()], [C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6)

