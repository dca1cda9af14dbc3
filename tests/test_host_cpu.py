"""CPU tests of the host layer: the C-ABI library loads without a GPU and exports every declared symbol,
the registry reproduces the reference's fingerprints (tests/golden/fingerprints.json, generated from the
reference's own host sources), SHA-256 known answers, the hash table, datatype helpers, and the error
behaviour of the handle API when no device is present."""
import ctypes as C
import json
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "fingerprints.json")))


@pytest.fixture(scope="module")
def L():
    from dataflow_lib_b200 import _lib
    return _lib.lib


def test_library_exports_every_declared_symbol(L):
    """Every function prototype in include/*.h must resolve in the shared object."""
    declared = set()
    for hdr in ("dataflow_b200_kernels.h", "dataflow_api.h"):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"typedef[^;]*;", "", text)
        declared |= set(re.findall(r"\b([a-z_][a-z0-9_]*)\s*\([^;{]*\)\s*;", text))
    declared -= {"defined"}
    assert len(declared) > 60
    missing = [n for n in sorted(declared) if not hasattr(L, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    from dataflow_lib_b200 import _lib
    bound = set(_lib.KERNEL_ABI) | set(_lib.HOST_ABI)
    assert declared <= bound, f"no ctypes signature for {sorted(declared - bound)}"
    assert L.dfb200_target_arch() == b"sm_100a"


def test_library_has_no_undefined_cuda_driver_dependency():
    """The library must load on a machine without libcuda (driver entry points are resolved lazily)."""
    from dataflow_lib_b200 import _lib
    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "libcuda.so" not in out and "libcudart" not in out and "not found" not in out, out


def test_struct_layouts_match_reference(tmp_path):
    """sizeof/offsetof of every ABI struct: include/dataflow_abi.h against the reference's headers (golden)."""
    exe = str(tmp_path / "abi_layout")
    subprocess.check_call(["gcc", f"-I{ROOT}/include", os.path.join(ROOT, "tests", "golden", "abi_layout.c"), "-o", exe])
    mine = json.loads(subprocess.check_output([exe]))
    assert mine == GOLDEN["layout"]
    assert mine["sizeof(Op_Skeleton_Header)"] == 388 and mine["sizeof(Op_Skeleton)"] == 420 and mine["sizeof(Op)"] == 680
    from dataflow_lib_b200 import abi           # the ctypes mirror used by the Python tests
    assert C.sizeof(abi.OpSkeletonHeader) == 388 and C.sizeof(abi.OpSkeleton) == 420 and C.sizeof(abi.Op) == 680
    assert C.sizeof(abi.Table) == mine["sizeof(Table)"] and C.sizeof(abi.CudaDeviceInfo) == mine["sizeof(Cuda_Device_Info)"]
    assert C.sizeof(abi.CudaFunction) == mine["sizeof(Cuda_Function)"] and C.sizeof(abi.DataflowHandleStruct) == mine["sizeof(Dataflow_Handle)"]
    assert abi.DataflowHandleStruct.op_table.offset == mine["offsetof(Dataflow_Handle,op_table)"]
    assert abi.DataflowHandleStruct.submit_op.offset == mine["offsetof(Dataflow_Handle,submit_op)"]
    assert abi.CudaFunction.op_skeleton.offset == mine["offsetof(Cuda_Function,op_skeleton)"]


def test_sha256_known_answers(L):
    """FIPS 180-4 example digests plus boundary lengths cross-checked against hashlib."""
    import hashlib
    out = (C.c_uint8 * 32)()
    L.dataflow_sha256(b"abc", 3, out)
    assert bytes(out).hex() == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    L.dataflow_sha256(b"", 0, out)
    assert bytes(out).hex() == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    rng = np.random.default_rng(0)
    for n in (1, 55, 56, 57, 63, 64, 65, 119, 120, 127, 128, 388, 1000):
        msg = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        L.do_fingerprinting(msg, n, out, 0)
        assert bytes(out) == hashlib.sha256(msg).digest(), n
    fp = bytes(range(32))
    assert L.fingerprint_to_least_sig64(fp, 32) == int.from_bytes(fp[24:], "big")
    assert L.get_fingerprint_num_bytes(0) == 32 and L.get_fingerprint_type_name(0) == b"SHA256"


def test_datatype_names_and_sizes_match_reference(L):
    for k, name in GOLDEN["datatype_names"].items():
        assert L.dataflow_datatype_as_string(int(k)).decode() == name, k
    for k, size in GOLDEN["datatype_sizes"].items():
        assert L.dataflow_sizeof_element(int(k)) == size, k


def test_skeleton_fingerprints_match_reference(L):
    """Every (op, datatype) identity of the reference: nickname, argument list and SHA-256 are bit-identical."""
    from dataflow_lib_b200 import abi
    assert len(GOLDEN["skeletons"]) == 59
    seen = set()
    for rec in GOLDEN["skeletons"]:
        sk = abi.OpSkeleton()
        C.memset(C.byref(sk), 0xCD, C.sizeof(sk))
        assert L.set_native_op_skeleton(C.byref(sk), rec["op"].encode(), rec["fwd_dt"], rec["bwd_dt"]) == 0
        assert sk.header.op_nickname.decode() == rec["nickname"]
        assert sk.header.num_args == rec["num_args"]
        assert list(sk.header.arg_dtypes) == rec["arg_dtypes"]
        assert bytes(sk.identifier.fingerprint).hex() == rec["fingerprint"], rec["nickname"]
        seen.add(rec["fingerprint"])
    assert len(seen) == 59
    # spot values quoted in the survey of the reference
    by_nick = {r["nickname"]: r["fingerprint"] for r in GOLDEN["skeletons"]}
    assert by_nick["rms_norm_BF16"] == "f1b2adb5a53567728addb01da4e7e41fbe1cf74ce1dc68feb65eb76628d8d5ad"
    assert by_nick["swiglu_bwd_x_FP8E4M3_BF16"] == "32d7bf510467c9646f2f96c7c2af5c57df11a1cb364ae8b4dd561f1e5c95f904"
    sk = abi.OpSkeleton()
    assert L.set_native_op_skeleton(C.byref(sk), b"no_such_op", 3, 3) == -1
    # the fused op has its own identity, distinct from every reference op
    L.set_native_softmax_cross_entropy_skeleton(C.byref(sk), 5, 5)
    assert sk.header.op_nickname == b"softmax_cross_entropy_BF16_BF16" and bytes(sk.identifier.fingerprint).hex() not in seen


def test_hash_table(L):
    """insert / find / duplicate / remove with collisions, growth and wrap-around."""
    from dataflow_lib_b200 import abi
    HASH = C.CFUNCTYPE(C.c_uint64, C.c_void_p, C.c_uint64)
    hash_fn = HASH(lambda key, size: C.cast(key, C.POINTER(C.c_uint64))[0] % 7 % size)     # heavy collisions
    t = abi.Table()
    assert L.init_table(C.byref(t), C.cast(hash_fn, C.c_void_p), 8, 16, 8, 64, 0.5, 0.25) == 0
    val = lambda k: (C.c_uint64 * 2)(k * 3, k * 5)
    keys = list(range(100, 140))
    for k in keys:
        assert L.insert_table(C.byref(t), C.byref(C.c_uint64(k)), val(k)) == 0
    assert t.cnt == 40 and t.size == 64
    assert L.insert_table(C.byref(t), C.byref(C.c_uint64(105)), val(105)) == -1        # duplicate
    ret = C.c_void_p()
    for k in keys:
        idx = L.find_table(C.byref(t), C.byref(C.c_uint64(k)), False, C.byref(ret))
        assert idx >= 0 and C.cast(ret, C.POINTER(C.c_uint64))[0] == k * 3
    buf = (C.c_uint64 * 2)()
    assert L.find_table(C.byref(t), C.byref(C.c_uint64(117)), True, buf) >= 0 and list(buf) == [351, 585]
    assert L.find_table(C.byref(t), C.byref(C.c_uint64(999)), False, C.byref(ret)) == -1 and not ret.value
    for k in keys[::2]:
        assert L.remove_table(C.byref(t), C.byref(C.c_uint64(k)), buf) == 0 and buf[0] == k * 3
    assert L.remove_table(C.byref(t), C.byref(C.c_uint64(100)), buf) == -1
    for k in keys:
        found = L.find_table(C.byref(t), C.byref(C.c_uint64(k)), False, C.byref(ret)) >= 0
        assert found == (k in keys[1::2]), k
    assert t.cnt == 20
    for k in range(200, 244):
        assert L.insert_table(C.byref(t), C.byref(C.c_uint64(k)), val(k)) == 0
    assert t.cnt == 64 and L.insert_table(C.byref(t), C.byref(C.c_uint64(500)), val(500)) == -1   # full at max size
    L.destroy_table(C.byref(t))
    assert not t.items


def test_host_datatype_conversion(L):
    """fp32 <-> bf16/fp16 round-to-nearest-even, against the oracle's converters (themselves checked against torch)."""
    import oracle as O
    import torch
    rng = np.random.default_rng(1)
    f = (rng.standard_normal(200000) * np.exp(rng.standard_normal(200000) * 6)).astype(np.float32)
    f[:8] = [0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 1e-8, 6e-8]
    for dt, tdt in ((5, torch.bfloat16), (4, torch.float16)):
        out = np.empty(f.size, np.uint16)
        assert L.dataflow_convert_datatype(out.ctypes.data, f.ctypes.data, dt, 3, f.size, 4) == 0
        assert np.array_equal(out, O.from_f32(f, dt))
        assert np.array_equal(out, torch.from_numpy(f).to(tdt).view(torch.int16).numpy().view(np.uint16))
        back = np.empty(f.size, np.float32)
        assert L.dataflow_convert_datatype(back.ctypes.data, out.ctypes.data, 3, dt, f.size, 3) == 0
        assert np.array_equal(back.view(np.uint32), O.to_f32(out, dt).view(np.uint32))
    assert L.solo_fp32_to_bf16(1.0) == 0x3F80 and L.solo_bf16_to_fp32(0x3F80) == 1.0
    assert L.solo_fp32_to_fp16(1.0) == 0x3C00 and L.solo_fp16_to_fp32(0x3C00) == 1.0
    assert L.solo_fp16_to_bf16(0x3C00) == 0x3F80 and L.solo_bf16_to_fp16(0x3F80) == 0x3C00
    assert L.dataflow_convert_datatype(back.ctypes.data, out.ctypes.data, 6, 3, 4, 1) == -1    # no fp8 on the host, as in the reference


def test_reference_host_conversion_agrees_where_it_is_rne():
    """The reference's own converter (AVX-512 path, RNE) gives the same bf16/fp16 bits as this library's."""
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libref_host.so")
    flags = open("/proc/cpuinfo").read()
    if not os.path.exists(ref_path) or "avx512_bf16" not in flags or "avx512_fp16" not in flags:
        pytest.skip("reference host library or AVX-512 bf16/fp16 not available here")
    from dataflow_lib_b200 import _lib
    ref = C.CDLL(ref_path)
    ref.dataflow_convert_datatype.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_long, C.c_int]
    f = (np.random.default_rng(2).standard_normal(1 << 16) * 3).astype(np.float32)
    for dt in (5, 4):
        a, b = np.empty(f.size, np.uint16), np.empty(f.size, np.uint16)
        assert ref.dataflow_convert_datatype(a.ctypes.data, f.ctypes.data, dt, 3, f.size, 2) == 0
        assert _lib.lib.dataflow_convert_datatype(b.ctypes.data, f.ctypes.data, dt, 3, f.size, 2) == 0
        assert np.array_equal(a, b)


def test_handle_api_fails_cleanly_without_a_device(L, capfd):
    """No GPU here: init reports -1 (message on stderr) instead of crashing; submit on a dead handle is -1."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from dataflow_lib_b200 import abi
    h = abi.DataflowHandleStruct()
    assert L.init_cuda_dataflow_handle(C.byref(h), abi.COMPUTE_CUDA, 0, 0, 0, 2, None, None) == -1
    assert "Error" in capfd.readouterr().err
    assert L.init_cuda_dataflow_handle(C.byref(h), abi.COMPUTE_CUDA, 0, 0, 0, 9999, None, None) == -1
    assert L.submit_swiglu(C.byref(abi.DataflowHandleStruct()), 0, 5, 1, 8, None, None, None) == -1
    assert L.register_native_ops(C.byref(abi.DataflowHandleStruct()), None, None) == -1
    # the kernel launchers validate arguments before touching CUDA
    assert L.dfb200_swiglu(5, 1, 7, None, None, None, None) == -1
    assert b"NULL tensor argument" in L.dfb200_last_error()
    assert L.dfb200_swiglu(5, 1, 7, 0x1001, 0x1000, 0x1000, None) == -1       # an odd address for a 16-bit tensor
    assert b"not aligned to its element size" in L.dfb200_last_error()
    assert L.dfb200_rope(5, 63 * 4, 63, 63, 0, 10000, 0x1000, 0x2000, 0x3000, None) == -1 and b"must be even" in L.dfb200_last_error()
    assert L.dfb200_rms_norm(1, 1, 8, 1e-5, None, None, None, None, None, None) == -2
    # the fused op keeps the on-chip forms' row limit in every datatype (the long-row geometries must not widen it silently)
    for dt in (3, 4, 5, 6):
        assert L.dfb200_softmax_cross_entropy(dt, 5 if dt == 6 else dt, 1, 8 * 40000, 0x1000, 0x3000, 0x2000, None, None, None, 0, None) != 0
        assert b"exceeds the supported maximum of 262144" in L.dfb200_last_error()


def test_own_op_identities_are_stable(L):
    """Identities this library adds (ops whose kernels the reference has but never gave a skeleton, and the fused op): the
    nickname, argument list and fingerprint are part of the registry contract, so they are pinned here; each fingerprint is
    also the plain SHA-256 of the 388-byte header (checked with hashlib)."""
    import hashlib
    from dataflow_lib_b200 import abi
    want = {
        ("set_native_select_experts_skeleton", (5,)): ("select_experts_BF16", [26, 26, 26, 5, 5, 10, 13, 13, 13],
                                                        "4683b3047ffaec6f53315b8cfabe6a675b9a72e499f59203dbc4dbd5a95c73ab"),
        ("set_native_softmax_argmax_skeleton", (5,)): ("softmax_argmax_BF16_FP32", [26, 26, 5, 3, 9],
                                                        "13b5caeb8d64aaa103411c0bb1c5399a625a0e6318a6d041425527b2f1df6580"),
        ("set_native_softmax_argmax_skeleton", (4,)): ("softmax_argmax_FP16_FP32", [26, 26, 4, 3, 9],
                                                        "00bf0355dfb6b3de7356d47462035a81c77a2c8541b5f4721b14bd6834c9e97c"),
        ("set_native_softmax_cross_entropy_skeleton", (5, 5)): ("softmax_cross_entropy_BF16_BF16", [26, 26, 5, 9, 5, 3, 3],
                                                                "e769fbd45e29682394e79ad43293bd5d087f6af5cacea9039631b052b9377975"),
        ("set_native_rms_norm_bwd_w_sums_skeleton", (5, 5)): ("rms_norm_bwd_w_sums_BF16_BF16", [26, 26, 16, 3, 5, 5, 3],
                                                              "5a19551fe3c12e4ee113b9b1c15ddb8fe120304066491a8172d3027234afdec6"),
        ("set_native_rms_norm_bwd_x_w_skeleton", (5, 5)): ("rms_norm_bwd_x_w_BF16_BF16", [26, 26, 16, 3, 3, 5, 5, 5, 5, 5],
                                                           "2a16dacd8e5d5d29ec0f6d84674816de4944caa6ca9f5dfd8d3379ba3da61616"),
        ("set_native_rms_norm_bwd_x_w_skeleton", (6, 4)): ("rms_norm_bwd_x_w_FP8E4M3_FP16", [26, 26, 16, 3, 3, 6, 6, 4, 4, 4],
                                                           "7c45bab4018365bb664dd1a3984fbb530765aca83bf9a76064031b4ecbafd5dd"),
        ("set_native_rms_norm_bwd_x_w_sums_skeleton", (5, 5)): ("rms_norm_bwd_x_w_sums_BF16_BF16", [26, 26, 16, 3, 3, 5, 5, 5, 5, 3],
                                                                "24bd0572d6d2ae63bb6059c51c9063f3be724592c00386c3bdc8e8d0bf91e665"),
    }
    for (fn, args), (nick, dts, digest) in want.items():
        sk = abi.OpSkeleton()
        C.memset(C.byref(sk), 0xAB, C.sizeof(sk))
        getattr(L, fn)(C.byref(sk), *args)
        assert sk.header.op_nickname.decode() == nick
        assert list(sk.header.arg_dtypes)[:sk.header.num_args] == dts and all(d == 0 for d in list(sk.header.arg_dtypes)[sk.header.num_args:])
        assert bytes(sk.identifier.fingerprint).hex() == digest == hashlib.sha256(bytes(sk.header)).hexdigest()


def test_reference_external_wrappers_link_against_this_library():
    """The reference's external-op wrappers and skeletons (matmul, attention), compiled unchanged, resolve what they need
    (do_fingerprinting) from this library: the matmul identity they produce is the reference's."""
    so = os.path.join(ROOT, "oracle", "_ref", "libref_external_ops.so")
    if not os.path.exists(so):
        pytest.skip("reference wrappers not built (make -C oracle ref)")
    from dataflow_lib_b200 import abi
    ext = C.CDLL(so)
    sk = abi.OpSkeleton()
    ext.set_external_matmul_skeleton(C.byref(sk))
    assert sk.header.op_nickname == b"matmul" and sk.header.num_args == 19
    assert bytes(sk.identifier.fingerprint).hex() == "2a113b16e997d04b8408f9aa299dd5a80bb77d29c95c8cc78270410ef84f3590"
    for name in ("submit_matmul", "submit_attention", "submit_attention_bwd"):
        assert hasattr(ext, name)


def test_external_op_skeletons_match_the_reference(L):
    """set_external_{matmul,flash3_attention_fwd,flash3_attention_bwd}_skeleton of this library: nickname, argument list and
    fingerprint pinned (the matmul digest is the one the reference's own wrapper produces, see the test above), each digest the
    plain SHA-256 of the header; when the reference's wrappers were compiled here, all three skeletons are compared with theirs
    byte for byte (als244/dataflow_lib src/set_ops/src/set_external_op_skeletons.c:4-243)."""
    import hashlib
    from dataflow_lib_b200 import abi
    D = abi.DataflowDatatype
    IS, FS, VP, INT, U64, U64S = int(D.INT_SCALAR), int(D.FP32_SCALAR), int(D.VOID), int(D.INT), int(D.UINT64), int(D.UINT64_SCALAR)
    want = {
        "set_external_matmul_skeleton": ("matmul", [IS] * 11 + [FS, FS] + [VP] * 4 + [U64, VP]),
        "set_external_flash3_attention_fwd_skeleton": ("flash3_attention_fwd", [IS] * 4 + [INT, INT, IS, INT, INT, IS, IS, IS, IS] + [VP] * 5 + [U64S, VP]),
        "set_external_flash3_attention_bwd_skeleton": ("flash3_attention_bwd", [IS] * 4 + [INT, INT, IS, INT, INT, IS, IS, IS, IS] + [VP] * 9 + [U64S, VP]),
    }
    so = os.path.join(ROOT, "oracle", "_ref", "libref_external_ops.so")
    ext = C.CDLL(so) if os.path.exists(so) else None
    for fn, (nick, dts) in want.items():
        sk = abi.OpSkeleton()
        C.memset(C.byref(sk), 0xAB, C.sizeof(sk))
        getattr(L, fn)(C.byref(sk))
        assert sk.header.op_nickname.decode() == nick and sk.header.num_args == len(dts)
        names = [abi.DataflowDatatype(d).name for d in list(sk.header.arg_dtypes)[:sk.header.num_args]]
        assert list(sk.header.arg_dtypes)[:sk.header.num_args] == dts, names
        assert bytes(sk.identifier.fingerprint).hex() == hashlib.sha256(bytes(sk.header)).hexdigest()
        if ext is not None:
            theirs = abi.OpSkeleton()
            C.memset(C.byref(theirs), 0, C.sizeof(theirs))
            getattr(ext, fn)(C.byref(theirs))
            assert bytes(theirs) == bytes(sk), fn
    sk = abi.OpSkeleton()
    L.set_external_matmul_skeleton(C.byref(sk))
    assert bytes(sk.identifier.fingerprint).hex() == "2a113b16e997d04b8408f9aa299dd5a80bb77d29c95c8cc78270410ef84f3590"


def test_external_op_wrappers_build_the_reference_argument_lists(L):
    """submit_matmul / submit_attention / submit_attention_bwd hand the handle an Op whose op_args point at the values in the
    reference's order (src/dataflow_ops/src/matmul_op.c:33-51, attention_op.c:55-74, 107-130); checked with a handle whose submit_op
    is a Python callback. An unregistered op (callback returns non-zero) makes the wrapper return -1."""
    from dataflow_lib_b200 import abi
    seen = {}

    def capture(handle, op_ptr, stream_id):
        op = op_ptr.contents
        n = op.op_skeleton.header.num_args
        seen["nick"], seen["stream"] = op.op_skeleton.header.op_nickname.decode(), stream_id
        seen["args"] = [op.op_args[i] for i in range(n)]
        dts = list(op.op_skeleton.header.arg_dtypes)[:n]
        vals = []
        for a, dt in zip(seen["args"], dts):
            name = abi.DataflowDatatype(dt).name
            ctype = {"INT_SCALAR": C.c_int, "FP32_SCALAR": C.c_float, "UINT64": C.c_uint64, "UINT64_SCALAR": C.c_uint64}.get(name, C.c_void_p)
            vals.append(C.cast(a, C.POINTER(ctype)).contents.value)
        seen["vals"] = vals
        return seen.get("rc", 0)

    h = abi.DataflowHandleStruct()
    cb = type(h.submit_op)(capture)
    h.submit_op = cb
    BF16, FP32, NONE = int(abi.DataflowDatatype.BF16), int(abi.DataflowDatatype.FP32), int(abi.DataflowDatatype.NONE)
    assert L.submit_matmul(C.byref(h), 3, BF16, BF16, NONE, BF16, FP32, 1, 0, 64, 32, 16, 1.5, 0.25, 0x1000, 0x2000, None, 0x4000, 4096, 0x5000) == 0
    assert seen["nick"] == "matmul" and seen["stream"] == 3
    assert seen["vals"] == [0, BF16, BF16, NONE, BF16, FP32, 1, 0, 64, 32, 16, 1.5, 0.25, 0x1000, 0x2000, None, 0x4000, 4096, 0x5000]
    assert L.submit_attention(C.byref(h), 1, BF16, 2, 100, 120, 0x10, 0x20, 60, 0x30, 0x40, 70, 32, 8, 128, 0x50, 0x60, 0x70, 0x80, 0x90, 77, 0xA0) == 0
    assert seen["nick"] == "flash3_attention_fwd"
    assert seen["vals"] == [BF16, 2, 100, 120, 0x10, 0x20, 60, 0x30, 0x40, 70, 32, 8, 128, 0x50, 0x60, 0x70, 0x80, 0x90, 77, 0xA0]
    assert L.submit_attention_bwd(C.byref(h), 1, BF16, 2, 100, 120, 0x10, 0x20, 60, 0x30, 0x40, 70, 32, 8, 128, 0x50, 0x60, 0x70, 0x80, 0x90,
                                  0xB0, 0xC0, 0xD0, 0xE0, 88, 0xF0) == 0
    assert seen["nick"] == "flash3_attention_bwd"
    assert seen["vals"] == [BF16, 2, 100, 120, 0x10, 0x20, 60, 0x30, 0x40, 70, 32, 8, 128, 0x50, 0x60, 0x70, 0x80, 0x90, 0xB0, 0xC0, 0xD0, 0xE0, 88, 0xF0]
    # this library's fused norm backward: the argument list of rms_norm_bwd_x with the weight gradient appended
    assert L.submit_rms_norm_bwd_x_w(C.byref(h), 2, BF16, BF16, 100, 4096, 1e-5, 0x10, 0x20, 0x30, 0x40, 0x50, 0x60, 0x70) == 0
    assert seen["nick"] == "rms_norm_bwd_x_w_BF16_BF16" and seen["stream"] == 2
    assert seen["vals"][:2] == [100, 4096] and abs(seen["vals"][2] - 1e-5) < 1e-12 and seen["vals"][3:] == [0x10, 0x20, 0x30, 0x40, 0x50, 0x60, 0x70]
    assert L.submit_rms_norm_bwd_x_w_sums(C.byref(h), 0, BF16, BF16, 7, 64, 1e-5, 0x10, 0x20, 0x30, 0x40, 0x50, 0x60, 0x70) == 0
    assert seen["nick"] == "rms_norm_bwd_x_w_sums_BF16_BF16" and seen["vals"][3:] == [0x10, 0x20, 0x30, 0x40, 0x50, 0x60, 0x70]
    seen["rc"] = -1
    assert L.submit_matmul(C.byref(h), 0, BF16, BF16, NONE, BF16, FP32, 0, 0, 8, 8, 8, 1.0, 0.0, None, None, None, None, 0, None) == -1


def test_register_native_ops_with_the_reference_callers_arguments(L, capfd, tmp_path):
    """A caller written against the reference passes its cubin and launch-config library
    (src/set_ops/src/set_native_op_skeletons.c:40-170). Those are not this library: registration then takes the ops from the shared
    object that holds register_native_ops, says so in one line, and registers the full set."""
    from dataflow_lib_b200 import abi, _lib
    seen = {}

    def on_register(handle, path, n, skeletons, symbols, init_symbols):
        seen["path"], seen["n"] = path.decode(), n
        seen["symbols"] = {symbols[i].decode() for i in range(n)}
        return n

    h = abi.DataflowHandleStruct()
    cb = type(h.register_external_code)(on_register)
    h.register_external_code = cb
    own = os.path.realpath(_lib.LIB_PATH)
    cubin = tmp_path / "cuda_kernels.cubin"
    cubin.write_bytes(b"\x7fELF not a shared object")
    for arg in (b"lib/cuda_kernels.cubin", str(cubin).encode(), b"libm.so.6"):       # missing file, not loadable, loadable but without the ops
        seen.clear()
        assert L.register_native_ops(C.byref(h), arg, b"lib/cuda_kernels_config.so") == 96
        assert os.path.realpath(seen["path"]) == own and seen["n"] == 96 and "dataflow_b200_rms_norm" in seen["symbols"]
        assert "registering them from this library instead" in capfd.readouterr().err
    for arg in (None, own.encode()):                                                  # the documented forms: no notice
        seen.clear()
        assert L.register_native_ops(C.byref(h), arg, None) == 96
        assert os.path.realpath(seen["path"]) == own
        assert "Notice" not in capfd.readouterr().err


def _head_containers(abi, T=8, d=16, V=64):
    BF16, FP32 = int(abi.DataflowDatatype.BF16), int(abi.DataflowDatatype.FP32)
    head = abi.TransformerHead(BF16, BF16, FP32, 1e-5, abi.EmbeddingConfig(V, d), None, 0x1000, 0x2000)
    act = abi.TransformerHeadActivations(T, None, 0x3000, 0x3100, 0x3200, 0x3300, 0x3400, 4096)
    xin = abi.TransformerBlockTransition(None, 0x4000)
    out = abi.TransformerModelOutput(None, None, 0x5000, 0x5100, 0x5200, 0.0)
    ghead = abi.TransformerHead(BF16, BF16, FP32, 1e-5, abi.EmbeddingConfig(V, d), None, 0x6000, 0x6100)
    gact = abi.TransformerHeadActivations(T, None, 0x7000, None, None, 0x7300, 0x7400, 8192)
    gs, gs2 = abi.TransformerBlockTransition(None, 0x8000), abi.TransformerBlockTransition(None, 0x9000)
    return head, act, xin, out, ghead, gact, gs, gs2


def test_transformer_head_submits_the_reference_chain(L):
    """submit_transformer_head on a handle made of Python callbacks: the ops arrive in the reference's order
    (src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:316-492) with the buffers wired as documented, the copy of
    the head gradient is ordered after the compute stream, and a failing step stops the chain with that step's code."""
    from dataflow_lib_b200 import abi
    log = []

    def on_op(handle, op_ptr, stream_id):
        op = op_ptr.contents
        n = op.op_skeleton.header.num_args
        ptrs = []
        for i, dt in enumerate(list(op.op_skeleton.header.arg_dtypes)[:n]):
            name = abi.DataflowDatatype(dt).name
            if not name.endswith("_SCALAR") and name != "UINT64":
                ptrs.append(C.cast(op.op_args[i], C.POINTER(C.c_void_p)).contents.value)
        nick = op.op_skeleton.header.op_nickname.decode()
        log.append((nick, stream_id, ptrs))
        return -7 if nick == fail_on[0] else 0

    fail_on = [None]
    h = abi.DataflowHandleStruct()
    state = C.c_int(0)
    cbs = {
        "submit_op": type(h.submit_op)(on_op),
        "get_stream_state": type(h.get_stream_state)(lambda hh, s: (log.append(("state", s, [])), C.addressof(state))[1]),
        "submit_dependency": type(h.submit_dependency)(lambda hh, s, st: (log.append(("dep", s, [st])), 0)[1]),
        "submit_peer_transfer": type(h.submit_peer_transfer)(lambda hh, s, dst, src, n: (log.append(("copy", s, [dst, src, n])), 0)[1]),
    }
    for k, v in cbs.items():
        setattr(h, k, v)
    head, act, xin, out, ghead, gact, gs, gs2 = _head_containers(abi)
    T, d, V = 8, 16, 64
    r = C.byref
    # forward only
    assert L.submit_transformer_head(r(h), 2, 3, r(xin), r(head), r(act), r(out), None, None, None, None) == 0
    assert [e[0] for e in log] == ["rms_norm_BF16", "matmul", "softmax_BF16_BF16"] and all(e[1] == 2 for e in log)
    assert log[0][2] == [0x1000, 0x4000, 0x3000, 0x3100, 0x3200]          # weight, X, out, weighted sums, rms values
    assert log[1][2] == [0x2000, 0x3000, None, 0x3300, 0x3400]            # A = w_head, B = head_norm_out, C, D = logits, workspace
    assert log[2][2] == [0x3300, 0x5100]
    # forward + backward with the copy to the next location
    log.clear()
    assert L.submit_transformer_head(r(h), 2, 3, r(xin), r(head), r(act), r(out), r(ghead), r(gact), r(gs), r(gs2)) == 0
    assert [e[0] for e in log] == ["rms_norm_BF16", "matmul", "softmax_cross_entropy_BF16_BF16", "matmul", "matmul", "rms_norm_bwd_x_BF16_BF16",
                                   "rms_norm_bwd_w_BF16_BF16", "state", "dep", "copy"]
    assert log[2][2] == [0x3300, 0x5000, 0x5100, 0x5200, None]            # logits, labels, dlogits, row losses, no loss sum
    assert log[3][2] == [0x2000, 0x5100, None, 0x7000, 0x7400]            # d(head_norm_out) = w_head . dlogits
    assert log[4][2] == [0x3000, 0x5100, 0x6100, 0x6100, 0x7400]          # dW_head += head_norm_out . dlogits^T
    assert log[5][2] == [0x3100, 0x3200, 0x1000, 0x4000, 0x7000, 0x8000]  # sums, rms, weight, X, upstream, dX
    assert log[6][2] == [0x3200, 0x4000, 0x7000, 0x6000]                  # rms, X, upstream, dW_norm
    assert log[7][1] == 2 and log[8][1] == 3 and log[8][2] == [C.addressof(state)]
    assert log[9][1] == 3 and log[9][2] == [0x9000, 0x8000, T * d * 2]
    # a failing step ends the chain with its code
    log.clear()
    fail_on[0] = "softmax_cross_entropy_BF16_BF16"
    assert L.submit_transformer_head(r(h), 0, 1, r(xin), r(head), r(act), r(out), r(ghead), r(gact), r(gs), None) == -1
    assert [e[0] for e in log] == ["rms_norm_BF16", "matmul", "softmax_cross_entropy_BF16_BF16"]
    # a backward pass without its containers is refused before anything is submitted
    log.clear()
    assert L.submit_transformer_head(r(h), 0, 1, r(xin), r(head), r(act), r(out), r(ghead), None, None, None) == -1 and not log


# ---- the block callers on a handle made of callbacks ------------------------------------------------------------------------

def _callback_handle(abi, log, fail_on):
    """A Dataflow_Handle whose function table is Python: every op, memset, copy, stream state and dependency is appended to `log`
    as (name, stream, values). Op values: every argument in order, scalars by value and pointers as integers."""
    h = abi.DataflowHandleStruct()
    state = C.c_int(0)

    def on_op(handle, op_ptr, stream_id):
        op = op_ptr.contents
        n = op.op_skeleton.header.num_args
        vals = []
        for i, dt in enumerate(list(op.op_skeleton.header.arg_dtypes)[:n]):
            name = abi.DataflowDatatype(dt).name
            ctype = {"INT_SCALAR": C.c_int, "FP32_SCALAR": C.c_float, "UINT64": C.c_uint64, "UINT64_SCALAR": C.c_uint64}.get(name, C.c_void_p)
            vals.append(C.cast(op.op_args[i], C.POINTER(ctype)).contents.value)
        nick = op.op_skeleton.header.op_nickname.decode()
        log.append((nick, stream_id, vals))
        return -7 if nick == fail_on[0] else 0

    cbs = {
        "submit_op": type(h.submit_op)(on_op),
        "get_stream_state": type(h.get_stream_state)(lambda hh, s: (log.append(("state", s, [])), C.addressof(state))[1]),
        "submit_dependency": type(h.submit_dependency)(lambda hh, s, st: (log.append(("dep", s, [st])), 0)[1]),
        "submit_peer_transfer": type(h.submit_peer_transfer)(lambda hh, s, dst, src, n: (log.append(("copy", s, [dst, src, n])), 0)[1]),
        "set_mem": type(h.set_mem)(lambda hh, s, p, v, n: (log.append(("set_mem", s, [p, v, n])), 0)[1]),
    }
    for k, v in cbs.items():
        setattr(h, k, v)
    return h, cbs, C.addressof(state)


def _block_containers(abi, base, T=8, nq=4, nkv=2, hd=8, f=48):
    """A block (or gradient block) and its activation containers with recognisable fake addresses starting at `base`."""
    BF16, FP32 = int(abi.DataflowDatatype.BF16), int(abi.DataflowDatatype.FP32)
    keep = []
    one = lambda addr: (keep.append((C.c_void_p * 1)(addr)), C.cast(keep[-1], C.POINTER(C.c_void_p)))[1]
    blk = abi.TransformerBlock()
    c = blk.config
    c.block_dt, c.compute_dt, c.eps, c.theta = BF16, FP32, 1e-5, 10000
    c.num_q_heads, c.num_kv_heads, c.head_dim, c.model_dim, c.kv_dim, c.ffn_dim = nq, nkv, hd, nq * hd, nkv * hd, f
    blk.w_attn_norm, blk.w_q, blk.w_k, blk.w_v, blk.w_o, blk.w_ffn_norm = (base + 0x10 * i for i in range(1, 7))
    blk.w_1, blk.w_2, blk.w_3 = one(base + 0x70), one(base + 0x80), one(base + 0x90)
    bc = abi.SeqBatchConfig(2, T, T + 4, base + 0x100, base + 0x110, base + 0x120, 5, base + 0x130, base + 0x140, 7)
    sv = abi.SeqBatchSavedActivations()
    sv.attn_norm_weighted_sums, sv.attn_norm_rms_vals, sv.x_q, sv.x_k_local, sv.x_v_local = (base + 0x200 + 0x10 * i for i in range(5))
    sv.softmax_lse, sv.x_attn_out, sv.x_o, sv.ffn_norm_weighted_sums, sv.ffn_norm_rms_vals = (base + 0x250 + 0x10 * i for i in range(5))
    sv.x_1, sv.x_2, sv.x_3 = one(base + 0x2a0), one(base + 0x2b0), one(base + 0x2c0)
    ctx = abi.SeqBatchContext(None, None, 0, base + 0x300, base + 0x310)
    ws = abi.SeqBatchActivationWorkspace(None, None, 0, base + 0x400, base + 0x410, base + 0x420, base + 0x430, base + 0x440, 4096)
    act = abi.TransformerBlockActivations(C.pointer(blk), C.pointer(bc), C.pointer(sv), C.pointer(ctx), C.pointer(ws))
    keep += [blk, bc, sv, ctx, ws]
    return blk, act, keep


def test_transformer_struct_mirrors_match_the_header(tmp_path):
    """The ctypes mirrors used by the tests have the sizes the C header gives the structs."""
    from dataflow_lib_b200 import abi
    names = {"Seq_Batch_Config": abi.SeqBatchConfig, "Seq_Batch_Saved_Activations": abi.SeqBatchSavedActivations,
             "Seq_Batch_Context": abi.SeqBatchContext, "Seq_Batch_Activation_Workspace": abi.SeqBatchActivationWorkspace,
             "MoE_Config": abi.MoEConfig, "Transformer_Block_Config": abi.TransformerBlockConfig, "Transformer_Block": abi.TransformerBlock,
             "Transformer_Block_Activations": abi.TransformerBlockActivations, "Transformer_Head": abi.TransformerHead,
             "Transformer_Head_Activations": abi.TransformerHeadActivations, "Transformer_Block_Transition": abi.TransformerBlockTransition,
             "Transformer_Model_Output": abi.TransformerModelOutput}
    src = tmp_path / "sizes.c"
    src.write_text('#include "dataflow_transformer.h"\n#include <stdio.h>\nint main(void) {\n' +
                   "".join(f'printf("{n} %zu\\n", sizeof({n}));\n' for n in names) +
                   'printf("w_1 %zu x_o %zu\\n", offsetof(Transformer_Block, w_1), offsetof(Seq_Batch_Saved_Activations, x_o));\nreturn 0; }\n')
    exe = str(tmp_path / "sizes")
    subprocess.check_call(["gcc", f"-I{ROOT}/include", str(src), "-o", exe])
    out = dict(line.split(" ", 1) for line in subprocess.check_output([exe], text=True).strip().splitlines())
    for n, t in names.items():
        assert int(out[n]) == C.sizeof(t), n
    assert out["w_1"] == f"{abi.TransformerBlock.w_1.offset} x_o {abi.SeqBatchSavedActivations.x_o.offset}"


def test_transformer_block_forward_submits_the_reference_chain(L):
    """submit_transformer_block on a handle made of callbacks: op order of src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:72-283,
    buffer wiring, RoPE in place on x_q / x_k_local, residual projections with beta = 1 and C = the residual, K / V projections with
    kv_dim outputs, the workspace zeroed before the attention, the output copy ordered after the compute stream."""
    from dataflow_lib_b200 import abi
    log, fail_on = [], [None]
    h, cbs, state = _callback_handle(abi, log, fail_on)
    B = 0x10000
    blk, act, keep = _block_containers(abi, B)
    T, d, kv, f = 8, 32, 16, 48
    BF16, FP32, NONE = int(abi.DataflowDatatype.BF16), int(abi.DataflowDatatype.FP32), int(abi.DataflowDatatype.NONE)
    xin, xout = abi.TransformerBlockTransition(None, 0x5000), abi.TransformerBlockTransition(None, 0x6000)
    r = C.byref
    assert L.submit_transformer_block(r(h), 2, 3, r(xin), r(blk), r(act), r(xout)) == 0
    names = [e[0] for e in log]
    assert names == ["rms_norm_BF16", "matmul", "matmul", "matmul", "rope_BF16", "set_mem", "flash3_attention_fwd", "matmul", "rms_norm_BF16",
                     "matmul", "matmul", "swiglu_BF16", "matmul", "state", "dep", "copy"]
    assert all(e[1] == 2 for e in log[:14]) and log[14][1] == 3 and log[15][1] == 3

    def mm(e):      # (to_trans_a, to_trans_b, M, K, N, alpha, beta, c_dt, A, B, C, D)
        v = e[2]
        return (v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[3], v[13], v[14], v[15], v[16])

    x_temp, x_mlp = B + 0x400, B + 0x410
    sums_a, rms_a, x_q, x_k, x_v, lse, attn_out, x_o, sums_f, rms_f = (B + 0x200 + 0x10 * i for i in range(10))
    x_1, x_2, x_3 = B + 0x2a0, B + 0x2b0, B + 0x2c0
    assert log[0][2] == [T, d, pytest.approx(1e-5), B + 0x10, 0x5000, x_temp, sums_a, rms_a]
    assert mm(log[1]) == (1, 0, d, d, T, 1.0, 0.0, NONE, B + 0x20, x_temp, None, x_q)
    assert mm(log[2]) == (1, 0, kv, d, T, 1.0, 0.0, NONE, B + 0x30, x_temp, None, x_k)
    assert mm(log[3]) == (1, 0, kv, d, T, 1.0, 0.0, NONE, B + 0x40, x_temp, None, x_v)
    assert log[4][2] == [T * d, d, 8, 2, 10000, B + 0x100, x_q, x_k]                      # in place on the projections' outputs
    assert log[5][2] == [B + 0x440, 0, 4096]
    assert log[6][2] == [BF16, 2, T, T + 4, B + 0x110, B + 0x120, 5, B + 0x130, B + 0x140, 7, 4, 2, 8, x_q, B + 0x300, B + 0x310, attn_out, lse, 4096, B + 0x440]
    assert mm(log[7]) == (1, 0, d, d, T, 1.0, 1.0, BF16, B + 0x50, attn_out, 0x5000, x_o)    # + the block input (residual)
    assert log[8][2] == [T, d, pytest.approx(1e-5), B + 0x60, x_o, x_temp, sums_f, rms_f]
    assert mm(log[9]) == (1, 0, f, d, T, 1.0, 0.0, NONE, B + 0x70, x_temp, None, x_1)
    assert mm(log[10]) == (1, 0, f, d, T, 1.0, 0.0, NONE, B + 0x90, x_temp, None, x_3)
    assert log[11][2] == [T, f, x_1, x_3, x_mlp]
    assert mm(log[12]) == (1, 0, d, f, T, 1.0, 1.0, BF16, B + 0x80, x_mlp, x_o, x_2)          # + x_o (residual)
    assert log[13][1] == 2 and log[14][2] == [state] and log[15][2] == [0x6000, x_2, T * d * 2]
    # a failing step ends the chain with its code; no output transition = no copy
    log.clear()
    fail_on[0] = "flash3_attention_fwd"
    assert L.submit_transformer_block(r(h), 0, 1, r(xin), r(blk), r(act), r(xout)) == -1
    assert [e[0] for e in log][-1] == "flash3_attention_fwd" and len(log) == 7
    log.clear()
    fail_on[0] = None
    assert L.submit_transformer_block(r(h), 0, 1, r(xin), r(blk), r(act), None) == 0 and "copy" not in [e[0] for e in log]
    assert L.submit_transformer_block(r(h), 0, 1, r(xin), r(blk), None, None) == -1


def test_transformer_block_backward_chains(L):
    """submit_transformer_block_bwd_x and _bwd_w on a handle made of callbacks (dataflow_transformer.c:565-1003): step order, the two
    RMSNorm input-gradient ops accumulating into the stream gradient, accumulated (C = D, beta = 1) W_3 / W_k / W_v products, d(x_o)
    kept for the W_o weight gradient, the two recompute RMSNorm calls with NULL statistics, and the weight-gradient products."""
    from dataflow_lib_b200 import abi
    log, fail_on = [], [None]
    h, cbs, state = _callback_handle(abi, log, fail_on)
    W, G, GW = 0x10000, 0x20000, 0x30000                     # forward containers, gradient containers, gradient weights
    blk, act, k1 = _block_containers(abi, W)
    _, gact, k2 = _block_containers(abi, G)
    gblk, _, k3 = _block_containers(abi, GW)
    T, d, kv, f = 8, 32, 16, 48
    BF16, NONE = int(abi.DataflowDatatype.BF16), int(abi.DataflowDatatype.NONE)
    dstream, xin, dnext = abi.TransformerBlockTransition(None, 0x5000), abi.TransformerBlockTransition(None, 0x6000), abi.TransformerBlockTransition(None, 0x7000)
    r = C.byref
    assert L.submit_transformer_block_bwd_x(r(h), 2, 3, r(blk), r(dstream), r(act), r(xin), r(gact), r(gblk), r(dnext)) == 0
    names = [e[0] for e in log]
    assert names == ["matmul", "swiglu_bwd_x_BF16_BF16", "matmul", "matmul", "rms_norm_bwd_x_BF16_BF16", "rms_norm_bwd_w_BF16_BF16", "copy",
                     "matmul", "set_mem", "flash3_attention_bwd", "rope_bwd_x_BF16", "matmul", "matmul", "matmul",
                     "rms_norm_bwd_x_BF16_BF16", "rms_norm_bwd_w_BF16_BF16", "rms_norm_BF16", "rms_norm_BF16", "state", "dep", "copy"]

    def mm(e):
        v = e[2]
        return (v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[3], v[13], v[14], v[15], v[16])

    sv = lambda base, i: base + 0x200 + 0x10 * i          # attn sums, attn rms, x_q, x_k_local, x_v_local, lse, attn_out, x_o, ffn sums, ffn rms
    g_temp, g_mlp, re_attn, re_ffn, g_ws = G + 0x400, G + 0x410, G + 0x420, G + 0x430, G + 0x440
    dX = 0x5000
    assert mm(log[0]) == (0, 0, f, d, T, 1.0, 0.0, NONE, W + 0x80, dX, None, g_mlp)                     # d(swiglu out) = dOut W_2
    assert log[1][2] == [T, f, W + 0x2a0, W + 0x2c0, g_mlp, G + 0x2a0, G + 0x2c0]
    assert mm(log[2]) == (0, 0, d, f, T, 1.0, 0.0, NONE, W + 0x70, G + 0x2a0, None, g_temp)
    assert mm(log[3]) == (0, 0, d, f, T, 1.0, 1.0, BF16, W + 0x90, G + 0x2c0, g_temp, g_temp)           # accumulated
    assert log[4][2] == [T, d, pytest.approx(1e-5), sv(W, 8), sv(W, 9), W + 0x60, sv(W, 7), g_temp, dX]   # accumulates into the stream gradient
    assert log[5][2] == [T, d, pytest.approx(1e-5), sv(W, 9), sv(W, 7), g_temp, GW + 0x60]
    assert log[6][1] == 2 and log[6][2] == [sv(G, 7), dX, T * d * 2]                                      # d(x_o) kept
    assert mm(log[7]) == (0, 0, d, d, T, 1.0, 0.0, NONE, W + 0x50, sv(G, 7), None, g_temp)
    assert log[8][2] == [g_ws, 0, 4096]
    assert log[9][2] == [BF16, 2, T, T + 4, G + 0x110, G + 0x120, 5, G + 0x130, G + 0x140, 7, 4, 2, 8, sv(W, 2), W + 0x300, W + 0x310, sv(W, 6), sv(W, 5),
                         g_temp, sv(G, 2), G + 0x300, G + 0x310, 4096, g_ws]
    assert log[10][2] == [T * d, d, 8, 2, 10000, G + 0x100, sv(G, 2), sv(G, 3)]
    assert mm(log[11]) == (0, 0, d, d, T, 1.0, 0.0, NONE, W + 0x20, sv(G, 2), None, g_temp)
    assert mm(log[12]) == (0, 0, d, kv, T, 1.0, 1.0, BF16, W + 0x30, sv(G, 3), g_temp, g_temp)
    assert mm(log[13]) == (0, 0, d, kv, T, 1.0, 1.0, BF16, W + 0x40, sv(G, 4), g_temp, g_temp)
    assert log[14][2] == [T, d, pytest.approx(1e-5), sv(W, 0), sv(W, 1), W + 0x10, 0x6000, g_temp, dX]
    assert log[15][2] == [T, d, pytest.approx(1e-5), sv(W, 1), 0x6000, g_temp, GW + 0x10]
    assert log[16][2] == [T, d, pytest.approx(1e-5), W + 0x10, 0x6000, re_attn, None, None]
    assert log[17][2] == [T, d, pytest.approx(1e-5), W + 0x60, sv(W, 7), re_ffn, None, None]
    assert log[19][1] == 3 and log[20][1] == 3 and log[20][2] == [0x7000, dX, T * d * 2]
    assert all(e[1] == 2 for e in log[:19])

    # weight gradients
    log.clear()
    dout = abi.TransformerBlockTransition(None, 0x8000)
    assert L.submit_transformer_block_bwd_w(r(h), 4, r(dout), r(act), r(gact), r(gblk)) == 0
    assert [e[0] for e in log] == ["swiglu_BF16"] + ["matmul"] * 7 and all(e[1] == 4 for e in log)
    assert log[0][2] == [T, f, W + 0x2a0, W + 0x2c0, g_mlp]
    wg = lambda e: mm(e)
    assert wg(log[1]) == (0, 1, f, T, d, 1.0, 1.0, BF16, g_mlp, 0x8000, GW + 0x80, GW + 0x80)            # dW_2 [d, f] += dOut^T h
    assert wg(log[2]) == (0, 1, d, T, f, 1.0, 1.0, BF16, re_ffn, G + 0x2a0, GW + 0x70, GW + 0x70)
    assert wg(log[3]) == (0, 1, d, T, f, 1.0, 1.0, BF16, re_ffn, G + 0x2c0, GW + 0x90, GW + 0x90)
    assert wg(log[4]) == (0, 1, d, T, d, 1.0, 1.0, BF16, sv(W, 6), sv(G, 7), GW + 0x50, GW + 0x50)
    assert wg(log[5]) == (0, 1, d, T, kv, 1.0, 1.0, BF16, re_attn, sv(G, 4), GW + 0x40, GW + 0x40)
    assert wg(log[6]) == (0, 1, d, T, kv, 1.0, 1.0, BF16, re_attn, sv(G, 3), GW + 0x30, GW + 0x30)
    assert wg(log[7]) == (0, 1, d, T, d, 1.0, 1.0, BF16, re_attn, sv(G, 2), GW + 0x20, GW + 0x20)
    # failures propagate
    log.clear()
    fail_on[0] = "flash3_attention_bwd"
    assert L.submit_transformer_block_bwd_x(r(h), 2, 3, r(blk), r(dstream), r(act), r(xin), r(gact), r(gblk), None) == -1
    assert [e[0] for e in log][-1] == "flash3_attention_bwd"
    assert L.submit_transformer_block_bwd_w(r(h), 4, r(dout), r(act), None, r(gblk)) == -1
